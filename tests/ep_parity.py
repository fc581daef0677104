"""The expert-parallel layer on `world` ranks against the CPU oracle: one small layer (T=384 tokens per rank, d=256,
8 experts, top-2, ffn 128), two steps so that every buffer, local and remote, is reused. Used by the 2-GPU test and by
bench.py after its timed region (every rank checks its own outputs; raises AssertionError on a mismatch).

Tokens are independent, so rank r's outputs (out, dXn) must equal the oracle's single-GPU layer on rank r's batch with
all experts; the expert weight gradients on the owning rank must equal the sum of the oracle's gradients over all
ranks' batches; the per-expert row counts seen by the owner must equal the sum of the ranks' counts (bit-exact)."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def check_expert_parallel(dist, rank, world, transport, num_experts=8):
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_chain_close, assert_close, bf16_bits_to_f32 as f32
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.ep import ExpertParallelMoELayer
    from oracle import oracle as orc

    T, d, E, k, f = 384, 256, num_experts, 2, 128
    assert E % world == 0
    El = E // world
    wrng = np.random.default_rng(99)
    Wr = rand_bf16(wrng, (E, d), 0.06)
    W1, W3, W2 = rand_bf16(wrng, (E, f, d), 0.06), rand_bf16(wrng, (E, f, d), 0.06), rand_bf16(wrng, (E, d, f), 0.06)
    batches = []
    for r in range(world):
        rng = np.random.default_rng(1000 + r)
        batches.append((rand_bf16(rng, (T, d)), rand_bf16(rng, (T, d))))
    X, dOut = batches[rank]
    sl = slice(rank * El, (rank + 1) * El)
    # "c": the buffers of the fused transport driven by b200_ep_moe_block_fwd / _bwd (barriers, counts exchange, plan
    # and router-gradient sum by the library's own kernels, no torch.distributed call inside the step)
    c_driver = transport == "c"
    layer = ExpertParallelMoELayer(T, d, E, k, f, dist, device=torch.device("cuda", torch.cuda.current_device()),
                                   transport="fused" if c_driver else transport)
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    dXn = torch.empty_like(out)
    dWr = torch.zeros((E, d), dtype=torch.bfloat16, device="cuda")
    dW1, dW3 = (torch.zeros((El, f, d), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    dW2 = torch.zeros((El, d, f), dtype=torch.bfloat16, device="cuda")
    Xd, dOd, Wrd = dev_bf16(X), dev_bf16(dOut), dev_bf16(Wr)
    W1d, W3d, W2d = dev_bf16(W1[sl]), dev_bf16(W3[sl]), dev_bf16(W2[sl])
    for _ in range(2):  # the second pass reuses every buffer, local and remote
        for t_ in (out, dWr, dW1, dW3, dW2):
            t_.zero_()
        if c_driver:
            blk = layer.c_block(Wrd, W1d, W3d, W2d)
            ops.ep_moe_block_fwd(blk, Xd, out)
            ops.ep_moe_block_bwd(blk, Xd, dOd, dXn, dWr, dW1, dW3, dW2)
        else:
            layer.forward(Xd, Wrd, W1d, W3d, W2d, out)
            layer.backward(Xd, Wrd, W1d, W3d, W2d, dOd, dXn, dWr, dW1, dW3, dW2)
    layer.check()  # no GEMM wait gave up, no receive buffer overflowed

    # oracle: every rank's batch through the single-GPU layer; this rank's logits come from its own GPU run
    grads = dict(dW1=np.zeros_like(W1), dW3=np.zeros_like(W3), dW2=np.zeros_like(W2), dWr=np.zeros_like(Wr))
    total_counts = np.zeros(E, np.int64)
    mine = None
    gathered = [torch.zeros((T, E), dtype=torch.float32, device="cuda") for _ in range(world)]
    dist.all_gather(gathered, layer.home.logits)
    for r in range(world):
        Xr, dOr = batches[r]
        fwd = orc.moe_forward(Xr, Wr, W1, W3, W2, k, logits=gathered[r].cpu().numpy())
        bwd = orc.moe_backward(Xr, Wr, W1, W3, W2, k, fwd, dOr, grads=grads)
        total_counts += fwd["counts"][:E]
        if r == rank:
            mine = (fwd, bwd["dXn"].copy())
    local_counts = layer._c_local["local_counts"] if c_driver else layer.x.local_counts
    np.testing.assert_array_equal(local_counts.cpu().numpy(), total_counts[sl])
    np.testing.assert_array_equal(layer.home.token_mapping.cpu().numpy(), mine[0]["token_mapping"])
    assert_chain_close(f32(host_bits(out)), f32(mine[0]["out"]), what="out")
    assert_close(f32(host_bits(out)), f32(mine[0]["out"]), rtol=2e-2, atol=4e-3, what="out")
    assert_chain_close(f32(host_bits(dXn)), f32(mine[1]), what="dXn")
    for got, ref, what in [(dW1, grads["dW1"][sl], "dW1"), (dW3, grads["dW3"][sl], "dW3"), (dW2, grads["dW2"][sl], "dW2")]:
        assert_chain_close(f32(host_bits(got)), f32(ref), what=what)
    assert_chain_close(f32(host_bits(dWr)), f32(grads["dWr"]), limit=5e-2, what="dWr")
