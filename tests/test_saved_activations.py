"""The saved-activation levels of the MoE part of a block (the reference's SavedActivationLevel,
libdataflowmodels/include/transformer/seq_batch_structs.h:199-204).

CPU: the size of the saved set per level against a restatement of the reference's layout (prep_seq_batch.c:230-283,
320-365: routing tensors in its order, 256-byte aligned, x1 / x3 only at FULL). GPU: forward, offload the saved set to
pinned host memory, overwrite every buffer of the block, bring the set back, recompute what the level did not keep,
run the backward: the weight gradients must equal, bit for bit, those of a backward that ran straight after the
forward.
"""
import ctypes as C

import numpy as np
import pytest

NONE, INP_ONLY, INP_ATTN_ONLY, FULL = 0, 1, 2, 3


def expected_bytes(T, E, k, f, level):
    if level == NONE:
        return 0
    R = T * k
    sizes = [4 * T * E, 2 * R, 4 * R, 4 * (E + 1), 4 * E, 4 * R, 4 * R]
    if level == FULL:
        sizes += [2 * R * f, 2 * R * f]
    at = 0
    for s in sizes:
        at = (at + 255) // 256 * 256 + s
    return at


@pytest.mark.parametrize("shape", [(300, 16, 4, 192), (8192, 64, 8, 1408), (1, 2, 1, 8)])
def test_saved_set_sizes_follow_the_reference_layout(shape):
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    T, E, k, f = shape
    for level in (NONE, INP_ONLY, INP_ATTN_ONLY, FULL):
        assert lib.b200_moe_saved_activations_bytes(T, E, k, f, level) == expected_bytes(T, E, k, f, level)
    assert lib.b200_moe_saved_activations_bytes(T, E, k, f, 7) == 0
    # the two lower levels keep the same MoE tensors; FULL adds x1 and x3
    assert expected_bytes(T, E, k, f, INP_ONLY) == expected_bytes(T, E, k, f, INP_ATTN_ONLY) < expected_bytes(T, E, k, f, FULL)


@pytest.mark.gpu
@pytest.mark.parametrize("level", [INP_ONLY, INP_ATTN_ONLY, FULL])
def test_offload_restore_recompute_then_backward(level):
    import torch

    from gpu_util import dev_bf16, rand_bf16, require_b200

    require_b200()
    from ml_dataflow_b200 import _lib, ops
    from ml_dataflow_b200.moe_layer import MoELayer

    lib = _lib.load()
    T, d, E, k, f = 700, 256, 16, 4, 192
    rng = np.random.default_rng(21)
    X, dOut = dev_bf16(rand_bf16(rng, (T, d))), dev_bf16(rand_bf16(rng, (T, d)))
    Wr = dev_bf16(rand_bf16(rng, (E, d), 0.05))
    W1, W3 = dev_bf16(rand_bf16(rng, (E, f, d), 0.05)), dev_bf16(rand_bf16(rng, (E, f, d), 0.05))
    W2 = dev_bf16(rand_bf16(rng, (E, d, f), 0.05))
    layer = MoELayer(T, d, E, k, f)
    blk = layer.block(Wr, W1, W3, W2)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def grads():
        return [torch.zeros_like(Wr), torch.zeros_like(W1), torch.zeros_like(W3), torch.zeros_like(W2)]

    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    ops.moe_block_fwd(blk, X, out)
    # reference run: backward straight after the forward
    dXn_a, Ga = torch.empty_like(out), grads()
    ops.moe_block_bwd(blk, X, dOut, dXn_a, *Ga)
    # offload what the level keeps, then lose everything the block holds
    nbytes = lib.b200_moe_saved_activations_bytes(T, E, k, f, level)
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    assert lib.b200_moe_block_save_activations(C.byref(blk), level, C.c_void_p(host.data_ptr()), nbytes, stream) == 0
    torch.cuda.synchronize()
    for name in ("logits", "weights", "chosen", "counts", "cumsum", "expert_mapping", "token_mapping", "zone", "x1", "x3",
                 "h", "Y", "dYz", "dx1", "dx3", "dZ"):
        getattr(layer, name).view(torch.uint8).fill_(0x5A)
    assert lib.b200_moe_block_restore_activations(C.byref(blk), level, C.c_void_p(host.data_ptr()), nbytes, stream) == 0
    assert lib.b200_moe_block_recompute_level(C.byref(blk), C.c_void_p(X.data_ptr()), level, stream) == 0
    dXn_b, Gb = torch.empty_like(out), grads()
    ops.moe_block_bwd(blk, X, dOut, dXn_b, *Gb)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    for a, b, what in zip(Ga[1:], Gb[1:], ("dW1", "dW3", "dW2")):
        assert torch.equal(a, b), what
    # the router gradients pass through fp32 atomics: equal up to summation order
    torch.testing.assert_close(dXn_b.float(), dXn_a.float(), rtol=2e-2, atol=1e-3)
    torch.testing.assert_close(Gb[0].float(), Ga[0].float(), rtol=2e-2, atol=1e-3)
    # a buffer that is too small, and level NONE, are refused
    assert lib.b200_moe_block_save_activations(C.byref(blk), level, C.c_void_p(host.data_ptr()), nbytes - 1, stream) == -1
    assert lib.b200_moe_block_save_activations(C.byref(blk), NONE, C.c_void_p(host.data_ptr()), nbytes, stream) == -1
    assert lib.b200_moe_block_recompute_level(C.byref(blk), C.c_void_p(X.data_ptr()), NONE, stream) == -1
