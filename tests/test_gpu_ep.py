"""GPU, 2 ranks over NCCL: the expert-parallel layer against the single-GPU CPU oracle on every rank's tokens.

Tokens are independent, so rank r's outputs (out, dXn) must equal the oracle's single-GPU layer on rank r's batch
with all experts; the expert weight gradients on the owning rank must equal the sum of the oracle's gradients over
all ranks' batches; the per-expert row counts seen by the owner must equal the sum of the ranks' counts (bit-exact).
All transports are covered: expert outputs stored into the home rank's buffer by the GEMM epilogue ("fused"), rows
written / read directly in the owner's NVLink-mapped buffer ("p2p") and rows moved by NCCL point-to-point batches
("nccl"). Two steps are run so that buffer reuse across steps is exercised.
Skipped on a box with fewer than two GPUs.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir, transport):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from ep_parity import check_expert_parallel

        check_expert_parallel(dist, rank, world, transport)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _overflow_worker(rank, world, port, result_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sys
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from gpu_util import dev_bf16, rand_bf16
        from ml_dataflow_b200.ep import ExpertParallelMoELayer

        T, d, E, k, f = 384, 256, 8, 2, 128
        El = E // world
        rng = np.random.default_rng(5 + rank)
        X, dOut = dev_bf16(rand_bf16(rng, (T, d))), dev_bf16(rand_bf16(rng, (T, d)))
        wr = np.random.default_rng(1)
        Wr = dev_bf16(rand_bf16(wr, (E, d), 0.06))
        W1, W3 = (dev_bf16(rand_bf16(rng, (El, f, d), 0.06)) for _ in range(2))
        W2 = dev_bf16(rand_bf16(rng, (El, d, f), 0.06))
        # receive buffers of 64 rows where about 768 arrive: the step must run to the end, touch nothing outside
        # its buffers, and report the overflow when asked
        layer = ExpertParallelMoELayer(T, d, E, k, f, dist, device=torch.device("cuda", rank), transport="fused",
                                       recv_capacity_factor=0.0)
        assert layer.cap < 400
        out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
        dXn = torch.empty_like(out)
        dWr = torch.zeros((E, d), dtype=torch.bfloat16, device="cuda")
        dW1, dW3 = (torch.zeros((El, f, d), dtype=torch.bfloat16, device="cuda") for _ in range(2))
        dW2 = torch.zeros((El, d, f), dtype=torch.bfloat16, device="cuda")
        layer.forward(X, Wr, W1, W3, W2, out)
        layer.backward(X, Wr, W1, W3, W2, dOut, dXn, dWr, dW1, dW3, dW2)
        torch.cuda.synchronize()
        assert int(layer.x.local_counts.sum()) <= layer.cap
        raised = False
        try:
            layer.check()
        except RuntimeError as e:
            raised = "too small" in str(e)
        assert raised
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_receive_buffer_overflow_is_reported_not_overrun(tmp_path):
    """A failure made on the host side (buffers sized far too small): rows that do not fit are dropped by the senders
    and by the clipped counts, the kernels stay inside their buffers, `check()` raises."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_overflow_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


@pytest.mark.parametrize("transport", ["fused", "p2p", "nccl", "c"])
def test_expert_parallel_two_ranks(tmp_path, transport):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), transport), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
