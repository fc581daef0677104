"""GPU, one device: the small kernels of the C expert-parallel driver (csrc/ep_block.cu) with the "ranks" emulated
as buffers of one GPU. No kernel here waits on another launch: the barrier kernel is only run (a) with world 1,
where its own store satisfies its wait, and (b) against a flag that nothing sets and a limit of 20 ms, where it must
give up, report status 1 and leave the device usable.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _setup():
    import torch

    from gpu_util import require_b200

    require_b200()
    from ml_dataflow_b200 import _lib, ops

    return torch, _lib.load(), ops


def _table(ptrs):
    return (C.c_ulonglong * len(ptrs))(*ptrs)


def _stream(torch):
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_plan_kernel_matches_the_host_plan():
    torch, lib, ops = _setup()
    rng = np.random.default_rng(3)
    for world, El, cap in [(2, 4, 10 ** 6), (8, 8, 10 ** 6), (4, 3, 500), (1, 16, 10 ** 6)]:
        E = world * El
        counts = rng.integers(0, 200, size=(world, E)).astype(np.int32)  # [source][global expert]
        g = torch.from_numpy(counts).cuda()
        for rank in range(world):
            lc, lcs = (torch.full((El,), -1, dtype=torch.int32, device="cuda") for _ in range(2))
            db = torch.full((E,), -1, dtype=torch.int32, device="cuda")
            ov = torch.zeros(1, dtype=torch.int32, device="cuda")
            assert lib.b200_ep_plan(C.c_void_p(g.data_ptr()), world, rank, El, cap, C.c_void_p(lc.data_ptr()),
                                    C.c_void_p(lcs.data_ptr()), C.c_void_p(db.data_ptr()), C.c_void_p(ov.data_ptr()),
                                    _stream(torch)) == 0
            a = counts.astype(np.int64).reshape(world, world, El)  # [source][owner][local expert]
            per_expert = a[:, rank, :].sum(axis=0)
            cum = np.minimum(np.cumsum(per_expert), cap)
            np.testing.assert_array_equal(lcs.cpu().numpy(), cum)
            np.testing.assert_array_equal(lc.cpu().numpy(), np.diff(np.concatenate([[0], cum])))
            per_owner = a.sum(axis=0)
            owner_base = np.cumsum(per_owner, axis=1) - per_owner
            before_me = a[:rank].sum(axis=0)
            np.testing.assert_array_equal(db.cpu().numpy(), (owner_base + before_me).reshape(-1))
            assert int(ov.item()) == int(per_expert.sum() > cap)


def test_router_gradient_sum_in_rank_order():
    torch, lib, ops = _setup()
    world, n = 4, 64 * 256
    parts = [torch.randn(n, device="cuda").to(torch.bfloat16) for _ in range(world)]
    dWr = torch.randn(n, device="cuda").to(torch.bfloat16)
    ref = dWr.float()
    for p in parts:
        ref = ref + p.float()
    tab = _table([p.data_ptr() for p in parts])
    assert lib.b200_ep_reduce_router_grad(tab, world, n, C.c_void_p(dWr.data_ptr()), _stream(torch)) == 0
    assert torch.equal(dWr, ref.to(torch.bfloat16))
    assert lib.b200_ep_reduce_router_grad(tab, world, n + 4, C.c_void_p(dWr.data_ptr()), _stream(torch)) == -1


def test_barrier_alone_and_payload():
    torch, lib, ops = _setup()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    mine = torch.arange(9, dtype=torch.int32, device="cuda")
    got = torch.zeros(9, dtype=torch.int32, device="cuda")
    for i in range(3):
        assert lib.b200_ep_barrier(_table([flags.data_ptr()]), 1, 0, C.c_void_p(epoch.data_ptr()),
                                   C.c_void_p(mine.data_ptr()), 9, _table([got.data_ptr()]), _stream(torch)) == 0
    assert ops.ep_status() == 0
    assert int(epoch.item()) == 3 and int(flags[0].item()) == 3 and torch.equal(got, mine)


def test_barrier_gives_up_when_a_rank_never_arrives():
    torch, lib, ops = _setup()
    # "rank 1" is a second flag array on this GPU that nothing ever writes into rank 0's slot 1 for
    mine = torch.zeros(4, dtype=torch.int32, device="cuda")
    other = torch.zeros(4, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.b200_ep_set_barrier_timeout_ms(20) == 0
    try:
        assert lib.b200_ep_barrier(_table([mine.data_ptr(), other.data_ptr()]), 2, 0, C.c_void_p(epoch.data_ptr()), None,
                                   0, None, _stream(torch)) == 0
        assert ops.ep_status() == 1   # synchronises: the kernel returned on its own
        assert ops.ep_status() == 0   # reading clears it
        assert int(other[0].item()) == 1 and int(mine[0].item()) == 1 and int(mine[1].item()) == 0
        # the device is still usable
        assert int((torch.ones(8, device="cuda") * 2).sum().item()) == 16
    finally:
        lib.b200_ep_set_barrier_timeout_ms(2000)
