"""CPU, world_size 2 over gloo: the expert-parallel row exchange (bookkeeping + transport) without any GPU.

Each rank builds a zone whose rows encode (source rank, global expert, index inside the expert); after `dispatch`
every rank must hold, for each of its experts, the rows of source 0 followed by the rows of source 1 in their
original order; `combine` must put every row back where it came from. Identity experts stand in for the GEMMs.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, E, d, seed, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ml_dataflow_b200.ep import RowExchange

        rng = np.random.default_rng(seed + rank)
        counts = rng.integers(0, 7, size=E).astype(np.int32)
        counts[rng.integers(0, E)] = 0  # an empty expert
        R = int(counts.sum())
        zone = torch.zeros((R, d), dtype=torch.float32)
        r = 0
        for e in range(E):
            for i in range(counts[e]):
                zone[r, 0], zone[r, 1], zone[r, 2] = rank, e, i
                r += 1
        x = RowExchange(dist, E, torch.device("cpu")).plan(torch.from_numpy(counts))
        El = E // world
        # every rank learns every rank's counts to predict what it must receive
        allc = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(allc, torch.from_numpy(counts))
        allc = torch.stack(allc).numpy()
        expect_rows = []
        for j in range(El):
            e = rank * El + j
            for s in range(world):
                expect_rows += [(s, e, i) for i in range(allc[s, e])]
        assert x.rows_recv == len(expect_rows)
        assert x.local_counts.tolist() == [int(allc[:, rank * El + j].sum()) for j in range(El)]
        assert x.local_cumsum.tolist() == np.cumsum(x.local_counts.numpy()).tolist()
        # dst_base: where THIS rank's rows of every expert start inside the owner's buffer == the owner's recv_off
        offs = [None] * world
        dist.all_gather_object(offs, x.recv_off)
        for e in range(E):
            assert int(x.dst_base[e]) == offs[e // El][rank][e % El], (rank, e)
        recv = torch.full((x.rows_recv + 3, d), -1.0)
        x.dispatch(zone, recv)
        got = [tuple(int(v) for v in recv[i, :3]) for i in range(x.rows_recv)]
        assert got == expect_rows, (rank, got[:8], expect_rows[:8])
        assert (recv[x.rows_recv:] == -1).all()
        # the peer-memory kernels address rows without any message: a routed row r of expert e sits at row
        # dst_base[e] + (r - first_row[e]) of rank e // El (csrc/ep_p2p.cu, locate()). Check that arithmetic
        # against what the message transport delivered, and the row tags the fused return path relies on:
        # tag (home rank << 40 | home row) stored at that position must name every home row exactly once.
        first_row = np.concatenate([[0], np.cumsum(counts)[:-1]])
        recvs = [None] * world
        dist.all_gather_object(recvs, recv[:x.rows_recv, :3].numpy().copy())
        tags_here = {}
        r = 0
        for e in range(E):
            for i in range(counts[e]):
                owner, row = e // El, int(x.dst_base[e]) + (r - int(first_row[e]))
                assert tuple(int(v) for v in recvs[owner][row]) == (rank, e, i)
                tags_here[(owner, row)] = (rank << 40) | r
                r += 1
        all_tags = [None] * world
        dist.all_gather_object(all_tags, tags_here)
        mine = sorted(t for tg in all_tags for (owner, _), t in tg.items() if owner == rank)
        assert len(mine) == x.rows_recv                      # every received row has a tag
        positions = sorted(row for tg in all_tags for (owner, row) in tg if owner == rank)
        assert positions == list(range(x.rows_recv))         # at distinct, dense positions
        homes = sorted((t >> 40, t & ((1 << 40) - 1)) for t in tags_here.values())
        assert homes == [(rank, i) for i in range(R)]        # and this rank's rows each get exactly one way back
        # the device-side plan (no host read of the counts) must agree with the host plan, and clip to a capacity
        y = RowExchange(dist, E, torch.device("cpu")).plan_on_device(torch.from_numpy(counts), 1 << 30)
        assert y.local_counts.tolist() == x.local_counts.tolist()
        assert y.local_cumsum.tolist() == x.local_cumsum.tolist()
        assert y.dst_base.tolist() == x.dst_base.tolist()
        assert int(y.rows_recv_dev) == x.rows_recv
        small = max(1, x.rows_recv // 2)
        z = RowExchange(dist, E, torch.device("cpu")).plan_on_device(torch.from_numpy(counts), small)
        assert int(z.rows_recv_dev) == x.rows_recv                     # the true total is still reported
        assert z.local_cumsum.tolist() == [min(c, small) for c in x.local_cumsum.tolist()]
        assert int(z.local_counts.sum()) == min(small, x.rows_recv) and (z.local_counts >= 0).all()
        # identity experts, then the way back
        back = torch.full((R, d), -5.0)
        x.combine(recv, back)
        assert torch.equal(back, zone)
        # 1-D payloads (the per-row router dot products) travel the same way
        vec = torch.arange(R, dtype=torch.float32) + 1000 * rank
        rv = torch.zeros(x.rows_recv)
        x.dispatch(vec, rv)
        bv = torch.zeros(R)
        x.combine(rv, bv)
        assert torch.equal(bv, vec)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("E,seed", [(4, 0), (16, 3)])
def test_row_exchange_two_ranks_gloo(tmp_path, E, seed):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), E, 8, seed, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
