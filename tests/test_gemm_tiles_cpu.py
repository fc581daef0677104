"""CPU: the GEMM kernels' tile scheduler, run on the host through b200_gemm_enumerate_tiles (the same Sched code the
device executes). Every output element must belong to exactly one tile, tiles must stay inside their expert, the
loaded width must cover the valid width in the granule the TMA boxes need, and reduction ranges must partition the
reduction."""
import ctypes

import numpy as np
import pytest

DENSE, GROUPED_M, GROUPED_K = 0, 1, 2


def tiles(mode, pair, M, N, K, dual_b=0, counts=None, splits=0, split_len=0):
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    G = 1 if counts is None else len(counts)
    c = None if counts is None else np.ascontiguousarray(counts, np.int32)
    ci = None if counts is None else np.cumsum(c).astype(np.int32)
    cap = 1 << 16  # pair: 0 = single-CTA tiles, 1 = CTA pairs, 2 = CTA pairs with two column tiles per unit
    out = np.zeros((cap, 9), np.int32)
    p = lambda a: None if a is None else a.ctypes.data_as(ctypes.c_void_p)
    n = lib.b200_gemm_enumerate_tiles(mode, pair, M, N, K, dual_b, G, p(c), p(ci), splits, split_len, cap, p(out))
    assert 0 <= n <= cap
    return out[:n]


@pytest.mark.parametrize("pair", [0, 1, 2])
@pytest.mark.parametrize("N,dual_b", [(1408, 1), (4096, 0), (1408, 0), (72, 0), (200, 1)])
def test_row_grouped_tiles_cover_every_expert_exactly(pair, N, dual_b):
    rng = np.random.default_rng(N + pair)
    counts = rng.integers(0, 700, size=12).astype(np.int32)
    counts[[2, 7]] = 0
    counts[3], counts[4], counts[5] = 1, 128, 257
    K = 512
    t = tiles(GROUPED_M, pair, 0, N, K, dual_b, counts)
    tile_rows = 256 if pair else 128
    width = 128 if dual_b else 256
    granule = 128 if (pair and not dual_b) else 64
    base = np.concatenate([[0], np.cumsum(counts)[:-1]])
    cover = np.zeros((int(counts.sum()), N), np.int16)
    for g, a0, o0, mv, n0, nv, nw, k0, kl in t:
        assert a0 == o0 and 0 < mv <= tile_rows and 0 < nv <= width
        assert base[g] <= o0 and o0 + mv <= base[g] + counts[g]          # never into a neighbour's rows
        assert (o0 - base[g]) % tile_rows == 0 and n0 % width == 0
        assert nw >= nv and nw % granule == 0 and nw - nv < granule and nw <= (256 if not dual_b else 128)
        assert k0 == 0 and kl == K
        cover[o0:o0 + mv, n0:n0 + nv] += 1
    assert (cover == 1).all()
    # processing order: column tiles of one row tile are adjacent (they share the A rows in L2)
    key = [(int(r[2]), int(r[4])) for r in t]
    assert key == sorted(key)


@pytest.mark.parametrize("pair", [0, 1, 2])
def test_reduction_grouped_tiles(pair):
    counts = np.array([0, 1, 63, 64, 65, 130, 0, 1000], np.int32)
    M, N = 1408, 4096
    t = tiles(GROUPED_K, pair, M, N, 0, 0, counts)
    tile_rows = 256 if pair else 128
    base = np.concatenate([[0], np.cumsum(counts)[:-1]])
    per = -(-M // tile_rows) * -(-N // 256)
    assert len(t) == len(counts) * per          # empty experts keep their tiles (the kernel skips k_len == 0)
    for e in range(len(counts)):
        te = t[e * per:(e + 1) * per]
        assert (te[:, 0] == e).all() and (te[:, 7] == base[e]).all() and (te[:, 8] == counts[e]).all()
        cover = np.zeros((M, N), np.int16)
        for g, a0, o0, mv, n0, nv, nw, k0, kl in te:
            cover[o0:o0 + mv, n0:n0 + nv] += 1
        assert (cover == 1).all()


@pytest.mark.parametrize("pair", [0, 1, 2])
@pytest.mark.parametrize("K,splits,split_len", [(8192, 8, 1024), (5000, 4, 1280), (4096, 0, 0)])
def test_dense_tiles_and_split_reduction(pair, K, splits, split_len):
    M, N = 300, 520          # output rows, output columns in the kernel's row-major view
    t = tiles(DENSE, pair, M, N, K, 0, None, splits, split_len)
    parts = max(1, splits)
    cover = np.zeros((parts, M, N), np.int16)
    for g, a0, o0, mv, n0, nv, nw, k0, kl in t:
        assert 0 <= g < parts
        if splits:
            assert k0 == g * split_len and k0 % 64 == 0 and kl == min(split_len, K - k0) and kl > 0
        else:
            assert k0 == 0 and kl == K
        cover[g, o0:o0 + mv, n0:n0 + nv] += 1
    assert (cover == 1).all()
    if splits:
        ranges = sorted({(int(r[7]), int(r[8])) for r in t})
        assert ranges[0][0] == 0 and ranges[-1][0] + ranges[-1][1] == K
        assert all(a[0] + a[1] == b[0] for a, b in zip(ranges[:-1], ranges[1:]))   # the ranges partition [0, K)


def test_bad_arguments_are_refused():
    from ml_dataflow_b200 import _lib

    out = np.zeros(9, np.int32)
    assert _lib.load().b200_gemm_enumerate_tiles(7, 0, 1, 1, 1, 0, 1, None, None, 0, 0, 1,
                                                 out.ctypes.data_as(ctypes.c_void_p)) == -1
    assert _lib.load().b200_gemm_enumerate_tiles(GROUPED_M, 0, 1, 1, 1, 0, 4, None, None, 0, 0, 1,
                                                 out.ctypes.data_as(ctypes.c_void_p)) == -1
