"""GPU parity: the tcgen05 GEMM (dense matmul op in all four layouts, grouped expert GEMMs) against the oracle.

bf16 outputs are compared at 2e-2 relative / 1e-3 absolute (fp32 accumulation on both sides, different
summation order); fp32 outputs at 1e-3 / 1e-3.
"""
import numpy as np
import pytest
import torch

from gpu_util import dev, dev_bf16, host_bits, rand_bf16, require_b200
from helpers import assert_close, assert_close_with_slack, bf16_bits_to_f32

pytestmark = pytest.mark.gpu


DEFAULT_WIDE_MASK = 0  # the library default: one column tile per unit everywhere


@pytest.fixture(params=["pair", "wide", "single"], autouse=True)
def gemm_tile_mode(request):
    """Every test runs with CTA-pair tiles of one column tile per unit (cta_group::2), with CTA pairs and two column
    tiles per unit forced on for every kind of launch however small ("wide"), and with single-CTA tiles."""
    if torch.cuda.is_available():
        from ml_dataflow_b200 import ops

        ops.gemm_set_pair_mode(request.param != "single")
        ops.gemm_set_wide_mode(15 if request.param == "wide" else 0)
        yield request.param
        ops.gemm_set_pair_mode(True)
        ops.gemm_set_wide_mode(DEFAULT_WIDE_MASK)
    else:
        yield request.param


def gemm_ok(ops):
    st = ops.gemm_status()
    assert st == 0, f"a GEMM kernel gave up waiting (status {st})"


@pytest.mark.parametrize("ta,tb", [(1, 0), (0, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("M,K,N", [(64, 64, 128), (256, 128, 128), (1408, 4096, 300), (4096, 1408, 129), (72, 200, 40),
                                   (520, 264, 1000), (64, 4096, 777)])
def test_matmul_layouts(oracle, ta, tb, M, K, N):
    require_b200()
    from ml_dataflow_b200 import ops

    if tb and N % 8:
        N = (N + 7) // 8 * 8
    rng = np.random.default_rng(M + 3 * K + 7 * N + ta * 2 + tb)
    A = rand_bf16(rng, (M, K) if ta else (K, M), std=0.5)   # column-major KxM when transposed == row-major [M][K]
    B = rand_bf16(rng, (K, N) if tb else (N, K), std=0.5)
    D_ref = np.zeros((N, M), np.uint16)
    oracle.matmul(ta, tb, M, K, N, 1.0, 0.0, A, B, None, D_ref)
    D = torch.zeros((N, M), dtype=torch.bfloat16, device="cuda")
    ops.matmul(ta, tb, M, K, N, 1.0, 0.0, dev_bf16(A), dev_bf16(B), None, D)
    gemm_ok(ops)
    assert_close(bf16_bits_to_f32(host_bits(D)), bf16_bits_to_f32(D_ref), what=f"matmul ta={ta} tb={tb}")


def test_matmul_alpha_beta_inplace_and_fp32_out(oracle):
    require_b200()
    from ml_dataflow_b200 import ops

    M, K, N = 256, 320, 200
    rng = np.random.default_rng(2)
    A, B = rand_bf16(rng, (M, K), 0.3), rand_bf16(rng, (N, K), 0.3)
    C = rand_bf16(rng, (N, M))
    ref = C.copy()
    oracle.matmul(1, 0, M, K, N, 0.5, 1.0, A, B, ref, ref)
    Dd = dev_bf16(C.copy())
    ops.matmul(1, 0, M, K, N, 0.5, 1.0, dev_bf16(A), dev_bf16(B), Dd, Dd)  # C = D, beta = 1
    gemm_ok(ops)
    assert_close(bf16_bits_to_f32(host_bits(Dd)), bf16_bits_to_f32(ref), what="beta=1 in place")
    # fp32 output (the router logits form: bf16 x bf16 -> fp32)
    ref32 = np.zeros((N, M), np.float32)
    oracle.matmul(1, 0, M, K, N, 1.0, 0.0, A, B, None, ref32)
    D32 = torch.zeros((N, M), dtype=torch.float32, device="cuda")
    ops.matmul(1, 0, M, K, N, 1.0, 0.0, dev_bf16(A), dev_bf16(B), None, D32)
    gemm_ok(ops)
    assert_close(D32.cpu().numpy(), ref32, rtol=1e-3, atol=1e-3, what="fp32 out")


def test_router_gemm_shape(oracle):
    """logits[T, E] = Xn Wr^T with fp32 output at a production shape (E = 64, d = 4096)."""
    require_b200()
    from ml_dataflow_b200 import ops

    T, d, E = 1000, 4096, 64
    rng = np.random.default_rng(4)
    Xn, Wr = rand_bf16(rng, (T, d)), rand_bf16(rng, (E, d), 0.02)
    ref = oracle.linear_fwd(Xn, Wr, out_dtype=np.float32)
    out = torch.zeros((T, E), dtype=torch.float32, device="cuda")
    ops.matmul(1, 0, E, d, T, 1.0, 0.0, dev_bf16(Wr), dev_bf16(Xn), None, out)
    gemm_ok(ops)
    assert_close(out.cpu().numpy(), ref, rtol=1e-3, atol=1e-3, what="router logits")


def make_counts(rng, E, R, empty=()):
    p = rng.random(E) + 0.05
    for e in empty:
        p[e] = 0
    counts = rng.multinomial(R, p / p.sum()).astype(np.int32)
    return counts, np.cumsum(counts).astype(np.int32)


@pytest.mark.parametrize("R,d,f,E,empty", [(300, 128, 64, 4, ()), (1000, 256, 192, 8, (0, 5)), (2500, 1024, 1408, 16, (15,)),
                                           (129, 4096, 1408, 2, ())])
def test_grouped_forward(oracle, R, d, f, E, empty):
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(R + d + f)
    counts, cincl = make_counts(rng, E, R, empty)
    Z = rand_bf16(rng, (R, d))
    W1, W3, W2 = rand_bf16(rng, (E, f, d), 0.03), rand_bf16(rng, (E, f, d), 0.03), rand_bf16(rng, (E, d, f), 0.03)
    x1, x3, h = (torch.zeros((R, f), dtype=torch.bfloat16, device="cuda") for _ in range(3))
    Y = torch.zeros((R, d), dtype=torch.bfloat16, device="cuda")
    ops.moe_experts_fwd(R, d, f, E, dev_bf16(Z), dev_bf16(W1), dev_bf16(W3), dev_bf16(W2), f * d, f * d, d * f,
                        dev(counts), dev(cincl), x1, x3, h, Y)
    gemm_ok(ops)
    # each op is checked on the inputs the GPU path actually fed it, so every comparison is strict
    x1g, x3g, hg = host_bits(x1), host_bits(x3), host_bits(h)
    x1r, x3r = np.zeros((R, f), np.uint16), np.zeros((R, f), np.uint16)
    Yr = np.zeros((R, d), np.uint16)
    b = 0
    for e in range(E):
        n = int(counts[e])
        if n:
            x1r[b:b + n] = oracle.linear_fwd(Z[b:b + n], W1[e])
            x3r[b:b + n] = oracle.linear_fwd(Z[b:b + n], W3[e])
            Yr[b:b + n] = oracle.linear_fwd(np.ascontiguousarray(hg[b:b + n]), W2[e])
        b += n
    assert_close(bf16_bits_to_f32(x1g), bf16_bits_to_f32(x1r), what="x1")
    assert_close(bf16_bits_to_f32(x3g), bf16_bits_to_f32(x3r), what="x3")
    assert_close(bf16_bits_to_f32(hg), bf16_bits_to_f32(oracle.swiglu(x1g, x3g)), what="h")
    assert_close(bf16_bits_to_f32(host_bits(Y)), bf16_bits_to_f32(Yr), what="Y")


@pytest.mark.parametrize("R,d,f,E,empty", [(300, 128, 64, 4, ()), (1000, 256, 192, 8, (2,)), (2500, 1024, 1408, 16, (0, 15))])
def test_grouped_backward(oracle, R, d, f, E, empty):
    """bwd_x + bwd_w against the oracle ops chained in the reference's order (with Y recomputed for dP)."""
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(R * 3 + d + f)
    counts, cincl = make_counts(rng, E, R, empty)
    dOutRows = rand_bf16(rng, (R, d))            # upstream gradient rows, already in expert order
    Zx = rand_bf16(rng, (R, d))
    roww = (rng.random(R, dtype=np.float32) * 0.5 + 0.05).astype(np.float32)
    from helpers import f32_to_bf16_bits
    dYs = f32_to_bf16_bits(bf16_bits_to_f32(dOutRows) * roww[:, None])  # what router_bwd_x leaves in the zone
    x1, x3 = rand_bf16(rng, (R, f)), rand_bf16(rng, (R, f))
    W1, W3, W2 = rand_bf16(rng, (E, f, d), 0.03), rand_bf16(rng, (E, f, d), 0.03), rand_bf16(rng, (E, d, f), 0.03)
    g1, g3, g2 = rand_bf16(rng, (E, f, d), 0.1), rand_bf16(rng, (E, f, d), 0.1), rand_bf16(rng, (E, d, f), 0.1)

    hr = oracle.swiglu(x1, x3)
    dx1, dx3, hs = (torch.zeros((R, f), dtype=torch.bfloat16, device="cuda") for _ in range(3))
    dZ = torch.zeros((R, d), dtype=torch.bfloat16, device="cuda")
    dP = torch.zeros(R, dtype=torch.float32, device="cuda")
    dYd, Zxd, cd, cid = dev_bf16(dYs), dev_bf16(Zx), dev(counts), dev(cincl)
    W1d, W3d, W2d = dev_bf16(W1), dev_bf16(W3), dev_bf16(W2)
    ops.moe_experts_bwd_x(R, d, f, E, dYd, torch.from_numpy(roww).cuda(), dev_bf16(x1), dev_bf16(x3), W1d, W3d, W2d,
                          f * d, f * d, d * f, cd, cid, dx1, dx3, hs, dP, dZ)
    G1, G3, G2 = dev_bf16(g1), dev_bf16(g3), dev_bf16(g2)
    ops.moe_experts_bwd_w(R, d, f, E, dYd, hs, Zxd, dx1, dx3, G1, G3, G2, f * d, f * d, d * f, cd, cid)
    gemm_ok(ops)
    dx1g, dx3g, hsg = host_bits(dx1), host_bits(dx3), host_bits(hs)

    # oracle, op by op, every op on the inputs the GPU op consumed
    dx1r, dx3r = np.zeros((R, f), np.uint16), np.zeros((R, f), np.uint16)
    dZr, dz1 = np.zeros((R, d), np.uint16), np.zeros((R, d), np.uint16)
    dPr = np.zeros(R, np.float32)
    g1r, g3r, g2r = g1.copy(), g3.copy(), g2.copy()
    b = 0
    for e in range(E):
        n = int(counts[e])
        if n:
            sl = slice(b, b + n)
            y = oracle.linear_fwd(hr[sl], W2[e])
            dPr[sl] = (bf16_bits_to_f32(y) * bf16_bits_to_f32(dOutRows[sl])).sum(axis=1)
            oracle.linear_wgrad(np.ascontiguousarray(hsg[sl]), dYs[sl], g2r[e])
            dh = oracle.linear_dgrad(dYs[sl], W2[e])
            dx1r[sl], dx3r[sl] = oracle.swiglu_bwd_x(x1[sl], x3[sl], dh)
            dz = oracle.linear_dgrad(np.ascontiguousarray(dx1g[sl]), W1[e])
            dz1[sl] = dz
            dZr[sl] = oracle.linear_dgrad(np.ascontiguousarray(dx3g[sl]), W3[e], accumulate_into=dz)
            oracle.linear_wgrad(Zx[sl], np.ascontiguousarray(dx1g[sl]), g1r[e])
            oracle.linear_wgrad(Zx[sl], np.ascontiguousarray(dx3g[sl]), g3r[e])
        b += n
    f32 = bf16_bits_to_f32
    assert_close(dP.cpu().numpy(), dPr, rtol=2e-2, atol=2e-2 * float(np.abs(dPr).mean() + 1e-6), what="dP")
    assert_close(f32(host_bits(hs)), f32(hr), what="hs")
    assert_close(f32(dx1g), f32(dx1r), what="dx1")  # differs from the oracle only through one rounding of dh
    assert_close(f32(dx3g), f32(dx3r), what="dx3")
    # the kernel adds dx1 W1 and dx3 W3 in one fp32 accumulator; the reference rounds the first product to bf16
    # before adding the second (two GEMM calls, beta = 1): allow one bf16 ulp of that intermediate
    assert_close_with_slack(f32(host_bits(dZ)), f32(dZr), np.abs(f32(dz1)) * 2.0 ** -8, what="dZ")
    assert_close(f32(host_bits(G2)), f32(g2r), what="dW2")
    assert_close(f32(host_bits(G1)), f32(g1r), what="dW1")
    assert_close(f32(host_bits(G3)), f32(g3r), what="dW3")


def _tags(rank_of_row, dest_row):
    return torch.from_numpy((rank_of_row.astype(np.int64) << 40) | dest_row.astype(np.int64)).cuda()


@pytest.mark.parametrize("R,d,f,E", [(700, 256, 192, 4), (2100, 1024, 1408, 8), (3000, 128, 64, 200)])
def test_grouped_scatter_forms_match_in_place_forms(R, d, f, E):
    """The *_scatter entry points store Y / dZ rows where their tags say (two destination buffers standing in for two
    ranks); values must be bit-identical to the in-place entry points."""
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(R + 7)
    counts, cincl = make_counts(rng, E, R, (1,))
    Z, dYs = dev_bf16(rand_bf16(rng, (R, d))), dev_bf16(rand_bf16(rng, (R, d)))
    W1, W3, W2 = (dev_bf16(rand_bf16(rng, s, 0.03)) for s in ((E, f, d), (E, f, d), (E, d, f)))
    cd, cid = dev(counts), dev(cincl)
    ones = torch.ones(R, dtype=torch.float32, device="cuda")
    x1, x3, h, dx1, dx3 = (torch.zeros((R, f), dtype=torch.bfloat16, device="cuda") for _ in range(5))
    Y, dZ = (torch.zeros((R, d), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    dP = torch.zeros(R, dtype=torch.float32, device="cuda")
    ops.moe_experts_fwd(R, d, f, E, Z, W1, W3, W2, f * d, f * d, d * f, cd, cid, x1, x3, h, Y)
    ops.moe_experts_bwd_x(R, d, f, E, dYs, ones, x1, x3, W1, W3, W2, f * d, f * d, d * f, cd, cid, dx1, dx3, None, dP, dZ)

    # a random permutation of the rows over two buffers
    perm = rng.permutation(R)
    half = (R + 1) // 2
    rank_of_row, dest_row = (perm >= half).astype(np.int64), np.where(perm >= half, perm - half, perm)
    tags = _tags(rank_of_row, dest_row)
    bufs = [torch.full((half, d), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    ptrs = [b.data_ptr() for b in bufs]
    x1b, x3b, hb = (torch.zeros_like(x1) for _ in range(3))
    ops.moe_experts_fwd_scatter(R, d, f, E, Z, W1, W3, W2, f * d, f * d, d * f, cd, cid, x1b, x3b, hb, tags, ptrs, half)
    gemm_ok(ops)
    got = torch.cat(bufs)[torch.from_numpy(perm).cuda()]
    assert torch.equal(got.view(torch.int16), Y.view(torch.int16))
    assert torch.equal(hb.view(torch.int16), h.view(torch.int16))

    for b in bufs:
        b.fill_(7.0)
    dPb = torch.zeros_like(dP)
    dx1b, dx3b = torch.zeros_like(dx1), torch.zeros_like(dx3)
    ops.moe_experts_bwd_x_scatter(R, d, f, E, dYs, ones, x1, x3, W1, W3, W2, f * d, f * d, d * f, cd, cid, dx1b, dx3b,
                                  None, dPb, tags, ptrs, half)
    gemm_ok(ops)
    got = torch.cat(bufs)[torch.from_numpy(perm).cuda()]
    assert torch.equal(got.view(torch.int16), dZ.view(torch.int16))
    assert torch.equal(dx1b.view(torch.int16), dx1.view(torch.int16))


def test_scatter_refuses_a_tag_outside_the_destination():
    """A tag naming a rank or a row outside the destination buffers is not stored; the status word reports it."""
    require_b200()
    from ml_dataflow_b200 import ops

    R, d, f, E = 300, 128, 64, 2
    rng = np.random.default_rng(5)
    counts, cincl = make_counts(rng, E, R)
    Z = dev_bf16(rand_bf16(rng, (R, d)))
    W1, W3, W2 = (dev_bf16(rand_bf16(rng, s, 0.03)) for s in ((E, f, d), (E, f, d), (E, d, f)))
    x1, x3, h = (torch.zeros((R, f), dtype=torch.bfloat16, device="cuda") for _ in range(3))
    rank_of_row, dest_row = np.zeros(R, np.int64), np.arange(R, dtype=np.int64)
    rank_of_row[10] = 3          # only one destination buffer is given
    dest_row[20] = R + 5         # past the end of the buffer
    guard = torch.full((R + 64, d), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.moe_experts_fwd_scatter(R, d, f, E, Z, W1, W3, W2, f * d, f * d, d * f, dev(counts), dev(cincl), x1, x3, h,
                                _tags(rank_of_row, dest_row), [guard.data_ptr()], R)
    assert ops.gemm_status() == 5
    assert ops.gemm_status() == 0  # reading clears it
    g = guard.float().cpu().numpy()
    assert (g[10] == 7.0).all() and (g[20] == 7.0).all() and (g[R:] == 7.0).all()
    assert (g[11] != 7.0).any()


def test_grouped_ops_on_the_reference_packed_expert_layout():
    """The reference stores an expert's w1, w3, w2 back to back (prep_transformer.c:155-159), so each of the three
    weight arrays is addressed as base + e * (3 f d). Forward, backward-x and backward-w on that layout must give the
    bits they give on three separate arrays."""
    require_b200()
    from ml_dataflow_b200 import ops

    R, d, f, E = 1500, 512, 320, 6
    rng = np.random.default_rng(77)
    counts, cincl = make_counts(rng, E, R, (3,))
    Z, dYs = dev_bf16(rand_bf16(rng, (R, d))), dev_bf16(rand_bf16(rng, (R, d)))
    W1, W3, W2 = (dev_bf16(rand_bf16(rng, s, 0.03)) for s in ((E, f, d), (E, f, d), (E, d, f)))
    packed = torch.cat([W1.reshape(E, -1), W3.reshape(E, -1), W2.reshape(E, -1)], dim=1).contiguous()
    stride = 3 * f * d
    P1, P3, P2 = packed[0, 0:], packed[0, f * d:], packed[0, 2 * f * d:]  # views: only their addresses are used
    gpacked = torch.zeros_like(packed)
    Q1, Q3, Q2 = gpacked[0, 0:], gpacked[0, f * d:], gpacked[0, 2 * f * d:]
    cd, cid = dev(counts), dev(cincl)
    ones = torch.ones(R, dtype=torch.float32, device="cuda")

    def run(w1, w3, w2, s1, s3, s2, g1, g3, g2):
        x1, x3, h, dx1, dx3, hs = (torch.zeros((R, f), dtype=torch.bfloat16, device="cuda") for _ in range(6))
        Y, dZ = (torch.zeros((R, d), dtype=torch.bfloat16, device="cuda") for _ in range(2))
        dP = torch.zeros(R, dtype=torch.float32, device="cuda")
        ops.moe_experts_fwd(R, d, f, E, Z, w1, w3, w2, s1, s3, s2, cd, cid, x1, x3, h, Y)
        ops.moe_experts_bwd_x(R, d, f, E, dYs, ones, x1, x3, w1, w3, w2, s1, s3, s2, cd, cid, dx1, dx3, hs, dP, dZ)
        ops.moe_experts_bwd_w(R, d, f, E, dYs, hs, Z, dx1, dx3, g1, g3, g2, s1, s3, s2, cd, cid)
        gemm_ok(ops)
        return Y, dZ

    G1, G3, G2 = torch.zeros_like(W1), torch.zeros_like(W3), torch.zeros_like(W2)
    Ya, dZa = run(W1, W3, W2, f * d, f * d, d * f, G1, G3, G2)
    Yb, dZb = run(P1, P3, P2, stride, stride, stride, Q1, Q3, Q2)
    eq = lambda a, b: torch.equal(a.contiguous().view(torch.int16), b.contiguous().view(torch.int16))
    assert eq(Ya, Yb) and eq(dZa, dZb)
    assert eq(gpacked[:, :f * d], G1.reshape(E, -1))
    assert eq(gpacked[:, f * d:2 * f * d], G3.reshape(E, -1))
    assert eq(gpacked[:, 2 * f * d:], G2.reshape(E, -1))


@pytest.mark.parametrize("ta,tb", [(1, 0), (0, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("M,K,N,d_fp32", [(64, 4096, 1024, True), (4096, 8192, 64, False), (256, 5000 // 8 * 8, 264, False)])
def test_matmul_with_split_reduction(oracle, ta, tb, M, K, N, d_fp32):
    """Few output tiles + long reduction + a workspace: the reduction is split over the SMs and summed by a second
    kernel. Same answer as the oracle (router logits and router weight-gradient shapes among the cases), also with
    alpha, beta and C aliasing D, and the same bits on a second run (the partial sums are added in a fixed order)."""
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(M + K + N + 2 * ta + tb)
    A = rand_bf16(rng, (M, K) if ta else (K, M), std=0.5)
    B = rand_bf16(rng, (K, N) if tb else (N, K), std=0.5)
    ws = torch.empty(16 << 20, dtype=torch.uint8, device="cuda")
    Ad, Bd = dev_bf16(A), dev_bf16(B)
    if d_fp32:
        D_ref = np.zeros((N, M), np.float32)
        oracle.matmul(ta, tb, M, K, N, 1.0, 0.0, A, B, None, D_ref)
        D = torch.zeros((N, M), dtype=torch.float32, device="cuda")
        ops.matmul(ta, tb, M, K, N, 1.0, 0.0, Ad, Bd, None, D, ws)
        gemm_ok(ops)
        assert_close(D.cpu().numpy(), D_ref, rtol=1e-3, atol=1e-3 * np.sqrt(K) * 0.25, what="split-k fp32")
        return
    C0 = rand_bf16(rng, (N, M), std=2.0)
    D_ref = C0.copy()
    oracle.matmul(ta, tb, M, K, N, 0.5, 1.0, A, B, C0, D_ref)
    D = dev_bf16(C0.copy())
    ops.matmul(ta, tb, M, K, N, 0.5, 1.0, Ad, Bd, D, D, ws)     # C aliases D
    gemm_ok(ops)
    assert_close(bf16_bits_to_f32(host_bits(D)), bf16_bits_to_f32(D_ref), what=f"split-k ta={ta} tb={tb}")
    D2 = dev_bf16(C0.copy())
    ops.matmul(ta, tb, M, K, N, 0.5, 1.0, Ad, Bd, D2, D2, ws)
    assert torch.equal(D.view(torch.int16), D2.view(torch.int16))
    # without a workspace the plain form runs and agrees to rounding
    D3 = dev_bf16(C0.copy())
    ops.matmul(ta, tb, M, K, N, 0.5, 1.0, Ad, Bd, D3, D3)
    gemm_ok(ops)
    assert_close(bf16_bits_to_f32(host_bits(D3)), bf16_bits_to_f32(host_bits(D)), what="split vs plain")


def test_weight_gradients_at_every_kind_of_reduction_tail(oracle):
    """Per-expert row counts chosen to end a reduction slab at every interesting place: empty, a single row, one short
    of / exactly / one past a 16-row group and a 64-row slab, two slabs (one pipeline stage) and a bit more. The rows
    of the next expert that share the last slab must not leak into the gradient."""
    require_b200()
    from ml_dataflow_b200 import ops

    counts = np.array([0, 1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 0, 200, 3], np.int32)
    E, R = len(counts), int(counts.sum())
    cincl = np.cumsum(counts).astype(np.int32)
    d, f = 256, 320
    rng = np.random.default_rng(4242)
    dY, Z = rand_bf16(rng, (R, d), 2.0), rand_bf16(rng, (R, d), 2.0)
    hs, dx1, dx3 = rand_bf16(rng, (R, f), 2.0), rand_bf16(rng, (R, f), 2.0), rand_bf16(rng, (R, f), 2.0)
    g1, g3, g2 = rand_bf16(rng, (E, f, d), 0.1), rand_bf16(rng, (E, f, d), 0.1), rand_bf16(rng, (E, d, f), 0.1)
    G1, G3, G2 = dev_bf16(g1.copy()), dev_bf16(g3.copy()), dev_bf16(g2.copy())
    ops.moe_experts_bwd_w(R, d, f, E, dev_bf16(dY), dev_bf16(hs), dev_bf16(Z), dev_bf16(dx1), dev_bf16(dx3), G1, G3, G2,
                          f * d, f * d, d * f, dev(counts), dev(cincl))
    gemm_ok(ops)
    b = 0
    for e in range(E):
        n = int(counts[e])
        sl = slice(b, b + n)
        if n:
            oracle.linear_wgrad(np.ascontiguousarray(hs[sl]), np.ascontiguousarray(dY[sl]), g2[e])
            oracle.linear_wgrad(np.ascontiguousarray(Z[sl]), np.ascontiguousarray(dx1[sl]), g1[e])
            oracle.linear_wgrad(np.ascontiguousarray(Z[sl]), np.ascontiguousarray(dx3[sl]), g3[e])
        b += n
    for got, ref, what in ((G1, g1, "dW1"), (G3, g3, "dW3"), (G2, g2, "dW2")):
        gb = host_bits(got)
        for e in range(E):
            if counts[e] == 0:
                np.testing.assert_array_equal(gb[e], ref[e], err_msg=f"{what}[{e}] of an empty expert changed")
            else:
                assert_close(bf16_bits_to_f32(gb[e]), bf16_bits_to_f32(ref[e]), what=f"{what}[{e}] ({counts[e]} rows)")
