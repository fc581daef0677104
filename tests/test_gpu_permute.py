"""GPU parity: gather, combine, per-expert variants, router_bwd_x and SwiGLU against the CPU oracle."""
import numpy as np
import pytest
import torch

from gpu_util import dev, dev_bf16, host_bits, rand_bf16, require_b200
from helpers import assert_close, bf16_bits_to_f32

pytestmark = pytest.mark.gpu


def routing(oracle, rng, T, E, k):
    logits = rng.standard_normal((T, E), dtype=np.float32)
    w, ch, counts, cexcl, _ = oracle.select_experts(logits, k)
    em, tm, cincl = oracle.build_expert_mapping(ch, E, cexcl)
    return w, ch, counts, cexcl, cincl, em, tm


@pytest.mark.parametrize("T,d,E,k", [(1, 8, 2, 1), (33, 64, 16, 2), (300, 1024, 16, 2), (257, 4096, 64, 8), (64, 8200, 8, 3)])
def test_prepare_and_merge(oracle, T, d, E, k):
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(T * 7 + d)
    w, ch, counts, cexcl, cincl, em, tm = routing(oracle, rng, T, E, k)
    X = rand_bf16(rng, (T, d))
    zone_ref = oracle.prepare_experts(X, tm)
    zone = torch.zeros((T * k, d), dtype=torch.bfloat16, device="cuda")
    ops.prepare_experts(T, d, k, dev_bf16(X), dev(tm), zone)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_bits(zone), zone_ref)  # a copy: bit-exact

    # combine with weights on top of a residual, then the un-weighted (NULL) form
    Y = rand_bf16(rng, (T * k, d))
    resid = rand_bf16(rng, (T, d))
    for weights in (w, None):
        ref = oracle.merge_experts(Y, tm, weights, resid.copy())
        out = dev_bf16(resid.copy())
        ops.merge_experts(T, d, k, dev_bf16(Y), dev(tm), None if weights is None else torch.from_numpy(weights).cuda(), out)
        torch.cuda.synchronize()
        # same fp32 operation order as the oracle -> identical up to fma contraction
        assert_close(bf16_bits_to_f32(host_bits(out)), bf16_bits_to_f32(ref), rtol=1e-2, atol=1e-3, what="merge")


@pytest.mark.parametrize("T,d,E,k", [(1, 8, 2, 1), (300, 1024, 16, 2), (257, 4096, 64, 8)])
def test_unpermute_overwrites_with_the_bits_of_merge_onto_zeros(oracle, T, d, E, k):
    """The backward's un-permute in one pass (no read of the output, no memset) against the reference's sequence:
    zero dX, merge_experts with NULL weights - bit for bit, and against the oracle."""
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(T + d)
    _, _, _, _, _, _, tm = routing(oracle, rng, T, E, k)
    dZ = rand_bf16(rng, (T * k, d))
    tmd, dZd = dev(tm), dev_bf16(dZ)
    two_pass = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    ops.merge_experts(T, d, k, dZd, tmd, None, two_pass)
    one_pass = dev_bf16(rand_bf16(rng, (T, d)))  # garbage that must not show through
    ops.unpermute_experts(T, d, k, dZd, tmd, one_pass)
    torch.cuda.synchronize()
    assert torch.equal(one_pass, two_pass)
    ref = oracle.merge_experts(dZ, tm, None, np.zeros((T, d), np.uint16))
    assert_close(bf16_bits_to_f32(host_bits(one_pass)), bf16_bits_to_f32(ref), rtol=1e-2, atol=1e-3, what="unpermute")


def test_per_expert_zone_and_merge_result(oracle):
    require_b200()
    from ml_dataflow_b200 import ops

    T, d, E, k = 200, 512, 8, 2
    rng = np.random.default_rng(5)
    w, ch, counts, cexcl, cincl, em, tm = routing(oracle, rng, T, E, k)
    X = rand_bf16(rng, (T, d))
    Xd, emd, cd, cid = dev_bf16(X), dev(em), dev(counts), dev(cincl)
    out_ref = rand_bf16(rng, (T, d))
    out = dev_bf16(out_ref.copy())
    for e in range(E):
        n = int(counts[e])
        zr = oracle.prepare_expert_zone(X, e, counts, cincl, em)
        z = torch.zeros((max(n, 1), d), dtype=torch.bfloat16, device="cuda")
        ops.prepare_expert_zone(d, Xd, e, cd, cid, emd, z)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(host_bits(z)[:n], zr)
        if n:
            oracle.merge_expert_result(zr, e, cincl, em, w, ch, out_ref)
            ops.merge_expert_result(n, d, k, z, e, cid, emd, torch.from_numpy(w).cuda(), dev(ch), out)
    torch.cuda.synchronize()
    assert_close(bf16_bits_to_f32(host_bits(out)), bf16_bits_to_f32(out_ref), rtol=1e-2, atol=1e-3, what="merge_expert_result")


def test_router_bwd_x(oracle):
    require_b200()
    from ml_dataflow_b200 import ops

    T, d, E, k = 150, 1024, 8, 2
    rng = np.random.default_rng(9)
    w, ch, counts, cexcl, cincl, em, tm = routing(oracle, rng, T, E, k)
    Y = rand_bf16(rng, (T * k, d), std=0.5)
    dOut = rand_bf16(rng, (T, d))
    dXr_ref = np.zeros((T, E), np.uint16)
    zone_ref = Y.copy()
    dXr = torch.zeros((T, E), dtype=torch.bfloat16, device="cuda")
    zone = dev_bf16(Y.copy())
    for e in range(E):
        n, b = int(counts[e]), int(cexcl[e])
        if n == 0:
            continue
        ze = np.ascontiguousarray(zone_ref[b:b + n])
        oracle.router_bwd_x(n, d, E, k, e, cincl, em, ch, w, ze, dOut, dXr_ref, ze)
        zone_ref[b:b + n] = ze
        ops.router_bwd_x(n, d, E, k, e, dev(cincl), dev(em), dev(ch), torch.from_numpy(w).cuda(), zone[b:b + n],
                         dev_bf16(dOut), dXr, zone[b:b + n])
    torch.cuda.synchronize()
    assert_close(bf16_bits_to_f32(host_bits(dXr)), bf16_bits_to_f32(dXr_ref), rtol=2e-2, atol=2e-2, what="dX_routed")
    assert_close(bf16_bits_to_f32(host_bits(zone)), bf16_bits_to_f32(zone_ref), what="scaled dOut rows")


@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 1408), (512, 1024)])
def test_swiglu_fwd_bwd(oracle, rows, cols):
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(rows + cols)
    x1, x3, dy = rand_bf16(rng, (rows, cols), 2.0), rand_bf16(rng, (rows, cols)), rand_bf16(rng, (rows, cols))
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device="cuda")
    ops.swiglu(rows, cols, dev_bf16(x1), dev_bf16(x3), out)
    d1 = torch.empty_like(out)
    d3 = torch.empty_like(out)
    ops.swiglu_bwd_x(rows, cols, dev_bf16(x1), dev_bf16(x3), dev_bf16(dy), d1, d3)
    torch.cuda.synchronize()
    assert_close(bf16_bits_to_f32(host_bits(out)), bf16_bits_to_f32(oracle.swiglu(x1, x3)), what="swiglu")
    r1, r3 = oracle.swiglu_bwd_x(x1, x3, dy)
    assert_close(bf16_bits_to_f32(host_bits(d1)), bf16_bits_to_f32(r1), what="dx1")
    assert_close(bf16_bits_to_f32(host_bits(d3)), bf16_bits_to_f32(r3), what="dx3")


def test_prepare_experts_weighted(oracle):
    """Gather with the gate weight applied: bf16(X[t,:] * w[t,j]), the row rewrite of the reference's router_bwd_x."""
    require_b200()
    from ml_dataflow_b200 import ops
    from helpers import f32_to_bf16_bits

    T, d, E, k = 123, 1032, 16, 4
    rng = np.random.default_rng(21)
    w, ch, counts, cexcl, cincl, em, tm = routing(oracle, rng, T, E, k)
    X = rand_bf16(rng, (T, d))
    ref = np.zeros((T * k, d), np.uint16)
    for t in range(T):
        for j in range(k):
            ref[tm[t, j]] = f32_to_bf16_bits(bf16_bits_to_f32(X[t]) * w[t, j])
    zone = torch.zeros((T * k, d), dtype=torch.bfloat16, device="cuda")
    ops.prepare_experts_weighted(T, d, k, dev_bf16(X), dev(tm), torch.from_numpy(w).cuda(), zone)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_bits(zone), ref)


def test_gather_combine_skewed_load_identity_experts_full_size():
    """T=65536, d=4096, 64 experts, top-8, Zipf(1.1) expert popularity, identity experts (BASELINE config 3).

    Size-independent properties: the gathered zone holds exactly the rows the mapping names (checked on sampled
    rows and through a column checksum), counts add up, the heaviest expert is several times the mean, and the
    weighted combine of the untouched zone returns every token row (gate weights sum to 1) within one bf16 ulp."""
    require_b200()
    from ml_dataflow_b200 import ops

    T, d, E, k = 65536, 4096, 64, 8
    gen = torch.Generator(device="cuda").manual_seed(0xB2000010)
    logits = torch.randn((T, E), generator=gen, device="cuda")
    rank = torch.randperm(E, generator=torch.Generator().manual_seed(0xB2000011)).float() + 1.0
    logits += torch.log(rank.pow(-1.1) / rank.pow(-1.1).sum()).cuda()[None, :]
    X = torch.randn((T, d), generator=gen, device="cuda").to(torch.bfloat16)
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    ch = torch.empty((T, k), dtype=torch.int16, device="cuda")
    counts = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    cumsum = torch.zeros(E, dtype=torch.int32, device="cuda")
    em = torch.empty(T * k, dtype=torch.int32, device="cuda")
    tm = torch.empty((T, k), dtype=torch.int32, device="cuda")
    ws = torch.empty(ops.build_expert_mapping_workspace_bytes(T, E, k), dtype=torch.uint8, device="cuda")
    ops.select_experts(T, E, k, logits, w, ch, counts, cumsum, None)
    ops.build_expert_mapping(T, E, k, ch, cumsum, em, tm, ws)
    zone = torch.empty((T * k, d), dtype=torch.bfloat16, device="cuda")
    ops.prepare_experts(T, d, k, X, tm, zone)
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    ops.merge_experts(T, d, k, zone, tm, w, out)
    torch.cuda.synchronize()

    c = counts[:E].cpu().numpy().astype(np.int64)
    assert c.sum() == T * k
    np.testing.assert_array_equal(cumsum.cpu().numpy(), np.cumsum(c))
    assert c.max() > 3 * c.mean() and c.min() < c.mean()  # the load really is skewed
    # every zone row is the row of the token expert_mapping names
    rows = torch.randint(0, T * k, (4096,), generator=torch.Generator().manual_seed(1)).cuda()
    assert torch.equal(zone[rows], X[em[rows].long()])
    # checksum over all rows: column sums of the zone == sum over tokens of k * X (fp64 on the device)
    zs = torch.zeros(d, dtype=torch.float64, device="cuda")
    for r0 in range(0, T * k, 32768):
        zs += zone[r0:r0 + 32768].double().sum(dim=0)
    xs = torch.zeros(d, dtype=torch.float64, device="cuda")
    for r0 in range(0, T, 32768):
        xs += X[r0:r0 + 32768].double().sum(dim=0) * k
    assert torch.allclose(zs, xs, rtol=0, atol=1e-6)
    # identity experts: sum_j w_j * x == x up to the rounding of the result
    xf, of = X.float(), out.float()
    assert ((of - xf).abs() <= xf.abs() * 2.0 ** -7 + 1e-30).all()
