"""GPU parity of the whole MoE layer (forward + backward) against the CPU oracle and the golden fixtures.

Routing is bit-exact given the same logits, so each test feeds the oracle the fp32 logits the GPU router GEMM
produced (compared separately at 1e-3) and then demands: identical chosen experts / counts / cumsums / mappings,
and every op's bf16 output within 2e-2 relative + 1e-3 absolute of the oracle op applied to the same inputs. The
end-to-end chain (GPU chain vs oracle chain) is additionally held to a relative Frobenius error, because bf16
values that round the other way early in a chain move later sums by more than the element-wise bound near zero.
"""
import os

import numpy as np
import pytest
import torch

from gpu_util import dev_bf16, host_bits, host_u16, rand_bf16, require_b200
from helpers import assert_close, assert_close_with_slack, bf16_bits_to_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["pair", "single"], autouse=True)
def gemm_tile_mode(request):
    """Every test runs with CTA-pair tiles (cta_group::2, the default) and with single-CTA tiles."""
    if torch.cuda.is_available():
        from ml_dataflow_b200 import ops

        ops.gemm_set_pair_mode(request.param == "pair")
        yield request.param
        ops.gemm_set_pair_mode(True)
    else:
        yield request.param
GOLD = os.path.join(os.path.dirname(__file__), "golden")
f32 = bf16_bits_to_f32


def run_layer(path, T, d, E, k, f, X, Wr, W1, W3, W2, dOut, g0, logits=None):
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    layer = MoELayer(T, d, E, k, f)
    layer.keep_pre_gate = True
    Xd, Wrd, W1d, W3d, W2d, dOd = (dev_bf16(a) for a in (X, Wr, W1, W3, W2, dOut))
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    dXn = torch.empty((T, d), dtype=torch.bfloat16, device="cuda")
    G = {n: dev_bf16(g0[n].copy()) for n in ("dWr", "dW1", "dW3", "dW2")}
    lg = None if logits is None else torch.from_numpy(logits).cuda()
    if path == "fast":
        layer.forward(Xd, Wrd, W1d, W3d, W2d, out, logits=lg)
        layer.backward(Xd, Wrd, W1d, W3d, W2d, dOd, dXn, G["dWr"], G["dW1"], G["dW3"], G["dW2"])
    else:
        layer.forward_reference_order(Xd, Wrd, W1d, W3d, W2d, out, logits=lg)
        layer.backward_reference_order(Xd, Wrd, W1d, W3d, W2d, dOd, dXn, G["dWr"], G["dW1"], G["dW3"], G["dW2"])
    st = ops.gemm_status()
    assert st == 0, f"GEMM status {st}"
    return layer, out, dXn, G


def compare_with_oracle(oracle, layer, out, dXn, G, X, Wr, W1, W3, W2, dOut, g0, k, path):
    """Every op against the oracle on the inputs the GPU op consumed (element-wise, strict), then the whole chain
    against the oracle's own chain (relative Frobenius error)."""
    from helpers import assert_chain_close, f32_to_bf16_bits

    T, d = X.shape
    E, f = W1.shape[0], W1.shape[1]
    logits = layer.logits.cpu().numpy()
    assert_close(logits, oracle.linear_fwd(X, Wr, out_dtype=np.float32), rtol=1e-3, atol=1e-3, what="router logits")
    fwd = oracle.moe_forward(X, Wr, W1, W3, W2, k, logits=logits)
    # ---- integers: bit-exact
    np.testing.assert_array_equal(host_u16(layer.chosen), fwd["chosen"])
    np.testing.assert_array_equal(layer.counts.cpu().numpy()[:E], fwd["counts"][:E])
    np.testing.assert_array_equal(layer.cumsum.cpu().numpy(), fwd["cumsum_incl"])
    np.testing.assert_array_equal(layer.token_mapping.cpu().numpy(), fwd["token_mapping"])
    np.testing.assert_array_equal(layer.expert_mapping.cpu().numpy(), fwd["expert_mapping"])
    np.testing.assert_allclose(layer.weights.cpu().numpy(), fwd["weights"], rtol=1e-5, atol=1e-7)
    np.testing.assert_array_equal(host_bits(layer.zone), fwd["zone"])
    # ---- forward ops
    x1g, x3g, hg, Yg = (host_bits(getattr(layer, n)) for n in ("x1", "x3", "h", "Y"))
    assert_close(f32(x1g), f32(fwd["x1"]), what="x1")
    assert_close(f32(x3g), f32(fwd["x3"]), what="x3")
    assert_close(f32(hg), f32(oracle.swiglu(x1g, x3g)), what="h")
    cnt, base = fwd["host_counts"], fwd["cumsum_excl"]
    tm, em, ch = fwd["token_mapping"], fwd["expert_mapping"], fwd["chosen"]
    w = layer.weights.cpu().numpy()  # the gate weights the GPU ops consumed (oracle's agree to 1e-5)

    def per_expert(fn, rows_out, cols_out):
        res = np.zeros((rows_out, cols_out), np.uint16)
        for e in range(E):
            n, b = int(cnt[e]), int(base[e])
            if n:
                res[b:b + n] = fn(e, slice(b, b + n))
        return res

    Yr = per_expert(lambda e, sl: oracle.linear_fwd(np.ascontiguousarray(hg[sl]), W2[e]), T * k, d)
    assert_close(f32(Yg), f32(Yr), what="Y")
    assert_close(f32(host_bits(out)), f32(oracle.merge_experts(Yg, tm, w, np.zeros((T, d), np.uint16))), what="out")
    assert_chain_close(f32(host_bits(out)), f32(fwd["out"]), what="out (chain)")

    # ---- backward ops
    dx1g, dx3g, dZg = host_bits(layer.dx1), host_bits(layer.dx3), host_bits(layer.dZ)
    dlg, dXng = host_bits(layer.dX_routed), host_bits(dXn)
    pre = host_bits(layer.dX_routed_pre)
    dYs = np.zeros((T * k, d), np.uint16)  # w * dOut rows in expert order
    for j in range(k):
        dYs[tm[:, j]] = f32_to_bf16_bits(f32(dOut) * w[:, j:j + 1])
    if path == "fast":
        np.testing.assert_array_equal(host_bits(layer.dYz), dYs)
    # dP before the gate Jacobian: <Y, dOut> per routed (token, expert), stored bf16 like the reference
    dots = (f32(Yg)[tm.reshape(-1)].reshape(T, k, d) * f32(dOut)[:, None, :]).sum(axis=2)
    pre_ref = np.zeros((T, E), np.float32)
    np.put_along_axis(pre_ref, ch.astype(np.int64), dots, axis=1)
    assert_close(f32(pre), pre_ref, rtol=2e-2, atol=2e-2 * float(np.abs(dots).mean()), what="dX_routed before gate")
    assert_close(f32(dlg), f32(oracle.router_gate_bwd_x(ch, w, pre.copy())), what="dlogits")
    dh = per_expert(lambda e, sl: oracle.linear_dgrad(np.ascontiguousarray(dYs[sl]), W2[e]), T * k, f)
    r1, r3 = oracle.swiglu_bwd_x(x1g, x3g, dh)
    assert_close(f32(dx1g), f32(r1), what="dx1")
    assert_close(f32(dx3g), f32(r3), what="dx3")
    dz1 = per_expert(lambda e, sl: oracle.linear_dgrad(np.ascontiguousarray(dx1g[sl]), W1[e]), T * k, d)
    dZr = per_expert(lambda e, sl: oracle.linear_dgrad(np.ascontiguousarray(dx3g[sl]), W3[e],
                                                       accumulate_into=np.ascontiguousarray(dz1[sl]).copy()), T * k, d)
    if path == "fast":
        # one fp32 accumulator for dx1 W1 + dx3 W3; the reference rounds the first product to bf16 in between
        assert_close_with_slack(f32(dZg), f32(dZr), np.abs(f32(dz1)) * 2.0 ** -8, what="dZ")
    else:
        assert_close(f32(dZg), f32(dZr), what="dZ")
    dXr = oracle.merge_experts(dZg, tm, None, np.zeros((T, d), np.uint16))
    oracle.linear_dgrad(dlg, Wr, accumulate_into=dXr)
    assert_close(f32(dXng), f32(dXr), what="dXn")
    gr = {n: g0[n].copy() for n in g0}
    for e in range(E):
        n, b = int(cnt[e]), int(base[e])
        if n:
            sl = slice(b, b + n)
            oracle.linear_wgrad(np.ascontiguousarray(hg[sl]), np.ascontiguousarray(dYs[sl]), gr["dW2"][e])
            oracle.linear_wgrad(fwd["zone"][sl], np.ascontiguousarray(dx1g[sl]), gr["dW1"][e])
            oracle.linear_wgrad(fwd["zone"][sl], np.ascontiguousarray(dx3g[sl]), gr["dW3"][e])
    oracle.linear_wgrad(X, dlg, gr["dWr"])
    for n in ("dW1", "dW3", "dW2", "dWr"):
        assert_close(f32(host_bits(G[n])), f32(gr[n]), what=n)

    # ---- the whole chain against the oracle's own chain
    bwd = oracle.moe_backward(X, Wr, W1, W3, W2, k, fwd, dOut, grads={n: g0[n].copy() for n in g0})
    for got, ref, what, lim in [(dXng, bwd["dXn"], "dXn", 1e-2), (host_bits(G["dW1"]), bwd["dW1"], "dW1", 1e-2),
                                (host_bits(G["dW3"]), bwd["dW3"], "dW3", 1e-2), (host_bits(G["dW2"]), bwd["dW2"], "dW2", 1e-2),
                                (dlg, bwd["dlogits"], "dlogits", 5e-2), (host_bits(G["dWr"]), bwd["dWr"], "dWr", 5e-2)]:
        assert_chain_close(f32(got), f32(ref), limit=lim, what=what + " (chain)")


def make_case(seed, T, d, E, k, f, wstd=0.02, grad_init=0.0):
    rng = np.random.default_rng(seed)
    X, dOut = rand_bf16(rng, (T, d)), rand_bf16(rng, (T, d))
    Wr = rand_bf16(rng, (E, d), wstd)
    W1, W3, W2 = rand_bf16(rng, (E, f, d), wstd), rand_bf16(rng, (E, f, d), wstd), rand_bf16(rng, (E, d, f), wstd)
    g0 = dict(dWr=rand_bf16(rng, (E, d), grad_init), dW1=rand_bf16(rng, (E, f, d), grad_init),
              dW3=rand_bf16(rng, (E, f, d), grad_init), dW2=rand_bf16(rng, (E, d, f), grad_init))
    return X, Wr, W1, W3, W2, dOut, g0


@pytest.mark.parametrize("path", ["fast", "reference_order"])
@pytest.mark.parametrize("T,d,E,k,f", [(200, 128, 8, 2, 64), (512, 256, 16, 4, 192)])
def test_layer_small(oracle, path, T, d, E, k, f):
    require_b200()
    X, Wr, W1, W3, W2, dOut, g0 = make_case(T + d, T, d, E, k, f, wstd=0.06, grad_init=0.05)
    layer, out, dXn, G = run_layer(path, T, d, E, k, f, X, Wr, W1, W3, W2, dOut, g0)
    compare_with_oracle(oracle, layer, out, dXn, G, X, Wr, W1, W3, W2, dOut, g0, k, path)


def test_layer_config1_fast_path(oracle):
    """BASELINE config 1: T=2048, d=1024, 16 experts, top-2, ffn 1024, weights N(0, 0.02)."""
    require_b200()
    T, d, E, k, f = 2048, 1024, 16, 2, 1024
    X, Wr, W1, W3, W2, dOut, g0 = make_case(1, T, d, E, k, f)
    layer, out, dXn, G = run_layer("fast", T, d, E, k, f, X, Wr, W1, W3, W2, dOut, g0)
    compare_with_oracle(oracle, layer, out, dXn, G, X, Wr, W1, W3, W2, dOut, g0, k, "fast")


@pytest.mark.parametrize("name", ["moe_mlp_small", "moe_mlp_k4", "moe_mlp_e64k8"])
def test_layer_against_reference_pytorch_golden(name):
    """The CUDA layer against tensors produced by the reference's own PyTorch MoE layer (tests/golden)."""
    require_b200()
    g = np.load(os.path.join(GOLD, name + ".npz"))
    T, d, E, k, f = [int(v) for v in g["shape"]]
    zeros = dict(dWr=np.zeros((E, d), np.uint16), dW1=np.zeros((E, f, d), np.uint16),
                 dW3=np.zeros((E, f, d), np.uint16), dW2=np.zeros((E, d, f), np.uint16))
    layer, out, dXn, G = run_layer("fast", T, d, E, k, f, g["X"], g["Wr"], g["W1"], g["W3"], g["W2"], g["dOut"], zeros,
                                   logits=np.ascontiguousarray(g["logits"]))
    ch = host_u16(layer.chosen).astype(np.int32)
    np.testing.assert_array_equal(np.sort(ch, axis=1), np.sort(g["selected"], axis=1))

    def rms(a):
        return float(np.sqrt(np.mean(np.asarray(a, np.float64) ** 2)))

    def rel_fro(a, b):
        return float(np.linalg.norm(a.astype(np.float64) - b) / (np.linalg.norm(b.astype(np.float64)) + 1e-30))

    pairs = [(out, g["out"], "out"), (dXn, g["dX"], "dX"), (G["dW1"], g["dW1"], "dW1"), (G["dW3"], g["dW3"], "dW3"),
             (G["dW2"], g["dW2"], "dW2")]
    for got, ref, what in pairs:
        a, b = f32(host_bits(got)), f32(ref)
        assert rel_fro(a, b) < 8e-3, what
        assert_close(a, b, atol=4e-2 * rms(b), what=what)
    assert rel_fro(f32(host_bits(G["dWr"])), g["dWr"]) < 8e-3


def test_layer_properties_full_size():
    """BASELINE config 2 shape (T=8192, d=4096, 64 experts, top-8, ffn 1408): size-independent properties.

    counts sum to T*k; token_mapping is a permutation of 0..R-1 consistent with expert_mapping; gate weights sum
    to 1; forward is linear in the gate weights' residual (out with residual r equals out without + r up to one
    rounding); un-permute(permute(x)) == k * x.
    """
    require_b200()
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    T, d, E, k, f = 8192, 4096, 64, 8, 1408
    gen = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn((T, d), generator=gen, device="cuda").to(torch.bfloat16)
    Wr = (torch.randn((E, d), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    W1 = (torch.randn((E, f, d), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    W3 = (torch.randn((E, f, d), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    W2 = (torch.randn((E, d, f), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    layer = MoELayer(T, d, E, k, f)
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    layer.forward(X, Wr, W1, W3, W2, out)
    assert ops.gemm_status() == 0
    counts = layer.counts[:E].cpu().numpy()
    assert counts.sum() == T * k
    np.testing.assert_array_equal(layer.cumsum.cpu().numpy(), np.cumsum(counts))
    tm = layer.token_mapping.cpu().numpy().reshape(-1)
    em = layer.expert_mapping.cpu().numpy()
    np.testing.assert_array_equal(np.sort(tm), np.arange(T * k))
    np.testing.assert_array_equal(em[tm], np.repeat(np.arange(T), k))
    ch = host_u16(layer.chosen).reshape(-1).astype(np.int64)
    np.testing.assert_array_equal(np.searchsorted(np.cumsum(counts), tm, side="right"), ch)
    np.testing.assert_allclose(layer.weights.sum(dim=1).cpu().numpy(), 1.0, rtol=1e-5)
    assert torch.isfinite(out.float()).all()
    # permute then un-permute with unit weights gives k copies of every row
    back = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    ops.merge_experts(T, d, k, layer.zone, layer.token_mapping, None, back)
    torch.cuda.synchronize()
    assert torch.equal(back, (X.float() * k).to(torch.bfloat16))
    # expert outputs against a torch fp32 evaluation of three sampled experts
    base = np.concatenate([[0], np.cumsum(counts)])
    for e in (0, 31, 63):
        n = int(counts[e])
        if n == 0:
            continue
        z = layer.zone[base[e]:base[e] + n].float()
        x1 = (z @ W1[e].float().T).to(torch.bfloat16).float()
        x3 = (z @ W3[e].float().T).to(torch.bfloat16).float()
        h = (torch.nn.functional.silu(x1) * x3).to(torch.bfloat16).float()
        y = (h @ W2[e].float().T)
        got = layer.Y[base[e]:base[e] + n].float()
        err = (got - y).abs()
        assert (err <= 1e-3 + 2e-2 * y.abs()).float().mean() > 0.999, f"expert {e}"


@pytest.mark.parametrize("T,d,E,k,f", [(512, 256, 16, 4, 192), (2048, 1024, 16, 2, 1024)])
def test_c_block_driver_matches_fast_path(T, d, E, k, f):
    """b200_moe_block_fwd / _bwd (one C call per direction) issue the same kernels in the same order as the Python
    fast path, which the tests above hold to the oracle: everything that does not pass through the fp32 atomics of
    the router dot product must be bit-identical, the router gradients equal to rounding."""
    require_b200()
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    X, Wr, W1, W3, W2, dOut, g0 = make_case(T * 3 + f, T, d, E, k, f, wstd=0.05, grad_init=0.05)
    Xd, Wrd, W1d, W3d, W2d, dOd = (dev_bf16(a) for a in (X, Wr, W1, W3, W2, dOut))
    res = []
    for use_block in (False, True):
        layer = MoELayer(T, d, E, k, f)
        out = dev_bf16(X.copy())  # the residual
        dXn = torch.empty((T, d), dtype=torch.bfloat16, device="cuda")
        G = {n: dev_bf16(g0[n].copy()) for n in ("dWr", "dW1", "dW3", "dW2")}
        if use_block:
            blk = layer.block(Wrd, W1d, W3d, W2d)
            ops.moe_block_fwd(blk, Xd, out)
            ops.moe_block_bwd(blk, Xd, dOd, dXn, G["dWr"], G["dW1"], G["dW3"], G["dW2"])
        else:
            layer.forward(Xd, Wrd, W1d, W3d, W2d, out)
            layer.backward(Xd, Wrd, W1d, W3d, W2d, dOd, dXn, G["dWr"], G["dW1"], G["dW3"], G["dW2"])
        assert ops.gemm_status() == 0
        res.append((layer, out, dXn, G))
    (la, oa, xa, ga), (lb, ob, xb, gb) = res
    same = lambda p, q: torch.equal(p.view(torch.uint8), q.view(torch.uint8))
    for name in ("logits", "weights", "chosen", "cumsum", "expert_mapping", "token_mapping", "zone", "x1", "x3", "h", "Y",
                 "dYz", "dx1", "dx3", "dZ"):
        assert same(getattr(la, name), getattr(lb, name)), name
    assert same(la.counts[:E], lb.counts[:E])
    assert same(oa, ob)
    for n in ("dW1", "dW3", "dW2"):
        assert same(ga[n], gb[n]), n
    assert_close(f32(host_bits(xb)), f32(host_bits(xa)), rtol=2e-2, atol=1e-3, what="dXn")
    assert_close(f32(host_bits(gb["dWr"])), f32(host_bits(ga["dWr"])), rtol=2e-2, atol=1e-3, what="dWr")
    # recompute after the workspace has been clobbered: bit-identical zone / x1 / x3 / h, then the same backward
    blk = lb.block(Wrd, W1d, W3d, W2d)
    keep = {n: getattr(lb, n).clone() for n in ("zone", "x1", "x3", "h")}
    for level, clobbered in ((0, ("zone", "h")), (1, ("zone", "h", "x1", "x3"))):
        for n in clobbered:
            getattr(lb, n).fill_(3.0)
        ops.moe_block_recompute(blk, Xd, level)
        for n in keep:
            assert same(getattr(lb, n), keep[n]), (level, n)
    G2 = {n: dev_bf16(g0[n].copy()) for n in ("dWr", "dW1", "dW3", "dW2")}
    ops.moe_block_bwd(blk, Xd, dOd, xb, G2["dWr"], G2["dW1"], G2["dW3"], G2["dW2"])
    for n in ("dW1", "dW3", "dW2"):
        assert same(G2[n], gb[n]), n
    # forward-only use: no backward workspace, no weight gradients wanted
    blk = lb.block(Wrd, W1d, W3d, W2d)
    blk.dY_zone = None
    out2 = dev_bf16(X.copy())
    ops.moe_block_fwd(blk, Xd, out2)
    assert same(out2, ob)
    with pytest.raises(RuntimeError):
        ops.moe_block_bwd(blk, Xd, dOd, xb, gb["dWr"], None, None, None)


def test_block_backward_overwrite_equals_zero_then_accumulate():
    """b200_moe_block_bwd_overwrite writes the same weight gradients that b200_moe_block_bwd adds to zeroed buffers,
    bit for bit, whatever the buffers held before."""
    import torch

    from gpu_util import require_b200

    require_b200()
    from ml_dataflow_b200 import _lib, ops
    from ml_dataflow_b200.moe_layer import MoELayer

    T, d, E, k, f = 512, 256, 8, 2, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    n = lambda shape, std: (torch.randn(shape, generator=g, device="cuda") * std).to(torch.bfloat16)
    X, dOut, Wr = n((T, d), 1.0), n((T, d), 1.0), n((E, d), 0.1)
    W1, W3, W2 = n((E, f, d), 0.1), n((E, f, d), 0.1), n((E, d, f), 0.1)
    layer = MoELayer(T, d, E, k, f, device="cuda")
    blk = layer.block(Wr, W1, W3, W2)
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    ops.moe_block_fwd(blk, X, out)
    grads_a = [torch.zeros_like(t) for t in (Wr, W1, W3, W2)]
    dXa = torch.empty_like(X)
    ops.moe_block_bwd(blk, X, dOut, dXa, *grads_a)
    grads_b = [torch.full_like(t, 5.0) for t in (Wr, W1, W3, W2)]
    dXb = torch.empty_like(X)
    import ctypes as C

    p = lambda t: C.c_void_p(t.data_ptr())
    rc = _lib.load().b200_moe_block_bwd_overwrite(C.byref(blk), p(X), p(dOut), p(dXb), *[p(t) for t in grads_b],
                                                  C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    assert torch.equal(dXa, dXb)
    for a, b, name in zip(grads_a, grads_b, ("dWr", "dW1", "dW3", "dW2")):
        assert torch.equal(a, b), name
