"""CPU: the oracle against independent statements of the same maths.

The oracle (oracle/moe_oracle.c) is what every GPU kernel is compared with, so it is itself cross-checked here, on
small cases, against (a) a literal pure-Python walk through the reference's selection rule, read off
select_experts.cu:135-166 (first k experts fill the slots in order; a later value must be strictly
greater than the running minimum to enter; it replaces the slot holding the minimum, ties among equal minima going to
the slot with the larger expert index), (b) float64 numpy for the linear algebra, and (c) torch autograd on the CPU for
the two hand-derived backward formulas (SwiGLU and the softmax-over-the-chosen-k gate). None of this needs a GPU.
"""
import numpy as np
import pytest
import torch

from helpers import assert_close, bf16_bits_to_f32, f32_to_bf16_bits


def select_by_hand(row, k):
    """Slot-ordered top-k of one logit row by the reference's sequential rule."""
    vals, inds = [], []
    for e, v in enumerate(row):
        v = float(v)
        if len(vals) < k:
            if v == float("-inf"):
                continue  # a slot is only taken by a value greater than the initial -inf
            vals.append(v)
            inds.append(e)
            continue
        lo = min(vals)
        if not v > lo:
            continue
        slot = max((j for j in range(k) if vals[j] == lo), key=lambda j: inds[j])
        vals[slot], inds[slot] = v, e
    return vals, inds


@pytest.mark.parametrize("T,E,k,kind", [(64, 16, 2, "normal"), (64, 64, 8, "normal"), (48, 64, 8, "ties"),
                                        (16, 8, 8, "normal"), (32, 64, 8, "equal"), (32, 32, 4, "descending")])
def test_select_experts_follows_the_sequential_rule(oracle, T, E, k, kind):
    rng = np.random.default_rng(T + E + k)
    if kind == "normal":
        logits = rng.standard_normal((T, E)).astype(np.float32)
    elif kind == "ties":
        logits = rng.integers(-2, 3, size=(T, E)).astype(np.float32)  # many equal values
    elif kind == "equal":
        logits = np.full((T, E), 0.25, np.float32)
    else:
        logits = np.tile(np.arange(E, 0, -1, dtype=np.float32), (T, 1))
    w, ch, counts, cexcl, host_counts = oracle.select_experts(logits, k)
    for t in range(T):
        vals, inds = select_by_hand(logits[t], k)
        assert list(ch[t]) == inds, (t, list(ch[t]), inds)
        v = np.array(vals, np.float64)
        p = np.exp(v - v.max())
        np.testing.assert_allclose(w[t], p / p.sum(), rtol=2e-6, atol=1e-7)
    hist = np.bincount(ch.reshape(-1).astype(np.int64), minlength=E)
    np.testing.assert_array_equal(counts[:E], hist)
    np.testing.assert_array_equal(host_counts[:E], hist)
    np.testing.assert_array_equal(cexcl, np.cumsum(hist) - hist)
    if kind == "equal":
        assert (ch == np.arange(k)).all()  # nothing ever displaces the first k


def test_mapping_is_the_stable_counting_sort(oracle):
    rng = np.random.default_rng(7)
    T, E, k = 200, 16, 4
    logits = rng.standard_normal((T, E)).astype(np.float32)
    _, ch, counts, cexcl, _ = oracle.select_experts(logits, k)
    em, tm, cincl = oracle.build_expert_mapping(ch, E, cexcl)
    np.testing.assert_array_equal(cincl, np.cumsum(counts[:E]))
    cursor = list(cexcl)
    for t in range(T):
        for j in range(k):
            e = int(ch[t, j])
            assert tm[t, j] == cursor[e] and em[cursor[e]] == t
            cursor[e] += 1
    np.testing.assert_array_equal(np.sort(tm.reshape(-1)), np.arange(T * k))


def test_gather_then_weighted_combine_of_identity_experts_returns_the_tokens(oracle):
    rng = np.random.default_rng(11)
    T, d, E, k = 64, 96, 8, 3
    logits = rng.standard_normal((T, E)).astype(np.float32)
    w, ch, counts, cexcl, _ = oracle.select_experts(logits, k)
    em, tm, _ = oracle.build_expert_mapping(ch, E, cexcl)
    X = f32_to_bf16_bits(rng.standard_normal((T, d)).astype(np.float32))
    zone = oracle.prepare_experts(X, tm)
    np.testing.assert_array_equal(zone[tm[:, 1]], X)  # every copy is the token's row, bit for bit
    out = oracle.merge_experts(zone, tm, w, np.zeros((T, d), np.uint16))
    x = bf16_bits_to_f32(X)
    assert (np.abs(bf16_bits_to_f32(out) - x) <= np.abs(x) * 2.0 ** -7 + 1e-30).all()  # weights sum to 1
    back = oracle.merge_experts(zone, tm, None, np.zeros((T, d), np.uint16))
    np.testing.assert_array_equal(back, f32_to_bf16_bits(x * k))  # NULL weights mean 1.0


@pytest.mark.parametrize("ta,tb", [(1, 0), (0, 0), (0, 1), (1, 1)])
def test_matmul_against_float64(oracle, ta, tb):
    rng = np.random.default_rng(3 + 2 * ta + tb)
    M, K, N = 24, 40, 16
    A = f32_to_bf16_bits(rng.standard_normal((M, K) if ta else (K, M)).astype(np.float32))
    B = f32_to_bf16_bits(rng.standard_normal((K, N) if tb else (N, K)).astype(np.float32))
    C0 = f32_to_bf16_bits(rng.standard_normal((N, M)).astype(np.float32))
    a = bf16_bits_to_f32(A).astype(np.float64)
    b = bf16_bits_to_f32(B).astype(np.float64)
    # a column-major matrix is the transpose of the row-major array holding it: op(A) is M x K, op(B) is K x N,
    # and the column-major M x N result is the row-major array [N][M]
    op_a = a if ta else a.T
    op_b = b if tb else b.T
    ref = (op_a @ op_b).T
    ref = 0.5 * ref + 2.0 * bf16_bits_to_f32(C0)
    D = C0.copy()
    oracle.matmul(ta, tb, M, K, N, 0.5, 2.0, A, B, C0, D)
    assert_close(bf16_bits_to_f32(D), ref, rtol=1e-2, atol=1e-2, what=f"matmul ta={ta} tb={tb}")


def test_swiglu_backward_against_autograd(oracle):
    rng = np.random.default_rng(5)
    rows, cols = 12, 32
    x1 = f32_to_bf16_bits(rng.standard_normal((rows, cols)).astype(np.float32))
    x3 = f32_to_bf16_bits(rng.standard_normal((rows, cols)).astype(np.float32))
    dy = f32_to_bf16_bits(rng.standard_normal((rows, cols)).astype(np.float32))
    a = torch.tensor(bf16_bits_to_f32(x1), dtype=torch.float64, requires_grad=True)
    b = torch.tensor(bf16_bits_to_f32(x3), dtype=torch.float64, requires_grad=True)
    h = torch.nn.functional.silu(a) * b
    h.backward(torch.tensor(bf16_bits_to_f32(dy), dtype=torch.float64))
    assert_close(bf16_bits_to_f32(oracle.swiglu(x1, x3)), h.detach().numpy(), what="swiglu")
    g1, g3 = oracle.swiglu_bwd_x(x1, x3, dy)
    assert_close(bf16_bits_to_f32(g1), a.grad.numpy(), what="d swiglu / d x1")
    assert_close(bf16_bits_to_f32(g3), b.grad.numpy(), what="d swiglu / d x3")


def test_gate_backward_against_autograd(oracle):
    """dL/dlogit over the k chosen experts of a softmax taken over those k only (router_gate_bwd_x.cu:7-57)."""
    rng = np.random.default_rng(9)
    T, E, k = 40, 16, 4
    logits = rng.standard_normal((T, E)).astype(np.float32)
    w, ch, *_ = oracle.select_experts(logits, k)
    dP = f32_to_bf16_bits(rng.standard_normal((T, E)).astype(np.float32))  # dL/dw on the chosen columns
    got = bf16_bits_to_f32(oracle.router_gate_bwd_x(ch, w, dP.copy()))
    lg = torch.tensor(logits, dtype=torch.float64, requires_grad=True)
    idx = torch.tensor(ch.astype(np.int64))
    wk = torch.softmax(torch.gather(lg, 1, idx), dim=1)
    up = torch.gather(torch.tensor(bf16_bits_to_f32(dP), dtype=torch.float64), 1, idx)
    (wk * up).sum().backward()
    ref = lg.grad.numpy()
    chosen_mask = np.zeros((T, E), bool)
    np.put_along_axis(chosen_mask, ch.astype(np.int64), True, axis=1)
    assert_close(got[chosen_mask], ref[chosen_mask], rtol=2e-2, atol=2e-3, what="gate backward")
    np.testing.assert_array_equal(got[~chosen_mask], bf16_bits_to_f32(dP)[~chosen_mask])  # other columns untouched


def test_layer_backward_against_autograd_in_float64(oracle):
    """The oracle's whole backward (the reference block's op order, bf16 storage) against torch autograd of the same
    layer in float64, routing held fixed: every gradient within the bf16 chain tolerance."""
    from helpers import rel_fro

    rng = np.random.default_rng(21)
    T, d, E, k, f = 48, 32, 4, 2, 24
    mk = lambda shape, s: f32_to_bf16_bits((rng.standard_normal(shape) * s).astype(np.float32))
    X, dOut, Wr = mk((T, d), 1.0), mk((T, d), 1.0), mk((E, d), 0.3)
    W1, W3, W2 = mk((E, f, d), 0.2), mk((E, f, d), 0.2), mk((E, d, f), 0.2)
    fwd = oracle.moe_forward(X, Wr, W1, W3, W2, k)
    bwd = oracle.moe_backward(X, Wr, W1, W3, W2, k, fwd, dOut)
    t64 = lambda a: torch.tensor(bf16_bits_to_f32(a), dtype=torch.float64, requires_grad=True)
    x, wr, w1, w3, w2 = t64(X), t64(Wr), t64(W1), t64(W3), t64(W2)
    idx = torch.tensor(fwd["chosen"].astype(np.int64))
    gates = torch.softmax(torch.gather(x @ wr.T, 1, idx), dim=1)
    out = torch.zeros((T, d), dtype=torch.float64)
    for j in range(k):
        e = idx[:, j]
        h = torch.nn.functional.silu(torch.einsum("td,tfd->tf", x, w1[e])) * torch.einsum("td,tfd->tf", x, w3[e])
        out = out + gates[:, j:j + 1] * torch.einsum("tf,tdf->td", h, w2[e])
    assert rel_fro(bf16_bits_to_f32(fwd["out"]), out.detach().numpy()) < 1e-2
    out.backward(torch.tensor(bf16_bits_to_f32(dOut), dtype=torch.float64))
    for name, ref in (("dXn", x.grad), ("dW1", w1.grad), ("dW3", w3.grad), ("dW2", w2.grad), ("dWr", wr.grad)):
        r = rel_fro(bf16_bits_to_f32(bwd[name]), ref.numpy())
        assert r < (5e-2 if name == "dWr" else 1.5e-2), f"{name}: relative Frobenius error {r:.2e}"
