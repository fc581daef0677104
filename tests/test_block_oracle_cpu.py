"""CPU: the block-op oracle (oracle/block_oracle.c) against independent statements of the same maths in float64 numpy
and torch autograd: RMSNorm forward / backward (autograd of x * rsqrt(mean(x^2) + eps) * w), RoPE as a complex
rotation, softmax + cross-entropy gradient (softmax - onehot), AdamW (torch.optim.AdamW on float32 copies), the
embedding gather and its scatter-add. The oracle rounds to bf16 where the reference's kernels do, so comparisons are to
bf16 resolution."""
import numpy as np
import pytest
import torch


def _bits(a):
    from helpers import f32_to_bf16_bits

    return f32_to_bf16_bits(np.asarray(a, np.float32))


def _f32(b):
    from helpers import bf16_bits_to_f32

    return bf16_bits_to_f32(b)


def test_rms_norm_forward_backward_against_autograd(oracle):
    rng = np.random.default_rng(0)
    rows, cols, eps = 37, 256, 1e-5
    X, w, up = _bits(rng.standard_normal((rows, cols)) * 1.5), _bits(rng.standard_normal(cols)), _bits(rng.standard_normal((rows, cols)))
    out, rms = oracle.rms_norm(w, X, eps)
    x = torch.tensor(_f32(X), dtype=torch.float64, requires_grad=True)
    wt = torch.tensor(_f32(w), dtype=torch.float64, requires_grad=True)
    y = x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + eps) * wt
    np.testing.assert_allclose(rms, torch.rsqrt((x * x).mean(dim=1) + eps).detach().numpy(), rtol=1e-6)
    np.testing.assert_allclose(_f32(out), y.detach().numpy(), rtol=8e-3, atol=1e-6)
    y.backward(torch.tensor(_f32(up), dtype=torch.float64))
    zero = np.zeros((rows, cols), np.uint16)
    dX, x_out = oracle.rms_norm_bwd_x(rms, w, X, up, zero, want_x_out=True)
    np.testing.assert_array_equal(x_out, out)
    np.testing.assert_allclose(_f32(dX), x.grad.numpy(), rtol=1e-2, atol=2e-3)
    dW = oracle.rms_norm_bwd_w(rms, X, up, np.zeros(cols, np.uint16))
    np.testing.assert_allclose(_f32(dW), wt.grad.numpy(), rtol=1e-2, atol=2e-2)
    # accumulation into existing gradients: one rounding of (old + new)
    old = _bits(rng.standard_normal((rows, cols)))
    dX2, _ = oracle.rms_norm_bwd_x(rms, w, X, up, old)
    np.testing.assert_allclose(_f32(dX2), _f32(old) + x.grad.numpy(), rtol=1e-2, atol=8e-3)
    np.testing.assert_array_equal(oracle.rms_norm_recompute(w, rms, X), out)


def test_rope_is_a_complex_rotation(oracle):
    rng = np.random.default_rng(1)
    tokens, heads, kv_heads, hd, theta = 19, 4, 2, 64, 10000
    q, k = _bits(rng.standard_normal((tokens, heads * hd))), _bits(rng.standard_normal((tokens, kv_heads * hd)))
    pos = rng.integers(0, 4096, tokens).astype(np.int32)
    rq, rk = oracle.rope(hd, kv_heads, theta, pos, q, k)
    inv = theta ** (-np.arange(0, hd, 2, dtype=np.float64) / hd)
    rot = np.exp(1j * pos[:, None].astype(np.float64) * inv[None, :])  # [tokens, hd/2]
    for got, src, h in ((rq, q, heads), (rk, k, kv_heads)):
        z = _f32(src).astype(np.float64).reshape(tokens, h, hd // 2, 2)
        zc = (z[..., 0] + 1j * z[..., 1]) * rot[:, None, :]
        ref = np.stack([zc.real, zc.imag], axis=-1).reshape(tokens, h * hd)
        # fp32 angles of up to 4096 rad carry ~2e-4 of absolute error before the bf16 rounding
        np.testing.assert_allclose(_f32(got), ref, rtol=8e-3, atol=3e-3)
    # the backward is the inverse rotation
    bq, _ = oracle.rope(hd, kv_heads, theta, pos, rq, None, backward=True)
    np.testing.assert_allclose(_f32(bq), _f32(q), rtol=2e-2, atol=2e-2)
    same, _ = oracle.rope(hd, kv_heads, theta, np.zeros(tokens, np.int32), q, None)
    np.testing.assert_array_equal(same, q)


def test_softmax_cross_entropy_gradient(oracle):
    rng = np.random.default_rng(2)
    rows, cols = 9, 1003
    X = _bits(rng.standard_normal((rows, cols)) * 3)
    labels = rng.integers(0, cols, rows).astype(np.uint32)
    p = oracle.softmax(X)
    ref = torch.softmax(torch.tensor(_f32(X), dtype=torch.float64), dim=1).numpy()
    np.testing.assert_allclose(_f32(p), ref, rtol=8e-3, atol=1e-9)
    g, loss = oracle.cross_entropy_loss(p, labels)
    onehot = np.zeros((rows, cols))
    onehot[np.arange(rows), labels] = 1.0
    np.testing.assert_allclose(_f32(g), _f32(p) - onehot, rtol=8e-3, atol=1e-9)
    np.testing.assert_allclose(loss[:rows], -np.log(_f32(p)[np.arange(rows), labels]), rtol=1e-6)
    np.testing.assert_allclose(loss[rows], loss[:rows].mean(), rtol=1e-6)


@pytest.mark.parametrize("step", [1, 10])
def test_adamw_matches_torch(oracle, step):
    rng = np.random.default_rng(3)
    n = 4096
    p0, g = _bits(rng.standard_normal(n) * 0.02), _bits(rng.standard_normal(n) * 0.01)
    m0, v0 = _bits(rng.standard_normal(n) * 0.01), _bits(np.abs(rng.standard_normal(n)) * 1e-4)
    lr, b1, b2, wd, eps = 3e-4, 0.9, 0.95, 0.1, 1e-8
    p, m, v = oracle.adamw_step(step, lr, b1, b2, wd, eps, p0, g, m0, v0)
    param = torch.nn.Parameter(torch.tensor(_f32(p0), dtype=torch.float64))
    opt = torch.optim.AdamW([param], lr=lr, betas=(b1, b2), eps=eps, weight_decay=wd)
    param.grad = torch.tensor(_f32(g), dtype=torch.float64)
    st = opt.state[param]
    st["step"] = torch.tensor(float(step - 1))
    st["exp_avg"] = torch.tensor(_f32(m0), dtype=torch.float64)
    st["exp_avg_sq"] = torch.tensor(_f32(v0), dtype=torch.float64)
    opt.step()
    np.testing.assert_allclose(_f32(m), st["exp_avg"].numpy(), rtol=8e-3, atol=1e-9)
    np.testing.assert_allclose(_f32(v), st["exp_avg_sq"].numpy(), rtol=8e-3, atol=1e-12)
    np.testing.assert_allclose(_f32(p), param.detach().numpy(), rtol=8e-3, atol=1e-7)


def test_embedding_gather_and_scatter_add(oracle):
    rng = np.random.default_rng(4)
    tokens, vocab, dim = 200, 17, 32
    ids = rng.integers(0, vocab, tokens).astype(np.uint32)
    table = _bits(rng.standard_normal((vocab, dim)))
    sorted_ids, mapping, starts = oracle.sort_tokens(ids)
    assert np.all(np.diff(sorted_ids.astype(np.int64)) >= 0) and np.array_equal(ids[mapping], sorted_ids)
    np.testing.assert_array_equal(oracle.embedding_table(sorted_ids, mapping, starts, table, tokens), table[ids])
    grads = _bits(rng.standard_normal((tokens, dim)))
    gt = oracle.embedding_table_bwd_w(sorted_ids, mapping, starts, grads, np.zeros((vocab, dim), np.uint16))
    ref = np.zeros((vocab, dim))
    np.add.at(ref, ids, _f32(grads).astype(np.float64))
    # bf16 running sums of about a dozen terms: a few ulp of the largest partial sum
    np.testing.assert_allclose(_f32(gt), ref, rtol=3e-2, atol=6e-2)
    absent = np.setdiff1d(np.arange(vocab), ids)
    assert not _f32(gt)[absent].any()
