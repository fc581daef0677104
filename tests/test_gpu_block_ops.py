"""GPU: the bandwidth-bound block and head ops (csrc/block_ops.cu) against the CPU oracle (oracle/block_oracle.c) on
the same seeded inputs, through the C ABI. bf16 tensors to |a-b| <= 1e-3 + 2e-2 |b|; what is pure copying or bf16
arithmetic in a fixed order (embedding forward / backward, the label entry of the cross-entropy) bit-exact.
Shapes: the decoder configuration of the full training step (d=2048, 16 query / 4 kv heads of 128) at a few hundred
rows, ragged sizes, and rows longer than a thread block keeps in registers.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(oracle):
    import torch

    from gpu_util import require_b200

    require_b200()
    from ml_dataflow_b200 import ops

    return torch, ops, oracle


def _f32(bits):
    from helpers import bf16_bits_to_f32

    return bf16_bits_to_f32(bits)


@pytest.mark.parametrize("rows,cols", [(300, 2048), (257, 4096), (33, 8192), (5, 16384), (64, 72), (1, 8)])
def test_rms_norm_forward_and_recompute(env, rows, cols):
    torch, ops, orc = env
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close

    rng = np.random.default_rng(rows * 31 + cols)
    X, w = rand_bf16(rng, (rows, cols), 1.5), rand_bf16(rng, (cols,), 1.0)
    ref_out, ref_rms = orc.rms_norm(w, X, 1e-5)
    Xd, wd = dev_bf16(X), dev_bf16(w)
    out = torch.zeros_like(Xd)
    rms = torch.zeros(rows, dtype=torch.float32, device="cuda")
    ops.rms_norm(rows, cols, 1e-5, wd, Xd, out, rms)
    np.testing.assert_allclose(rms.cpu().numpy(), ref_rms, rtol=2e-6)
    assert_close(_f32(host_bits(out)), _f32(ref_out), what="rms_norm")
    # without the rms output, and the recompute from kept values: the same bits as the forward
    out2 = torch.zeros_like(Xd)
    ops.rms_norm(rows, cols, 1e-5, wd, Xd, out2, None)
    assert torch.equal(out, out2)
    out3 = torch.zeros_like(Xd)
    ops.rms_norm_recompute(rows, cols, wd, rms, Xd, out3)
    assert torch.equal(out, out3)
    assert_close(_f32(host_bits(out3)), _f32(orc.rms_norm_recompute(w, ref_rms, X)), what="rms_norm_recompute")


@pytest.mark.parametrize("rows,cols", [(300, 2048), (129, 4096), (17, 8192), (64, 72)])
def test_rms_norm_backward(env, rows, cols):
    torch, ops, orc = env
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close, assert_chain_close

    rng = np.random.default_rng(rows + cols)
    X, w = rand_bf16(rng, (rows, cols), 1.5), rand_bf16(rng, (cols,), 1.0)
    up, dX0 = rand_bf16(rng, (rows, cols), 1.0), rand_bf16(rng, (rows, cols), 0.5)
    dW0 = rand_bf16(rng, (cols,), 0.5)
    _, rms = orc.rms_norm(w, X, 1e-5)
    ref_dX, ref_xout = orc.rms_norm_bwd_x(rms, w, X, up, dX0, want_x_out=True)
    ref_dW = orc.rms_norm_bwd_w(rms, X, up, dW0)
    Xd, wd, upd, rmsd = dev_bf16(X), dev_bf16(w), dev_bf16(up), torch.from_numpy(rms).cuda()
    dX, xout = dev_bf16(dX0), torch.zeros_like(Xd)
    ops.rms_norm_bwd_x(rows, cols, 1e-5, rmsd, wd, Xd, upd, dX, xout)
    assert_close(_f32(host_bits(dX)), _f32(ref_dX), what="rms_norm_bwd_x dX (accumulated)")
    assert_close(_f32(host_bits(xout)), _f32(ref_xout), what="rms_norm_bwd_x X_out")
    dXb = dev_bf16(dX0)
    ops.rms_norm_bwd_x(rows, cols, 1e-5, rmsd, wd, Xd, upd, dXb, None)
    assert torch.equal(dX, dXb)
    # weight gradient: with the workspace that fills the GPU and with one that holds three slices only
    full = ops.rms_norm_bwd_w_workspace_bytes(rows, cols)
    results = []
    for nbytes in (full, 3 * cols * 4):
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        dW = dev_bf16(dW0)
        ops.rms_norm_bwd_w(rows, cols, 1e-5, rmsd, Xd, upd, dW, ws)
        assert_chain_close(_f32(host_bits(dW)), _f32(ref_dW), limit=4e-3, what="rms_norm_bwd_w")
        assert_close(_f32(host_bits(dW)), _f32(ref_dW), rtol=2e-2, atol=2e-2, what="rms_norm_bwd_w")
        results.append(dW)
    # the same launch twice gives the same bits (fixed summation order)
    ws = torch.empty(full, dtype=torch.uint8, device="cuda")
    again = dev_bf16(dW0)
    ops.rms_norm_bwd_w(rows, cols, 1e-5, rmsd, Xd, upd, again, ws)
    assert torch.equal(again, results[0])
    with pytest.raises(RuntimeError):
        ops.rms_norm_bwd_w(rows, cols, 1e-5, rmsd, Xd, upd, again, torch.empty(cols * 4 - 4, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("tokens,heads,kv_heads,head_dim,theta", [(300, 16, 4, 128, 500000), (77, 8, 8, 64, 10000),
                                                                  (5, 2, 1, 256, 10000)])
def test_rope_forward_backward(env, tokens, heads, kv_heads, head_dim, theta):
    torch, ops, orc = env
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close

    rng = np.random.default_rng(tokens + head_dim)
    q, k = rand_bf16(rng, (tokens, heads * head_dim)), rand_bf16(rng, (tokens, kv_heads * head_dim))
    pos = rng.integers(0, 8192, size=tokens).astype(np.int32)
    pos[:3] = [0, 1, 8191][: min(3, tokens)]
    posd = torch.from_numpy(pos).cuda()
    for backward in (False, True):
        ref_q, ref_k = orc.rope(head_dim, kv_heads, theta, pos, q, k, backward=backward)
        qd, kd = dev_bf16(q), dev_bf16(k)
        (ops.rope_bwd_x if backward else ops.rope)(tokens, heads * head_dim, head_dim, kv_heads, theta, posd, qd, kd)
        # libm on the host and CUDA's sincosf / powf agree to a few ulp of the angle; at 8191 rad that is 1e-3 in sin
        assert_close(_f32(host_bits(qd)), _f32(ref_q), rtol=2e-2, atol=4e-3, what="rope q")
        assert_close(_f32(host_bits(kd)), _f32(ref_k), rtol=2e-2, atol=4e-3, what="rope k")
        qd2 = dev_bf16(q)
        (ops.rope_bwd_x if backward else ops.rope)(tokens, heads * head_dim, head_dim, kv_heads, theta, posd, qd2, None)
        assert torch.equal(qd, qd2)
    # position 0 is the identity; forward then backward returns the input up to two roundings
    qd = dev_bf16(q)
    ops.rope(tokens, heads * head_dim, head_dim, kv_heads, theta, posd, qd, None)
    assert np.array_equal(host_bits(qd)[0], q[0])
    ops.rope_bwd_x(tokens, heads * head_dim, head_dim, kv_heads, theta, posd, qd, None)
    assert_close(_f32(host_bits(qd)), _f32(q), rtol=2e-2, atol=2e-2, what="rope round trip")


@pytest.mark.parametrize("rows,cols", [(40, 128256), (300, 4096), (7, 50304), (3, 1001), (2, 5)])
def test_softmax_cross_entropy_average(env, rows, cols):
    torch, ops, orc = env
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close

    rng = np.random.default_rng(rows + cols)
    X = rand_bf16(rng, (rows, cols), 2.0)
    labels = rng.integers(0, cols, size=rows).astype(np.uint32)
    ref_p = orc.softmax(X)
    Xd = dev_bf16(X)
    p = torch.zeros_like(Xd)
    ops.softmax(rows, cols, Xd, p)
    assert_close(_f32(host_bits(p)), _f32(ref_p), rtol=2e-2, atol=1e-6, what="softmax")
    sums = p.float().sum(dim=1).cpu().numpy()
    np.testing.assert_allclose(sums, 1.0, atol=5e-3)
    # in place
    Xi = dev_bf16(X)
    ops.softmax(rows, cols, Xi, Xi)
    assert torch.equal(Xi, p)
    # loss and gradient on identical probabilities (the oracle's): the label entry is bf16 arithmetic, bit-exact
    ref_g, ref_loss = orc.cross_entropy_loss(ref_p, labels)
    pd = dev_bf16(ref_p)
    loss = torch.zeros(rows + 1, dtype=torch.float32, device="cuda")
    ops.cross_entropy_loss(rows, cols, pd, torch.from_numpy(labels.view(np.int32)).cuda(), loss)
    ops.set_average_loss(rows, loss)
    assert np.array_equal(host_bits(pd), ref_g)
    np.testing.assert_allclose(loss.cpu().numpy(), ref_loss, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("n,step", [(1 << 20, 1), (1000003, 7), (5, 300)])
def test_adamw_step(env, n, step):
    torch, ops, orc = env
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close

    rng = np.random.default_rng(n + step)
    param, grad = rand_bf16(rng, (n,), 0.02), rand_bf16(rng, (n,), 1e-2)
    mean, var = rand_bf16(rng, (n,), 1e-2), orc.to_bf16(np.abs(rng.standard_normal(n).astype(np.float32)) * 1e-4)
    hp = dict(lr=3e-4, b1=0.9, b2=0.95, wd=0.1, eps=1e-8)
    rp, rm, rv = orc.adamw_step(step, hp["lr"], hp["b1"], hp["b2"], hp["wd"], hp["eps"], param, grad, mean, var)
    pd, gd, md, vd = dev_bf16(param), dev_bf16(grad), dev_bf16(mean), dev_bf16(var)
    ops.adamw_step(n, step, hp["lr"], hp["b1"], hp["b2"], hp["wd"], hp["eps"], pd, gd, md, vd)
    for got, ref, what in ((pd, rp, "param"), (md, rm, "mean"), (vd, rv, "var")):
        g, r = host_bits(got), ref
        # the same fp32 formula on both sides, but the compilers fuse multiply-adds differently: an element whose
        # fp32 value sits next to a bf16 rounding boundary may land on the other side (one bf16 ulp), most do not
        assert (g != r).mean() < 2e-2, what
        assert_close(_f32(g), _f32(r), rtol=1e-2, atol=1e-8, what=what)
    with pytest.raises(RuntimeError):
        ops.adamw_step(n, 0, hp["lr"], hp["b1"], hp["b2"], hp["wd"], hp["eps"], pd, gd, md, vd)


@pytest.mark.parametrize("tokens,vocab,dim", [(4096, 1000, 2048), (333, 128256, 256), (64, 7, 64)])
def test_embedding_forward_backward(env, tokens, vocab, dim):
    torch, ops, orc = env
    from gpu_util import dev, dev_bf16, host_bits, rand_bf16

    rng = np.random.default_rng(tokens + vocab)
    ids = rng.integers(0, vocab, size=tokens).astype(np.uint32)
    ids[: tokens // 4] = ids[0]  # a heavily repeated token
    table = rand_bf16(rng, (vocab, dim), 0.02)
    sorted_ids, mapping, starts = orc.sort_tokens(ids)
    nu = len(starts) - 1
    as_dev = lambda a: torch.from_numpy(a.view(np.int32)).cuda()
    out = torch.zeros((tokens, dim), dtype=torch.bfloat16, device="cuda")
    ops.embedding_table(nu, dim, as_dev(sorted_ids), as_dev(mapping), as_dev(starts), dev_bf16(table), out)
    assert np.array_equal(host_bits(out), table[ids])
    assert np.array_equal(host_bits(out), orc.embedding_table(sorted_ids, mapping, starts, table, tokens))
    grad_stream, gtab0 = rand_bf16(rng, (tokens, dim), 1.0), rand_bf16(rng, (vocab, dim), 0.5)
    ref = orc.embedding_table_bwd_w(sorted_ids, mapping, starts, grad_stream, gtab0)
    gtab = dev_bf16(gtab0)
    ops.embedding_table_bwd_w(nu, dim, as_dev(sorted_ids), as_dev(mapping), as_dev(starts), dev_bf16(grad_stream), gtab)
    assert np.array_equal(host_bits(gtab), ref)


def test_block_ops_reject_bad_arguments(env):
    torch, ops, orc = env
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    import ctypes as C

    p = C.c_void_p(x.data_ptr())
    assert lib.b200_rms_norm(3, 4, 64, 1e-5, p, p, p, None, None) == -1       # fp32 is not implemented
    assert lib.b200_rms_norm(5, 4, 60, 1e-5, p, p, p, None, None) == -1       # columns not a multiple of 8
    assert lib.b200_rms_norm(5, 4, 64, 1e-5, p, C.c_void_p(x.data_ptr() + 2), p, None, None) == -1  # unaligned
    assert lib.b200_rope(5, 4, 64, 48, 1, 10000, p, p, None, None) == -1      # head_dim does not divide model_dim
    assert lib.b200_rms_norm(5, 0, 64, 1e-5, p, p, p, None, None) == 0        # no rows: nothing to do
