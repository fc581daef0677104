"""GPU: pins the block-op oracle (oracle/block_oracle.c) against the reference's OWN kernels.

`oracle/_ref/ref_*.cubin` are the reference's norm / rope / loss / optimizer / embedding kernels compiled from its
sources in place with its own flags (`make -C oracle ref`; built where the reference tree exists, shipped as binaries),
loaded with the CUDA driver API and launched with the reference's launch shapes
(backends/nvidia/src/ops/src/native/src/norm/rms_norm_config.c, attention_misc/attn_misc_config.c,
loss_misc/loss_misc_config.c, optimizer/adamw_step_config.c, preprocess/embedding_table_config.c).

The reference is built with --use_fast_math: its expf, powf, sincosf and divisions are the approximate hardware forms.
The oracle uses libm, so floating-point results are compared to the bf16 tolerance of the layer; for RoPE the
reference's fast sine/cosine lose about |angle| * 2^-22 of absolute accuracy (1e-3 .. 2e-3 at positions of a few
thousand), which the comparison allows for explicitly. Copies and bf16 arithmetic in a fixed order (embedding, the
label entry of the cross-entropy) must be bit-exact.
"""
import ctypes as C
import os

import numpy as np
import pytest

from test_reference_kernels_gpu import REF_DIR, Driver, _ptr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def drv():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if not os.path.exists(os.path.join(REF_DIR, "ref_rms_norm.cubin")):
        pytest.skip("reference cubins are built only where the reference tree is present")
    torch.cuda.init()
    torch.zeros(1, device="cuda")
    return Driver()


def _f32(bits):
    from helpers import bf16_bits_to_f32

    return bf16_bits_to_f32(bits)


def _sm_count():
    import torch

    return torch.cuda.get_device_properties(0).multi_processor_count


def test_reference_rms_norm_forward_backward(drv, oracle):
    import torch
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_chain_close, assert_close

    rows, cols, eps = 300, 2048, 1e-5
    rng = np.random.default_rng(5)
    X, w = rand_bf16(rng, (rows, cols), 1.5), rand_bf16(rng, (cols,), 1.0)
    up, dX0, dW0 = rand_bf16(rng, (rows, cols)), rand_bf16(rng, (rows, cols), 0.5), rand_bf16(rng, (cols,), 0.5)
    Xd, wd, upd = dev_bf16(X), dev_bf16(w), dev_bf16(up)
    out = torch.zeros_like(Xd)
    rms = torch.zeros(rows, dtype=torch.float32, device="cuda")
    fn = drv.function("ref_rms_norm.cubin", "default_rms_norm_bf16_kernel")
    drv.launch(fn, rows, 256, 4 * cols + 128, 0, [C.c_int(rows), C.c_int(cols), C.c_float(eps), _ptr(wd), _ptr(Xd), _ptr(out),
                                                   _ptr(rms)])
    torch.cuda.synchronize()
    ref_out, ref_rms = oracle.rms_norm(w, X, eps)
    np.testing.assert_allclose(rms.cpu().numpy(), ref_rms, rtol=1e-5)
    assert_close(_f32(host_bits(out)), _f32(ref_out), what="reference rms_norm vs oracle")
    # backward-x on the reference's own rms values
    dX, xout = dev_bf16(dX0), torch.zeros_like(Xd)
    fn = drv.function("ref_rms_norm_bwd_x.cubin", "default_rms_norm_bwd_x_bf16_bf16_kernel")
    drv.launch(fn, rows, 256, 4 * cols + 128, 0, [C.c_int(rows), C.c_int(cols), C.c_float(eps), _ptr(rms), _ptr(wd), _ptr(Xd),
                                                   _ptr(upd), _ptr(dX), _ptr(xout)])
    torch.cuda.synchronize()
    ref_dX, ref_xout = oracle.rms_norm_bwd_x(rms.cpu().numpy(), w, X, up, dX0, want_x_out=True)
    assert_close(_f32(host_bits(dX)), _f32(ref_dX), what="reference rms_norm_bwd_x vs oracle")
    assert_close(_f32(host_bits(xout)), _f32(ref_xout), what="reference rms_norm_bwd_x X_out vs oracle")
    # backward-w: partial sums per block, then the combine kernel
    blocks = min(_sm_count(), rows)
    per_block = -(-rows // blocks)
    ws = torch.zeros((blocks, cols), dtype=torch.float32, device="cuda")
    nblk = torch.zeros(1, dtype=torch.int32, device="cuda")
    dW = dev_bf16(dW0)
    fn = drv.function("ref_rms_norm_bwd_w.cubin", "default_rms_norm_bwd_w_bf16_bf16_kernel")
    drv.launch(fn, blocks, 1024, 4 * cols + 4 * per_block, 0, [C.c_int(rows), C.c_int(cols), C.c_float(eps), _ptr(rms), _ptr(Xd),
                                                                _ptr(upd), _ptr(ws), _ptr(nblk)])
    fn = drv.function("ref_rms_norm_bwd_w_combine.cubin", "default_rms_norm_bwd_w_combine_bf16_kernel")
    drv.launch(fn, -(-cols // 32), 1024, 0, 0, [_ptr(nblk), C.c_int(cols), _ptr(ws), _ptr(dW)])
    torch.cuda.synchronize()
    assert int(nblk.item()) == blocks
    ref_dW = oracle.rms_norm_bwd_w(rms.cpu().numpy(), X, up, dW0)
    assert_chain_close(_f32(host_bits(dW)), _f32(ref_dW), limit=4e-3, what="reference rms_norm_bwd_w vs oracle")


@pytest.mark.parametrize("backward", [False, True])
def test_reference_rope(drv, oracle, backward):
    import torch
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close_with_slack

    tokens, heads, kv_heads, head_dim, theta = 300, 16, 4, 128, 500000
    rng = np.random.default_rng(9 + backward)
    q, k = rand_bf16(rng, (tokens, heads * head_dim)), rand_bf16(rng, (tokens, kv_heads * head_dim))
    pos = rng.integers(0, 8192, size=tokens).astype(np.int32)
    pos[:2] = [0, 8191]
    qd, kd, posd = dev_bf16(q), dev_bf16(k), torch.from_numpy(pos).cuda()
    name = "default_rope_bwd_x_bf16_kernel" if backward else "default_rope_bf16_kernel"
    fn = drv.function("ref_rope_bwd_x.cubin" if backward else "ref_rope.cubin", name)
    drv.launch(fn, tokens, 128, 0, 0, [C.c_int(tokens), C.c_int(heads * head_dim), C.c_int(head_dim), C.c_int(kv_heads),
                                       C.c_int(theta), _ptr(posd), _ptr(qd), _ptr(kd)])
    torch.cuda.synchronize()
    ref_q, ref_k = oracle.rope(head_dim, kv_heads, theta, pos, q, k, backward=backward)
    # fast-math sine / cosine: absolute error of about |angle| * 2^-21 in each, times the magnitude of the pair
    for got, ref, src, what in ((qd, ref_q, q, "q"), (kd, ref_k, k, "k")):
        mag = np.abs(_f32(src)).reshape(tokens, -1, 2).sum(axis=2).repeat(2, axis=1)
        slack = mag * (pos.astype(np.float64)[:, None] * 2.0 ** -21 + 2e-3)
        assert_close_with_slack(_f32(host_bits(got)), _f32(ref), slack, what=f"reference rope {what} vs oracle")
    # positions where the angle is small agree to the plain tolerance
    small = pos < 64
    if small.any():
        from helpers import assert_close

        assert_close(_f32(host_bits(qd))[small], _f32(ref_q)[small], rtol=2e-2, atol=4e-3, what="reference rope (small angles)")


def test_reference_softmax_and_cross_entropy(drv, oracle):
    import torch
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close

    rows, cols = 24, 128256
    rng = np.random.default_rng(11)
    X = rand_bf16(rng, (rows, cols), 2.0)
    labels = rng.integers(0, cols, size=rows).astype(np.uint32)
    Xd = dev_bf16(X)
    p = torch.zeros_like(Xd)
    fn = drv.function("ref_softmax.cubin", "default_softmax_bf16_bf16_kernel")
    drv.launch(fn, rows, 1024, 0, 0, [C.c_int(rows), C.c_int(cols), _ptr(Xd), _ptr(p)])
    torch.cuda.synchronize()
    assert_close(_f32(host_bits(p)), _f32(oracle.softmax(X)), rtol=2e-2, atol=1e-6, what="reference softmax vs oracle")
    # cross-entropy on the reference's own probabilities: loss to fp32 tolerance (fast logf), gradient entry bit-exact
    probs = host_bits(p).copy()
    ref_g, ref_loss = oracle.cross_entropy_loss(probs, labels)
    loss = torch.zeros(rows + 1, dtype=torch.float32, device="cuda")
    lab = torch.from_numpy(labels.view(np.int32)).cuda()
    fn = drv.function("ref_cross_entropy.cubin", "default_cross_entropy_loss_bf16_kernel")
    drv.launch(fn, _sm_count(), 256, 0, 0, [C.c_int(rows), C.c_int(cols), _ptr(p), _ptr(lab), _ptr(loss)])
    fn = drv.function("ref_cross_entropy.cubin", "default_set_average_loss_kernel")
    drv.launch(fn, 1, 1024, 0, 0, [C.c_int(rows), _ptr(loss)])
    torch.cuda.synchronize()
    assert np.array_equal(host_bits(p), ref_g)
    np.testing.assert_allclose(loss.cpu().numpy(), ref_loss, rtol=1e-4, atol=1e-5)


def test_reference_adamw(drv, oracle):
    import torch
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close

    n, step = 1 << 20, 3
    rng = np.random.default_rng(13)
    param, grad, mean = rand_bf16(rng, (n,), 0.02), rand_bf16(rng, (n,), 1e-2), rand_bf16(rng, (n,), 1e-2)
    var = oracle.to_bf16(np.abs(rng.standard_normal(n).astype(np.float32)) * 1e-4)
    lr, b1, b2, wd, eps = 3e-4, 0.9, 0.95, 0.1, 1e-8
    pd, gd, md, vd = dev_bf16(param), dev_bf16(grad), dev_bf16(mean), dev_bf16(var)
    fn = drv.function("ref_adamw_step.cubin", "default_adamw_step_bf16_bf16_bf16_bf16_kernel")
    drv.launch(fn, _sm_count(), 1024, 0, 0, [C.c_uint64(n), C.c_int(step), C.c_float(lr), C.c_float(b1), C.c_float(b2),
                                            C.c_float(wd), C.c_float(eps), _ptr(pd), _ptr(gd), _ptr(md), _ptr(vd)])
    torch.cuda.synchronize()
    rp, rm, rv = oracle.adamw_step(step, lr, b1, b2, wd, eps, param, grad, mean, var)
    for got, ref, what in ((pd, rp, "param"), (md, rm, "mean"), (vd, rv, "var")):
        assert_close(_f32(host_bits(got)), _f32(ref), rtol=1e-2, atol=1e-8, what=f"reference adamw {what} vs oracle")
        assert (host_bits(got) != ref).mean() < 2e-2, what


def test_reference_embedding(drv, oracle):
    import torch
    from gpu_util import dev_bf16, host_bits, rand_bf16

    tokens, vocab, dim = 2048, 500, 1024
    rng = np.random.default_rng(17)
    ids = rng.integers(0, vocab, size=tokens).astype(np.uint32)
    ids[:300] = ids[0]
    table = rand_bf16(rng, (vocab, dim), 0.02)
    sorted_ids, mapping, starts = oracle.sort_tokens(ids)
    nu = len(starts) - 1
    as_dev = lambda a: torch.from_numpy(a.view(np.int32)).cuda()
    sid, smap, sst, tab = as_dev(sorted_ids), as_dev(mapping), as_dev(starts), dev_bf16(table)
    out = torch.zeros((tokens, dim), dtype=torch.bfloat16, device="cuda")
    fn = drv.function("ref_embedding_table.cubin", "default_embedding_table_bf16_kernel")
    drv.launch(fn, nu, 1024, 2 * dim, 0, [C.c_int(nu), C.c_int(dim), _ptr(sid), _ptr(smap), _ptr(sst), _ptr(tab), _ptr(out)])
    torch.cuda.synchronize()
    assert np.array_equal(host_bits(out), oracle.embedding_table(sorted_ids, mapping, starts, table, tokens))
    grad_stream, gtab0 = rand_bf16(rng, (tokens, dim), 1.0), rand_bf16(rng, (vocab, dim), 0.5)
    gs, gtab = dev_bf16(grad_stream), dev_bf16(gtab0)
    fn = drv.function("ref_embedding_table_bwd_w.cubin", "default_embedding_table_bwd_w_bf16_kernel")
    drv.launch(fn, nu, 1024, 2 * dim, 0, [C.c_int(nu), C.c_int(dim), _ptr(sid), _ptr(smap), _ptr(sst), _ptr(gs), _ptr(gtab)])
    torch.cuda.synchronize()
    assert np.array_equal(host_bits(gtab), oracle.embedding_table_bwd_w(sorted_ids, mapping, starts, grad_stream, gtab0))
