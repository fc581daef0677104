"""The reference's own submitters driving the B200 kernels through the external-op adapter.

`oracle/_ref/libdropin.so` is built from the reference's sources in place (its op table, SHA-256 fingerprinting,
skeleton setters and `dataflow_submit_*` functions) plus a minimal handle; `libb200moe_dataflow.so` is this
repository's C adapter compiled against the reference's headers. Both are built where the reference tree exists and
travel as binaries. CPU: the adapter registers the twelve drop-in ops under the reference's fingerprints and three
additive grouped ops (all experts of one pass per call) under skeletons of the same style. GPU: calling the
reference's `dataflow_submit_default_select_experts`, `..._build_expert_mapping`, `..._prepare_experts`,
`dataflow_submit_matmul` and `..._merge_experts` produces the oracle's results.
"""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "oracle", "_ref", "libdropin.so")
ADAPTER = os.path.join(ROOT, "ml_dataflow_b200", "lib", "libb200moe_dataflow.so")
DATAFLOW_FP32, DATAFLOW_BF16, DATAFLOW_NONE = 3, 5, 0


def _load():
    if not (os.path.exists(DROPIN) and os.path.exists(ADAPTER)):
        pytest.skip("drop-in binaries are built only where the reference tree is present")
    lib = C.CDLL(DROPIN, mode=C.RTLD_GLOBAL)
    lib.dropin_create_handle.restype = C.c_void_p
    lib.dropin_create_handle.argtypes = [C.c_void_p, C.c_char_p]
    lib.dropin_num_ops.argtypes = [C.c_void_p]
    return lib


def test_adapter_registers_every_op_under_the_reference_fingerprints():
    lib = _load()
    h = lib.dropin_create_handle(None, ADAPTER.encode())
    assert h, "registration failed"
    assert lib.dropin_num_ops(h) == 15


@pytest.mark.gpu
def test_reference_submitters_reach_the_b200_kernels(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gpu_util import dev_bf16, host_bits, host_u16, rand_bf16
    from helpers import assert_close, bf16_bits_to_f32

    lib = _load()
    h = lib.dropin_create_handle(C.c_void_p(torch.cuda.current_stream().cuda_stream), ADAPTER.encode())
    assert h
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float

    def p(t):
        return vp(t.data_ptr())

    T, d, E, k = 300, 256, 16, 4
    rng = np.random.default_rng(17)
    X, Wr = rand_bf16(rng, (T, d)), rand_bf16(rng, (E, d), 0.05)
    Xd, Wrd = dev_bf16(X), dev_bf16(Wr)
    logits = torch.zeros((T, E), dtype=torch.float32, device="cuda")
    # router GEMM through dataflow_submit_matmul (bf16 x bf16 -> fp32, transa=1)
    lib.dataflow_submit_matmul.argtypes = [vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, f32, vp, vp,
                                           vp, vp, C.c_uint64, vp]
    rc = lib.dataflow_submit_matmul(h, 0, DATAFLOW_BF16, DATAFLOW_BF16, DATAFLOW_NONE, DATAFLOW_FP32, DATAFLOW_FP32, 1, 0,
                                    E, d, T, 1.0, 0.0, p(Wrd), p(Xd), None, p(logits), 0, None)
    assert rc == 0
    w = torch.zeros((T, k), dtype=torch.float32, device="cuda")
    ch = torch.zeros((T, k), dtype=torch.int16, device="cuda")
    counts = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    cumsum = torch.zeros(E, dtype=torch.int32, device="cuda")
    hostc = torch.zeros(E, dtype=torch.int32, device="cuda")
    lib.dataflow_submit_default_select_experts.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp]
    assert lib.dataflow_submit_default_select_experts(h, 0, DATAFLOW_FP32, T, E, k, p(logits), p(w), p(ch), p(counts),
                                                      p(cumsum), p(hostc)) == 0
    em = torch.zeros(T * k, dtype=torch.int32, device="cuda")
    tm = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    lib.dataflow_submit_default_build_expert_mapping.argtypes = [vp, i32, i32, i32, i32, vp, vp, vp, vp]
    assert lib.dataflow_submit_default_build_expert_mapping(h, 0, T, E, k, p(ch), p(cumsum), p(em), p(tm)) == 0
    zone = torch.zeros((T * k, d), dtype=torch.bfloat16, device="cuda")
    lib.dataflow_submit_default_prepare_experts.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp]
    assert lib.dataflow_submit_default_prepare_experts(h, 0, DATAFLOW_BF16, DATAFLOW_BF16, T, d, k, p(Xd), p(tm),
                                                       p(zone)) == 0
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    lib.dataflow_submit_default_merge_experts.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp]
    assert lib.dataflow_submit_default_merge_experts(h, 0, DATAFLOW_BF16, DATAFLOW_BF16, T, d, k, p(zone), p(tm), p(w),
                                                     p(out)) == 0
    # an op the backend does not implement for this dtype is refused with -1, like a missing table entry
    assert lib.dataflow_submit_default_prepare_experts(h, 0, DATAFLOW_FP32, DATAFLOW_FP32, T, d, k, p(Xd), p(tm),
                                                       p(zone)) == -1
    assert lib.dataflow_submit_default_select_experts(h, 5, DATAFLOW_FP32, T, E, k, p(logits), p(w), p(ch), p(counts),
                                                      p(cumsum), p(hostc)) == -1  # stream id out of range
    torch.cuda.synchronize()

    lg = logits.cpu().numpy()
    assert_close(lg, oracle.linear_fwd(X, Wr, out_dtype=np.float32), rtol=1e-3, atol=1e-3, what="logits")
    ow, och, ocounts, ocexcl, _ = oracle.select_experts(lg, k)
    oem, otm, ocincl = oracle.build_expert_mapping(och, E, ocexcl)
    np.testing.assert_array_equal(host_u16(ch), och)
    np.testing.assert_array_equal(counts.cpu().numpy()[:E], ocounts[:E])
    np.testing.assert_array_equal(hostc.cpu().numpy(), ocounts[:E])
    np.testing.assert_array_equal(cumsum.cpu().numpy(), ocincl)
    np.testing.assert_array_equal(tm.cpu().numpy(), otm)
    np.testing.assert_array_equal(em.cpu().numpy(), oem)
    np.testing.assert_array_equal(host_bits(zone), oracle.prepare_experts(X, otm))
    # identity experts: combining the gathered rows with the gate weights returns sum_j w_j * x = x
    ref = oracle.merge_experts(oracle.prepare_experts(X, otm), otm, w.cpu().numpy(), np.zeros((T, d), np.uint16))
    assert_close(bf16_bits_to_f32(host_bits(out)), bf16_bits_to_f32(ref), rtol=1e-2, atol=1e-3, what="merge")


@pytest.mark.gpu
def test_grouped_expert_ops_are_reached_through_submit_op():
    """The additive grouped ops go through handle->submit_op like every other op: the adapter's own submitters
    (dataflow_submit_b200_moe_experts_fwd / _bwd_x / _bwd_w) build the skeleton, the handle finds the registered
    function by fingerprint, and the results equal a direct call of the C ABI bit for bit."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ml_dataflow_b200 import ops

    lib = _load()
    h = lib.dropin_create_handle(C.c_void_p(torch.cuda.current_stream().cuda_stream), ADAPTER.encode())
    assert h
    ad = C.CDLL(ADAPTER)
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64

    def p(t):
        return None if t is None else vp(t.data_ptr())

    R, d, f, E = 900, 256, 192, 6
    g = torch.Generator(device="cuda").manual_seed(3)

    def nrm(shape, std):
        return (torch.randn(shape, generator=g, device="cuda") * std).to(torch.bfloat16)

    counts = torch.tensor([100, 0, 333, 200, 17, 250], dtype=torch.int32, device="cuda")
    cumsum = torch.cumsum(counts, 0).to(torch.int32)
    zone, dY = nrm((R, d), 1.0), nrm((R, d), 1.0)
    W1, W3, W2 = nrm((E, f, d), 0.05), nrm((E, f, d), 0.05), nrm((E, d, f), 0.05)
    roww = torch.rand((R,), generator=g, device="cuda") + 0.1

    def bufs():
        x = [torch.zeros((R, f), dtype=torch.bfloat16, device="cuda") for _ in range(5)]   # x1 x3 h dx1 dx3
        y = [torch.zeros((R, d), dtype=torch.bfloat16, device="cuda") for _ in range(2)]   # Y dZ
        gr = [torch.zeros_like(W1), torch.zeros_like(W3), torch.zeros_like(W2)]
        return x, y, gr, torch.zeros((R,), dtype=torch.float32, device="cuda")

    (x1, x3, hh, dx1, dx3), (Y, dZ), (dW1, dW3, dW2), dP = bufs()
    ops.moe_experts_fwd(R, d, f, E, zone, W1, W3, W2, f * d, f * d, d * f, counts, cumsum, x1, x3, hh, Y)
    ops.moe_experts_bwd_x(R, d, f, E, dY, roww, x1, x3, W1, W3, W2, f * d, f * d, d * f, counts, cumsum, dx1, dx3, None,
                          dP, dZ)
    ops.moe_experts_bwd_w(R, d, f, E, dY, hh, zone, dx1, dx3, dW1, dW3, dW2, f * d, f * d, d * f, counts, cumsum)
    (x1b, x3b, hb, dx1b, dx3b), (Yb, dZb), (dW1b, dW3b, dW2b), dPb = bufs()
    ad.dataflow_submit_b200_moe_experts_fwd.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, i64, i64, i64,
                                                        vp, vp, vp, vp, vp, vp]
    assert ad.dataflow_submit_b200_moe_experts_fwd(h, 0, DATAFLOW_BF16, R, d, f, E, p(zone), p(W1), p(W3), p(W2), f * d,
                                                   f * d, d * f, p(counts), p(cumsum), p(x1b), p(x3b), p(hb), p(Yb)) == 0
    ad.dataflow_submit_b200_moe_experts_bwd_x.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp,
                                                          i64, i64, i64, vp, vp, vp, vp, vp, vp, vp]
    assert ad.dataflow_submit_b200_moe_experts_bwd_x(h, 0, DATAFLOW_BF16, R, d, f, E, p(dY), p(roww), p(x1b), p(x3b),
                                                     p(W1), p(W3), p(W2), f * d, f * d, d * f, p(counts), p(cumsum),
                                                     p(dx1b), p(dx3b), None, p(dPb), p(dZb)) == 0
    ad.dataflow_submit_b200_moe_experts_bwd_w.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp,
                                                          vp, i64, i64, i64, vp, vp]
    assert ad.dataflow_submit_b200_moe_experts_bwd_w(h, 0, DATAFLOW_BF16, R, d, f, E, p(dY), p(hb), p(zone), p(dx1b),
                                                     p(dx3b), p(dW1b), p(dW3b), p(dW2b), f * d, f * d, d * f, p(counts),
                                                     p(cumsum)) == 0
    # an fp32 variant has no registered function: the lookup fails like any unknown op
    assert ad.dataflow_submit_b200_moe_experts_fwd(h, 0, DATAFLOW_FP32, R, d, f, E, p(zone), p(W1), p(W3), p(W2), f * d,
                                                   f * d, d * f, p(counts), p(cumsum), p(x1b), p(x3b), p(hb), p(Yb)) == -1
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0
    for a, b, what in [(x1, x1b, "x1"), (x3, x3b, "x3"), (hh, hb, "h"), (Y, Yb, "Y"), (dx1, dx1b, "dx1"), (dx3, dx3b, "dx3"),
                       (dZ, dZb, "dZ"), (dW1, dW1b, "dW1"), (dW3, dW3b, "dW3"), (dW2, dW2b, "dW2")]:
        assert torch.equal(a, b), what
    torch.testing.assert_close(dP, dPb, rtol=1e-4, atol=1e-4)  # fp32 atomics: equal up to summation order
