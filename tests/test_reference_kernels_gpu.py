"""GPU: pins the CPU oracle against the reference's OWN kernels.

`oracle/_ref/ref_*.cubin` are the reference's MoE and SwiGLU kernels compiled from its sources in place
(`make -C oracle ref`; built where the reference tree exists, shipped as binaries). They are loaded with the CUDA
driver API and launched with the reference's launch shapes
(backends/nvidia/src/ops/src/native/src/moe/moe_config.c) on well-formed inputs. The oracle must reproduce:
  * select_experts (fp32): chosen_experts slot for slot, counts, exclusive cumsum - bit-exact; gate weights to 1e-5
    (the reference is built with --use_fast_math);
  * build_expert_mapping: the same rows per expert as a set (the reference's order inside an expert is atomic
    arrival order), inclusive cumsum;
  * prepare_experts / merge_experts / router_bwd_x / router_gate_bwd_x / swiglu / swiglu_bwd_x on the oracle's own
    mapping: bit-exact copies, tolerance for arithmetic.
This is the check that the restatement in oracle/moe_oracle.c says what the reference's kernels do.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


class Driver:
    def __init__(self):
        self.cu = C.CDLL("libcuda.so.1")
        self.modules = {}

    def function(self, cubin, name):
        if cubin not in self.modules:
            mod = C.c_void_p()
            rc = self.cu.cuModuleLoad(C.byref(mod), os.path.join(REF_DIR, cubin).encode())
            assert rc == 0, f"cuModuleLoad({cubin}) -> {rc}"
            self.modules[cubin] = mod
        fn = C.c_void_p()
        rc = self.cu.cuModuleGetFunction(C.byref(fn), self.modules[cubin], name.encode())
        assert rc == 0, f"cuModuleGetFunction({name}) -> {rc}"
        return fn

    def launch(self, fn, grid, block, smem, stream, args):
        """args: list of ctypes scalars (c_int / c_void_p)."""
        arr = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])
        rc = self.cu.cuLaunchKernel(fn, grid, 1, 1, block, 1, 1, smem, C.c_void_p(stream), arr, None)
        assert rc == 0, f"cuLaunchKernel -> {rc}"


@pytest.fixture(scope="module")
def drv():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if not os.path.exists(os.path.join(REF_DIR, "ref_select_experts.cubin")):
        pytest.skip("reference cubins are built only where the reference tree is present")
    torch.cuda.init()
    torch.zeros(1, device="cuda")  # make the primary context current for the driver API
    return Driver()


def _ptr(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("T,E,k", [(4096, 64, 8), (5000, 16, 2), (4097, 64, 1)])
@pytest.mark.parametrize("ties", [False, True])
def test_reference_select_experts_and_mapping(drv, oracle, T, E, k, ties):
    import torch
    from gpu_util import host_u16

    rng = np.random.default_rng(T + E + k + ties)
    if ties:
        logits = rng.integers(-3, 4, size=(T, E)).astype(np.float32)  # heavy ties: the tie rule decides
    else:
        logits = rng.standard_normal((T, E), dtype=np.float32)
    lg = torch.from_numpy(logits).cuda()
    w = torch.zeros((T, k), dtype=torch.float32, device="cuda")
    ch = torch.zeros((T, k), dtype=torch.int16, device="cuda")
    counts = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    cumsum = torch.zeros(E, dtype=torch.int32, device="cuda")
    hostc = torch.zeros(E, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    warps = 8
    smem = E * 4 + warps * (32 * 4 + k * 4 + k * 2)
    fn = drv.function("ref_select_experts.cubin", "default_select_experts_fp32_kernel")
    drv.launch(fn, sm, warps * 32, smem, stream,
               [C.c_int(T), C.c_int(E), C.c_int(k), _ptr(lg), _ptr(w), _ptr(ch), _ptr(counts), _ptr(cumsum), _ptr(hostc)])
    torch.cuda.synchronize()
    ow, och, ocounts, ocexcl, _ = oracle.select_experts(logits, k)
    np.testing.assert_array_equal(host_u16(ch), och)
    np.testing.assert_array_equal(counts.cpu().numpy()[:E], ocounts[:E])
    np.testing.assert_array_equal(cumsum.cpu().numpy(), ocexcl)
    np.testing.assert_array_equal(hostc.cpu().numpy(), ocounts[:E])
    np.testing.assert_allclose(w.cpu().numpy(), ow, rtol=1e-5, atol=1e-6)

    # build_expert_mapping: same rows per expert, any order inside an expert
    em = torch.full((T * k,), -1, dtype=torch.int32, device="cuda")
    tm = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
    fn = drv.function("ref_build_expert_mapping.cubin", "default_build_expert_mapping_kernel")
    drv.launch(fn, (T + 255) // 256, 256, 0, stream,
               [C.c_int(T), C.c_int(E), C.c_int(k), _ptr(ch), _ptr(cumsum), _ptr(em), _ptr(tm)])
    torch.cuda.synchronize()
    oem, otm, ocincl = oracle.build_expert_mapping(och, E, ocexcl)
    np.testing.assert_array_equal(cumsum.cpu().numpy(), ocincl)
    em_h, tm_h = em.cpu().numpy(), tm.cpu().numpy()
    np.testing.assert_array_equal(np.sort(tm_h.reshape(-1)), np.arange(T * k))
    np.testing.assert_array_equal(em_h[tm_h.reshape(-1)], np.repeat(np.arange(T), k))
    base = 0
    for e in range(E):
        n = int(ocounts[e])
        np.testing.assert_array_equal(np.sort(em_h[base:base + n]), np.sort(oem[base:base + n]))
        base += n


def test_reference_permute_combine_and_router_backward(drv, oracle):
    import torch
    from gpu_util import dev, dev_bf16, host_bits, rand_bf16
    from helpers import assert_close, bf16_bits_to_f32

    T, d, E, k = 700, 1024, 16, 4
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    w, ch, counts, cexcl, _ = oracle.select_experts(logits, k)
    em, tm, cincl = oracle.build_expert_mapping(ch, E, cexcl)
    X, Y, resid, dOut = (rand_bf16(rng, s) for s in ((T, d), (T * k, d), (T, d), (T, d)))
    stream = torch.cuda.current_stream().cuda_stream
    tmd, wd, chd, emd, cid = dev(tm), torch.from_numpy(w).cuda(), dev(ch), dev(em), dev(cincl)

    zone = torch.zeros((T * k, d), dtype=torch.bfloat16, device="cuda")
    Xd = dev_bf16(X)
    fn = drv.function("ref_prepare_expert_zone.cubin", "default_prepare_experts_bf16_bf16_kernel")
    drv.launch(fn, T, 128, d * 2, stream, [C.c_int(T), C.c_int(d), C.c_int(k), _ptr(Xd), _ptr(tmd), _ptr(zone)])
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host_bits(zone), oracle.prepare_experts(X, tm))

    for weights in (w, None):
        out = dev_bf16(resid.copy())
        Yd = dev_bf16(Y)
        fn = drv.function("ref_merge_expert_result.cubin", "default_merge_experts_bf16_bf16_kernel")
        wptr = _ptr(wd) if weights is not None else C.c_void_p(0)
        drv.launch(fn, T, 128, d * 4, stream, [C.c_int(T), C.c_int(d), C.c_int(k), _ptr(Yd), _ptr(tmd), wptr, _ptr(out)])
        torch.cuda.synchronize()
        ref = oracle.merge_experts(Y, tm, weights, resid.copy())
        assert_close(bf16_bits_to_f32(host_bits(out)), bf16_bits_to_f32(ref), rtol=1e-2, atol=1e-3, what="merge_experts")

    # router_bwd_x per expert, then the gate Jacobian
    dXr = torch.zeros((T, E), dtype=torch.bfloat16, device="cuda")
    dXr_ref = np.zeros((T, E), np.uint16)
    zone2 = dev_bf16(Y.copy())
    zone_ref = Y.copy()
    dOd = dev_bf16(dOut)
    fn = drv.function("ref_router_bwd_x.cubin", "default_router_bwd_x_bf16_bf16_kernel")
    for e in range(E):
        n, b = int(counts[e]), int(cexcl[e])
        if n == 0:
            continue
        ze = np.ascontiguousarray(zone_ref[b:b + n])
        oracle.router_bwd_x(n, d, E, k, e, cincl, em, ch, w, ze, dOut, dXr_ref, ze)
        zone_ref[b:b + n] = ze
        zptr = C.c_void_p(zone2.data_ptr() + b * d * 2)
        drv.launch(fn, n, 256, d * 2 + 33 * 4, stream,
                   [C.c_int(n), C.c_int(d), C.c_int(E), C.c_int(k), C.c_int(e), _ptr(cid), _ptr(emd), _ptr(chd), _ptr(wd),
                    zptr, _ptr(dOd), _ptr(dXr), zptr])
    torch.cuda.synchronize()
    assert_close(bf16_bits_to_f32(host_bits(dXr)), bf16_bits_to_f32(dXr_ref), rtol=2e-2, atol=2e-2, what="dX_routed")
    # the reference multiplies by the gate weight rounded to bf16, in bf16 (router_bwd_x.cu:83-86)
    assert_close(bf16_bits_to_f32(host_bits(zone2)), bf16_bits_to_f32(zone_ref), rtol=2e-2, atol=1e-3, what="scaled rows")
    fn = drv.function("ref_router_gate_bwd_x.cubin", "default_router_gate_bwd_x_bf16_bf16_kernel")
    pre = host_bits(dXr).copy()
    drv.launch(fn, T, 32, 0, stream, [C.c_int(T), C.c_int(E), C.c_int(k), _ptr(chd), _ptr(wd), _ptr(dXr)])
    torch.cuda.synchronize()
    assert_close(bf16_bits_to_f32(host_bits(dXr)), bf16_bits_to_f32(oracle.router_gate_bwd_x(ch, w, pre)), what="gate bwd")


def test_reference_swiglu(drv, oracle):
    import torch
    from gpu_util import dev_bf16, host_bits, rand_bf16
    from helpers import assert_close, bf16_bits_to_f32

    rows, cols = 300, 1408
    rng = np.random.default_rng(8)
    x1, x3, dy = rand_bf16(rng, (rows, cols), 2.0), rand_bf16(rng, (rows, cols)), rand_bf16(rng, (rows, cols))
    stream = torch.cuda.current_stream().cuda_stream
    out, d1, d3 = (torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda") for _ in range(3))
    a, b, g = dev_bf16(x1), dev_bf16(x3), dev_bf16(dy)
    fn = drv.function("ref_swiglu.cubin", "default_swiglu_bf16_kernel")
    drv.launch(fn, rows, 256, 0, stream, [C.c_int(rows), C.c_int(cols), _ptr(a), _ptr(b), _ptr(out)])
    fn = drv.function("ref_swiglu_bwd_x.cubin", "default_swiglu_bwd_x_bf16_bf16_kernel")
    drv.launch(fn, rows, 256, 0, stream, [C.c_int(rows), C.c_int(cols), _ptr(a), _ptr(b), _ptr(g), _ptr(d1), _ptr(d3)])
    torch.cuda.synchronize()
    assert_close(bf16_bits_to_f32(host_bits(out)), bf16_bits_to_f32(oracle.swiglu(x1, x3)), what="swiglu")
    r1, r3 = oracle.swiglu_bwd_x(x1, x3, dy)
    assert_close(bf16_bits_to_f32(host_bits(d1)), bf16_bits_to_f32(r1), what="dx1")
    assert_close(bf16_bits_to_f32(host_bits(d3)), bf16_bits_to_f32(r3), what="dx3")
