"""GPU: the scratch-free build_expert_mapping entry point against the regular one.

b200_build_expert_mapping_static serves callers that have no way to pass device scratch (an op slot with a fixed
argument list) and may not allocate while submitting work; its tables live in an array inside the library. The
test drives both entry points straight through the C ABI on the same inputs and demands identical integers, twice
in a row with different routing so that the second call runs over what the first one left in the array. It also
checks that an oversized problem is refused. This file sorts last on purpose: a failure here cannot hide any other
test when pytest stops at the first failure, and the test is self-contained so it also passes on its own.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _run_both(lib, chosen_np, E, cumsum_excl_np):
    T, k = chosen_np.shape
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    chosen = torch.from_numpy(chosen_np.view(np.int16)).cuda()
    results = []
    for variant in ("scratch", "static"):
        cumsum = torch.from_numpy(cumsum_excl_np.copy()).cuda()
        em = torch.full((T * k,), -3, dtype=torch.int32, device="cuda")
        tm = torch.full((T, k), -3, dtype=torch.int32, device="cuda")
        if variant == "scratch":
            nbytes = lib.b200_build_expert_mapping_workspace_bytes(T, E, k)
            ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            rc = lib.b200_build_expert_mapping(T, E, k, _ptr(chosen), _ptr(cumsum), _ptr(em), _ptr(tm), _ptr(ws),
                                               nbytes, stream)
        else:
            rc = lib.b200_build_expert_mapping_static(T, E, k, _ptr(chosen), _ptr(cumsum), _ptr(em), _ptr(tm), stream)
        assert rc == 0
        torch.cuda.synchronize()
        results.append((em.cpu().numpy(), tm.cpu().numpy(), cumsum.cpu().numpy()))
    return results


def test_static_scratch_mapping_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    E, k = 64, 8
    rng = np.random.default_rng(2024)
    for T in (4096, 1537):  # two calls in a row; the second sees the first one's leftovers in the array
        chosen = np.argsort(rng.random((T, E)), axis=1)[:, :k].astype(np.uint16)
        counts = np.bincount(chosen.reshape(-1), minlength=E).astype(np.int32)
        excl = (np.cumsum(counts) - counts).astype(np.int32)
        (em_a, tm_a, cs_a), (em_b, tm_b, cs_b) = _run_both(lib, chosen, E, excl)
        np.testing.assert_array_equal(em_b, em_a)
        np.testing.assert_array_equal(tm_b, tm_a)
        np.testing.assert_array_equal(cs_b, cs_a)
        np.testing.assert_array_equal(cs_b, np.cumsum(counts))
        np.testing.assert_array_equal(np.sort(tm_b.reshape(-1)), np.arange(T * k))

    # a problem whose tables do not fit the built-in array is refused, nothing is launched
    cap = lib.b200_build_expert_mapping_static_capacity_bytes()
    T_big, E_big = 1 << 20, 4096
    assert lib.b200_build_expert_mapping_workspace_bytes(T_big, E_big, k) > cap
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.b200_build_expert_mapping_static(T_big, E_big, k, _ptr(dummy), _ptr(dummy), _ptr(dummy), _ptr(dummy),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -1
    torch.cuda.synchronize()
