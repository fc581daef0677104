"""Helpers for the GPU parity tests: numpy (oracle side) <-> torch (device side) conversions."""
import numpy as np
import torch


def dev_bf16(bits):
    """uint16 bf16 bit patterns (numpy) -> cuda bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def host_bits(t):
    """cuda bf16 tensor -> uint16 bit patterns (numpy)."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def dev(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    return torch.from_numpy(a).cuda()


def host_u16(t):
    return t.detach().contiguous().cpu().numpy().view(np.uint16)


def rand_bf16(rng, shape, std=1.0):
    """Seeded N(0, std) rounded to bf16; returns uint16 bit patterns."""
    from helpers import f32_to_bf16_bits

    return f32_to_bf16_bits((rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32))


def require_b200():
    import pytest

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ml_dataflow_b200 import ops

    sm, major, minor = ops.device_info()
    assert major == 10, f"these kernels are built for sm_100a only (device is sm_{major}{minor})"
