"""Shared test helpers: tolerance checks and bf16 <-> numpy conversions."""
import numpy as np

# The contract for every bf16 tensor of the layer: |a-b| <= ATOL + RTOL*|b|
RTOL, ATOL = 2e-2, 1e-3


def bf16_bits_to_f32(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(a):
    """Round-to-nearest-even, NaN-preserving (numpy restatement used only by tests)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def close_frac(a, b, rtol=RTOL, atol=ATOL):
    """Fraction of elements outside tolerance, and the worst excess ratio."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    err = np.abs(a - b)
    lim = atol + rtol * np.abs(b)
    bad = err > lim
    return float(bad.mean()), float((err / lim).max()) if err.size else 0.0


def assert_close(a, b, rtol=RTOL, atol=ATOL, max_bad_frac=0.0, what=""):
    frac, worst = close_frac(a, b, rtol, atol)
    assert frac <= max_bad_frac, f"{what}: {frac:.3e} of elements outside tol (worst {worst:.2f}x)"


# Chained comparisons (a tensor computed from earlier GPU results against the oracle's own chain): a bf16 value
# that rounds the other way upstream shifts a few downstream elements by one ulp of a larger term, so a tiny
# fraction may sit just outside the element-wise bound. Everything else must be inside it.
CHAIN_BAD_FRAC, CHAIN_WORST = 1e-3, 8.0


def assert_close_chained(a, b, rtol=RTOL, atol=ATOL, what=""):
    frac, worst = close_frac(a, b, rtol, atol)
    assert frac <= CHAIN_BAD_FRAC and worst <= CHAIN_WORST, (
        f"{what}: {frac:.3e} of elements outside tol (worst {worst:.2f}x)")
    a64, b64 = np.asarray(a, np.float64), np.asarray(b, np.float64)
    rel = np.linalg.norm(a64 - b64) / (np.linalg.norm(b64) + 1e-30)
    assert rel < 4e-3, f"{what}: relative Frobenius error {rel:.2e}"
