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


# End-to-end comparisons (a whole chain of GPU ops against the oracle's own chain): a bf16 value that rounds the
# other way early in the chain moves downstream sums by an ulp of their largest term, which the element-wise bound
# cannot absorb near zero. Chains are therefore held to a relative Frobenius error; every single op is checked
# element-wise on identical inputs elsewhere in the same tests.
def rel_fro(a, b):
    a64, b64 = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a64 - b64) / (np.linalg.norm(b64) + 1e-30))


def assert_chain_close(a, b, limit=1e-2, what=""):
    r = rel_fro(a, b)
    assert r < limit, f"{what}: relative Frobenius error {r:.2e} >= {limit:.0e}"


def assert_close_with_slack(a, b, slack, rtol=RTOL, atol=ATOL, what=""):
    """|a-b| <= atol + rtol*|b| + slack, `slack` an element-wise array (e.g. one bf16 ulp of an intermediate)."""
    a, b, slack = (np.asarray(x, np.float64) for x in (a, b, slack))
    err = np.abs(a - b)
    lim = atol + rtol * np.abs(b) + slack
    bad = err > lim
    assert not bad.any(), f"{what}: {bad.mean():.3e} of elements outside tol (worst {(err / lim).max():.2f}x)"
