"""CPU: pins the oracle against tensors produced by the reference's PyTorch MoE layer.

The fixtures come from tests/golden/make_golden.py. PyTorch accumulates the combine and the
gradients with bf16 roundings between terms where the reference kernels (and the oracle) use one
fp32 accumulation, and it rounds silu and the gate product to bf16 separately, so sums with cancellation differ
by a few bf16 ulps of their largest term. The check is therefore a relative Frobenius error
below 8e-3 (bf16 has 2^-8 = 3.9e-3) plus an element-wise bound of 2e-2 relative + 4e-2 of the
tensor's rms. Exact integer outputs (expert sets, counts) are compared exactly.
"""
import os

import numpy as np
import pytest

from helpers import assert_close, bf16_bits_to_f32

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def rms(a):
    return float(np.sqrt(np.mean(np.asarray(a, np.float64) ** 2)))


def rel_fro(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))


@pytest.mark.parametrize("name", ["moe_mlp_small", "moe_mlp_k4", "moe_mlp_e64k8"])
def test_oracle_matches_reference_pytorch_layer(oracle, name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    T, d, E, k, f = [int(v) for v in g["shape"]]
    X, Wr, W1, W3, W2, dOut = g["X"], g["Wr"], g["W1"], g["W3"], g["W2"], g["dOut"]

    # router GEMM of the oracle against the reference's logits
    logits = oracle.linear_fwd(X, Wr, out_dtype=np.float32)
    np.testing.assert_allclose(logits, g["logits"], rtol=1e-4, atol=1e-4)

    fwd = oracle.moe_forward(X, Wr, W1, W3, W2, k, logits=np.ascontiguousarray(g["logits"]))
    # same expert set per token, same gate weight per (token, expert)
    order_o = np.argsort(fwd["chosen"].astype(np.int32), axis=1)
    order_g = np.argsort(g["selected"], axis=1)
    np.testing.assert_array_equal(np.take_along_axis(fwd["chosen"].astype(np.int32), order_o, 1),
                                  np.take_along_axis(g["selected"], order_g, 1))
    np.testing.assert_allclose(np.take_along_axis(fwd["weights"], order_o, 1),
                               np.take_along_axis(g["routing_weights"], order_g, 1), rtol=1e-5, atol=1e-6)
    assert int(fwd["counts"][:E].sum()) == T * k

    out_o, out_g = bf16_bits_to_f32(fwd["out"]), bf16_bits_to_f32(g["out"])
    assert_close(out_o, out_g, atol=4e-2 * rms(out_g), what="out")
    assert rel_fro(out_o, out_g) < 8e-3

    bwd = oracle.moe_backward(X, Wr, W1, W3, W2, k, fwd, dOut)
    for key_o, key_g in [("dXn", "dX"), ("dW1", "dW1"), ("dW3", "dW3"), ("dW2", "dW2")]:
        a, b = bf16_bits_to_f32(bwd[key_o]), bf16_bits_to_f32(g[key_g])
        assert_close(a, b, atol=4e-2 * rms(b), what=key_o)
        assert rel_fro(a, b) < 8e-3, key_o
    # router weight gradient: reference keeps it in fp32, oracle in bf16 with bf16 dlogits
    a, b = bf16_bits_to_f32(bwd["dWr"]), g["dWr"]
    assert rel_fro(a, b) < 8e-3
