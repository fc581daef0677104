"""GPU: backward of the whole MoE layer at the benchmark's sizes (T=8192 and T=32768, d=4096, 64 experts, top-8,
ffn 1408), checked on three sampled experts and on the router gradients.

The CPU oracle needs minutes for these shapes (6.8 and 27 TFLOP of fp32 loops), so the checker here is a plain
fp32 torch evaluation on the GPU of the same maths the oracle restates, applied to the inputs each GPU op consumed
(the oracle itself is compared with the kernels, element-wise, at smaller sizes in test_gpu_gemm.py and
test_gpu_layer.py). What is covered per sampled expert e (rows [base_e, base_e + n_e) of the expert-ordered arrays):
  dh = dY_e W2_e -> (dx1, dx3) = swiglu'(x1, x3, bf16(dh));  dZ_e = dx1 W1_e + dx3 W3_e;
  dW2_e = dY_e^T h_e;  dW1_e = dx1^T Z_e;  dW3_e = dx3^T Z_e;  dP[r] = <Y[r], dOut[token(r)]>
and for the whole batch: the gate Jacobian, dWr = dL^T Xn and the router part of dXn.
Tolerance: |a - b| <= 1e-3 + 2e-2 |b| on at least 99.9 % of the elements (a bf16 input that rounds the other way
moves a few sums by more), plus a relative Frobenius error below 1e-2 (5e-2 for the router gradients, whose dot
products go through a cancelling subtraction).
"""
import numpy as np
import pytest
import torch

from gpu_util import require_b200

pytestmark = pytest.mark.gpu


def _close(got, ref, what, frac=0.999, fro=1e-2):
    got, ref = got.float(), ref.float()
    err = (got - ref).abs()
    ok = (err <= 1e-3 + 2e-2 * ref.abs()).float().mean().item()
    rel = ((got - ref).norm() / (ref.norm() + 1e-30)).item()
    assert ok >= frac, f"{what}: only {ok:.5f} of the elements within tolerance"
    assert rel < fro, f"{what}: relative Frobenius error {rel:.2e}"


def _bf(x):
    return x.to(torch.bfloat16).float()


@pytest.mark.parametrize("T", [8192, 32768])
def test_layer_backward_full_size(T):
    require_b200()
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    d, E, k, f = 4096, 64, 8, 1408
    gen = torch.Generator(device="cuda").manual_seed(11 + T)

    def normal(shape, std):
        return (torch.randn(shape, generator=gen, device="cuda") * std).to(torch.bfloat16)

    X, dOut, Wr = normal((T, d), 1.0), normal((T, d), 1.0), normal((E, d), 0.02)
    W1, W3, W2 = normal((E, f, d), 0.02), normal((E, f, d), 0.02), normal((E, d, f), 0.02)
    layer = MoELayer(T, d, E, k, f)
    layer.keep_pre_gate = True
    out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
    dXn = torch.empty_like(out)
    dWr = torch.zeros_like(Wr)
    dW1, dW3, dW2 = torch.zeros_like(W1), torch.zeros_like(W3), torch.zeros_like(W2)
    layer.forward(X, Wr, W1, W3, W2, out)
    layer.backward(X, Wr, W1, W3, W2, dOut, dXn, dWr, dW1, dW3, dW2)
    assert ops.gemm_status() == 0
    counts = layer.counts[:E].cpu().numpy()
    assert counts.sum() == T * k
    base = np.concatenate([[0], np.cumsum(counts)])
    em = layer.expert_mapping.long()
    w_rows = layer.row_w
    for e in (0, 29, 63):
        n = int(counts[e])
        assert n > 0
        sl = slice(int(base[e]), int(base[e]) + n)
        tok = em[sl]
        # dY rows = bf16(w * dOut[token]) in expert order
        dY = _bf(dOut[tok].float() * w_rows[sl].unsqueeze(1))
        _close(layer.dYz[sl], dY, f"expert {e}: weighted gather", frac=0.9999, fro=1e-3)
        x1, x3, Z, h = layer.x1[sl].float(), layer.x3[sl].float(), layer.zone[sl].float(), layer.h[sl].float()
        dh = _bf(layer.dYz[sl].float() @ W2[e].float())
        s = torch.sigmoid(x1)
        silu = x1 * s
        _close(layer.dx3[sl], dh * silu, f"expert {e}: dx3")
        _close(layer.dx1[sl], dh * x3 * (s + x1 * s * (1 - s)), f"expert {e}: dx1")
        dx1, dx3 = layer.dx1[sl].float(), layer.dx3[sl].float()
        _close(layer.dZ[sl], dx1 @ W1[e].float() + dx3 @ W3[e].float(), f"expert {e}: dZ")
        _close(dW2[e], layer.dYz[sl].float().T @ h, f"expert {e}: dW2")
        _close(dW1[e], dx1.T @ Z, f"expert {e}: dW1")
        _close(dW3[e], dx3.T @ Z, f"expert {e}: dW3")
        # router dot product on the forward's expert output, as the reference forms it (router_bwd_x.cu:41-64)
        # there Y is the bf16-rounded forward output, here the dot product is taken on the fp32 accumulator side
        # (<h, dh> / w): the two differ by the rounding of Y, about 2^-9 |Y_i dOut_i| per term, summed at random
        terms = layer.Y[sl].float() * dOut[tok].float()
        dP_ref = terms.sum(dim=1)
        slack = 6.0 * 2.0 ** -9 * terms.pow(2).sum(dim=1).sqrt()
        err = (layer.dP[sl] - dP_ref).abs()
        assert (err <= 1e-3 + 2e-2 * dP_ref.abs() + slack).float().mean().item() >= 0.999, f"expert {e}: dP"
        assert ((layer.dP[sl] - dP_ref).norm() / dP_ref.norm()).item() < 2e-2, f"expert {e}: dP (norm)"
    # un-permute: dXn before the router part is the sum of a token's k dZ rows; the router adds dL . Wr
    dL = layer.dX_routed.float()
    tm = layer.token_mapping.long()
    dX_experts = layer.dZ.float()[tm.reshape(-1)].reshape(T, k, d).sum(dim=1)
    _close(dXn, _bf(dX_experts) + dL @ Wr.float(), "dXn", frac=0.995)
    _close(dWr, dL.T @ X.float(), "dWr", frac=0.99, fro=5e-2)
    # gate Jacobian on the k chosen columns, other columns zero (router_gate_bwd_x.cu:7-57)
    pre = layer.dX_routed_pre.float()
    ch = layer.chosen.view(torch.int16).long() & 0xFFFF
    p = layer.weights
    dp = torch.gather(pre, 1, ch)
    g = p * (dp - (dp * p).sum(dim=1, keepdim=True))
    ref = torch.zeros_like(pre).scatter_(1, ch, g)
    _close(layer.dX_routed, ref, "gate backward", frac=0.99, fro=2e-2)
