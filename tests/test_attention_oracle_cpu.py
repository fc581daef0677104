"""CPU: the attention oracle (oracle/block_oracle.c) against float64 softmax attention and torch autograd: packed
variable-length sequences, grouped query heads, causal with the last query aligned to the last key, and the full
(non-causal) form. The oracle rounds the probabilities to bf16 before they multiply V / dO, as the published
algorithm does, so the comparison is to bf16 resolution."""
import numpy as np
import pytest
import torch


def _bits(a):
    from helpers import f32_to_bf16_bits

    return f32_to_bf16_bits(np.asarray(a, np.float32))


def _f32(b):
    from helpers import bf16_bits_to_f32

    return bf16_bits_to_f32(b)


def reference_attention(q, k, v, q_off, q_len, k_off, k_len, Hq, Hkv, hd, causal, dO=None):
    """float64 torch: returns O (and dQ, dK, dV when dO is given)."""
    q = torch.tensor(q, dtype=torch.float64, requires_grad=True)
    k = torch.tensor(k, dtype=torch.float64, requires_grad=True)
    v = torch.tensor(v, dtype=torch.float64, requires_grad=True)
    out = torch.zeros_like(q)
    lse = torch.zeros((Hq, q.shape[0]), dtype=torch.float64)
    group = Hq // Hkv
    for s in range(len(q_len)):
        Tq, Tk = q_len[s], k_len[s]
        for h in range(Hq):
            qs = q[q_off[s]:q_off[s] + Tq, h * hd:(h + 1) * hd]
            g = h // group
            ks = k[k_off[s]:k_off[s] + Tk, g * hd:(g + 1) * hd]
            vs = v[k_off[s]:k_off[s] + Tk, g * hd:(g + 1) * hd]
            sc = qs @ ks.T / np.sqrt(hd)
            if causal:
                i = torch.arange(Tq)[:, None]
                j = torch.arange(Tk)[None, :]
                sc = sc.masked_fill(j > i + (Tk - Tq), float("-inf"))
            lse[h, q_off[s]:q_off[s] + Tq] = torch.logsumexp(sc, dim=1).detach()
            out[q_off[s]:q_off[s] + Tq, h * hd:(h + 1) * hd] = torch.softmax(sc, dim=1) @ vs
    if dO is None:
        return out.detach().numpy(), lse.numpy()
    out.backward(torch.tensor(dO, dtype=torch.float64))
    return out.detach().numpy(), lse.numpy(), q.grad.numpy(), k.grad.numpy(), v.grad.numpy()


CASES = [
    # q_len, k_len, Hq, Hkv, hd, causal
    ([37, 5, 64], [37, 5, 64], 4, 2, 32, True),
    ([16, 9], [40, 9], 2, 1, 16, True),     # keys beyond the queries (a cached prefix)
    ([21], [21], 3, 3, 8, False),
]


@pytest.mark.parametrize("q_len,k_len,Hq,Hkv,hd,causal", CASES)
def test_attention_oracle_forward_backward(oracle, q_len, k_len, Hq, Hkv, hd, causal):
    rng = np.random.default_rng(sum(q_len) + hd)
    q_off = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(int).tolist()
    k_off = np.concatenate([[0], np.cumsum(k_len)[:-1]]).astype(int).tolist()
    tq, tk = sum(q_len), sum(k_len)
    Q, K, V = (_bits(rng.standard_normal((n, H * hd))) for n, H in ((tq, Hq), (tk, Hkv), (tk, Hkv)))
    dO = _bits(rng.standard_normal((tq, Hq * hd)))
    O, lse = oracle.attention_fwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Q, K, V, causal)
    ro, rl, rdq, rdk, rdv = reference_attention(_f32(Q), _f32(K), _f32(V), q_off, q_len, k_off, k_len, Hq, Hkv, hd, causal,
                                                _f32(dO))
    np.testing.assert_allclose(lse, rl, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(_f32(O), ro, rtol=2e-2, atol=8e-3)
    dQ, dK, dV = oracle.attention_bwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Q, K, V, O, lse, dO, causal)
    for got, ref, what in ((dQ, rdq, "dQ"), (dK, rdk, "dK"), (dV, rdv, "dV")):
        err = np.linalg.norm(_f32(got) - ref) / (np.linalg.norm(ref) + 1e-30)
        assert err < 1e-2, f"{what}: relative error {err:.2e}"
