"""GPU: b200_attention_fwd / _bwd (csrc/attention.cu) against the CPU oracle on the same seeded inputs: packed
variable-length sequences with ragged lengths (not multiples of 8), grouped query heads (16 query / 4 key-value heads
of 128 as in the decoder configuration, and smaller shapes), causal and full, keys beyond the queries. Outputs and
gradients to the layer's bf16 tolerance as relative Frobenius error plus an element bound; the log-sum-exp to 1e-4."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CASES = [
    # q_len, k_len, Hq, Hkv, hd, causal
    ([300, 77, 1], [300, 77, 1], 16, 4, 128, True),
    ([129], [129], 4, 4, 64, False),
    ([64, 40], [200, 40], 8, 2, 128, True),
    ([513], [513], 2, 1, 128, True),
    ([4200, 100], [4300, 100], 2, 1, 32, True),   # more than one chunk of query rows, keys beyond the queries
    ([16], [8300], 2, 1, 32, True),               # more keys than a block keeps in registers
    ([0, 257], [5, 700], 4, 2, 128, False),       # fused kernels: a sequence without queries, several key blocks, no mask
    ([385, 130], [900, 130], 8, 2, 128, True),    # fused kernels: three query tiles, keys beyond the queries, ragged ends
    ([40], [40], 2, 2, 128, True),                # fused kernels: fewer rows in the whole batch than one tile
    (list(range(1, 61)), [n + (n % 3) * 50 for n in range(1, 61)], 4, 2, 128, True),  # more sequences than one launch's table
]


def _f32(b):
    from helpers import bf16_bits_to_f32

    return bf16_bits_to_f32(b)


@pytest.mark.parametrize("q_len,k_len,Hq,Hkv,hd,causal", CASES)
def test_attention_forward_backward(oracle, q_len, k_len, Hq, Hkv, hd, causal):
    import torch

    from gpu_util import dev_bf16, host_bits, rand_bf16, require_b200
    from helpers import assert_chain_close, assert_close

    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(sum(q_len) * 3 + hd)
    q_off = np.concatenate([[0], np.cumsum(q_len)[:-1]]).astype(int).tolist()
    k_off = np.concatenate([[0], np.cumsum(k_len)[:-1]]).astype(int).tolist()
    tq, tk = sum(q_len), sum(k_len)
    Q, K, V = rand_bf16(rng, (tq, Hq * hd)), rand_bf16(rng, (tk, Hkv * hd)), rand_bf16(rng, (tk, Hkv * hd))
    dO = rand_bf16(rng, (tq, Hq * hd))
    ref_O, ref_lse = oracle.attention_fwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Q, K, V, causal)
    Qd, Kd, Vd, dOd = dev_bf16(Q), dev_bf16(K), dev_bf16(V), dev_bf16(dO)
    O = torch.zeros_like(Qd)
    lse = torch.zeros((Hq, tq), dtype=torch.float32, device="cuda")
    nbytes = ops.attention_workspace_bytes(True, Hq, Hkv, hd, tq, max(q_len), max(k_len))
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    ops.attention_fwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Qd, Kd, Vd, O, lse, causal, ws)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0 and ops.attention_status() == 0
    np.testing.assert_allclose(lse.cpu().numpy(), ref_lse, rtol=1e-4, atol=1e-4)
    assert_chain_close(_f32(host_bits(O)), _f32(ref_O), limit=6e-3, what="attention output")
    assert_close(_f32(host_bits(O)), _f32(ref_O), rtol=2e-2, atol=8e-3, what="attention output")
    # backward on the oracle's forward results, so that both sides start from identical tensors
    ref_dQ, ref_dK, ref_dV = oracle.attention_bwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Q, K, V, ref_O, ref_lse, dO, causal)
    dQ, dK, dV = torch.full_like(Qd, 7.0), torch.full_like(Kd, 7.0), torch.full_like(Vd, 7.0)
    ops.attention_bwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Qd, Kd, Vd, dev_bf16(ref_O), torch.from_numpy(ref_lse).cuda(),
                      dOd, dQ, dK, dV, causal, ws)
    torch.cuda.synchronize()
    assert ops.gemm_status() == 0 and ops.attention_status() == 0
    for got, ref, what in ((dQ, ref_dQ, "dQ"), (dK, ref_dK, "dK"), (dV, ref_dV, "dV")):
        assert_chain_close(_f32(host_bits(got)), _f32(ref), limit=8e-3, what=what)
        assert_close(_f32(host_bits(got)), _f32(ref), rtol=2e-2, atol=3e-2, max_bad_frac=2e-3, what=what)
    # a workspace that is too small is refused
    with pytest.raises(RuntimeError):
        ops.attention_bwd(q_off, q_len, k_off, k_len, Hq, Hkv, hd, Qd, Kd, Vd, dev_bf16(ref_O), torch.from_numpy(ref_lse).cuda(),
                          dOd, dQ, dK, dV, causal, ws[:1024])
