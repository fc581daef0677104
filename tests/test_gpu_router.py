"""GPU parity: router select, mapping and gate backward against the CPU oracle (bit-exact integers)."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host_u16, require_b200

pytestmark = pytest.mark.gpu


def run_select(ops, logits_np, k):
    T, E = logits_np.shape
    logits = torch.from_numpy(logits_np).cuda()
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    ch = torch.empty((T, k), dtype=torch.int16, device="cuda")
    counts = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    cumsum = torch.zeros(E, dtype=torch.int32, device="cuda")
    hostc = torch.zeros(E, dtype=torch.int32, device="cuda")
    ops.select_experts(T, E, k, logits, w, ch, counts, cumsum, hostc)
    torch.cuda.synchronize()
    return w.cpu().numpy(), host_u16(ch), counts.cpu().numpy(), cumsum.cpu().numpy(), hostc.cpu().numpy()


def check_select(ops, oracle, logits, k):
    w, ch, counts, cumsum, hostc = run_select(ops, logits, k)
    ow, och, ocounts, ocumsum, ohost = oracle.select_experts(logits, k)
    E = logits.shape[1]
    np.testing.assert_array_equal(ch, och)
    np.testing.assert_array_equal(counts[:E], ocounts[:E])
    np.testing.assert_array_equal(cumsum, ocumsum)
    np.testing.assert_array_equal(hostc, ohost)
    np.testing.assert_allclose(w, ow, rtol=1e-5, atol=1e-7)
    return ch, cumsum


def run_mapping(ops, chosen_np, E, cumsum_np):
    T, k = chosen_np.shape
    ch = dev(chosen_np)
    cumsum = torch.from_numpy(cumsum_np.copy()).cuda()
    em = torch.full((T * k,), -7, dtype=torch.int32, device="cuda")
    tm = torch.full((T, k), -7, dtype=torch.int32, device="cuda")
    ws = torch.empty(ops.build_expert_mapping_workspace_bytes(T, E, k), dtype=torch.uint8, device="cuda")
    ops.build_expert_mapping(T, E, k, ch, cumsum, em, tm, ws)
    torch.cuda.synchronize()
    return em.cpu().numpy(), tm.cpu().numpy(), cumsum.cpu().numpy()


def check_mapping(ops, oracle, chosen, E, cumsum_excl):
    em, tm, cincl = run_mapping(ops, chosen, E, cumsum_excl)
    oem, otm, ocincl = oracle.build_expert_mapping(chosen, E, cumsum_excl)
    np.testing.assert_array_equal(tm, otm)
    n_routed = int((chosen < E).sum())
    np.testing.assert_array_equal(em[:n_routed], oem[:n_routed])
    np.testing.assert_array_equal(cincl, ocincl)


@pytest.mark.parametrize("T", [1, 2, 31, 33, 130, 1000])
@pytest.mark.parametrize("E,k", [(2, 1), (2, 2), (16, 2), (64, 8), (100, 5), (64, 1), (256, 8), (40, 32)])
def test_select_and_mapping_small_grid(oracle, T, E, k):
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(1000 * T + 10 * E + k)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    ch, cumsum = check_select(ops, oracle, logits, k)
    check_mapping(ops, oracle, ch, E, cumsum)


def test_select_ties_and_degenerate_rows(oracle):
    require_b200()
    from ml_dataflow_b200 import ops

    T, E, k = 257, 64, 8
    # pure tie-break: all logits equal -> experts 0..k-1 in slot order
    logits = np.full((T, E), 0.25, np.float32)
    ch, cumsum = check_select(ops, oracle, logits, k)
    assert (ch == np.arange(k, dtype=np.uint16)[None, :]).all()
    check_mapping(ops, oracle, ch, E, cumsum)
    # heavy ties from quantised logits
    rng = np.random.default_rng(7)
    logits = rng.integers(-2, 3, size=(T, E)).astype(np.float32)
    ch, cumsum = check_select(ops, oracle, logits, k)
    check_mapping(ops, oracle, ch, E, cumsum)
    # every token prefers expert 5, the rest random
    logits = rng.standard_normal((T, E), dtype=np.float32)
    logits[:, 5] += 100.0
    ch, cumsum = check_select(ops, oracle, logits, k)
    assert (ch == 5).sum() == T
    check_mapping(ops, oracle, ch, E, cumsum)
    # rows with fewer than k finite logits: unfilled slots keep 0xFFFF and are not counted
    logits = np.full((T, E), -np.inf, np.float32)
    logits[:, 3] = 1.0
    logits[:, 9] = 2.0
    w, chg, counts, cs, hc = run_select(ops, logits, k)
    ow, och, ocounts, ocs, ohc = oracle.select_experts(logits, k)
    np.testing.assert_array_equal(chg, och)
    np.testing.assert_array_equal(counts[:E], ocounts[:E])
    assert counts[:E].sum() == 2 * T
    check_mapping(ops, oracle, chg, E, cs)


@pytest.mark.parametrize("T,E,k", [(2048, 16, 2), (8192, 64, 8), (65536, 64, 8)])
def test_select_and_mapping_config_shapes(oracle, T, E, k):
    require_b200()
    from ml_dataflow_b200 import ops

    rng = np.random.default_rng(T + E)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    if T == 65536:  # skewed popularity: Zipf(1.1) bias over a seeded expert ranking
        rank = rng.permutation(E) + 1
        p = rank.astype(np.float64) ** -1.1
        logits += np.log(p / p.sum()).astype(np.float32)[None, :]
    ch, cumsum = check_select(ops, oracle, logits, k)
    check_mapping(ops, oracle, ch, E, cumsum)


def test_select_bf16_logits(oracle):
    require_b200()
    from ml_dataflow_b200 import ops
    from helpers import bf16_bits_to_f32, f32_to_bf16_bits

    T, E, k = 500, 64, 8
    rng = np.random.default_rng(3)
    bits = f32_to_bf16_bits(rng.standard_normal((T, E), dtype=np.float32))
    logits16 = torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    ch = torch.empty((T, k), dtype=torch.int16, device="cuda")
    counts = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    cumsum = torch.zeros(E, dtype=torch.int32, device="cuda")
    ops.select_experts(T, E, k, logits16, w, ch, counts, cumsum, None)
    torch.cuda.synchronize()
    ow, och, ocounts, _, _ = oracle.select_experts(bf16_bits_to_f32(bits), k)
    np.testing.assert_array_equal(host_u16(ch), och)
    np.testing.assert_array_equal(counts.cpu().numpy()[:E], ocounts[:E])
    np.testing.assert_allclose(w.cpu().numpy(), ow, rtol=1e-5, atol=1e-7)


def test_router_gate_bwd(oracle):
    require_b200()
    from ml_dataflow_b200 import ops
    from helpers import assert_close, bf16_bits_to_f32, f32_to_bf16_bits

    T, E, k = 777, 64, 8
    rng = np.random.default_rng(11)
    logits = rng.standard_normal((T, E), dtype=np.float32)
    w, ch, *_ = oracle.select_experts(logits, k)
    dP = f32_to_bf16_bits(rng.standard_normal((T, E), dtype=np.float32))
    ref = oracle.router_gate_bwd_x(ch, w, dP.copy())
    d = torch.from_numpy(dP.view(np.int16).copy()).cuda().view(torch.bfloat16)
    ops.router_gate_bwd_x(T, E, k, dev(ch), torch.from_numpy(w).cuda(), d)
    torch.cuda.synchronize()
    got = d.view(torch.int16).cpu().numpy().view(np.uint16)
    assert_close(bf16_bits_to_f32(got), bf16_bits_to_f32(ref), what="gate bwd")


def test_argument_errors():
    require_b200()
    from ml_dataflow_b200 import ops

    x = torch.zeros((4, 8), dtype=torch.float32, device="cuda")
    w = torch.zeros((4, 2), dtype=torch.float32, device="cuda")
    ch = torch.zeros((4, 2), dtype=torch.int16, device="cuda")
    c = torch.zeros(9, dtype=torch.int32, device="cuda")
    cs = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        ops.select_experts(4, 8, 9, x, w, ch, c, cs, None)  # top_k > n_experts
    with pytest.raises(RuntimeError):
        ops.select_experts(4, 5000, 2, x, w, ch, c, cs, None)  # too many experts
    with pytest.raises(RuntimeError):
        ops.prepare_experts(4, 12, 2, x, cs, x)  # model_dim not a multiple of 8
