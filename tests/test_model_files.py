"""The reference's model directory (config.txt, layers/<i>/combined_layer.weight) read by the library's loader.

tests/golden/model_tiny/ was written by the reference's own models/init_model.py (tests/golden/make_model_dir.py).
CPU: the parsed configuration, the byte offsets (against a restatement of the writer's order in numpy and of the
reference's alignment rule) and the weight pointers the loader binds. GPU: a layer loaded from the file gives the
same forward, bit for bit, as the same tensors uploaded one by one.
"""
import ctypes as C
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
MODEL = os.path.join(HERE, "golden", "model_tiny")
LAYER0 = os.path.join(MODEL, "layers", "0", "combined_layer.weight")


def lib_and_types():
    from ml_dataflow_b200 import _lib

    return _lib.load(), _lib


def parse():
    lib, L = lib_and_types()
    cfg = L.ModelConfig()
    assert lib.b200_parse_model_config(os.path.join(MODEL, "config.txt").encode(), C.byref(cfg)) == 0
    return lib, L, cfg


def writer_order_offsets(cfg, alignment):
    """Offsets of every tensor in the writer's order (init_model.py:198-318: norm, q, k, v, o, ffn norm, router, then
    w1, w3, w2 per expert), each start rounded up as prep_transformer.c:3-20 does. Returns ({name: offset}, total)."""
    d, hd, f = cfg.model_dim, cfg.head_dim, cfg.expert_dim
    attn, kv, E = cfg.num_q_heads * hd, cfg.num_kv_heads * hd, cfg.num_routed_experts
    sizes = [("attn_norm", d), ("w_q", attn * d), ("w_k", kv * d), ("w_v", kv * d), ("w_o", d * attn), ("ffn_norm", d),
             ("router", E * d)]
    for e in range(E):
        sizes += [(f"w1_{e}", f * d), (f"w3_{e}", f * d), (f"w2_{e}", d * f)]
    off, at = {}, 0
    for name, n in sizes:
        off[name] = at
        at += 2 * n
        if alignment and at % alignment:
            at += alignment - at % alignment
    return off, at


def test_config_txt_is_parsed_field_for_field():
    _, _, cfg = parse()
    assert (cfg.embed_dtype, cfg.attn_dtype, cfg.router_dtype, cfg.expert_dtype, cfg.head_dtype) == (b"bf16",) * 5
    assert (cfg.vocab_size, cfg.num_layers, cfg.model_dim, cfg.head_dim, cfg.num_q_heads, cfg.num_kv_heads) == (0, 1, 64, 32, 1, 1)
    assert (cfg.qk_norm_type, cfg.qk_norm_weight_type, cfg.expert_mlp_type) == (b"none", b"none", b"swiglu")
    assert (cfg.num_shared_experts, cfg.num_routed_experts, cfg.top_k_routed_experts, cfg.expert_dim) == (0, 8, 2, 32)
    assert cfg.rope_theta == 10000 and abs(cfg.rms_norm_epsilon - 1e-5) < 1e-9


def test_a_malformed_or_missing_config_is_refused(tmp_path):
    lib, L = lib_and_types()
    cfg = L.ModelConfig()
    assert lib.b200_parse_model_config(str(tmp_path / "nope.txt").encode(), C.byref(cfg)) == -1
    bad = tmp_path / "config.txt"
    bad.write_text(open(os.path.join(MODEL, "config.txt")).read().replace("Num Layers", "Layers"))
    assert lib.b200_parse_model_config(str(bad).encode(), C.byref(cfg)) == -1


@pytest.mark.parametrize("alignment", [0, 16, 256])
def test_layout_follows_the_writer_order_and_the_alignment_rule(alignment):
    lib, L, cfg = parse()
    lay = L.MoeLayerLayout()
    assert lib.b200_moe_layer_file_layout(C.byref(cfg), alignment, C.byref(lay)) == 0
    off, total = writer_order_offsets(cfg, alignment)
    for name in ("attn_norm", "w_q", "w_k", "w_v", "w_o", "ffn_norm", "router"):
        assert getattr(lay, name) == off[name], name
    assert (lay.w1_first, lay.w3_first, lay.w2_first) == (off["w1_0"], off["w3_0"], off["w2_0"])
    for e in range(cfg.num_routed_experts):
        assert lay.w1_first + e * lay.expert_stride_bytes == off[f"w1_{e}"]
        assert lay.w3_first + e * lay.expert_stride_bytes == off[f"w3_{e}"]
        assert lay.w2_first + e * lay.expert_stride_bytes == off[f"w2_{e}"]
    assert lay.aligned_bytes == total and lay.num_experts_in_file == 8 and lay.first_routed_expert == 0
    assert lay.raw_bytes == os.path.getsize(LAYER0)
    if alignment in (0, 16):  # every tensor of this model is a multiple of 16 bytes: the file is the laid-out block
        assert lay.aligned_bytes == os.path.getsize(LAYER0)


def test_file_is_read_whole_and_weights_are_bound():
    lib, L, cfg = parse()
    lay = L.MoeLayerLayout()
    assert lib.b200_moe_layer_file_layout(C.byref(cfg), 16, C.byref(lay)) == 0
    buf = np.zeros(lay.aligned_bytes // 2 + 8, np.uint16)
    base = buf.ctypes.data + (-buf.ctypes.data) % 16
    assert lib.b200_read_layer_file(LAYER0.encode(), C.c_void_p(base), lay.aligned_bytes) == 0
    raw = np.fromfile(LAYER0, np.uint16)
    start = (base - buf.ctypes.data) // 2
    np.testing.assert_array_equal(buf[start:start + raw.size], raw)
    # a file of another length is refused
    assert lib.b200_read_layer_file(LAYER0.encode(), C.c_void_p(base), lay.aligned_bytes - 2) == -1
    assert lib.b200_read_layer_file(LAYER0.encode(), C.c_void_p(base), lay.aligned_bytes + 2) == -1
    blk = L.MoeBlock()
    assert lib.b200_moe_block_bind_weights(C.byref(blk), C.byref(cfg), C.byref(lay), C.c_void_p(base)) == 0
    assert (blk.model_dim, blk.num_experts, blk.top_k, blk.ffn_dim) == (64, 8, 2, 32)
    assert blk.Wr == base + lay.router and blk.W1 == base + lay.w1_first and blk.W3 == base + lay.w3_first
    assert blk.W2 == base + lay.w2_first
    assert blk.w1_stride_elems == blk.w3_stride_elems == blk.w2_stride_elems == 3 * 32 * 64
    # an unaligned base is refused: the kernels need 16-byte aligned tensors
    assert lib.b200_moe_block_bind_weights(C.byref(blk), C.byref(cfg), C.byref(lay), C.c_void_p(base + 2)) == -1


@pytest.mark.gpu
def test_layer_loaded_from_the_file_matches_tensors_uploaded_one_by_one():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gpu_util import dev_bf16, rand_bf16
    from ml_dataflow_b200 import ops
    from ml_dataflow_b200.moe_layer import MoELayer

    lib, L, cfg = parse()
    lay = L.MoeLayerLayout()
    assert lib.b200_moe_layer_file_layout(C.byref(cfg), 16, C.byref(lay)) == 0
    host = torch.empty(lay.aligned_bytes, dtype=torch.uint8).pin_memory()
    assert lib.b200_read_layer_file(LAYER0.encode(), C.c_void_p(host.data_ptr()), lay.aligned_bytes) == 0
    dev = host.cuda()
    T, d, E, k, f = 96, cfg.model_dim, cfg.num_routed_experts, cfg.top_k_routed_experts, cfg.expert_dim
    X = dev_bf16(rand_bf16(np.random.default_rng(1), (T, d)))
    # reference path of the comparison: slice the file in the writer's order and upload every tensor on its own
    raw = np.fromfile(LAYER0, np.uint16)
    off, _ = writer_order_offsets(cfg, 0)
    pick = lambda name, shape: dev_bf16(raw[off[name] // 2: off[name] // 2 + int(np.prod(shape))].reshape(shape))
    Wr = pick("router", (E, d))
    W1 = torch.stack([pick(f"w1_{e}", (f, d)) for e in range(E)])
    W3 = torch.stack([pick(f"w3_{e}", (f, d)) for e in range(E)])
    W2 = torch.stack([pick(f"w2_{e}", (d, f)) for e in range(E)])
    outs = []
    for from_file in (False, True):
        layer = MoELayer(T, d, E, k, f)
        blk = layer.block(Wr, W1, W3, W2)
        if from_file:
            assert lib.b200_moe_block_bind_weights(C.byref(blk), C.byref(cfg), C.byref(lay), C.c_void_p(dev.data_ptr())) == 0
        out = torch.zeros((T, d), dtype=torch.bfloat16, device="cuda")
        ops.moe_block_fwd(blk, X, out)
        torch.cuda.synchronize()
        assert ops.gemm_status() == 0
        outs.append((out, layer.logits.clone(), layer.x1.clone()))
    assert torch.equal(outs[0][1], outs[1][1]) and torch.equal(outs[0][2], outs[1][2]) and torch.equal(outs[0][0], outs[1][0])
    assert outs[0][0].float().abs().max() > 0
