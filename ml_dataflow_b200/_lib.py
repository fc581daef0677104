"""Loads the C-ABI library and declares the argument types of every entry point in include/b200_moe.h.

There is no fallback: if the library is missing the import of any op fails with an error that says how to build it.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200moe.so")

_vp, _i, _f, _i64, _u64, _sz = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_uint64, C.c_size_t

# name -> (restype, argtypes); mirrors include/b200_moe.h
SIGNATURES = {
    "b200_device_info": (_i, [_vp, _vp, _vp]),
    "b200_select_experts": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_build_expert_mapping_workspace_bytes": (_sz, [_i, _i, _i]),
    "b200_build_expert_mapping": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200_build_expert_mapping_static_capacity_bytes": (_sz, []),
    "b200_build_expert_mapping_static": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "b200_prepare_experts": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_prepare_experts_weighted": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "b200_prepare_expert_zone": (_i, [_i, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "b200_merge_experts": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "b200_unpermute_experts": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_merge_expert_result": (_i, [_i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_router_bwd_x": (_i, [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_router_gate_bwd_x": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_swiglu": (_i, [_i, _i, _vp, _vp, _vp, _vp]),
    "b200_swiglu_bwd_x": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_matmul": (_i, [_i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _u64, _vp, _vp]),
    "b200_matmul_strided": (_i, [_i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _i64, _i, _vp, _i64, _vp, _vp, _i64, _vp]),
    "b200_gemm_status": (_i, [_vp]),
    "b200_gemm_set_pair_mode": (_i, [_i]),
    "b200_gemm_set_wide_mode": (_i, [_i]),
    "b200_moe_experts_fwd": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_moe_experts_bwd_x": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp,
                                    _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_moe_experts_bwd_w": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp,
                                    _vp]),
    "b200_moe_experts_bwd_w_overwrite": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp,
                                    _vp]),
    "b200_ep_dispatch_rows": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i, _i, _vp]),
    "b200_ep_combine_rows": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _vp, _vp]),
    "b200_ep_gather_router_grad": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _vp, _vp]),
    "b200_ep_publish_row_tags": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i64, _vp]),
    "b200_moe_experts_fwd_scatter": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp,
                                          _vp, _vp, _i, _i64, _vp]),
    "b200_moe_experts_bwd_x_scatter": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp,
                                            _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _vp]),
    "b200_gemm_enumerate_tiles": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "b200_moe_block_fwd": (_i, [_vp, _vp, _vp, _vp]),
    "b200_moe_block_recompute": (_i, [_vp, _vp, _i, _vp]),
    "b200_moe_block_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_moe_block_bwd_overwrite": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_moe_saved_activations_bytes": (_u64, [_i, _i, _i, _i, _i]),
    "b200_moe_block_save_activations": (_i, [_vp, _i, _vp, _u64, _vp]),
    "b200_moe_block_restore_activations": (_i, [_vp, _i, _vp, _u64, _vp]),
    "b200_moe_block_recompute_level": (_i, [_vp, _vp, _i, _vp]),
    "b200_parse_model_config": (_i, [C.c_char_p, _vp]),
    "b200_moe_layer_file_layout": (_i, [_vp, _i, _vp]),
    "b200_read_layer_file": (_i, [C.c_char_p, _vp, _u64]),
    "b200_moe_block_bind_weights": (_i, [_vp, _vp, _vp, _vp]),
    "b200_ep_barrier": (_i, [_vp, _i, _i, _vp, _vp, _i, _vp, _vp]),
    "b200_ep_set_barrier_timeout_ms": (_i, [_i]),
    "b200_ep_status": (_i, [_vp]),
    "b200_ep_plan": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _vp, _vp, _vp]),
    "b200_ep_reduce_router_grad": (_i, [_vp, _i, _i64, _vp, _vp]),
    "b200_ep_moe_block_fwd": (_i, [_vp, _vp, _vp, _vp]),
    "b200_ep_moe_block_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_rms_norm": (_i, [_i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp]),
    "b200_rms_norm_recompute": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "b200_rms_norm_bwd_x": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_rms_norm_bwd_w_workspace_bytes": (_u64, [_i, _i]),
    "b200_rms_norm_bwd_w": (_i, [_i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _u64, _vp, _vp]),
    "b200_rope": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_rope_bwd_x": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_softmax": (_i, [_i, _i, _i, _i, _vp, _vp, _vp]),
    "b200_cross_entropy_loss": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_set_average_loss": (_i, [_i, _vp, _vp]),
    "b200_adamw_step": (_i, [_i, _i, _i, _i, _u64, _i, _f, _f, _f, _f, _f, _vp, _vp, _vp, _vp, _vp]),
    "b200_embedding_table": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_embedding_table_bwd_w": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_attention_workspace_bytes": (_u64, [_i, _i, _i, _i, _i, _i, _i]),
    "b200_attention_fwd": (_i, [_i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _u64, _vp, _vp]),
    "b200_attention_bwd": (_i, [_i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                _vp, _i, _u64, _vp, _vp]),
    "b200_attention_status": (_i, [_vp]),
    "b200_transformer_block_fwd": (_i, [_vp, _vp, _vp, _vp]),
    "b200_transformer_block_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_scatter_row_weights": (_i, [_i, _i, _vp, _vp, _vp, _vp]),
    "b200_gather_router_grad": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
}



class MoeBlock(C.Structure):
    """ctypes mirror of B200MoeBlock in include/b200_moe.h (same field order)."""
    _fields_ = [
        ("total_tokens", _i), ("model_dim", _i), ("num_experts", _i), ("top_k", _i), ("ffn_dim", _i),
        ("Wr", _vp), ("W1", _vp), ("W3", _vp), ("W2", _vp),
        ("w1_stride_elems", _i64), ("w3_stride_elems", _i64), ("w2_stride_elems", _i64),
        ("logits", _vp), ("token_expert_weights", _vp), ("chosen_experts", _vp), ("expert_counts", _vp),
        ("expert_counts_cumsum", _vp), ("host_expert_counts", _vp), ("expert_mapping", _vp), ("token_mapping", _vp),
        ("zone", _vp), ("x1", _vp), ("x3", _vp), ("h", _vp), ("Y", _vp),
        ("mapping_workspace", _vp), ("mapping_workspace_bytes", _sz),
        ("matmul_workspace", _vp), ("matmul_workspace_bytes", _sz),
        ("dY_zone", _vp), ("row_weights", _vp), ("dP", _vp), ("dx1", _vp), ("dx3", _vp), ("dZ", _vp),
        ("dX_routed", _vp),
    ]


class TransformerBlock(C.Structure):
    """ctypes mirror of B200TransformerBlock in include/b200_moe.h (same field order)."""
    _fields_ = [
        ("total_tokens", _i), ("model_dim", _i), ("num_q_heads", _i), ("num_kv_heads", _i), ("head_dim", _i), ("theta", _i),
        ("eps", C.c_float), ("num_seqs", _i), ("max_seqlen", _i),
        ("seq_offsets", _vp), ("seq_lens", _vp), ("positions", _vp),
        ("attn_norm", _vp), ("wq", _vp), ("wk", _vp), ("wv", _vp), ("wo", _vp), ("ffn_norm", _vp),
        ("rms1", _vp), ("rms2", _vp), ("q", _vp), ("k", _vp), ("v", _vp), ("attn", _vp), ("lse", _vp),
        ("x_mid", _vp), ("xn2", _vp), ("xn", _vp), ("attn_workspace", _vp), ("attn_workspace_bytes", _u64),
        ("moe", MoeBlock),
    ]


class TransformerBlockGrads(C.Structure):
    _fields_ = [(n, _vp) for n in ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "router", "W1", "W3", "W2")] + [("overwrite", _i)]


class TransformerBlockScratch(C.Structure):
    _fields_ = [(n, _vp) for n in ("dxn", "dattn", "dq", "dk", "dv", "norm_workspace")] + [("norm_workspace_bytes", _u64)]


class EpMoeBlock(C.Structure):
    """ctypes mirror of B200EpMoeBlock in include/b200_moe.h (same field order)."""
    _fields_ = [
        ("world", _i), ("rank", _i),
        ("total_tokens", _i), ("model_dim", _i), ("num_experts", _i), ("top_k", _i), ("ffn_dim", _i),
        ("capacity_rows", _i64),
        ("Wr", _vp), ("W1", _vp), ("W3", _vp), ("W2", _vp),
        ("w1_stride_elems", _i64), ("w3_stride_elems", _i64), ("w2_stride_elems", _i64),
        ("logits", _vp), ("token_expert_weights", _vp), ("chosen_experts", _vp), ("expert_counts", _vp),
        ("expert_counts_cumsum", _vp), ("expert_mapping", _vp), ("token_mapping", _vp),
        ("mapping_workspace", _vp), ("mapping_workspace_bytes", _sz),
        ("matmul_workspace", _vp), ("matmul_workspace_bytes", _sz),
        ("dX_routed", _vp),
        ("gathered_counts", _vp), ("local_counts", _vp), ("local_cumsum", _vp), ("dst_base", _vp), ("overflow", _vp),
        ("barrier_epoch", _vp), ("peer_flags", _vp), ("peer_counts", _vp),
        ("zone_recv", _vp), ("tags_recv", _vp), ("x1", _vp), ("x3", _vp), ("h", _vp),
        ("peer_zone", _vp), ("peer_tags", _vp),
        ("Y_home", _vp), ("peer_Y_home", _vp),
        ("dY_recv", _vp), ("dP_recv", _vp), ("dx1", _vp), ("dx3", _vp), ("ones", _vp), ("dZ_home", _vp),
        ("dWr_partial", _vp),
        ("peer_dY", _vp), ("peer_dP", _vp), ("peer_dZ_home", _vp), ("peer_dWr", _vp),
    ]


class ModelConfig(C.Structure):
    """ctypes mirror of B200ModelConfig (config.txt of a reference model directory)."""
    _fields_ = [
        ("embed_dtype", C.c_char * 16), ("attn_dtype", C.c_char * 16), ("router_dtype", C.c_char * 16),
        ("expert_dtype", C.c_char * 16), ("head_dtype", C.c_char * 16),
        ("vocab_size", _i), ("num_layers", _i), ("model_dim", _i), ("head_dim", _i), ("num_q_heads", _i),
        ("num_kv_heads", _i), ("qk_norm_type", C.c_char * 16), ("qk_norm_weight_type", C.c_char * 16),
        ("num_shared_experts", _i), ("num_routed_experts", _i), ("top_k_routed_experts", _i), ("expert_dim", _i),
        ("expert_mlp_type", C.c_char * 16), ("rope_theta", _i), ("rms_norm_epsilon", _f),
    ]


class MoeLayerLayout(C.Structure):
    """ctypes mirror of B200MoeLayerLayout (byte offsets inside combined_layer.weight)."""
    _fields_ = [
        ("attn_norm", _u64), ("w_q", _u64), ("w_k", _u64), ("w_v", _u64), ("w_o", _u64), ("ffn_norm", _u64),
        ("router", _u64), ("w1_first", _u64), ("w3_first", _u64), ("w2_first", _u64), ("expert_stride_bytes", _u64),
        ("num_experts_in_file", _i), ("first_routed_expert", _i), ("raw_bytes", _u64), ("aligned_bytes", _u64),
    ]


_lib = None


def load():
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ml_dataflow_b200.build` "
                "(nvcc, sm_100a). There is no CPU or library fallback for these ops."
            )
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
