"""torch-tensor front end of the C ABI (include/b200_moe.h).

One function per reference op, same argument order and meaning as the reference's
`dataflow_submit_*` functions (libdataflowops/include/dataflow_ops.h:216-294, 70-77) minus the
handle: tensors stand for the device pointers, the CUDA stream is torch's current stream. A
non-zero return from the library raises `RuntimeError` (the reference returns -1). torch is only
used for device memory and streams; every op runs a hand-written sm_100a kernel through ctypes.
"""
import ctypes as C

import torch

from . import _lib

DT_NONE, DT_FP32, DT_BF16 = 0, 3, 5


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t):
    if t is None:
        return DT_NONE
    if t.dtype == torch.float32:
        return DT_FP32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


LAUNCHES = 0  # kernels of this library launched so far (reset it to count a region)
_KERNELS_PER_CALL = {"build_expert_mapping": 2, "moe_experts_fwd": 2, "moe_experts_bwd_x": 2}


def _check(rc, name, launches=None):
    global LAUNCHES
    if rc != 0:
        raise RuntimeError(f"{name} failed (see stderr)")
    LAUNCHES += _KERNELS_PER_CALL.get(name, 1) if launches is None else launches


def device_info():
    sm, major, minor = C.c_int(), C.c_int(), C.c_int()
    _check(_lib.load().b200_device_info(C.byref(sm), C.byref(major), C.byref(minor)), "b200_device_info", 0)
    return sm.value, major.value, minor.value


def gemm_status():
    """Synchronises and returns the status word of the GEMM kernels (0 = every wait completed)."""
    st = C.c_int()
    _check(_lib.load().b200_gemm_status(C.byref(st)), "b200_gemm_status", 0)
    return st.value


def attention_status():
    """Synchronises and returns the status word of the fused attention kernels (0 = every wait completed)."""
    st = C.c_int()
    _check(_lib.load().b200_attention_status(C.byref(st)), "b200_attention_status", 0)
    return st.value


def gemm_set_pair_mode(on):
    """1: CTA pairs (cta_group::2, 256-row tiles); 0: single-CTA 128-row tiles."""
    _check(_lib.load().b200_gemm_set_pair_mode(int(bool(on))), "b200_gemm_set_pair_mode", 0)


def gemm_set_wide_mode(mask):
    """Bit 0 / 1 / 2: forward+dgrad / weight-gradient / dense launches use 256 x 512 units per CTA pair; bit 3: even
    when that leaves too few units to fill the GPU (tests on small shapes)."""
    _check(_lib.load().b200_gemm_set_wide_mode(int(mask)), "b200_gemm_set_wide_mode", 0)


def select_experts(total_tokens, n_experts, top_k_experts, X_routed, token_expert_weights, chosen_experts,
                   expert_counts, expert_counts_cumsum, host_expert_counts=None):
    _check(_lib.load().b200_select_experts(_dt(X_routed), total_tokens, n_experts, top_k_experts, _p(X_routed),
                                           _p(token_expert_weights), _p(chosen_experts), _p(expert_counts),
                                           _p(expert_counts_cumsum), _p(host_expert_counts), _stream()),
           "select_experts")


def build_expert_mapping_workspace_bytes(total_tokens, num_routed_experts, num_selected_experts):
    return int(_lib.load().b200_build_expert_mapping_workspace_bytes(total_tokens, num_routed_experts,
                                                                     num_selected_experts))


def build_expert_mapping(total_tokens, num_routed_experts, num_selected_experts, chosen_experts,
                         expert_counts_cumsum, expert_mapping, token_mapping, workspace):
    _check(_lib.load().b200_build_expert_mapping(total_tokens, num_routed_experts, num_selected_experts,
                                                 _p(chosen_experts), _p(expert_counts_cumsum), _p(expert_mapping),
                                                 _p(token_mapping), _p(workspace),
                                                 workspace.numel() * workspace.element_size(), _stream()),
           "build_expert_mapping")


def prepare_experts(total_tokens, model_dim, num_selected_experts, X, token_mapping, expert_zone):
    _check(_lib.load().b200_prepare_experts(total_tokens, model_dim, num_selected_experts, _p(X), _p(token_mapping),
                                            _p(expert_zone), _stream()), "prepare_experts")


def prepare_experts_weighted(total_tokens, model_dim, num_selected_experts, X, token_mapping, token_expert_weights,
                             expert_zone):
    _check(_lib.load().b200_prepare_experts_weighted(total_tokens, model_dim, num_selected_experts, _p(X),
                                                     _p(token_mapping), _p(token_expert_weights), _p(expert_zone),
                                                     _stream()), "prepare_experts_weighted")


def prepare_expert_zone(model_dim, X, expert_id, expert_counts, expert_counts_cumsum, expert_mapping, expert_zone):
    _check(_lib.load().b200_prepare_expert_zone(model_dim, _p(X), expert_id, _p(expert_counts),
                                                _p(expert_counts_cumsum), _p(expert_mapping), _p(expert_zone),
                                                _stream()), "prepare_expert_zone")


def merge_experts(num_tokens, model_dim, top_k_experts, expert_zones, token_mapping, token_expert_weights,
                  X_combined):
    _check(_lib.load().b200_merge_experts(num_tokens, model_dim, top_k_experts, _p(expert_zones), _p(token_mapping),
                                          _p(token_expert_weights), _p(X_combined), _stream()), "merge_experts")


def unpermute_experts(num_tokens, model_dim, top_k_experts, expert_zones, token_mapping, X_out):
    """X_out[t] = sum of the token's k zone rows (overwrites; the backward's un-permute without the memset)."""
    _check(_lib.load().b200_unpermute_experts(num_tokens, model_dim, top_k_experts, _p(expert_zones), _p(token_mapping),
                                              _p(X_out), _stream()), "unpermute_experts")


def merge_expert_result(num_tokens, model_dim, top_k_experts, expert_zone, expert_id, expert_counts_cumsum,
                        expert_mapping, token_expert_weights, chosen_experts, X_combined):
    _check(_lib.load().b200_merge_expert_result(num_tokens, model_dim, top_k_experts, _p(expert_zone), expert_id,
                                                _p(expert_counts_cumsum), _p(expert_mapping),
                                                _p(token_expert_weights), _p(chosen_experts), _p(X_combined),
                                                _stream()), "merge_expert_result")


def router_bwd_x(num_expert_tokens, model_dim, num_routed_experts, top_k_active, expert_id, expert_counts_cumsum,
                 expert_mapping, chosen_experts, token_expert_weights, expert_out, upstream_dX, dX_routed,
                 dX_expert_out):
    _check(_lib.load().b200_router_bwd_x(num_expert_tokens, model_dim, num_routed_experts, top_k_active, expert_id,
                                         _p(expert_counts_cumsum), _p(expert_mapping), _p(chosen_experts),
                                         _p(token_expert_weights), _p(expert_out), _p(upstream_dX), _p(dX_routed),
                                         _p(dX_expert_out), _stream()), "router_bwd_x")


def router_gate_bwd_x(num_tokens, num_routed_experts, top_k_active, chosen_experts, token_expert_weights, dX_routed):
    _check(_lib.load().b200_router_gate_bwd_x(num_tokens, num_routed_experts, top_k_active, _p(chosen_experts),
                                              _p(token_expert_weights), _p(dX_routed), _stream()),
           "router_gate_bwd_x")


def swiglu(num_rows, num_cols, x_w1, x_w3, out):
    _check(_lib.load().b200_swiglu(num_rows, num_cols, _p(x_w1), _p(x_w3), _p(out), _stream()), "swiglu")


def swiglu_bwd_x(num_rows, num_cols, x_w1, x_w3, upstream_dX, dX_w1, dX_w3):
    _check(_lib.load().b200_swiglu_bwd_x(num_rows, num_cols, _p(x_w1), _p(x_w3), _p(upstream_dX), _p(dX_w1),
                                         _p(dX_w3), _stream()), "swiglu_bwd_x")


def matmul(to_trans_a, to_trans_b, M, K, N, alpha, beta, A, B, Cm, D, workspace=None):
    """Column-major D[MxN] = alpha * op(A) * op(B) + beta * C, the reference's matmul op.
    workspace (a uint8 tensor, optional): fp32 scratch that lets a GEMM with few output tiles and a long reduction
    split the reduction over the SMs."""
    wbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _check(_lib.load().b200_matmul(_dt(A), _dt(B), _dt(Cm), _dt(D), to_trans_a, to_trans_b, M, K, N, alpha, beta,
                                   _p(A), _p(B), _p(Cm), _p(D), wbytes, _p(workspace), _stream()), "matmul")


def moe_experts_fwd(total_rows, model_dim, ffn_dim, num_experts, zone, W1, W3, W2, w1_stride, w3_stride, w2_stride,
                    expert_counts, expert_counts_cumsum, x1, x3, h, Y):
    _check(_lib.load().b200_moe_experts_fwd(total_rows, model_dim, ffn_dim, num_experts, _p(zone), _p(W1), _p(W3),
                                            _p(W2), w1_stride, w3_stride, w2_stride, _p(expert_counts),
                                            _p(expert_counts_cumsum), _p(x1), _p(x3), _p(h), _p(Y), _stream()),
           "moe_experts_fwd")


def moe_experts_bwd_x(total_rows, model_dim, ffn_dim, num_experts, dY_zone, row_weights, x1, x3, W1, W3, W2,
                      w1_stride, w3_stride, w2_stride, expert_counts, expert_counts_cumsum, dx1, dx3, hs, dP, dZ):
    _check(_lib.load().b200_moe_experts_bwd_x(total_rows, model_dim, ffn_dim, num_experts, _p(dY_zone),
                                              _p(row_weights), _p(x1), _p(x3), _p(W1), _p(W3), _p(W2), w1_stride,
                                              w3_stride, w2_stride, _p(expert_counts), _p(expert_counts_cumsum),
                                              _p(dx1), _p(dx3), _p(hs), _p(dP), _p(dZ), _stream()),
           "moe_experts_bwd_x")


def moe_experts_bwd_w(total_rows, model_dim, ffn_dim, num_experts, dY_zone, hs, zone_x, dx1, dx3, dW1, dW3, dW2,
                      dw1_stride, dw3_stride, dw2_stride, expert_counts, expert_counts_cumsum):
    _check(_lib.load().b200_moe_experts_bwd_w(total_rows, model_dim, ffn_dim, num_experts, _p(dY_zone), _p(hs),
                                              _p(zone_x), _p(dx1), _p(dx3), _p(dW1), _p(dW3), _p(dW2), dw1_stride,
                                              dw3_stride, dw2_stride, _p(expert_counts), _p(expert_counts_cumsum),
                                              _stream()), "moe_experts_bwd_w",
           sum(g is not None for g in (dW1, dW3, dW2)))


def scatter_row_weights(num_tokens, top_k, token_mapping, token_expert_weights, row_weights):
    _check(_lib.load().b200_scatter_row_weights(num_tokens, top_k, _p(token_mapping), _p(token_expert_weights),
                                                _p(row_weights), _stream()), "scatter_row_weights")


def gather_router_grad(num_tokens, num_routed_experts, top_k, token_mapping, chosen_experts, dP, dX_routed):
    _check(_lib.load().b200_gather_router_grad(num_tokens, num_routed_experts, top_k, _p(token_mapping),
                                               _p(chosen_experts), _p(dP), _p(dX_routed), _stream()),
           "gather_router_grad")


def _peer_array(ptrs):
    return (C.c_ulonglong * len(ptrs))(*[int(p) for p in ptrs])


def ep_dispatch_rows(total_tokens, model_dim, top_k, X, token_expert_weights, token_mapping, chosen_experts,
                     expert_counts, expert_counts_cumsum, dst_base, peer_buffers, num_experts, experts_per_rank,
                     capacity_rows, local_expert_range=None):
    """peer_buffers: list of device addresses, one per rank (this rank's own buffer included).
    local_expert_range: (begin, end) of the owners' local expert indices to move; None = all."""
    lo, hi = (0, experts_per_rank) if local_expert_range is None else local_expert_range
    _check(_lib.load().b200_ep_dispatch_rows(total_tokens, model_dim, top_k, _p(X), _p(token_expert_weights),
                                             _p(token_mapping), _p(chosen_experts), _p(expert_counts),
                                             _p(expert_counts_cumsum), _p(dst_base), _peer_array(peer_buffers),
                                             len(peer_buffers), num_experts, experts_per_rank, capacity_rows, lo, hi,
                                             _stream()),
           "ep_dispatch_rows", 1 if hi > lo else 0)


def ep_combine_rows(num_tokens, model_dim, top_k, token_expert_weights, token_mapping, chosen_experts, expert_counts,
                    expert_counts_cumsum, dst_base, peer_buffers, num_experts, experts_per_rank, capacity_rows,
                    X_combined):
    _check(_lib.load().b200_ep_combine_rows(num_tokens, model_dim, top_k, _p(token_expert_weights), _p(token_mapping),
                                            _p(chosen_experts), _p(expert_counts), _p(expert_counts_cumsum),
                                            _p(dst_base), _peer_array(peer_buffers), len(peer_buffers), num_experts,
                                            experts_per_rank, capacity_rows, _p(X_combined), _stream()),
           "ep_combine_rows")


def ep_gather_router_grad(num_tokens, top_k, token_expert_weights, token_mapping, chosen_experts, expert_counts,
                          expert_counts_cumsum, dst_base, peer_dP_buffers, num_experts, experts_per_rank, capacity_rows,
                          dX_routed):
    _check(_lib.load().b200_ep_gather_router_grad(num_tokens, top_k, _p(token_expert_weights), _p(token_mapping),
                                                  _p(chosen_experts), _p(expert_counts), _p(expert_counts_cumsum),
                                                  _p(dst_base), _peer_array(peer_dP_buffers), len(peer_dP_buffers),
                                                  num_experts, experts_per_rank, capacity_rows, _p(dX_routed), _stream()),
           "ep_gather_router_grad")


def ep_publish_row_tags(num_tokens, top_k, my_rank, token_mapping, chosen_experts, expert_counts, expert_counts_cumsum,
                        dst_base, peer_tag_buffers, num_experts, experts_per_rank, capacity_rows):
    """Writes (my_rank << 40 | zone row) for every routed pair into the owner's tag array (peer stores)."""
    _check(_lib.load().b200_ep_publish_row_tags(num_tokens, top_k, my_rank, _p(token_mapping), _p(chosen_experts),
                                                _p(expert_counts), _p(expert_counts_cumsum), _p(dst_base),
                                                _peer_array(peer_tag_buffers), len(peer_tag_buffers), num_experts,
                                                experts_per_rank, capacity_rows, _stream()), "ep_publish_row_tags")


def moe_experts_fwd_scatter(total_rows, model_dim, ffn_dim, num_experts, zone, W1, W3, W2, w1_stride, w3_stride,
                            w2_stride, expert_counts, expert_counts_cumsum, x1, x3, h, row_tags, dest_buffers,
                            rows_per_buffer):
    """moe_experts_fwd whose Y rows go to the rows of dest_buffers (device addresses, one per rank) their tags name."""
    _check(_lib.load().b200_moe_experts_fwd_scatter(total_rows, model_dim, ffn_dim, num_experts, _p(zone), _p(W1),
                                                    _p(W3), _p(W2), w1_stride, w3_stride, w2_stride,
                                                    _p(expert_counts), _p(expert_counts_cumsum), _p(x1), _p(x3), _p(h),
                                                    _p(row_tags), _peer_array(dest_buffers), len(dest_buffers),
                                                    rows_per_buffer, _stream()), "moe_experts_fwd_scatter", 2)


def moe_experts_bwd_x_scatter(total_rows, model_dim, ffn_dim, num_experts, dY_zone, row_weights, x1, x3, W1, W3, W2,
                              w1_stride, w3_stride, w2_stride, expert_counts, expert_counts_cumsum, dx1, dx3, hs, dP,
                              row_tags, dest_buffers, rows_per_buffer):
    """moe_experts_bwd_x whose dZ rows go to the rows of dest_buffers their tags name."""
    _check(_lib.load().b200_moe_experts_bwd_x_scatter(total_rows, model_dim, ffn_dim, num_experts, _p(dY_zone),
                                                      _p(row_weights), _p(x1), _p(x3), _p(W1), _p(W3), _p(W2),
                                                      w1_stride, w3_stride, w2_stride, _p(expert_counts),
                                                      _p(expert_counts_cumsum), _p(dx1), _p(dx3), _p(hs), _p(dP),
                                                      _p(row_tags), _peer_array(dest_buffers), len(dest_buffers),
                                                      rows_per_buffer, _stream()), "moe_experts_bwd_x_scatter", 2)


def moe_block_fwd(block, Xn, X_combined):
    """block: a filled `_lib.MoeBlock` (see MoELayer.block). One C call issues the whole forward."""
    _check(_lib.load().b200_moe_block_fwd(C.byref(block), _p(Xn), _p(X_combined), _stream()), "moe_block_fwd", 8)


def moe_block_bwd(block, Xn, dOut, dXn, dWr, dW1, dW3, dW2):
    _check(_lib.load().b200_moe_block_bwd(C.byref(block), _p(Xn), _p(dOut), _p(dXn), _p(dWr), _p(dW1), _p(dW3),
                                          _p(dW2), _stream()), "moe_block_bwd",
           10 + sum(g is not None for g in (dW1, dW3, dW2)))


def moe_block_recompute(block, Xn, recompute_x1_x3):
    """Re-forms zone and h (and x1, x3 when asked) after the forward's workspace has been reused."""
    _check(_lib.load().b200_moe_block_recompute(C.byref(block), _p(Xn), int(bool(recompute_x1_x3)), _stream()),
           "moe_block_recompute", 2)


def ep_moe_block_fwd(block, Xn, X_combined):
    """block: a filled `_lib.EpMoeBlock` (see ExpertParallelMoELayer.c_block). The whole expert-parallel forward of
    this rank in one C call: 13 launches, three of them barrier kernels."""
    _check(_lib.load().b200_ep_moe_block_fwd(C.byref(block), _p(Xn), _p(X_combined), _stream()), "ep_moe_block_fwd", 13)


def ep_moe_block_bwd(block, Xn, dOut, dXn, dWr, dW1, dW3, dW2):
    _check(_lib.load().b200_ep_moe_block_bwd(C.byref(block), _p(Xn), _p(dOut), _p(dXn), _p(dWr), _p(dW1), _p(dW3),
                                             _p(dW2), _stream()), "ep_moe_block_bwd",
           14 + sum(g is not None for g in (dW1, dW3, dW2)))


def ep_status():
    """Synchronises; returns (and clears) the status word of the barrier kernels: 1 = a wait ran out of time."""
    v = C.c_int(0)
    _check(_lib.load().b200_ep_status(C.byref(v)), "b200_ep_status", 0)
    return v.value


# ---- the bandwidth-bound ops of the block around the MoE feed-forward and of the head (bf16) ----------------------
def rms_norm(n_rows, n_cols, eps, rms_weight, X, out, rms_vals=None):
    _check(_lib.load().b200_rms_norm(DT_BF16, n_rows, n_cols, eps, _p(rms_weight), _p(X), _p(out), _p(rms_vals), _stream()),
           "rms_norm")


def rms_norm_recompute(n_rows, n_cols, rms_weight, rms_vals, X, out):
    _check(_lib.load().b200_rms_norm_recompute(DT_BF16, n_rows, n_cols, _p(rms_weight), _p(rms_vals), _p(X), _p(out),
                                               _stream()), "rms_norm_recompute")


def rms_norm_bwd_x(n_rows, n_cols, eps, fwd_rms_vals, rms_weight, X_inp, upstream_dX, dX, X_out=None):
    _check(_lib.load().b200_rms_norm_bwd_x(DT_BF16, DT_BF16, n_rows, n_cols, eps, _p(fwd_rms_vals), _p(rms_weight), _p(X_inp),
                                           _p(upstream_dX), _p(dX), _p(X_out), _stream()), "rms_norm_bwd_x")


def rms_norm_bwd_w_workspace_bytes(n_rows, n_cols):
    return int(_lib.load().b200_rms_norm_bwd_w_workspace_bytes(n_rows, n_cols))


def rms_norm_bwd_w(n_rows, n_cols, eps, fwd_rms_vals, X_inp, upstream_dX, dW, workspace):
    _check(_lib.load().b200_rms_norm_bwd_w(DT_BF16, DT_BF16, n_rows, n_cols, eps, _p(fwd_rms_vals), _p(X_inp), _p(upstream_dX),
                                           _p(dW), workspace.numel() * workspace.element_size(), _p(workspace), _stream()),
           "rms_norm_bwd_w", 2)


def rope(num_tokens, model_dim, head_dim, num_kv_heads, theta, seq_positions, X_q, X_k):
    _check(_lib.load().b200_rope(DT_BF16, num_tokens, model_dim, head_dim, num_kv_heads, theta, _p(seq_positions), _p(X_q),
                                 _p(X_k), _stream()), "rope")


def rope_bwd_x(num_tokens, model_dim, head_dim, num_kv_heads, theta, seq_positions, dX_q, dX_k):
    _check(_lib.load().b200_rope_bwd_x(DT_BF16, num_tokens, model_dim, head_dim, num_kv_heads, theta, _p(seq_positions),
                                       _p(dX_q), _p(dX_k), _stream()), "rope_bwd_x")


def softmax(n_rows, n_cols, X, out):
    _check(_lib.load().b200_softmax(DT_BF16, DT_BF16, n_rows, n_cols, _p(X), _p(out), _stream()), "softmax")


def cross_entropy_loss(n_rows, n_cols, pred_logits, labels, loss_vec):
    _check(_lib.load().b200_cross_entropy_loss(DT_BF16, n_rows, n_cols, _p(pred_logits), _p(labels), _p(loss_vec), _stream()),
           "cross_entropy_loss")


def set_average_loss(n_tokens, loss_vec):
    _check(_lib.load().b200_set_average_loss(n_tokens, _p(loss_vec), _stream()), "set_average_loss")


def adamw_step(num_els, step_num, lr, beta1, beta2, weight_decay, epsilon, param, grad, mean, var):
    _check(_lib.load().b200_adamw_step(DT_BF16, DT_BF16, DT_BF16, DT_BF16, num_els, step_num, lr, beta1, beta2, weight_decay,
                                       epsilon, _p(param), _p(grad), _p(mean), _p(var), _stream()), "adamw_step")


def embedding_table(num_unique_tokens, embed_dim, sorted_token_ids, sorted_token_mapping, unique_token_sorted_inds_start,
                    table, output):
    _check(_lib.load().b200_embedding_table(DT_BF16, num_unique_tokens, embed_dim, _p(sorted_token_ids),
                                            _p(sorted_token_mapping), _p(unique_token_sorted_inds_start), _p(table),
                                            _p(output), _stream()), "embedding_table")


def embedding_table_bwd_w(num_unique_tokens, embed_dim, sorted_token_ids, sorted_token_mapping,
                          unique_token_sorted_inds_start, grad_stream, grad_table):
    _check(_lib.load().b200_embedding_table_bwd_w(DT_BF16, num_unique_tokens, embed_dim, _p(sorted_token_ids),
                                                  _p(sorted_token_mapping), _p(unique_token_sorted_inds_start),
                                                  _p(grad_stream), _p(grad_table), _stream()), "embedding_table_bwd_w")


# ---- attention (packed variable-length sequences; sequence offsets / lengths are host lists) ------------------------
def _int_array(values):
    return (C.c_int * len(values))(*[int(v) for v in values])


def transformer_block_fwd(block, x, out):
    """block: _lib.TransformerBlock; out = block(x)."""
    _check(_lib.load().b200_transformer_block_fwd(C.byref(block), _p(x), _p(out), _stream()), "transformer_block_fwd", 20)


def transformer_block_bwd(block, x, dx, grads, scratch):
    """dx: the gradient at the block's output on entry, at its input on return; grads are accumulated into."""
    _check(_lib.load().b200_transformer_block_bwd(C.byref(block), _p(x), _p(dx), C.byref(grads), C.byref(scratch), _stream()),
           "transformer_block_bwd", 45)


def attention_workspace_bytes(is_training, num_q_heads, num_kv_heads, head_dim, max_total_q, max_seqlen_q, max_seqlen_k):
    return int(_lib.load().b200_attention_workspace_bytes(int(bool(is_training)), num_q_heads, num_kv_heads, head_dim,
                                                          max_total_q, max_seqlen_q, max_seqlen_k))


def attention_fwd(q_offsets, q_lens, k_offsets, k_lens, num_q_heads, num_kv_heads, head_dim, x_q, x_k, x_v, x_attn_out,
                  softmax_lse, is_causal, workspace):
    n = len(q_lens)
    _check(_lib.load().b200_attention_fwd(DT_BF16, n, x_q.shape[0], x_k.shape[0], _int_array(q_offsets), _int_array(q_lens),
                                          max(q_lens), _int_array(k_offsets), _int_array(k_lens), max(k_lens), num_q_heads,
                                          num_kv_heads, head_dim, _p(x_q), _p(x_k), _p(x_v), _p(x_attn_out), _p(softmax_lse),
                                          int(bool(is_causal)), workspace.numel() * workspace.element_size(), _p(workspace),
                                          _stream()), "attention_fwd", 3 * n * num_q_heads)


def attention_bwd(q_offsets, q_lens, k_offsets, k_lens, num_q_heads, num_kv_heads, head_dim, x_q, x_k, x_v, x_attn_out,
                  softmax_lse, dx_out, dx_q, dx_k, dx_v, is_causal, workspace):
    n = len(q_lens)
    _check(_lib.load().b200_attention_bwd(DT_BF16, n, x_q.shape[0], x_k.shape[0], _int_array(q_offsets), _int_array(q_lens),
                                          max(q_lens), _int_array(k_offsets), _int_array(k_lens), max(k_lens), num_q_heads,
                                          num_kv_heads, head_dim, _p(x_q), _p(x_k), _p(x_v), _p(x_attn_out), _p(softmax_lse),
                                          _p(dx_out), _p(dx_q), _p(dx_k), _p(dx_v), int(bool(is_causal)),
                                          workspace.numel() * workspace.element_size(), _p(workspace), _stream()),
           "attention_bwd", n * (9 * num_q_heads + 2 * num_kv_heads))
