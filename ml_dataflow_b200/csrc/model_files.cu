// Reading the reference's model directory: config.txt and layers/<i>/combined_layer.weight. Host code only.
//
// What it follows (reference project paths):
//   * config.txt is one sscanf of 20 "Name: value" lines (libdataflowmodels/src/transformer/src/prep_seq_batch.c:
//     84-130), written by models/init_model.py:153-156.
//   * a block's weights are one file in the order attention norm, q, k, v, o, ffn norm, router, then per expert
//     w1, w3, w2 (libdataflowmodels/src/transformer/src/prep_transformer.c:140-159; writer models/init_model.py:
//     198-318), each tensor starting at the running offset rounded up to the pointer alignment
//     (prep_transformer.c:3-20) and the file read in one piece into the bound buffer (prep_transformer.c:368-388).
// Only the MoE part of the block is used by this library: the offsets of the ffn norm, the router weight and the
// experts, and the stride between experts, which is what B200MoeBlock's weight pointers need.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "../../include/b200_moe.h"

static int dtype_bytes(const char *name) {
  if (!strcmp(name, "bf16") || !strcmp(name, "fp16")) return 2;
  if (!strcmp(name, "fp32")) return 4;
  return 0;
}

extern "C" int b200_parse_model_config(const char *config_txt_path, B200ModelConfig *out) {
  B200_REQUIRE(config_txt_path && out, "parse_model_config: null argument");
  FILE *fh = fopen(config_txt_path, "rb");
  B200_REQUIRE(fh != nullptr, "parse_model_config: could not open %s", config_txt_path);
  char text[4096];
  const size_t n = fread(text, 1, sizeof(text) - 1, fh);
  fclose(fh);
  text[n] = '\0';
  memset(out, 0, sizeof(*out));
  // the same twenty fields, in the same order, as the reference's parser
  const int got = sscanf(text,
                         "Embed Dtype: %15s\nAttn Dtype: %15s\nRouter Dtype: %15s\nExpert Dtype: %15s\nHead Dtype: %15s\n"
                         "Vocab Size: %d\nNum Layers: %d\nModel Dim: %d\nHead Dim: %d\nNum Q Heads: %d\nNum KV Heads: %d\n"
                         "QK Norm Type: %15s\nQK Norm Weight Type: %15s\nNum Shared Experts: %d\nNum Routed Experts: %d\n"
                         "Top K Routed Experts: %d\nExpert Dim: %d\nExpert MLP Type: %15s\nRope Theta: %d\n"
                         "RMS Norm Epsilon: %f\n",
                         out->embed_dtype, out->attn_dtype, out->router_dtype, out->expert_dtype, out->head_dtype,
                         &out->vocab_size, &out->num_layers, &out->model_dim, &out->head_dim, &out->num_q_heads,
                         &out->num_kv_heads, out->qk_norm_type, out->qk_norm_weight_type, &out->num_shared_experts,
                         &out->num_routed_experts, &out->top_k_routed_experts, &out->expert_dim, out->expert_mlp_type,
                         &out->rope_theta, &out->rms_norm_epsilon);
  B200_REQUIRE(got == 20, "parse_model_config: %s does not match the expected format (%d of 20 fields)", config_txt_path,
               got);
  return 0;
}

// running offset -> offset of the next tensor; sizes of zero take no space (prep_transformer.c:3-20)
static uint64_t place(uint64_t size, uint64_t *aligned, uint64_t *raw, uint64_t alignment) {
  const uint64_t at = *aligned;
  if (size == 0) return at;
  *raw += size;
  *aligned += size;
  if (alignment > 0 && *aligned % alignment) *aligned += alignment - *aligned % alignment;
  return at;
}

extern "C" int b200_moe_layer_file_layout(const B200ModelConfig *cfg, int pointer_alignment, B200MoeLayerLayout *out) {
  B200_REQUIRE(cfg && out, "moe_layer_file_layout: null argument");
  B200_REQUIRE(pointer_alignment >= 0, "moe_layer_file_layout: negative alignment");
  const uint64_t attn_el = dtype_bytes(cfg->attn_dtype), router_el = dtype_bytes(cfg->router_dtype),
                 expert_el = dtype_bytes(cfg->expert_dtype);
  B200_REQUIRE(attn_el && expert_el && (router_el || cfg->num_routed_experts == 0),
               "moe_layer_file_layout: unknown dtype (attn %s, router %s, expert %s)", cfg->attn_dtype, cfg->router_dtype,
               cfg->expert_dtype);
  B200_REQUIRE(cfg->model_dim > 0 && cfg->head_dim > 0 && cfg->num_q_heads > 0 && cfg->num_kv_heads > 0 &&
                   cfg->expert_dim > 0 && cfg->num_routed_experts >= 0 && cfg->num_shared_experts >= 0,
               "moe_layer_file_layout: bad dimensions");
  B200_REQUIRE(!strcmp(cfg->expert_mlp_type, "swiglu"), "moe_layer_file_layout: expert MLP type %s is not supported",
               cfg->expert_mlp_type);
  // per-head / per-token q,k norm weights sit between v and o in the writer (init_model.py:247-268); the reference's
  // own loader has no slot for them, and neither has this one
  B200_REQUIRE(!strcmp(cfg->qk_norm_weight_type, "none"), "moe_layer_file_layout: q/k norm weights (%s) are not supported",
               cfg->qk_norm_weight_type);
  const uint64_t d = (uint64_t)cfg->model_dim, attn_dim = (uint64_t)cfg->num_q_heads * cfg->head_dim,
                 kv_dim = (uint64_t)cfg->num_kv_heads * cfg->head_dim, f = (uint64_t)cfg->expert_dim;
  const uint64_t al = (uint64_t)pointer_alignment;
  uint64_t aligned = 0, raw = 0;
  memset(out, 0, sizeof(*out));
  out->attn_norm = place(d * attn_el, &aligned, &raw, al);
  out->w_q = place(d * attn_dim * attn_el, &aligned, &raw, al);
  out->w_k = place(d * kv_dim * attn_el, &aligned, &raw, al);
  out->w_v = place(d * kv_dim * attn_el, &aligned, &raw, al);
  out->w_o = place(attn_dim * d * attn_el, &aligned, &raw, al);
  out->ffn_norm = place(d * attn_el, &aligned, &raw, al);
  out->router = place(d * (uint64_t)cfg->num_routed_experts * router_el, &aligned, &raw, al);
  const int experts = cfg->num_shared_experts + cfg->num_routed_experts;
  out->num_experts_in_file = experts;
  for (int e = 0; e < experts; e++) {
    const uint64_t w1 = place(f * d * expert_el, &aligned, &raw, al);
    const uint64_t w3 = place(f * d * expert_el, &aligned, &raw, al);
    const uint64_t w2 = place(d * f * expert_el, &aligned, &raw, al);
    if (e == 0) {
      out->w1_first = w1;
      out->w3_first = w3;
      out->w2_first = w2;
    } else if (e == 1) {
      out->expert_stride_bytes = w1 - out->w1_first;
    }
  }
  if (experts == 1) out->expert_stride_bytes = aligned - out->w1_first;
  // shared experts come first in the file (init_model.py:285), the routed ones after them
  out->first_routed_expert = cfg->num_shared_experts;
  out->raw_bytes = raw;
  out->aligned_bytes = aligned;
  return 0;
}

extern "C" int b200_read_layer_file(const char *path, void *host_buffer, uint64_t bytes) {
  B200_REQUIRE(path && host_buffer, "read_layer_file: null argument");
  FILE *fh = fopen(path, "rb");
  B200_REQUIRE(fh != nullptr, "read_layer_file: could not open %s", path);
  const size_t got = fread(host_buffer, 1, (size_t)bytes, fh);
  // one byte more would mean the file holds something this layout does not describe
  char extra;
  const size_t more = fread(&extra, 1, 1, fh);
  fclose(fh);
  B200_REQUIRE(got == (size_t)bytes, "read_layer_file: %s holds %zu bytes, the layout needs %llu", path, got,
               (unsigned long long)bytes);
  B200_REQUIRE(more == 0, "read_layer_file: %s is longer than the %llu bytes of the layout", path,
               (unsigned long long)bytes);
  return 0;
}

extern "C" int b200_moe_block_bind_weights(B200MoeBlock *block, const B200ModelConfig *cfg,
                                           const B200MoeLayerLayout *layout, const void *layer_base) {
  B200_REQUIRE(block && cfg && layout && layer_base, "moe_block_bind_weights: null argument");
  B200_REQUIRE(dtype_bytes(cfg->expert_dtype) == 2 && dtype_bytes(cfg->router_dtype) == 2 &&
                   !strcmp(cfg->expert_dtype, "bf16") && !strcmp(cfg->router_dtype, "bf16"),
               "moe_block_bind_weights: the kernels take bf16 router and expert weights (file has %s, %s)",
               cfg->router_dtype, cfg->expert_dtype);
  B200_REQUIRE(cfg->num_routed_experts >= 1, "moe_block_bind_weights: the layer has no routed experts");
  B200_REQUIRE(layout->expert_stride_bytes % 16 == 0 && layout->router % 16 == 0 && layout->w1_first % 16 == 0 &&
                   layout->w3_first % 16 == 0 && layout->w2_first % 16 == 0 && b200_aligned16(layer_base),
               "moe_block_bind_weights: tensors must start on 16-byte boundaries (use a pointer alignment that is a "
               "multiple of 16, and an aligned buffer)");
  const unsigned char *base = static_cast<const unsigned char *>(layer_base);
  const uint64_t skip = (uint64_t)layout->first_routed_expert * layout->expert_stride_bytes;
  block->model_dim = cfg->model_dim;
  block->num_experts = cfg->num_routed_experts;
  block->top_k = cfg->top_k_routed_experts;
  block->ffn_dim = cfg->expert_dim;
  block->Wr = base + layout->router;
  block->W1 = base + layout->w1_first + skip;
  block->W3 = base + layout->w3_first + skip;
  block->W2 = base + layout->w2_first + skip;
  block->w1_stride_elems = block->w3_stride_elems = block->w2_stride_elems = (int64_t)(layout->expert_stride_bytes / 2);
  return 0;
}
