"""A MoE decoder training step on the sm_100a ops: embedding -> n_layers x (RMSNorm, q/k/v projections, RoPE, causal
attention with grouped query heads, output projection + residual, RMSNorm, MoE feed-forward + residual) -> RMSNorm,
vocabulary projection, softmax, cross-entropy -> the backward of all of it -> AdamW.

It follows the op order of the reference's transformer driver (libdataflowmodels/src/transformer/src/
dataflow_transformer.c: embedding 2283-2342, block forward 2343-2584 and 2588-2986, head 3721-3963, block backward
3386-3719 and 4060-4185, optimizer step) with every op going through this library's C ABI (ops.py); torch only holds
the buffers. Like moe_layer.py it is the test and benchmark harness of the ops, not a second implementation: the
parity test (tests/test_gpu_decoder.py) compares a small model against float32 torch autograd with the routing held
fixed. No activation offload or recompute: every layer keeps what its backward reads (the memory planner of the
reference is out of scope).

Weight layouts are the reference's (models/init_model.py:279-306): projections [out_features][in_features], experts
W1 / W3 [E][f][d], W2 [E][d][f], embedding and head [vocab][d], all bf16.
"""
import math
from dataclasses import dataclass

import torch

from . import ops
from .moe_layer import MoELayer


@dataclass
class DecoderConfig:
    n_layers: int
    d: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    n_experts: int
    top_k: int
    ffn: int
    vocab: int
    eps: float = 1e-5
    theta: int = 500000


def _randn(gen, shape, std, dev):
    return (torch.randn(shape, generator=gen, device=dev) * std).to(torch.bfloat16)


class Decoder:
    """Weights, gradients, optimizer state and the per-layer saved activations for batches of up to `max_tokens`."""

    PARAMS = ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "router", "W1", "W3", "W2")

    def __init__(self, cfg, max_tokens, max_seqlen, device="cuda", seed=0, std=0.02, c_blocks=True):
        """c_blocks: run each block through the C driver (b200_transformer_block_fwd / _bwd, one call per block and
        direction) instead of op by op from here; both issue the same ops in the same order."""
        self.cfg, self.T, self.max_seqlen = cfg, max_tokens, max_seqlen
        self.c_blocks = c_blocks
        self.dev = dev = torch.device(device)
        gen = torch.Generator(device=dev).manual_seed(seed)
        c = cfg
        Dq, Dk = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        self.Dq, self.Dk = Dq, Dk
        ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=dev)
        self.layers = []
        for _ in range(c.n_layers):
            self.layers.append(dict(
                attn_norm=ones(c.d), wq=_randn(gen, (Dq, c.d), std, dev), wk=_randn(gen, (Dk, c.d), std, dev),
                wv=_randn(gen, (Dk, c.d), std, dev), wo=_randn(gen, (c.d, Dq), std, dev), ffn_norm=ones(c.d),
                router=_randn(gen, (c.n_experts, c.d), std, dev), W1=_randn(gen, (c.n_experts, c.ffn, c.d), std, dev),
                W3=_randn(gen, (c.n_experts, c.ffn, c.d), std, dev), W2=_randn(gen, (c.n_experts, c.d, c.ffn), std, dev)))
        self.embed = _randn(gen, (c.vocab, c.d), std, dev)
        self.final_norm = ones(c.d)
        self.head = _randn(gen, (c.vocab, c.d), std, dev)
        self.grads = [{k: torch.zeros_like(v) for k, v in L.items()} for L in self.layers]
        self.g_embed, self.g_final_norm, self.g_head = (torch.zeros_like(t) for t in (self.embed, self.final_norm, self.head))
        self.opt_state = None
        self.step_num = 0
        T = max_tokens
        bf, f32 = torch.bfloat16, torch.float32
        buf = lambda shape, dt=bf: torch.empty(shape, dtype=dt, device=dev)
        # saved per layer: block input, both rms values, rotated q / k, v, attention output and its log-sum-exp, the
        # stream after the attention residual, the normed input of the MoE part; the MoE layer keeps its own set
        self.saved = [dict(x=buf((T, c.d)), rms1=buf((T,), f32), q=buf((T, Dq)), k=buf((T, Dk)), v=buf((T, Dk)),
                           attn=buf((T, Dq)), lse=buf((c.n_heads, T), f32), x_mid=buf((T, c.d)), rms2=buf((T,), f32),
                           xn2=buf((T, c.d)), moe=MoELayer(T, c.d, c.n_experts, c.top_k, c.ffn, device=dev))
                      for _ in range(c.n_layers)]
        self.x_final = buf((T, c.d))
        self.rms_f = buf((T,), f32)
        self.xn = buf((T, c.d))
        self.logits = buf((T, c.vocab))
        self.loss = torch.zeros(T + 1, dtype=f32, device=dev)
        # backward scratch shared by the layers
        self.dx, self.dxn, self.dattn = buf((T, c.d)), buf((T, c.d)), buf((T, Dq))
        self.dq, self.dk, self.dv = buf((T, Dq)), buf((T, Dk)), buf((T, Dk))
        self.attn_ws = torch.empty(max(256, ops.attention_workspace_bytes(True, c.n_heads, c.n_kv_heads, c.head_dim, T, max_seqlen, max_seqlen)), dtype=torch.uint8,
                                   device=dev)
        self.norm_ws = torch.empty(ops.rms_norm_bwd_w_workspace_bytes(T, c.d), dtype=torch.uint8, device=dev)

    def _c_structs(self):
        """The blocks as the C driver takes them (rebuilt per batch: the sequence description is per batch)."""
        import ctypes as C

        from . import _lib

        c, T = self.cfg, self.T
        p = lambda t: t.data_ptr()
        n = len(self.seq_lens)
        self._seq_arrays = ((C.c_int * n)(*self.seq_offs), (C.c_int * n)(*self.seq_lens))  # kept alive with the structs
        offs, lens = (C.cast(a, C.c_void_p) for a in self._seq_arrays)
        blocks, grads = [], []
        for L, S, G in zip(self.layers, self.saved, self.grads):
            moe = S["moe"].block(L["router"], L["W1"], L["W3"], L["W2"])
            blocks.append(_lib.TransformerBlock(
                T, c.d, c.n_heads, c.n_kv_heads, c.head_dim, c.theta, c.eps, n, max(self.seq_lens), offs, lens,
                p(self.positions), p(L["attn_norm"]), p(L["wq"]), p(L["wk"]), p(L["wv"]), p(L["wo"]), p(L["ffn_norm"]),
                p(S["rms1"]), p(S["rms2"]), p(S["q"]), p(S["k"]), p(S["v"]), p(S["attn"]), p(S["lse"]), p(S["x_mid"]),
                p(S["xn2"]), p(self.xn), p(self.attn_ws), self.attn_ws.numel(), moe))
            # one batch per step here: the blocks write their weight gradients, so nothing has to be zeroed first
            grads.append(_lib.TransformerBlockGrads(*[p(G[k]) for k in self.PARAMS], 1))
        scratch = _lib.TransformerBlockScratch(p(self.dxn), p(self.dattn), p(self.dq), p(self.dk), p(self.dv), p(self.norm_ws),
                                               self.norm_ws.numel())
        return blocks, grads, scratch

    # ------------------------------------------------------------------------------------------------ helpers
    @staticmethod
    def _linear(x, w, out, residual=None):
        """out[T][o] = x[T][i] . w[o][i]^T (+ residual)."""
        T, i = x.shape
        o = w.shape[0]
        ops.matmul(1, 0, o, i, T, 1.0, 1.0 if residual is not None else 0.0, w, x, residual, out)

    @staticmethod
    def _linear_dx(dy, w, dx, accumulate):
        """dx[T][i] (+)= dy[T][o] . w[o][i]."""
        T, o = dy.shape
        i = w.shape[1]
        ops.matmul(0, 0, i, o, T, 1.0, 1.0 if accumulate else 0.0, w, dy, dx if accumulate else None, dx)

    @staticmethod
    def _linear_dw(dy, x, dw):
        """dw[o][i] += dy[T][o]^T . x[T][i]."""
        T, o = dy.shape
        i = x.shape[1]
        ops.matmul(0, 1, i, T, o, 1.0, 1.0, x, dy, dw, dw)

    def _sort_tokens(self, token_ids):
        sorted_ids, order = torch.sort(token_ids.to(torch.int64), stable=True)
        first = torch.ones_like(sorted_ids, dtype=torch.bool)
        first[1:] = sorted_ids[1:] != sorted_ids[:-1]
        starts = torch.cat([torch.nonzero(first).flatten(), torch.tensor([sorted_ids.numel()], device=self.dev)])
        return sorted_ids.to(torch.int32), order.to(torch.int32), starts.to(torch.int32), int(starts.numel()) - 1

    # ------------------------------------------------------------------------------------------------ forward
    def forward(self, token_ids, labels, seq_lens):
        """token_ids, labels: int32 [T] on the device; seq_lens: host list of the packed sequences' lengths.
        Leaves the average loss in self.loss[T] and dLoss/dlogits (summed loss) in self.logits."""
        c, T = self.cfg, token_ids.numel()
        assert T == self.T and sum(seq_lens) == T and max(seq_lens) <= self.max_seqlen
        self.seq_lens = list(seq_lens)
        self.seq_offs = [sum(seq_lens[:i]) for i in range(len(seq_lens))]
        self.positions = torch.cat([torch.arange(n, dtype=torch.int32) for n in seq_lens]).to(self.dev)
        self.tokens = self._sort_tokens(token_ids)
        sid, smap, starts, nu = self.tokens
        x = self.saved[0]["x"]
        ops.embedding_table(nu, c.d, sid, smap, starts, self.embed, x)
        if self.c_blocks:
            self._blocks, self._block_grads, self._block_scratch = self._c_structs()
        for li, (L, S) in enumerate(zip(self.layers, self.saved)):
            x = S["x"]
            if self.c_blocks:
                out = self.saved[li + 1]["x"] if li + 1 < c.n_layers else self.x_final
                ops.transformer_block_fwd(self._blocks[li], x, out)
                continue
            ops.rms_norm(T, c.d, c.eps, L["attn_norm"], x, self.xn, S["rms1"])
            self._linear(self.xn, L["wq"], S["q"])
            self._linear(self.xn, L["wk"], S["k"])
            self._linear(self.xn, L["wv"], S["v"])
            ops.rope(T, self.Dq, c.head_dim, c.n_kv_heads, c.theta, self.positions, S["q"], S["k"])
            ops.attention_fwd(self.seq_offs, self.seq_lens, self.seq_offs, self.seq_lens, c.n_heads, c.n_kv_heads, c.head_dim,
                              S["q"], S["k"], S["v"], S["attn"], S["lse"], True, self.attn_ws)
            self._linear(S["attn"], L["wo"], S["x_mid"], residual=x)
            ops.rms_norm(T, c.d, c.eps, L["ffn_norm"], S["x_mid"], S["xn2"], S["rms2"])
            out = self.saved[li + 1]["x"] if li + 1 < c.n_layers else self.x_final
            out.copy_(S["x_mid"])  # the MoE combine accumulates onto the residual
            S["moe"].forward(S["xn2"], L["router"], L["W1"], L["W3"], L["W2"], out)
        ops.rms_norm(T, c.d, c.eps, self.final_norm, self.x_final, self.xn, self.rms_f)
        self._linear(self.xn, self.head, self.logits)
        ops.softmax(T, c.vocab, self.logits, self.logits)
        ops.cross_entropy_loss(T, c.vocab, self.logits, labels, self.loss)
        ops.set_average_loss(T, self.loss)
        return self.loss[T]

    # ------------------------------------------------------------------------------------------------ backward
    def backward(self):
        """Gradients of the SUMMED token losses (what the reference's cross-entropy leaves in the logits buffer),
        accumulated into self.grads / g_embed / g_final_norm / g_head."""
        c, T = self.cfg, self.T
        dlogits = self.logits
        # head: xn still holds the final norm's output
        self._linear_dw(dlogits, self.xn, self.g_head)
        self._linear_dx(dlogits, self.head, self.dxn, accumulate=False)
        self.dx.zero_()
        ops.rms_norm_bwd_w(T, c.d, c.eps, self.rms_f, self.x_final, self.dxn, self.g_final_norm, self.norm_ws)
        ops.rms_norm_bwd_x(T, c.d, c.eps, self.rms_f, self.final_norm, self.x_final, self.dxn, self.dx, None)
        for li in reversed(range(c.n_layers)):
            L, S, G = self.layers[li], self.saved[li], self.grads[li]
            x, moe = S["x"], S["moe"]
            if self.c_blocks:
                ops.transformer_block_bwd(self._blocks[li], x, self.dx, self._block_grads[li], self._block_scratch)
                continue
            # MoE part: dx is the gradient at the block's output; it also flows through the residual unchanged
            moe.backward(S["xn2"], L["router"], L["W1"], L["W3"], L["W2"], self.dx, self.dxn, G["router"], G["W1"], G["W3"],
                         G["W2"])
            ops.rms_norm_bwd_w(T, c.d, c.eps, S["rms2"], S["x_mid"], self.dxn, G["ffn_norm"], self.norm_ws)
            ops.rms_norm_bwd_x(T, c.d, c.eps, S["rms2"], L["ffn_norm"], S["x_mid"], self.dxn, self.dx, None)
            # attention part: x_mid = x + attn . wo^T
            self._linear_dw(self.dx, S["attn"], G["wo"])
            self._linear_dx(self.dx, L["wo"], self.dattn, accumulate=False)
            ops.attention_bwd(self.seq_offs, self.seq_lens, self.seq_offs, self.seq_lens, c.n_heads, c.n_kv_heads, c.head_dim,
                              S["q"], S["k"], S["v"], S["attn"], S["lse"], self.dattn, self.dq, self.dk, self.dv, True,
                              self.attn_ws)
            ops.rope_bwd_x(T, self.Dq, c.head_dim, c.n_kv_heads, c.theta, self.positions, self.dq, self.dk)
            ops.rms_norm_recompute(T, c.d, L["attn_norm"], S["rms1"], x, self.xn)
            self._linear_dw(self.dq, self.xn, G["wq"])
            self._linear_dw(self.dk, self.xn, G["wk"])
            self._linear_dw(self.dv, self.xn, G["wv"])
            self._linear_dx(self.dq, L["wq"], self.dxn, accumulate=False)
            self._linear_dx(self.dk, L["wk"], self.dxn, accumulate=True)
            self._linear_dx(self.dv, L["wv"], self.dxn, accumulate=True)
            ops.rms_norm_bwd_w(T, c.d, c.eps, S["rms1"], x, self.dxn, G["attn_norm"], self.norm_ws)
            ops.rms_norm_bwd_x(T, c.d, c.eps, S["rms1"], L["attn_norm"], x, self.dxn, self.dx, None)
        sid, smap, starts, nu = self.tokens
        ops.embedding_table_bwd_w(nu, c.d, sid, smap, starts, self.dx, self.g_embed)

    # ------------------------------------------------------------------------------------------------ optimizer
    def _all_params(self):
        for L, G in zip(self.layers, self.grads):
            for name in self.PARAMS:
                yield L[name], G[name]
        yield self.embed, self.g_embed
        yield self.final_norm, self.g_final_norm
        yield self.head, self.g_head

    def adamw_step(self, lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1, eps=1e-8):
        if self.opt_state is None:
            self.opt_state = [(torch.zeros_like(p), torch.zeros_like(p)) for p, _ in self._all_params()]
        self.step_num += 1
        for (p, g), (m, v) in zip(self._all_params(), self.opt_state):
            ops.adamw_step(p.numel(), self.step_num, lr, beta1, beta2, weight_decay, eps, p, g, m, v)

    def zero_grads(self):
        """Zeroes what the backward accumulates into. With the C block driver the blocks' gradients are written, not
        accumulated (B200TransformerBlockGrads.overwrite), and only the embedding, final norm and head remain."""
        if self.c_blocks:
            for g in (self.g_embed, self.g_final_norm, self.g_head):
                g.zero_()
            return
        for _, g in self._all_params():
            g.zero_()

    def num_params(self):
        return sum(p.numel() for p, _ in self._all_params())

    def flops_per_token(self):
        """Forward + backward matmul flop per token (6 per active weight), attention at the mean causal span
        excluded."""
        c = self.cfg
        per_layer = c.d * (2 * self.Dq + 2 * self.Dk) + c.n_experts * c.d + c.top_k * 3 * c.d * c.ffn
        return 6 * (c.n_layers * per_layer + c.vocab * c.d)
