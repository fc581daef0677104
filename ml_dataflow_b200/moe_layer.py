"""The MoE layer as the reference's transformer block drives it, on the sm_100a ops.

Two drivers over the same buffers:

* `forward` / `backward` - the fast path: grouped expert GEMMs (two launches per direction
  instead of the reference's host loop of 3-7 cuBLASLt calls per expert), no host sync, no
  recompute of the W2 forward in backward.
* `forward_reference_order` / `backward_reference_order` - the exact op sequence of
  libdataflowmodels/src/transformer/src/dataflow_transformer.c (forward 2710-2974, backward-x
  3399-3719, backward-w 4062-4185) issued op by op through the drop-in entry points, with the
  host read of the per-expert counts the reference performs (2789). It exists to show that each
  replaced op slots into the reference's own call order.

Shapes: Xn [T, d] bf16, Wr [E, d], W1/W3 [E, f, d], W2 [E, d, f] bf16 (the reference's weight
layouts, models/init_model.py:279-306). All buffers are allocated once in the constructor.
"""
import torch

from . import ops


class MoELayer:
    def __init__(self, T, d, E, k, f, device="cuda"):
        self.T, self.d, self.E, self.k, self.f = T, d, E, k, f
        R = T * k
        self.R = R
        dev = torch.device(device)
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32

        def buf(shape, dt):
            return torch.empty(shape, dtype=dt, device=dev)

        # saved by forward (the reference's Seq_Batch_Saved_Activations MoE fields)
        self.logits = buf((T, E), f32)
        self.weights = buf((T, k), f32)
        self.chosen = buf((T, k), torch.int16)  # uint16 bit patterns
        self.counts = torch.zeros(E + 1, dtype=i32, device=dev)
        self.cumsum = torch.zeros(E, dtype=i32, device=dev)
        self.host_counts = torch.zeros(E, dtype=i32).pin_memory() if dev.type == "cuda" else torch.zeros(E, dtype=i32)
        self.dev_counts_copy = torch.zeros(E, dtype=i32, device=dev)
        self.expert_mapping = buf((R,), i32)
        self.token_mapping = buf((T, k), i32)
        self.map_ws = torch.empty(ops.build_expert_mapping_workspace_bytes(T, E, k), dtype=torch.uint8, device=dev)
        self.mm_ws = torch.empty(16 << 20, dtype=torch.uint8, device=dev)  # split-K scratch of the router GEMMs
        self.zone = buf((R, d), bf)
        self.x1 = buf((R, f), bf)
        self.x3 = buf((R, f), bf)
        self.h = buf((R, f), bf)
        self.Y = buf((R, d), bf)
        # backward working set
        self.dYz = buf((R, d), bf)
        self.row_w = buf((R,), f32)
        self.dP = buf((R,), f32)
        self.dx1 = buf((R, f), bf)
        self.dx3 = buf((R, f), bf)
        self.hs = buf((R, f), bf)
        self.dh = None  # [R, f], allocated on first use by the reference-order backward only
        self.dZ = buf((R, d), bf)
        self.dX_routed = buf((T, E), bf)
        self.profile = None  # list of (name, event) when a caller wants per-op timing (see mark())
        self.keep_pre_gate = False  # tests set this to look at dX_routed before the gate Jacobian is applied
        self.dX_routed_pre = None

    def mark(self, name):
        """Records a CUDA event labelled `name` on the current stream when profiling is switched on."""
        if self.profile is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.profile.append((name, ev))

    def block(self, Wr, W1, W3, W2):
        """The layer's buffers as the C structure `b200_moe_block_fwd` / `b200_moe_block_bwd` take."""
        from . import _lib

        p = lambda t: None if t is None else t.data_ptr()
        d, f = self.d, self.f
        return _lib.MoeBlock(
            self.T, self.d, self.E, self.k, self.f, p(Wr), p(W1), p(W3), p(W2), f * d, f * d, d * f,
            p(self.logits), p(self.weights), p(self.chosen), p(self.counts), p(self.cumsum), None,
            p(self.expert_mapping), p(self.token_mapping), p(self.zone), p(self.x1), p(self.x3), p(self.h), p(self.Y),
            p(self.map_ws), self.map_ws.numel(), p(self.mm_ws), self.mm_ws.numel(), p(self.dYz), p(self.row_w), p(self.dP), p(self.dx1), p(self.dx3),
            p(self.dZ), p(self.dX_routed))

    # ------------------------------------------------------------------ routing (shared)
    def route(self, Xn, Wr, logits=None):
        T, d, E, k = self.T, self.d, self.E, self.k
        self.mark("router_gemm")
        if logits is None:
            # logits[T,E] = Xn . Wr^T, fp32 out (reference call: transa=1, M=E, K=d, N=T)
            ops.matmul(1, 0, E, d, T, 1.0, 0.0, Wr, Xn, None, self.logits, self.mm_ws)
        else:
            self.logits.copy_(logits)
        self.mark("select_experts")
        self.counts.zero_()
        self.cumsum.zero_()
        ops.select_experts(T, E, k, self.logits, self.weights, self.chosen, self.counts, self.cumsum,
                           self.dev_counts_copy)
        self.mark("build_expert_mapping")
        ops.build_expert_mapping(T, E, k, self.chosen, self.cumsum, self.expert_mapping, self.token_mapping,
                                 self.map_ws)

    # ------------------------------------------------------------------ fast path
    def forward(self, Xn, Wr, W1, W3, W2, out, logits=None):
        """out[T,d] (bf16, pre-loaded with the residual or zeros) += combined expert outputs."""
        T, d, E, k, f, R = self.T, self.d, self.E, self.k, self.f, self.R
        self.route(Xn, Wr, logits)
        self.mark("prepare_experts")
        ops.prepare_experts(T, d, k, Xn, self.token_mapping, self.zone)
        self.mark("experts_fwd_gemm")
        ops.moe_experts_fwd(R, d, f, E, self.zone, W1, W3, W2, f * d, f * d, d * f, self.counts, self.cumsum,
                            self.x1, self.x3, self.h, self.Y)
        self.mark("merge_experts")
        ops.merge_experts(T, d, k, self.Y, self.token_mapping, self.weights, out)
        self.mark("fwd_end")
        return out

    def backward(self, Xn, Wr, W1, W3, W2, dOut, dXn, dWr, dW1, dW3, dW2):
        """dXn is overwritten; dWr, dW1, dW3, dW2 (bf16) are accumulated into, like the reference's beta=1 GEMMs."""
        T, d, E, k, f, R = self.T, self.d, self.E, self.k, self.f, self.R
        # dY rows = w * dOut in expert order (what the reference's router_bwd_x leaves in the zone)
        self.mark("prepare_experts_weighted")
        ops.prepare_experts_weighted(T, d, k, dOut, self.token_mapping, self.weights, self.dYz)
        ops.scatter_row_weights(T, k, self.token_mapping, self.weights, self.row_w)
        self.dP.zero_()
        self.mark("experts_bwd_x_gemm")
        ops.moe_experts_bwd_x(R, d, f, E, self.dYz, self.row_w, self.x1, self.x3, W1, W3, W2, f * d, f * d, d * f,
                              self.counts, self.cumsum, self.dx1, self.dx3, None, self.dP, self.dZ)
        # h is still resident from the forward (the reference recomputes it instead)
        self.mark("experts_bwd_w_gemm")
        ops.moe_experts_bwd_w(R, d, f, E, self.dYz, self.h, self.zone, self.dx1, self.dx3, dW1, dW3, dW2,
                              f * d, f * d, d * f, self.counts, self.cumsum)
        self.mark("unpermute")
        ops.unpermute_experts(T, d, k, self.dZ, self.token_mapping, dXn)
        self.mark("router_grad")
        self.dX_routed.zero_()
        ops.gather_router_grad(T, E, k, self.token_mapping, self.chosen, self.dP, self.dX_routed)
        if self.keep_pre_gate:
            self.dX_routed_pre = self.dX_routed.clone()
        ops.router_gate_bwd_x(T, E, k, self.chosen, self.weights, self.dX_routed)
        # dXn += dL . Wr   (reference: transa=0, transb=0, M=d, K=E, N=T, beta=1, C=D)
        ops.matmul(0, 0, d, E, T, 1.0, 1.0, Wr, self.dX_routed, dXn, dXn)
        # dWr += dL^T . Xn (reference: transa=0, transb=1, M=d, K=T, N=E, beta=1, C=D)
        ops.matmul(0, 1, d, T, E, 1.0, 1.0, Xn, self.dX_routed, dWr, dWr, self.mm_ws)
        self.mark("bwd_end")
        return dXn

    # ------------------------------------------------------------------ the reference's own op order
    def forward_reference_order(self, Xn, Wr, W1, W3, W2, out, logits=None):
        T, d, E, k, f = self.T, self.d, self.E, self.k, self.f
        self.route(Xn, Wr, logits)
        self.host_counts.copy_(self.counts[:E], non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the reference's sync_stream (dataflow_transformer.c:2789)
        ops.prepare_experts(T, d, k, Xn, self.token_mapping, self.zone)
        base = 0
        for e in range(E):
            n = int(self.host_counts[e])
            if n == 0:
                continue
            z, x1, x3, h = self.zone[base:base + n], self.x1[base:base + n], self.x3[base:base + n], self.h[base:base + n]
            ops.matmul(1, 0, f, d, n, 1.0, 0.0, W1[e], z, None, x1)
            ops.matmul(1, 0, f, d, n, 1.0, 0.0, W3[e], z, None, x3)
            ops.swiglu(n, f, x1, x3, h)
            ops.matmul(1, 0, d, f, n, 1.0, 0.0, W2[e], h, None, self.Y[base:base + n])
            base += n
        ops.merge_experts(T, d, k, self.Y, self.token_mapping, self.weights, out)
        return out

    def backward_reference_order(self, Xn, Wr, W1, W3, W2, dOut, dXn, dWr, dW1, dW3, dW2):
        T, d, E, k, f = self.T, self.d, self.E, self.k, self.f
        self.dX_routed.zero_()
        zone = self.dZ  # plays the reference's expert zone: holds Y, then dY, then dZ
        base = 0
        for e in range(E):
            n = int(self.host_counts[e])
            if n == 0:
                continue
            sl = slice(base, base + n)
            x1, x3, tmp = self.x1[sl], self.x3[sl], self.hs[sl]
            ops.swiglu(n, f, x1, x3, tmp)  # recompute h, then the expert output
            ops.matmul(1, 0, d, f, n, 1.0, 0.0, W2[e], tmp, None, zone[sl])
            ops.router_bwd_x(n, d, E, k, e, self.cumsum, self.expert_mapping, self.chosen, self.weights, zone[sl],
                             dOut, self.dX_routed, zone[sl])
            ops.matmul(0, 1, f, n, d, 1.0, 1.0, tmp, zone[sl], dW2[e], dW2[e])  # dW2 += dY^T h
            if self.dh is None:
                self.dh = torch.empty_like(self.h)
            dh = self.dh[sl]
            ops.matmul(0, 0, f, d, n, 1.0, 0.0, W2[e], zone[sl], None, dh)  # dh = dY W2
            ops.swiglu_bwd_x(n, f, x1, x3, dh, self.dx1[sl], self.dx3[sl])
            ops.matmul(0, 0, d, f, n, 1.0, 0.0, W1[e], self.dx1[sl], None, zone[sl])
            ops.matmul(0, 0, d, f, n, 1.0, 1.0, W3[e], self.dx3[sl], zone[sl], zone[sl])
            base += n
        dXn.zero_()
        ops.merge_experts(T, d, k, zone, self.token_mapping, None, dXn)
        if self.keep_pre_gate:
            self.dX_routed_pre = self.dX_routed.clone()
        ops.router_gate_bwd_x(T, E, k, self.chosen, self.weights, self.dX_routed)
        ops.matmul(0, 0, d, E, T, 1.0, 1.0, Wr, self.dX_routed, dXn, dXn)
        # backward-w
        ops.prepare_experts(T, d, k, Xn, self.token_mapping, self.zone)
        base = 0
        for e in range(E):
            n = int(self.host_counts[e])
            if n == 0:
                continue
            sl = slice(base, base + n)
            ops.matmul(0, 1, d, n, f, 1.0, 1.0, self.zone[sl], self.dx1[sl], dW1[e], dW1[e])
            ops.matmul(0, 1, d, n, f, 1.0, 1.0, self.zone[sl], self.dx3[sl], dW3[e], dW3[e])
            base += n
        ops.matmul(0, 1, d, T, E, 1.0, 1.0, Xn, self.dX_routed, dWr, dWr, self.mm_ws)
        return dXn
