"""Expert-parallel MoE layer: experts sharded over the ranks of one node, tokens data-parallel.

The reference is single-GPU (its `MoE_Config.num_local_experts / local_expert_inds`,
libdataflowmodels/include/dataflow_models.h:51-67, are placeholders), so the per-token maths is the
only behaviour to match; the exchange is new. Rank g owns experts [g*E/G, (g+1)*E/G) with their
W1/W3/W2 and gradients; the router weight is replicated and its gradient all-reduced.

Per layer and direction there is one exchange each way:

  route locally (global expert ids) -> counts[E] -> counts exchange (G x E/G ints)
  -> rows already sit expert-contiguous in the zone, so the block of rows for (destination rank h,
     local expert j) is one contiguous slice; it is sent straight into the receiver's region of
     expert j, at the offset of this source rank. The receive buffer is therefore expert-contiguous
     (source-major inside an expert) with no second permutation, and the grouped GEMMs run on it
     unchanged with per-expert counts summed over sources.
  -> grouped expert GEMMs on the received rows -> the reverse exchange -> local weighted combine.

Three transports for the rows:
  * "fused" (default): as "p2p" on the way out; on the way back the LAST GEMM of each pass does the exchange itself: its
    epilogue stores every output row (Y forward, dZ backward) straight into the zone-ordered buffer of the token's
    home rank (peer stores, tile by tile under the MMAs of the next tile), guided by a per-row tag the home rank
    published next to the row. After one barrier the combine / un-permute is a purely local kernel.
  * "p2p": the receive buffers are NVLink-mapped into every rank (torch symmetric memory gives the
    peer addresses). The gather kernel stores each row straight into its owner's buffer and the combine kernel loads
    each expert output row straight from its owner (csrc/ep_p2p.cu): no staging copy, no collective on the data path,
    only a stream-ordered barrier between the phases.
  * "nccl": rows are first gathered locally and then moved with NCCL point-to-point batches.

`RowExchange` holds only the bookkeeping and the point-to-point batches (torch.distributed
`batch_isend_irecv`: one NCCL group per exchange over NVLink; also runs on gloo for the CPU tests).
Only the "nccl" transport needs the row counts on the host (to size its messages): its `plan()` reads
the exchanged counts back once per layer - the same place where the reference's block synchronises to
read `host_expert_counts` (dataflow_transformer.c:2789). The peer-memory transports use
`plan_on_device()` and never leave the stream.
"""
import torch


class RowExchange:
    """Bookkeeping + transport of routed rows between `world` ranks owning `E // world` experts each."""

    def __init__(self, dist, num_experts, device):
        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        assert num_experts % self.world == 0, "experts must divide evenly over the ranks"
        self.E = num_experts
        self.E_loc = num_experts // self.world
        self.device = device

    # -------------------------------------------------------------------------------- plan
    def plan(self, counts_dev):
        """counts_dev: int32 [E] per-expert row counts of this rank's tokens (device tensor).

        Exchanges the counts, then fills (host lists / device tensors):
          send_off[h][j], send_cnt[h][j] : slice of the local zone holding rows for rank h's expert j
          recv_off[s][j], recv_cnt[s][j] : slice of the receive buffer for rows from rank s, local expert j
          local_counts, local_cumsum     : int32 [E_loc] device tensors for the grouped GEMMs (inclusive cumsum)
          rows_recv                      : total received rows
        """
        G, El = self.world, self.E_loc
        mine = counts_dev[: self.E].to(torch.int32).contiguous()
        gathered = torch.empty(G * self.E, dtype=torch.int32, device=mine.device)
        self.dist.all_gather_into_tensor(gathered, mine)
        all_counts = gathered.cpu().view(G, G, El)  # [source rank][destination rank][local expert]  (host sync)
        send_cnt = all_counts[self.rank]                     # [h][j]
        recv_cnt = all_counts[:, self.rank, :].contiguous()  # [s][j]
        send_off = (torch.cumsum(send_cnt.reshape(-1), 0) - send_cnt.reshape(-1)).view(G, El)
        per_expert = recv_cnt.sum(dim=0)                     # [j]
        expert_base = torch.cumsum(per_expert, 0) - per_expert
        within = torch.cumsum(recv_cnt, 0) - recv_cnt        # offset of source s inside expert j
        recv_off = expert_base.view(1, El) + within
        self.send_cnt, self.send_off = send_cnt.tolist(), send_off.tolist()
        self.recv_cnt, self.recv_off = recv_cnt.tolist(), recv_off.tolist()
        self.rows_recv = int(per_expert.sum())
        self.rows_send = int(send_cnt.sum())
        self.local_counts = per_expert.to(torch.int32).to(self.device)
        self.local_cumsum = torch.cumsum(per_expert, 0).to(torch.int32).to(self.device)
        # first row, in the OWNER's buffer, of this rank's rows of every global expert (used by the peer-memory kernels)
        per_owner = all_counts.sum(dim=0)                               # [h][j] rows of owner h's expert j
        owner_base = torch.cumsum(per_owner, 1) - per_owner             # [h][j]
        before_me = all_counts[: self.rank].sum(dim=0)                  # rows of lower source ranks
        self.dst_base = (owner_base + before_me).reshape(-1).to(torch.int32).to(self.device)
        return self

    def plan_on_device(self, counts_dev, capacity_rows):
        """The part of `plan` the peer-memory transports need, computed on the device with no host read:
        `local_counts`, `local_cumsum` (int32 [E_loc], clipped to `capacity_rows`), `dst_base` (int32 [E]) and
        `rows_recv_dev` (0-dim int64 tensor, unclipped). The layer then launches everything with its buffer capacity as the row bound; the kernels take the
        real per-expert counts from these tensors."""
        G, El = self.world, self.E_loc
        mine = counts_dev[: self.E].to(torch.int32).contiguous()
        gathered = torch.empty(G * self.E, dtype=torch.int32, device=mine.device)
        self.dist.all_gather_into_tensor(gathered, mine)
        all_counts = gathered.view(G, G, El).to(torch.int64)  # [source rank][destination rank][local expert]
        per_expert = all_counts[:, self.rank, :].sum(dim=0)
        self.rows_recv_dev = per_expert.sum()
        # what the GEMMs are told never reaches past the buffer: rows that do not fit are dropped by the senders
        # (capacity bound of the peer-memory kernels) and by these clipped counts alike
        cum = torch.cumsum(per_expert, 0).clamp(max=int(capacity_rows))
        self.local_cumsum = cum.to(torch.int32)
        self.local_counts = (cum - torch.cat([cum.new_zeros(1), cum[:-1]])).to(torch.int32)
        per_owner = all_counts.sum(dim=0)
        owner_base = torch.cumsum(per_owner, 1) - per_owner
        before_me = all_counts[: self.rank].sum(dim=0)
        self.dst_base = (owner_base + before_me).reshape(-1).to(torch.int32)
        return self

    # -------------------------------------------------------------------------------- transport
    def _exchange(self, src, dst, out_cnt, out_off, in_cnt, in_off):
        """Rows src[out_off[p][j] : +out_cnt[p][j]] go to rank p; rows from rank p land in dst[in_off[p][j] : ...]."""
        dist = self.dist
        ops = []
        for j in range(self.E_loc):
            n = out_cnt[self.rank][j]
            if n:
                dst[in_off[self.rank][j]: in_off[self.rank][j] + n].copy_(
                    src[out_off[self.rank][j]: out_off[self.rank][j] + n])
        for step in range(1, self.world):
            to, frm = (self.rank + step) % self.world, (self.rank - step) % self.world
            for j in range(self.E_loc):
                if out_cnt[to][j]:
                    ops.append(dist.P2POp(dist.isend, src[out_off[to][j]: out_off[to][j] + out_cnt[to][j]], to))
                if in_cnt[frm][j]:
                    ops.append(dist.P2POp(dist.irecv, dst[in_off[frm][j]: in_off[frm][j] + in_cnt[frm][j]], frm))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return dst

    def dispatch(self, zone_rows, recv_rows):
        """Local zone (expert-contiguous over all E experts) -> receive buffer (this rank's experts)."""
        return self._exchange(zone_rows, recv_rows, self.send_cnt, self.send_off, self.recv_cnt, self.recv_off)

    def combine(self, recv_rows, zone_rows):
        """The reverse exchange: rows computed by the owning rank go back to their slot in the source's zone."""
        return self._exchange(recv_rows, zone_rows, self.recv_cnt, self.recv_off, self.send_cnt, self.send_off)


class ExpertParallelMoELayer:
    """Same call surface as `MoELayer`, with W1/W3/W2 and their gradients holding only this rank's experts."""

    def __init__(self, T, d, E, k, f, dist, device="cuda", recv_capacity_factor=1.5, transport="fused", slices=1):
        self.T, self.d, self.E, self.k, self.f = T, d, E, k, f
        self.dist = dist
        self.dev = torch.device(device)
        self.transport = transport
        self.x = RowExchange(dist, E, self.dev)
        self.E_loc = self.x.E_loc
        self.R = T * k
        if transport not in ("fused", "p2p", "nccl"):
            raise ValueError(f"unknown expert-parallel transport {transport!r}")
        self.home = _HomeSide(T, d, E, k, self.dev, staging=(transport == "nccl"))
        self.cap = int(self.R * recv_capacity_factor) + 256
        bf, f32 = torch.bfloat16, torch.float32

        def buf(shape, dt):
            return torch.empty(shape, dtype=dt, device=self.dev)

        self.peers = {}
        if transport in ("fused", "p2p"):
            import torch.distributed._symmetric_memory as symm_mem

            def shared(name, shape, dt):
                t = symm_mem.empty(shape, dtype=dt, device=self.dev)
                hdl = symm_mem.rendezvous(t, dist.group.WORLD)
                self.peers[name] = [int(p) for p in hdl.buffer_ptrs]
                self._handles = getattr(self, "_handles", []) + [hdl]
                return t
        else:
            def shared(name, shape, dt):
                return buf(shape, dt)

        # buffers other ranks write into / read from
        self.zone_r = shared("zone", (self.cap, d), bf)   # received rows (kept for backward-w)
        self.dY_r = shared("dY", (self.cap, d), bf)
        self.dP_r = shared("dP", (self.cap,), f32)
        if transport == "fused":
            # the GEMM epilogues store Y / dZ rows straight into the home rank's zone-ordered buffers
            self.tags_r = shared("tags", (self.cap,), torch.int64)
            self.Y_h = shared("Yh", (self.R, d), bf)
            self.dZ_h = shared("dZh", (self.R, d), bf)
        else:
            self.Y_r = shared("Y", (self.cap, d), bf)
            self.dZ_r = shared("dZ", (self.cap, d), bf)
        # local only
        self.x1, self.x3, self.h = buf((self.cap, f), bf), buf((self.cap, f), bf), buf((self.cap, f), bf)
        self.dx1, self.dx3 = buf((self.cap, f), bf), buf((self.cap, f), bf)
        self.ones = torch.ones(self.cap, dtype=f32, device=self.dev)
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.overflowed = torch.zeros((), dtype=torch.bool, device=self.dev)
        self.rows = 0
        self.profile = None
        # "fused": the outward exchange can run in slices of local experts on a side stream, slice c+1 under the GEMMs
        # of slice c (the copy blocks are small enough to share the SMs with the persistent GEMM CTAs). Measured on
        # 2 GPUs the copies are hidden but slow the GEMMs, which are bound by the same L2 paths, by as much as they
        # hide (1 slice 36.8 ms/step, 4 slices 38.2, 8 slices 39.1), hence one slice by default.
        n_sl = max(1, min(int(slices), self.E_loc))
        edges = [round(i * self.E_loc / n_sl) for i in range(n_sl + 1)]
        self.slices = [(a, b) for a, b in zip(edges[:-1], edges[1:]) if b > a]
        if transport == "fused":
            self.side = torch.cuda.Stream(device=self.dev)
            self.side_group = dist.new_group()  # its own communicator: side-stream barriers never queue behind main's
            self._flag_side = torch.zeros(1, dtype=torch.int32, device=self.dev)

    def c_block(self, Wr, W1, W3, W2):
        """Fills a `B200EpMoeBlock` for b200_ep_moe_block_fwd / _bwd over this layer's buffers ("fused" transport
        only): the same step with the barriers, the counts exchange, the plan and the router-gradient sum done by
        the library's own kernels over peer memory instead of torch.distributed. Collective: every rank calls it."""
        import ctypes as C

        from . import _lib

        if self.transport != "fused":
            raise ValueError("the C block runs on the buffers of the 'fused' transport")
        if not hasattr(self, "_c_shared"):
            import torch.distributed._symmetric_memory as symm_mem

            def shared(name, shape, dt):
                t = symm_mem.empty(shape, dtype=dt, device=self.dev)
                t.zero_()
                hdl = symm_mem.rendezvous(t, self.dist.group.WORLD)
                self.peers[name] = [int(p) for p in hdl.buffer_ptrs]
                self._handles.append(hdl)
                return t

            G = self.x.world
            self._c_shared = dict(flags=shared("flags", (max(G, 4),), torch.int32),
                                  gathered=shared("gathered", (G, self.E), torch.int32),
                                  dWr_part=shared("dWr_part", (self.E, self.d), torch.bfloat16))
            self._c_local = dict(
                local_counts=torch.zeros(self.E_loc, dtype=torch.int32, device=self.dev),
                local_cumsum=torch.zeros(self.E_loc, dtype=torch.int32, device=self.dev),
                dst_base=torch.zeros(self.E, dtype=torch.int32, device=self.dev),
                overflow=torch.zeros(1, dtype=torch.int32, device=self.dev),
                epoch=torch.zeros(1, dtype=torch.int32, device=self.dev))
            torch.cuda.synchronize(self.dev)
            self.dist.barrier()  # every rank's flag array is zero before the first barrier kernel runs
        hm, sh, lo = self.home, self._c_shared, self._c_local
        ptr = lambda t: t.data_ptr()
        self._c_tables = {n: (C.c_ulonglong * len(v))(*v) for n, v in self.peers.items()}
        tab = lambda n: C.cast(self._c_tables[n], C.c_void_p)
        b = _lib.EpMoeBlock()
        b.world, b.rank = self.x.world, self.x.rank
        b.total_tokens, b.model_dim, b.num_experts, b.top_k, b.ffn_dim = self.T, self.d, self.E, self.k, self.f
        b.capacity_rows = self.cap
        b.Wr, b.W1, b.W3, b.W2 = ptr(Wr), ptr(W1), ptr(W3), ptr(W2)
        b.w1_stride_elems = b.w3_stride_elems = self.f * self.d
        b.w2_stride_elems = self.d * self.f
        b.logits, b.token_expert_weights, b.chosen_experts = ptr(hm.logits), ptr(hm.weights), ptr(hm.chosen)
        b.expert_counts, b.expert_counts_cumsum = ptr(hm.counts), ptr(hm.cumsum)
        b.expert_mapping, b.token_mapping = ptr(hm.expert_mapping), ptr(hm.token_mapping)
        b.mapping_workspace, b.mapping_workspace_bytes = ptr(hm.map_ws), hm.map_ws.numel()
        b.matmul_workspace, b.matmul_workspace_bytes = ptr(hm.mm_ws), hm.mm_ws.numel()
        b.dX_routed = ptr(hm.dX_routed)
        b.gathered_counts = ptr(sh["gathered"])
        b.local_counts, b.local_cumsum, b.dst_base = ptr(lo["local_counts"]), ptr(lo["local_cumsum"]), ptr(lo["dst_base"])
        b.overflow, b.barrier_epoch = ptr(lo["overflow"]), ptr(lo["epoch"])
        b.peer_flags, b.peer_counts = tab("flags"), tab("gathered")
        b.zone_recv, b.tags_recv = ptr(self.zone_r), ptr(self.tags_r)
        b.x1, b.x3, b.h = ptr(self.x1), ptr(self.x3), ptr(self.h)
        b.peer_zone, b.peer_tags = tab("zone"), tab("tags")
        b.Y_home, b.peer_Y_home = ptr(self.Y_h), tab("Yh")
        b.dY_recv, b.dP_recv, b.dx1, b.dx3, b.ones = ptr(self.dY_r), ptr(self.dP_r), ptr(self.dx1), ptr(self.dx3), ptr(self.ones)
        b.dZ_home, b.dWr_partial = ptr(self.dZ_h), ptr(sh["dWr_part"])
        b.peer_dY, b.peer_dP, b.peer_dZ_home, b.peer_dWr = tab("dY"), tab("dP"), tab("dZh"), tab("dWr_part")
        return b

    def check(self):
        """Synchronises and raises if a step received more rows than the buffers hold (the extra rows were dropped,
        never written out of bounds) or if a GEMM kernel gave up a bounded wait."""
        from . import ops

        if hasattr(self, "_c_local") and int(self._c_local["overflow"].item()):
            raise RuntimeError(f"expert-parallel receive buffer too small (capacity {self.cap} rows): rows were dropped")
        if hasattr(self, "_c_local") and ops.ep_status():
            raise RuntimeError("a barrier kernel of the expert-parallel layer ran out of time")
        if bool(self.overflowed.item()):
            raise RuntimeError(f"expert-parallel receive buffer too small (capacity {self.cap} rows): rows were dropped")
        st = ops.gemm_status()
        if st:
            raise RuntimeError(f"a GEMM kernel gave up waiting (status {st})")

    def _barrier(self):
        """Stream-ordered barrier over all ranks: everything enqueued before it on every rank has finished (and its
        peer stores have landed) before anything enqueued after it starts."""
        self.dist.all_reduce(self._flag)

    def _sliced_dispatch(self, rows, row_weights, peer_buffers, publish_tags):
        """Enqueues, on the side stream, the outward exchange slice by slice (each followed by a barrier) and
        returns one event per slice: once it has fired, this rank's buffer holds every rank's rows of that slice."""
        from . import ops

        hm, x = self.home, self.x
        T, d, E, k = self.T, self.d, self.E, self.k
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        events = []
        with torch.cuda.stream(self.side):
            self.side.wait_event(start)
            for i, (a, b) in enumerate(self.slices):
                ops.ep_dispatch_rows(T, d, k, rows, row_weights, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum,
                                     x.dst_base, peer_buffers, E, self.E_loc, self.cap, (a, b))
                if publish_tags and i == 0:
                    ops.ep_publish_row_tags(T, k, self.dist.get_rank(), hm.token_mapping, hm.chosen, hm.counts,
                                            hm.cumsum, x.dst_base, self.peers["tags"], E, self.E_loc, self.cap)
                self.dist.all_reduce(self._flag_side, group=self.side_group)
                ev = torch.cuda.Event()
                ev.record(self.side)
                events.append(ev)
        return events

    def mark(self, name):
        if self.profile is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.profile.append((name, ev))

    def forward(self, Xn, Wr, W1, W3, W2, out):
        from . import ops

        hm, x = self.home, self.x
        T, d, E, k, f = self.T, self.d, self.E, self.k, self.f
        self.mark("router_gemm")
        hm.route(Xn, Wr)
        fused = self.transport == "fused"
        p2p = fused or self.transport == "p2p"
        if not p2p:
            self.mark("prepare_experts")
            ops.prepare_experts(T, d, k, Xn, hm.token_mapping, hm.zone)
        self.mark("dispatch")
        # the counts exchange also orders this step after every rank's previous step (its buffers are free again)
        if p2p:
            # no host read of the counts: every launch below is bounded by the buffer capacity and reads the real
            # counts on the device; an overflow is recorded in self.overflowed and raised by check()
            x.plan_on_device(hm.counts, self.cap)
            self.overflowed |= x.rows_recv_dev > self.cap
            n = self.cap
        else:
            x.plan(hm.counts)
            if x.rows_recv > self.cap:
                raise RuntimeError(f"expert-parallel receive buffer too small: {x.rows_recv} rows > capacity {self.cap}")
            n = x.rows_recv
        self.rows = n
        if fused:
            ready = self._sliced_dispatch(Xn, None, self.peers["zone"], publish_tags=True)
            for (a, b), ev in zip(self.slices, ready):
                self.mark("dispatch")
                torch.cuda.current_stream().wait_event(ev)
                self.mark("experts_fwd_gemm")
                ops.moe_experts_fwd_scatter(n, d, f, b - a, self.zone_r, W1[a:b], W3[a:b], W2[a:b], f * d, f * d, d * f,
                                            x.local_counts[a:b], x.local_cumsum[a:b], self.x1, self.x3, self.h,
                                            self.tags_r, self.peers["Yh"], self.R)
            self.mark("return")
            self._barrier()  # every rank's epilogue stores into Y_h have landed
            self.mark("merge_experts")
            ops.merge_experts(T, d, k, self.Y_h, hm.token_mapping, hm.weights, out)
            self.mark("fwd_end")
            return out
        if p2p:
            ops.ep_dispatch_rows(T, d, k, Xn, None, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum, x.dst_base,
                                 self.peers["zone"], E, self.E_loc, self.cap)
            self._barrier()
        else:
            x.dispatch(hm.zone, self.zone_r)
        self.mark("experts_fwd_gemm")
        ops.moe_experts_fwd(n, d, f, self.E_loc, self.zone_r, W1, W3, W2, f * d, f * d, d * f, x.local_counts,
                            x.local_cumsum, self.x1, self.x3, self.h, self.Y_r)
        self.mark("return")
        if p2p:
            self._barrier()
            ops.ep_combine_rows(T, d, k, hm.weights, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum, x.dst_base,
                                self.peers["Y"], E, self.E_loc, self.cap, out)
        else:
            x.combine(self.Y_r, hm.Y)
            self.mark("merge_experts")
            ops.merge_experts(T, d, k, hm.Y, hm.token_mapping, hm.weights, out)
        self.mark("fwd_end")
        return out

    def backward(self, Xn, Wr, W1, W3, W2, dOut, dXn, dWr, dW1, dW3, dW2):
        from . import ops

        hm, x = self.home, self.x
        T, d, E, k, f = self.T, self.d, self.E, self.k, self.f
        n = self.rows
        fused = self.transport == "fused"
        p2p = fused or self.transport == "p2p"
        if fused:
            self.dP_r[:n].zero_()
            ready = self._sliced_dispatch(dOut, hm.weights, self.peers["dY"], publish_tags=False)
            for (a, b), ev in zip(self.slices, ready):
                self.mark("dispatch_bwd")
                torch.cuda.current_stream().wait_event(ev)
                self.mark("experts_bwd_x_gemm")
                # the gate weight of a row lives on its home rank: accumulate w*<Y,dOut> here, divide there
                ops.moe_experts_bwd_x_scatter(n, d, f, b - a, self.dY_r, self.ones, self.x1, self.x3, W1[a:b], W3[a:b],
                                              W2[a:b], f * d, f * d, d * f, x.local_counts[a:b], x.local_cumsum[a:b],
                                              self.dx1, self.dx3, None, self.dP_r, self.tags_r, self.peers["dZh"],
                                              self.R)
                self.mark("experts_bwd_w_gemm")
                ops.moe_experts_bwd_w(n, d, f, b - a, self.dY_r, self.h, self.zone_r, self.dx1, self.dx3, dW1[a:b],
                                      dW3[a:b], dW2[a:b], f * d, f * d, d * f, x.local_counts[a:b],
                                      x.local_cumsum[a:b])
            self.mark("return_bwd")
            self._barrier()
            self.mark("unpermute")
            ops.unpermute_experts(T, d, k, self.dZ_h, hm.token_mapping, dXn)
            self.mark("router_grad")
            hm.dX_routed.zero_()
            ops.ep_gather_router_grad(T, k, hm.weights, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum, x.dst_base,
                                      self.peers["dP"], E, self.E_loc, self.cap, hm.dX_routed)
            return self._router_backward(Xn, Wr, dXn, dWr)
        if p2p:
            self.mark("dispatch_bwd")
            ops.ep_dispatch_rows(T, d, k, dOut, hm.weights, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum,
                                 x.dst_base, self.peers["dY"], E, self.E_loc, self.cap)
            self._barrier()
        else:
            self.mark("prepare_experts_weighted")
            ops.prepare_experts_weighted(T, d, k, dOut, hm.token_mapping, hm.weights, hm.dYz)
            ops.scatter_row_weights(T, k, hm.token_mapping, hm.weights, hm.row_w)
            self.mark("dispatch_bwd")
            x.dispatch(hm.dYz, self.dY_r)
        self.mark("experts_bwd_x_gemm")
        self.dP_r[:n].zero_()
        # the gate weight of a row lives on its home rank: accumulate w*<Y,dOut> here, divide there
        ops.moe_experts_bwd_x(n, d, f, self.E_loc, self.dY_r, self.ones, self.x1, self.x3, W1, W3, W2, f * d, f * d,
                              d * f, x.local_counts, x.local_cumsum, self.dx1, self.dx3, None, self.dP_r, self.dZ_r)
        self.mark("experts_bwd_w_gemm")
        ops.moe_experts_bwd_w(n, d, f, self.E_loc, self.dY_r, self.h, self.zone_r, self.dx1, self.dx3, dW1, dW3, dW2,
                              f * d, f * d, d * f, x.local_counts, x.local_cumsum)
        self.mark("return_bwd")
        if p2p:
            self._barrier()
            dXn.zero_()
            ops.ep_combine_rows(T, d, k, None, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum, x.dst_base,
                                self.peers["dZ"], E, self.E_loc, self.cap, dXn)
            self.mark("router_grad")
            hm.dX_routed.zero_()
            ops.ep_gather_router_grad(T, k, hm.weights, hm.token_mapping, hm.chosen, hm.counts, hm.cumsum, x.dst_base,
                                      self.peers["dP"], E, self.E_loc, self.cap, hm.dX_routed)
        else:
            x.combine(self.dZ_r, hm.dZ)
            x.combine(self.dP_r, hm.dP)
            self.mark("unpermute")
            hm.dP.div_(hm.row_w)
            dXn.zero_()
            ops.merge_experts(T, d, k, hm.dZ, hm.token_mapping, None, dXn)
            self.mark("router_grad")
            hm.dX_routed.zero_()
            ops.gather_router_grad(T, E, k, hm.token_mapping, hm.chosen, hm.dP, hm.dX_routed)
        return self._router_backward(Xn, Wr, dXn, dWr)

    def _router_backward(self, Xn, Wr, dXn, dWr):
        from . import ops

        hm = self.home
        T, d, E, k = self.T, self.d, self.E, self.k
        ops.router_gate_bwd_x(T, E, k, hm.chosen, hm.weights, hm.dX_routed)
        ops.matmul(0, 0, d, E, T, 1.0, 1.0, Wr, hm.dX_routed, dXn, dXn)
        hm.dWr_local.zero_()
        ops.matmul(0, 1, d, T, E, 1.0, 0.0, Xn, hm.dX_routed, None, hm.dWr_local, hm.mm_ws)
        self.dist.all_reduce(hm.dWr_local)  # the replicated router weight sees every rank's tokens
        dWr.add_(hm.dWr_local)
        self.mark("bwd_end")
        return dXn


class _HomeSide:
    """Token-side state of one rank: routing results, the expert-ordered zone and its backward twins."""

    def __init__(self, T, d, E, k, dev, staging=True):
        from . import ops

        self.T, self.d, self.E, self.k = T, d, E, k
        R = T * k
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32

        def buf(shape, dt):
            return torch.empty(shape, dtype=dt, device=dev)

        self.logits = buf((T, E), f32)
        self.weights = buf((T, k), f32)
        self.chosen = buf((T, k), torch.int16)
        self.counts = torch.zeros(E + 1, dtype=i32, device=dev)
        self.cumsum = torch.zeros(E, dtype=i32, device=dev)
        self.expert_mapping = buf((R,), i32)
        self.token_mapping = buf((T, k), i32)
        self.map_ws = torch.empty(ops.build_expert_mapping_workspace_bytes(T, E, k), dtype=torch.uint8, device=dev)
        self.mm_ws = torch.empty(16 << 20, dtype=torch.uint8, device=dev)  # split-K scratch of the router GEMMs
        if staging:  # local copies of the routed rows, only needed when rows travel through NCCL
            self.zone, self.Y, self.dYz, self.dZ = (buf((R, d), bf) for _ in range(4))
            self.row_w, self.dP = buf((R,), f32), buf((R,), f32)
        self.dX_routed = buf((T, E), bf)
        self.dWr_local = buf((E, d), bf)

    def route(self, Xn, Wr):
        from . import ops

        T, d, E, k = self.T, self.d, self.E, self.k
        ops.matmul(1, 0, E, d, T, 1.0, 0.0, Wr, Xn, None, self.logits, self.mm_ws)
        self.counts.zero_()
        self.cumsum.zero_()
        ops.select_experts(T, E, k, self.logits, self.weights, self.chosen, self.counts, self.cumsum, None)
        ops.build_expert_mapping(T, E, k, self.chosen, self.cumsum, self.expert_mapping, self.token_mapping,
                                 self.map_ws)
