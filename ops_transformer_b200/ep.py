"""Expert-parallel MoE expert FFN over the GPUs of one node: one process per GPU, experts split evenly over the
ranks, token rows exchanged with an all-to-all before and after the two grouped GEMM operators.

Pipeline per step (the roles of the reference's MoeDistributeDispatch / MoeReRouting / GroupedMatmulSwigluQuant /
GroupedMatmul / MoeDistributeCombine sequence, mc2/moe_distribute_dispatch_v2/README.md:167-186 and
moe/moe_re_routing/README.md:12-26):

  1. every (token, slot) pair becomes a row; rows are sorted by destination expert (so by destination rank),
  2. the per-(rank, expert) row counts are exchanged (small all-to-all), rows (int8 + fp32 per-token scale) follow
     with an all-to-all-v and land in local HBM,
  3. received rows are (source rank major, expert minor); they are re-ordered to expert major and the expert
     row counts become the running-total group_list,
  4. grouped_matmul_swiglu_quant (gate/up) then grouped_matmul W8A8 (down) run on the local experts,
  5. results go back through the inverse re-order and an all-to-all-v, arriving in the order the rows were sent.

Tokens are processed in chunks so that the exchange of one chunk overlaps the GEMMs of another.  With a world size
of 1 there is no exchange.  The row bookkeeping is plain tensor code so that it also runs on CPU with the gloo
backend, where the tests drive it with a CPU stand-in for step 4.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


@dataclass
class ChunkPlan:
    order: torch.Tensor         # [rows] position in (token, slot) space of every sent row, sorted by expert
    src_token: torch.Tensor     # [rows] token of every sent row
    send_counts: torch.Tensor   # [world, experts_per_rank] rows this rank sends to (rank, local expert)


def dispatch_plan(topk_ids: torch.Tensor, n_experts: int, world: int) -> ChunkPlan:
    """Sort the (token, slot) pairs of a chunk by destination expert.  Expert e lives on rank e // (n_experts/world)."""
    T, k = topk_ids.shape
    flat = topk_ids.reshape(-1).to(torch.int64)
    order = torch.sort(flat, stable=True).indices
    # histogram by scatter-add: unlike bincount it needs no look at the values on the host, so it can be graph-captured
    counts = torch.zeros(n_experts, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))
    counts = counts.reshape(world, n_experts // world)
    return ChunkPlan(order=order, src_token=order // k, send_counts=counts)


def reorder_index(recv_counts: torch.Tensor, n_rows: Optional[int] = None):
    """recv_counts[src, e] rows arrive source-rank major.  Returns (dst, group_list): dst[i] is the expert-major
    position of received row i (the MoeReRouting offsets, moe/moe_re_routing/README.md:12-26), group_list the
    running totals of rows per local expert."""
    G, E = recv_counts.shape
    flat = recv_counts.reshape(-1)                                   # (src, e) order
    src_off = torch.cumsum(flat, 0) - flat                           # start of each segment as received
    em = recv_counts.t().contiguous().reshape(-1)                    # (e, src) order
    dst_off_em = torch.cumsum(em, 0) - em
    dst_off = dst_off_em.reshape(E, G).t().contiguous().reshape(-1)  # back to (src, e) indexing
    if n_rows is None and flat.device.type == "cpu":
        n_rows = int(flat.sum().item())
    # with n_rows given, repeat_interleave does not have to synchronise with the device to size its result
    seg = torch.repeat_interleave(torch.arange(G * E, device=flat.device), flat, output_size=n_rows)
    i = torch.arange(seg.numel(), device=flat.device)
    dst = dst_off[seg] + (i - src_off[seg])
    group_list = torch.cumsum(recv_counts.sum(0), 0).to(torch.int64)
    return dst, group_list


class ExpertParallelFFN:
    """Holds this rank's expert weights and runs the dispatch -> FFN -> return pipeline."""

    def __init__(self, n_experts: int, w1, w1_scale, w2, w2_scale, *, group=None, chunks: int = 1,
                 compute: Optional[Callable] = None, options=None):
        """``options``: per-call ``LaunchOptions`` for the two GEMM operators, e.g. a CTA cap that leaves a few SMs to the
        all-to-all kernels running beside them."""
        self.group = group
        self.options = options
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_experts = n_experts
        self.e_local = n_experts // self.world
        assert self.e_local * self.world == n_experts
        self.w1, self.w1_scale, self.w2, self.w2_scale = w1, w1_scale, w2, w2_scale
        self.chunks = chunks
        self.compute = compute or self._gpu_compute
        self.timers = None  # set to a dict to collect per-phase wall times (synchronises after every phase)
        self.trace = None   # set to a list to collect (label, CUDA event) marks without synchronising

    def _mark(self, label):
        """Diagnostic trace: with self.trace set to a list, record a CUDA event on the current stream (no sync)."""
        if self.trace is not None and torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace.append((label, ev))

    def _tick(self, name, t0):
        """Diagnostic timing: with timers enabled, wait for the device and add the phase's wall time."""
        if self.timers is None:
            return t0
        import time
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        t1 = time.perf_counter()
        self.timers[name] = self.timers.get(name, 0.0) + (t1 - t0) * 1e3
        return t1

    # -- step 4 on the GPU: the two operators through the C ABI ------------------------------------------------
    def _gpu_compute(self, x, xs, group_list, out_row_index):
        """gate/up GEMM + SwiGLU + requant, then the down GEMM; with ``out_row_index`` the down GEMM scatters its
        result rows (row r -> row out_row_index[r]) so that no separate un-permute pass is needed."""
        from . import acl
        q, qs = acl.grouped_matmul_swiglu_quant(x, self.w1, self.w1_scale, xs, group_list, options=self.options)
        return acl.grouped_matmul_v4(q, self.w2, self.w2_scale, qs, group_list, group_list_type=0, out_row_index=out_row_index,
                                     options=self.options)

    def _a2a(self, out, inp, out_splits, in_splits, async_op=False):
        return dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group, async_op=async_op)

    def forward(self, x: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor) -> List[dict]:
        """x int8 [T, H], x_scale fp32 [T], topk_ids [T, k] global expert ids.  Returns one dict per chunk with
        'y' (bf16 [rows, H_out], rows in the order they were sent = sorted by expert) and 'plan' (ChunkPlan)."""
        import time
        G, E, C = self.world, self.e_local, self.chunks
        T = x.shape[0]
        dev = x.device
        use_cuda = dev.type == "cuda"
        t = time.perf_counter()
        self._mark("start")
        bounds = [T * c // C for c in range(C + 1)]
        plans = [dispatch_plan(topk_ids[bounds[c]:bounds[c + 1]], self.n_experts, G) for c in range(C)]
        t = self._tick("plan", t)

        if G == 1:
            # One rank: nothing to exchange, rows sorted by expert are already expert major.
            results = []
            for c, p in enumerate(plans):
                tok = p.src_token + bounds[c]
                sx = x.index_select(0, tok)
                ss = x_scale.index_select(0, tok)
                t = self._tick("gather_send", t)
                group_list = torch.cumsum(p.send_counts.reshape(-1), 0).to(torch.int64)
                y = self.compute(sx, ss, group_list, None)
                t = self._tick("gemms", t)
                results.append({"y": y, "plan": p, "rows_computed": int(sx.shape[0]), "tokens": bounds[c + 1] - bounds[c]})
            return results

        # counts of all chunks in one small exchange; the split sizes are needed on the host
        send_counts = torch.stack([p.send_counts for p in plans], 1).contiguous()      # [G(dst), C, E]
        recv_counts = torch.empty_like(send_counts)                                    # [G(src), C, E]
        self._a2a(recv_counts, send_counts, None, None)
        send_h = send_counts.sum(2).cpu()   # [G, C] rows to each rank
        recv_h = recv_counts.sum(2).cpu()   # [G, C] rows from each rank
        t = self._tick("counts_exchange", t)
        self._mark("counts_done")

        # dispatch of every chunk is issued up front; compute of chunk c starts when its rows have landed
        inflight = []
        for c, p in enumerate(plans):
            tok = p.src_token + bounds[c]
            sx = x.index_select(0, tok)
            ss = x_scale.index_select(0, tok)
            t = self._tick("gather_send", t)
            n_recv = int(recv_h[:, c].sum())
            rx = torch.empty((n_recv, x.shape[1]), dtype=x.dtype, device=dev)
            rs = torch.empty((n_recv,), dtype=x_scale.dtype, device=dev)
            in_sp, out_sp = send_h[:, c].tolist(), recv_h[:, c].tolist()
            w1 = self._a2a(rx, sx, out_sp, in_sp, async_op=use_cuda)
            w2 = self._a2a(rs, ss, out_sp, in_sp, async_op=use_cuda)
            inflight.append((rx, rs, w1, w2, sx, ss, in_sp, out_sp))
            if self.timers is not None:
                for w in (w1, w2):
                    if w is not None:
                        w.wait()
            t = self._tick("a2a_dispatch", t)

        results = []
        returns = []
        for c, p in enumerate(plans):
            rx, rs, w1, w2, sx, ss, in_sp, out_sp = inflight[c]
            for w in (w1, w2):
                if w is not None:
                    w.wait()
            self._mark(f"c{c}_dispatch_landed")
            n_rows = int(rx.shape[0])
            dst, group_list = reorder_index(recv_counts[:, c, :], n_rows=n_rows)
            # inverse permutation: expert-major position -> position as received (source-rank major)
            inv = torch.empty_like(dst)
            inv[dst] = torch.arange(n_rows, device=dev)
            xs_sorted = rx.index_select(0, inv)
            ss_sorted = rs.index_select(0, inv)
            t = self._tick("reorder_in", t)
            self._mark(f"c{c}_reordered")
            # the down projection writes result row r straight to row inv[r], i.e. back in source-rank-major order
            y_back = self.compute(xs_sorted, ss_sorted, group_list, inv)
            t = self._tick("gemms", t)
            self._mark(f"c{c}_gemms_done")
            out = torch.empty((sx.shape[0], y_back.shape[1]), dtype=y_back.dtype, device=dev)
            w3 = self._a2a(out, y_back, in_sp, out_sp, async_op=use_cuda)
            if self.timers is not None and w3 is not None:
                w3.wait()
            t = self._tick("a2a_return", t)
            returns.append(w3)
            results.append({"y": out, "plan": p, "rows_computed": n_rows, "tokens": bounds[c + 1] - bounds[c],
                            "keep": (y_back, sx, ss, xs_sorted, ss_sorted)})
        for c, w in enumerate(returns):
            if w is not None:
                w.wait()
            self._mark(f"c{c}_return_landed")
        return results


ROW_BITS = 40  # a destination is (gpu << ROW_BITS) | row


def _count_tables(all_counts: torch.Tensor):
    G, _, E = all_counts.shape
    c = all_counts.to(torch.int64)
    tot = c.sum(0)                                                    # [dst, e] rows of expert e on dst
    expert_off = torch.cumsum(tot, 1) - tot                           # [dst, e] start of expert e in dst's buffer
    src_off = torch.cumsum(c, 0) - c                                  # [src, dst, e] rows of lower ranks inside the expert
    send_flat = c.reshape(G, G * E)
    send_start = (torch.cumsum(send_flat, 1) - send_flat).reshape(G, G, E)   # [src, dst, e] start in src's send order
    return c, tot, expert_off, src_off, send_start


def fused_send_map(all_counts: torch.Tensor, rank: int, n_send: int):
    """send_dest[i]: where send row i of this rank (rows sorted by global expert) lands, (dst << 40) | row in dst's
    expert-major activation buffer (MoeReRouting's DstOffset, moe/moe_re_routing/README.md:12-26).  all_counts[src, dst, e]
    = rows that rank src sends to local expert e of rank dst.  Nothing is read on the host."""
    G, _, E = all_counts.shape
    dev = all_counts.device
    c, tot, expert_off, src_off, _ = _count_tables(all_counts)
    seg_len = c[rank].reshape(-1)                                     # my send order is made of (dst, e) segments
    seg_end = torch.cumsum(seg_len, 0)
    i = torch.arange(n_send, device=dev)
    seg = torch.searchsorted(seg_end, i, right=True).clamp_(max=G * E - 1)
    within = i - (seg_end[seg] - seg_len[seg])
    base = (expert_off + src_off[rank]).reshape(-1)                   # [(dst, e)]
    send_dest = ((seg // E) << ROW_BITS) | (base[seg] + within)
    return torch.where(i < seg_end[-1], send_dest, torch.full_like(send_dest, -1))


def fused_return_map(all_counts: torch.Tensor, rank: int, capacity: int):
    """(ret_dest [capacity], group_list [E], n_recv [1]) of this rank as a receiver: ret_dest[p] = (src << 40) | row says
    where the result of activation row p goes back - the position the row had in src's send order (-1 beyond n_recv);
    group_list = running totals of rows per local expert."""
    G, _, E = all_counts.shape
    dev = all_counts.device
    c, tot, _, _, send_start = _count_tables(all_counts)
    rlen = c[:, rank, :].t().reshape(-1)                              # my activation buffer is ordered (e, src)
    rend = torch.cumsum(rlen, 0)
    p = torch.arange(capacity, device=dev)
    rseg = torch.searchsorted(rend, p, right=True).clamp_(max=G * E - 1)
    rwithin = p - (rend[rseg] - rlen[rseg])
    back = send_start[:, rank, :].t().reshape(-1)                     # [(e, src)] start of that segment in src's send order
    ret_dest = ((rseg % G) << ROW_BITS) | (back[rseg] + rwithin)
    ret_dest = torch.where(p < rend[-1], ret_dest, torch.full_like(ret_dest, -1))
    return ret_dest, torch.cumsum(tot[rank], 0), rend[-1:].clone()


def fused_maps(all_counts: torch.Tensor, rank: int, n_send: int, capacity: int):
    """Both row maps of the peer-memory pipeline: (send_dest, ret_dest, group_list, n_recv)."""
    return (fused_send_map(all_counts, rank, n_send),) + fused_return_map(all_counts, rank, capacity)


class FusedExpertParallelFFN:
    """Expert-parallel FFN over peer memory: no collective moves token rows.

      1. rows sorted by expert (as in ExpertParallelFFN); the per-(rank, expert) counts are all-gathered (a few KB),
      2. one dispatch kernel stores every row straight into its place in the owning GPU's expert-major buffer
         (gather + exchange + re-order in one pass of NVLink stores),
      3. a barrier orders the GPUs, then grouped_matmul_swiglu_quant and grouped_matmul run on the local experts; the
         down projection's epilogue stores each result row into the buffer of the GPU that sent the token,
      4. a second barrier; every rank then finds its results, in send order, in its own result buffer.

    Two ways to overlap the exchange with the GEMMs, both as "pieces" whose dispatch runs on a second stream beside the
    GEMMs of the piece before: ``chunks`` splits the tokens (rows per expert shrink with it, which costs tile efficiency),
    ``expert_parts`` splits every rank's experts into ranges (groups keep their length: piece p holds the pairs routed to
    the p-th range of local experts of every rank, its rows are dispatched while the GEMMs of range p-1 run).

    Nothing is read back to the host during a step.  Buffers are sized for `capacity` received rows per rank; rows
    beyond it are dropped and counted, so capacity must cover the worst expected imbalance.  The reference's dispatch is
    dropless in this mode, so a caller must read the counter: every result dict carries it as ``dropped_rows`` (an int32
    device tensor, cumulative since construction; anything but 0 means results are missing).
    """

    def __init__(self, n_experts: int, hidden: int, hidden_out: int, w1, w1_scale, w2, w2_scale, *, tokens: int, top_k: int,
                 capacity: int, group=None, chunks: int = 1, expert_parts: int = 1, reserve_sms: int = 0):
        """capacity: rows this rank can receive per step (all pieces together).  chunks > 1 splits the tokens,
        expert_parts > 1 the local experts of every rank (not both); the dispatch of piece c+1 then runs on a second
        stream beside the GEMMs of piece c.  reserve_sms > 0: with expert_parts, the SMs that dispatch is confined to, the
        gate/up GEMM running beside it being capped to the others.  Measured: neither form of the overlap pays on this
        hardware (8 GPUs: 9.1 ms per step with two expert ranges against 6.75 ms with one; 2 GPUs: 6.8 ms, with 16 reserved
        SMs 9.4 ms, against 6.5 ms) - the dispatch kernel and the persistent GEMM queue for the same SMs, and a dispatch
        confined to a few SMs cannot keep NVLink busy - so one piece is the default."""
        import ctypes as C

        from .peer import PeerBuffer
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_experts, self.e_local = n_experts, n_experts // self.world
        self.hidden, self.hidden_out = hidden, hidden_out
        self.w1, self.w1_scale, self.w2, self.w2_scale = w1, w1_scale, w2, w2_scale
        self.tokens, self.top_k = tokens, top_k
        self.reserve_sms = reserve_sms
        self.parts = expert_parts
        if expert_parts > 1:
            if chunks != 1 or self.e_local % expert_parts:
                raise ValueError("expert_parts needs chunks == 1 and a number of local experts it divides")
            chunks = expert_parts                               # one piece per expert range
        self.chunks = chunks
        self.n_send = tokens * top_k
        if self.parts > 1:
            # every piece sees all tokens; its pairs are those routed to its expert range, at most all of them
            self.bounds = [0] * (chunks + 1)
            self.e_piece = self.e_local // self.parts           # local experts per piece
            self.piece_pairs = [self.n_send] * chunks
            self.token_base = [0] * chunks
            self.result_base = [c * self.n_send for c in range(chunks)]
            result_rows = chunks * self.n_send
        else:
            self.bounds = [tokens * c // chunks for c in range(chunks + 1)]
            self.e_piece = self.e_local
            self.piece_pairs = [(self.bounds[c + 1] - self.bounds[c]) * top_k for c in range(chunks)]
            self.token_base = self.bounds[:-1]
            self.result_base = [self.bounds[c] * top_k for c in range(chunks)]
            result_rows = self.n_send
        self.result_rows = result_rows
        self.capacity = capacity
        self.cap_c = (capacity + chunks - 1) // chunks          # rows per piece buffer
        self.buf_x = PeerBuffer(chunks * self.cap_c * hidden, group)
        self.buf_s = PeerBuffer(chunks * self.cap_c * 4, group)
        self.buf_y = PeerBuffer(result_rows * hidden_out * 2, group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.act = self.buf_x.view(torch.int8, (chunks, self.cap_c, hidden))
        self.act_scale = self.buf_s.view(torch.float32, (chunks, self.cap_c))
        self.result = self.buf_y.view(torch.bfloat16, (result_rows, hidden_out))
        # per chunk: every rank's activation / scale buffer of that chunk
        self._x_ptrs = [(C.c_void_p * self.world)(*[C.c_void_p(p + c * self.cap_c * hidden) for p in self.buf_x.ptrs])
                        for c in range(chunks)]
        self._s_ptrs = [(C.c_void_p * self.world)(*[C.c_void_p(p + c * self.cap_c * 4) for p in self.buf_s.ptrs])
                        for c in range(chunks)]
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        # routing state written by the library's count / route kernels (two launches per chunk instead of a sort and
        # some sixty small tensor kernels); route_kernels=False keeps the tensor formulation used by the CPU tests
        self.route_kernels = True
        i64 = dict(dtype=torch.int64, device=dev)
        self._r = []
        for c in range(chunks):
            n_c = self.piece_pairs[c]
            self._r.append(dict(n=n_c, hist=torch.empty(((n_c + 1023) // 1024, self.world * self.e_piece), dtype=torch.int32, device=dev),
                                src_token=torch.zeros(n_c, **i64), order=torch.zeros(n_c, **i64), send_dest=torch.empty(n_c, **i64),
                                ret_dest=torch.empty(self.cap_c, **i64), group_list=torch.empty(self.e_piece, **i64),
                                first_row=torch.empty(1, **i64)))
        self._totals = torch.empty((chunks, self.world, self.e_piece), **i64)
        # for the combine (forward(..., topk_weights=...)): the row of every (token, slot) pair in the result buffer, the
        # combined tokens, and a counter of send positions that named no pair
        self._pair_row = torch.empty(self.n_send, dtype=torch.int32, device=dev)
        self.combined = None
        self.bad_pairs = torch.zeros(1, dtype=torch.int32, device=dev)
        self._side = torch.cuda.Stream() if chunks > 1 else None
        self._graph = None
        self.trace = None   # set to a list to collect (label, CUDA event) marks without synchronising

    def _mark(self, label):
        if self.trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace.append((label, ev))

    def _barrier(self):
        """Stream-ordered barrier across the ranks: completes on the current stream only after every rank's earlier
        work on the stream it called this from (the kernels that store into peer memory) has finished."""
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def _dispatch(self, c, x, x_scale, plan, send_dest, first_row, max_blocks=0):
        import ctypes as C

        from . import _lib, acl
        p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        n = int(plan.src_token.shape[0])
        rc = _lib.lib().gmmB200EpDispatch(p(x), p(x_scale), p(plan.src_token), p(send_dest), n, self.hidden, self.cap_c,
                                          self._x_ptrs[c], self._s_ptrs[c], self.world, p(self.overflow), p(first_row),
                                          max_blocks, stream)
        if rc != 0:
            raise acl.AclnnError(rc, "gmmB200EpDispatch")

    def forward(self, x: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor, topk_weights: Optional[torch.Tensor] = None):
        """topk_weights (fp32 [tokens, top_k], optional): also combine every token's result rows into one row,
        result["combined"] = bf16(sum_s weights[t, s] * y[row of (t, s)]) - the last step of the reference's
        MoeDistributeCombineV2 (mc2/moe_distribute_combine_v2/README.md:12-17).  Dropped rows are left out of the sum."""
        from . import acl
        G, E, C_ = self.world, self.e_local, self.chunks
        k = self.top_k
        self._mark("start")
        if self.route_kernels:
            return self._forward_kernels(x, x_scale, topk_ids, topk_weights)
        if topk_weights is not None:
            raise ValueError("the combine needs the routing kernels (route_kernels = True)")
        if self.parts > 1:
            raise ValueError("expert_parts needs the routing kernels (route_kernels = True)")
        # routing plans and row maps of all chunks first (small kernels), one count exchange for all chunks
        plans = [dispatch_plan(topk_ids[self.bounds[c]:self.bounds[c + 1]], self.n_experts, G) for c in range(C_)]
        self._mark("plan")
        mine = torch.stack([pl.send_counts for pl in plans]).contiguous()                 # [C, G(dst), E]
        if G > 1:
            allc = torch.empty((G,) + tuple(mine.shape), dtype=mine.dtype, device=x.device)  # [G(src), C, G(dst), E]
            dist.all_gather_into_tensor(allc, mine, group=self.group)
        else:
            allc = mine.reshape(1, C_, 1, E)
        self._mark("counts_gathered")
        send_dest, first_row, tok = [], [], []
        for c, pl in enumerate(plans):
            n_c = (self.bounds[c + 1] - self.bounds[c]) * k
            send_dest.append(fused_send_map(allc[:, c], self.rank, n_c))
            # start with the rows of the next rank (then wrap around), so that the ranks fan out over different destinations
            per_dst = pl.send_counts.sum(1)
            first_row.append((torch.cumsum(per_dst, 0) - per_dst)[(self.rank + 1) % G].reshape(1).to(torch.int64).contiguous())
            pl.src_token = pl.src_token + self.bounds[c]
        self._mark("send_map")

        self._dispatch(0, x, x_scale, plans[0], send_dest[0], first_row[0])
        self._mark("dispatch_kernel")
        main = torch.cuda.current_stream()
        landed = [None] * C_
        group_lists = []
        for c in range(C_):
            ret_dest, group_list, _ = fused_return_map(allc[:, c], self.rank, self.cap_c)   # while rows are still arriving
            ret_dest = torch.where(ret_dest >= 0, ret_dest + self.bounds[c] * k, ret_dest)  # rows of chunk c in the result buffer
            if c == 0:
                self._mark("return_map")
                self._barrier()   # all rows of chunk 0 for my experts have landed
                self._mark("barrier1")
            else:
                main.wait_event(landed[c])
            if c + 1 < C_:
                # the next chunk's dispatch (and the barrier after it) runs beside this chunk's GEMMs
                self._side.wait_stream(main)
                with torch.cuda.stream(self._side):
                    self._dispatch(c + 1, x, x_scale, plans[c + 1], send_dest[c + 1], first_row[c + 1])
                    self._barrier()
                    landed[c + 1] = torch.cuda.Event()
                    landed[c + 1].record()
            q, qs = acl.grouped_matmul_swiglu_quant(self.act[c], self.w1, self.w1_scale, self.act_scale[c], group_list)
            self._mark(f"swiglu_quant{c}")
            acl.grouped_matmul_v4(q, self.w2, self.w2_scale, qs, group_list, group_list_type=0, out_row_index=ret_dest,
                                  out_peers=self.buf_y.ptrs, out=None, out_rows=self.result_rows)
            self._mark(f"down_gemm{c}")
            group_lists.append(group_list)
        self._barrier()   # every rank's results have landed, and everyone is done reading its activation buffers
        self._mark("barrier2")
        chunk_out = [{"y": self.result[self.bounds[c] * k:self.bounds[c + 1] * k], "plan": plans[c]} for c in range(C_)]
        return {"y": self.result, "plan": plans[0], "group_list": group_lists[0], "group_lists": group_lists, "chunks": chunk_out,
                "dropped_rows": self.overflow}

    def combine(self, res: dict, topk_weights: torch.Tensor) -> torch.Tensor:
        """The combine on the result of a forward() or replay(): the row of every pair from the send orders of all pieces,
        then one weighted sum per token (bf16 [tokens, hidden_out]).  forward(..., topk_weights=...) calls it itself."""
        plans = [ch["plan"] for ch in res["chunks"]]
        import ctypes as C

        from . import _lib, acl
        L = _lib.lib()
        p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        w = topk_weights.to(torch.float32).contiguous()
        if tuple(w.shape) != (self.tokens, self.top_k):
            raise ValueError(f"topk_weights must be [{self.tokens}, {self.top_k}]")
        if self.combined is None:
            self.combined = torch.empty((self.tokens, self.hidden_out), dtype=torch.bfloat16, device=w.device)
        self._pair_row.fill_(-1)
        in_use = []
        for c in range(self.chunks):
            # expert ranges number their pairs over all tokens; token chunks inside the chunk
            pair0 = 0 if self.parts > 1 else self.bounds[c] * self.top_k
            n_pairs = self.n_send if self.parts > 1 else self.piece_pairs[c]
            rows = self._totals[c].sum().reshape(1)
            in_use.append(rows)
            rc = L.gmmB200EpInverseMap(p(plans[c].order), p(rows), self.piece_pairs[c], self.result_base[c], n_pairs,
                                       C.c_void_p(self._pair_row.data_ptr() + 4 * pair0), p(self.bad_pairs), st)
            if rc != 0:
                raise acl.AclnnError(rc, "gmmB200EpInverseMap")
        rc = L.gmmB200EpCombine(p(self.result), p(self._pair_row), p(w), p(self.combined), self.tokens, self.top_k, self.hidden_out,
                                self.result_rows, st)
        if rc != 0:
            raise acl.AclnnError(rc, "gmmB200EpCombine")
        return self.combined

    def _forward_kernels(self, x, x_scale, topk_ids, topk_weights=None):
        """forward() with the routing done by gmmB200EpCount / gmmB200EpRoute."""
        import ctypes as C

        from . import _lib, acl
        L = _lib.lib()
        G, E, C_, k = self.world, self.e_local, self.chunks, self.top_k
        p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)  # noqa: E731
        topk_ids = topk_ids.contiguous()
        Ep = self.e_piece
        if self.parts > 1:
            # piece c = the pairs routed to local experts [c*Ep, (c+1)*Ep) of any rank, renumbered rank*Ep + (local - c*Ep);
            # the other pairs read as -1, which the count and route kernels skip
            flat = topk_ids.reshape(-1)
            owner, local = flat // E, flat % E
            piece_of = local // Ep
            renum = owner * Ep + (local - piece_of * Ep)
            tk = [torch.where(piece_of == c, renum, torch.full_like(renum, -1)) for c in range(C_)]
        else:
            tk = [topk_ids[self.bounds[c]:self.bounds[c + 1]] for c in range(C_)]
        for c in range(C_):
            rc = L.gmmB200EpCount(p(tk[c]), self._r[c]["n"], G * Ep, p(self._r[c]["hist"]), p(self._totals[c]), st())
            if rc != 0:
                raise acl.AclnnError(rc, "gmmB200EpCount")
        self._mark("plan")
        if G > 1:
            allc = torch.empty((G, C_, G, Ep), dtype=torch.int64, device=x.device)
            dist.all_gather_into_tensor(allc, self._totals, group=self.group)
        else:
            allc = self._totals.reshape(1, C_, 1, Ep)
        self._mark("counts_gathered")
        plans = []
        for c in range(C_):
            r = self._r[c]
            ac = allc[:, c].contiguous()
            if self.parts > 1:
                r["send_dest"].fill_(-1)   # positions beyond the piece's pairs must read as "no row"
            rc = L.gmmB200EpRoute(p(tk[c]), p(r["hist"]), p(ac), r["n"], k, G, Ep, self.rank, self.cap_c, self.token_base[c],
                                  self.result_base[c], p(r["src_token"]), p(r["order"]), p(r["send_dest"]), p(r["ret_dest"]),
                                  p(r["group_list"]), p(r["first_row"]), st())
            if rc != 0:
                raise acl.AclnnError(rc, "gmmB200EpRoute")
            plans.append(ChunkPlan(order=r["order"], src_token=r["src_token"], send_counts=self._totals[c]))
        self._mark("send_map")
        self._dispatch(0, x, x_scale, plans[0], self._r[0]["send_dest"], self._r[0]["first_row"])
        self._mark("dispatch_kernel")
        main = torch.cuda.current_stream()
        landed = [None] * C_
        for c in range(C_):
            r = self._r[c]
            if c == 0:
                self._barrier()   # all rows of chunk 0 for my experts have landed
                self._mark("barrier1")
            else:
                main.wait_event(landed[c])
            beside = None
            if c + 1 < C_:
                cap = self.parts > 1 and self.reserve_sms > 0
                self._side.wait_stream(main)
                with torch.cuda.stream(self._side):
                    self._dispatch(c + 1, x, x_scale, plans[c + 1], self._r[c + 1]["send_dest"], self._r[c + 1]["first_row"],
                                   max_blocks=8 * self.reserve_sms if cap else 0)
                    self._barrier()
                    landed[c + 1] = torch.cuda.Event()
                    landed[c + 1].record()
                if cap:
                    n_sm = torch.cuda.get_device_properties(x.device).multi_processor_count
                    beside = acl.LaunchOptions(max_ctas=max(2, n_sm - self.reserve_sms))
            e0, e1 = (c * Ep, (c + 1) * Ep) if self.parts > 1 else (0, E)
            q, qs = acl.grouped_matmul_swiglu_quant(self.act[c], self.w1[e0:e1], self.w1_scale[e0:e1], self.act_scale[c], r["group_list"],
                                                    options=beside)
            self._mark(f"swiglu_quant{c}")
            acl.grouped_matmul_v4(q, self.w2[e0:e1], self.w2_scale[e0:e1], qs, r["group_list"], group_list_type=0,
                                  out_row_index=r["ret_dest"], out_peers=self.buf_y.ptrs, out=None, out_rows=self.result_rows)
            self._mark(f"down_gemm{c}")
        self._barrier()   # every rank's results have landed, and everyone is done reading its activation buffers
        self._mark("barrier2")
        group_lists = [self._r[c]["group_list"] for c in range(C_)]
        # per piece: its result rows (in its send order), the plan, and how many of the rows are in use (a device scalar;
        # with expert_parts a piece holds only the pairs routed to its expert range)
        chunk_out = [{"y": self.result[self.result_base[c]:self.result_base[c] + self.piece_pairs[c]], "plan": plans[c],
                      "rows_in_use": self._totals[c].sum()} for c in range(C_)]
        out = {"y": self.result, "plan": plans[0], "group_list": group_lists[0], "group_lists": group_lists, "chunks": chunk_out,
               "dropped_rows": self.overflow}
        if topk_weights is not None:
            out["combined"] = self.combine(out, topk_weights)
            out["bad_pairs"] = self.bad_pairs
            self._mark("combine")
        return out

    def capture(self, x: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor, topk_weights: Optional[torch.Tensor] = None):
        """Record one step into a CUDA graph.  Shapes are static (buffers are sized by capacity and nothing is read on
        the host), so the whole step - routing plan, count exchange, row maps, dispatch, both GEMMs, barriers - replays
        with one launch and no Python in between.  Inputs are copied into fixed tensors before every replay."""
        self._gx, self._gs, self._gt = torch.empty_like(x), torch.empty_like(x_scale), torch.empty_like(topk_ids)
        self._gx.copy_(x); self._gs.copy_(x_scale); self._gt.copy_(topk_ids)
        self._gw = None
        if topk_weights is not None:
            self._gw = topk_weights.to(torch.float32).contiguous().clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):   # warm-up outside capture: lazy initialisation of kernels, NCCL and the workspace pool
                self.forward(self._gx, self._gs, self._gt, self._gw)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._graph_out = self.forward(self._gx, self._gs, self._gt, self._gw)
        return self

    def replay(self, x: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor, topk_weights: Optional[torch.Tensor] = None):
        self._gx.copy_(x, non_blocking=True); self._gs.copy_(x_scale, non_blocking=True); self._gt.copy_(topk_ids, non_blocking=True)
        if self._gw is not None and topk_weights is not None:
            self._gw.copy_(topk_weights, non_blocking=True)
        self._graph.replay()
        return self._graph_out

    def close(self):
        self._graph = None
        for b in (self.buf_x, self.buf_s, self.buf_y):
            b.close()
