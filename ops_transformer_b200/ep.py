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
    counts = torch.bincount(flat, minlength=n_experts).reshape(world, n_experts // world)
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
                 compute: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_experts = n_experts
        self.e_local = n_experts // self.world
        assert self.e_local * self.world == n_experts
        self.w1, self.w1_scale, self.w2, self.w2_scale = w1, w1_scale, w2, w2_scale
        self.chunks = chunks
        self.compute = compute or self._gpu_compute
        self.timers = None  # set to a dict to collect per-phase wall times (synchronises after every phase)

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
    def _gpu_compute(self, x, xs, group_list):
        from . import acl
        q, qs = acl.grouped_matmul_swiglu_quant(x, self.w1, self.w1_scale, xs, group_list)
        return acl.grouped_matmul_v4(q, self.w2, self.w2_scale, qs, group_list, group_list_type=0)

    def _a2a(self, out, inp, out_splits, in_splits, async_op=False):
        if self.world == 1:
            out.copy_(inp)
            return None
        return dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group, async_op=async_op)

    def forward(self, x: torch.Tensor, x_scale: torch.Tensor, topk_ids: torch.Tensor) -> List[dict]:
        """x int8 [T, H], x_scale fp32 [T], topk_ids [T, k] global expert ids.  Returns one dict per chunk with
        'y' (bf16 [rows, H_out], rows in the order they were sent = sorted by expert) and 'plan' (ChunkPlan)."""
        import time
        G, E, C = self.world, self.e_local, self.chunks
        T = x.shape[0]
        dev = x.device
        t = time.perf_counter()
        bounds = [T * c // C for c in range(C + 1)]
        plans = [dispatch_plan(topk_ids[bounds[c]:bounds[c + 1]], self.n_experts, G) for c in range(C)]
        t = self._tick("plan", t)

        # counts of all chunks in one small exchange; the split sizes are needed on the host
        send_counts = torch.stack([p.send_counts for p in plans], 1).contiguous()      # [G(dst), C, E]
        recv_counts = torch.empty_like(send_counts)                                    # [G(src), C, E]
        self._a2a(recv_counts, send_counts, None, None)
        send_h = send_counts.sum(2).cpu()   # [G, C] rows to each rank
        recv_h = recv_counts.sum(2).cpu()   # [G, C] rows from each rank
        recv_counts_h = recv_counts.cpu()
        t = self._tick("counts_exchange", t)

        use_cuda = dev.type == "cuda"

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
            w1 = self._a2a(rx, sx, out_sp, in_sp, async_op=use_cuda and G > 1)
            w2 = self._a2a(rs, ss, out_sp, in_sp, async_op=use_cuda and G > 1)
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
            dst, group_list = reorder_index(recv_counts[:, c, :], n_rows=int(rx.shape[0]))
            if G > 1:
                xs_sorted = torch.empty_like(rx); xs_sorted.index_copy_(0, dst, rx)
                ss_sorted = torch.empty_like(rs); ss_sorted.index_copy_(0, dst, rs)
            else:
                xs_sorted, ss_sorted = rx, rs   # one source: already expert major
            t = self._tick("reorder_in", t)
            y = self.compute(xs_sorted, ss_sorted, group_list)
            t = self._tick("gemms", t)
            y_back = y.index_select(0, dst) if G > 1 else y
            t = self._tick("reorder_out", t)
            out = torch.empty((sx.shape[0], y.shape[1]), dtype=y.dtype, device=dev)
            w3 = self._a2a(out, y_back, in_sp, out_sp, async_op=use_cuda and G > 1)
            if self.timers is not None and w3 is not None:
                w3.wait()
            t = self._tick("a2a_return", t)
            returns.append(w3)
            results.append({"y": out, "plan": p, "rows_computed": int(rx.shape[0]), "keep": (y_back, sx, ss)})
        for w in returns:
            if w is not None:
                w.wait()
        return results


# ----------------------------------------------------------------------------------------------------------------
# benchmark entry (bench.py --gpus N under torchrun, or N = 1)
# ----------------------------------------------------------------------------------------------------------------

def bench_main(args):
    import json
    import time

    import numpy as np

    from . import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_experts, H, I, top_k, T = 256, 7168, 2048, 8, args.ep_tokens
    e_local = n_experts // world
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    w1 = torch.randint(-127, 128, (e_local, H, 2 * I), dtype=torch.int8, device=dev, generator=g)
    w2 = torch.randint(-127, 128, (e_local, I, H), dtype=torch.int8, device=dev, generator=g)
    w1s = torch.empty((e_local, 2 * I), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    w2s = torch.empty((e_local, H), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    x = torch.randint(-127, 128, (T, H), dtype=torch.int8, device=dev, generator=g)
    xs = torch.empty((T,), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    _, top = synth.topk_softmax_counts(T, n_experts, top_k, seed=rank, idx=7)
    topk = torch.from_numpy(top.astype(np.int64)).to(dev)

    ffn = ExpertParallelFFN(n_experts, w1, w1s, w2, w2s, chunks=args.ep_chunks)
    for _ in range(max(args.warmup, 3)):
        res = ffn.forward(x, xs, topk)
    torch.cuda.synchronize()
    rows_local = sum(r["rows_computed"] for r in res)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(args.steps):
        res = ffn.forward(x, xs, topk)
    ev1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / args.steps * 1e3
    ms = ev0.elapsed_time(ev1) / args.steps
    stats = torch.tensor([ms, float(rows_local)], dtype=torch.float64, device=dev)
    if world > 1:
        allst = [torch.empty_like(stats) for _ in range(world)]
        dist.all_gather(allst, stats)
        ms_max = max(float(s[0]) for s in allst)
        rows_total = sum(float(s[1]) for s in allst)
    else:
        ms_max, rows_total = ms, float(rows_local)
    ops_total = 2.0 * rows_total * (H * 2 * I + I * H)
    phases = None
    if args.ep_phases:
        ffn.timers = {}
        for _ in range(3):
            ffn.forward(x, xs, topk)
        phases = {k: v / 3 for k, v in ffn.timers.items()}
        ffn.timers = None
    if rank == 0:
        tops = ops_total / (ms_max * 1e-3) / 1e12
        line = {
            "metric": "int8 GMM+SwiGLU-quant TOPS", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"c5 expert-parallel FFN: 256 experts over {world} GPU(s), {T} tokens per GPU, top-8, "
                                   f"swiglu_quant K=7168 N=4096 then down GEMM K=2048 N=7168, {args.ep_chunks} chunk(s)",
                       "l2": "inputs larger than L2", "tokens_per_s": T * world / (ms_max * 1e-3),
                       "rows_total": rows_total, "host_ms_per_step": wall, "phase_ms_serialised": phases},
            "gpu_launches": 3 * args.ep_chunks * args.steps,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
