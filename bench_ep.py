"""Benchmark harness of the expert-parallel FFN (bench.py --gpus N under torchrun, or --workload c5 on one GPU).

256 experts split evenly over the ranks, 16384 tokens per rank, top-8 routing: token rows (int8 + fp32 scale) go to the
GPU that owns their expert, grouped_matmul_swiglu_quant (K=7168, N=4096) and the down grouped_matmul (K=2048, N=7168) run
there, result rows come back.  After the timed region every rank checks a sample of the rows it got back against the CPU
oracle (gate/up with SwiGLU and requantisation, then the down GEMM, on the sampled tokens): the rows sampled were sent to
experts of the NEXT rank, so the check covers the dispatch stores, both GEMM kernels and the cross-GPU stores of the
down-GEMM epilogue.  The check sits outside the timed region.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

N_EXPERTS, HIDDEN, INTER, TOP_K = 256, 7168, 2048, 8


def default_chunks(world: int) -> int:
    """Token chunks per step of the NCCL variant: enough rows per local expert and chunk to keep the GEMM tiles full."""
    return {1: 1, 2: 1, 4: 2}.get(world, 4)


def make_rank_data(dev, world, rank, tokens):
    """Seeded synthetic weights of rank ``rank``'s experts and that rank's tokens (DeepSeek-V3 shapes)."""
    from ops_transformer_b200 import synth
    e_local = N_EXPERTS // world
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    d = {}
    d["w1"] = torch.randint(-127, 128, (e_local, HIDDEN, 2 * INTER), dtype=torch.int8, device=dev, generator=g)
    d["w2"] = torch.randint(-127, 128, (e_local, INTER, HIDDEN), dtype=torch.int8, device=dev, generator=g)
    d["w1s"] = torch.empty((e_local, 2 * INTER), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    d["w2s"] = torch.empty((e_local, HIDDEN), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    d["x"] = torch.randint(-127, 128, (tokens, HIDDEN), dtype=torch.int8, device=dev, generator=g)
    d["xs"] = torch.empty((tokens,), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    _, top = synth.topk_softmax_counts(tokens, N_EXPERTS, TOP_K, seed=rank, idx=7)
    d["topk"] = torch.from_numpy(top.astype(np.int64)).to(dev)
    wts = torch.empty((tokens, TOP_K), dtype=torch.float32, device=dev).uniform_(0.05, 1.0, generator=g)
    d["topk_w"] = wts / wts.sum(dim=1, keepdim=True)   # routing weights of the combine (they sum to 1 per token)
    return d


def build_ffn(args, d, tokens, world):
    from ops_transformer_b200 import ep
    if args.ep_impl == "fused":
        chunks = args.ep_chunks if args.ep_chunks > 0 else 1   # measured on 8 GPUs: 1 chunk 7.1 ms, 2 chunks 7.6 ms, 4 chunks 8.7 ms
        parts = getattr(args, "ep_parts", 0)
        if parts <= 0:
            parts = 1   # expert ranges (--ep-parts 2: the second range is dispatched beside the GEMMs of the first); on 2 GPUs, where
                        # half of the rows stay local, the split costs more than the overlap gains (6.81 vs 6.48 ms per step)
        ffn = ep.FusedExpertParallelFFN(N_EXPERTS, HIDDEN, HIDDEN, d["w1"], d["w1s"], d["w2"], d["w2s"], tokens=tokens, top_k=TOP_K,
                                        capacity=2 * tokens * TOP_K, chunks=chunks, expert_parts=parts)
        pieces = max(chunks, parts)
        return ffn, (f"dispatch by peer stores, results stored into the owners' buffers by the down-GEMM epilogue, {chunks} "
                     f"token chunk(s), {parts} expert range(s) per rank with the next piece's dispatch beside the GEMMs"), 3 * pieces
    chunks = args.ep_chunks if args.ep_chunks > 0 else default_chunks(world)
    reserve = args.ep_reserve_sms if args.ep_reserve_sms >= 0 else (16 if world > 1 and chunks > 1 else 0)
    options = None
    if reserve > 0:
        # leave a few SMs to the all-to-all kernels so that they can run beside the persistent GEMM kernels
        from ops_transformer_b200 import LaunchOptions
        n_sm = torch.cuda.get_device_properties(d["x"].device).multi_processor_count
        options = LaunchOptions(max_ctas=max(2, n_sm - reserve))
    ffn = ep.ExpertParallelFFN(N_EXPERTS, d["w1"], d["w1s"], d["w2"], d["w2s"], chunks=chunks, options=options)
    return ffn, f"NCCL all-to-all around the operators, {chunks} chunk(s), {reserve} SMs left to the exchange", 2 * chunks


def _rows_of(res):
    if isinstance(res, dict):
        return sum(int(g[-1].item()) for g in res["group_lists"])
    return sum(r["rows_computed"] for r in res)


def timed_steps(ffn, d, steps, warmup, world, use_graph=False):
    if use_graph and hasattr(ffn, "capture"):
        ffn.capture(d["x"], d["xs"], d["topk"])
        fwd = ffn.replay
    else:
        fwd = ffn.forward
    for _ in range(max(warmup, 3)):
        res = fwd(d["x"], d["xs"], d["topk"])
    torch.cuda.synchronize()
    rows = _rows_of(res)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(steps):
        res = fwd(d["x"], d["xs"], d["topk"])
    ev1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / steps * 1e3
    return ev0.elapsed_time(ev1) / steps, wall, rows, res


def e2e_steps(ffn, d, steps):
    """The same step through the public classes with host buffers, every step: pinned H2D of tokens, scales, routing (and
    routing weights), the FFN, D2H of the result.  The fused layer returns what a caller of the reference's
    dispatch -> FFN -> combine chain gets back, one combined bf16 row per token (the weighted sum of its top-k result
    rows, FusedExpertParallelFFN.combine); the NCCL variant has no combine and returns all result rows."""
    combine = hasattr(ffn, "combine")
    hx = torch.empty_like(d["x"], device="cpu").pin_memory(); hx.copy_(d["x"])
    hs = torch.empty_like(d["xs"], device="cpu").pin_memory(); hs.copy_(d["xs"])
    ht = torch.empty_like(d["topk"], device="cpu").pin_memory(); ht.copy_(d["topk"])
    hw = torch.empty_like(d["topk_w"], device="cpu").pin_memory(); hw.copy_(d["topk_w"])
    dx, ds, dt, dw = torch.empty_like(d["x"]), torch.empty_like(d["xs"]), torch.empty_like(d["topk"]), torch.empty_like(d["topk_w"])
    host_out = None
    last = {}

    def step():
        nonlocal host_out
        dx.copy_(hx, non_blocking=True); ds.copy_(hs, non_blocking=True); dt.copy_(ht, non_blocking=True)
        if combine:
            dw.copy_(hw, non_blocking=True)
        res = ffn.replay(dx, ds, dt) if getattr(ffn, "_graph", None) is not None else ffn.forward(dx, ds, dt)
        if combine:
            ys = [ffn.combine(res, dw)]
        else:
            ys = [res["y"]] if isinstance(res, dict) else [r["y"] for r in res]
        if host_out is None:
            host_out = [torch.empty_like(y, device="cpu").pin_memory() for y in ys]
        for h, y in zip(host_out, ys):
            h.copy_(y, non_blocking=True)
        torch.cuda.synchronize()
        last["res"], last["out"] = res, ys

    step()
    if dist.is_initialized():
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) / steps * 1e3
    h2d = hx.numel() + hs.numel() * 4 + ht.numel() * 8 + (hw.numel() * 4 if combine else 0)
    d2h = sum(h.numel() * h.element_size() for h in host_out)
    checked = verify_combined(ffn, last["res"], d, host_out[0]) if combine else None
    return ms, h2d, d2h, checked


def verify_combined(ffn, res, d, host_combined, n_tokens=64, seed=0):
    """Combined rows of a token sample (as they arrived on the host) against the oracle's combine of the returned rows
    (which verify_returned_rows checks against the oracle FFN): bit for bit."""
    from oracle import oracle as O
    k = ffn.top_k
    pair_row = np.full(ffn.tokens * k, -1, np.int64)
    for c, ch in enumerate(res["chunks"]):
        n = int(ch["rows_in_use"].item())
        order = ch["plan"].order[:n].cpu().numpy()
        pair0 = 0 if ffn.parts > 1 else ffn.bounds[c] * k
        pair_row[pair0 + order] = ffn.result_base[c] + np.arange(n)
    rng = np.random.default_rng(seed + ffn.rank)
    toks = np.unique(np.concatenate([[0, ffn.tokens - 1], rng.integers(0, ffn.tokens, size=n_tokens)]))
    rows = pair_row.reshape(ffn.tokens, k)[toks]                       # [n, k] rows of the result buffer
    flat = torch.from_numpy(np.maximum(rows, 0).reshape(-1)).to(res["y"].device)
    y_sel = res["y"][flat].view(torch.int16).cpu().numpy().view(np.uint16)
    local = np.where(rows >= 0, np.arange(rows.size).reshape(rows.shape), -1)
    want = O.ep_combine(y_sel, local, d["topk_w"][torch.from_numpy(toks).to(res["y"].device)].cpu().numpy())
    got = host_combined[torch.from_numpy(toks)].view(torch.int16).numpy().view(np.uint16)
    return {"tokens": int(toks.size), "mismatches": int((got != want).any(axis=1).sum())}


def verify_returned_rows(res, d, dev, world, rank, tokens, experts_checked=4, rows_per_expert=24, seed=0):
    """Check result rows this rank got back against the CPU oracle.  The rows are those this rank sent to a few experts of
    rank (rank + 1) % world (its own experts when world == 1): the sender holds the token rows, the owner's weights are
    regenerated from their seed, the oracle runs swiglu_quant then the down GEMM on the sampled tokens.  The bar is the
    benchmark's bf16 tolerance (rtol 4e-3 / atol 1e-2): the requantised intermediate may differ from the oracle's by one
    LSB on at most 0.01 % of its elements, which moves a result by far less."""
    from oracle import oracle as O
    from oracle import sampled_check as SC
    O.build()
    O.use_all_cores()
    chunks = res["chunks"] if isinstance(res, dict) else res
    topk_flat = d["topk"].reshape(-1)
    owner = (rank + 1) % world
    e_local = N_EXPERTS // world
    dw = d if owner == rank else make_rank_data(dev, world, owner, tokens)   # the owner's weights, from their seed
    rng = np.random.default_rng(seed + rank)
    local_ids = sorted(set([0, e_local - 1] + [int(v) for v in rng.integers(0, e_local, size=max(experts_checked - 2, 0))]))
    # every piece (token chunk or expert range) holds its own send order and result rows
    pieces = []
    tok_off = 0
    for ch in chunks:
        plan = ch["plan"]
        order = plan.order.to(torch.int64)
        n_use = int(ch["rows_in_use"].item()) if "rows_in_use" in ch else int(order.shape[0])
        if isinstance(res, dict):
            pair, tok = order[:n_use], plan.src_token.to(torch.int64)[:n_use]
        else:   # the NCCL variant numbers pairs and tokens inside its token chunk
            pair, tok = order[:n_use] + tok_off * TOP_K, plan.src_token.to(torch.int64)[:n_use] + tok_off
            tok_off += int(ch.get("tokens", 0))
        pieces.append((topk_flat[pair], tok, ch["y"]))           # global expert of every send row, its token, the results
    sel_x, sel_xs, sel_y, sel_counts = [], [], [], []
    for le in local_ids:
        n_le = 0
        for expert_of_row, tok, y in pieces:
            pos = torch.nonzero(expert_of_row == owner * e_local + le).reshape(-1)
            if pos.numel() == 0:
                continue
            n = int(pos.numel())
            pick = sorted(set([0, n - 1] + [int(v) for v in rng.integers(0, n, size=rows_per_expert)]))
            pos = pos[torch.tensor(pick, device=pos.device)]
            sel_x.append(d["x"][tok[pos]]); sel_xs.append(d["xs"][tok[pos]]); sel_y.append(y[pos])
            n_le += len(pick)
        sel_counts.append(n_le)
    sel_rows = sel_x
    if not sel_rows:
        return {"rows": 0, "mismatches": 0, "note": "no rows for the sampled experts"}
    x_rows = torch.cat(sel_x).cpu().numpy()
    xs_rows = torch.cat(sel_xs).cpu().numpy()
    idx = torch.tensor(local_ids, device=dev)
    w1 = dw["w1"][idx].cpu().numpy(); w1s = dw["w1s"][idx].cpu().numpy()
    w2 = dw["w2"][idx].cpu().numpy(); w2s = dw["w2s"][idx].cpu().numpy()
    gl = np.cumsum(np.asarray(sel_counts, np.int64))
    r1 = O.swiglu_quant(x_rows, w1, w1s, xs_rows, gl)
    got = torch.cat(sel_y).view(torch.int16).cpu().numpy().view(np.uint16)
    out = SC.check_gmm_rows(r1["q"], w2, w2s, r1["q_scale"], np.asarray(sel_counts, np.int64), got)
    out["experts_of_rank"] = owner
    del dw
    return out


def one_gpu_summary(args, dev, verify=True):
    """The expert-parallel workload on one GPU (all 256 experts local): tokens/s, ms per step and TOPS."""
    T = args.ep_tokens
    d1 = make_rank_data(dev, 1, 0, T)
    f1, _, _ = build_ffn(args, d1, T, 1)
    ms1, _, rows1, res = timed_steps(f1, d1, max(3, min(args.steps, 10)), 3, 1)
    out = {"ms_per_step": ms1, "tokens_per_s": T / (ms1 * 1e-3),
           "tops": rows1 * 2.0 * (HIDDEN * 2 * INTER + INTER * HIDDEN) / (ms1 * 1e-3) / 1e12}
    if verify:
        out["verified"] = verify_returned_rows(res, d1, dev, 1, 0, T)
    if hasattr(f1, "close"):
        f1.close()
    del f1, d1, res
    torch.cuda.empty_cache()
    return out


def bench_main(args, ClockSampler, cpu_baseline_sample, measured_peaks, extra_c2=None):
    """``extra_c2``: optional callable returning the C2 one-GPU summary, shown as an extra when this line headlines C5 at N=1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    T = args.ep_tokens
    ops_per_row = 2.0 * (HIDDEN * 2 * INTER + INTER * HIDDEN)

    # The same workload on one GPU (all 256 experts local, no exchange), measured by rank 0 before the group forms:
    # the reference point for the scaling of this line.
    n1 = None
    if world > 1 and rank == 0 and not args.ep_skip_n1:
        n1 = one_gpu_summary(args, dev, verify=False)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    d = make_rank_data(dev, world, rank, T)
    ffn, how, launches_per_step = build_ffn(args, d, T, world)
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        sampler.mark_begin()
    ms, wall, rows_local, res = timed_steps(ffn, d, args.steps, args.warmup, world, use_graph=args.ep_graph and world > 1)
    if sampler:
        sampler.mark_end()
        clocks = sampler.stop()
    # value check of what was just timed (outside the timed region): every rank, rows that crossed to the next rank and back
    verified = {"rows": 0, "mismatches": 0, "note": "skipped (--no-verify)"}
    if not args.no_verify:
        torch.cuda.synchronize()
        verified = verify_returned_rows(res, d, dev, world, rank, T)
    e2e_ms, h2d, d2h, combined_checked = e2e_steps(ffn, d, 3)
    dropped = int(ffn.overflow.item()) if hasattr(ffn, "overflow") else 0
    trace = None
    if args.ep_phases and hasattr(ffn, "trace"):
        for _ in range(2):
            ffn.forward(d["x"], d["xs"], d["topk"])   # eager warm-up (the timed steps may have been graph replays)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ffn.trace = []
        ffn.forward(d["x"], d["xs"], d["topk"])
        torch.cuda.synchronize()
        tr = ffn.trace
        mine = [(b[0], round(a[1].elapsed_time(b[1]), 3)) for a, b in zip(tr[:-1], tr[1:])]
        ffn.trace = None
        if world > 1:
            allt = [None] * world
            dist.all_gather_object(allt, mine)
            trace = [(mine[i][0], min(t_[i][1] for t_ in allt), max(t_[i][1] for t_ in allt)) for i in range(len(mine))]
        else:
            trace = mine
    stats = torch.tensor([ms, float(rows_local), float(dropped), e2e_ms, float(verified["rows"]), float(verified["mismatches"]),
                          float(verified.get("not_bit_identical", 0)), float(combined_checked["tokens"] if combined_checked else 0),
                          float(combined_checked["mismatches"] if combined_checked else 0)], dtype=torch.float64, device=dev)
    if world > 1:
        allst = [torch.empty_like(stats) for _ in range(world)]
        dist.all_gather(allst, stats)
    else:
        allst = [stats]
    ms_max = max(float(s_[0]) for s_ in allst)
    rows_total = sum(float(s_[1]) for s_ in allst)
    dropped = sum(float(s_[2]) for s_ in allst)
    e2e_max = max(float(s_[3]) for s_ in allst)
    if rank == 0:
        tops = rows_total * ops_per_row / (ms_max * 1e-3) / 1e12
        peaks = measured_peaks()
        int8_peak = 2.0 * peaks["bf16_tflops_sustained"]   # a multi-millisecond step runs under the power cap
        line = {
            "metric": "int8 GMM+SwiGLU-quant TOPS", "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"c5 expert-parallel FFN: 256 experts over {world} GPU(s), {T} tokens per GPU, top-8, swiglu_quant "
                                   f"K=7168 N=4096 then down GEMM K=2048 N=7168; {how}",
                       "l2": "inputs larger than L2", "tokens_per_s": T * world / (ms_max * 1e-3), "rows_total": rows_total,
                       "host_ms_per_step": wall, "dropped_rows": dropped, "phase_ms": trace,
                       "cuda_graph": bool(args.ep_graph and args.ep_impl == "fused" and world > 1),
                       "verified": {"rows": int(sum(float(s_[4]) for s_ in allst)), "mismatches": int(sum(float(s_[5]) for s_ in allst)),
                                    "not_bit_identical": int(sum(float(s_[6]) for s_ in allst)), "ranks": world,
                                    "what": "per rank, result rows of tokens sent to experts of the next rank, against the CPU oracle "
                                            "(swiglu_quant then down GEMM), bf16 rtol 4e-3 / atol 1e-2"}},
            "roofline": {"bound": "tensor", "achieved": tops / world, "peak": int8_peak, "unit": "TFLOP/s", "frac": tops / world / int8_peak,
                         "traffic": None, "kernel": "whole step per GPU (dispatch, two GEMM kernels, exchange)",
                         "peak_basis": f"2 x sustained bf16 of {peaks['source']} ({peaks['bf16_tflops_sustained']} TFLOP/s); int8 ops "
                                       "counted as 2 per multiply-add"},
            "e2e": {"value": rows_total * ops_per_row / (e2e_max * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_max,
                    "h2d_bytes_per_step": int(h2d) * world, "d2h_bytes_per_step": int(d2h) * world,
                    "result": ("one combined bf16 row per token (weighted sum of its top-k result rows, on the device after the "
                               "step)" if combined_checked else "all result rows"),
                    "combined_verified": ({"tokens": int(sum(float(s_[7]) for s_ in allst)),
                                           "mismatches": int(sum(float(s_[8]) for s_ in allst)),
                                           "bar": "bit-identical to the oracle's combine of the returned rows"}
                                          if combined_checked else None)},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "ep": {"tokens_per_s": T * world / (ms_max * 1e-3), "one_gpu_same_workload": n1,
                   "scaling_vs_one_gpu": (T * world / (ms_max * 1e-3)) / n1["tokens_per_s"] if n1 else None},
        }
    if hasattr(ffn, "close"):
        ffn.close()
    del ffn, d, res
    torch.cuda.empty_cache()
    if rank == 0:
        if world == 1 and extra_c2 is not None:
            line["extra"] = {"c2": extra_c2()}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sample("c5")
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
