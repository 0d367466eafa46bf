#!/usr/bin/env python
"""Benchmark of the grouped int8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input (seeded, DeepSeek-V3 shaped; no
dataset or checkpoint is involved).  At N=1 the default workload is the DeepSeek-V3 prefill gate/up projection
through grouped_matmul_swiglu_quant: 4096 tokens x top-8 over 32 local experts = 32768 rows, K=7168, N=4096.
At N>1 (launched under torchrun, one rank per GPU) the workload is the expert-parallel FFN: 256 experts split
over the ranks, 16384 tokens per rank, rows exchanged over NVLink, swiglu_quant then the down GEMM, results
returned (bench_ep.py).  Launched under torchrun with a world size of 1 the same expert-parallel workload is the
headline (all 256 experts on the one GPU), so that a scaling series started that way compares like with like; the
prefill workload is then an extra of the line.  Rank 0 prints one JSON line.

Every timed workload is value-checked after its timed region against the CPU oracle on a sample of rows
(`config.verified`, `extra.*.verified`); the check is outside the timed region.

`--impl reference` times the reference's CPU golden path instead: the CPU restatement of the reference kernels
(oracle/) with all host threads, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


# DRAM traffic per launch of the GEMM kernel: CONSTANTS copied from the committed ncu captures, not measured by this script.
# The full-size launches are too large to capture, so the reduced cases are scaled by the units processed (rows, or non-empty
# experts for the weight-streaming decode case); traffic grows in proportion to them.  name -> (bytes, source file).
NCU_DRAM_BYTES_PER_LAUNCH = {
    "c2_small": (454.0e6, "profiles/ncu_gmm_kernel_c2_small_swiglu_quant.md"),
    "c2": (4 * 454.0e6, "profiles/ncu_gmm_kernel_c2_small_swiglu_quant.md, x4 by rows"),
    "c3_small": (217.8e6, "profiles/ncu_gmm_kernel_c3_small_w8a8_bf16.md"),
    "c3": (4 * 217.8e6, "profiles/ncu_gmm_kernel_c3_small_w8a8_bf16.md, x4 by rows"),
    "c4_swiglu_small": (859.8e6, "profiles/ncu_gmm_kernel_c4_small_decode_swiglu_quant.md"),
    "c4_swiglu": (859.8e6 * 165 / 29, "profiles/ncu_gmm_kernel_c4_small_decode_swiglu_quant.md, x165/29 by non-empty experts"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.t0 = self.t1 = None
        self.stamps = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"], samples=0)
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [l for (t, l) in self.lines if self.t0 is not None and self.t0 - 0.05 <= t <= (self.t1 or t) + 0.25]
        if not rows:
            rows = [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            f = [c.strip() for c in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ------------------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------------------

def gen_device_inputs(torch, dev, M, K, N, E, seed):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
    w = torch.randint(-127, 128, (E, K, N), dtype=torch.int8, device=dev, generator=g)
    ws = torch.empty((E, N), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    xs = torch.empty((M,), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    return x, w, ws, xs


def cpu_sample_swiglu(counts, K, N, rows_per_expert, seed):
    """Bounded CPU sample of the swiglu workload: the first `rows_per_expert` rows of every expert."""
    from ops_transformer_b200 import synth
    c = np.minimum(np.asarray(counts), rows_per_expert)
    M = int(c.sum())
    E = len(c)
    x = synth.int8_tensor((M, K), seed, 1)
    w = synth.int8_tensor((E, K, N), seed, 2)
    ws = synth.scale_tensor((E, N), seed, 3)
    xs = synth.scale_tensor((M,), seed, 4)
    return x, w, ws, xs, np.cumsum(c)


C5_WORKLOAD = ("c5 expert-parallel FFN: 256 experts, 16384 tokens per GPU, top-8, swiglu_quant K=7168 N=4096 then down GEMM "
               "K=2048 N=7168")


def launched_by_torchrun() -> bool:
    return "TORCHELASTIC_RUN_ID" in os.environ or ("LOCAL_RANK" in os.environ and "WORLD_SIZE" in os.environ)


def headline_is_c5(args) -> bool:
    """The expert-parallel workload is the headline at N>1, under torchrun at any world size, and when asked for by name."""
    return args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1 or launched_by_torchrun() or args.workload == "c5"


def c5_cpu_sample(rows_per_expert=64):
    """32 of c5's 256 experts with `rows_per_expert` rows each, both operators at full K and N."""
    from ops_transformer_b200 import synth
    cfg = synth.CONFIGS["c2"]
    counts = synth.config_counts("c2", 0)
    K, N = cfg["K"], cfg["N"]
    x, w, ws, xs, gl = cpu_sample_swiglu(counts, K, N, rows_per_expert, 0)
    w2 = synth.int8_tensor((len(counts), N // 2, K), 0, 5)
    ws2 = synth.scale_tensor((len(counts), K), 0, 6)
    M = x.shape[0]
    ops = 2.0 * M * K * N + 2.0 * M * (N // 2) * K
    sample = f"32 of the 256 experts, first {rows_per_expert} rows of each ({M} rows), both operators at full K and N"
    return (x, w, ws, xs, gl, w2, ws2), ops, sample


def run_reference_arm(args):
    """The reference's CPU golden path (CPU restatement of its kernels) on a bounded sample of this arm's workload: the
    gate/up operator of c2 at N=1; where the GPU arm headlines c5, the expert FFN of c5 (gate/up with SwiGLU and
    requantisation, then the down GEMM on its int8 result), as the GPU arm runs it."""
    from oracle import oracle as O
    from ops_transformer_b200 import synth
    O.build()
    O.use_all_cores()
    multi = headline_is_c5(args)
    rows_per_expert = 64
    if multi:
        (x, w, ws, xs, gl, w2, ws2), ops_per_step, sample = c5_cpu_sample(rows_per_expert)
        sample += ", per step"
        workload = C5_WORKLOAD
    else:
        cfg = synth.CONFIGS["c2"]
        counts = synth.config_counts("c2", 0)
        x, w, ws, xs, gl = cpu_sample_swiglu(counts, cfg["K"], cfg["N"], rows_per_expert, 0)
        ops_per_step = 2.0 * x.shape[0] * cfg["K"] * cfg["N"]
        workload = "c2: DeepSeek-V3 prefill gate/up, grouped_matmul_swiglu_quant, 32768 rows, 32 experts, K=7168, N=4096"
        sample = f"first {rows_per_expert} rows of each of the 32 experts ({x.shape[0]} of 32768 rows), full K and N, per step"

    def step():
        r = O.swiglu_quant(x, w, ws, xs, gl)
        if multi:
            O.gmm_w8a8(r["q"], w2, ws2, r["q_scale"], gl, 0)

    for _ in range(args.warmup if args.warmup < 2 else 1):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    tops = ops_per_step / dt / 1e12
    line = {
        "impl": "reference", "metric": "int8 GMM+SwiGLU-quant TOPS", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def cpu_baseline_sample(name="c2", seconds_budget=15.0):
    """The oracle (CPU restatement of the reference kernels) timed on a bounded sample of workload `name`."""
    from oracle import oracle as O
    from ops_transformer_b200 import synth
    O.build()
    O.use_all_cores()
    if name == "c5":
        (x, w, ws, xs, gl, w2, ws2), ops, sample = c5_cpu_sample()

        def fn():
            r = O.swiglu_quant(x, w, ws, xs, gl)
            O.gmm_w8a8(r["q"], w2, ws2, r["q_scale"], gl, 0)
        total_ops, label = ops, "c5: " + sample
    else:
        finalize = name.startswith("c3_finalize")
        base = name.replace("_finalize", "")
        cfg = synth.CONFIGS[base]
        counts = synth.config_counts(base, 0)
        swiglu = base in ("c2", "c4_swiglu", "c2_small", "c4_swiglu_small")
        rows_per_expert = 64
        x, w, ws, xs, gl = cpu_sample_swiglu(counts, cfg["K"], cfg["N"], rows_per_expert, 0)
        M = x.shape[0]
        if finalize:
            rng = np.random.default_rng(5)
            batch = max(1, M // 8)
            ri = (rng.permutation(M) % batch).astype(np.int64)
            lg = rng.uniform(0.05, 0.55, size=M).astype(np.float32)
            sh = O.f32_to_bf16_bits(rng.standard_normal((batch, cfg["N"])).astype(np.float32))
            cnt = np.diff(np.concatenate([[0], gl]))
            fn = lambda: O.gmm_finalize_routing(x, w, ws, xs, cnt, ri, batch, shared_input=sh, logit=lg)  # noqa: E731
        elif swiglu:
            fn = lambda: O.swiglu_quant(x, w, ws, xs, gl)  # noqa: E731
        else:
            fn = lambda: O.gmm_w8a8(x, w, ws, xs, gl, 0)  # noqa: E731
        total_ops = 2.0 * M * cfg["K"] * cfg["N"]
        total = int(np.asarray(counts).sum())
        label = f"{name}: first {rows_per_expert} rows of each expert ({M} of {total} rows), full K/N"
    t0 = time.perf_counter()
    reps = 0
    while True:
        fn()
        reps += 1
        if time.perf_counter() - t0 > seconds_budget or reps >= 5:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": total_ops / dt / 1e12, "unit": "TOPS", "cores": O.num_threads(), "kind": "port",
            "sample": f"{label}, {reps} repetitions"}


# ------------------------------------------------------------------------------------------------------------
# value checks of what was timed (outside the timed region; the only use of oracle/ besides the CPU baselines)
# ------------------------------------------------------------------------------------------------------------

def verify_rows(torch, kind, counts, x, w_nd, ws, xs, out0, out1):
    """Row sample of a finished launch against the CPU oracle: per expert the first and last row, the rows either side of
    every 128/256-row tile edge and 32 random ones (every row when there are at most 2048)."""
    from oracle import oracle as O
    from oracle import sampled_check as SC
    O.build()
    O.use_all_cores()
    rows = SC.sample_rows(counts, n_random=32, seed=0, max_rows_all=2048)
    sc = SC.counts_of_sample(rows, counts)
    sel = torch.from_numpy(rows).to(x.device)
    x_rows = x.index_select(0, sel).cpu().numpy()
    xs_rows = xs.index_select(0, sel).cpu().numpy()
    w_h, ws_h = w_nd.cpu().numpy(), ws.cpu().numpy()
    if kind == "swiglu":
        return SC.check_swiglu_rows(x_rows, w_h, ws_h, xs_rows, sc, out0.index_select(0, sel).cpu().numpy(),
                                    out1.index_select(0, sel).cpu().numpy())
    got = out0.index_select(0, sel).view(torch.int16).cpu().numpy().view(np.uint16)
    return SC.check_gmm_rows(x_rows, w_h, ws_h, xs_rows, sc, got)


def verify_finalize(torch, counts, x, w_nd, ws, xs, row_index, logit, shared, out0, n_dst=48):
    """Finalize routing: a sample of destination rows, each with every GEMM row that is combined into it."""
    from oracle import oracle as O
    O.build()
    O.use_all_cores()
    batch = out0.shape[0]
    rng = np.random.default_rng(0)
    dst = np.unique(np.concatenate([[0, batch - 1], rng.integers(0, batch, size=n_dst)])).astype(np.int64)
    ri = row_index.cpu().numpy()
    rows = np.nonzero(np.isin(ri, dst))[0].astype(np.int64)          # ascending: expert order is kept
    ends = np.cumsum(np.asarray(counts, np.int64))
    sc = np.bincount(np.searchsorted(ends, rows, side="right"), minlength=len(ends)).astype(np.int64)
    remap = np.searchsorted(dst, ri[rows]).astype(np.int64)
    sel = torch.from_numpy(rows).to(x.device)
    dsel = torch.from_numpy(dst).to(x.device)
    sh_bits = shared.index_select(0, dsel).view(torch.int16).cpu().numpy().view(np.uint16)
    ref = O.gmm_finalize_routing(x.index_select(0, sel).cpu().numpy(), w_nd.cpu().numpy(), ws.cpu().numpy(),
                                 xs.index_select(0, sel).cpu().numpy(), sc, remap, len(dst), shared_input=sh_bits,
                                 logit=logit.index_select(0, sel).cpu().numpy())
    got = out0.index_select(0, dsel).cpu().numpy()
    bound = 4.0 * 2.0 ** -23 * ref["abs_sum"] + 1e-30   # unordered fp32 sums of up to top-k + 1 terms
    bad = int(np.count_nonzero(~(np.abs(got.astype(np.float64) - ref["y"].astype(np.float64)) <= bound)))
    return {"rows": int(len(dst)), "gemm_rows": int(len(rows)), "mismatches": bad,
            "bar": "|got - oracle| <= 4 * 2^-23 * sum|terms| (atomic adds in any order)"}


def measure_workload(args, name, steps, weight_format="nd", with_e2e=False, verify=True):
    """Times one operator workload on cuda:0: whole steps and, with events the library records around it, the tensor-core
    kernel alone.  Returns a dict with the timings, the roofline block, the value check and (optionally) the end-to-end leg."""
    import torch

    import ops_transformer_b200 as ops
    from ops_transformer_b200 import LaunchOptions, synth

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    finalize = name in ("c3_finalize", "c3_finalize_small")  # the down projection of c3 fused with the weighted combine
    base = name.replace("_finalize", "")
    cfg = synth.CONFIGS[base]
    counts = synth.config_counts(base, 0)
    E, K, N = cfg["E"], cfg["K"], cfg["N"]
    M = int(counts.sum())
    swiglu = name in ("c2", "c4_swiglu", "c2_small", "c4_swiglu_small")
    x, w, ws, xs = gen_device_inputs(torch, dev, M, K, N, E, 0)
    w_nd = w
    gl = torch.from_numpy(np.cumsum(counts)).to(dev)
    nonempty = int((counts > 0).sum())
    wkw = {}
    if weight_format == "nz":  # the layout the reference's A8W8 SwiGLU operator asks for; cast once, outside the timing
        w = ops.format_cast_nz(w)
        wkw = {"weight_format": ops.ACL_FORMAT_FRACTAL_NZ}
    row_index = logit = shared = None
    if finalize:
        topk = 8
        batch = M // topk
        g = torch.Generator(device="cpu").manual_seed(5)
        row_index = (torch.randperm(M, generator=g) % batch).to(dev)
        logit = torch.rand(M, generator=g).mul_(0.5).add_(0.05).to(dev)
        shared = torch.randn(batch, N, generator=g).to(torch.bfloat16).to(dev)
        out0 = torch.empty((batch, N), dtype=torch.float32, device=dev)
        out1 = None
        out_bytes = batch * N * 4 + batch * N * 2 + M * 12   # fp32 result, bf16 shared rows, logits and row indices
        wflat = (2 if weight_format == "nz" else 0)
        gl_counts = torch.from_numpy(np.asarray(counts, np.int64)).to(dev)
        fin_ws = torch.zeros(256, dtype=torch.uint8, device=dev)
    elif swiglu:
        out0 = torch.empty((M, N // 2), dtype=torch.int8, device=dev)
        out1 = torch.empty((M,), dtype=torch.float32, device=dev)
        out_bytes = M * (N // 2) + M * 4
    else:
        out0 = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        out1 = None
        out_bytes = M * N * 2
    ops_per_step = 2.0 * M * K * N
    alg_bytes = M * K + nonempty * K * N + nonempty * N * 4 + M * 4 + out_bytes + E * 8

    def step(options=None):
        if finalize:
            ops.grouped_matmul_finalize_routing_flat(x, w, wflat, ws, gl_counts, row_index, out0, pertoken_scale=xs,
                                                     shared_input=shared, logit=logit, workspace=fin_ws, options=options)
            return fin_ws
        if swiglu:
            return ops.grouped_matmul_swiglu_quant(x, w, ws, xs, gl, output=out0, output_scale=out1, return_workspace=True,
                                                   options=options, **wkw)[-1]
        return ops.grouped_matmul_v4(x, w, ws, xs, gl, out=out0, return_workspace=True, options=options, **wkw)[-1]

    # L2 policy: for the prefill workloads one step streams > 1 GB, far more than the 126 MB L2; for the small
    # decode workloads a 256 MB buffer is rewritten between timed steps.
    flush = None
    if alg_bytes < 4 * 126e6:
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        wsb = step()
    ops.check_status(wsb)

    # kernel-only events (recorded by the library around the tensor-core kernel, per call) + whole-step events
    k_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    s_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in k_ev:
        a.record(); b.record()  # materialise the handles
    opts = [LaunchOptions(start_event=a.cuda_event, stop_event=b.cuda_event) for a, b in k_ev]
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    torch.cuda.synchronize()
    sampler.mark_begin()
    for i in range(steps):
        if flush is not None:
            flush.fill_(i & 0xff)
        s_ev[i][0].record()
        step(opts[i])
        s_ev[i][1].record()
    torch.cuda.synchronize()
    sampler.mark_end()
    clocks = sampler.stop()
    step_ms = [a.elapsed_time(b) for a, b in s_ev]
    kern_ms = [a.elapsed_time(b) for a, b in k_ev]
    ms = float(np.mean(step_ms))
    kms = float(np.mean(kern_ms))
    ops.check_status(wsb)

    verified = None
    if verify:
        if finalize:
            verified = verify_finalize(torch, counts, x, w_nd, ws, xs, row_index, logit, shared, out0)
        else:
            verified = verify_rows(torch, "swiglu" if swiglu else "gmm", counts, x, w_nd, ws, xs, out0, out1)

    res = {"name": name, "E": E, "K": K, "N": N, "M": M, "nonempty": nonempty, "swiglu": swiglu, "finalize": finalize,
           "ms": ms, "kernel_ms": kms, "kern_ms_list": kern_ms, "ops": ops_per_step, "alg_bytes": alg_bytes, "clocks": clocks,
           "flush": flush is not None, "verified": verified, "tokens": cfg.get("tokens", 0), "steps": steps, "warmup": warmup,
           "weight_format": weight_format}

    if with_e2e:
        # end to end through the public API with host buffers: pinned H2D of the step's inputs, the two-phase call,
        # D2H of the results, all inside the timed region.
        hx = torch.empty_like(x, device="cpu").pin_memory(); hx.copy_(x)
        hxs = torch.empty_like(xs, device="cpu").pin_memory(); hxs.copy_(xs)
        hgl = torch.empty_like(gl, device="cpu").pin_memory(); hgl.copy_(gl)
        ho0 = torch.empty_like(out0, device="cpu").pin_memory()
        ho1 = torch.empty_like(out1, device="cpu").pin_memory() if out1 is not None else None
        dx, dxs, dgl = torch.empty_like(x), torch.empty_like(xs), torch.empty_like(gl)
        pipe = None
        if not finalize and args.e2e_pieces > 1:   # the pipelined helper slices the weight by experts, in either layout
            # the call a user with host-resident rows makes: the operator split by experts into a copy-in / operator /
            # copy-out pipeline (ops_transformer_b200/hostio.py); every piece goes through the aclnn entry points
            from ops_transformer_b200.hostio import HostPipelinedGroupedOp
            pipe = HostPipelinedGroupedOp("swiglu_quant" if swiglu else "gmm", w, ws, M, pieces=args.e2e_pieces)

        def e2e_step():
            if pipe is not None:
                pipe.run(hx, hxs, counts, ho0, ho1)
                return
            dx.copy_(hx, non_blocking=True); dxs.copy_(hxs, non_blocking=True); dgl.copy_(hgl, non_blocking=True)
            if finalize:
                ops.grouped_matmul_finalize_routing_flat(dx, w, wflat, ws, gl_counts, row_index, out0, pertoken_scale=dxs,
                                                         shared_input=shared, logit=logit, workspace=fin_ws)
                ho0.copy_(out0, non_blocking=True)
            elif swiglu:
                ops.grouped_matmul_swiglu_quant(dx, w, ws, dxs, dgl, output=out0, output_scale=out1, **wkw)
                ho0.copy_(out0, non_blocking=True); ho1.copy_(out1, non_blocking=True)
            else:
                ops.grouped_matmul_v4(dx, w, ws, dxs, dgl, out=out0, **wkw)
                ho0.copy_(out0, non_blocking=True)
            torch.cuda.synchronize()

        e2e_step()
        e_steps = max(3, min(steps, 10))
        t0 = time.perf_counter()
        for _ in range(e_steps):
            e2e_step()
        e2e_ms = (time.perf_counter() - t0) / e_steps * 1e3
        h2d = hx.numel() + hxs.numel() * 4 + hgl.numel() * 8
        d2h = ho0.numel() * ho0.element_size() + (ho1.numel() * 4 if ho1 is not None else 0)
        res["e2e"] = {"value": ops_per_step / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
                      "pieces": args.e2e_pieces if pipe is not None else 1,
                      "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)}
        if not finalize and out1 is not None and verify:
            # the pipelined end-to-end leg must produce the same values as the single call just verified
            res["e2e"]["matches_device_run"] = bool(torch.equal(ho0.to(dev), out0))
    del x, w, w_nd, ws, xs, out0, out1, flush
    torch.cuda.empty_cache()
    return res


def roofline_of(res):
    """The roofline block of a measured workload: achieved = algorithmic ops (or bytes) per launch / the kernel's own
    CUDA-event duration; peak = the measured figure of MEASURED_PEAKS.json (fallback constants if that file is absent)."""
    peaks = measured_peaks()
    clocks = res["clocks"]
    kms, kern_ms = res["kernel_ms"], res["kern_ms_list"]
    # tcgen05 int8 runs at twice the bf16 rate.  Two measured bf16 figures exist: a burst one (best of 10 at full clock) and
    # a sustained one (seconds of back-to-back GEMMs under the power cap).  Which regime the timed region ran in is read
    # off the clocks sampled during it: power-capped with the SM clock well below its maximum = sustained, otherwise burst.
    capped = "sw_power_cap" in (clocks.get("reasons") or []) and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and \
        clocks["sm_mhz"] < 0.9 * clocks["sm_max_mhz"]
    int8_burst, int8_sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
    int8_peak = int8_sustained if capped else int8_burst
    t_tensor = res["ops"] / (int8_burst * 1e12)
    t_hbm = res["alg_bytes"] / (peaks["hbm_gbs"] * 1e9)
    if t_tensor >= t_hbm:
        ach = res["ops"] / (kms * 1e-3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": int8_peak, "unit": "TFLOP/s",
                "peak_basis": (f"2 x bf16 {'sustained' if capped else 'burst'} of {peaks['source']} "
                               f"({peaks['bf16_tflops_sustained'] if capped else peaks['bf16_tflops']} TFLOP/s): the timed region ran "
                               f"{'power-capped at ' + str(clocks.get('sm_mhz')) + ' MHz' if capped else 'at full clock'}; "
                               "int8 ops counted as 2 per multiply-add"),
                "frac_vs_burst": ach / int8_burst, "frac_vs_sustained": ach / int8_sustained}
    else:
        roof = {"bound": "hbm", "achieved": res["alg_bytes"] / (kms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "peak_basis": f"copy bandwidth, {peaks['source']}"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    traffic = NCU_DRAM_BYTES_PER_LAUNCH.get(res["name"]) if res["weight_format"] == "nd" else None
    roof["traffic"] = traffic[0] if traffic else None
    roof["traffic_source"] = f"constant from {traffic[1]} (not measured by this run)" if traffic else None
    roof["kernel"] = "gmm_w8a8_sm100_kernel"
    roof["kernel_ms"] = kms
    roof["kernel_ms_p10_p50_p90"] = [float(np.percentile(kern_ms, q)) for q in (10, 50, 90)]
    roof["algorithmic_bytes"] = res["alg_bytes"]
    roof["algorithmic_ops"] = res["ops"]
    return roof


def extra_block(res):
    """Short form of a measured workload for the `extra` object of the headline line."""
    roof = roofline_of(res)
    out = {"workload": f"{res['name']}: E={res['E']} K={res['K']} N={res['N']} rows={res['M']} non-empty experts={res['nonempty']}",
           "steps": res["steps"], "kernel_ms": res["kernel_ms"], "ms_per_step": res["ms"], "bound": roof["bound"],
           "achieved": roof["achieved"], "unit": roof["unit"], "peak": roof["peak"], "frac": roof["frac"],
           "l2": "256 MB flush write between steps" if res["flush"] else "inputs larger than L2",
           "sm_mhz": res["clocks"].get("sm_mhz"), "reasons": res["clocks"].get("reasons"), "verified": res["verified"]}
    if roof["bound"] == "tensor":
        out["frac_vs_burst"], out["frac_vs_sustained"] = roof["frac_vs_burst"], roof["frac_vs_sustained"]
    return out


def c2_summary(args):
    return extra_block(measure_workload(args, "c2", min(args.steps, 100), with_e2e=False, verify=not args.no_verify))


def bench_single(args):
    name = args.workload or "c2"
    res = measure_workload(args, name, args.steps, args.weight_format, with_e2e=True, verify=not args.no_verify)
    roof = roofline_of(res)
    ms, swiglu, finalize = res["ms"], res["swiglu"], res["finalize"]
    tops = res["ops"] / (ms * 1e-3) / 1e12
    line = {
        "metric": "int8 GMM+SwiGLU-quant TOPS" if swiglu else ("int8 GMM+finalize-routing TOPS" if finalize else "int8 GMM W8A8 TOPS"),
        "value": tops, "unit": "TOPS", "n_gpus": 1, "steps": args.steps, "warmup": res["warmup"],
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": f"{name}: E={res['E']} K={res['K']} N={res['N']} rows={res['M']} non-empty experts={res['nonempty']}",
                   "weight_format": "FRACTAL_NZ" if args.weight_format == "nz" else "ND",
                   "l2": "256 MB flush write between steps" if res["flush"] else "inputs larger than L2",
                   "tokens_per_s": (res["tokens"] / (ms * 1e-3)) if res["tokens"] else None,
                   "verified": res["verified"]},
        "roofline": roof,
        "e2e": res["e2e"],
        # one kernel per operator call (the int8 requant is fused into the GEMM kernel); finalize routing adds the kernel
        # that initialises the fp32 result
        "gpu_launches": args.steps * (2 if finalize else 1),
        "clocks": res["clocks"],
        "pct_of_nominal_int8_peak": tops / 4500.0 * 100.0,
    }
    if name == "c2" and not args.no_extras:
        # the other claims of the benchmark definition, measured in the same run on this GPU
        extra = {}
        for wl in ("c3", "c4_swiglu", "c4_down", "c3_finalize"):
            extra[wl] = extra_block(measure_workload(args, wl, min(args.steps, 100), verify=not args.no_verify))
        extra["c2_fractal_nz"] = extra_block(measure_workload(args, "c2", min(args.steps, 100), "nz", verify=not args.no_verify))
        extra["init_routing"] = measure_init_routing(args, min(args.steps, 100), verify=not args.no_verify)
        line["extra"] = extra
    if name == "c2" and not args.no_ep:
        # the expert-parallel workload (config 5) on this one GPU: the reference point of the multi-GPU lines
        import torch

        import bench_ep
        line["ep"] = {"workload": "c5 on one GPU: 256 local experts, 16384 tokens, top-8, swiglu_quant then down GEMM",
                      **bench_ep.one_gpu_summary(args, torch.device("cuda:0"), verify=not args.no_verify)}
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_sample(name)
    print(json.dumps(line))


def cpu_baseline_init_routing(n, k, h, E, alg_bytes):
    """The oracle's MoeInitRoutingV3 on the first 512 tokens of the workload (same seed), single thread."""
    from oracle import oracle as O
    O.build()
    import torch
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(n, h, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(n)]).to(torch.int32)
    m = 512
    xb = x[:m].view(torch.int16).numpy().view(np.uint16)
    ib = idx[:m].numpy()
    t0 = time.perf_counter()
    reps = 0
    while True:
        O.moe_init_routing_v3(xb, ib, E, (0, E), True)
        reps += 1
        if time.perf_counter() - t0 > 10.0 or reps >= 5:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": alg_bytes * (m / n) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": f"first {m} of {n} tokens, {reps} repetitions"}


def measure_init_routing(args, steps, verify=True):
    """The producer of c2's inputs: 4096 bf16 tokens x top-8 over 32 experts, hidden 7168, dynamic per-row int8 quantisation
    (MoeInitRoutingV3).  HBM-bound byte work: every token row is read from DRAM once (its 8 uses hit the L2), every
    output row written once."""
    import torch

    import ops_transformer_b200 as ops

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    n, k, h, E = 4096, 8, 7168, 32
    g = torch.Generator(device="cpu").manual_seed(0)
    hx = torch.randn(n, h, generator=g).to(torch.bfloat16)
    hidx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(n)]).to(torch.int32)
    x, idx = hx.to(dev), hidx.to(dev)
    outs = (torch.empty((n * k, h), dtype=torch.int8, device=dev), torch.empty((n * k,), dtype=torch.int32, device=dev),
            torch.empty((E,), dtype=torch.int64, device=dev), torch.empty((n * k,), dtype=torch.float32, device=dev))
    alg_bytes = n * h * 2 + n * k * h + n * k * (4 + 4 + 4) + E * 8
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def step():
        ops.moe_init_routing_v3(x, idx, expert_num=E, active_expert_range=(0, E), quant_mode=1, outputs=outs)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    # The launches of one call are replayed as a CUDA graph: through Python the host needs longer to issue them
    # than the GPU needs to run them, and the events would then time the host.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    graph.replay()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    sampler.mark_begin()
    for i in range(steps):
        flush.fill_(i & 0xff)
        ev[i][0].record()
        graph.replay()
        ev[i][1].record()
    torch.cuda.synchronize()
    sampler.mark_end()
    clocks = sampler.stop()
    ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))
    verified = None
    if verify:
        from oracle import oracle as O
        O.build()
        ref = O.moe_init_routing_v3(hx.view(torch.int16).numpy().view(np.uint16), hidx.numpy(), E, (0, E), True)
        got = [t.cpu().numpy() for t in outs]
        bad = sum(int(np.count_nonzero(a != b)) for a, b in zip(got, (ref["expanded_x"], ref["expanded_row_idx"], ref["counts"],
                                                                     ref["expanded_scale"])))
        verified = {"rows": n * k, "mismatches": bad, "bar": "all four outputs bit-identical to the oracle"}
    peaks = measured_peaks()
    gbs = alg_bytes / (ms * 1e-3) / 1e9
    del flush, outs, x
    torch.cuda.empty_cache()
    return {"workload": f"init_routing: {n} tokens x top-{k}, {E} experts, hidden {h}", "steps": steps, "ms_per_step": ms,
            "bound": "hbm", "achieved": gbs, "unit": "GB/s", "peak": peaks["hbm_gbs"], "frac": gbs / peaks["hbm_gbs"],
            "l2": "256 MB flush write between steps", "launch": "CUDA graph replay of one operator call",
            "algorithmic_bytes": alg_bytes, "rows_per_s": n * k / (ms * 1e-3), "clocks": clocks, "verified": verified}


def bench_init_routing(args):
    r = measure_init_routing(args, args.steps, verify=not args.no_verify)
    n, k, h, E = 4096, 8, 7168, 32
    print(json.dumps({
        "metric": "MoeInitRoutingV3 dynamic-quant GB/s", "value": r["achieved"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16->int8", "data": "synthetic",
        "config": {"workload": r["workload"], "l2": r["l2"], "launch": r["launch"], "verified": r["verified"]},
        "roofline": {"bound": "hbm", "achieved": r["achieved"], "peak": r["peak"], "unit": "GB/s", "frac": r["frac"],
                     "traffic": None, "algorithmic_bytes": r["algorithmic_bytes"], "kernel": "routing_quant_kernel (+ count, scan, scatter)",
                     "peak_basis": f"copy bandwidth, {measured_peaks()['source']}"},
        "gpu_launches": args.steps * 4, "clocks": r["clocks"], "rows_per_s": r["rows_per_s"],
        "cpu_baseline": None if args.no_cpu_baseline else cpu_baseline_init_routing(n, k, h, E, r["algorithmic_bytes"])}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, help="c2 (default at N=1), c3, c4_swiglu, c4_down, c3_finalize, init_routing")
    ap.add_argument("--weight-format", default="nd", choices=["nd", "nz"], help="N=1: weight layout [E,K,N] or FRACTAL_NZ")
    ap.add_argument("--e2e-pieces", type=int, default=8,
                    help="N=1 end-to-end leg: expert ranges pipelined as copy-in / operator / copy-out (1 = one whole call)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check of the timed results (it runs outside the timed region)")
    ap.add_argument("--no-extras", action="store_true", help="N=1: skip the extra workloads (c3, c4, finalize routing, NZ weights, init routing)")
    ap.add_argument("--no-ep", action="store_true", help="N=1: skip the one-GPU run of the expert-parallel workload")
    ap.add_argument("--ep-tokens", type=int, default=16384, help="tokens per GPU of the expert-parallel workload")
    ap.add_argument("--ep-chunks", type=int, default=0, help="token chunks pipelined against the exchange (0 = by world size)")
    ap.add_argument("--ep-parts", type=int, default=0,
                    help="fused variant: expert ranges per rank pipelined against the exchange (0 = default, one range)")
    ap.add_argument("--ep-reserve-sms", type=int, default=-1, help="SMs left free for the exchange kernels (-1 = automatic)")
    ap.add_argument("--ep-impl", default="fused", choices=["fused", "nccl"],
                    help="fused: rows move by peer stores inside our kernels; nccl: NCCL all-to-all around the operators")
    ap.add_argument("--ep-graph", type=int, default=1, help="1: replay the fused expert-parallel step as a CUDA graph")
    ap.add_argument("--ep-skip-n1", action="store_true", help="N>1: skip rank 0's one-GPU run of the same workload")
    ap.add_argument("--ep-phases", action="store_true", help="also report serialised per-phase times (diagnostic)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args)
        return
    if headline_is_c5(args):
        import bench_ep
        world = int(os.environ.get("WORLD_SIZE", "1"))
        extra = (lambda: c2_summary(args)) if world == 1 and launched_by_torchrun() and not args.no_extras else None
        bench_ep.bench_main(args, ClockSampler, cpu_baseline_sample, measured_peaks, extra_c2=extra)
        return
    if args.workload == "init_routing":
        bench_init_routing(args)
        return
    bench_single(args)


if __name__ == "__main__":
    main()
