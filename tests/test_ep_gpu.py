"""Expert-parallel FFN on the GPU: the single-rank path (no exchange) against the oracle, and - when the machine has
two GPUs - two NCCL ranks against the oracle applied to each rank's rows with all experts."""
import os
import subprocess
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)  # this file is also run as a script by the two-rank test

from ops_transformer_b200 import ep, synth  # noqa: E402

pytestmark = pytest.mark.gpu

N_EXPERTS, H, I, TOP_K, T = 8, 256, 128, 2, 300


def _weights():
    return (synth.int8_tensor((N_EXPERTS, H, 2 * I), 80, 1), synth.int8_tensor((N_EXPERTS, I, H), 80, 2),
            synth.scale_tensor((N_EXPERTS, 2 * I), 80, 3), synth.scale_tensor((N_EXPERTS, H), 80, 4))


def _inputs(rank):
    x = synth.int8_tensor((T, H), 90 + rank, 1)
    xs = synth.scale_tensor((T,), 90 + rank, 2)
    rng = np.random.default_rng(95 + rank)
    topk = np.stack([rng.choice(N_EXPERTS, TOP_K, replace=False) for _ in range(T)]).astype(np.int64)
    return x, xs, topk


def _check(O, res, chunks, x, xs, topk, w1, s1, w2, s2):
    bounds = [T * c // chunks for c in range(chunks + 1)]
    for c, r in enumerate(res):
        p = r["plan"]
        tok = p.src_token.cpu().numpy() + bounds[c]
        experts = topk[bounds[c]:bounds[c + 1]].reshape(-1)[p.order.cpu().numpy()]
        gl = np.cumsum(np.bincount(experts, minlength=N_EXPERTS))
        q = O.swiglu_quant(x[tok], w1, s1, xs[tok], gl)
        exp = O.gmm_w8a8(q["q"], w2, s2, q["q_scale"], gl, 0)["y"]
        got = r["y"].view(torch.int16).cpu().numpy().view(np.uint16)
        a, b = O.bf16_bits_to_f32(got), O.bf16_bits_to_f32(exp)
        # a 1-LSB difference in an int8 activation (allowed on 0.01 % of them) moves a few bf16 results slightly
        bad = np.abs(a - b) > 1e-2 + 4e-3 * np.abs(b)
        assert bad.mean() < 1e-3, f"{bad.sum()} of {bad.size} results outside tolerance"
        assert (got == exp).mean() > 0.995


@pytest.mark.parametrize("chunks", [1, 2])
def test_single_rank_ffn_matches_oracle(oracle, chunks):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    w1, w2, s1, s2 = _weights()
    x, xs, topk = _inputs(0)
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    ffn = ep.ExpertParallelFFN(N_EXPERTS, t(w1), t(s1), t(w2), t(s2), chunks=chunks)
    res = ffn.forward(t(x), t(xs), t(topk))
    torch.cuda.synchronize()
    _check(oracle, res, chunks, x, xs, topk, w1, s1, w2, s2)


def _check_parts(O, res, x, xs, topk, w1, s1, w2, s2):
    """Expert-range pieces: every piece holds, in its own send order, the pairs routed to its range of local experts."""
    seen = 0
    for ch in res["chunks"]:
        n = int(ch["rows_in_use"].item())
        order = ch["plan"].order.cpu().numpy()[:n]
        tok = ch["plan"].src_token.cpu().numpy()[:n]
        experts = topk.reshape(-1)[order]
        assert (tok == order // TOP_K).all() and (np.diff(experts) >= 0).all()
        gl = np.cumsum(np.bincount(experts, minlength=N_EXPERTS))
        q = O.swiglu_quant(x[tok], w1, s1, xs[tok], gl)
        exp = O.gmm_w8a8(q["q"], w2, s2, q["q_scale"], gl, 0)["y"]
        got = ch["y"][:n].view(torch.int16).cpu().numpy().view(np.uint16)
        a, b = O.bf16_bits_to_f32(got), O.bf16_bits_to_f32(exp)
        bad = np.abs(a - b) > 1e-2 + 4e-3 * np.abs(b)
        assert bad.mean() < 1e-3 and (got == exp).mean() > 0.995
        seen += n
    assert seen == T * TOP_K, "the pieces together hold every (token, slot) pair once"


def _check_combined(O, ffn, res, wts):
    """res["combined"] against the oracle's combine of the returned rows, bit for bit; the pair -> row map is rebuilt here
    from the pieces' send orders."""
    pair_row = np.full(T * TOP_K, -1, np.int64)
    for c, ch in enumerate(res["chunks"]):
        n = int(ch["rows_in_use"].item()) if "rows_in_use" in ch else int(ch["plan"].order.shape[0])
        order = ch["plan"].order.cpu().numpy()[:n]
        pair0 = 0 if ffn.parts > 1 else ffn.bounds[c] * TOP_K
        pair_row[pair0 + order] = ffn.result_base[c] + np.arange(n)
    assert (pair_row >= 0).all() and int(res["bad_pairs"].item()) == 0
    y_bits = res["y"].view(torch.int16).cpu().numpy().view(np.uint16)
    want = O.ep_combine(y_bits, pair_row.reshape(T, TOP_K), wts)
    got = res["combined"].view(torch.int16).cpu().numpy().view(np.uint16)
    assert got.shape == want.shape and np.array_equal(got, want)


def _run_fused(O, dev, rank, world, w1, s1, w2, s2, x, xs, topk, chunks=1, route_kernels=True, parts=1):
    el = N_EXPERTS // world
    lo, hi = rank * el, (rank + 1) * el
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    ffn = ep.FusedExpertParallelFFN(N_EXPERTS, H, H, t(w1[lo:hi]), t(s1[lo:hi]), t(w2[lo:hi]), t(s2[lo:hi]), tokens=T, top_k=TOP_K,
                                    capacity=2 * T * TOP_K, chunks=chunks, expert_parts=parts)
    ffn.route_kernels = route_kernels
    wts = np.random.default_rng(97 + rank).uniform(0.05, 1.0, size=(T, TOP_K)).astype(np.float32) if route_kernels else None
    for _ in range(2):  # twice: the second step runs over the first one's buffers
        res = ffn.forward(t(x), t(xs), t(topk), None if wts is None else t(wts))
    torch.cuda.synchronize()
    assert int(ffn.overflow.item()) == 0
    if wts is not None:
        _check_combined(O, ffn, res, wts)
    if parts > 1:
        _check_parts(O, res, x, xs, topk, w1, s1, w2, s2)
        ffn.close()
        return
    outs = []
    for c, ch in enumerate(res["chunks"]):  # _check expects chunk-local token numbers in the plan
        pl = ch["plan"]
        outs.append({"y": ch["y"], "plan": ep.ChunkPlan(order=pl.order, src_token=pl.src_token - ffn.bounds[c], send_counts=pl.send_counts)})
    _check(O, outs, chunks, x, xs, topk, w1, s1, w2, s2)
    for c, ch in enumerate(res["chunks"]):  # the send order is a permutation of the chunk's pairs, grouped by expert
        order = ch["plan"].order.cpu().numpy()
        lo, hi = ffn.bounds[c], ffn.bounds[c + 1]
        assert sorted(order.tolist()) == list(range((hi - lo) * TOP_K))
        assert (np.diff(topk[lo:hi].reshape(-1)[order]) >= 0).all()
    ffn.close()


@pytest.mark.parametrize("chunks", [1, 3])
def test_single_rank_fused_ffn_matches_oracle(oracle, chunks):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    w1, w2, s1, s2 = _weights()
    x, xs, topk = _inputs(0)
    _run_fused(oracle, torch.device("cuda:0"), 0, 1, w1, s1, w2, s2, x, xs, topk, chunks=chunks)
    _run_fused(oracle, torch.device("cuda:0"), 0, 1, w1, s1, w2, s2, x, xs, topk, chunks=chunks, route_kernels=False)


@pytest.mark.parametrize("parts", [2, 4])
def test_single_rank_fused_ffn_expert_ranges(oracle, parts):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    w1, w2, s1, s2 = _weights()
    x, xs, topk = _inputs(0)
    _run_fused(oracle, torch.device("cuda:0"), 0, 1, w1, s1, w2, s2, x, xs, topk, parts=parts)


def _rank_main():
    import torch.distributed as dist
    from oracle import oracle as O
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    w1, w2, s1, s2 = _weights()
    el = N_EXPERTS // world
    lo, hi = rank * el, (rank + 1) * el
    x, xs, topk = _inputs(rank)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    ffn = ep.ExpertParallelFFN(N_EXPERTS, t(w1[lo:hi]), t(s1[lo:hi]), t(w2[lo:hi]), t(s2[lo:hi]), chunks=2)
    res = ffn.forward(t(x), t(xs), t(topk))
    torch.cuda.synchronize()
    _check(O, res, 2, x, xs, topk, w1, s1, w2, s2)
    _run_fused(O, dev, rank, world, w1, s1, w2, s2, x, xs, topk)
    _run_fused(O, dev, rank, world, w1, s1, w2, s2, x, xs, topk, chunks=2)
    _run_fused(O, dev, rank, world, w1, s1, w2, s2, x, xs, topk, route_kernels=False)
    _run_fused(O, dev, rank, world, w1, s1, w2, s2, x, xs, topk, parts=2)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


def test_two_rank_nccl_ffn_matches_oracle(oracle):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29655", os.path.abspath(__file__)]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    _rank_main()
