"""Parity at the sizes the benchmark definition names, through the aclnn entry points.

The oracle cannot run 32768 x 7168 x 4096 in seconds, so every full-size launch is compared on a ROW SAMPLE: both
operators treat each row on its own, hence the oracle applied to the selected rows (same weights, full K and N) must
reproduce those rows of the large launch.  Per expert the sample holds the first and last row, the rows either side of
every 128- and 256-row tile edge and 32 random rows; rows beyond group_list[-1] must keep their sentinel values.
Bars as everywhere: int32 bit-exact, bf16 within rtol 4e-3 / atol 1e-2 (and expected bit-identical), requant scales 1e-6
relative, int8 at most 1 LSB apart on at most 0.01 % of elements.

Inputs are generated on the device (uniform int8 in [-127, 127], fp32 scales in [1e-3, 1e-2], the routing of
ops_transformer_b200.synth) and only the sampled rows and the weights travel to the host.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from ops_transformer_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu

TAIL = 37  # rows past group_list[-1] that no launch may touch


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _inputs(dev, counts, K, N, seed):
    E, M = len(counts), int(np.sum(counts)) + TAIL
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
    w = torch.randint(-127, 128, (E, K, N), dtype=torch.int8, device=dev, generator=g)
    ws = torch.empty((E, N), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    xs = torch.empty((M,), dtype=torch.float32, device=dev).uniform_(1e-3, 1e-2, generator=g)
    gl = torch.from_numpy(np.cumsum(counts).astype(np.int64)).to(dev)
    return x, w, ws, xs, gl


def _sample(counts, dev):
    from oracle import sampled_check as SC
    rows = SC.sample_rows(counts, n_random=32, seed=1, max_rows_all=2048)
    return rows, SC.counts_of_sample(rows, counts), torch.from_numpy(rows).to(dev)


def run_swiglu_config(counts, K, N, seed, weight="nd", api=""):
    import ops_transformer_b200 as ops
    from oracle import sampled_check as SC
    dev = _dev()
    counts = np.asarray(counts, np.int64)
    x, w, ws, xs, gl = _inputs(dev, counts, K, N, seed)
    M, covered = x.shape[0], int(counts.sum())
    q = torch.full((M, N // 2), -77, dtype=torch.int8, device=dev)
    qs = torch.full((M,), -5.0, dtype=torch.float32, device=dev)
    kw = {}
    wt = w
    if weight == "nz":
        wt = ops.format_cast_nz(w)
        kw = {"api": api} if api == "WeightNZ" else {"weight_format": ops.ACL_FORMAT_FRACTAL_NZ}
    _, _, wsb = ops.grouped_matmul_swiglu_quant(x, wt, ws, xs, gl, output=q, output_scale=qs, return_workspace=True, **kw)
    ops.check_status(wsb)
    assert bool((q[covered:] == -77).all()) and bool((qs[covered:] == -5.0).all()), "rows beyond group_list[-1] were written"
    rows, sc, sel = _sample(counts, dev)
    r = SC.check_swiglu_rows(x.index_select(0, sel).cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(),
                             xs.index_select(0, sel).cpu().numpy(), sc, q.index_select(0, sel).cpu().numpy(),
                             qs.index_select(0, sel).cpu().numpy())
    assert r["mismatches"] == 0 and r["int8_off_by_more"] == 0 and r["scale_max_rel"] <= SC.QSCALE_RTOL, r
    assert r["int8_off_by_one"] <= SC.Q_LSB_FRACTION * r["int8_elements"], r
    return r


def run_gmm_config(counts, K, N, seed, out_dtype="bf16", weight="nd"):
    import ops_transformer_b200 as ops
    from oracle import sampled_check as SC
    dev = _dev()
    counts = np.asarray(counts, np.int64)
    x, w, ws, xs, gl = _inputs(dev, counts, K, N, seed)
    M, covered = x.shape[0], int(counts.sum())
    if out_dtype == "int32":
        out = torch.full((M, N), -123456789, dtype=torch.int32, device=dev)
    else:
        out = torch.full((M, N), 0x7fc1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    kw = {}
    wt = w
    if weight == "nz":
        wt = ops.format_cast_nz(w)
        kw = {"weight_format": ops.ACL_FORMAT_FRACTAL_NZ}
    floating = out_dtype != "int32"
    _, wsb = ops.grouped_matmul_v4(x, wt, ws if floating else None, xs if floating else None, gl, out=out,
                                   out_dtype=out.dtype, return_workspace=True, **kw)
    ops.check_status(wsb)
    tail = out[covered:]
    if floating:
        assert bool((tail.view(torch.int16) == 0x7fc1).all()), "rows beyond group_list[-1] were written"
    else:
        assert bool((tail == -123456789).all()), "rows beyond group_list[-1] were written"
    rows, sc, sel = _sample(counts, dev)
    got = out.index_select(0, sel)
    got = got.cpu().numpy() if not floating else got.view(torch.int16).cpu().numpy().view(np.uint16)
    r = SC.check_gmm_rows(x.index_select(0, sel).cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(),
                          xs.index_select(0, sel).cpu().numpy(), sc, got, y_dtype=out_dtype)
    assert r["mismatches"] == 0, r
    assert r["not_bit_identical"] == 0, r
    return r


# ---- configs[1]: DeepSeek-V3 prefill gate/up, 32768 rows over 32 experts, K=7168, N=4096 --------------------------------

@pytest.mark.parametrize("weight", ["nd", "nz"])
def test_config_c2_swiglu_quant_full_size(oracle, weight):
    c = synth.CONFIGS["c2"]
    counts = synth.config_counts("c2", 0)
    assert counts.sum() == 32768 and len(counts) == 32
    r = run_swiglu_config(counts, c["K"], c["N"], seed=11, weight=weight)
    assert r["rows"] > 1000


# ---- configs[2]: the down projection, same routing, K=2048, N=7168 ------------------------------------------------------

def test_config_c3_down_gemm_full_size_bf16(oracle):
    c = synth.CONFIGS["c3"]
    run_gmm_config(synth.config_counts("c3", 0), c["K"], c["N"], seed=12)


def test_config_c3_down_gemm_full_size_int32_accumulators(oracle):
    c = synth.CONFIGS["c3"]
    run_gmm_config(synth.config_counts("c3", 0), c["K"], c["N"], seed=13, out_dtype="int32")


# ---- configs[3]: decode, 1024 rows over 256 experts, Zipf(1.1), many empty groups: every row is checked ------------------

@pytest.mark.parametrize("weight", ["nd", "nz"])
def test_config_c4_decode_swiglu_quant_full_size(oracle, weight):
    c = synth.CONFIGS["c4_swiglu"]
    counts = synth.config_counts("c4_swiglu", 0)
    assert counts.sum() == 1024 and (counts == 0).sum() > 50
    r = run_swiglu_config(counts, c["K"], c["N"], seed=14, weight=weight)
    assert r["rows"] == 1024


def test_config_c4_decode_down_gemm_full_size(oracle):
    c = synth.CONFIGS["c4_down"]
    r = run_gmm_config(synth.config_counts("c4_down", 0), c["K"], c["N"], seed=15)
    assert r["rows"] == 1024


# ---- the shape of the reference's own example: E=4, M=8192, K=7168, N=4096, FRACTAL_NZ weight ----------------------------
# gmm/grouped_matmul_swiglu_quant/examples/test_aclnn_grouped_matmul_swiglu_quant.cpp:85-88 (the example's tensors are all
# zero, its group list included, so the call touches no row; both that literal call and a filled one are run)

def test_reference_example_shape_filled(oracle):
    run_swiglu_config([2048, 1901, 2243, 2000], 7168, 4096, seed=16, weight="nz", api="WeightNZ")


def test_reference_example_shape_literal_zero_group_list(oracle):
    import ops_transformer_b200 as ops
    dev = _dev()
    E, M, K, N = 4, 8192, 7168, 4096
    x = torch.zeros((M, K), dtype=torch.int8, device=dev)
    w = torch.zeros((E, N // 32, K // 16, 16, 32), dtype=torch.int8, device=dev)
    ws = torch.zeros((E, N), dtype=torch.float32, device=dev)
    xs = torch.zeros((M,), dtype=torch.float32, device=dev)
    gl = torch.zeros((E,), dtype=torch.int64, device=dev)
    q = torch.full((M, N // 2), -77, dtype=torch.int8, device=dev)
    qs = torch.full((M,), -5.0, dtype=torch.float32, device=dev)
    _, _, wsb = ops.grouped_matmul_swiglu_quant(x, w, ws, xs, gl, output=q, output_scale=qs, return_workspace=True,
                                                weight_format=ops.ACL_FORMAT_FRACTAL_NZ)
    ops.check_status(wsb)
    assert bool((q == -77).all()) and bool((qs == -5.0).all())


# ---- configs[4] on one GPU: the expert-parallel FFN with all 256 experts local, checked like the benchmark checks it ----

def test_config_c5_expert_parallel_ffn_one_gpu_full_size(oracle):
    import argparse

    import bench_ep
    dev = _dev()
    args = argparse.Namespace(ep_impl="fused", ep_chunks=0, ep_reserve_sms=-1)
    tokens = 16384
    d = bench_ep.make_rank_data(dev, 1, 0, tokens)
    ffn, _, _ = bench_ep.build_ffn(args, d, tokens, 1)
    for _ in range(2):
        res = ffn.forward(d["x"], d["xs"], d["topk"])
    torch.cuda.synchronize()
    assert int(res["dropped_rows"].item()) == 0
    v = bench_ep.verify_returned_rows(res, d, dev, 1, 0, tokens, experts_checked=8, rows_per_expert=40)
    ffn.close()
    assert v["rows"] > 100 and v["mismatches"] == 0, v
    assert v["not_bit_identical"] <= 0.005 * v["rows"] * bench_ep.HIDDEN, v
