"""Parity of the CUDA path (through the C ABI) against the CPU oracle on identical seeded inputs.

Bars: int32 accumulators bit-exact; bf16 results within rtol 4e-3 / atol 1e-2 of the oracle (they are in fact
expected to be bit-identical, which is asserted too); per-token requant scales within 1e-6 relative; int8
requant values identical except at most 1 LSB on at most 0.01 % of elements; rows that group_list does not
cover keep their previous contents.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from ops_transformer_b200 import synth  # noqa: E402

pytestmark = pytest.mark.gpu

BF16_RTOL, BF16_ATOL = 4e-3, 1e-2
QSCALE_RTOL = 1e-6
Q_LSB_FRACTION = 1e-4


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _bf16_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def make_inputs(M, K, N, E, seed=0):
    x = synth.int8_tensor((M, K), seed, 1)
    w = synth.int8_tensor((E, K, N), seed, 2)
    ws = synth.scale_tensor((E, N), seed, 3)
    xs = synth.scale_tensor((M,), seed, 4)
    return x, w, ws, xs


def nd_to_nz(w):
    """[E, K, N] -> FRACTAL_NZ storage [E, N/32, K/16, 16, 32]."""
    E, K, N = w.shape
    return np.ascontiguousarray(w.reshape(E, K // 16, 16, N // 32, 32).transpose(0, 3, 1, 2, 4))


def check_gmm(oracle, x, w, ws, xs, gl, gl_type=0, bias=None, act_type=0, w_trans=False, out_dtype="bf16",
              scale_bf16=False, expect_exact=True, w_nz=False, api="V4", **api_kw):
    import ops_transformer_b200 as ops
    dev = _dev()
    M, K = x.shape
    E = w.shape[0]
    N = w.shape[2]
    gl = np.asarray(gl, np.int64)
    if scale_bf16:
        ws_bits = oracle.f32_to_bf16_bits(ws)
        ws_o = ws_bits
        ws_t = torch.from_numpy(ws_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    else:
        ws_o = ws
        ws_t = torch.from_numpy(ws).to(dev)
    w_o = np.ascontiguousarray(w.transpose(0, 2, 1)) if w_trans else w
    bias_t = None
    bias_o = None
    if bias is not None:
        if bias.dtype == np.int32:
            bias_o = bias
            bias_t = torch.from_numpy(bias).to(dev)
        else:  # bf16 bits
            bias_o = bias
            bias_t = torch.from_numpy(bias.view(np.int16)).to(dev).view(torch.bfloat16)
    ref = oracle.gmm_w8a8(x, w_o, ws_o, xs, gl, gl_type, bias=bias_o, act_type=act_type, w_trans=w_trans,
                          y_dtype=out_dtype, want_acc=True)
    xt = torch.from_numpy(x).to(dev)
    if w_trans:
        wt = torch.from_numpy(w_o).to(dev).transpose(1, 2)  # view [E, K, N] with strides (N*K, 1, K)
    elif w_nz:
        wt = torch.from_numpy(nd_to_nz(w)).to(dev)
        if api != "WeightNz":
            api_kw["weight_format"] = ops.ACL_FORMAT_FRACTAL_NZ
    else:
        wt = torch.from_numpy(w).to(dev)
    xst = torch.from_numpy(xs).to(dev) if xs is not None else None
    glt = torch.from_numpy(gl).to(dev)
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "int32": torch.int32}[out_dtype]
    sentinel = 0x7fc1 if out_dtype != "int32" else -123456789
    floating = out_dtype != "int32"
    if floating:
        out = torch.full((M, N), 0, dtype=torch.int16, device=dev)
        out.fill_(np.int16(np.uint16(sentinel).view(np.int16)).item())
        out = out.view(tdt)
    else:
        out = torch.full((M, N), sentinel, dtype=torch.int32, device=dev)
    y, wsb = ops.grouped_matmul_v4(xt, wt, ws_t if floating else None, xst if floating else None,
                                   glt, bias=bias_t, group_list_type=gl_type, act_type=act_type, out=out,
                                   out_dtype=tdt, return_workspace=True, api=api, **api_kw)
    ops.check_status(wsb)
    rs, rc = oracle.group_layout(gl[: E if E > 1 else 1], gl_type, M)
    covered = np.zeros(M, bool)
    for s, r in zip(rs, rc):
        covered[s:s + r] = True
    if out_dtype == "int32":
        got = y.cpu().numpy()
        assert np.array_equal(got[covered], ref["y"][covered]), "int32 accumulators differ"
        assert (got[~covered] == sentinel).all(), "rows outside group_list were written"
        return
    got_bits = _bf16_bits(y)
    if out_dtype == "f16":
        got = got_bits.view(np.float16).astype(np.float32)
        exp = ref["y"].view(np.float16).astype(np.float32)
    else:
        got = oracle.bf16_bits_to_f32(got_bits)
        exp = oracle.bf16_bits_to_f32(ref["y"])
    err = np.abs(got[covered] - exp[covered])
    assert (err <= BF16_ATOL + BF16_RTOL * np.abs(exp[covered])).all(), f"bf16 max err {err.max()}"
    assert (got_bits[~covered] == sentinel).all(), "rows outside group_list were written"
    if expect_exact:
        nbad = int(np.count_nonzero(got_bits[covered] != ref["y"][covered]))
        assert nbad == 0, f"{nbad} bf16 values are not bit-identical to the oracle"


def check_swiglu(oracle, x, w, ws, xs, gl, ws_dtype="f32", w_nz=False, api=""):
    import ops_transformer_b200 as ops
    dev = _dev()
    M, K = x.shape
    N = w.shape[2]
    H = N // 2
    gl = np.asarray(gl, np.int64)
    if ws_dtype == "bf16":
        bits = oracle.f32_to_bf16_bits(ws)
        ws_o = bits
        ws_t = torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)
    elif ws_dtype == "f16":
        ws_o = ws.astype(np.float16)
        ws_t = torch.from_numpy(ws_o).to(dev)
    else:
        ws_o = ws
        ws_t = torch.from_numpy(ws).to(dev)
    ref = oracle.swiglu_quant(x, w, ws_o, xs, gl)
    q0 = torch.full((M, H), -77, dtype=torch.int8, device=dev)
    qs0 = torch.full((M,), -5.0, dtype=torch.float32, device=dev)
    kw = {}
    if w_nz:
        wt = torch.from_numpy(nd_to_nz(w)).to(dev)
        kw["api"] = api
        if api != "WeightNZ":
            kw["weight_format"] = ops.ACL_FORMAT_FRACTAL_NZ
    else:
        wt = torch.from_numpy(w).to(dev)
    q, qs, wsb = ops.grouped_matmul_swiglu_quant(torch.from_numpy(x).to(dev), wt, ws_t,
                                                 torch.from_numpy(xs).to(dev), torch.from_numpy(gl).to(dev), output=q0,
                                                 output_scale=qs0, return_workspace=True, **kw)
    ops.check_status(wsb)
    rs, rc = oracle.group_layout(gl, 0, M)
    covered = np.zeros(M, bool)
    for s, r in zip(rs, rc):
        covered[s:s + r] = True
    qg, qsg = q.cpu().numpy(), qs.cpu().numpy()
    assert (qg[~covered] == -77).all() and (qsg[~covered] == -5.0).all(), "rows outside group_list were written"
    if covered.any():
        rel = np.abs(qsg[covered] - ref["q_scale"][covered]) / np.abs(ref["q_scale"][covered])
        assert rel.max() <= QSCALE_RTOL, f"q_scale max rel err {rel.max()}"
        d = np.abs(qg[covered].astype(np.int32) - ref["q"][covered].astype(np.int32))
        assert d.max() <= 1, f"int8 outputs differ by {d.max()} LSB"
        frac = np.count_nonzero(d) / d.size
        assert frac <= Q_LSB_FRACTION, f"{frac:.2e} of int8 outputs differ by 1 LSB"


# ----------------------------------------------------------------------------------------------------------
# grouped_matmul W8A8
# ----------------------------------------------------------------------------------------------------------

def test_gmm_single_tile_int32(oracle):
    x, w, ws, xs = make_inputs(128, 128, 256, 1, seed=1)
    check_gmm(oracle, x, w, ws, xs, [128], out_dtype="int32")


def test_gmm_single_tile_bf16(oracle):
    x, w, ws, xs = make_inputs(128, 128, 256, 1, seed=2)
    check_gmm(oracle, x, w, ws, xs, [128])


def test_gmm_single_tile_transposed_weight(oracle):
    x, w, ws, xs = make_inputs(128, 256, 256, 1, seed=3)
    check_gmm(oracle, x, w, ws, xs, [128], w_trans=True, out_dtype="int32")


@pytest.mark.parametrize("gl_type", [0, 1])
def test_gmm_config1_cpu_golden_case(oracle, gl_type):
    c = synth.CONFIGS["c1"]
    counts = np.asarray(c["counts"])
    x, w, ws, xs = make_inputs(int(counts.sum()), c["K"], c["N"], c["E"], seed=0)
    check_gmm(oracle, x, w, ws, xs, synth.group_list_from_counts(counts, gl_type), gl_type)
    check_gmm(oracle, x, w, ws, xs, synth.group_list_from_counts(counts, gl_type), gl_type, out_dtype="int32")


def test_gmm_ragged_groups_and_tails(oracle):
    counts = [0, 5, 130, 0, 1, 257]
    M = sum(counts) + 9  # 9 trailing rows not covered
    x, w, ws, xs = make_inputs(M, 144, 272, len(counts), seed=4)  # K and N not multiples of the tile
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0)
    check_gmm(oracle, x, w, ws, xs, counts, 1, out_dtype="int32")


def test_gmm_bf16_scale_reference_dtype_pair(oracle):
    # the reference's own aclnn case: x[84,5120] w[4,5120,2560], bf16 scale, group list {50,65,69,84}
    x, w, ws, xs = make_inputs(84, 5120, 2560, 4, seed=5)
    check_gmm(oracle, x, w, ws, xs, [50, 65, 69, 84], 0, scale_bf16=True)


def test_gmm_reference_kernel_ut_shapes(oracle):
    counts = [40, 40] + [20] * 14
    x, w, ws, xs = make_inputs(360, 1024, 8192, 16, seed=6)
    check_gmm(oracle, x, w, ws, xs, counts, 1, scale_bf16=True)
    x, w, ws, xs = make_inputs(360, 8192, 1024, 16, seed=7)
    check_gmm(oracle, x, w, ws, xs, counts, 1, scale_bf16=True)


def test_gmm_unaligned_shapes_take_the_cuda_core_path(oracle):
    # K=5, N=10 (not 16-byte aligned) are legal in the reference's kernel tests
    x, w, ws, xs = make_inputs(16, 5, 10, 2, seed=8)
    check_gmm(oracle, x, w, ws, xs, [8, 8], 1, scale_bf16=True)
    x, w, ws, xs = make_inputs(16, 10, 10, 2, seed=9)
    check_gmm(oracle, x, w, ws, xs, [8, 8], 1, act_type=1)


def test_gmm_bias_and_relu(oracle):
    counts = [70, 0, 200]
    x, w, ws, xs = make_inputs(270, 256, 512, 3, seed=10)
    b32 = np.random.default_rng(11).integers(-100000, 100000, size=(3, 512)).astype(np.int32)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, bias=b32)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, bias=b32, out_dtype="int32")
    bbf = oracle.f32_to_bf16_bits(np.random.default_rng(12).uniform(-50, 50, size=(3, 512)).astype(np.float32))
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, bias=bbf, act_type=1)


def test_gmm_transposed_weight_multi_group(oracle):
    counts = [100, 37, 300]
    x, w, ws, xs = make_inputs(437, 512, 768, 3, seed=13)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, w_trans=True)


def test_gmm_many_tiles_more_than_sms(oracle):
    counts = [513, 1000, 129, 0, 700]
    x, w, ws, xs = make_inputs(sum(counts), 256, 1024, 5, seed=14)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0)


def test_gmm_max_group_count(oracle):
    E = 1024
    counts = np.zeros(E, np.int64)
    counts[[0, 17, 500, 1023]] = [3, 129, 1, 64]
    x = synth.int8_tensor((int(counts.sum()), 128), 15, 1)
    w = synth.int8_tensor((E, 128, 32), 15, 2)
    ws = synth.scale_tensor((E, 32), 15, 3)
    xs = synth.scale_tensor((int(counts.sum()),), 15, 4)
    check_gmm(oracle, x, w, ws, xs, counts, 1)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0)


def test_gmm_row_scatter_extension(oracle):
    # result row r lands in row perm[r]: the un-permute after the down projection folded into the epilogue
    import ops_transformer_b200 as ops
    dev = _dev()
    counts = [150, 3, 200]
    M = sum(counts)
    x, w, ws, xs = make_inputs(M, 256, 528, 3, seed=16)
    gl = np.cumsum(counts)
    perm = np.random.default_rng(17).permutation(M).astype(np.int64)
    ref = oracle.gmm_w8a8(x, w, ws, xs, gl, 0)["y"]
    for dt, odt in ((torch.bfloat16, "bf16"), (torch.int32, "int32")):
        y = ops.grouped_matmul_v4(torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev),
                                  torch.from_numpy(ws).to(dev) if odt == "bf16" else None,
                                  torch.from_numpy(xs).to(dev) if odt == "bf16" else None, torch.from_numpy(gl).to(dev),
                                  out_dtype=dt, out_row_index=torch.from_numpy(perm).to(dev))
        torch.cuda.synchronize()
        if odt == "bf16":
            got = _bf16_bits(y)
            assert np.array_equal(got[perm], ref)
        else:
            refi = oracle.gmm_w8a8(x, w, ws, xs, gl, 0, y_dtype="int32")["y"]
            assert np.array_equal(y.cpu().numpy()[perm], refi)


# ----------------------------------------------------------------------------------------------------------
# grouped_matmul_swiglu_quant
# ----------------------------------------------------------------------------------------------------------

def test_swiglu_reference_small_case(oracle):
    # m=16, k=256, n=512, e=4 (the reference's kernel unit test shape)
    x, w, ws, xs = make_inputs(16, 256, 512, 4, seed=20)
    check_swiglu(oracle, x, w, ws, xs, [4, 8, 12, 16])


def test_swiglu_reference_api_case(oracle):
    x, w, ws, xs = make_inputs(192, 2048, 2048, 4, seed=21)
    check_swiglu(oracle, x, w, ws, xs, [24, 48, 72, 96])  # rows 96.. stay untouched


def test_swiglu_config1_shape(oracle):
    x, w, ws, xs = make_inputs(256, 1024, 2048, 4, seed=0)
    check_swiglu(oracle, x, w, ws, xs, np.cumsum([64, 32, 96, 64]))


def test_swiglu_ragged_empty_groups_short_list(oracle):
    counts = [0, 3, 0, 131, 260]
    x, w, ws, xs = make_inputs(sum(counts) + 5, 144, 608, 8, seed=22)  # list shorter than E, K/N tails
    check_swiglu(oracle, x, w, ws, xs, np.cumsum(counts))


@pytest.mark.parametrize("ws_dtype", ["bf16", "f16"])
def test_swiglu_half_precision_weight_scale(oracle, ws_dtype):
    x, w, ws, xs = make_inputs(200, 512, 1024, 2, seed=23)
    check_swiglu(oracle, x, w, ws, xs, [120, 200], ws_dtype=ws_dtype)


def test_swiglu_unaligned_takes_cuda_core_path(oracle):
    x, w, ws, xs = make_inputs(20, 24, 36, 2, seed=24)
    check_swiglu(oracle, x, w, ws, xs, [7, 20])


def test_swiglu_deepseek_width_few_rows(oracle):
    # decode-like: full K=7168 / N=4096 with a handful of rows per expert, some experts empty
    counts = [3, 0, 17, 1, 0, 40]
    x, w, ws, xs = make_inputs(sum(counts), 7168, 4096, 6, seed=25)
    check_swiglu(oracle, x, w, ws, xs, np.cumsum(counts))


def test_swiglu_many_row_blocks_and_tiles(oracle):
    # more tiles than SMs and several row blocks per expert: exercises the row-block completion counters
    counts = [700, 0, 1300, 129, 512]
    x, w, ws, xs = make_inputs(sum(counts) + 3, 256, 2048, 5, seed=27)
    check_swiglu(oracle, x, w, ws, xs, np.cumsum(counts))


def test_swiglu_repeated_calls_reuse_workspace(oracle):
    # the same workspace is used by consecutive calls of different shapes; counters and maxima must be reset
    x, w, ws, xs = make_inputs(400, 384, 1024, 3, seed=28)
    check_swiglu(oracle, x, w, ws, xs, [100, 250, 400])
    x, w, ws, xs = make_inputs(90, 128, 512, 2, seed=29)
    check_swiglu(oracle, x, w, ws, xs, [40, 90])
    x, w, ws, xs = make_inputs(400, 384, 1024, 3, seed=30)
    check_swiglu(oracle, x, w, ws, xs, [10, 20, 390])


def test_gmm_deepseek_down_width_few_rows(oracle):
    counts = [3, 0, 17, 1, 0, 40]
    x, w, ws, xs = make_inputs(sum(counts), 2048, 7168, 6, seed=26)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0)


# ----------------------------------------------------------------------------------------------------------
# FRACTAL_NZ weights, the V5 / WeightNz / WeightNZ entry points, float16 results, activations
# ----------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("ctas", ["1", "2"])
def test_gmm_fractal_nz_weight(oracle, monkeypatch, ctas):
    monkeypatch.setenv("GMM_B200_CTAS", ctas)
    counts = [0, 5, 130, 0, 1, 600]
    x, w, ws, xs = make_inputs(sum(counts) + 9, 144, 288, len(counts), seed=40)  # K and N tails inside the NZ boxes
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, w_nz=True)
    check_gmm(oracle, x, w, ws, xs, counts, 1, w_nz=True, out_dtype="int32")
    check_gmm(oracle, x, w, ws, xs, counts, 1, w_nz=True, api="WeightNz", tuning_config=[128], quant_group_size=0)


def test_gmm_fractal_nz_deep_k(oracle):
    counts = [300, 40, 513]
    x, w, ws, xs = make_inputs(sum(counts), 2048, 1024, 3, seed=41)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, w_nz=True, scale_bf16=True)


def test_gmm_fractal_nz_cuda_core_path(oracle):
    # the smallest legal FRACTAL_NZ weight: one 16 x 32 fractal per expert
    x, w, ws, xs = make_inputs(24, 16, 32, 2, seed=42)
    check_gmm(oracle, x, w, ws, xs, [10, 24], 0, w_nz=True)


def test_gmm_v5_tuning_config(oracle):
    counts = [100, 37, 300]
    x, w, ws, xs = make_inputs(437, 512, 768, 3, seed=43)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, api="V5", tuning_config=[146])
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, api="V5", tuning_config=[512])   # the hint selects CTA pairs
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, api="V5")


def test_gmm_float16_result(oracle):
    counts = [70, 0, 200, 3]
    x, w, ws, xs = make_inputs(sum(counts) + 2, 256, 528, 4, seed=44)
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, out_dtype="f16")
    bbf = oracle.f32_to_bf16_bits(np.random.default_rng(45).uniform(-5, 5, size=(4, 528)).astype(np.float32))
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, out_dtype="f16", bias=bbf, act_type=1)


@pytest.mark.parametrize("act_type", [2, 4, 5])
def test_gmm_activations(oracle, act_type):
    # GELU (tanh form), fast GELU, SiLU: expf differs by an ulp between libm and the GPU, so bit identity is not asked
    counts = [70, 0, 200]
    x, w, ws, xs = make_inputs(270, 256, 512, 3, seed=46 + act_type)
    ws = (ws * 0.3).astype(np.float32)  # keeps many values inside the curved part of the activations
    check_gmm(oracle, x, w, ws, xs, np.cumsum(counts), 0, act_type=act_type, expect_exact=False)
    x, w, ws, xs = make_inputs(16, 10, 10, 2, seed=50 + act_type)  # CUDA-core path
    check_gmm(oracle, x, w, ws, xs, [8, 8], 1, act_type=act_type, expect_exact=False)


@pytest.mark.parametrize("ctas", ["1", "2"])
@pytest.mark.parametrize("api", ["", "WeightNZ"])
def test_swiglu_fractal_nz_weight(oracle, monkeypatch, ctas, api):
    monkeypatch.setenv("GMM_B200_CTAS", ctas)
    counts = [0, 3, 0, 131, 600]
    x, w, ws, xs = make_inputs(sum(counts) + 5, 144, 576, 8, seed=55)  # list shorter than E, K/N tails
    check_swiglu(oracle, x, w, ws, xs, np.cumsum(counts), w_nz=True, api=api)


def test_swiglu_fractal_nz_reference_api_case(oracle):
    # the reference's WeightNZ example: E=4, M=192 (96 covered), K=2048, N=2048
    x, w, ws, xs = make_inputs(192, 2048, 2048, 4, seed=56)
    check_swiglu(oracle, x, w, ws, xs, [24, 48, 72, 96], w_nz=True, api="WeightNZ")


def test_swiglu_fractal_nz_n_multiple_of_32_only(oracle):
    # N = 96: N/2 = 48 is not a multiple of 32, the tensor-core path declines and the CUDA-core kernel runs
    x, w, ws, xs = make_inputs(20, 32, 96, 2, seed=57)
    check_swiglu(oracle, x, w, ws, xs, [7, 20], w_nz=True)


# ----------------------------------------------------------------------------------------------------------
# grouped_matmul_finalize_routing (down GEMM + weighted combine)
# ----------------------------------------------------------------------------------------------------------

def check_finalize(oracle, M, K, N, E, counts, topk, seed, *, shared_rows=0, shared_offset=0, shared_weight=1.0, use_logit=True,
                   use_bias=False, use_pts=True, idx32=False, scale_bf16=False, api="", flat_layout=None, view_3d=True,
                   batch=None, y_misaligned=False):
    """fp32 sums of up to topk + 1 terms in an order that differs from the oracle's: every element must lie within
    4 ulp-sized steps of the sum of magnitudes (4 * 2^-23 * abs_sum) of the oracle's value."""
    import ops_transformer_b200 as ops
    dev = _dev()
    rng = np.random.default_rng(seed)
    x, w, ws, xs = make_inputs(M, K, N, E, seed=seed)
    if batch is None:
        batch = M // topk
    scatter = use_logit
    ri = (rng.permutation(M) % batch).astype(np.int64) if scatter else rng.permutation(M)[:M].astype(np.int64)
    logit = rng.uniform(0.05, 0.6, size=M).astype(np.float32) if use_logit else None
    shared = oracle.f32_to_bf16_bits(rng.uniform(-40, 40, size=(shared_rows, N)).astype(np.float32)) if scatter else None
    bias = oracle.f32_to_bf16_bits(rng.uniform(-20, 20, size=(E, N)).astype(np.float32)) if use_bias else None
    gl = np.asarray(counts, np.int64)
    ws_o = oracle.f32_to_bf16_bits(ws) if scale_bf16 else ws
    y_rows = batch if scatter else M
    y0 = np.full((y_rows, N), 3.5, np.float32)
    ref = oracle.gmm_finalize_routing(x, w, ws_o, xs if use_pts else None, gl, ri.astype(np.int32) if idx32 else ri, y_rows, bias=bias,
                                      shared_input=shared, shared_offset=shared_offset, shared_weight=shared_weight, logit=logit,
                                      y_init=y0)
    t = lambda a: None if a is None else torch.from_numpy(a).to(dev)  # noqa: E731
    bf = lambda a: None if a is None else torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)  # noqa: E731
    ws_t = bf(ws_o) if scale_bf16 else t(ws)
    out = torch.from_numpy(y0).to(dev)
    if y_misaligned:  # a result that starts 4 bytes into an allocation: 4-byte but not 16-byte aligned
        flat = torch.empty(y0.size + 4, dtype=torch.float32, device=dev)
        out = flat[1:1 + y0.size].view(y_rows, N)
        out.copy_(torch.from_numpy(y0))
        assert out.data_ptr() % 16 == 4
    ri_t = t(ri.astype(np.int32)) if idx32 else t(ri)
    kw = dict(bias=bf(bias), pertoken_scale=t(xs) if use_pts else None, shared_input=bf(shared), logit=t(logit),
              shared_input_weight=shared_weight, shared_input_offset=shared_offset)
    if flat_layout is None:
        y, wsb = ops.grouped_matmul_finalize_routing(t(x), t(nd_to_nz(w)), ws_t, t(gl), ri_t, y_rows, out=out, api=api, view_3d=view_3d,
                                                     return_workspace=True, **kw)
        ops.check_status(wsb)
    else:
        wt = t(nd_to_nz(w)) if flat_layout == 2 else t(w)
        y = ops.grouped_matmul_finalize_routing_flat(t(x), wt, flat_layout, ws_t, t(gl), ri_t, out, **kw)
        torch.cuda.synchronize()
    got = y.cpu().numpy()
    tol = 4 * 2.0 ** -23 * ref["abs_sum"] + 1e-30
    err = np.abs(got.astype(np.float64) - ref["y"].astype(np.float64))
    assert (err <= tol).all(), f"max excess {float((err - tol).max())}"
    if not scatter:  # rows nobody wrote keep their contents
        covered = np.zeros(M, bool)
        covered[ri[: int(gl.sum())]] = True
        assert (got[~covered] == 3.5).all()


@pytest.mark.parametrize("ctas", ["1", "2"])
def test_finalize_routing_reference_example_shape(oracle, monkeypatch, ctas):
    # the reference's example: m=192, k=2048, n=7168, e=4, batch=24 (top-8), 8 shared rows
    monkeypatch.setenv("GMM_B200_CTAS", ctas)
    check_finalize(oracle, 192, 2048, 7168, 4, [48, 40, 64, 40], 8, 60, shared_rows=8, shared_offset=4, shared_weight=0.5)


@pytest.mark.parametrize("ctas", ["1", "2"])
def test_finalize_routing_ragged_groups_bias_int32_index(oracle, monkeypatch, ctas):
    monkeypatch.setenv("GMM_B200_CTAS", ctas)
    counts = [0, 5, 530, 0, 1, 260]          # 4 trailing rows in no group; tails in both tile sizes
    check_finalize(oracle, sum(counts) + 4, 144, 288, 6, counts, 4, 61, shared_rows=50, shared_offset=10, use_bias=True, idx32=True,
                   scale_bf16=True, api="V2")


def test_finalize_routing_without_per_token_scale_and_5d_view(oracle):
    check_finalize(oracle, 256, 256, 512, 3, [100, 56, 100], 2, 62, shared_rows=128, use_pts=False, view_3d=False)


def test_finalize_routing_plain_store_scene(oracle):
    # neither shared input nor logits: rows are stored at row_index, nothing is initialised
    check_finalize(oracle, 300, 256, 512, 3, [100, 37, 150], 1, 63, use_logit=False)
    check_finalize(oracle, 300, 256, 512, 3, [100, 37, 150], 1, 64, use_logit=False, use_bias=True, idx32=True)


@pytest.mark.parametrize("layout", [0, 2])
def test_finalize_routing_flat_entry_point(oracle, layout):
    check_finalize(oracle, 512, 512, 1024, 4, [128, 200, 0, 184], 8, 65, shared_rows=64, flat_layout=layout, use_bias=True)


def test_finalize_routing_result_view_not_16_byte_aligned(oracle):
    # the tensor-core path needs 16-byte aligned rows; such a view takes the CUDA-core kernels, including the scalar
    # initialisation of the result
    check_finalize(oracle, 96, 128, 256, 2, [40, 56], 4, 67, shared_rows=16, shared_offset=3, y_misaligned=True)


def test_finalize_routing_batch_smaller_than_rows_per_token(oracle):
    # many rows per destination: 64 destinations for 1024 rows (16 atomics per element)
    check_finalize(oracle, 1024, 128, 256, 2, [500, 524], 16, 66, shared_rows=64, shared_weight=2.0)


# ----------------------------------------------------------------------------------------------------------
# moe_init_routing_v3 (producer of the path's inputs): every output is integer or exactly rounded, so bit-exact
# ----------------------------------------------------------------------------------------------------------

def check_init_routing(oracle, n, k, h, E, rng_, seed, *, quant=True, x_kind="bf16", smooth=False, row_idx_type=1, count_type=1,
                       per_token_scale=False, zero_row=True):
    import ops_transformer_b200 as ops
    dev = _dev()
    rng = np.random.default_rng(seed)
    xf = (rng.standard_normal((n, h)) * rng.uniform(0.1, 4.0, size=(n, 1))).astype(np.float32)
    if zero_row and n > 2:
        xf[2] = 0.0
    idx = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    if x_kind == "bf16":
        x_o = oracle.f32_to_bf16_bits(xf)
        x_t = torch.from_numpy(x_o.view(np.int16)).to(dev).view(torch.bfloat16)
    elif x_kind == "f16":
        x_o = xf.astype(np.float16)
        x_t = torch.from_numpy(x_o).to(dev)
    elif x_kind == "int8":
        x_o = rng.integers(-127, 128, size=(n, h)).astype(np.int8)
        x_t = torch.from_numpy(x_o).to(dev)
    else:
        x_o = xf
        x_t = torch.from_numpy(xf).to(dev)
    sc = None
    if smooth:
        sc = rng.uniform(0.5, 2.0, size=(rng_[1] - rng_[0], h)).astype(np.float32)
    elif per_token_scale:
        sc = rng.uniform(0.5, 2.0, size=(n,)).astype(np.float32)
    ref = oracle.moe_init_routing_v3(x_o, idx, E, rng_, quant, row_idx_type=row_idx_type, count_type=count_type, scale=sc)
    rows = ref["rows"]
    ex = torch.full((n * k, h), -77, dtype=torch.int8, device=dev) if quant else torch.zeros((n * k, h), dtype=x_t.dtype, device=dev)
    ri = torch.full((n * k,), -9, dtype=torch.int32, device=dev)
    cnt = torch.full(ref["counts"].shape, -9, dtype=torch.int64, device=dev)
    es = torch.full((n * k,), -5.0, dtype=torch.float32, device=dev)
    ops.moe_init_routing_v3(x_t, torch.from_numpy(idx).to(dev), expert_num=E, active_expert_range=rng_, quant_mode=1 if quant else -1,
                            scale=None if sc is None else torch.from_numpy(sc).to(dev), expert_tokens_num_type=count_type,
                            row_idx_type=row_idx_type, outputs=(ex, ri, cnt, es))
    torch.cuda.synchronize()
    assert np.array_equal(cnt.cpu().numpy(), ref["counts"])
    assert np.array_equal(ri.cpu().numpy(), ref["expanded_row_idx"])
    got = ex.view(torch.int16).cpu().numpy().view(np.uint16) if x_kind == "bf16" and not quant else ex.cpu().numpy()
    assert np.array_equal(got, ref["expanded_x"]), "expanded rows differ"
    if quant or sc is not None:
        assert np.array_equal(es.cpu().numpy(), ref["expanded_scale"])
    return rows


def test_init_routing_dynamic_quant_deepseek_width(oracle):
    rows = check_init_routing(oracle, 96, 8, 7168, 256, (0, 256), 70)
    assert rows == 96 * 8


def test_init_routing_active_range_smooth_scale_and_gather_index(oracle):
    check_init_routing(oracle, 300, 4, 512, 64, (16, 48), 71, smooth=True, row_idx_type=0, count_type=2)
    check_init_routing(oracle, 300, 4, 512, 64, (16, 48), 72, smooth=True, x_kind="f32")
    check_init_routing(oracle, 5, 2, 20, 8, (1, 8), 73, x_kind="f16", row_idx_type=0)      # h not a multiple of 4


def test_init_routing_many_blocks_keep_pair_order(oracle):
    # 40000 pairs = 40 blocks of 1024: the order of equal experts must hold across warps and blocks
    check_init_routing(oracle, 5000, 8, 64, 32, (0, 32), 74)
    check_init_routing(oracle, 5000, 8, 64, 2048, (100, 1900), 75, count_type=2)
    check_init_routing(oracle, 4000, 8, 64, 256, (3, 250), 80, count_type=2)   # scan folded into the scatter kernel, key-value counts
    check_init_routing(oracle, 9000, 8, 64, 256, (0, 256), 79, count_type=2)   # table too large for the folded scan
    check_init_routing(oracle, 9000, 8, 64, 32, (1, 31), 82, count_type=2)     # folded scan over 71 blocks


def test_init_routing_without_quantisation(oracle):
    check_init_routing(oracle, 200, 4, 256, 32, (0, 32), 76, quant=False, per_token_scale=True)
    check_init_routing(oracle, 200, 4, 256, 32, (4, 20), 77, quant=False, x_kind="int8", row_idx_type=0)
    check_init_routing(oracle, 64, 2, 100, 16, (0, 16), 78, quant=False, x_kind="f32")


def test_init_routing_feeds_the_grouped_gemms(oracle):
    # bf16 tokens -> init routing (int8 rows, scales, counts) -> swiglu_quant -> finalize routing back to token order
    import ops_transformer_b200 as ops
    dev = _dev()
    rng = np.random.default_rng(79)
    n, k, h, inter, E = 64, 4, 512, 256, 8
    xf = rng.standard_normal((n, h)).astype(np.float32)
    xb = oracle.f32_to_bf16_bits(xf)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    w1 = synth.int8_tensor((E, h, 2 * inter), 79, 2)
    s1 = synth.scale_tensor((E, 2 * inter), 79, 3)
    w2 = synth.int8_tensor((E, inter, h), 79, 5)
    s2 = synth.scale_tensor((E, h), 79, 6)
    logit = rng.uniform(0.1, 0.4, size=(n, k)).astype(np.float32)
    # oracle chain
    r = oracle.moe_init_routing_v3(xb, idx, E, (0, E), True, row_idx_type=1)
    gl = np.cumsum(r["counts"])
    a = oracle.swiglu_quant(r["expanded_x"], w1, s1, r["expanded_scale"], gl)
    pair = r["expanded_row_idx"]
    fin = oracle.gmm_finalize_routing(a["q"], w2, s2, a["q_scale"], r["counts"], (pair // k).astype(np.int64), n,
                                      shared_input=oracle.f32_to_bf16_bits(np.zeros((n, h), np.float32)), logit=logit.ravel()[pair])
    # GPU chain
    t = lambda v: torch.from_numpy(v).to(dev)  # noqa: E731
    ex, ri, cnt, es = ops.moe_init_routing_v3(torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16), t(idx), expert_num=E,
                                              active_expert_range=(0, E), quant_mode=1)
    q, qs = ops.grouped_matmul_swiglu_quant(ex, t(w1), t(s1), es, torch.cumsum(cnt, 0))
    tok = torch.div(ri, k, rounding_mode="floor").to(torch.int64)
    y = ops.grouped_matmul_finalize_routing(q, t(nd_to_nz(w2)), t(s2), cnt, tok, n, pertoken_scale=qs,
                                            shared_input=torch.zeros((n, h), dtype=torch.bfloat16, device=dev),
                                            logit=t(logit.ravel())[ri.to(torch.int64)])
    torch.cuda.synchronize()
    assert np.array_equal(ex.cpu().numpy(), r["expanded_x"]) and np.array_equal(cnt.cpu().numpy(), r["counts"])
    d = np.abs(q.cpu().numpy().astype(np.int32) - a["q"].astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) <= max(1, int(1e-4 * d.size))
    err = np.abs(y.cpu().numpy().astype(np.float64) - fin["y"])
    # a 1-LSB difference of the int8 intermediate moves an output by about one part in 127 of a term
    assert (err <= 4 * 2.0 ** -23 * fin["abs_sum"] + (np.count_nonzero(d) > 0) * 2e-2 * fin["abs_sum"]).all()


# ----------------------------------------------------------------------------------------------------------
# non-contiguous views: inputs are made contiguous inside the executor, results are copied back into strided outputs
# ----------------------------------------------------------------------------------------------------------

def _strided(tensor_2d):
    """The same values as a view over every second column of a wider buffer."""
    wide = torch.empty((tensor_2d.shape[0], 2 * tensor_2d.shape[1]), dtype=tensor_2d.dtype, device=tensor_2d.device)
    view = wide[:, ::2]
    view.copy_(tensor_2d)
    assert not view.is_contiguous()
    return view


def test_strided_views_grouped_matmul(oracle):
    import ops_transformer_b200 as ops
    dev = _dev()
    counts = [70, 0, 200]
    M = sum(counts) + 6
    x, w, ws, xs = make_inputs(M, 256, 512, 3, seed=80)
    gl = np.cumsum(counts)
    ref = oracle.gmm_w8a8(x, w, ws, xs, gl, 0)["y"]
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    out_wide = torch.full((M, 1024), 0x7fc1, dtype=torch.int16, device=dev)
    out = out_wide.view(torch.bfloat16)[:, ::2]
    xs_wide = torch.zeros((M, 3), dtype=torch.float32, device=dev)
    xs_wide[:, 1] = t(xs)
    y, wsb = ops.grouped_matmul_v4(_strided(t(x)), t(w), _strided(t(ws)), xs_wide[:, 1], t(gl), out=out, return_workspace=True)
    ops.check_status(wsb)
    bits = out_wide.cpu().numpy().view(np.uint16)
    rows = sum(counts)
    assert np.array_equal(bits[:rows, ::2], ref[:rows])
    assert (bits[rows:, ::2] == 0x7fc1).all(), "rows outside group_list must keep their contents"
    assert (bits[:, 1::2] == 0x7fc1).all(), "the gaps of the strided output must not be written"


def test_strided_views_swiglu_quant(oracle):
    import ops_transformer_b200 as ops
    dev = _dev()
    x, w, ws, xs = make_inputs(200, 256, 1024, 2, seed=81)
    gl = np.array([120, 190], np.int64)
    ref = oracle.swiglu_quant(x, w, ws, xs, gl)
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    q_wide = torch.full((200, 1024), -77, dtype=torch.int8, device=dev)
    qs_wide = torch.full((200, 2), -5.0, dtype=torch.float32, device=dev)
    _, _, wsb = ops.grouped_matmul_swiglu_quant(_strided(t(x)), t(w), t(ws), t(xs), t(gl), output=q_wide[:, ::2], output_scale=qs_wide[:, 0],
                                                return_workspace=True)
    ops.check_status(wsb)
    qg, qsg = q_wide.cpu().numpy(), qs_wide.cpu().numpy()
    rel = np.abs(qsg[:190, 0] - ref["q_scale"][:190]) / ref["q_scale"][:190]
    d = np.abs(qg[:190, ::2].astype(np.int32) - ref["q"][:190].astype(np.int32))
    assert rel.max() <= QSCALE_RTOL and d.max() <= 1 and np.count_nonzero(d) / d.size <= Q_LSB_FRACTION
    assert (qg[190:] == -77).all() and (qg[:, 1::2] == -77).all() and (qsg[190:] == -5.0).all() and (qsg[:, 1] == -5.0).all()


def test_strided_views_init_routing(oracle):
    import ops_transformer_b200 as ops
    dev = _dev()
    rng = np.random.default_rng(82)
    n, k, h, E = 50, 2, 64, 8
    xb = oracle.f32_to_bf16_bits(rng.standard_normal((n, h)).astype(np.float32))
    idx = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    ref = oracle.moe_init_routing_v3(xb, idx, E, (0, E), True)
    x_t = _strided(torch.from_numpy(xb.view(np.int16)).to(dev).view(torch.bfloat16))
    idx_t = _strided(torch.from_numpy(idx).to(dev))
    ex_wide = torch.full((n * k, 2 * h), -77, dtype=torch.int8, device=dev)
    ri = torch.empty((n * k,), dtype=torch.int32, device=dev)
    cnt = torch.empty((E,), dtype=torch.int64, device=dev)
    es = torch.empty((n * k,), dtype=torch.float32, device=dev)
    ops.moe_init_routing_v3(x_t, idx_t, expert_num=E, active_expert_range=(0, E), quant_mode=1, outputs=(ex_wide[:, ::2], ri, cnt, es))
    torch.cuda.synchronize()
    got = ex_wide.cpu().numpy()
    assert np.array_equal(got[:, ::2], ref["expanded_x"]) and (got[:, 1::2] == -77).all()
    assert np.array_equal(ri.cpu().numpy(), ref["expanded_row_idx"]) and np.array_equal(es.cpu().numpy(), ref["expanded_scale"])


# ----------------------------------------------------------------------------------------------------------
# the committed golden fixtures, straight through the C ABI (no oracle involved)
# ----------------------------------------------------------------------------------------------------------

def test_golden_fixtures_on_the_gpu():
    import json
    import os

    import ops_transformer_b200 as ops
    dev = _dev()
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    with open(os.path.join(golden, "manifest.json")) as f:
        manifest = json.load(f)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    bf = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.bfloat16)  # noqa: E731
    seen = set()
    for case in manifest["cases"]:
        d = np.load(os.path.join(golden, case["file"]))
        seen.add(case["op"])
        if case["op"] == "moe_init_routing_v3":
            n, k, h, E = case["n"], case["k"], case["h"], case["E"]
            fill = case["fill"]
            outs = (torch.full((n * k, h), fill["expanded_x"], dtype=torch.int8, device=dev),
                    torch.full((n * k,), fill["expanded_row_idx"], dtype=torch.int32, device=dev),
                    torch.full(d["counts"].shape, fill["counts"], dtype=torch.int64, device=dev),
                    torch.full((n * k,), fill["expanded_scale"], dtype=torch.float32, device=dev))
            ops.moe_init_routing_v3(bf(d["x_bf16_bits"]), t(d["expert_idx"]), expert_num=E, active_expert_range=tuple(case["active_range"]),
                                    quant_mode=1, scale=t(d["scale"]), expert_tokens_num_type=case["count_type"],
                                    row_idx_type=case["row_idx_type"], outputs=outs)
            torch.cuda.synchronize()
            for got, key in zip(outs, ("expanded_x", "expanded_row_idx", "counts", "expanded_scale")):
                assert np.array_equal(got.cpu().numpy(), d[key]), (case["file"], key)
            continue
        if case["op"] == "ep_combine":
            import ctypes as C

            from ops_transformer_b200 import _lib
            y_dev, rows_dev, w_dev = bf(d["y_bf16_bits"]), t(d["pair_row"]), t(d["weights"])
            out = torch.full((case["tokens"], case["h"]), -1.0, dtype=torch.bfloat16, device=dev)
            p = lambda a: C.c_void_p(a.data_ptr())  # noqa: E731
            rc = _lib.lib().gmmB200EpCombine(p(y_dev), p(rows_dev), p(w_dev), p(out), case["tokens"], case["k"], case["h"], case["rows"],
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
            torch.cuda.synchronize()
            assert np.array_equal(_bf16_bits(out), d["out_bf16_bits"]), case["file"]
            continue
        x, w, ws, xs, gl = d["x"], d["w"], d["w_scale"], d["x_scale"], d["group_list"]
        if case["op"] == "grouped_matmul_finalize_routing":
            y = ops.grouped_matmul_finalize_routing(t(x), t(nd_to_nz(w)), t(ws), t(gl), t(d["row_index"]), case["batch"],
                                                    bias=bf(d["bias_bf16_bits"]), pertoken_scale=t(xs), shared_input=bf(d["shared_bf16_bits"]),
                                                    logit=t(d["logit"]), shared_input_weight=case["shared_weight"],
                                                    shared_input_offset=case["shared_offset"])
            torch.cuda.synchronize()
            err = np.abs(y.cpu().numpy().astype(np.float64) - d["y"])
            assert (err <= 4 * 2.0 ** -23 * d["abs_sum"] + 1e-30).all(), case["file"]
        elif case["op"] == "grouped_matmul":
            glt = int(case["group_list_type"])
            y = ops.grouped_matmul_v4(t(x), t(w), t(ws), t(xs), t(gl), group_list_type=glt)
            acc = ops.grouped_matmul_v4(t(x), t(w), None, None, t(gl), group_list_type=glt, out_dtype=torch.int32)
            torch.cuda.synchronize()
            rows = int(gl[-1]) if glt == 0 else int(gl.sum())
            assert np.array_equal(acc.cpu().numpy()[:rows], d["acc"][:rows]), case["file"]
            assert np.array_equal(_bf16_bits(y)[:rows], d["y_bf16_bits"][:rows]), case["file"]
        else:
            q, qs = ops.grouped_matmul_swiglu_quant(t(x), t(w), t(ws), t(xs), t(gl))
            torch.cuda.synchronize()
            rows = int(gl[-1])
            rel = np.abs(qs.cpu().numpy()[:rows] - d["q_scale"][:rows]) / d["q_scale"][:rows]
            dd = np.abs(q.cpu().numpy()[:rows].astype(np.int32) - d["q"][:rows].astype(np.int32))
            assert rel.max() <= QSCALE_RTOL and dd.max() <= 1 and np.count_nonzero(dd) <= max(1, int(Q_LSB_FRACTION * dd.size)), case["file"]
    assert seen == {"grouped_matmul", "grouped_matmul_swiglu_quant", "moe_init_routing_v3", "grouped_matmul_finalize_routing",
                    "ep_combine"}


def test_host_pipelined_pieces_equal_the_whole_call(oracle):
    # rows in pinned host memory, the call split by experts into a copy-in / operator / copy-out pipeline
    import ops_transformer_b200 as ops
    from ops_transformer_b200.hostio import HostPipelinedGroupedOp
    dev = _dev()
    counts = np.array([100, 0, 37, 300, 5, 64, 0, 129])
    M = int(counts.sum())
    x, w, ws, xs = make_inputs(M, 256, 512, len(counts), seed=90)
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    hx, hxs = torch.from_numpy(x).pin_memory(), torch.from_numpy(xs).pin_memory()
    for op in ("swiglu_quant", "gmm"):
        pipe = HostPipelinedGroupedOp(op, t(w), t(ws), M, pieces=3)
        if op == "swiglu_quant":
            h0 = torch.zeros((M, 256), dtype=torch.int8).pin_memory()
            h1 = torch.zeros((M,), dtype=torch.float32).pin_memory()
            pipe.run(hx, hxs, counts, h0, h1)
            q, qs = ops.grouped_matmul_swiglu_quant(t(x), t(w), t(ws), t(xs), t(np.cumsum(counts)))
            torch.cuda.synchronize()
            assert np.array_equal(h1.numpy(), qs.cpu().numpy())
            d = np.abs(h0.numpy().astype(np.int32) - q.cpu().numpy().astype(np.int32))
            assert d.max() <= 1 and np.count_nonzero(d) <= max(1, int(Q_LSB_FRACTION * d.size))
            ref = oracle.swiglu_quant(x, w, ws, xs, np.cumsum(counts))
            assert np.abs(h1.numpy() - ref["q_scale"]).max() <= QSCALE_RTOL * ref["q_scale"].max()
        else:
            h0 = torch.zeros((M, 512), dtype=torch.bfloat16).pin_memory()
            pipe.run(hx, hxs, counts, h0)
            ref = oracle.gmm_w8a8(x, w, ws, xs, np.cumsum(counts), 0)["y"]
            assert np.array_equal(h0.view(torch.int16).numpy().view(np.uint16), ref)
    # the same pipeline over a FRACTAL_NZ weight (the 5-D storage is sliced by experts like the 3-D one)
    pipe = HostPipelinedGroupedOp("swiglu_quant", ops.format_cast_nz(t(w)), t(ws), M, pieces=3)
    h0 = torch.zeros((M, 256), dtype=torch.int8).pin_memory()
    h1 = torch.zeros((M,), dtype=torch.float32).pin_memory()
    pipe.run(hx, hxs, counts, h0, h1)
    q, qs = ops.grouped_matmul_swiglu_quant(t(x), t(w), t(ws), t(xs), t(np.cumsum(counts)))
    torch.cuda.synchronize()
    assert np.array_equal(h1.numpy(), qs.cpu().numpy()) and np.array_equal(h0.numpy(), q.cpu().numpy())


# ----------------------------------------------------------------------------------------------------------
# seeded random sweep over shapes, group lists, layouts, tile shapes and options
# ----------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_sweep_of_shapes_and_options(oracle, monkeypatch, seed):
    rng = np.random.default_rng(seed)
    for it in range(25):
        E = int(rng.integers(1, 12))
        K = int(rng.choice([16, 48, 128, 144, 256, 512, 1040]))
        N = int(rng.choice([32, 64, 96, 256, 288, 512, 1056]))
        counts = rng.integers(0, int(rng.choice([3, 140, 300, 700])), size=E).astype(np.int64)
        counts[rng.random(E) < 0.3] = 0
        if counts.sum() == 0:
            counts[0] = 5
        M = int(counts.sum()) + int(rng.integers(0, 7))
        x, w, ws, xs = make_inputs(M, K, N, E, seed=1000 * seed + it)
        monkeypatch.setenv("GMM_B200_CTAS", str(rng.choice(["1", "2"])))
        monkeypatch.setenv("GMM_B200_HYBRID", str(rng.choice(["0", "1"])))
        gl_type = int(rng.integers(0, 2))
        gl = counts if gl_type == 1 else np.cumsum(counts)
        nz = bool(rng.random() < 0.4)
        mode = str(rng.choice(["gmm", "gmm_i32", "gmm_f16", "swiglu", "finalize"]))
        if mode == "gmm":
            bias = rng.integers(-1000, 1000, size=(E, N)).astype(np.int32) if rng.random() < 0.3 else None
            check_gmm(oracle, x, w, ws, xs, gl, gl_type, w_nz=nz, bias=bias, act_type=int(rng.choice([0, 1])),
                      w_trans=(not nz and rng.random() < 0.3))
        elif mode == "gmm_i32":
            check_gmm(oracle, x, w, ws, xs, gl, gl_type, w_nz=nz, out_dtype="int32")
        elif mode == "gmm_f16":
            check_gmm(oracle, x, w, ws, xs, gl, gl_type, w_nz=nz, out_dtype="f16")
        elif mode == "swiglu":
            check_swiglu(oracle, x, w, ws, xs, np.cumsum(counts), w_nz=nz, ws_dtype=str(rng.choice(["f32", "bf16", "f16"])))
        elif N >= 256:
            topk = int(rng.choice([1, 2, 4]))
            rows = (int(counts.sum()) // topk) * topk
            extra = int(counts.sum()) - rows
            for i in range(E):
                d = min(extra, int(counts[i]))
                counts[i] -= d
                extra -= d
            if rows == 0:
                continue
            check_finalize(oracle, rows, K, N, E, counts, topk, 2000 * seed + it, shared_rows=max(1, rows // topk // 2),
                           use_bias=bool(rng.random() < 0.5), idx32=bool(rng.random() < 0.5), use_pts=bool(rng.random() < 0.8),
                           flat_layout=(int(rng.choice([0, 2])) if rng.random() < 0.5 else None))
    for it in range(8):
        E = int(rng.choice([8, 32, 256, 300, 1024]))
        n, k, h = int(rng.integers(1, 400)), min(int(rng.choice([1, 2, 4, 8])), E), int(rng.choice([16, 20, 64, 100, 512, 1024]))
        a = int(rng.integers(0, E - 1))
        b = int(rng.integers(a + 1, E + 1))
        quant = bool(rng.random() < 0.7)
        kind = str(rng.choice(["bf16", "f16", "f32"] if quant else ["bf16", "f16", "f32", "int8"]))
        check_init_routing(oracle, n, k, h, E, (a, b), 3000 * seed + it, quant=quant, x_kind=kind, smooth=bool(quant and rng.random() < 0.5),
                           row_idx_type=int(rng.integers(0, 2)), count_type=int(rng.integers(1, 3)),
                           per_token_scale=bool(not quant and rng.random() < 0.5))
