"""CPU checks of the oracle itself: against what the reference's own tests pin (group_list semantics from the
operator README, workspace byte counts and tiling keys from the tiling unit tests), against an independent
numpy formulation, against the committed golden fixtures, and of each rounding rule on hand-picked values."""
import json
import os

import numpy as np
import pytest

from ops_transformer_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


# ---- what the reference pins -----------------------------------------------------------------------------

def test_group_list_readme_example(oracle):
    # gmm/grouped_matmul_swiglu_quant/README.md:38-48: groupList=[3,4,4,6] -> rows [0,3) [3,4) [4,4) [4,6)
    rs, rc = oracle.group_layout([3, 4, 4, 6], 0, 6)
    assert rs.tolist() == [0, 3, 4, 4] and rc.tolist() == [3, 1, 0, 2]
    # README.md:50-57: groupList=[12,14,18] with 30 rows -> rows 18.. are never written
    rs, rc = oracle.group_layout([12, 14, 18], 0, 30)
    assert int(rs[-1] + rc[-1]) == 18


def test_group_list_count_type(oracle):
    # aclnn_grouped_matmul_v4.h:55-57: groupListType 1 = per-group counts
    rs, rc = oracle.group_layout([64, 32, 96, 64], 1, 256)
    assert rs.tolist() == [0, 64, 96, 192] and rc.tolist() == [64, 32, 96, 64]
    rs0, rc0 = oracle.group_layout(np.cumsum([64, 32, 96, 64]), 0, 256)
    assert rs0.tolist() == rs.tolist() and rc0.tolist() == rc.tolist()


def test_group_list_is_clipped_to_the_tensor(oracle):
    rs, rc = oracle.group_layout([5, 3, 40], 0, 20)       # not monotone, overshoots M
    assert rc.tolist() == [5, 0, 17] and (rs + rc).max() <= 20
    rs, rc = oracle.group_layout([5, -3, 40], 1, 20)
    assert rc.tolist() == [5, 0, 15] and rs.tolist() == [0, 5, 5]


def test_reference_workspace_known_answers(oracle):
    # tests/ut/op_host/test_grouped_matmul_swiglu_quant_tiling.cpp:70, :99 (A8W8 cases) of the reference
    assert oracle.ref_swiglu_workspace_bytes(16, 512) == 16809984
    assert oracle.ref_swiglu_workspace_bytes(16, 4096) == 17039360
    assert oracle.ref_swiglu_tiling_key(16, 512) == 0 and oracle.ref_swiglu_tiling_key(16, 4096) == 0
    # key 1 iff m > 2*mLimit; at N=4096 mLimit = 2048 (grouped_matmul_swiglu_quant_tiling.cpp:211, :232)
    assert oracle.ref_swiglu_tiling_key(4096, 4096) == 0 and oracle.ref_swiglu_tiling_key(4097, 4096) == 1
    assert oracle.ref_swiglu_workspace_bytes(32768, 4096) == 16 * 2**20 + 64 * 2**20


# ---- rounding rules ----------------------------------------------------------------------------------------

def test_bf16_round_to_nearest_even(oracle):
    L = oracle.lib()
    assert L.oracle_f32_to_bf16(1.0) == 0x3F80
    assert L.oracle_f32_to_bf16(np.float32(1.00390625)) == 0x3F80        # 1 + 2^-8: tie -> even (down)
    assert L.oracle_f32_to_bf16(np.float32(1.01171875)) == 0x3F82        # 1 + 3*2^-8: tie -> even (up)
    assert L.oracle_f32_to_bf16(float(np.nextafter(np.float32(1.00390625), np.float32(2)))) == 0x3F81  # just above the tie
    vals = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 1e3
    import torch
    exp = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_bits(vals), exp)
    assert all(L.oracle_f32_to_bf16(float(v)) == int(e) for v, e in zip(vals[:512], exp[:512]))


def test_fp16_then_int8_double_rounding(oracle):
    L = oracle.lib()
    vals = np.concatenate([np.random.default_rng(1).uniform(-130, 130, 20000), [0.5, 1.5, 2.5, -0.5, -2.5, 126.5, 127.49,
                          126.96875, 0.49999997, 1e-8, -1e-8, 65519.0, 65520.0, 1e9, 5.96e-8, 2.98e-8, 3.0e-8]]).astype(np.float32)
    for v in vals:
        h = L.oracle_f32_to_f16(float(v))
        assert h == int(np.float32(v).astype(np.float16).view(np.uint16)), v
        if abs(float(v)) < 1000:
            q = L.oracle_f16_to_i8(h)
            e = int(np.clip(np.rint(np.float32(np.float16(v))), -128, 127))
            assert q == e, (v, q, e)
    # double rounding differs from a single rounding: 0.50024 -> half 0.5 -> 0, although rint(0.50024) = 1
    assert L.oracle_f16_to_i8(L.oracle_f32_to_f16(0.50024)) == 0 and round(0.50024) == 1
    assert L.oracle_f16_to_i8(0x7E00) == 0  # NaN -> 0


# ---- against the independent numpy formulation ---------------------------------------------------------------

@pytest.mark.parametrize("gl_type", [0, 1])
def test_gmm_matches_numpy_formulation(oracle, gl_type):
    rng = np.random.default_rng(3)
    M, K, N, E = 70, 133, 48, 5
    x = synth.int8_tensor((M, K), 3, 1)
    w = synth.int8_tensor((E, K, N), 3, 2)
    ws = synth.scale_tensor((E, N), 3, 3)
    xs = synth.scale_tensor((M,), 3, 4)
    counts = np.array([10, 0, 33, 1, 20])
    gl = synth.group_list_from_counts(counts, gl_type)
    r = oracle.gmm_w8a8(x, w, ws, xs, gl, gl_type, want_acc=True, want_pre=True)
    acc, pre, y = oracle.np_gmm_w8a8(x, w, ws, xs, gl, gl_type)
    n = int(counts.sum())
    assert np.array_equal(r["acc"][:n], acc[:n]) and np.array_equal(r["pre"][:n], pre[:n]) and np.array_equal(r["y"][:n], y[:n])
    assert (r["y"][n:] == 0).all()
    # int32 bias joins the accumulator; bf16 bias is added in fp32 after both scales; relu before the cast
    b32 = rng.integers(-5000, 5000, size=(E, N)).astype(np.int32)
    r = oracle.gmm_w8a8(x, w, ws, xs, gl, gl_type, bias=b32, want_acc=True)
    acc, pre, y = oracle.np_gmm_w8a8(x, w, ws, xs, gl, gl_type, bias_i32=b32)
    assert np.array_equal(r["acc"][:n], acc[:n]) and np.array_equal(r["y"][:n], y[:n])
    bf = oracle.f32_to_bf16_bits(rng.uniform(-30, 30, size=(E, N)).astype(np.float32))
    r = oracle.gmm_w8a8(x, w, ws, xs, gl, gl_type, bias=bf, act_type=1)
    acc, pre, y = oracle.np_gmm_w8a8(x, w, ws, xs, gl, gl_type, bias_f32=oracle.bf16_bits_to_f32(bf), relu=True)
    assert np.array_equal(r["y"][:n], y[:n])
    # transposed storage gives the same numbers
    rt = oracle.gmm_w8a8(x, np.ascontiguousarray(w.transpose(0, 2, 1)), ws, xs, gl, gl_type, w_trans=True)
    r0 = oracle.gmm_w8a8(x, w, ws, xs, gl, gl_type)
    assert np.array_equal(rt["y"], r0["y"])


def test_gmm_activations_and_float16_result(oracle):
    # the activations against float64 evaluations of their published definitions; the float16 cast against numpy's
    M, K, N, E = 40, 64, 48, 2
    x = synth.int8_tensor((M, K), 5, 1)
    w = synth.int8_tensor((E, K, N), 5, 2)
    ws = (synth.scale_tensor((E, N), 5, 3) * 0.5).astype(np.float32)
    xs = synth.scale_tensor((M,), 5, 4)
    gl = [15, 40]
    pre = oracle.gmm_w8a8(x, w, ws, xs, gl, 0, want_pre=True)["pre"].astype(np.float64)
    want = {
        1: np.maximum(pre, 0),
        2: pre / (1 + np.exp(-1.59576912 * (pre + 0.044715 * pre ** 3))),
        4: pre / (1 + np.exp(-1.702 * pre)),
        5: pre / (1 + np.exp(-pre)),
    }
    assert np.abs(pre).max() > 3 and np.abs(pre).min() < 0.1   # both the flat and the curved parts are visited
    for act, exp in want.items():
        r = oracle.gmm_w8a8(x, w, ws, xs, gl, 0, act_type=act, want_pre=True)
        assert np.allclose(r["pre"], exp, rtol=2e-6, atol=1e-7), act
        assert np.array_equal(r["y"], oracle.f32_to_bf16_bits(r["pre"]))
        h = oracle.gmm_w8a8(x, w, ws, xs, gl, 0, act_type=act, y_dtype="f16", want_pre=True)
        assert np.array_equal(h["y"], h["pre"].astype(np.float16).view(np.uint16))
    # 2 (tanh form) equals 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) analytically
    tanh_form = 0.5 * pre * (1 + np.tanh(np.sqrt(2 / np.pi) * (pre + 0.044715 * pre ** 3)))
    assert np.allclose(want[2], tanh_form, rtol=1e-6, atol=1e-7)


def _finalize_inputs(seed, M, K, N, E, counts, topk, shared_rows):
    rng = np.random.default_rng(seed)
    x = synth.int8_tensor((M, K), seed, 1)
    w = synth.int8_tensor((E, K, N), seed, 2)
    ws = synth.scale_tensor((E, N), seed, 3)
    xs = synth.scale_tensor((M,), seed, 4)
    batch = M // topk
    row_index = rng.permutation(M).astype(np.int64) % batch      # every destination row receives topk rows
    logit = rng.uniform(0.05, 0.6, size=M).astype(np.float32)
    shared = rng.uniform(-40, 40, size=(shared_rows, N)).astype(np.float32)
    bias = rng.uniform(-20, 20, size=(E, N)).astype(np.float32)
    return x, w, ws, xs, np.asarray(counts, np.int64), row_index, logit, shared, bias, batch


def test_finalize_routing_matches_float64_formulation(oracle):
    M, K, N, E, topk = 96, 80, 64, 4, 4
    counts = [30, 0, 50, 10]                       # 6 trailing rows belong to no group
    x, w, ws, xs, gl, ri, logit, shared, bias, batch = _finalize_inputs(7, M, K, N, E, counts, topk, 10)
    sh_bits, b_bits = oracle.f32_to_bf16_bits(shared), oracle.f32_to_bf16_bits(bias)
    # scene 1: shared rows, logits, per-token scale, bias; shared rows sit at an offset
    r = oracle.gmm_finalize_routing(x, w, ws, xs, gl, ri, batch, bias=b_bits, shared_input=sh_bits, shared_offset=5,
                                    shared_weight=0.5, logit=logit, y_init=np.full((batch, N), 7.0, np.float32))
    want = oracle.np_gmm_finalize_routing(x, w, ws, xs, gl, ri, batch, bias_f32=oracle.bf16_bits_to_f32(b_bits),
                                          shared_f32=oracle.bf16_bits_to_f32(sh_bits), shared_offset=5, shared_weight=0.5,
                                          logit=logit)
    assert np.all(np.abs(r["y"] - want) <= 4e-7 * r["abs_sum"] + 1e-30)
    assert np.abs(want).max() > 1.0
    # rows that receive nothing and lie outside the shared range are zero, not the previous contents
    touched = np.zeros(batch, bool)
    touched[ri[:90]] = True
    touched[5:15] = True
    assert (r["y"][~touched] == 0).all()
    # int32 row index, count versus running-total group list, bf16 scale: same numbers
    r32 = oracle.gmm_finalize_routing(x, w, ws, xs, np.cumsum(gl), ri.astype(np.int32), batch, gl_type=0, bias=b_bits,
                                      shared_input=sh_bits, shared_offset=5, shared_weight=0.5, logit=logit)
    assert np.array_equal(r32["y"], r["y"])
    # scene 2: neither shared input nor logits: plain stores of (acc * scale) * per_token, other rows keep their contents
    perm = np.random.default_rng(8).permutation(M).astype(np.int64)
    r2 = oracle.gmm_finalize_routing(x, w, ws, xs, gl, perm, M, y_init=np.full((M, N), 7.0, np.float32))
    g = oracle.gmm_w8a8(x, w, ws, xs, gl, 1, want_pre=True)["pre"]
    assert np.array_equal(r2["y"][perm[:90]], g[:90])
    assert (r2["y"][perm[90:]] == 7.0).all()
    # out-of-range destinations are skipped
    bad = ri.copy(); bad[3] = batch + 5; bad[4] = -1
    rb = oracle.gmm_finalize_routing(x, w, ws, xs, gl, bad, batch, shared_input=sh_bits, logit=logit)
    assert np.isfinite(rb["y"]).all()


def test_moe_init_routing_matches_numpy_formulation(oracle):
    rng = np.random.default_rng(11)
    n, k, h, E = 37, 4, 48, 16
    x = rng.standard_normal((n, h)).astype(np.float32)
    x[5] = 0.0                                           # an all-zero row: scale 0, zeros
    idx = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    start, end = 3, 12
    flat = idx.ravel()
    keep = np.nonzero((flat >= start) & (flat < end))[0]
    order = keep[np.argsort(flat[keep], kind="stable")]   # stable sort of the active pairs by expert
    smooth = rng.uniform(0.5, 2.0, size=(end - start, h)).astype(np.float32)
    for sc in (None, smooth):
        r = oracle.moe_init_routing_v3(x, idx, E, (start, end), True, row_idx_type=1, count_type=1, scale=sc)
        assert r["rows"] == len(order)
        assert np.array_equal(r["expanded_row_idx"][:len(order)], order)
        assert (r["expanded_row_idx"][len(order):] == -9).all()
        assert np.array_equal(r["counts"], np.bincount(flat[keep] - start, minlength=end - start))
        for i, j in enumerate(order):
            v = x[j // k] if sc is None else (x[j // k] * sc[flat[j] - start]).astype(np.float32)
            s = np.float32(np.abs(v).max()) / np.float32(127.0)
            assert r["expanded_scale"][i] == s
            if s == 0:
                assert (r["expanded_x"][i] == 0).all()
                continue
            u = (v / s).astype(np.float32)
            hz = np.where(np.abs(u.astype(np.float16).astype(np.float32)) > np.abs(u),              # fp16 towards zero
                          np.nextafter(u.astype(np.float16), np.float16(0)), u.astype(np.float16)).astype(np.float32)
            q = np.trunc(hz + np.copysign(np.float32(0.5), hz))                                       # ties away from zero
            assert np.array_equal(r["expanded_x"][i], q.astype(np.int8)), i
        assert (r["expanded_x"][len(order):] == -77).all() and (r["expanded_scale"][len(order):] == -5.0).all()
    # gather-type row index and key-value counts
    r0 = oracle.moe_init_routing_v3(x, idx, E, (start, end), True, row_idx_type=0, count_type=2)
    inv = np.full(n * k, -1, np.int32)
    inv[order] = np.arange(len(order))
    assert np.array_equal(r0["expanded_row_idx"], inv)
    cnt = np.bincount(flat[keep] - start, minlength=end - start)
    nzp = [(e + start, c) for e, c in enumerate(cnt) if c]
    assert [tuple(p) for p in r0["counts"][:len(nzp)]] == nzp
    written = min(end - start + 1, E)
    assert (r0["counts"][len(nzp):written] == 0).all() and (r0["counts"][written:] == -9).all()
    # no quantisation: rows and per-token scales are copied; bf16 / int8 rows pass through untouched
    ps = rng.uniform(1, 2, size=n).astype(np.float32)
    xb = oracle.f32_to_bf16_bits(x)
    rc = oracle.moe_init_routing_v3(xb, idx, E, (0, E), False, scale=ps)
    full = np.argsort(flat, kind="stable")
    assert np.array_equal(rc["expanded_x"], xb[full // k]) and np.array_equal(rc["expanded_scale"], ps[full // k])
    # bf16 and fp16 inputs quantise like their float32 values
    rb = oracle.moe_init_routing_v3(xb, idx, E, (0, E), True)
    rf = oracle.moe_init_routing_v3(oracle.bf16_bits_to_f32(xb), idx, E, (0, E), True)
    assert np.array_equal(rb["expanded_x"], rf["expanded_x"]) and np.array_equal(rb["expanded_scale"], rf["expanded_scale"])


def test_gmm_scale_order_is_weight_then_token(oracle):
    # (acc*w_scale)*x_scale and (acc*x_scale)*w_scale differ in the last bit for some inputs; the two operators
    # use opposite orders (grouped_matmul_quant_mixcore.h:262,300 vs grouped_matmul_swiglu_quant.h:392,450).
    x = synth.int8_tensor((64, 256), 5, 1)
    w = synth.int8_tensor((1, 256, 64), 5, 2)
    ws = synth.scale_tensor((1, 64), 5, 3)
    xs = synth.scale_tensor((64,), 5, 4)
    r = oracle.gmm_w8a8(x, w, ws, xs, [64], 0, want_acc=True, want_pre=True)
    a = r["acc"].astype(np.float32)
    assert np.array_equal(r["pre"], (a * ws[0][None, :]) * xs[:, None])
    other = (a * xs[:, None]) * ws[0][None, :]
    assert np.count_nonzero(other != r["pre"]) > 0


def test_swiglu_matches_numpy_formulation(oracle):
    M, K, N, E = 90, 200, 96, 4
    x = synth.int8_tensor((M, K), 6, 1)
    w = synth.int8_tensor((E, K, N), 6, 2)
    ws = synth.scale_tensor((E, N), 6, 3)
    xs = synth.scale_tensor((M,), 6, 4)
    gl = [20, 20, 75, 80]
    r = oracle.swiglu_quant(x, w, ws, xs, gl, want_acc=True, want_s=True)
    q, qs, S = oracle.np_swiglu_quant(x, w, ws, xs, gl)
    acc = np.zeros((M, N), np.int64)
    for g, (s, n) in enumerate(oracle.np_group_ranges(gl, 0, M)):
        acc[s:s + n] = x[s:s + n].astype(np.int64) @ w[g].astype(np.int64)
    assert np.array_equal(r["acc"][:80], acc[:80])
    # exp differs between libm and numpy by an ulp or two: 1e-6 on the scales, 1 LSB on a few outputs
    assert np.max(np.abs(S[:80] - r["s"][:80]) / np.maximum(np.abs(S[:80]), 1e-30)) < 1e-6
    assert np.max(np.abs(qs[:80] - r["q_scale"][:80]) / qs[:80]) < 1e-6
    d = np.abs(q[:80].astype(int) - r["q"][:80].astype(int))
    assert d.max() <= 1 and np.count_nonzero(d) <= 2
    assert (r["q"][80:] == 0).all() and (r["q_scale"][80:] == 0).all()
    # exact identities of the quantisation step given the oracle's own S
    s = r["s"][:80]
    amax = np.abs(s).max(axis=1)
    assert np.array_equal(r["q_scale"][:80], amax / np.float32(127.0))
    assert (np.abs(r["q"][:80]).max(axis=1) == 127).all()


def test_swiglu_zero_row_maps_nan_to_zero(oracle):
    x = np.zeros((4, 32), np.int8)
    w = synth.int8_tensor((1, 32, 32), 7, 2)
    ws = synth.scale_tensor((1, 32), 7, 3)
    xs = synth.scale_tensor((4,), 7, 4)
    r = oracle.swiglu_quant(x, w, ws, xs, [4])
    assert (r["q_scale"] == 0).all() and (r["q"] == 0).all()


# ---- committed golden fixtures ---------------------------------------------------------------------------------

def test_golden_fixtures(oracle):
    with open(os.path.join(GOLDEN, "manifest.json")) as f:
        manifest = json.load(f)
    assert manifest["cases"], "no golden cases"
    for case in manifest["cases"]:
        d = np.load(os.path.join(GOLDEN, case["file"]))
        if case["op"] == "moe_init_routing_v3":
            r = oracle.moe_init_routing_v3(d["x_bf16_bits"], d["expert_idx"], case["E"], tuple(case["active_range"]), bool(case["quant"]),
                                           row_idx_type=case["row_idx_type"], count_type=case["count_type"], scale=d["scale"])
            for key in ("expanded_x", "expanded_row_idx", "counts", "expanded_scale"):
                assert np.array_equal(r[key], d[key]), key
            assert r["rows"] == int(d["rows"])
            continue
        if case["op"] == "ep_combine":
            assert np.array_equal(oracle.ep_combine(d["y_bf16_bits"], d["pair_row"], d["weights"]), d["out_bf16_bits"])
            continue
        x, w, ws, xs, gl = d["x"], d["w"], d["w_scale"], d["x_scale"], d["group_list"]
        if case["op"] == "grouped_matmul_finalize_routing":
            r = oracle.gmm_finalize_routing(x, w, ws, xs, gl, d["row_index"], case["batch"], bias=d["bias_bf16_bits"],
                                            shared_input=d["shared_bf16_bits"], shared_offset=case["shared_offset"],
                                            shared_weight=case["shared_weight"], logit=d["logit"])
            assert np.array_equal(r["y"], d["y"])
            continue
        if case["op"] == "grouped_matmul":
            r = oracle.gmm_w8a8(x, w, ws, xs, gl, int(case["group_list_type"]), want_acc=True)
            assert np.array_equal(r["acc"], d["acc"]) and np.array_equal(r["y"], d["y_bf16_bits"])
        else:
            r = oracle.swiglu_quant(x, w, ws, xs, gl)
            assert np.array_equal(r["q"], d["q"]) and np.array_equal(r["q_scale"], d["q_scale"])


# ---------------------------------------------------------------------------------------------------------
# Row-sampled checks of full-size launches (oracle/sampled_check.py): the sampling itself and the row-independence
# the method rests on
# ---------------------------------------------------------------------------------------------------------

def test_sample_rows_covers_edges_of_every_expert():
    from oracle import sampled_check as SC
    counts = np.array([300, 0, 1, 513, 129], np.int64)
    rows = SC.sample_rows(counts, n_random=4, seed=3)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    assert (np.diff(rows) > 0).all() and rows.min() >= 0 and rows.max() < counts.sum()
    for s, r in zip(starts, counts):
        if r == 0:
            continue
        must = {s, s + r - 1} | {s + m + d for m in range(128, r, 128) for d in (-1, 0)}
        assert must <= set(rows.tolist())
    assert (SC.counts_of_sample(rows, counts) <= counts).all() and SC.counts_of_sample(rows, counts).sum() == len(rows)
    assert (SC.counts_of_sample(rows, counts)[[1]] == 0).all()
    # few rows: everything is taken
    assert np.array_equal(SC.sample_rows([3, 0, 5], max_rows_all=16), np.arange(8))


def test_oracle_on_sampled_rows_equals_sampled_rows_of_the_oracle(oracle):
    """Both operators treat every row on its own: the oracle on a subset of rows (same weights) reproduces those rows."""
    from oracle import sampled_check as SC
    from ops_transformer_b200 import synth
    counts = np.array([70, 0, 33, 140], np.int64)
    M, K, N, E = int(counts.sum()), 96, 64, 4
    x, w = synth.int8_tensor((M, K), 7, 1), synth.int8_tensor((E, K, N), 7, 2)
    ws, xs = synth.scale_tensor((E, N), 7, 3), synth.scale_tensor((M,), 7, 4)
    gl = np.cumsum(counts)
    full_s = oracle.swiglu_quant(x, w, ws, xs, gl)
    full_g = oracle.gmm_w8a8(x, w, ws, xs, gl, 0)["y"]
    rows = SC.sample_rows(counts, n_random=5, seed=1)
    sc = SC.counts_of_sample(rows, counts)
    r = SC.check_swiglu_rows(x[rows], w, ws, xs[rows], sc, full_s["q"][rows], full_s["q_scale"][rows])
    assert r["mismatches"] == 0 and r["int8_off_by_one"] == 0 and r["rows"] == len(rows)
    g = SC.check_gmm_rows(x[rows], w, ws, xs[rows], sc, full_g[rows])
    assert g["mismatches"] == 0 and g["not_bit_identical"] == 0
    # a wrong row is caught
    bad = full_g[rows].copy()
    bad[3] ^= 0x0040
    assert SC.check_gmm_rows(x[rows], w, ws, xs[rows], sc, bad)["not_bit_identical"] > 0
    qbad = full_s["q"][rows].copy()
    qbad[2, :] = np.where(qbad[2, :] > 100, qbad[2, :] - 3, qbad[2, :] + 3)
    assert SC.check_swiglu_rows(x[rows], w, ws, xs[rows], sc, qbad, full_s["q_scale"][rows])["mismatches"] > 0


def test_ep_combine_weighted_sum_in_slot_order(oracle):
    """Two tokens, three slots: products and sums rounded one at a time in slot order, missing rows left out, bf16 RNE."""
    y = np.array([[1.0, 3.0], [0.5, -2.0], [4.0, 1.0], [8.0, 8.0]], np.float32)
    pair_row = np.array([[0, 2, 1], [3, -1, 99]])
    w = np.array([[0.5, 0.25, 2.0], [0.125, 7.0, 7.0]], np.float32)
    got = oracle.bf16_bits_to_f32(oracle.ep_combine(oracle.f32_to_bf16_bits(y), pair_row, w))
    want = np.array([[0.5 + 1.0 + 1.0, 1.5 + 0.25 - 4.0], [1.0, 1.0]], np.float32)
    assert np.array_equal(got, want)
    # the order of the additions is the slot order: a sum that depends on it
    big = oracle.f32_to_bf16_bits(np.array([[2.0 ** 24], [1.0], [-(2.0 ** 24)]], np.float32))
    r = oracle.bf16_bits_to_f32(oracle.ep_combine(big, np.array([[0, 1, 2]]), np.ones((1, 3), np.float32)))
    assert r[0, 0] == 0.0      # (2^24 + 1) rounds to 2^24, then - 2^24
    r = oracle.bf16_bits_to_f32(oracle.ep_combine(big, np.array([[0, 2, 1]]), np.ones((1, 3), np.float32)))
    assert r[0, 0] == 1.0
