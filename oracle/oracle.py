"""ctypes front-end of the CPU oracle (TEST INFRASTRUCTURE, not product code).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import this
module.  It loads ``libgmm_oracle.so`` (built from ``gmm_oracle.c`` by the Makefile beside it) and also
holds an independent, slow numpy formulation of the same arithmetic that the CPU tests use to
cross-check the C code on small cases.

Parity unpinned: the reference ships no golden vectors for either operator; see the header of
``gmm_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libgmm_oracle.so")

DT_F32, DT_F16, DT_I32, DT_BF16 = 0, 1, 3, 27


def build(force: bool = False) -> str:
    """Compile the oracle library if it is missing or older than its source."""
    src = os.path.join(_HERE, "gmm_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libgmm_oracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        p, i64, i32 = C.c_void_p, C.c_int64, C.c_int
        L.oracle_group_layout.argtypes = [p, i64, i32, i64, p, p]
        L.oracle_gmm_w8a8.argtypes = [p, p, p, i32, p, p, i32, p, i64, i32, i64, i64, i64, i64, i32, i32, i32, p, p, p]
        L.oracle_swiglu_quant.argtypes = [p, p, p, i32, p, p, i64, i64, i64, i64, i64, i32, p, p, p, p]
        L.oracle_ref_swiglu_workspace_bytes.argtypes = [i64, i64]
        L.oracle_ref_swiglu_workspace_bytes.restype = i64
        L.oracle_ref_swiglu_tiling_key.argtypes = [i64, i64]
        L.oracle_f32_to_bf16.argtypes = [C.c_float]
        L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f16_to_i8.argtypes = [C.c_uint16]
        L.oracle_f16_to_i8.restype = C.c_int8
        L.oracle_force_generic_gemm.argtypes = [i32]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _scale_dtype(a) -> int:
    if a.dtype == np.float32:
        return DT_F32
    if a.dtype == np.float16:
        return DT_F16
    if a.dtype == np.uint16:  # bf16 bit patterns
        return DT_BF16
    raise TypeError(f"scale dtype {a.dtype}")


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Make the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS said; returns the count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def group_layout(group_list, gl_type: int, M: int):
    gl = np.ascontiguousarray(group_list, dtype=np.int64)
    rs = np.zeros(len(gl), np.int64)
    rc = np.zeros(len(gl), np.int64)
    lib().oracle_group_layout(_ptr(gl), len(gl), gl_type, M, _ptr(rs), _ptr(rc))
    return rs, rc


def gmm_w8a8(x, w, scale, per_token_scale, group_list, gl_type=0, bias=None, act_type=0, w_trans=False,
             y_dtype="bf16", y_init=None, want_acc=False, want_pre=False):
    """grouped_matmul W8A8.  ``w`` is [E,K,N] int8 (or [E,N,K] when ``w_trans``).  bf16 tensors (scale, bias,
    result) travel as uint16 bit patterns.  Returns a dict with y and, when asked, acc / pre."""
    x = np.ascontiguousarray(x, np.int8)
    w = np.ascontiguousarray(w, np.int8)
    M, K = x.shape
    E = w.shape[0]
    N = w.shape[1] if w_trans else w.shape[2]
    gl = np.ascontiguousarray(group_list, np.int64)
    scale = np.ascontiguousarray(scale)
    pts = None if per_token_scale is None else np.ascontiguousarray(per_token_scale, np.float32)
    bias_dt = -1
    if bias is not None:
        bias = np.ascontiguousarray(bias)
        bias_dt = DT_I32 if bias.dtype == np.int32 else DT_BF16
    if y_dtype in ("bf16", "f16"):  # both travel as uint16 bit patterns
        y = np.zeros((M, N), np.uint16) if y_init is None else np.array(y_init, np.uint16, copy=True)
        ydt = DT_BF16 if y_dtype == "bf16" else DT_F16
    else:
        y = np.zeros((M, N), np.int32) if y_init is None else np.array(y_init, np.int32, copy=True)
        ydt = DT_I32
    acc = np.zeros((M, N), np.int32) if want_acc else None
    pre = np.zeros((M, N), np.float32) if want_pre else None
    rc = lib().oracle_gmm_w8a8(_ptr(x), _ptr(w), _ptr(scale), _scale_dtype(scale), _ptr(pts), _ptr(bias), bias_dt,
                               _ptr(gl), len(gl), gl_type, M, K, N, E, act_type, int(w_trans), ydt, _ptr(y),
                               _ptr(acc), _ptr(pre))
    if rc != 0:
        raise ValueError("oracle_gmm_w8a8 rejected the arguments")
    return {"y": y, "acc": acc, "pre": pre}


def gmm_finalize_routing(x, w, scale, per_token, group_list, row_index, y_rows, gl_type=1, bias=None, shared_input=None,
                         shared_offset=0, shared_weight=1.0, logit=None, y_init=None):
    """grouped_matmul_finalize_routing W8A8.  ``w`` int8 [E,K,N]; bf16 tensors (scale if uint16, bias, shared_input) are
    uint16 bit patterns.  Returns dict(y fp32 [y_rows, N], abs_sum float64: sum of the magnitudes of the terms of every
    element, the scale of the rounding differences an unordered summation may show)."""
    x = np.ascontiguousarray(x, np.int8)
    w = np.ascontiguousarray(w, np.int8)
    M, K = x.shape
    E, _, N = w.shape
    gl = np.ascontiguousarray(group_list, np.int64)
    scale = np.ascontiguousarray(scale)
    pts = None if per_token is None else np.ascontiguousarray(per_token, np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.uint16)
    sh = None if shared_input is None else np.ascontiguousarray(shared_input, np.uint16)
    lg = None if logit is None else np.ascontiguousarray(logit, np.float32)
    ri = np.ascontiguousarray(row_index)
    if ri.dtype not in (np.int64, np.int32):
        raise TypeError("row_index must be int64 or int32")
    y = np.zeros((y_rows, N), np.float32) if y_init is None else np.array(y_init, np.float32, copy=True)
    abs_sum = np.zeros((y_rows, N), np.float64)
    fn = lib().oracle_gmm_finalize_routing
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int,
                   C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                   C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p]
    fn.restype = C.c_int
    rc = fn(_ptr(x), _ptr(w), _ptr(scale), _scale_dtype(scale), _ptr(bias), _ptr(pts), _ptr(gl), len(gl), gl_type, _ptr(sh),
            0 if sh is None else sh.shape[0], shared_offset, float(shared_weight), _ptr(lg), _ptr(ri), int(ri.dtype == np.int32),
            M, K, N, E, _ptr(y), y_rows, _ptr(abs_sum))
    if rc != 0:
        raise ValueError("oracle_gmm_finalize_routing rejected the arguments")
    return {"y": y, "abs_sum": abs_sum}


def np_gmm_finalize_routing(x, w, scale_f32, per_token, group_list, row_index, y_rows, gl_type=1, bias_f32=None,
                            shared_f32=None, shared_offset=0, shared_weight=1.0, logit=None):
    """Independent float64 formulation of the same operator (for tolerance checks of the C restatement)."""
    M, K = x.shape
    N = w.shape[2]
    add = shared_f32 is not None or logit is not None
    y = np.zeros((y_rows, N), np.float64)
    if shared_f32 is not None:
        y[shared_offset:shared_offset + shared_f32.shape[0]] = shared_f32.astype(np.float64) * float(np.float32(shared_weight))
    for g, (s, r) in enumerate(np_group_ranges(group_list, gl_type, M)):
        if r <= 0:
            continue
        a = (x[s:s + r].astype(np.int64) @ w[g].astype(np.int64)).astype(np.float64)
        t = a * np.asarray(scale_f32[g], np.float64)[None, :]
        rowscale = np.ones(r) if per_token is None else np.asarray(per_token[s:s + r], np.float64)
        lg = np.ones(r) if logit is None else np.asarray(logit[s:s + r], np.float64)
        t = t * (rowscale * lg)[:, None]
        if bias_f32 is not None:
            t = t + lg[:, None] * np.asarray(bias_f32[g], np.float64)[None, :]
        for i in range(r):
            d = int(row_index[s + i])
            if 0 <= d < y_rows:
                if add:
                    y[d] += t[i]
                else:
                    y[d] = t[i]
    return y


def moe_init_routing_v3(x, expert_idx, expert_num, active_range, quant, row_idx_type=1, count_type=1, scale=None):
    """moe_init_routing_v3.  ``x`` [n,h] float32, float16, uint16 (bf16 bits) or int8; returns dict(expanded_x, expanded_row_idx,
    counts, expanded_scale, rows).  Rows beyond ``rows`` keep the fill values (-77 / -5.0 / -9)."""
    x = np.ascontiguousarray(x)
    idx = np.ascontiguousarray(expert_idx, np.int32)
    n, h = x.shape
    k = idx.shape[1]
    dt = {np.dtype(np.float32): DT_F32, np.dtype(np.float16): DT_F16, np.dtype(np.uint16): DT_BF16, np.dtype(np.int8): 2}[x.dtype]
    start, end = active_range
    sc = None if scale is None else np.ascontiguousarray(scale, np.float32)
    ex = np.full((n * k, h), -77, np.int8) if quant else np.zeros((n * k, h), x.dtype)
    ri = np.full((n * k,), -9, np.int32)
    counts = np.full((end - start,) if count_type == 1 else (expert_num, 2), -9, np.int64)
    es = np.full((n * k,), -5.0, np.float32)
    fn = lib().oracle_moe_init_routing_v3
    fn.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p] + [C.c_int64] * 6 + [C.c_int] * 3 + [C.c_void_p] * 4
    fn.restype = C.c_int64
    rows = fn(_ptr(x), dt, _ptr(idx), _ptr(sc), n, k, h, expert_num, start, end, int(quant), row_idx_type, count_type, _ptr(ex),
              _ptr(ri), _ptr(counts), _ptr(es))
    return {"expanded_x": ex, "expanded_row_idx": ri, "counts": counts, "expanded_scale": es, "rows": int(rows)}


def swiglu_quant(x, w, w_scale, x_scale, group_list, w_trans=False, q_init=None, qs_init=None, want_acc=False,
                 want_s=False):
    """grouped_matmul_swiglu_quant A8W8.  Returns dict(q int8 [M,N/2], q_scale f32 [M], acc, s)."""
    x = np.ascontiguousarray(x, np.int8)
    w = np.ascontiguousarray(w, np.int8)
    M, K = x.shape
    E = w.shape[0]
    N = w.shape[1] if w_trans else w.shape[2]
    gl = np.ascontiguousarray(group_list, np.int64)
    w_scale = np.ascontiguousarray(w_scale)
    xs = np.ascontiguousarray(x_scale, np.float32)
    q = np.zeros((M, N // 2), np.int8) if q_init is None else np.array(q_init, np.int8, copy=True)
    qs = np.zeros((M,), np.float32) if qs_init is None else np.array(qs_init, np.float32, copy=True)
    acc = np.zeros((M, N), np.int32) if want_acc else None
    s = np.zeros((M, N // 2), np.float32) if want_s else None
    rc = lib().oracle_swiglu_quant(_ptr(x), _ptr(w), _ptr(w_scale), _scale_dtype(w_scale), _ptr(xs), _ptr(gl),
                                   len(gl), M, K, N, E, int(w_trans), _ptr(q), _ptr(qs), _ptr(acc), _ptr(s))
    if rc != 0:
        raise ValueError("oracle_swiglu_quant rejected the arguments")
    return {"q": q, "q_scale": qs, "acc": acc, "s": s}


def ref_swiglu_workspace_bytes(m: int, n: int) -> int:
    return int(lib().oracle_ref_swiglu_workspace_bytes(m, n))


def ref_swiglu_tiling_key(m: int, n: int) -> int:
    return int(lib().oracle_ref_swiglu_tiling_key(m, n))


# --------------------------------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16): bit patterns in uint16
# --------------------------------------------------------------------------------------------------

def f32_to_bf16_bits(a) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(a, np.float32))
    if nan.any():
        r = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)
    return r


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def ep_combine(y_bits, pair_row, weights) -> np.ndarray:
    """The combine that ends the expert-parallel path: per token, sum = 0; for every slot in slot order
    sum = sum + float(row) * weight (fp32 Muls, then fp32 Add: mc2/moe_distribute_combine_v2/op_kernel/
    moe_distribute_combine_v2.h:1130-1134, 1195); the result is cast to bf16 with round-to-nearest-even (:1258).
    y_bits: uint16 [rows, h] bf16 bit patterns; pair_row: int [tokens, k] row of every (token, slot) pair, negative or
    beyond the rows = no row; weights: fp32 [tokens, k].  Returns uint16 [tokens, h]."""
    y_bits = np.ascontiguousarray(y_bits, np.uint16)
    pair_row = np.asarray(pair_row)
    weights = np.asarray(weights, np.float32)
    tokens, k = pair_row.shape
    acc = np.zeros((tokens, y_bits.shape[1]), np.float32)
    for s in range(k):
        rows = pair_row[:, s]
        ok = (rows >= 0) & (rows < y_bits.shape[0])
        v = bf16_bits_to_f32(y_bits[np.where(ok, rows, 0)])
        prod = (v * weights[:, s:s + 1]).astype(np.float32)      # one rounding
        acc = np.where(ok[:, None], (acc + prod).astype(np.float32), acc)   # one rounding
    return f32_to_bf16_bits(acc)


# --------------------------------------------------------------------------------------------------
# Independent numpy formulation (slow; small cases only).  Written separately from the C code: int64
# matmul for the accumulators, numpy float32 element-wise ops (each one separately rounded), numpy's own
# float16 cast and np.rint for the double rounding.
# --------------------------------------------------------------------------------------------------

def np_group_ranges(group_list, gl_type, M):
    out, prev, run = [], 0, 0
    for v in np.asarray(group_list, np.int64):
        v = int(np.int32(v))
        if gl_type == 0:
            s, r = prev, v - prev
            prev = v
        else:
            s, r = run, v
            run += max(v, 0)
        r = max(r, 0)
        s = min(max(s, 0), M)
        r = min(r, M - s)
        out.append((s, r))
    return out


def np_gmm_w8a8(x, w, scale_f32, per_token_scale, group_list, gl_type=0, bias_i32=None, bias_f32=None, relu=False):
    M, K = x.shape
    N = w.shape[2]
    acc = np.zeros((M, N), np.int64)
    pre = np.zeros((M, N), np.float32)
    for g, (s, r) in enumerate(np_group_ranges(group_list, gl_type, M)):
        if r <= 0:
            continue
        a = x[s:s + r].astype(np.int64) @ w[g].astype(np.int64)
        if bias_i32 is not None:
            a = a + bias_i32[g].astype(np.int64)
        acc[s:s + r] = a
        t = a.astype(np.int32).astype(np.float32) * np.asarray(scale_f32[g], np.float32)[None, :]
        t = t * np.asarray(per_token_scale[s:s + r], np.float32)[:, None]
        if bias_f32 is not None:
            t = t + np.asarray(bias_f32[g], np.float32)[None, :]
        if relu:
            t = np.maximum(t, np.float32(0))
        pre[s:s + r] = t
    return acc.astype(np.int32), pre, f32_to_bf16_bits(pre)


def np_swiglu_quant(x, w, w_scale_f32, x_scale, group_list):
    M, K = x.shape
    N = w.shape[2]
    H = N // 2
    q = np.zeros((M, H), np.int8)
    qs = np.zeros((M,), np.float32)
    S = np.zeros((M, H), np.float32)
    one = np.float32(1.0)
    for g, (s, r) in enumerate(np_group_ranges(group_list, 0, M)):
        if r <= 0:
            continue
        a = (x[s:s + r].astype(np.int64) @ w[g].astype(np.int64)).astype(np.int32).astype(np.float32)
        t = a * np.asarray(x_scale[s:s + r], np.float32)[:, None]
        t = t * np.asarray(w_scale_f32[g], np.float32)[None, :]
        act, gate = t[:, :H], t[:, H:]
        sw = act / (one + np.exp(-act, dtype=np.float32))
        sv = (gate * sw).astype(np.float32)
        S[s:s + r] = sv
        amax = np.max(np.abs(sv), axis=1)
        scale = (amax / np.float32(127.0)).astype(np.float32)
        qs[s:s + r] = scale
        with np.errstate(divide="ignore", invalid="ignore"):
            rcp = (one / scale).astype(np.float32)
            u = (sv * rcp[:, None]).astype(np.float32)
        h = u.astype(np.float16)
        qi = np.rint(h.astype(np.float32))
        qi = np.where(np.isnan(qi), 0, qi)
        q[s:s + r] = np.clip(qi, -128, 127).astype(np.int8)
    return q, qs, S
