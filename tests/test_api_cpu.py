"""Host-side behaviour of the C ABI that needs no GPU: the library loads and exports every declared symbol, and
the first-phase calls return the reference's status codes for valid and invalid parameter sets (the cases follow
gmm/grouped_matmul/tests/utest_aclnn/ts_aclnn_grouped_matmul.cpp and
gmm/grouped_matmul_swiglu_quant/tests/ut/op_host/op_api/test_aclnn_grouped_matmul_swiglu_quant.cpp of the reference).
Phase 1 never dereferences tensor data, so host tensors stand in for device tensors here."""
import ctypes as C
import os
import re

import pytest
import torch

from ops_transformer_b200 import _lib, acl

OK, NULLPTR, INVALID = 0, 161001, 161002
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(gmm_lib):
    declared = set()
    for d, _, files in os.walk(os.path.join(ROOT, "include")):
        for f in files:
            text = open(os.path.join(d, f)).read()
            text = re.sub(r"#define ACL_FUNC_VISIBILITY.*", "", text)
            declared |= set(re.findall(r"ACL_FUNC_VISIBILITY[^;(]*?\b(\w+)\s*\(", text))
    assert declared, "no declarations found"
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(gmm_lib, name), f"{name} is declared but not exported"
    assert gmm_lib.gmmB200Version() >= 100


def _v4_phase1(x, w, scale, pts, gl, out, bias=None, split_item=3, group_type=0, gl_type=0, act=0, extra=None, api="V4",
               fmt_w=_lib.ACL_FORMAT_ND, tuning=None, quant_group_size=0):
    L = _lib.lib()
    mk = lambda t: acl.create_tensor_list([t]) if t is not None else None  # noqa: E731
    hx, hb, hs, hp, hy = mk(x), mk(bias), mk(scale), mk(pts), mk(out)
    hw = acl.create_tensor_list([w], fmt_w) if w is not None else None
    hg = acl.create_tensor(gl) if gl is not None else None
    size, ex = C.c_uint64(123), C.c_void_p(0)
    args = [hx, hw, hb, hs, None, None, None, hp, hg, None, None, None, split_item, group_type, gl_type, act, hy, None, None]
    if extra:
        for k, v in extra.items():
            args[k] = v
    ht = L.aclCreateIntArray((C.c_int64 * len(tuning))(*tuning), len(tuning)) if tuning is not None else None
    if api == "V5":
        args = args[:16] + [ht] + args[16:]
    elif api == "WeightNz":
        args = args[:16] + [ht, quant_group_size] + args[16:]
    rc = getattr(L, f"aclnnGroupedMatmul{api}GetWorkspaceSize")(*args, C.byref(size), C.byref(ex))
    if ht:
        L.aclDestroyIntArray(ht)
    if rc == OK:
        assert L.aclDestroyAclOpExecutor(ex) == OK
    for h in (hx, hw, hb, hs, hp, hy):
        if h:
            L.aclDestroyTensorList(h)
    if hg:
        L.aclDestroyTensor(hg)
    return rc, size.value


def _v4_tensors(M=84, K=5120, N=2560, E=4, scale_dtype=torch.bfloat16, out_dtype=torch.bfloat16):
    return dict(x=torch.empty((M, K), dtype=torch.int8), w=torch.empty((E, K, N), dtype=torch.int8),
                scale=torch.empty((E, N), dtype=scale_dtype), pts=torch.empty((M,), dtype=torch.float32),
                gl=torch.tensor([50, 65, 69, 84][:E], dtype=torch.int64), out=torch.empty((M, N), dtype=out_dtype))


def test_v4_reference_valid_case():
    # Test_GMMV4_04 of the reference: int8, bf16 scale, fp32 per-token scale, bf16 out, group list {50,65,69,84}
    rc, size = _v4_phase1(**_v4_tensors())
    assert rc == OK and size >= 256 and size % 256 == 0
    rc, _ = _v4_phase1(**_v4_tensors(scale_dtype=torch.float32))  # fp32 scale with bf16 result: accepted extension
    assert rc == OK
    rc, _ = _v4_phase1(**_v4_tensors(), gl_type=1)
    assert rc == OK


def test_v4_null_and_empty_arguments():
    t = _v4_tensors()
    assert _v4_phase1(**{**t, "x": None})[0] == NULLPTR
    assert _v4_phase1(**{**t, "w": None})[0] == NULLPTR
    assert _v4_phase1(**{**t, "out": None})[0] == NULLPTR
    assert _v4_phase1(**{**t, "gl": None})[0] == INVALID      # required group list missing -> invalid, not nullptr
    assert _v4_phase1(**{**t, "scale": None})[0] == INVALID   # quant case without scale
    L = _lib.lib()
    hx = acl.create_tensor_list([t["x"]])
    rc = L.aclnnGroupedMatmulV4GetWorkspaceSize(hx, hx, None, None, None, None, None, None, None, None, None, None, 3, 0, 0, 0, hx,
                                                None, None, None, None)
    assert rc == NULLPTR  # workspaceSize / executor pointers missing
    L.aclDestroyTensorList(hx)


@pytest.mark.parametrize("kw", [
    dict(group_type=1), dict(group_type=5), dict(group_type=-1), dict(split_item=0), dict(split_item=1),
    dict(gl_type=2), dict(gl_type=7), dict(act=-1), dict(act=3), dict(act=6),
])
def test_v4_invalid_attributes(kw):
    assert _v4_phase1(**_v4_tensors(), **kw)[0] == INVALID


def test_v4_invalid_shapes_and_dtypes():
    t = _v4_tensors()
    assert _v4_phase1(**{**t, "x": torch.empty((84, 5000), dtype=torch.int8)})[0] == INVALID          # K mismatch
    assert _v4_phase1(**{**t, "out": torch.empty((80, 2560), dtype=torch.bfloat16)})[0] == INVALID    # M mismatch
    assert _v4_phase1(**{**t, "out": torch.empty((84, 2000), dtype=torch.bfloat16)})[0] == INVALID    # N mismatch
    assert _v4_phase1(**{**t, "out": torch.empty((84, 2560), dtype=torch.float32)})[0] == INVALID     # y dtype
    assert _v4_phase1(**{**t, "pts": torch.empty((84,), dtype=torch.float16)})[0] == INVALID          # per-token dtype
    assert _v4_phase1(**{**t, "pts": torch.empty((80,), dtype=torch.float32)})[0] == INVALID
    assert _v4_phase1(**{**t, "pts": torch.empty((84, 1), dtype=torch.float32)})[0] == INVALID
    assert _v4_phase1(**{**t, "gl": torch.tensor([50, 65, 84], dtype=torch.int64)})[0] == INVALID     # len != E
    assert _v4_phase1(**{**t, "gl": torch.tensor([50, 65, 69, 84], dtype=torch.int32)})[0] == INVALID
    assert _v4_phase1(**{**t, "gl": torch.zeros((4, 1), dtype=torch.int64)})[0] == INVALID
    assert _v4_phase1(**{**t, "scale": torch.empty((4, 2560), dtype=torch.int64)})[0] == INVALID
    assert _v4_phase1(**{**t, "scale": torch.empty((4, 100), dtype=torch.bfloat16)})[0] == INVALID
    assert _v4_phase1(**{**t, "x": torch.empty((84, 5120), dtype=torch.float16)})[0] == INVALID       # other dtype families
    assert _v4_phase1(**{**t, "bias": torch.empty((4, 2560), dtype=torch.float32)})[0] == INVALID
    assert _v4_phase1(**{**t, "bias": torch.empty((4, 2560), dtype=torch.int32)})[0] == OK
    big = _v4_tensors(M=4, K=65536, N=16, E=1)
    assert _v4_phase1(**big)[0] == INVALID                                                              # inner axis > 65535
    hx = acl.create_tensor_list([t["x"]])
    for slot in (4, 5, 6, 9, 10, 11, 17, 18):  # offset, antiquant*, activation*, dynQuant* must be null
        assert _v4_phase1(**t, extra={slot: hx})[0] == INVALID
    _lib.lib().aclDestroyTensorList(hx)


def test_v4_int32_result_needs_no_scales_and_empty_input_needs_no_workspace():
    t = _v4_tensors(out_dtype=torch.int32)
    assert _v4_phase1(**{**t, "scale": None, "pts": None})[0] == OK
    e = _v4_tensors(M=0)
    rc, size = _v4_phase1(**e)
    assert rc == OK and size == 0
    # K == 0: x has no elements, so the reference returns success with a workspace of 0 and launches nothing
    # (CheckZeroShape and its caller, aclnn_grouped_matmul.cpp:1535-1548, 1770-1772)
    z = _v4_tensors(K=0)
    rc, size = _v4_phase1(**z)
    assert rc == OK and size == 0


def test_v4_transposed_weight_view_and_unaligned_shapes():
    t = _v4_tensors()
    wt = torch.empty((4, 2560, 5120), dtype=torch.int8).transpose(1, 2)
    assert _v4_phase1(**{**t, "w": wt})[0] == OK
    # K=5, N=10 (the reference kernel UT shape): accepted, served by the CUDA-core kernels
    u = dict(x=torch.empty((16, 5), dtype=torch.int8), w=torch.empty((2, 5, 10), dtype=torch.int8),
             scale=torch.empty((2, 10), dtype=torch.bfloat16), pts=torch.empty((16,), dtype=torch.float32),
             gl=torch.tensor([8, 8], dtype=torch.int64), out=torch.empty((16, 10), dtype=torch.bfloat16))
    assert _v4_phase1(**u, gl_type=1)[0] == OK
    # a strided x is served through a contiguous copy in the workspace: the size grows by the copy (256-byte granules)
    xs = torch.empty((84, 2 * 5120), dtype=torch.int8)[:, ::2]
    rc0, size0 = _v4_phase1(**t)
    rc1, size1 = _v4_phase1(**{**t, "x": xs})
    assert rc0 == OK and rc1 == OK and size1 == size0 + (84 * 5120 + 255) // 256 * 256
    ys = torch.empty((84, 2 * 2560), dtype=torch.bfloat16)[:, ::2]
    rc2, size2 = _v4_phase1(**{**t, "out": ys})
    assert rc2 == OK and size2 == size0 + (84 * 2560 * 2 + 255) // 256 * 256


def _sw_phase1(x, w, ws, xs, gl, q, qs, fmt_w=_lib.ACL_FORMAT_ND, null=(), api=""):
    L = _lib.lib()
    hs = dict(x=x, w=w, ws=ws, xs=xs, gl=gl, q=q, qs=qs)
    h = {k: (acl.create_tensor(v, fmt=fmt_w if k == "w" else _lib.ACL_FORMAT_ND) if (v is not None and k not in null) else None)
         for k, v in hs.items()}
    size, ex = C.c_uint64(7), C.c_void_p(0)
    rc = getattr(L, f"aclnnGroupedMatmulSwigluQuant{api}GetWorkspaceSize")(h["x"], h["w"], None, None, h["ws"], h["xs"], h["gl"],
                                                                         h["q"], h["qs"], None, C.byref(size), C.byref(ex))
    if rc == OK:
        assert L.aclDestroyAclOpExecutor(ex) == OK
    for v in h.values():
        if v:
            L.aclDestroyTensor(v)
    return rc, size.value


def _sw_tensors(m=192, k=2048, n=2048, e=4, ws_dtype=torch.float32):
    return dict(x=torch.empty((m, k), dtype=torch.int8), w=torch.empty((e, k, n), dtype=torch.int8),
                ws=torch.empty((e, n), dtype=ws_dtype), xs=torch.empty((m,), dtype=torch.float32),
                gl=torch.tensor([24 * (i + 1) for i in range(e)], dtype=torch.int64),
                q=torch.empty((m, n // 2), dtype=torch.int8), qs=torch.empty((m,), dtype=torch.float32))


def test_swiglu_valid_cases():
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        rc, size = _sw_phase1(**_sw_tensors(ws_dtype=dt))
        assert rc == OK and size > 192 * 1024 * 4
    t = _sw_tensors()
    assert _sw_phase1(**{**t, "gl": torch.tensor([10, 20], dtype=torch.int64)})[0] == OK   # list shorter than E is legal


def test_swiglu_reference_api_ut_case_is_rejected():
    # the reference's op_api UT passes an int64 weightScale and an [m, n] output: neither is valid for A8W8
    t = _sw_tensors()
    assert _sw_phase1(**{**t, "ws": torch.empty((4, 2048), dtype=torch.int64)})[0] == INVALID
    assert _sw_phase1(**{**t, "q": torch.empty((192, 2048), dtype=torch.int8)})[0] == INVALID


def test_swiglu_empty_reduction_is_rejected():
    # k == 0 leaves no row maximum to quantise by: refused with a message, as the flat entry points do
    rc, _ = _sw_phase1(**_sw_tensors(k=0))
    assert rc == INVALID and "k must be positive" in _lib.last_error()
    size = C.c_uint64(0)
    assert _lib.lib().gmmB200GroupedMatmulSwigluQuantWorkspaceSize(4, 0, 32, 1, C.byref(size)) == INVALID
    assert _lib.lib().gmmB200GroupedMatmulW8A8WorkspaceSize(1 << 31, 16, 16, 1, 27, C.byref(size)) == INVALID   # m beyond int range


def test_executor_options_are_validated_on_the_host():
    L = _lib.lib()
    t = _sw_tensors()
    hs = {k: acl.create_tensor(v) for k, v in t.items()}
    size, ex = C.c_uint64(0), C.c_void_p(0)
    assert L.aclnnGroupedMatmulSwigluQuantGetWorkspaceSize(hs["x"], hs["w"], None, None, hs["ws"], hs["xs"], hs["gl"], hs["q"], hs["qs"],
                                                           None, C.byref(size), C.byref(ex)) == OK
    assert L.gmmB200SetExecutorOptions(ex, C.byref(_lib.LaunchOptions(max_ctas=16, wait_limit_cycles=1 << 20))) == OK
    assert L.gmmB200SetExecutorOptions(ex, None) == OK                                   # null = defaults
    assert L.gmmB200SetExecutorOptions(ex, C.byref(_lib.LaunchOptions(max_ctas=-1))) == INVALID
    half = _lib.LaunchOptions(start_event=C.c_void_p(8))                                 # a start event without a stop event
    assert L.gmmB200SetExecutorOptions(ex, C.byref(half)) == INVALID
    short = _lib.LaunchOptions(max_ctas=3)
    short.structSize = 4
    assert L.gmmB200SetExecutorOptions(ex, C.byref(short)) == INVALID
    assert L.gmmB200SetExecutorOptions(None, C.byref(short)) == NULLPTR
    assert L.aclDestroyAclOpExecutor(ex) == OK
    assert L.gmmB200SetExecutorOptions(ex, C.byref(_lib.LaunchOptions())) == INVALID     # no longer live
    for h in hs.values():
        L.aclDestroyTensor(h)


def test_swiglu_null_arguments():
    t = _sw_tensors()
    for name in ("x", "w", "ws", "xs", "gl", "q", "qs"):
        assert _sw_phase1(**t, null=(name,))[0] == NULLPTR


def test_swiglu_invalid_shapes_dtypes_limits():
    t = _sw_tensors()
    assert _sw_phase1(**{**t, "x": torch.empty((192, 2048, 1), dtype=torch.int8)})[0] == INVALID
    assert _sw_phase1(**{**t, "w": torch.empty((4, 2000, 2048), dtype=torch.int8)})[0] == INVALID
    assert _sw_phase1(**{**t, "xs": torch.empty((100,), dtype=torch.float32)})[0] == INVALID
    assert _sw_phase1(**{**t, "xs": torch.empty((192,), dtype=torch.float16)})[0] == INVALID
    assert _sw_phase1(**{**t, "qs": torch.empty((192,), dtype=torch.float16)})[0] == INVALID
    assert _sw_phase1(**{**t, "q": torch.empty((192, 1024), dtype=torch.int32)})[0] == INVALID
    assert _sw_phase1(**{**t, "gl": torch.tensor([1, 2, 3, 4, 5], dtype=torch.int64)})[0] == INVALID   # longer than E
    assert _sw_phase1(**{**t, "gl": torch.tensor([1, 2, 3, 4], dtype=torch.int32)})[0] == INVALID
    odd = _sw_tensors(m=8, k=64, n=34)
    odd["ws"] = torch.empty((4, 33), dtype=torch.float32)
    assert _sw_phase1(**odd)[0] == INVALID                                                                  # N odd
    assert _sw_phase1(**_sw_tensors(m=4, k=64, n=10242, e=1))[0] == INVALID                                 # N > 10240
    assert _sw_phase1(**_sw_tensors(m=2, k=65536, n=32, e=1))[0] == INVALID                                 # K >= 65536
    e = _sw_tensors(m=0)
    rc, size = _sw_phase1(**e)
    assert rc == OK and size == 0


def test_fractal_nz_weights_and_twin_entry_points():
    NZ = _lib.ACL_FORMAT_FRACTAL_NZ
    # swiglu: E=4, K=2048, N=2048 -> storage [4, 64, 128, 16, 32]
    t = _sw_tensors()
    w5 = torch.empty((4, 64, 128, 16, 32), dtype=torch.int8)
    assert _sw_phase1(**{**t, "w": w5}, fmt_w=NZ)[0] == OK
    assert _sw_phase1(**{**t, "w": w5}, api="WeightNZ")[0] == OK                 # storage counted as NZ whatever the format
    assert _sw_phase1(**{**t, "w": w5})[0] == INVALID                            # 5-D weight that is not NZ
    assert _sw_phase1(**t, api="WeightNZ")[0] == INVALID                         # WeightNZ wants a 5-D storage shape
    assert "storageShape" in _lib.last_error()
    assert _sw_phase1(**{**t, "w": torch.empty((4, 64, 127, 16, 32), dtype=torch.int8)}, fmt_w=NZ)[0] == INVALID
    assert _sw_phase1(**{**t, "w": torch.empty((4, 64, 128, 32, 16), dtype=torch.int8)}, fmt_w=NZ)[0] == INVALID
    assert _sw_phase1(**t, fmt_w=NZ)[0] == OK                                    # 3-D view over NZ storage
    odd = _sw_tensors(m=8, k=40, n=64, e=1)
    assert _sw_phase1(**odd, fmt_w=NZ)[0] == INVALID                             # K % 16 != 0
    assert _sw_phase1(**t, fmt_w=3)[0] == INVALID                                # another private format (NC1HWC0)
    # grouped_matmul: E=4, K=5120, N=2560 -> [4, 80, 320, 16, 32]
    v = _v4_tensors()
    v5d = torch.empty((4, 80, 320, 16, 32), dtype=torch.int8)
    for api in ("V4", "V5"):
        assert _v4_phase1(**{**v, "w": v5d}, fmt_w=NZ, api=api)[0] == OK
        assert _v4_phase1(**v, fmt_w=NZ, api=api)[0] == OK
        assert _v4_phase1(**{**v, "w": v5d}, api=api)[0] == INVALID
    assert _v4_phase1(**{**v, "w": v5d}, api="WeightNz")[0] == OK
    assert _v4_phase1(**v, api="WeightNz")[0] == OK
    assert _v4_phase1(**{**v, "w": v5d}, api="WeightNz", tuning=[21], quant_group_size=0)[0] == OK
    assert _v4_phase1(**{**v, "w": v5d}, api="WeightNz", quant_group_size=-1)[0] == INVALID
    assert _v4_phase1(**{**v, "w": v5d}, api="V5", fmt_w=NZ, tuning=[-3])[0] == INVALID
    assert _v4_phase1(**{**v, "w": torch.empty((4, 80, 319, 16, 32), dtype=torch.int8)}, api="WeightNz")[0] == INVALID
    u = dict(x=torch.empty((16, 24), dtype=torch.int8), w=torch.empty((2, 24, 32), dtype=torch.int8),
             scale=torch.empty((2, 32), dtype=torch.bfloat16), pts=torch.empty((16,), dtype=torch.float32),
             gl=torch.tensor([8, 16], dtype=torch.int64), out=torch.empty((16, 32), dtype=torch.bfloat16))
    assert _v4_phase1(**u, api="WeightNz")[0] == INVALID                         # K % 16 != 0
    assert _v4_phase1(**u)[0] == OK


def test_v4_float16_result_and_activations():
    t = _v4_tensors(scale_dtype=torch.float32, out_dtype=torch.float16)
    assert _v4_phase1(**t)[0] == OK
    assert _v4_phase1(**_v4_tensors(out_dtype=torch.float16))[0] == INVALID      # float16 result needs a float32 scale
    for act in (1, 2, 4, 5):
        assert _v4_phase1(**_v4_tensors(), act=act)[0] == OK
    assert _v4_phase1(**_v4_tensors(), act=3)[0] == INVALID
    assert "GELU_ERR_FUNC" in _lib.last_error()


def _fr_tensors(m=192, k=2048, n=7168, e=4, batch=24, shared=8):
    return dict(x=torch.empty((m, k), dtype=torch.int8), w=torch.empty((e, n // 32, k // 16, 16, 32), dtype=torch.int8),
                scale=torch.empty((e, n), dtype=torch.float32), bias=None, pts=torch.empty((m,), dtype=torch.float32),
                gl=torch.empty((e,), dtype=torch.int64), shared=torch.empty((shared, n), dtype=torch.bfloat16),
                logit=torch.empty((m,), dtype=torch.float32), ri=torch.empty((m,), dtype=torch.int64),
                out=torch.empty((batch, n), dtype=torch.float32))


def _fr_phase1(x, w, scale, bias, pts, gl, shared, logit, ri, out, dtype=0, weight=1.0, offset=0, tx=False, tw=False, gl_type=1,
               fmt_w=_lib.ACL_FORMAT_FRACTAL_NZ, view_3d=True, api="", tuning=None, v2_offset=None):
    L = _lib.lib()
    hs = []

    def mk(t, **kw):
        if t is None:
            return None
        h = acl.create_tensor(t, **kw)
        hs.append(h)
        return h
    view = None
    if w is not None and view_3d and w.dim() == 5:
        view = [w.shape[0], w.shape[2] * 16, w.shape[1] * 32]
    hw = mk(w, fmt=fmt_w, view_dims=view)
    hx, hsc, hb, hp, hg, hsh, hl, hr, hy = (mk(t) for t in (x, scale, bias, pts, gl, shared, logit, ri, out))
    size, ex = C.c_uint64(9), C.c_void_p(0)
    if api == "V2":
        ht = L.aclCreateIntArray((C.c_int64 * len(tuning))(*tuning), len(tuning)) if tuning is not None else None
        rc = L.aclnnGroupedMatmulFinalizeRoutingWeightNzV2GetWorkspaceSize(hx, hw, hsc, hb, mk(v2_offset), None, None, hp, hg, hsh, hl, hr,
                                                                           dtype, weight, offset, tx, tw, gl_type, ht, hy,
                                                                           C.byref(size), C.byref(ex))
        if ht:
            L.aclDestroyIntArray(ht)
    else:
        rc = L.aclnnGroupedMatmulFinalizeRoutingWeightNzGetWorkspaceSize(hx, hw, hsc, hb, hp, hg, hsh, hl, hr, dtype, weight, offset, tx,
                                                                         tw, gl_type, hy, C.byref(size), C.byref(ex))
    if rc == OK:
        assert L.aclDestroyAclOpExecutor(ex) == OK
    for h in hs:
        L.aclDestroyTensor(h)
    return rc, size.value


def test_finalize_routing_phase1_status_codes():
    NZ = _lib.ACL_FORMAT_FRACTAL_NZ
    t = _fr_tensors()   # the reference's example: m=192, k=2048, n=7168, e=4, batch=24, 8 shared rows
    rc, size = _fr_phase1(**t)
    assert rc == OK and size >= 256
    assert _fr_phase1(**t, view_3d=False)[0] == OK                                   # 5-dimensional view
    assert _fr_phase1(**t, api="V2", tuning=[48])[0] == OK
    assert _fr_phase1(**{**t, "scale": torch.empty((4, 7168), dtype=torch.bfloat16)})[0] == OK
    assert _fr_phase1(**{**t, "ri": torch.empty((192,), dtype=torch.int32)})[0] == OK
    assert _fr_phase1(**{**t, "bias": torch.empty((4, 7168), dtype=torch.bfloat16)})[0] == OK
    assert _fr_phase1(**{**t, "pts": None})[0] == OK
    assert _fr_phase1(**{**t, "shared": None, "logit": None})[0] == OK               # scene 2: plain stores
    # the two scenes are the only legal combinations of null arguments
    assert _fr_phase1(**{**t, "shared": None})[0] == NULLPTR
    assert _fr_phase1(**{**t, "logit": None})[0] == NULLPTR
    for name in ("x", "w", "scale", "gl", "ri"):
        assert _fr_phase1(**{**t, name: None})[0] == NULLPTR
    assert _fr_phase1(**{**t, "out": None})[0] == NULLPTR
    # attributes
    assert _fr_phase1(**t, dtype=1)[0] == INVALID
    assert _fr_phase1(**t, tx=True)[0] == INVALID
    assert _fr_phase1(**t, tw=True)[0] == INVALID
    assert _fr_phase1(**t, gl_type=0)[0] == INVALID
    assert "groupListType" in _lib.last_error()
    assert _fr_phase1(**t, offset=-1)[0] == INVALID
    assert _fr_phase1(**t, offset=17)[0] == INVALID                                  # 17 + 8 shared rows > batch 24
    assert _fr_phase1(**t, offset=16)[0] == OK
    assert _fr_phase1(**t, api="V2", tuning=[193])[0] == INVALID
    assert _fr_phase1(**t, api="V2", tuning=[-1])[0] == INVALID
    assert _fr_phase1(**t, api="V2", v2_offset=torch.empty((4, 1, 7168), dtype=torch.float32))[0] == INVALID
    # formats, dtypes, shapes
    assert _fr_phase1(**t, fmt_w=_lib.ACL_FORMAT_ND)[0] == INVALID                   # this entry point wants the NZ weight
    assert _fr_phase1(**{**t, "w": torch.empty((4, 2048, 7168), dtype=torch.int8)})[0] == INVALID   # NZ format over an ND storage shape
    assert _fr_phase1(**{**t, "out": torch.empty((24, 7168), dtype=torch.bfloat16)})[0] == INVALID
    assert _fr_phase1(**{**t, "scale": torch.empty((4, 7168), dtype=torch.int64)})[0] == INVALID
    assert _fr_phase1(**{**t, "bias": torch.empty((4, 7168), dtype=torch.float32)})[0] == INVALID
    assert _fr_phase1(**{**t, "ri": torch.empty((192,), dtype=torch.float32)})[0] == INVALID
    assert _fr_phase1(**{**t, "ri": torch.empty((100,), dtype=torch.int64)})[0] == INVALID
    assert _fr_phase1(**{**t, "logit": torch.empty((100,), dtype=torch.float32)})[0] == INVALID
    assert _fr_phase1(**{**t, "gl": torch.empty((3,), dtype=torch.int64)})[0] == INVALID
    assert _fr_phase1(**{**t, "shared": torch.empty((25, 7168), dtype=torch.bfloat16)})[0] == INVALID  # more shared rows than batch
    assert _fr_phase1(**{**t, "shared": torch.empty((8, 7000), dtype=torch.bfloat16)})[0] == INVALID
    assert _fr_phase1(**{**t, "out": torch.empty((193, 7168), dtype=torch.float32)})[0] == INVALID     # batch > m
    assert _fr_phase1(**{**t, "x": torch.empty((192, 2032), dtype=torch.int8)})[0] == INVALID          # k mismatch
    small = _fr_tensors(m=16, k=64, n=128, e=2, batch=4, shared=2)
    assert _fr_phase1(**small)[0] == INVALID                                                            # n < 256
    assert _fr_phase1(**_fr_tensors(m=16, k=64, n=256, e=2, batch=4, shared=2))[0] == OK
    assert _fr_phase1(**{**t, "shared": torch.empty((0, 7168), dtype=torch.bfloat16)})[0] == INVALID   # empty tensors are refused


def _ir_phase1(n=8, k=2, h=64, E=16, rng_=(0, 16), quant=1, x_dtype=torch.bfloat16, out_dtype=None, count_type=1, row_idx_type=1,
               drop=0, flag=True, active_num=None, scale=None, null=(), counts_shape=None, idx_dtype=torch.int32, **over):
    L = _lib.lib()
    if out_dtype is None:
        out_dtype = torch.int8 if quant == 1 else x_dtype
    t = dict(x=torch.empty((n, h), dtype=x_dtype), idx=torch.empty((n, k), dtype=idx_dtype), scale=scale,
             ex=torch.empty((n * k, h), dtype=out_dtype), ri=torch.empty((n * k,), dtype=torch.int32),
             cnt=torch.empty(counts_shape or (((rng_[1] - rng_[0]) if rng_ else 1,) if count_type == 1 else (E, 2)), dtype=torch.int64),
             es=torch.empty((n * k,), dtype=torch.float32))
    t.update(over)
    h_ = {name: (acl.create_tensor(v) if (v is not None and name not in null) else None) for name, v in t.items()}
    ra = L.aclCreateIntArray((C.c_int64 * len(rng_))(*rng_), len(rng_)) if rng_ is not None else None
    size, ex = C.c_uint64(5), C.c_void_p(0)
    rc = L.aclnnMoeInitRoutingV3GetWorkspaceSize(h_["x"], h_["idx"], h_["scale"], None, n * k if active_num is None else active_num, 0, E,
                                                 drop, count_type, flag, quant, ra, row_idx_type, h_["ex"], h_["ri"], h_["cnt"], h_["es"],
                                                 C.byref(size), C.byref(ex))
    if rc == OK:
        assert L.aclDestroyAclOpExecutor(ex) == OK
    for v in h_.values():
        if v:
            L.aclDestroyTensor(v)
    if ra:
        L.aclDestroyIntArray(ra)
    return rc, size.value


def test_moe_init_routing_v3_phase1_status_codes():
    rc, size = _ir_phase1()
    assert rc == OK and size >= 256
    assert _ir_phase1(quant=-1)[0] == OK
    assert _ir_phase1(quant=-1, x_dtype=torch.int8)[0] == OK
    assert _ir_phase1(x_dtype=torch.float32)[0] == OK and _ir_phase1(x_dtype=torch.float16)[0] == OK
    assert _ir_phase1(count_type=2)[0] == OK and _ir_phase1(row_idx_type=0)[0] == OK
    assert _ir_phase1(rng_=(4, 12), scale=torch.empty((8, 64), dtype=torch.float32))[0] == OK      # smooth scale [range, h]
    assert _ir_phase1(quant=-1, scale=torch.empty((8,), dtype=torch.float32))[0] == OK             # per-token scale [n]
    assert _ir_phase1(n=0)[0] == OK and _ir_phase1(n=0)[1] == 0
    for name in ("x", "idx", "ex", "ri", "cnt", "es"):
        assert _ir_phase1(null=(name,))[0] == NULLPTR
    assert _ir_phase1(idx_dtype=torch.int64)[0] == INVALID
    assert _ir_phase1(x_dtype=torch.int8)[0] == INVALID                                            # dynamic quant of int8 rows
    assert _ir_phase1(out_dtype=torch.bfloat16)[0] == INVALID                                      # quant output must be int8
    assert _ir_phase1(quant=-1, out_dtype=torch.float32)[0] == INVALID
    # the example of the reference's documentation (x float32 [3,2], top-4, quantMode -1, per-token scale [3], expertNum 256, range
    # [0,4) ...) declares an int8 expandedXOut: refused, float32 rows do not fit it; with a float32 output the call is accepted
    doc = dict(n=3, k=4, h=2, E=256, rng_=(0, 4), quant=-1, x_dtype=torch.float32, scale=torch.empty((3,), dtype=torch.float32))
    assert _ir_phase1(**doc, out_dtype=torch.int8)[0] == INVALID
    assert _ir_phase1(**doc)[0] == OK
    assert _ir_phase1(quant=0)[0] == INVALID and _ir_phase1(quant=2)[0] == INVALID                 # static quant is not supported
    assert _ir_phase1(drop=1)[0] == INVALID and _ir_phase1(flag=False)[0] == INVALID
    assert _ir_phase1(count_type=0)[0] == INVALID and _ir_phase1(row_idx_type=2)[0] == INVALID
    assert _ir_phase1(active_num=5)[0] == INVALID
    assert _ir_phase1(rng_=(4, 4))[0] == INVALID and _ir_phase1(rng_=(0, 17))[0] == INVALID and _ir_phase1(rng_=None)[0] == INVALID
    assert _ir_phase1(E=10241, rng_=(0, 16))[0] == INVALID
    assert _ir_phase1(count_type=2, E=5121, rng_=(0, 16))[0] == INVALID
    assert _ir_phase1(counts_shape=(15,))[0] == INVALID
    assert _ir_phase1(scale=torch.empty((16, 32), dtype=torch.float32))[0] == INVALID
    assert _ir_phase1(scale=torch.empty((16, 64), dtype=torch.float16))[0] == INVALID
    assert _ir_phase1(ex=torch.empty((15, 64), dtype=torch.int8))[0] == INVALID
    assert _ir_phase1(ri=torch.empty((16,), dtype=torch.int64))[0] == INVALID
    assert _ir_phase1(idx=torch.empty((7, 2), dtype=torch.int32))[0] == INVALID


def test_finalize_routing_reference_unit_test_cases():
    """The status codes the reference's own op_api unit tests pin for aclnnGroupedMatmulFinalizeRoutingWeightNz
    (gmm/grouped_matmul_finalize_routing/tests/ut/op_host/op_api/test_aclnn_grouped_matmul_finalize_routing_weight_nz_l2.cpp:41-621):
    m=192, k=2048, n=7168, e=4, bs=24, bsdp=8, weight viewed [e,k,n] over storage [e, n/32, k/16, 16, 32]."""
    i8, f32, bf = torch.int8, torch.float32, torch.bfloat16
    m, k, n, e, bs, bsdp = 192, 2048, 7168, 4, 24, 8
    t = _fr_tensors(m, k, n, e, bs, bsdp)
    assert _fr_phase1(**t)[0] == OK                                                              # normal_case_add_value (:41)
    assert _fr_phase1(**{**t, "logit": None, "ri": None})[0] == NULLPTR                          # shared_input_null (:68)
    assert _fr_phase1(**{**t, "bias": torch.empty((e, n), dtype=bf)})[0] == OK                   # bias_not_null (:94)
    assert _fr_phase1(**{**t, "w": torch.empty((e, k, n), dtype=i8)}, fmt_w=_lib.ACL_FORMAT_ND)[0] == INVALID   # x2_not_nz (:121)
    assert _fr_phase1(**{**t, "w": None})[0] == NULLPTR                                          # x2_null (:147)
    assert _fr_phase1(**t, dtype=1)[0] == INVALID                                                # dtype_not_0 (:172)
    assert _fr_phase1(**{**t, "scale": torch.empty((e + 1, n), dtype=f32)})[0] == INVALID        # scale_noteq_e (:198)
    assert _fr_phase1(**{**t, "pts": torch.empty((m + 1,), dtype=f32)})[0] == INVALID            # perTokenScale_noteq_m (:224)
    assert _fr_phase1(**{**t, "shared": torch.empty((bs + 1, n), dtype=bf)})[0] == INVALID       # shared_input_more_than_bs (:250)
    assert _fr_phase1(**{**t, "x": torch.empty((0, k), dtype=i8)})[0] == INVALID                 # view_shape_0 (:302)
    assert _fr_phase1(**{**t, "x": torch.empty((m,), dtype=i8)})[0] == INVALID                   # x12_viewdims_wrong (:328)
    assert _fr_phase1(**{**t, "shared": torch.empty((bsdp + 1, n + 1), dtype=bf)})[0] == INVALID  # shareinput_outputBS_noeq (:354)
    assert _fr_phase1(**{**t, "logit": torch.empty((m + 1,), dtype=f32)})[0] == INVALID          # logit_1stdim_noeq_xMdim (:380)
    assert _fr_phase1(**{**t, "ri": torch.empty((m + 1,), dtype=torch.int64)})[0] == INVALID     # rowindex1stdim_noeq_xMdim (:407)
    assert _fr_phase1(**{**t, "gl": torch.empty((e + 1,), dtype=torch.int64)})[0] == INVALID     # groupListdim_wrong (:434)
    assert _fr_phase1(**_fr_tensors(m, k, 224, e, bs, bsdp))[0] == INVALID                       # nvalid (:488, n = 7000 there): n % 32, n >= 256
    assert _fr_phase1(**{**t, "x": torch.empty((m, 4098), dtype=i8)})[0] == INVALID              # not_support_k_shape (:515)
    assert _fr_phase1(**{**t, "w": torch.empty((e, n // 32, k // 16, 16, 32), dtype=torch.int32)})[0] == INVALID   # x1_type_not_same_with_x2 (:542)
    assert _fr_phase1(**{**t, "x": torch.empty((m, k - 1), dtype=i8)})[0] == INVALID             # k_n_not_support_w8a8 (:596)


def test_second_phase_host_checks():
    L = _lib.lib()
    assert L.aclnnGroupedMatmulV4(None, 0, None, None) == NULLPTR
    assert L.aclnnGroupedMatmulSwigluQuant(None, 0, None, None) == NULLPTR
    # an executor built by one operator cannot be run by the other, and cannot be run twice
    t = _sw_tensors(m=0)
    h = {k: acl.create_tensor(v) for k, v in t.items()}
    size, ex = C.c_uint64(0), C.c_void_p(0)
    assert L.aclnnGroupedMatmulSwigluQuantGetWorkspaceSize(h["x"], h["w"], None, None, h["ws"], h["xs"], h["gl"], h["q"], h["qs"], None,
                                                           C.byref(size), C.byref(ex)) == OK
    assert L.aclnnGroupedMatmulV4(None, 0, ex, None) == INVALID
    assert L.aclnnGroupedMatmulSwigluQuant(None, 0, ex, None) == INVALID          # consumed by the failed call above
    assert L.aclnnGroupedMatmulSwigluQuantGetWorkspaceSize(h["x"], h["w"], None, None, h["ws"], h["xs"], h["gl"], h["q"], h["qs"], None,
                                                           C.byref(size), C.byref(ex)) == OK
    assert L.aclnnGroupedMatmulSwigluQuant(None, 0, ex, None) == OK               # empty problem: nothing to launch
    assert L.aclnnGroupedMatmulSwigluQuant(None, 0, ex, None) == INVALID          # single use
    for v in h.values():
        L.aclDestroyTensor(v)


def test_flat_entry_points_validate_on_the_host():
    L = _lib.lib()
    size = C.c_uint64(0)
    assert L.gmmB200GroupedMatmulSwigluQuantWorkspaceSize(32768, 7168, 4096, 32, C.byref(size)) == OK
    assert size.value >= 32768 * 2048 * 4
    assert L.gmmB200GroupedMatmulSwigluQuantWorkspaceSize(16, 64, 33, 1, C.byref(size)) == INVALID
    assert L.gmmB200GroupedMatmulW8A8WorkspaceSize(256, 1024, 2048, 4, _lib.ACL_BF16, C.byref(size)) == OK and size.value == 256
    assert L.gmmB200GroupedMatmulW8A8WorkspaceSize(256, 1024, 2048, 4, _lib.ACL_FLOAT16, C.byref(size)) == OK
    assert L.gmmB200GroupedMatmulW8A8WorkspaceSize(256, 1024, 2048, 4, _lib.ACL_FLOAT, C.byref(size)) == INVALID
    one = C.c_void_p(256)
    assert L.gmmB200GroupedMatmulW8A8(None, one, one, 0, one, None, 0, one, 1, 0, 1, 16, 16, 1, 0, 0, None, None, 0, 0, one, 27, one, 256, None, None) == NULLPTR
    assert L.gmmB200GroupedMatmulW8A8(one, one, one, 0, one, None, 0, one, 2, 0, 1, 16, 16, 1, 0, 0, None, None, 0, 0, one, 27, one, 256, None, None) == INVALID
    assert L.gmmB200GroupedMatmulSwigluQuant(one, one, one, 0, one, one, 1, 4, 16, 32, 1, 0, one, one, one, 16, None, None) == INVALID  # workspace too small
    assert "workspaceSize" in _lib.last_error()
