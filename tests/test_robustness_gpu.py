"""Failure handling of the CUDA path, exercised without faulting the GPU.

* A bounded device-side wait is made to run out by a host-made inconsistency (the copy-issuing warp of ONE CTA is told
  to leave one K block out of its last tile, so the warp that consumes the blocks waits for something that never comes):
  the kernel must return, gmmB200CheckStatus must report ACLNN_ERR_RUNTIME_ERROR (361001) with the record filled, and
  the next ordinary call on the same workspace must be correct.  No trap, no endless loop, no access outside the call's
  own buffers is involved.  The reference's counterpart is the timeout stamping of its dispatch kernel
  (mc2/moe_distribute_dispatch_v2/op_kernel/moe_distribute_dispatch_v2.h:44, 1103-1118).
* A scattered result row whose index names no peer GPU or no row of the result is skipped and reported, not stored.
* Per-call launch options: a CTA cap of 1 still gives the right result (also for the cross-CTA requantisation of
  swiglu_quant), and options are rejected on an executor that is no longer live.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from ops_transformer_b200 import _lib, synth  # noqa: E402

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _gmm_inputs(dev, M, K, N, E, seed):
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    x, w = synth.int8_tensor((M, K), seed, 1), synth.int8_tensor((E, K, N), seed, 2)
    ws, xs = synth.scale_tensor((E, N), seed, 3), synth.scale_tensor((M,), seed, 4)
    return (x, w, ws, xs), (t(x), t(w), t(ws), t(xs))


def test_bounded_wait_runs_out_and_the_workspace_stays_usable(oracle):
    import ops_transformer_b200 as ops
    dev = _dev()
    M, K, N, E = 96, 512, 256, 1           # one tile of four K blocks
    (x, w, ws, xs), (xt, wt, wst, xst) = _gmm_inputs(dev, M, K, N, E, 41)
    gl = torch.tensor([M], dtype=torch.int64, device=dev)
    out = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    wsb = torch.zeros(4096, dtype=torch.uint8, device=dev)
    # ~1 ms wait bound, one CTA, the producer leaves out the tile's last K block
    opts = ops.LaunchOptions(max_ctas=1, wait_limit_cycles=2_000_000, test_skip_k_blocks=1)
    ops.grouped_matmul_v4(xt, wt, wst, xst, gl, out=out, workspace=wsb, options=opts)
    with pytest.raises(ops.AclnnError) as ei:
        ops.check_status(wsb)
    assert ei.value.status == _lib.ACLNN_ERR_RUNTIME_ERROR
    code, cta, role, _ = ei.value.record
    assert code == 1 and cta == 0 and 300 <= role < 500, ei.value.record   # the MMA issuer (3xx) or an epilogue warp (4xx) gave up first
    # the context is intact and the same workspace serves the next, ordinary call
    out2 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    ops.grouped_matmul_v4(xt, wt, wst, xst, gl, out=out2, workspace=wsb)
    ops.check_status(wsb)
    ref = oracle.gmm_w8a8(x, w, ws, xs, np.array([M], np.int64), 0)["y"]
    assert np.array_equal(out2.view(torch.int16).cpu().numpy().view(np.uint16), ref)


def test_scatter_index_outside_the_result_is_skipped_and_reported(oracle):
    import ops_transformer_b200 as ops
    dev = _dev()
    M, K, N, E = 70, 256, 256, 2
    (x, w, ws, xs), (xt, wt, wst, xst) = _gmm_inputs(dev, M, K, N, E, 42)
    counts = np.array([30, 40], np.int64)
    gl = torch.from_numpy(np.cumsum(counts)).to(dev)
    perm = np.random.default_rng(3).permutation(M).astype(np.int64)
    bad_row = 17
    perm_bad = perm.copy()
    perm_bad[bad_row] = M + 5                       # beyond the result
    out = torch.full((M, N), 0x7fc1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    _, wsb = ops.grouped_matmul_v4(xt, wt, wst, xst, gl, out=out, out_row_index=torch.from_numpy(perm_bad).to(dev),
                                   return_workspace=True)
    with pytest.raises(ops.AclnnError) as ei:
        ops.check_status(wsb)
    assert ei.value.record[0] == 2 and ei.value.record[3] == bad_row, ei.value.record
    ref = oracle.gmm_w8a8(x, w, ws, xs, np.cumsum(counts), 0)["y"]
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    keep = np.arange(M) != bad_row
    assert np.array_equal(got[perm[keep]], ref[keep])
    assert (got[perm[bad_row]] == 0x7fc1).all(), "the row with the bad index must not be stored anywhere"
    # a gpu field that names no peer: same treatment
    peers_bad = perm.copy() | (np.int64(3) << 40)
    out3 = torch.full((M, N), 0x7fc1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    _, wsb = ops.grouped_matmul_v4(xt, wt, wst, xst, gl, out=None, out_row_index=torch.from_numpy(peers_bad).to(dev),
                                   out_peers=[out3.data_ptr()], out_rows=M, return_workspace=True)
    with pytest.raises(ops.AclnnError):
        ops.check_status(wsb)
    assert bool((out3.view(torch.int16) == 0x7fc1).all())


def test_dispatch_skips_and_counts_rows_with_a_bad_destination():
    dev = _dev()
    L = _lib.lib()
    rows, hidden, cap = 6, 64, 8
    x = torch.randint(-127, 128, (rows, hidden), dtype=torch.int8, device=dev)
    xs = torch.rand(rows, device=dev)
    src = torch.arange(rows, dtype=torch.int64, device=dev)
    dest = torch.tensor([0, 1, (5 << 40) | 2, 3, cap + 1, -1], dtype=torch.int64, device=dev)   # row 2: no such peer; row 4: beyond capacity
    bx = torch.full((cap, hidden), 99, dtype=torch.int8, device=dev)
    bs = torch.full((cap,), -1.0, dtype=torch.float32, device=dev)
    overflow = torch.zeros(1, dtype=torch.int32, device=dev)
    px, ps = (C.c_void_p * 1)(bx.data_ptr()), (C.c_void_p * 1)(bs.data_ptr())
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    rc = L.gmmB200EpDispatch(p(x), p(xs), p(src), p(dest), rows, hidden, cap, px, ps, 1, p(overflow), None, 0,
                             C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert int(overflow.item()) == 2
    assert torch.equal(bx[0], x[0]) and torch.equal(bx[1], x[1]) and torch.equal(bx[3], x[3])
    assert bool((bx[2] == 99).all()) and bool((bx[4:] == 99).all())


@pytest.mark.parametrize("ctas", ["1", "2"])
@pytest.mark.parametrize("max_ctas", [1, 3, 7])
def test_cta_cap_per_call_swiglu_quant(oracle, monkeypatch, max_ctas, ctas):
    """With fewer CTAs than N tiles of a row block the requantisation of a block depends on tiles the same CTA computes
    later; the kernel must not wait for them.  Both tile shapes (single CTAs, CTA pairs; a cap of 1 forces single CTAs)."""
    import ops_transformer_b200 as ops
    dev = _dev()
    monkeypatch.setenv("GMM_B200_CTAS", ctas)
    counts = np.array([300, 0, 130, 513], np.int64)
    M, K, N, E = int(counts.sum()), 256, 2048, 4     # 8 N tiles per row block
    (x, w, ws, xs), (xt, wt, wst, xst) = _gmm_inputs(dev, M, K, N, E, 43)
    gl = torch.from_numpy(np.cumsum(counts)).to(dev)
    q, qs, wsb = ops.grouped_matmul_swiglu_quant(xt, wt, wst, xst, gl, return_workspace=True,
                                                 options=ops.LaunchOptions(max_ctas=max_ctas, wait_limit_cycles=200_000_000))
    ops.check_status(wsb)
    ref = oracle.swiglu_quant(x, w, ws, xs, np.cumsum(counts))
    rel = np.abs(qs.cpu().numpy() - ref["q_scale"]) / np.abs(ref["q_scale"])
    assert rel.max() <= 1e-6
    d = np.abs(q.cpu().numpy().astype(np.int32) - ref["q"].astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) / d.size <= 1e-4


def test_two_swiglu_calls_overlapping_on_two_streams(oracle):
    """Two persistent launches that each want every SM: their CTAs are not all resident together.  Nothing in the kernel
    waits for another CTA (the wave pacing is a bounded hint), so both calls finish without a timeout and are correct."""
    import ops_transformer_b200 as ops
    dev = _dev()
    counts = np.array([700, 300, 0, 1100, 520], np.int64)
    M, K, N, E = int(counts.sum()), 1024, 2048, 5
    gl = torch.from_numpy(np.cumsum(counts)).to(dev)
    sets = [_gmm_inputs(dev, M, K, N, E, 44 + i) for i in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = []
    torch.cuda.synchronize()
    for rep in range(3):
        outs = []
        for (host, devt), st in zip(sets, streams):
            with torch.cuda.stream(st):
                wsb = torch.empty(64 << 20, dtype=torch.uint8, device=dev)   # one workspace per call
                q, qs, wsb = ops.grouped_matmul_swiglu_quant(*devt, gl, stream=st, workspace=wsb, return_workspace=True,
                                                             options=ops.LaunchOptions(wait_limit_cycles=400_000_000))
                outs.append((q, qs, wsb, st))
        for q, qs, wsb, st in outs:
            ops.check_status(wsb, stream=st)
    for (host, _), (q, qs, _, _) in zip(sets, outs):
        ref = oracle.swiglu_quant(*host, np.cumsum(counts))
        rel = np.abs(qs.cpu().numpy() - ref["q_scale"]) / np.abs(ref["q_scale"])
        assert rel.max() <= 1e-6
        d = np.abs(q.cpu().numpy().astype(np.int32) - ref["q"].astype(np.int32))
        assert d.max() <= 1 and np.count_nonzero(d) / d.size <= 1e-4


def test_options_are_per_executor_and_need_a_live_executor(gmm_lib):
    _dev()
    opts = _lib.LaunchOptions(max_ctas=4)
    assert gmm_lib.gmmB200SetExecutorOptions(None, C.byref(opts)) == _lib.ACLNN_ERR_PARAM_NULLPTR
    assert gmm_lib.gmmB200SetExecutorOptions(C.c_void_p(0x1000), C.byref(opts)) == _lib.ACLNN_ERR_PARAM_INVALID
