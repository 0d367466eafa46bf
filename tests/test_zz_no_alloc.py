"""The allocation-free entry point, gmmB200GroupedMatmulSwigluQuantNoAlloc, against the workspace-taking one.

Some callers of the library cannot allocate device memory when they invoke the operator (a frozen memory pool,
a host runtime that owns the allocator, a loop that cannot take cudaMalloc's device-wide synchronisation), so
this entry point keeps its scratch in a fixed array inside the library.  The test drives it through the C ABI
twice in a row, with different inputs, so that the second call runs over what the first one left behind in the
shared array, and compares each result with the existing entry point on the same inputs and with the CPU oracle,
within the same bars as the other parity tests (scales 1e-6 relative, int8 values at most 1 LSB apart on at most
0.01 % of elements; both GPU paths run the same kernels, so their results are in fact expected to be identical).
It also reads the kernels' status record through gmmB200NoAllocCheckStatus (the record lives in the built-in array,
which the caller cannot address) and checks that the device's free memory does not change across the second call.
This file is collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from ops_transformer_b200 import _lib, synth  # noqa: E402

pytestmark = pytest.mark.gpu


def _run_pair(L, dev, oracle, seed, M, K, N, E, counts, check_memory=False):
    hx, hw = synth.int8_tensor((M, K), seed, 1), synth.int8_tensor((E, K, N), seed, 2)
    hws, hxs = synth.scale_tensor((E, N), seed, 3), synth.scale_tensor((M,), seed, 4)
    x, w, ws, xs = (torch.from_numpy(a).to(dev) for a in (hx, hw, hws, hxs))
    gl = torch.from_numpy(np.cumsum(counts).astype(np.int64)).to(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731

    # existing entry point, caller-provided workspace
    size = C.c_uint64(0)
    assert L.gmmB200GroupedMatmulSwigluQuantWorkspaceSize(M, K, N, E, C.byref(size)) == 0
    wsb = torch.empty(int(size.value), dtype=torch.uint8, device=dev)
    q_ref = torch.full((M, N // 2), 99, dtype=torch.int8, device=dev)
    qs_ref = torch.full((M,), -1.0, dtype=torch.float32, device=dev)
    rc = L.gmmB200GroupedMatmulSwigluQuant(p(x), p(w), p(ws), _lib.ACL_FLOAT, p(xs), p(gl), len(counts), M, K, N, E, 0, p(q_ref),
                                           p(qs_ref), p(wsb), size.value, stream, None)
    assert rc == 0, _lib.last_error()
    assert L.gmmB200CheckStatus(p(wsb), size.value, stream, None) == 0, _lib.last_error()

    # allocation-free entry point
    q = torch.full((M, N // 2), 99, dtype=torch.int8, device=dev)
    qs = torch.full((M,), -1.0, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(dev)[0]
    rc = L.gmmB200GroupedMatmulSwigluQuantNoAlloc(p(x), p(w), p(ws), _lib.ACL_FLOAT, p(xs), p(gl), len(counts), M, K, N, E, p(q),
                                                  p(qs), stream)
    assert rc == 0, _lib.last_error()
    rec = (C.c_int32 * 4)()
    assert L.gmmB200NoAllocCheckStatus(stream, rec) == 0, (_lib.last_error(), list(rec))   # waits for the stream
    if check_memory:  # a steady-state call (the kernels are loaded by now) takes no device memory
        assert torch.cuda.mem_get_info(dev)[0] == free_before

    rows = int(np.sum(counts))
    a, b = qs.cpu().numpy(), qs_ref.cpu().numpy()
    assert (a[rows:] == -1.0).all() and (q.cpu().numpy()[rows:] == 99).all(), "rows outside group_list were written"
    rel = np.abs(a[:rows] - b[:rows]) / np.abs(b[:rows])
    assert rel.max() <= 1e-6
    d = np.abs(q.cpu().numpy()[:rows].astype(np.int32) - q_ref.cpu().numpy()[:rows].astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) / d.size <= 1e-4
    assert torch.equal(q, q_ref) and torch.equal(qs, qs_ref), "same kernels, same inputs: results should be identical"
    # and against the CPU oracle, like every other parity test
    ref = oracle.swiglu_quant(hx, hw, hws, hxs, np.cumsum(counts))
    rel = np.abs(a[:rows] - ref["q_scale"][:rows]) / np.abs(ref["q_scale"][:rows])
    assert rel.max() <= 1e-6
    d = np.abs(q.cpu().numpy()[:rows].astype(np.int32) - ref["q"][:rows].astype(np.int32))
    assert d.max() <= 1 and np.count_nonzero(d) / d.size <= 1e-4


def test_no_alloc_entry_matches_workspace_entry_twice_in_a_row(oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    L = _lib.lib()
    assert L.gmmB200NoAllocScratchBytes() == 32 * 1024 * 1024 + 64 * 1024
    # first call: more rows, large values left behind in the shared scratch
    _run_pair(L, dev, oracle, 31, 300, 512, 1024, 4, [100, 0, 150, 40])
    # second call straight after it: fewer rows, different shape, runs over the first call's leftovers
    _run_pair(L, dev, oracle, 32, 70, 256, 512, 3, [20, 30, 15], check_memory=True)


def test_no_alloc_entry_rejects_oversized_problem():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    L = _lib.lib()
    m, n = 8192, 4096
    assert 256 + 4 * m + 8 * (m // 128 + 4) + 4 * m * (n // 2) > L.gmmB200NoAllocScratchBytes()  # twice the built-in scratch
    one = C.c_void_p(256)  # never dereferenced: the size check comes before anything touches the device
    rc = L.gmmB200GroupedMatmulSwigluQuantNoAlloc(one, one, one, _lib.ACL_FLOAT, one, one, 1, m, 7168, n, 1, one, one, None)
    assert rc == _lib.ACLNN_ERR_PARAM_INVALID
    assert "scratch" in _lib.last_error()
