"""Expert-parallel row bookkeeping on CPU: two gloo ranks exchange rows, run a CPU stand-in for the two GEMM
operators (the oracle) on their local experts, return the results, and every rank checks what it gets back against
the oracle applied to its own rows with all experts in one process.  Also checks the re-order index maths."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ops_transformer_b200 import ep, synth

N_EXPERTS, H, I, TOP_K, T = 8, 64, 32, 2, 24


def _weights():
    w1 = synth.int8_tensor((N_EXPERTS, H, 2 * I), 50, 1)
    w2 = synth.int8_tensor((N_EXPERTS, I, H), 50, 2)
    s1 = synth.scale_tensor((N_EXPERTS, 2 * I), 50, 3)
    s2 = synth.scale_tensor((N_EXPERTS, H), 50, 4)
    return w1, w2, s1, s2


def _oracle_ffn(O, x, xs, gl, w1, s1, w2, s2):
    r = O.swiglu_quant(x, w1, s1, xs, gl)
    y = O.gmm_w8a8(r["q"], w2, s2, r["q_scale"], gl, 0)["y"]
    return y


def _rank_main(rank, world, port, chunks, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        w1, w2, s1, s2 = _weights()
        el = N_EXPERTS // world
        lo, hi = rank * el, (rank + 1) * el

        def compute(x, xs, gl, out_row_index):
            y = _oracle_ffn(O, x.numpy(), xs.numpy(), gl.numpy(), w1[lo:hi], s1[lo:hi], w2[lo:hi], s2[lo:hi])
            yt = torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)
            if out_row_index is None:
                return yt
            out = torch.empty_like(yt)
            out[out_row_index] = yt   # row r -> row out_row_index[r], what the GPU down projection does in its epilogue
            return out

        x = synth.int8_tensor((T, H), 60 + rank, 1)
        xs = synth.scale_tensor((T,), 60 + rank, 2)
        rng = np.random.default_rng(70 + rank)
        topk = np.stack([rng.choice(N_EXPERTS, TOP_K, replace=False) for _ in range(T)]).astype(np.int64)
        ffn = ep.ExpertParallelFFN(N_EXPERTS, None, None, None, None, chunks=chunks, compute=compute)
        res = ffn.forward(torch.from_numpy(x), torch.from_numpy(xs), torch.from_numpy(topk))
        ok = True
        bounds = [T * c // chunks for c in range(chunks + 1)]
        for c, r in enumerate(res):
            p = r["plan"]
            tok = p.src_token.numpy() + bounds[c]
            experts = topk[bounds[c]:bounds[c + 1]].reshape(-1)[p.order.numpy()]
            assert (np.diff(experts) >= 0).all()
            gl = np.cumsum(np.bincount(experts, minlength=N_EXPERTS))
            exp = _oracle_ffn(O, x[tok], xs[tok], gl, w1, s1, w2, s2)
            got = r["y"].view(torch.int16).numpy().view(np.uint16)
            ok = ok and np.array_equal(got, exp)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 3])
def test_two_rank_exchange_matches_single_process(chunks, oracle):
    world = 2
    port = 29610 + chunks
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, port, chunks, ret), nprocs=world, join=True)
    assert all(ret.get(r, False) for r in range(world)), dict(ret)


def test_reorder_index_is_the_rerouting_permutation():
    counts = torch.tensor([[2, 0, 3], [1, 4, 0]])  # [src, expert]
    dst, gl = ep.reorder_index(counts)
    # received order: (s0,e0)x2 (s0,e2)x3 (s1,e0)x1 (s1,e1)x4 ; expert-major: e0: s0x2 s1x1 | e1: s1x4 | e2: s0x3
    assert dst.tolist() == [0, 1, 7, 8, 9, 2, 3, 4, 5, 6]
    assert gl.tolist() == [3, 7, 10]
    assert sorted(dst.tolist()) == list(range(10))


def test_dispatch_plan_sorts_rows_by_expert():
    topk = torch.tensor([[5, 1], [0, 5], [3, 1]])
    p = ep.dispatch_plan(topk, 8, 2)
    assert topk.reshape(-1)[p.order].tolist() == [0, 1, 1, 3, 5, 5]
    assert p.src_token.tolist() == [1, 0, 2, 2, 0, 1]
    assert p.send_counts.tolist() == [[1, 2, 0, 1], [0, 2, 0, 0]]


def test_fused_maps_place_rows_expert_major_and_return_them_home():
    """Simulate G ranks on CPU: scatter every rank's send rows by send_dest, check the receiver's buffer is expert major
    with the right owners, then scatter 'results' by ret_dest and check every row comes back to its send position."""
    G, E, k, T = 4, 3, 2, 40
    rng = np.random.default_rng(5)
    topks = [np.stack([rng.choice(G * E, k, replace=False) for _ in range(T)]).astype(np.int64) for _ in range(G)]
    plans = [ep.dispatch_plan(torch.from_numpy(t), G * E, G) for t in topks]
    allc = torch.stack([p.send_counts for p in plans])                      # [src, dst, e]
    n_send, cap = T * k, 2 * T * k
    maps = [ep.fused_maps(allc, r, n_send, cap) for r in range(G)]
    act = np.full((G, cap, 3), -1, np.int64)                                # (src rank, send index, global expert)
    for r in range(G):
        send_dest = maps[r][0].numpy()
        experts = topks[r].reshape(-1)[plans[r].order.numpy()]
        assert (send_dest >= 0).all()
        for i, d in enumerate(send_dest):
            gpu, row = int(d >> ep.ROW_BITS), int(d & ((1 << ep.ROW_BITS) - 1))
            assert gpu == experts[i] // E
            assert act[gpu, row, 0] == -1, "two rows sent to the same place"
            act[gpu, row] = (r, i, experts[i])
    result = np.full((G, n_send, 2), -1, np.int64)
    for d in range(G):
        _, ret_dest, gl, n_recv = maps[d]
        n = int(n_recv)
        assert n == int(allc[:, d, :].sum()) and gl.tolist() == np.cumsum(allc[:, d, :].sum(0).numpy()).tolist()
        local_e = act[d, :n, 2] - d * E
        assert (act[d, :n, 0] >= 0).all() and (np.diff(local_e) >= 0).all(), "buffer is not expert major"
        starts = np.concatenate([[0], gl.numpy()])
        for e in range(E):
            seg = act[d, starts[e]:starts[e + 1]]
            assert (seg[:, 2] == d * E + e).all() and (np.diff(seg[:, 0]) >= 0).all()   # rank-minor inside an expert
        assert (ret_dest[n:] == -1).all()
        for p_, rd in enumerate(ret_dest[:n].numpy()):
            gpu, row = int(rd >> ep.ROW_BITS), int(rd & ((1 << ep.ROW_BITS) - 1))
            assert (gpu, row) == (act[d, p_, 0], act[d, p_, 1]), "result row does not go back to where it came from"
            result[gpu, row] = (d, p_)
    assert (result[:, :, 0] >= 0).all(), "some sent row got no result"
