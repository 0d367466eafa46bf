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

        def compute(x, xs, gl):
            y = _oracle_ffn(O, x.numpy(), xs.numpy(), gl.numpy(), w1[lo:hi], s1[lo:hi], w2[lo:hi], s2[lo:hi])
            return torch.from_numpy(y.view(np.int16)).view(torch.bfloat16)

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
