"""Writes the golden fixtures in this folder.

The reference ships no golden vectors for grouped_matmul or grouped_matmul_swiglu_quant and its kernels cannot
run outside the closed Ascend toolchain, so these fixtures come from the CPU oracle (oracle/gmm_oracle.c) on
seeded inputs.  They pin the oracle against accidental change and give the GPU tests a fixed target that does
not depend on the oracle being rebuilt on the test machine.  Run: python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402
from ops_transformer_b200 import synth  # noqa: E402


def main():
    cases = []
    specs = [
        ("gmm_cumsum_small", "grouped_matmul", 0, 24, 48, 32, 3, [5, 5, 20]),
        ("gmm_count_small", "grouped_matmul", 1, 40, 80, 48, 4, [7, 0, 30, 2]),
        ("gmm_tile_sized", "grouped_matmul", 0, 160, 128, 256, 2, [128, 150]),
        ("swiglu_small", "grouped_matmul_swiglu_quant", 0, 20, 64, 64, 3, [4, 4, 17]),
        ("swiglu_tile_sized", "grouped_matmul_swiglu_quant", 0, 140, 128, 256, 2, [130, 137]),
    ]
    for i, (name, op, gl_type, M, K, N, E, gl) in enumerate(specs):
        seed = 100 + i
        x = synth.int8_tensor((M, K), seed, 1)
        w = synth.int8_tensor((E, K, N), seed, 2)
        ws = synth.scale_tensor((E, N), seed, 3)
        xs = synth.scale_tensor((M,), seed, 4)
        gl = np.asarray(gl, np.int64)
        out = dict(x=x, w=w, w_scale=ws, x_scale=xs, group_list=gl)
        if op == "grouped_matmul":
            r = O.gmm_w8a8(x, w, ws, xs, gl, gl_type, want_acc=True)
            out.update(acc=r["acc"], y_bf16_bits=r["y"])
        else:
            r = O.swiglu_quant(x, w, ws, xs, gl)
            out.update(q=r["q"], q_scale=r["q_scale"])
        fn = name + ".npz"
        np.savez_compressed(os.path.join(HERE, fn), **out)
        cases.append(dict(file=fn, op=op, group_list_type=gl_type, M=M, K=K, N=N, E=E, seed=seed))
    # the producer and the consumer either side of the two operators
    rng = np.random.default_rng(7)
    n, k, h, E = 24, 2, 64, 6
    xb = O.f32_to_bf16_bits(rng.standard_normal((n, h)).astype(np.float32))
    idx = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    smooth = rng.uniform(0.5, 2.0, size=(4, h)).astype(np.float32)
    r = O.moe_init_routing_v3(xb, idx, E, (1, 5), True, row_idx_type=0, count_type=2, scale=smooth)
    np.savez_compressed(os.path.join(HERE, "init_routing_quant_small.npz"), x_bf16_bits=xb, expert_idx=idx, scale=smooth,
                        expanded_x=r["expanded_x"], expanded_row_idx=r["expanded_row_idx"], counts=r["counts"],
                        expanded_scale=r["expanded_scale"], rows=np.int64(r["rows"]))
    cases.append(dict(file="init_routing_quant_small.npz", op="moe_init_routing_v3", n=n, k=k, h=h, E=E, active_range=[1, 5],
                      quant=1, row_idx_type=0, count_type=2, fill=dict(expanded_x=-77, expanded_row_idx=-9, counts=-9, expanded_scale=-5.0)))
    M, K, N, E, topk = 64, 64, 256, 3, 4
    x = synth.int8_tensor((M, K), 120, 1)
    w = synth.int8_tensor((E, K, N), 120, 2)
    ws = synth.scale_tensor((E, N), 120, 3)
    xs = synth.scale_tensor((M,), 120, 4)
    counts = np.array([20, 0, 40], np.int64)
    ri = (rng.permutation(M) % (M // topk)).astype(np.int64)
    logit = rng.uniform(0.05, 0.6, size=M).astype(np.float32)
    shared = O.f32_to_bf16_bits(rng.uniform(-40, 40, size=(8, N)).astype(np.float32))
    bias = O.f32_to_bf16_bits(rng.uniform(-20, 20, size=(E, N)).astype(np.float32))
    f = O.gmm_finalize_routing(x, w, ws, xs, counts, ri, M // topk, bias=bias, shared_input=shared, shared_offset=4, shared_weight=0.5,
                               logit=logit)
    np.savez_compressed(os.path.join(HERE, "finalize_routing_small.npz"), x=x, w=w, w_scale=ws, x_scale=xs, group_list=counts,
                        row_index=ri, logit=logit, shared_bf16_bits=shared, bias_bf16_bits=bias, y=f["y"], abs_sum=f["abs_sum"])
    cases.append(dict(file="finalize_routing_small.npz", op="grouped_matmul_finalize_routing", M=M, K=K, N=N, E=E, batch=M // topk,
                      shared_offset=4, shared_weight=0.5, group_list_type=1,
                      note="y is the sum in row order; an unordered fp32 sum may differ by 4 * 2^-23 * abs_sum"))
    # the combine that ends the expert-parallel path: weighted sum of a token's result rows in slot order
    tokens, k, h, rows = 20, 4, 64, 70
    yb = O.f32_to_bf16_bits(rng.uniform(-300, 300, size=(rows, h)).astype(np.float32))
    pair_row = rng.permutation(tokens * k)[:tokens * k].reshape(tokens, k) % rows
    pair_row[3, 1] = -1            # a dropped row
    pair_row[7] = -1               # a token none of whose rows came back
    wts = rng.uniform(0.05, 1.0, size=(tokens, k)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "ep_combine_small.npz"), y_bf16_bits=yb, pair_row=pair_row.astype(np.int32), weights=wts,
                        out_bf16_bits=O.ep_combine(yb, pair_row, wts))
    cases.append(dict(file="ep_combine_small.npz", op="ep_combine", tokens=tokens, k=k, h=h, rows=rows))
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(dict(source="oracle/gmm_oracle.c, oracle/oracle.py (the reference has no golden vectors for these operators)",
                       cases=cases), f, indent=1)


if __name__ == "__main__":
    main()
