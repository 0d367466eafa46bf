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
    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(dict(source="oracle/gmm_oracle.c (the reference has no golden vectors for these operators)",
                       cases=cases), f, indent=1)


if __name__ == "__main__":
    main()
