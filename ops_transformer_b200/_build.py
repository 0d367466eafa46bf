"""Builds libgmm_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python -m ops_transformer_b200._build`` or through ``__graft_entry__.build()``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libgmm_b200.so")

SOURCES = ["gmm_sm100.cu", "gmm_simt.cu", "gmm_noalloc.cu", "ep_peer.cu", "moe_init_routing.cu", "view_copy.cu", "acl_shim.cpp", "op_api.cpp"]
HEADERS = ["gmm_common.h", "acl_shim.h"]

# -fmad=false: the epilogues reproduce the reference's separately rounded fp32 steps, so the compiler must not
# fuse a multiply and an add.  No fast-math.
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-fmad=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared", "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    inc = os.path.join(ROOT, "include")
    for d, _, files in os.walk(inc):
        deps += [os.path.join(d, f) for f in files]
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    extra = os.environ.get("GMM_B200_NVCC_EXTRA", "").split()  # e.g. -DGMM_DEBUG_KNOBS for kernel experiments
    cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + [
        "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", LIB_PATH,
    ] + [os.path.join(CSRC, s) for s in SOURCES]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libgmm_b200.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
