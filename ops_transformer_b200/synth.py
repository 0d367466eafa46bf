"""Seeded synthetic inputs with the shapes of DeepSeek-V3's MoE expert FFN (hidden 7168, expert intermediate
2048, 256 routed experts, top-8).  No dataset or checkpoint is involved: values are uniform int8 in [-127, 127]
and fp32 scales uniform in [1e-3, 1e-2]; routing is top-8 of a softmax over N(0,1) logits, or a Zipf(1.1)
choice for the skewed decode case.  One generator per tensor (seed*1000 + index) keeps tensors independent of
the order in which they are drawn.
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int, idx: int) -> np.random.Generator:
    return np.random.default_rng(seed * 1000 + idx)


def int8_tensor(shape, seed: int, idx: int) -> np.ndarray:
    return _rng(seed, idx).integers(-127, 128, size=shape, dtype=np.int8)


def scale_tensor(shape, seed: int, idx: int) -> np.ndarray:
    return _rng(seed, idx).uniform(1e-3, 1e-2, size=shape).astype(np.float32)


def topk_softmax_counts(tokens: int, experts: int, top_k: int, seed: int, idx: int = 7):
    """Per-expert row counts and the expert id of every (token, slot) pair for softmax/top-k routing."""
    logits = _rng(seed, idx).standard_normal((tokens, experts)).astype(np.float32)
    # softmax is monotone, so its top-k equals the logits' top-k
    top = np.argpartition(-logits, top_k - 1, axis=1)[:, :top_k]
    counts = np.bincount(top.reshape(-1), minlength=experts).astype(np.int64)
    return counts, top


def zipf_counts(tokens: int, experts: int, top_k: int, seed: int, s: float = 1.1, idx: int = 8):
    """Per token, ``top_k`` distinct experts drawn with p(e) proportional to (e+1)^-s."""
    r = _rng(seed, idx)
    p = (np.arange(experts, dtype=np.float64) + 1.0) ** (-s)
    p /= p.sum()
    picks = np.stack([r.choice(experts, size=top_k, replace=False, p=p) for _ in range(tokens)])
    counts = np.bincount(picks.reshape(-1), minlength=experts).astype(np.int64)
    return counts, picks


def group_list_from_counts(counts, gl_type: int) -> np.ndarray:
    counts = np.asarray(counts, np.int64)
    return np.cumsum(counts) if gl_type == 0 else counts.copy()


# The configurations named by the benchmark definition.  M = total rows, E = local experts.
CONFIGS = {
    "c1": dict(E=4, K=1024, N=2048, counts=[64, 32, 96, 64]),
    "c2": dict(E=32, K=7168, N=4096, tokens=4096, top_k=8, routing="softmax"),
    "c3": dict(E=32, K=2048, N=7168, tokens=4096, top_k=8, routing="softmax"),
    "c4_swiglu": dict(E=256, K=7168, N=4096, tokens=128, top_k=8, routing="zipf"),
    "c4_down": dict(E=256, K=2048, N=7168, tokens=128, top_k=8, routing="zipf"),
    # Reduced cases of the same kernels for profiler captures (a few hundred MB on the device, still > L2).
    "c2_small": dict(E=8, K=7168, N=4096, tokens=1024, top_k=8, routing="softmax"),
    "c3_small": dict(E=8, K=2048, N=7168, tokens=1024, top_k=8, routing="softmax"),
    "c4_swiglu_small": dict(E=32, K=7168, N=4096, tokens=16, top_k=8, routing="zipf"),
    "c4_down_small": dict(E=32, K=2048, N=7168, tokens=16, top_k=8, routing="zipf"),
}


def config_counts(name: str, seed: int = 0) -> np.ndarray:
    c = CONFIGS[name]
    if "counts" in c:
        return np.asarray(c["counts"], np.int64)
    if c["routing"] == "softmax":
        return topk_softmax_counts(c["tokens"], c["E"], c["top_k"], seed)[0]
    return zipf_counts(c["tokens"], c["E"], c["top_k"], seed)[0]
