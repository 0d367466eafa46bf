"""Row-sampled comparison of full-size GPU results with the CPU oracle (TEST INFRASTRUCTURE, not product code).

Both operators treat every row on its own (a row of grouped_matmul is one vector-matrix product with its expert's
weight; a row of grouped_matmul_swiglu_quant adds a row-local maximum), so a full-size launch can be checked by
running the oracle on a subset of its rows at the full K and N: the selected rows of every expert, in order, form a
smaller problem with the same weights whose results must equal the selected rows of the large one.

Used by the `-m gpu` tests of the benchmark configurations and by bench.py after its timed region.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O

# The bars of the benchmark definition.
BF16_RTOL, BF16_ATOL = 4e-3, 1e-2
QSCALE_RTOL = 1e-6
Q_LSB_FRACTION = 1e-4


def sample_rows(counts, n_random: int = 32, seed: int = 0, edges=(128, 256), max_rows_all: int = 0) -> np.ndarray:
    """Sorted row numbers to check: per expert its first and last row, the rows either side of every 128- and 256-row
    tile edge inside it, and ``n_random`` more drawn uniformly.  With at most ``max_rows_all`` rows in total every row."""
    counts = np.asarray(counts, np.int64)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    total = int(counts.sum())
    if total <= max_rows_all:
        return np.arange(total, dtype=np.int64)
    rng = np.random.default_rng(seed)
    picks = []
    for s, r in zip(starts, counts):
        s, r = int(s), int(r)
        if r <= 0:
            continue
        local = {0, r - 1}
        for e in edges:
            for m in range(e, r, e):
                local.add(m - 1)
                local.add(m)
        if r > len(local):
            local.update(int(v) for v in rng.integers(0, r, size=n_random))
        picks.extend(s + v for v in sorted(local))
    return np.asarray(sorted(set(picks)), np.int64)


def counts_of_sample(rows: np.ndarray, counts) -> np.ndarray:
    """How many of the sampled rows fall into each expert's range."""
    ends = np.cumsum(np.asarray(counts, np.int64))
    owner = np.searchsorted(ends, rows, side="right")
    return np.bincount(owner, minlength=len(ends)).astype(np.int64)


def check_swiglu_rows(x_rows, w, w_scale, x_scale_rows, sample_counts, q_rows, q_scale_rows) -> dict:
    """Oracle on the sampled rows (``x_rows`` int8 [r, K], in expert order) against the GPU's ``q_rows`` / ``q_scale_rows``.
    Returns counts; ``mismatches`` is 0 when the bars of the benchmark definition hold."""
    ref = O.swiglu_quant(x_rows, w, w_scale, x_scale_rows, np.cumsum(sample_counts))
    qs_ref, q_ref = ref["q_scale"], ref["q"]
    rel = np.abs(q_scale_rows - qs_ref) / np.maximum(np.abs(qs_ref), np.float32(1e-30))
    bad_scale = int(np.count_nonzero(~(rel <= QSCALE_RTOL)))
    d = np.abs(q_rows.astype(np.int32) - q_ref.astype(np.int32))
    off_by_one = int(np.count_nonzero(d == 1))
    bad_q = int(np.count_nonzero(d > 1))
    frac = off_by_one / max(d.size, 1)
    mism = bad_scale + bad_q + (off_by_one if frac > Q_LSB_FRACTION else 0)
    return {"rows": int(x_rows.shape[0]), "mismatches": int(mism), "scale_max_rel": float(rel.max()) if rel.size else 0.0,
            "int8_off_by_one": off_by_one, "int8_off_by_more": bad_q, "int8_elements": int(d.size)}


def check_gmm_rows(x_rows, w, w_scale, x_scale_rows, sample_counts, y_rows_bits, y_dtype: str = "bf16", w_trans: bool = False) -> dict:
    """Oracle grouped_matmul W8A8 on the sampled rows against the GPU's rows: bf16 bit patterns (uint16) or int32."""
    ref = O.gmm_w8a8(x_rows, w, w_scale, x_scale_rows, np.cumsum(sample_counts), 0, y_dtype=y_dtype, w_trans=w_trans)["y"]
    if y_dtype == "int32":
        bad = int(np.count_nonzero(y_rows_bits != ref))
        return {"rows": int(x_rows.shape[0]), "mismatches": bad, "not_bit_identical": bad}
    got, exp = O.bf16_bits_to_f32(y_rows_bits), O.bf16_bits_to_f32(ref)
    err = np.abs(got - exp)
    out_of_tol = int(np.count_nonzero(~(err <= BF16_ATOL + BF16_RTOL * np.abs(exp))))
    return {"rows": int(x_rows.shape[0]), "mismatches": out_of_tol, "not_bit_identical": int(np.count_nonzero(y_rows_bits != ref)),
            "max_abs_err": float(err.max()) if err.size else 0.0}
