"""Sampled parity checks of device results against the CPU oracle.  TEST INFRASTRUCTURE ONLY.

The fp64 golden GEMM costs O(M N K) on the host, so full-size results are checked on a
sub-matrix: rows spread over every 4096-row band of the output, columns stratified over the
whole width (one random column per stratum, so every range of 128-column weight blocks is
hit when there are at least as many strata as ranges).  Only the sampled operand rows travel
to the host; the weight scales are expanded to one row per sampled column and the oracle is
called with block_n = 1, which selects exactly the scale row the full layout would.

Used by the GPU tests and by the benchmark's parity gates (never by the package).
"""
from __future__ import annotations

import numpy as np

from . import quant_fp8_per_token_group, w8a8_block_fp8_gemm

ROW_TOL = 1e-2          # max |err| <= ROW_TOL * ||golden row||_inf        (reference tests/test_gemm.cpp:93-96 are looser)
FRO_TOL_16BIT = 2e-3    # relative Frobenius error, bf16 / fp16 output (rounding alone is ~1.7e-3)
FRO_TOL_F32 = 1e-5


def stratified(total: int, count: int, seed: int) -> np.ndarray:
    """`count` sorted distinct indices in [0, total), one drawn from each of `count` equal strata."""
    count = min(count, total)
    rng = np.random.default_rng(seed)
    edges = np.linspace(0, total, count + 1).astype(np.int64)
    lo, hi = edges[:-1], np.maximum(edges[1:], edges[:-1] + 1)
    return np.unique(np.minimum(lo + (rng.random(count) * (hi - lo)).astype(np.int64), total - 1))


def band_rows(m: int, per_band: int, seed: int, band: int = 4096) -> np.ndarray:
    """`per_band` rows from every `band`-row band of [0, m), always including the first and last row."""
    picks = [np.array([0, m - 1], dtype=np.int64)]
    for b0 in range(0, m, band):
        picks.append(b0 + stratified(min(band, m - b0), per_band, seed + b0))
    return np.unique(np.concatenate(picks))


def gemm_errors(got, want):
    """(max over rows of max|err| / ||want row||_inf, relative Frobenius error), in float64."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    row_inf = np.abs(want).max(axis=1)
    row_inf = np.where(row_inf == 0, 1.0, row_inf)
    return float((err.max(axis=1) / row_inf).max()), float(np.sqrt((err ** 2).sum() / max((want ** 2).sum(), 1e-300)))


def gemm_sample(a_q, a_scales, b_q, b_scales, c, rows, cols, threads: int = 8):
    """Errors of the device result `c` [M, N] on the sub-matrix rows x cols against the fp64 golden
    fed the same quantised operands.  All tensor arguments are torch CUDA tensors; `b_q` is
    [N, K] (a single matrix, e.g. one expert's).  Returns (row_err, frobenius_err)."""
    import torch
    dev = a_q.device
    r = torch.as_tensor(np.asarray(rows), device=dev, dtype=torch.long)
    cidx = torch.as_tensor(np.asarray(cols), device=dev, dtype=torch.long)
    aq = a_q.index_select(0, r).cpu().numpy()
    a_s = a_scales.index_select(0, r).cpu().numpy()
    bq = b_q.index_select(0, cidx).cpu().numpy()
    bs = b_scales.index_select(0, cidx // 128).cpu().numpy()          # one scale row per sampled column
    want = w8a8_block_fp8_gemm(aq, a_s, bq, bs, block_n=1, threads=threads)
    got = c.index_select(0, r).index_select(1, cidx).float().cpu().numpy()
    return gemm_errors(got, want)


def quant_rows_exact(x, q, scales, rows) -> bool:
    """True when the device quantisation (q, scales) of the 16-bit / fp32 activations x equals the
    oracle's on the sampled rows, byte for byte."""
    import torch
    r = torch.as_tensor(np.asarray(rows), device=x.device, dtype=torch.long)
    xs = x.index_select(0, r).float().cpu().numpy()                    # widening is exact
    want_q, want_s = quant_fp8_per_token_group(xs)
    return bool(np.array_equal(q.index_select(0, r).cpu().numpy(), want_q) and
                np.array_equal(scales.index_select(0, r).cpu().numpy(), want_s))
