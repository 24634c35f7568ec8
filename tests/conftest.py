import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; runs the CUDA path through the C ABI")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def config1_inputs():
    """Inputs of the CPU-runnable golden config (M=32, N=1024, K=1024, seed 0) as bf16 bit patterns."""
    import oracle
    rng = np.random.default_rng(0)
    m, n, k = 32, 1024, 1024
    a_bits = oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32))
    w_bits = oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32))
    return a_bits, w_bits


def gemm_errors(got, want):
    """(max over rows of max|err| / ||want row||_inf, relative Frobenius error), in float64."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    row_inf = np.abs(want).max(axis=1)
    row_inf = np.where(row_inf == 0, 1.0, row_inf)
    return float((err.max(axis=1) / row_inf).max()), float(np.sqrt((err ** 2).sum() / (want ** 2).sum()))


# Tolerances of the GEMM against the fp64 golden: max |err| <= 1e-2 * ||row||_inf and
# relative Frobenius error <= 2e-3 for bf16 output (bf16 rounding alone costs ~1.7e-3).
GEMM_ROW_TOL = 1e-2
GEMM_FRO_TOL_BF16 = 2e-3
GEMM_FRO_TOL_F32 = 1e-5
