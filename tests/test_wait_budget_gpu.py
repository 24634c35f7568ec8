"""The give-up path of the bounded waits, on a GPU, without faulting or hanging it.

Every wait inside the GEMM kernels has a budget; when it runs out the role records where it gave
up, all roles of the CTA wind down, tensor memory is freed and the kernel returns.  Here the
budget is set to about a millisecond and a test hook makes the TMA producers issue no load at
all, so that from the first instruction no role can make progress (nothing is in flight, nothing
is half done): every role runs out, the call returns, inferop_device_status reports
INFEROP_ERR_DEVICE_WAIT with the site, and the next ordinary call gives the right answer.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import GEMM_FRO_TOL_BF16, GEMM_ROW_TOL, gemm_errors

pytestmark = pytest.mark.gpu

# (what, options, M, N, K, sites a first giver-up may record)
CASES = [
    ("single-CTA large-tile kernel", {"gemm_path": 1, "gemm_pair": 0}, 128, 128, 256, {0x101, 0x201, 0x202, 0x301}),
    ("CTA-pair kernel", {"gemm_path": 1, "gemm_pair": 1}, 256, 256, 256, {0x121, 0x221, 0x222, 0x321}),
    ("small-M kernel", {"gemm_path": 2}, 8, 128, 256, {0x111, 0x211, 0x212, 0x311, 0x312, 0x411}),
]


def _inputs(m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32)))
    w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    dev = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (aq, a_s, bq, bs)]
    return dev, oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)


@pytest.mark.parametrize("what,options,m,n,k,sites", CASES, ids=[c[0] for c in CASES])
def test_waits_run_out_cleanly_and_the_next_call_is_right(what, options, m, n, k, sites):
    from inference_b200 import _capi, ops
    assert ops.has_cuda() and ops.device_sm_version(0) == 100, "needs a B200"
    torch.cuda.set_device(0)
    (aq, a_s, bq, bs), want = _inputs(m, n, k)
    ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)       # creates the context and the scratch
    assert ops.device_status()[0] == 0
    for key, val in options.items():
        ops.set_option(key, val)
    rec = (C.c_uint32 * 4)()
    try:
        ops.set_option("wait_budget_us", 1000)
        ops.set_option("debug_no_loads", 1)
        out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=out)           # enqueues; every role gives up after ~1 ms
        rc = _capi.lib.inferop_device_status(rec, 1)                 # synchronises
        assert rc == _capi.ERR_DEVICE_WAIT, f"{what}: status {rc}, record {[hex(v) for v in rec]}"
        assert rec[0] in sites, f"{what}: unexpected site {hex(rec[0])}"
        assert _capi.lib.inferop_device_status(rec, 0) == _capi.OK   # the record was reset
    finally:
        ops.set_option("debug_no_loads", 0)
        ops.set_option("wait_budget_us", 0)
    try:
        got = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
        assert ops.device_status()[0] == 0
        row, fro = gemm_errors(got.float().cpu().numpy(), want)
        assert row <= GEMM_ROW_TOL and fro <= GEMM_FRO_TOL_BF16
    finally:
        for key in options:
            ops.set_option(key, -1 if key == "gemm_pair" else 0)
