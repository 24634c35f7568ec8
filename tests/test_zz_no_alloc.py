"""The allocation-free entry point for a few tokens against the regular GEMM entry point.

Some users of this library run with every byte of device memory already owned by their own
pool, or inside a latency-critical loop where a driver allocation call is not acceptable; for
them inferop_w8a8_block_fp8_gemm_fixed_scratch keeps its split-tile scratch in a fixed array
inside the library image.  This test calls it through the C ABI twice in a row (the array
keeps the previous call's contents, so the second call exercises the re-use) and compares each
result with what inferop_w8a8_block_fp8_gemm returns for the same inputs, within the GEMM
tolerances used everywhere else in the suite.  It lives in a file of its own that pytest
collects last.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import GEMM_FRO_TOL_BF16, GEMM_ROW_TOL, gemm_errors

pytestmark = pytest.mark.gpu


def _case(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32)))
    w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    return [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (aq, a_s, bq, bs)]


@pytest.mark.parametrize("m,n,k", [(16, 1000, 1536), (3, 384, 2048), (32, 2500, 512)])
def test_fixed_scratch_entry_point_matches_regular_entry_point_twice(m, n, k):
    from inference_b200 import _capi
    lib = _capi.lib
    assert lib.inferop_has_cuda() and lib.inferop_device_sm_version(0) == 100, "needs a B200"
    torch.cuda.set_device(0)
    aq, a_s, bq, bs = _case(m, n, k, seed=m + n + k)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    _capi.check(lib.inferop_w8a8_block_fp8_gemm(want.data_ptr(), aq.data_ptr(), a_s.data_ptr(), bq.data_ptr(),
                                                bs.data_ptr(), m, n, k, 128, 128, 2, stream), "regular entry point")
    torch.cuda.synchronize()
    want_h = want.float().cpu().numpy()
    for call in range(2):
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        _capi.check(lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(got.data_ptr(), aq.data_ptr(), a_s.data_ptr(),
                                                                  bq.data_ptr(), bs.data_ptr(), m, n, k, 128, 128,
                                                                  2, stream), f"fixed-scratch entry point, call {call}")
        torch.cuda.synchronize()
        row, fro = gemm_errors(got.float().cpu().numpy(), want_h)
        assert row <= GEMM_ROW_TOL and fro <= GEMM_FRO_TOL_BF16, f"call {call}: row {row:.3e} frobenius {fro:.3e}"


def test_fixed_scratch_entry_point_rejects_sizes_beyond_its_limits():
    from inference_b200 import _capi
    lib = _capi.lib
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(p, p, p, p, p, 33, 256, 128, 128, 128, 2, None) == _capi.ERR_LIMIT
    assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(p, p, p, p, p, 4, 128 * 4096 + 1, 128, 128, 128, 2, None) == _capi.ERR_LIMIT
    assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(p, p, p, p, p, 4, 256, 100, 128, 128, 2, None) == _capi.ERR_SHAPE
    assert "limit" in _capi.status_string(_capi.ERR_LIMIT)
