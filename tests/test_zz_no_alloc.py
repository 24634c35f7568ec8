"""The allocation-free entry point for a few tokens against the regular GEMM entry point.

Some users of this library run with every byte of device memory already owned by their own
pool, or inside a latency-critical loop where a driver allocation call is not acceptable; for
them inferop_w8a8_block_fp8_gemm_fixed_scratch keeps its split-tile scratch in a fixed array
inside the library image.  This test calls it through the C ABI twice in a row (the array
keeps the previous call's contents, so the second call exercises the re-use) and compares each
result with what inferop_w8a8_block_fp8_gemm returns for the same inputs: both run the same
kernel with the same split of K, so the results must be equal bit for bit (a tolerance would
hide stale partial sums left in the shared array), and both must be within the GEMM tolerances
of the fp64 oracle.  It also checks that the calls leave the amount of free device memory
unchanged and that the bounded-wait record of this entry point reads "ok".  It lives in a file
of its own that pytest collects last.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from conftest import GEMM_FRO_TOL_BF16, GEMM_ROW_TOL, ROOT, gemm_errors

pytestmark = pytest.mark.gpu


def _case(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32)))
    w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=8)
    return [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (aq, a_s, bq, bs)], want


def _fixed(lib, out, aq, a_s, bq, bs, m, n, k, stream):
    return lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(out.data_ptr(), aq.data_ptr(), a_s.data_ptr(), bq.data_ptr(),
                                                         bs.data_ptr(), m, n, k, 128, 128, 2, stream)


@pytest.mark.parametrize("m,n,k", [(16, 1000, 1536), (3, 384, 2048), (32, 2500, 512)])
def test_fixed_scratch_entry_point_matches_regular_entry_point_twice(m, n, k):
    import ctypes as C
    from inference_b200 import _capi
    lib = _capi.lib
    assert lib.inferop_has_cuda() and lib.inferop_device_sm_version(0) == 100, "needs a B200"
    torch.cuda.set_device(0)
    (aq, a_s, bq, bs), oracle_c = _case(m, n, k, seed=m + n + k)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    _capi.check(lib.inferop_w8a8_block_fp8_gemm(want.data_ptr(), aq.data_ptr(), a_s.data_ptr(), bq.data_ptr(),
                                                bs.data_ptr(), m, n, k, 128, 128, 2, stream), "regular entry point")
    outs = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    _capi.check(_fixed(lib, outs[2], aq, a_s, bq, bs, m, n, k, stream), "fixed-scratch entry point, warm-up")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for call in range(2):
        _capi.check(_fixed(lib, outs[call], aq, a_s, bq, bs, m, n, k, stream), f"fixed-scratch entry point, call {call}")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before, "the allocation-free entry point took device memory"
    rec = (C.c_uint32 * 4)()
    assert lib.inferop_device_status(rec, 1) == _capi.OK and rec[0] == 0
    for call in range(2):
        assert torch.equal(outs[call].view(torch.int16), want.view(torch.int16)), f"call {call} differs from the regular entry point"
        row, fro = gemm_errors(outs[call].float().cpu().numpy(), oracle_c)
        assert row <= GEMM_ROW_TOL and fro <= GEMM_FRO_TOL_BF16, f"call {call}: row {row:.3e} frobenius {fro:.3e}"


_FRESH = r"""
import ctypes as C, sys
import numpy as np, torch
sys.path.insert(0, {root!r})
import oracle
from inference_b200 import _capi
lib = _capi.lib
torch.cuda.set_device(0)
rng = np.random.default_rng(5)
m, n, k = 8, 640, 1024
a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32)))
w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
aq, a_s = oracle.quant_fp8_per_token_group(a)
bq, bs = oracle.block_quant_weights(w)
want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
d = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (aq, a_s, bq, bs)]
outs = [torch.zeros((m, n), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
s = torch.cuda.current_stream().cuda_stream
def call(o):
    return lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(o.data_ptr(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(),
                                                         d[3].data_ptr(), m, n, k, 128, 128, 2, s)
assert call(outs[2]) == 0          # first call on this device: resolves the array's address, loads the kernel
torch.cuda.synchronize()
free = torch.cuda.mem_get_info()[0]
assert call(outs[0]) == 0 and call(outs[1]) == 0
torch.cuda.synchronize()
assert torch.cuda.mem_get_info()[0] >= free, "device memory was taken"
rec = (C.c_uint32 * 4)()
assert lib.inferop_device_status(rec, 1) == 0 and rec[0] == 0
for o in outs:
    err = np.abs(o.float().cpu().numpy().astype(np.float64) - want)
    assert (err.max(axis=1) / np.abs(want).max(axis=1)).max() <= 1e-2
assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
# empty sum: zeros, like the regular entry point
z = torch.ones((m, n), dtype=torch.bfloat16, device="cuda")
assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(z.data_ptr(), None, None, None, None, m, n, 0, 128, 128, 2, s) == 0
torch.cuda.synchronize()
assert bool((z == 0).all())
print("fresh-process ok")
"""


def test_fixed_scratch_entry_point_alone_in_a_fresh_process():
    """A process that never calls any other operator of the library (so nothing of the library
    has allocated on its behalf): results against the oracle, free memory unchanged, status ok."""
    out = subprocess.run([sys.executable, "-c", _FRESH.format(root=ROOT)], capture_output=True, text=True,
                         timeout=600, cwd=ROOT, env=dict(os.environ))
    assert out.returncode == 0 and "fresh-process ok" in out.stdout, out.stdout + out.stderr


def test_fixed_scratch_entry_point_rejects_sizes_beyond_its_limits():
    from inference_b200 import _capi
    lib = _capi.lib
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(p, p, p, p, p, 33, 256, 128, 128, 128, 2, None) == _capi.ERR_LIMIT
    assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(p, p, p, p, p, 4, 128 * 4096 + 1, 128, 128, 128, 2, None) == _capi.ERR_LIMIT
    assert lib.inferop_w8a8_block_fp8_gemm_fixed_scratch(p, p, p, p, p, 4, 256, 100, 128, 128, 2, None) == _capi.ERR_SHAPE
    assert "limit" in _capi.status_string(_capi.ERR_LIMIT)
