"""Parity of the CUDA GEMM (through the C ABI) with the fp64 golden of the oracle."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import (GEMM_FRO_TOL_BF16, GEMM_FRO_TOL_F32, GEMM_ROW_TOL, GOLDEN, config1_inputs,
                      gemm_errors)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    yield _ops
    _ops.set_option("gemm_block_n", 0)
    _ops.set_option("gemm_tma_store", -1)


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_case(m, n, k, seed, w_std=0.02, outliers=False):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    if outliers:
        a[:, rng.choice(k, max(1, k // 100), replace=False)] *= 20.0
    a = oracle.bf16_widen(oracle.bf16_narrow(a))
    w = oracle.bf16_widen(oracle.bf16_narrow((w_std * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    return aq, a_s, bq, bs


def run(ops, aq, a_s, bq, bs, out_dtype):
    c = ops.w8a8_block_fp8_gemm(cuda(aq), cuda(a_s), cuda(bq), cuda(bs), out_dtype)
    code = ops.device_status()
    assert code[0] == 0, f"a device-side wait ran out: {[hex(v) for v in code]}"
    return c.float().cpu().numpy()


def check(got, want, out_dtype):
    row, fro = gemm_errors(got, want)
    fro_tol = GEMM_FRO_TOL_F32 if out_dtype == torch.float32 else GEMM_FRO_TOL_BF16
    assert row <= GEMM_ROW_TOL and fro <= fro_tol, f"row err {row:.3e}, frobenius {fro:.3e}"
    return row, fro


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("tma_store", [0, 1])
def test_single_tile_and_small_shapes(ops, bn, tma_store):
    ops.set_option("gemm_block_n", bn)
    ops.set_option("gemm_tma_store", tma_store)
    for (m, n, k) in [(128, 128, 128), (128, 256, 256), (256, 256, 512), (32, 1024, 1024)]:
        aq, a_s, bq, bs = make_case(m, n, k, seed=m + n + k)
        want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=8)
        for dt in (torch.float32, torch.bfloat16):
            check(run(ops, aq, a_s, bq, bs, dt), want, dt)


@pytest.mark.parametrize("bn", [128, 256])
def test_golden_small_ragged(ops, bn):
    ops.set_option("gemm_block_n", bn)
    ops.set_option("gemm_tma_store", -1)
    g = np.load(os.path.join(GOLDEN, "gemm_small_golden.npz"))
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        check(run(ops, g["aq"], g["a_scales"], g["bq"], g["b_scales"], dt), g["c"], dt)


def test_config1_golden(ops):
    ops.set_option("gemm_block_n", 0)
    ops.set_option("gemm_tma_store", -1)
    with open(os.path.join(GOLDEN, "config1_golden.json")) as f:
        rec = json.load(f)
    a_bits, w_bits = config1_inputs()
    x = torch.from_numpy(a_bits.view(np.int16)).cuda().view(torch.bfloat16)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    bq, bs = oracle.block_quant_weights(oracle.bf16_widen(w_bits))
    aq_h, as_h = oracle.quant_fp8_per_token_group(oracle.bf16_widen(a_bits))
    assert np.array_equal(aq.cpu().numpy(), aq_h) and np.array_equal(a_s.cpu().numpy(), as_h)
    want = oracle.w8a8_block_fp8_gemm(aq_h, as_h, bq, bs, threads=8)
    got = ops.w8a8_block_fp8_gemm(aq, a_s, cuda(bq), cuda(bs), torch.bfloat16).float().cpu().numpy()
    row, fro = check(got, want, torch.bfloat16)
    # the first 8 columns stored from the reference itself
    import hashlib
    if hashlib.sha256(a_bits.tobytes()).hexdigest() == rec["sha256"]["a_bf16_bits"]:
        ref8 = np.array(rec["c_first8cols"], dtype=np.float32)
        assert np.array_equal(want[:, :8], ref8)
        assert gemm_errors(got[:, :8], ref8)[0] <= GEMM_ROW_TOL


@pytest.mark.parametrize("m,n,k,dt", [
    (100, 180, 256, torch.float32),   # the reference test's ragged case (N*2 not a multiple of 16)
    (100, 180, 256, torch.bfloat16),
    (1, 128, 128, torch.bfloat16),
    (1, 1, 128, torch.float32),
    (129, 257, 384, torch.bfloat16),
    (300, 1000, 1536, torch.bfloat16),
    (64, 3000, 2048, torch.float16),
])
def test_ragged_shapes(ops, m, n, k, dt):
    for bn in (128, 256):
        ops.set_option("gemm_block_n", bn)
        ops.set_option("gemm_tma_store", -1)
        aq, a_s, bq, bs = make_case(m, n, k, seed=m * 7 + n * 3 + k, outliers=True)
        want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=8)
        check(run(ops, aq, a_s, bq, bs, dt), want, dt)


def test_reference_test_tolerances(ops):
    """tests/test_gemm.cpp:93-96: N(0,1) weights, rtol/atol of the reference's own cross-checks."""
    ops.set_option("gemm_block_n", 0)
    for (m, n, k, dt, rtol, atol) in [(256, 256, 512, torch.float32, 2e-3, 2e-2),
                                      (256, 256, 512, torch.bfloat16, 1e-2, 3e-2),
                                      (100, 180, 256, torch.float32, 2e-3, 2e-2)]:
        aq, a_s, bq, bs = make_case(m, n, k, seed=99, w_std=1.0)
        want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=8)
        got = run(ops, aq, a_s, bq, bs, dt)
        assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want))


def test_untouched_outside_output_and_canaries(ops):
    """Output rows/columns past M, N are never written (canary-padded buffer)."""
    m, n, k = 100, 184, 256
    aq, a_s, bq, bs = make_case(m, n, k, seed=5)
    buf = torch.full((m * n + 4096,), -7.0, dtype=torch.bfloat16, device="cuda")
    out = buf[:m * n].view(m, n)
    for bn in (128, 256):
        ops.set_option("gemm_block_n", bn)
        ops.w8a8_block_fp8_gemm(cuda(aq), cuda(a_s), cuda(bq), cuda(bs), out=out)
        torch.cuda.synchronize()
        assert bool((buf[m * n:] == -7.0).all())
    want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    check(out.float().cpu().numpy(), want, torch.bfloat16)


def test_rejected_calls(ops):
    from inference_b200 import _capi
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    lib = _capi.lib
    assert lib.inferop_w8a8_block_fp8_gemm(p, p, p, p, p, 4, 4, 130, 128, 128, 2, None) == _capi.ERR_SHAPE
    assert lib.inferop_w8a8_block_fp8_gemm(p, p + 1, p, p, p, 4, 4, 128, 128, 128, 2, None) == _capi.ERR_POINTER
    assert lib.inferop_w8a8_block_fp8_gemm(p, None, p, p, p, 4, 4, 128, 128, 128, 2, None) == _capi.ERR_POINTER
    # K == 0: the empty sum
    out = torch.ones((4, 4), dtype=torch.bfloat16, device="cuda")
    assert lib.inferop_w8a8_block_fp8_gemm(out.data_ptr(), p, p, p, p, 4, 4, 0, 128, 128, 2, None) == 0
    torch.cuda.synchronize()
    assert bool((out == 0).all())


def test_repeatable_and_linear_in_scales(ops):
    """Same inputs -> same bits; doubling every activation scale doubles C exactly."""
    ops.set_option("gemm_block_n", 0)
    aq, a_s, bq, bs = make_case(384, 640, 1024, seed=21)
    c1 = ops.w8a8_block_fp8_gemm(cuda(aq), cuda(a_s), cuda(bq), cuda(bs), torch.float32)
    c2 = ops.w8a8_block_fp8_gemm(cuda(aq), cuda(a_s), cuda(bq), cuda(bs), torch.float32)
    c3 = ops.w8a8_block_fp8_gemm(cuda(aq), cuda(a_s * 2), cuda(bq), cuda(bs), torch.float32)
    assert torch.equal(c1, c2) and torch.equal(c3, c1 * 2)


@pytest.mark.parametrize("m,n,k", [(4096, 4096, 4096), (16, 18432, 7168), (4096, 18432, 7168)])
def test_large_shapes_sampled(ops, m, n, k):
    """Benchmark-sized shapes: sampled rows x columns against the fp64 golden, whole-matrix
    agreement between the two tile configurations."""
    from inference_b200 import synth
    x = synth.activations(m, k, seed=1)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    bq, bs = synth.quantised_weights(n, k, seed=1)
    ops.set_option("gemm_block_n", 128)
    c128 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
    ops.set_option("gemm_block_n", 256)
    c256 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
    assert ops.device_status()[0] == 0
    assert torch.equal(c128, c256)
    rng = np.random.default_rng(m + n)
    rows = np.sort(rng.choice(m, min(m, 24), replace=False))
    cols = np.sort(rng.choice(n, 512, replace=False))
    want = oracle.w8a8_block_fp8_gemm(aq.cpu().numpy(), a_s.cpu().numpy(), bq.cpu().numpy(),
                                      bs.cpu().numpy(), rows=rows, cols=cols, threads=8)
    got = c256[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].float().cpu().numpy()
    check(got, want, torch.bfloat16)
    ops.set_option("gemm_block_n", 0)


# ------------------------------------------------------------------ small-M (weight-streaming) path
@pytest.mark.parametrize("m", [1, 4, 16, 17, 33, 64, 65, 128])
@pytest.mark.parametrize("n,k", [(384, 512), (1000, 1536), (200, 128)])
def test_small_m_path_matches_oracle(ops, m, n, k):
    ops.set_option("gemm_path", 2)
    try:
        aq, a_s, bq, bs = make_case(m, n, k, seed=m * 31 + n + k, outliers=True)
        want = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=8)
        for dt in (torch.float32, torch.bfloat16):
            check(run(ops, aq, a_s, bq, bs, dt), want, dt)
    finally:
        ops.set_option("gemm_path", 0)


@pytest.mark.parametrize("m,n,k", [(16, 18432, 7168), (4, 7168, 18432), (64, 24576, 1536), (1, 7168, 18432)])
def test_small_m_path_on_the_decode_shapes(ops, m, n, k):
    """Decode sweep shapes: split tiles (N/128 < SM count) included.  The streaming kernel must be
    repeatable bit for bit (fixed reduction order) and agree with the large-tile kernel and the
    fp64 golden on sampled columns."""
    from inference_b200 import synth
    x = synth.activations(m, k, seed=3)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    bq, bs = synth.quantised_weights(n, k, seed=3)
    try:
        ops.set_option("gemm_path", 2)
        c1 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.float32)
        c2 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.float32)
        cb = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
        ops.set_option("gemm_path", 1)
        c3 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.float32)
    finally:
        ops.set_option("gemm_path", 0)
    assert ops.device_status()[0] == 0
    assert torch.equal(c1, c2)
    assert torch.allclose(c1, c3, rtol=1e-5, atol=1e-5 * float(c3.abs().max()))
    cols = np.sort(np.random.default_rng(n).choice(n, 384, replace=False))
    want = oracle.w8a8_block_fp8_gemm(aq.cpu().numpy(), a_s.cpu().numpy(), bq.cpu().numpy(),
                                      bs.cpu().numpy(), cols=cols, threads=8)
    idx = torch.from_numpy(cols).cuda()
    check(c1[:, idx].cpu().numpy(), want, torch.float32)
    check(cb[:, idx].float().cpu().numpy(), want, torch.bfloat16)


# ------------------------------------------------------------------ grouped (MoE) launch
def test_grouped_launch_equals_one_call_per_group(ops):
    """Variable rows per group incl. empty groups, tiles that end inside a 128-row box, and a
    group larger than one tile: identical bits to per-group calls, and within tolerance of the
    fp64 golden."""
    rng = np.random.default_rng(77)
    groups, n, k = 9, 512, 768
    counts = [0, 5, 128, 200, 1, 0, 131, 64, 300]
    m_total = sum(counts)
    a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m_total, k)).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bqs, bss = [], []
    for g in range(groups):
        w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
        q, s = oracle.block_quant_weights(w)
        bqs.append(q)
        bss.append(s)
    bq, bs = np.stack(bqs), np.stack(bss)
    d_aq, d_as, d_bq, d_bs = cuda(aq), cuda(a_s), cuda(bq), cuda(bs)
    for dt in (torch.bfloat16, torch.float32):
        canary = torch.full((m_total * n + 1024,), -3.0, dtype=dt, device="cuda")
        out = canary[:m_total * n].view(m_total, n)
        ops.w8a8_block_fp8_gemm_grouped(d_aq, d_as, d_bq, d_bs, counts, out=out)
        assert ops.device_status()[0] == 0
        assert bool((canary[m_total * n:] == -3.0).all())
        r = 0
        for g, mg in enumerate(counts):
            if mg == 0:
                continue
            ops.set_option("gemm_path", 1)   # the same (large-tile) kernel as the grouped launch
            try:
                single = ops.w8a8_block_fp8_gemm(d_aq[r:r + mg], d_as[r:r + mg], d_bq[g], d_bs[g], dt)
            finally:
                ops.set_option("gemm_path", 0)
            assert torch.equal(out[r:r + mg], single), f"group {g} differs from its own call"
            want = oracle.w8a8_block_fp8_gemm(aq[r:r + mg], a_s[r:r + mg], bq[g], bs[g], threads=8)
            check(out[r:r + mg].float().cpu().numpy(), want, dt)
            r += mg


def test_grouped_launch_rejects_bad_arguments(ops):
    import ctypes as C
    from inference_b200 import _capi
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    counts = (C.c_int64 * 2)(4, 4)
    lib = _capi.lib
    assert lib.inferop_w8a8_block_fp8_gemm_grouped(p, p, p, p, p, counts, 2, 200, 128, 128, 128, 2, None) == _capi.ERR_SHAPE
    assert lib.inferop_w8a8_block_fp8_gemm_grouped(p, p, p, p, p, None, 2, 256, 128, 128, 128, 2, None) == _capi.ERR_SHAPE
    bad = (C.c_int64 * 2)(4, -1)
    assert lib.inferop_w8a8_block_fp8_gemm_grouped(p, p, p, p, p, bad, 2, 256, 128, 128, 128, 2, None) == _capi.ERR_SHAPE


# ------------------------------------------------------------------ quantisation fused as the A prologue
@pytest.mark.parametrize("m", [1, 3, 16, 17, 32, 33, 129, 1024])
@pytest.mark.parametrize("n,k", [(384, 512), (1000, 1536), (18432, 7168)])
def test_fused_quant_prologue_is_bit_identical_to_the_two_calls(ops, m, n, k):
    from inference_b200 import synth
    x = synth.activations(m, k, seed=m + n)
    x[0, :128] = 0                      # an all-zero group
    if m > 1:
        x[1, 5] = float("nan")
    bq, bs = synth.quantised_weights(n, k, seed=2)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    for dt in (torch.bfloat16, torch.float32):
        ops.set_option("gemm_path", 2 if m <= 32 else 0)   # up to 32 tokens the one-launch form is the small-M kernel
        try:
            two = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, dt)
        finally:
            ops.set_option("gemm_path", 0)
        for in_kernel in ((0, 1) if m <= 32 else (0,)):   # the chained pair (default) and the one-launch form
            ops.set_option("fused_prologue", in_kernel)
            try:
                one = ops.w8a8_block_fp8_gemm_fused_quant(x, bq, bs, dt)
            finally:
                ops.set_option("fused_prologue", 0)
            assert ops.device_status()[0] == 0
            assert torch.equal(one.view(torch.int16 if dt == torch.bfloat16 else torch.int32),
                               two.view(torch.int16 if dt == torch.bfloat16 else torch.int32))
    ops.set_option("fused_prologue", 1 if m <= 32 else 0)
    xh = x.half()
    aq, a_s = ops.quant_fp8_per_token_group(xh)
    two = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.float32)
    try:
        one = ops.w8a8_block_fp8_gemm_fused_quant(xh, bq, bs, torch.float32)
    finally:
        ops.set_option("fused_prologue", 0)
    assert torch.equal(one.view(torch.int32), two.view(torch.int32))


@pytest.mark.parametrize("m,n,k", [(4, 7168, 18432), (16, 7168, 18432), (32, 7168, 18432), (16, 24576, 1536),
                                   (32, 24576, 1536), (5, 2048, 10240), (16, 128, 10240), (16, 128, 20480)])
def test_fused_quant_prologue_ring(ops, m, n, k):
    """Shapes that exercise the token-tile ring of the one-launch form: K parts of a split tile
    (72 blocks of 144), whole tiles with two tiles per CTA (the K range repeats), K ranges far
    longer than the ring: always the bits of the two separate calls, and of the quantiser + GEMM
    pair that the option selects."""
    from inference_b200 import synth
    x = synth.activations(m, k, seed=m + k)
    bq, bs = synth.quantised_weights(n, k, seed=3)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    two = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    ops.set_option("fused_prologue", 1)
    try:
        for rep in range(3):
            one = ops.w8a8_block_fp8_gemm_fused_quant(x, bq, bs)
            assert ops.device_status()[0] == 0
            assert torch.equal(one.view(torch.int16), two.view(torch.int16)), f"repeat {rep}"
    finally:
        ops.set_option("fused_prologue", 0)
    pair = ops.w8a8_block_fp8_gemm_fused_quant(x, bq, bs)   # default: quantiser + GEMM chained in one call
    assert torch.equal(pair.view(torch.int16), two.view(torch.int16))


def test_fused_quant_prologue_limits(ops):
    from inference_b200 import _capi
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    lib = _capi.lib
    assert lib.inferop_w8a8_block_fp8_gemm_fused_quant(p, p, 2, p, p, 4, 128 * 70000, 128, 128, 128, 2, None) == _capi.ERR_LIMIT
    assert lib.inferop_w8a8_block_fp8_gemm_fused_quant(p, p, 0, p, p, 4, 256, 128, 128, 128, 2, None) == _capi.ERR_DTYPE
    assert lib.inferop_w8a8_block_fp8_gemm_fused_quant(p, p, 2, p, p, 4, 256, 100, 128, 128, 2, None) == _capi.ERR_SHAPE


@pytest.mark.parametrize("m,n,k", [(16, 18432, 7168), (4, 24576, 1536), (64, 7168, 18432), (48, 18432, 7168)])
def test_back_to_back_steps_share_buffers_without_a_race(ops, m, n, k):
    """quant -> GEMM steps queued without a synchronisation, every step re-quantising different
    activations into the SAME q / scales buffers that the previous step's GEMM reads: the
    quantiser is launched with programmatic stream serialisation and may start under the tail of
    the small-M GEMM, so it must not write before that GEMM has completed.  Every step's result
    is compared with the same step run on its own."""
    from inference_b200 import synth
    bq, bs = synth.quantised_weights(n, k, seed=21)
    xs = [synth.activations(m, k, seed=30 + i) for i in range(4)]
    want = []
    for x in xs:
        aq, a_s = ops.quant_fp8_per_token_group(x)
        want.append(ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs))
        torch.cuda.synchronize()
    aq = torch.empty((m, k), dtype=torch.uint8, device="cuda")
    a_s = torch.empty((m, k // 128), dtype=torch.float32, device="cuda")
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in range(24)]
    for i, c in enumerate(outs):
        ops.quant_fp8_per_token_group(xs[i % 4], 128, aq, a_s)
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=c)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    for i, c in enumerate(outs):
        assert torch.equal(c, want[i % 4]), f"step {i} differs from the same step run alone"
    # the same chain replayed from a CUDA graph (programmatic edges are captured as such)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=outs[0])   # creates this stream's scratch before the capture
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i, c in enumerate(outs):
                ops.quant_fp8_per_token_group(xs[i % 4], 128, aq, a_s)
                ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=c)
        for c in outs:
            c.zero_()
        g.replay()
        g.replay()
        torch.cuda.synchronize()
    for i, c in enumerate(outs):
        assert torch.equal(c, want[i % 4]), f"graph replay: step {i} differs"
