"""RMSNorm, residual add + RMSNorm and the NeoX rotary embedding through the C ABI against the
oracle (reference/reference.cpp:11-53) and the reference's golden vectors, with the tolerances of
the reference's own GPU tests (tests/test_rmsnorm.cpp:96-99, tests/test_rope.cpp:82-83)."""
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-5, 1e-5), torch.float16: (3e-3, 3e-3), torch.bfloat16: (2e-2, 2e-2)}


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    return _ops


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def rounded(a, dtype):
    """The fp32 values a tensor of `dtype` holds after the inputs were rounded to it."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).float().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(33, 1024), (1, 7168), (5, 8192), (300, 128), (7, 16384), (3, 2048 * 16),
                                       (9, 130), (4, 1), (17, 1000)])
def test_rmsnorm_matches_the_oracle(ops, dtype, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    x = rounded(rng.standard_normal((rows, cols)).astype(np.float32), dtype)
    w = rounded(rng.uniform(0.5, 1.5, cols).astype(np.float32), dtype)
    want = oracle.rmsnorm(x, w, 1e-6)
    got = ops.rmsnorm(cuda(x, dtype), cuda(w, dtype), 1e-6).float().cpu().numpy()
    rtol, atol = TOL[dtype]
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)
    if dtype != torch.float32:
        # beyond the reference's tolerance: the 16-bit result is the rounded fp32 result up to one unit
        # in the last place (the row sum is added in a different order)
        exact = rounded(want, dtype)
        assert np.mean(got == exact) > 0.98


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(33, 1024), (2, 7168), (6, 130), (3, 2048 * 16)])
def test_fused_add_rmsnorm_matches_the_oracle(ops, dtype, rows, cols):
    rng = np.random.default_rng(rows * 11 + cols)
    res = rounded(rng.standard_normal((rows, cols)).astype(np.float32), dtype)
    x = rounded(rng.standard_normal((rows, cols)).astype(np.float32), dtype)
    w = rounded(rng.uniform(0.5, 1.5, cols).astype(np.float32), dtype)
    want_res, want_out = oracle.fused_add_rmsnorm(res, x, w, 1e-6)
    d_res = cuda(res, dtype)
    got_out = ops.fused_add_rmsnorm(d_res, cuda(x, dtype), cuda(w, dtype), 1e-6).float().cpu().numpy()
    got_res = d_res.float().cpu().numpy()
    assert np.array_equal(got_res, rounded(want_res, dtype)), "the residual is the rounded sum"
    rtol, atol = (1e-5, 1e-5) if dtype == torch.float32 else (3e-2, 3e-2)   # tests/test_rmsnorm.cpp:99
    np.testing.assert_allclose(got_out, want_out, rtol=rtol, atol=atol)
    # the output is computed from the stored (rounded) residual, as in the reference's kernel
    again = oracle.rmsnorm(got_res, w, 1e-6)
    rtol, atol = TOL[dtype]
    np.testing.assert_allclose(got_out, again, rtol=rtol, atol=atol)


def test_rmsnorm_golden_vectors(ops):
    g = np.load(os.path.join(GOLDEN, "norm_rope_golden.npz"))
    got = ops.rmsnorm(cuda(g["x"]), cuda(g["w"]), 1e-6).cpu().numpy()
    np.testing.assert_allclose(got, g["rms"], rtol=1e-5, atol=1e-5)
    res = cuda(g["res"])
    out = ops.fused_add_rmsnorm(res, cuda(g["x"]), cuda(g["w"]), 1e-6).cpu().numpy()
    assert np.array_equal(res.cpu().numpy(), g["fused_res"])
    np.testing.assert_allclose(out, g["fused_out"], rtol=1e-5, atol=1e-5)


def test_rmsnorm_leaves_the_neighbourhood_alone_and_takes_unaligned_rows(ops):
    rng = np.random.default_rng(5)
    rows, cols = 6, 1000          # 2000-byte rows of bf16: the element-wise kernel
    buf = torch.full((rows + 2, cols), 7.0, dtype=torch.bfloat16, device="cuda")
    x = cuda(rng.standard_normal((rows, cols)).astype(np.float32), torch.bfloat16)
    w = cuda(rng.uniform(0.5, 1.5, cols).astype(np.float32), torch.bfloat16)
    ops.rmsnorm(x, w, 1e-6, out=buf[1:rows + 1])
    assert bool((buf[0] == 7).all()) and bool((buf[rows + 1] == 7).all())
    want = oracle.rmsnorm(x.float().cpu().numpy(), w.float().cpu().numpy())
    np.testing.assert_allclose(buf[1:rows + 1].float().cpu().numpy(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("tokens,heads,dim,rot,base,yarn", [(64, 32, 128, 64, 10000.0, 1.0), (5, 3, 64, 64, 500000.0, 0.25),
                                                          (9, 1, 256, 2, 10000.0, 1.0), (3, 8, 96, 48, 10000.0, 1.0),
                                                          (17, 40, 128, 128, 10000.0, 1.0), (2, 9, 72, 36, 10000.0, 1.0)])
def test_rope_matches_the_oracle(ops, dtype, tokens, heads, dim, rot, base, yarn):
    rng = np.random.default_rng(tokens + heads + dim)
    q = rounded(rng.standard_normal((tokens, heads, dim)).astype(np.float32), dtype)
    pos = rng.integers(0, 131072, tokens).astype(np.int64)
    pos[0] = 0
    want = oracle.rope_neox(q, pos, rot, base, yarn)
    d_q = cuda(q, dtype)
    ops.rope_neox(d_q, cuda(pos), rot, base, yarn)
    got = d_q.float().cpu().numpy()
    assert np.array_equal(got[..., rot:], q[..., rot:]), "the tail beyond rotary_dim is untouched"
    assert np.array_equal(got[0], rounded(want[0], dtype)) or pos[0] != 0   # position 0: the identity
    if dtype == torch.float32:
        # the frequencies are the golden code's own (the C library's powf, computed on the host), so
        # fp32 agrees far inside the reference's tolerance (1e-4) even at positions beyond 100 000;
        # what is left is a unit or two in the last place of the device's sine and cosine
        np.testing.assert_allclose(got, want, rtol=5e-6, atol=5e-6)
        assert np.mean(got == want) > 0.5
    else:
        rtol, atol = TOL[dtype]
        np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)
        assert np.mean(got == rounded(want, dtype)) > 0.99


def test_rope_golden_vectors_and_properties(ops):
    g = np.load(os.path.join(GOLDEN, "norm_rope_golden.npz"))
    q = cuda(g["q"])
    ops.rope_neox(q, cuda(g["pos"]), 64)
    np.testing.assert_allclose(q.cpu().numpy(), g["rope"], rtol=5e-6, atol=5e-6)
    q2 = cuda(g["q2"])
    ops.rope_neox(q2, cuda(g["pos2"]), 64, 500000.0, 0.25)
    np.testing.assert_allclose(q2.cpu().numpy(), g["rope2"], rtol=5e-6, atol=5e-6)
    # pair norms are preserved (tests/test_rope.cpp:22-34)
    half = 32
    n0 = np.hypot(g["q"][..., :half].astype(np.float64), g["q"][..., half:64])
    n1 = np.hypot(q.cpu().numpy()[..., :half].astype(np.float64), q.cpu().numpy()[..., half:64])
    assert np.abs(n0 - n1).max() < 1e-4


def test_norm_and_rope_reject_bad_arguments(ops):
    from inference_b200 import _capi
    lib = _capi.lib
    t = torch.zeros(4096, dtype=torch.float32, device="cuda")
    p = t.data_ptr()
    assert lib.inferop_rmsnorm(p, p, p, 0, 0, 16, 1e-6, None) == _capi.ERR_SHAPE
    assert lib.inferop_rmsnorm(p, p, p, 5, 4, 16, 1e-6, None) == _capi.ERR_DTYPE
    assert lib.inferop_rmsnorm(None, p, p, 0, 4, 16, 1e-6, None) == _capi.ERR_POINTER
    assert lib.inferop_fused_add_rmsnorm(p, p, p, None, 0, 4, 16, 1e-6, None) == _capi.ERR_POINTER
    pos = torch.zeros(4, dtype=torch.int64, device="cuda").data_ptr()
    assert lib.inferop_rope_neox(p, pos, 0, 4, 2, 16, 18, 10000.0, 1.0, None) == _capi.ERR_SHAPE   # rotary_dim > head_dim
    assert lib.inferop_rope_neox(p, pos, 0, 4, 2, 16, 7, 10000.0, 1.0, None) == _capi.ERR_SHAPE    # odd
    assert lib.inferop_rope_neox(p, None, 0, 4, 2, 16, 8, 10000.0, 1.0, None) == _capi.ERR_POINTER
    torch.cuda.synchronize()
    assert bool((t == 0).all())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(33, 1024), (1, 7168), (300, 128), (7, 16384), (64, 2048), (5, 4096)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rmsnorm_with_quantisation_equals_the_two_calls(ops, dtype, rows, cols, with_residual):
    """The one-pass form gives the bytes and scales of rmsnorm (or fused_add_rmsnorm) followed by
    quant_fp8_per_token_group, bit for bit, and the same updated residual."""
    rng = np.random.default_rng(rows + cols)
    x = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).cuda().to(dtype)
    x[0, :128] = 0                                   # a group that normalises to zeros
    w = torch.from_numpy(rng.uniform(0.5, 1.5, cols).astype(np.float32)).cuda().to(dtype)
    if with_residual:
        res = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).cuda().to(dtype)
        res[0, :128] = 0
        r1, r2 = res.clone(), res.clone()
        y = ops.fused_add_rmsnorm(r1, x, w, 1e-6)
        q, s = ops.rmsnorm_quant(x, w, 1e-6, residual=r2)
        assert torch.equal(r1.view(torch.int16), r2.view(torch.int16))
    else:
        y = ops.rmsnorm(x, w, 1e-6)
        q, s = ops.rmsnorm_quant(x, w, 1e-6)
    q_want, s_want = ops.quant_fp8_per_token_group(y)
    assert torch.equal(s, s_want)
    assert torch.equal(q, q_want)
    # and the chain against the oracle: quantising the oracle's rounded norm gives the same scales up to the
    # rare element that rounds differently (the row sum is added in another order)
    got_s = s.cpu().numpy()
    xin = (x.float() + (res.float() if with_residual else 0)).to(dtype).float().cpu().numpy() if with_residual else x.float().cpu().numpy()
    gold = oracle.rmsnorm(xin, w.float().cpu().numpy(), 1e-6)
    _, s_gold = oracle.quant_fp8_per_token_group(rounded(gold, dtype))
    np.testing.assert_allclose(got_s, s_gold, rtol=2e-2, atol=1e-8)


def test_rmsnorm_with_quantisation_rejects_what_it_cannot_do(ops):
    from inference_b200 import _capi
    lib = _capi.lib
    t = torch.zeros(1 << 16, dtype=torch.bfloat16, device="cuda")
    p = t.data_ptr()
    assert lib.inferop_rmsnorm_quant(p, p, None, p, p, 2, 4, 1000, 128, 1e-6, None) == _capi.ERR_SHAPE     # cols % 128
    assert lib.inferop_rmsnorm_quant(p, p, None, p, p, 2, 4, 32768, 128, 1e-6, None) == _capi.ERR_SHAPE    # too wide
    assert lib.inferop_rmsnorm_quant(p, p, None, p, p, 0, 4, 1024, 128, 1e-6, None) == _capi.ERR_DTYPE     # fp32
    assert lib.inferop_rmsnorm_quant(p, p, None, p + 2, p, 2, 4, 1024, 128, 1e-6, None) == _capi.ERR_POINTER
    assert lib.inferop_rmsnorm_quant(p, p, None, p, p, 2, 4, 1024, 64, 1e-6, None) == _capi.ERR_SHAPE      # group size
