"""Parity of the CUDA quantiser (through the C ABI) with the oracle: bytes and scales bit-exact."""
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    return _ops


def to_dev(bits_or_f32, dt):
    if dt == torch.bfloat16:
        return torch.from_numpy(np.ascontiguousarray(bits_or_f32).view(np.int16)).cuda().view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(bits_or_f32)).cuda()


def check_exact(ops, x_dev, x_f32_host, gs=128):
    q, s = ops.quant_fp8_per_token_group(x_dev, gs)
    torch.cuda.synchronize()
    q_want, s_want = oracle.quant_fp8_per_token_group(x_f32_host, gs)
    q, s = q.cpu().numpy(), s.cpu().numpy()
    bad = np.flatnonzero(q.ravel() != q_want.ravel())
    assert bad.size == 0, f"{bad.size} byte mismatches, first at {bad[:5]}: got {q.ravel()[bad[:5]]} want {q_want.ravel()[bad[:5]]}"
    assert np.array_equal(s.view(np.uint32), s_want.view(np.uint32))
    return q, s


def test_hardware_converter_equals_software_encoder_on_all_floats(ops):
    import ctypes as C
    from inference_b200 import _capi
    out = (C.c_uint64 * 2)()
    _capi.check(_capi.lib.inferop_selftest_e4m3_cvt(0, 1 << 32, out), "selftest")
    assert out[0] == 0, f"{out[0]} non-NaN inputs convert differently"


@pytest.mark.parametrize("dt", [1, 2])
def test_reciprocal_division_equals_ieee_division_on_the_whole_16bit_domain(ops, dt):
    import ctypes as C
    from inference_b200 import _capi
    out = (C.c_uint64 * 3)()
    _capi.check(_capi.lib.inferop_selftest_quant_div(dt, out), "selftest")
    assert out[1] > 1 << 29, f"the sweep did not cover the domain ({out[1]} pairs)"
    assert out[0] == 0, (f"{out[0]} of {out[1]} (group maximum, element) pairs give a different byte, "
                         f"e.g. maximum bits {out[2] >> 32:#06x} element bits {out[2] & 0xFFFF:#06x}")


def test_golden_vectors_bf16_gs128_gs64_fp32(ops):
    g = np.load(os.path.join(GOLDEN, "quant_golden.npz"))
    x = to_dev(g["x_bf16_bits"], torch.bfloat16)
    q, s = ops.quant_fp8_per_token_group(x, 128)
    assert np.array_equal(q.cpu().numpy(), g["q"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), g["scales"].view(np.uint32))
    q, s = ops.quant_fp8_per_token_group(x, 64)
    assert np.array_equal(q.cpu().numpy(), g["q_gs64"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), g["scales_gs64"].view(np.uint32))
    q, s = ops.quant_fp8_per_token_group(to_dev(g["x_f32"], torch.float32), 128)
    assert np.array_equal(q.cpu().numpy(), g["q_f32"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), g["scales_f32"].view(np.uint32))


@pytest.mark.parametrize("rows,cols", [(1, 128), (3, 384), (64, 768), (17, 7168), (257, 1536), (4096, 7168)])
def test_bf16_matches_oracle(ops, rows, cols):
    rng = np.random.default_rng(rows * 100003 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[:, rng.choice(cols, max(1, cols // 100), replace=False)] *= 20.0  # outlier channels
    bits = oracle.bf16_narrow(x)
    check_exact(ops, to_dev(bits, torch.bfloat16), oracle.bf16_widen(bits))


@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_other_input_dtypes(ops, dt):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((64, 768)).astype(np.float32)  # the reference test's shape
    if dt == torch.float16:
        x = x.astype(np.float16).astype(np.float32)
        check_exact(ops, torch.from_numpy(x).cuda().half(), x)
    else:
        check_exact(ops, to_dev(x, dt), x)


def test_edge_values(ops):
    x = np.zeros((8, 256), np.float32)
    x[1, :] = np.random.default_rng(0).standard_normal(256) * 1e-38   # subnormal scales
    x[2, 3] = np.nan
    x[2, 4] = -np.nan
    x[2, 5:128] = 1.0
    x[3, 0] = np.inf
    x[3, 1] = -1.0
    x[3, 2] = -np.inf
    x[4, :] = -0.0
    x[5, :] = 3.3895314e38   # bf16 max
    x[6, 128:] = np.random.default_rng(1).standard_normal(128) * 1e30
    x[7, ::2] = 1e-45
    check_exact(ops, to_dev(x, torch.float32), x)
    bits = oracle.bf16_narrow(x)
    bits[2, 3] = 0x7FC0
    bits[2, 4] = 0xFFC0
    check_exact(ops, to_dev(bits, torch.bfloat16), oracle.bf16_widen(bits))


def test_generic_group_sizes(ops):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((5, 960)).astype(np.float32)
    for gs in (32, 64, 192, 960):
        check_exact(ops, to_dev(x, torch.float32), x, gs)


def test_rejected_shapes_raise_and_write_nothing(ops):
    from inference_b200 import _capi
    x = torch.zeros((4, 100), dtype=torch.bfloat16, device="cuda")
    q = torch.full((4, 100), 7, dtype=torch.uint8, device="cuda")
    s = torch.full((4, 1), 7.0, device="cuda")
    rc = _capi.lib.inferop_quant_fp8_per_token_group(q.data_ptr(), s.data_ptr(), x.data_ptr(), 2, 4, 100, 128, None)
    torch.cuda.synchronize()
    assert rc == _capi.ERR_SHAPE and bool((q == 7).all()) and bool((s == 7).all())


def test_dequant_matches_oracle(ops):
    rng = np.random.default_rng(12)
    x = rng.standard_normal((64, 768)).astype(np.float32)
    q, s = oracle.quant_fp8_per_token_group(x)
    want = oracle.dequant_fp8_per_token_group(q, s)
    got = ops.dequant_fp8_per_token_group(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), torch.float32)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    got = ops.dequant_fp8_per_token_group(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), torch.bfloat16)
    assert np.array_equal(got.cpu().view(torch.int16).numpy().view(np.uint16), oracle.bf16_narrow(want))


def test_full_size_properties(ops):
    """16384 x 7168 (the sharded config's activations): idempotent, scales are the row-group
    absmax * fl(1/448), sampled rows equal the oracle."""
    from inference_b200 import synth
    x = synth.activations(16384, 7168, seed=0)
    q, s = ops.quant_fp8_per_token_group(x)
    q2, s2 = ops.quant_fp8_per_token_group(x)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    amax = x.float().abs().view(16384, 56, 128).amax(dim=2)
    want_s = torch.where(amax == 0, torch.ones_like(amax), amax * torch.tensor(1.0 / 448.0, device="cuda"))
    assert torch.equal(s, want_s)
    rows = np.random.default_rng(0).choice(16384, 48, replace=False)
    xh = x[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    q_want, s_want = oracle.quant_fp8_per_token_group(xh)
    assert np.array_equal(q[torch.from_numpy(rows).cuda()].cpu().numpy(), q_want)
    assert np.array_equal(s[torch.from_numpy(rows).cuda()].cpu().numpy(), s_want)
