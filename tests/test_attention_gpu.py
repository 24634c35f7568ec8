"""Paged attention decode through the C ABI against the oracle (reference/reference.cpp:112-150) with
the cases and tolerances of the reference's own GPU test (tests/test_paged_attn.cpp:110-117) and more:
shuffled physical blocks, empty sequences, groups of 1 / 2 / 4 / 8 query heads per KV head, sequences
long enough to be cut into several token ranges."""
import numpy as np
import pytest
import torch

import oracle
from test_oracle_cpu import attn_case

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (2e-3, 2e-3), torch.float16: (5e-3, 5e-3), torch.bfloat16: (2e-2, 2e-2)}


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    return _ops


def rounded(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).float().numpy()


def run_case(ops, dtype, batch, heads, kv_heads, dim, block_size, lens, shuffle, seed=0):
    q, k, v, tables, sl = attn_case(batch, heads, kv_heads, dim, block_size, lens, seed=seed, shuffle=shuffle)
    q, k, v = rounded(q, dtype), rounded(k, dtype), rounded(v, dtype)
    scale = float(1.0 / np.sqrt(dim))
    want = oracle.paged_attn_decode(q, k, v, tables, sl, scale)
    cu = lambda a, dt=None: torch.from_numpy(a).cuda().to(dt) if dt is not None else torch.from_numpy(a).cuda()
    got = ops.paged_attn_decode(cu(q, dtype), cu(k, dtype), cu(v, dtype), cu(tables), cu(sl), scale)
    torch.cuda.synchronize()
    return got.float().cpu().numpy(), want


@pytest.mark.parametrize("case,dtype", [
    ((3, 32, 8, 128, 16, [1, 17, 129]), torch.float32),
    ((3, 32, 8, 128, 16, [1, 17, 129]), torch.bfloat16),
    ((2, 16, 4, 64, 16, [5, 64]), torch.bfloat16),
    ((2, 8, 8, 256, 16, [33, 200]), torch.bfloat16),
    ((1, 32, 8, 128, 16, [2048]), torch.bfloat16),
])
def test_the_reference_tests_own_cases(ops, case, dtype):
    got, want = run_case(ops, dtype, *case, shuffle=False)
    rtol, atol = TOL[dtype]
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads", [(8, 8), (8, 4), (16, 4), (32, 4), (6, 2), (5, 5), (12, 4)])
@pytest.mark.parametrize("dim", [64, 128, 256])
def test_head_groups_and_head_sizes(ops, dtype, heads, kv_heads, dim):
    got, want = run_case(ops, dtype, 3, heads, kv_heads, dim, 16, [1, 40, 333], shuffle=True, seed=heads + dim)
    rtol, atol = TOL[dtype]
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol)
    if dtype == torch.float32:
        np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5)   # far inside the reference's 2e-3


@pytest.mark.parametrize("block_size", [1, 8, 16, 32, 128])
def test_block_sizes_empty_sequences_and_long_ones(ops, block_size):
    lens = [0, 1, 4097, 0, 777, 9000]
    got, want = run_case(ops, torch.bfloat16, len(lens), 8, 2, 128, block_size, lens, shuffle=True, seed=block_size)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
    assert np.array_equal(got[0], np.zeros_like(got[0])) and np.array_equal(got[3], np.zeros_like(got[3]))


def test_a_single_long_sequence_is_cut_into_ranges_and_merged(ops):
    got, want = run_case(ops, torch.float32, 1, 16, 2, 128, 16, [20000], shuffle=True, seed=9)
    np.testing.assert_allclose(got, want, rtol=5e-5, atol=5e-5)
    # sequence lengths beyond the table are clamped to what the table covers
    q, k, v, tables, sl = attn_case(2, 4, 2, 64, 16, [48, 48], seed=3)
    scale = 0.125
    want = oracle.paged_attn_decode(q, k, v, tables, sl, scale)
    big = np.array([1000, 48], np.int32)
    cu = lambda a: torch.from_numpy(a).cuda()
    got = ops.paged_attn_decode(cu(q), cu(k), cu(v), cu(tables), cu(big), scale).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5)


def test_length_one_returns_the_value_row_and_outputs_stay_in_range(ops):
    q, k, v, tables, sl = attn_case(3, 32, 8, 128, 16, [1, 17, 129])
    cu = lambda a: torch.from_numpy(a).cuda()
    out = ops.paged_attn_decode(cu(q), cu(k), cu(v), cu(tables), cu(sl), float(1 / np.sqrt(128))).cpu().numpy()
    np.testing.assert_allclose(out[0, 0], v[tables[0, 0], 0, 0], atol=1e-5)
    assert out.min() >= v.min() - 1e-3 and out.max() <= v.max() + 1e-3


def test_rejected_calls(ops):
    from inference_b200 import _capi
    lib = _capi.lib
    t = torch.zeros(1 << 14, dtype=torch.float32, device="cuda")
    p = t.data_ptr()
    i = torch.zeros(16, dtype=torch.int32, device="cuda").data_ptr()
    assert lib.inferop_paged_attn_decode(p, p, p, p, i, i, 0, 1, 8, 3, 128, 16, 4, 0.1, None) == _capi.ERR_SHAPE    # 8 % 3
    assert lib.inferop_paged_attn_decode(p, p, p, p, i, i, 0, 1, 8, 4, 96, 16, 4, 0.1, None) == _capi.ERR_SHAPE     # head_dim
    assert lib.inferop_paged_attn_decode(p, p, p, p, i, i, 4, 1, 8, 4, 128, 16, 4, 0.1, None) == _capi.ERR_DTYPE
    assert lib.inferop_paged_attn_decode(p, p, p + 4, p, i, i, 0, 1, 8, 4, 128, 16, 4, 0.1, None) == _capi.ERR_POINTER
    assert lib.inferop_paged_attn_decode(p, p, p, p, None, i, 0, 1, 8, 4, 128, 16, 4, 0.1, None) == _capi.ERR_POINTER
    torch.cuda.synchronize()
    assert bool((t == 0).all())
