"""The all-gather variant of the GEMM: each rank's epilogue writes its column shard into every
rank's full result.  On one GPU the ranks are emulated as successive calls that write into
several buffers of the same device; with two or more GPUs the same check runs as one process
per GPU over peer-mapped buffers (worker: allgather_worker.py)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from conftest import GEMM_FRO_TOL_BF16, GEMM_ROW_TOL, gemm_errors

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    # the comparisons below are bit for bit: keep the plain GEMM on the same (large-tile) kernel
    # as the all-gather variant for the small row counts too
    _ops.set_option("gemm_path", 1)
    yield _ops
    _ops.set_option("gemm_path", 0)


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def case(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32)))
    w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    return aq, a_s, bq, bs


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("m,n_shard,k,dt", [(200, 384, 512, torch.bfloat16), (77, 128, 256, torch.float16),
                                            (300, 256, 384, torch.bfloat16)])
def test_emulated_ranks_fill_every_buffer_with_the_full_result(ops, world, m, n_shard, k, dt):
    from inference_b200 import shard
    n = n_shard * world
    aq, a_s, bq, bs = case(m, n, k, seed=world * 1000 + m)
    d_aq, d_as, d_bq, d_bs = cuda(aq), cuda(a_s), cuda(bq), cuda(bs)
    want_local = ops.w8a8_block_fp8_gemm(d_aq, d_as, d_bq, d_bs, dt)         # the plain GEMM
    # guard rows before and after every buffer: the peer stores must stay inside [M, N]
    bufs = [torch.full((m + 2, n), -7.0, dtype=dt, device="cuda") for _ in range(world)]
    ptrs = [b[1:].data_ptr() for b in bufs]
    for rank in range(world):
        wq, ws = shard.shard_weights(d_bq, d_bs, world, rank)
        ops.w8a8_block_fp8_gemm_allgather(ptrs, rank, d_aq, d_as, wq, ws, dt)
    assert ops.device_status()[0] == 0
    for b in bufs:
        assert torch.equal(b[1:m + 1], want_local), "a rank's buffer differs from the unsharded GEMM"
        assert bool((b[0] == -7.0).all()) and bool((b[m + 1] == -7.0).all()), "store outside the buffer"
    golden = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    row, fro = gemm_errors(bufs[-1][1:m + 1].float().cpu().numpy(), golden)
    assert row <= GEMM_ROW_TOL and fro <= GEMM_FRO_TOL_BF16 * (4 if dt == torch.float16 else 1)


@pytest.mark.parametrize("m", [1, 16, 50, 96])
def test_few_tokens_take_the_weight_streaming_kernel_and_fill_every_buffer(ops, m):
    from inference_b200 import shard
    world, n_shard, k = 4, 384, 1024
    aq, a_s, bq, bs = case(m, n_shard * world, k, seed=40 + m)
    d_aq, d_as, d_bq, d_bs = cuda(aq), cuda(a_s), cuda(bq), cuda(bs)
    ops.set_option("gemm_path", 0)
    try:
        want = ops.w8a8_block_fp8_gemm(d_aq, d_as, d_bq, d_bs)        # same kernel, unsharded
        bufs = [torch.full((m + 2, n_shard * world), -7.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for rank in range(world):
            wq, ws = shard.shard_weights(d_bq, d_bs, world, rank)
            ops.w8a8_block_fp8_gemm_allgather([b[1:].data_ptr() for b in bufs], rank, d_aq, d_as, wq, ws)
        assert ops.device_status()[0] == 0
    finally:
        ops.set_option("gemm_path", 1)
    golden = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    for b in bufs:
        assert bool((b[0] == -7.0).all()) and bool((b[m + 1] == -7.0).all())
        row, fro = gemm_errors(b[1:m + 1].float().cpu().numpy(), golden)
        assert row <= GEMM_ROW_TOL and fro <= GEMM_FRO_TOL_BF16
        # split tiles add their K parts in a fixed order, but the parts depend on the shard's tile
        # count: equal to the unsharded call up to the rounding of the output type
        assert torch.allclose(b[1:m + 1].float(), want.float(), rtol=2e-2, atol=1e-3)


def test_only_the_ranks_own_columns_are_written(ops):
    from inference_b200 import shard
    world, m, n_shard, k = 4, 130, 128, 256
    aq, a_s, bq, bs = case(m, n_shard * world, k, seed=5)
    d_aq, d_as, d_bq, d_bs = cuda(aq), cuda(a_s), cuda(bq), cuda(bs)
    bufs = [torch.full((m, n_shard * world), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    wq, ws = shard.shard_weights(d_bq, d_bs, world, 2)
    ops.w8a8_block_fp8_gemm_allgather([b.data_ptr() for b in bufs], 2, d_aq, d_as, wq, ws)
    lo, hi = shard.peer_columns(n_shard, 2)
    for b in bufs:
        assert bool((b[:, :lo] == 3.0).all()) and bool((b[:, hi:] == 3.0).all())
        assert not bool((b[:, lo:hi] == 3.0).all())


def test_strided_output_gemm_writes_only_its_column_block(ops):
    for (m, n, k, ldc, col0) in [(300, 256, 512, 1024, 512), (130, 128, 256, 136, 8), (16, 384, 512, 1152, 768)]:
        aq, a_s, bq, bs = [cuda(t) for t in case(m, n, k, seed=m + ldc)]
        want = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
        wide = torch.full((m, ldc), 5.0, dtype=torch.bfloat16, device="cuda")
        ops.w8a8_block_fp8_gemm_into(wide, col0, aq, a_s, bq, bs)
        torch.cuda.synchronize()
        assert torch.equal(wide[:, col0:col0 + n], want)
        assert bool((wide[:, :col0] == 5.0).all()) and bool((wide[:, col0 + n:] == 5.0).all())
    assert ops.device_status()[0] == 0


def test_panel_gather_by_the_copy_engines_on_one_rank_equals_the_plain_gemm(ops):
    """Without a process group the gather degrades to one destination (this rank's own buffer):
    panels of the GEMM copied in by the copy engines must reproduce the plain GEMM."""
    from inference_b200 import shard
    for (m, n, k, panels) in [(1024, 384, 512, 8), (256, 1152, 1024, 2), (130, 256, 256, 8)]:
        aq, a_s, bq, bs = [cuda(t) for t in case(m, n, k, seed=m + n)]
        want = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
        pg = shard.PanelGather(m, n, torch.bfloat16, "cuda", panels=panels)
        for _ in range(2):
            got = pg(aq, a_s, bq, bs)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
    assert ops.device_status()[0] == 0


def test_rejected_calls(ops):
    from inference_b200._capi import InferopError
    aq, a_s, bq, bs = case(64, 256, 256, seed=1)
    d = [cuda(x) for x in (aq, a_s, bq, bs)]
    buf = torch.zeros((64, 512), dtype=torch.bfloat16, device="cuda")
    canary = buf.clone()
    with pytest.raises(InferopError):      # rank outside the group
        ops.w8a8_block_fp8_gemm_allgather([buf.data_ptr()] * 2, 2, *d)
    with pytest.raises(InferopError):      # more destinations than the kernel carries
        ops.w8a8_block_fp8_gemm_allgather([buf.data_ptr()] * 9, 0, *d)
    with pytest.raises(InferopError):      # fp32 output is not offered by this variant
        ops.w8a8_block_fp8_gemm_allgather([buf.data_ptr()] * 2, 0, *d, out_dtype=torch.float32)
    with pytest.raises(InferopError):      # destination not 16-byte aligned
        ops.w8a8_block_fp8_gemm_allgather([buf.data_ptr() + 2, buf.data_ptr()], 0, *d)
    with pytest.raises(InferopError):      # shard width not a multiple of 128
        ops.w8a8_block_fp8_gemm_allgather([buf.data_ptr()] * 2, 0, d[0], d[1], d[2][:192], d[3])
    torch.cuda.synchronize()
    assert torch.equal(buf, canary)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_peer_mapped_buffers():
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29731",
           os.path.join(HERE, "allgather_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "allgather parity ok" in res.stdout
