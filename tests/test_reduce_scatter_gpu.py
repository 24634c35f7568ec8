"""Row-parallel (K-sharded) GEMM with the reduce-scatter done by the GEMM epilogue (fp32 partial
tiles stored into the row owner's slots) plus an ordered sum on the owner.  One GPU: the ranks are
emulated as successive calls writing into several slot buffers of the same device; two or more
GPUs: one process per GPU over peer-mapped slots (reduce_scatter_worker.py)."""
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
    _ops.set_option("gemm_path", 1)   # the partial GEMMs below must run on the kernel the scatter form uses
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


@pytest.mark.parametrize("world,m,n,k", [(1, 128, 256, 256), (2, 256, 384, 512), (4, 512, 200, 1024),
                                         (8, 1024, 7168, 1024), (3, 384, 132, 768)])
def test_emulated_ranks_scatter_then_ordered_sum(ops, world, m, n, k):
    from inference_b200 import shard
    aq, a_s, bq, bs = case(m, n, k, seed=world * 77 + n)
    d = [cuda(x) for x in (aq, a_s, bq, bs)]
    rows = m // world
    # owner d's slots, with guard rows before and after
    slots = [torch.full((world * rows + 2, n), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
    ptrs = [s[1:].data_ptr() for s in slots]
    partial = []
    for rank in range(world):
        sh = shard.shard_k(*d, world, rank)
        ops.w8a8_block_fp8_gemm_scatter(ptrs, rank, *sh)
        partial.append(ops.w8a8_block_fp8_gemm(*sh, out_dtype=torch.float32))   # the same partial, locally
    assert ops.device_status()[0] == 0
    golden = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    for owner in range(world):
        lo, hi = shard.owner_rows(m, world, owner)
        buf = slots[owner]
        assert bool(buf[0].isnan().all()) and bool(buf[-1].isnan().all()), "store outside the slots"
        view = buf[1:-1].view(world, rows, n)
        for rank in range(world):
            assert torch.equal(view[rank], partial[rank][lo:hi]), "slot differs from the rank's partial GEMM"
        got = ops.reduce_slots(view.contiguous())
        acc = partial[0][lo:hi].clone()
        for rank in range(1, world):
            acc = acc + partial[rank][lo:hi]
        assert torch.equal(got, acc.to(torch.bfloat16)), "ordered fp32 sum, one rounding"
        row, fro = gemm_errors(got.float().cpu().numpy(), golden[lo:hi])
        assert row <= GEMM_ROW_TOL and fro <= GEMM_FRO_TOL_BF16


def test_reduce_slots_output_types(ops):
    g = torch.Generator(device="cuda").manual_seed(3)
    slots = torch.randn((5, 64, 36), device="cuda", generator=g)
    acc = slots[0].clone()
    for r in range(1, 5):
        acc = acc + slots[r]
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        assert torch.equal(ops.reduce_slots(slots, dt), acc.to(dt))


def test_rejected_calls(ops):
    from inference_b200._capi import InferopError
    aq, a_s, bq, bs = case(256, 256, 256, seed=1)
    d = [cuda(x) for x in (aq, a_s, bq, bs)]
    buf = torch.zeros((256, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(InferopError):      # rows do not split into whole tiles per owner
        ops.w8a8_block_fp8_gemm_scatter([buf.data_ptr()] * 4, 0, *d)
    with pytest.raises(InferopError):      # rank outside the group
        ops.w8a8_block_fp8_gemm_scatter([buf.data_ptr()] * 2, 2, *d)
    with pytest.raises(InferopError):      # slots not 16-byte aligned
        ops.w8a8_block_fp8_gemm_scatter([buf.data_ptr() + 4, buf.data_ptr()], 0, *d)
    torch.cuda.synchronize()
    assert not bool(buf.any())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_processes_over_peer_mapped_slots():
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29741",
           os.path.join(HERE, "reduce_scatter_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "reduce-scatter parity ok" in res.stdout
