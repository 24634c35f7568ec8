"""Parity on the shapes the benchmark numbers are quoted on, through the C ABI.

The fp64 golden costs O(M N K) on the host, so these full-size results are checked on a
sub-matrix against the oracle (oracle/sampled.py: at least 16 rows from every 4096-row band,
columns stratified over the whole width, plus the first and last row), and through properties
that do not depend on the size: quantisation bytes equal to the oracle's on the sampled rows,
the CTA-pair kernel and the single-CTA kernel agree bit for bit on the whole matrix, the
grouped launch agrees bit for bit with one call per expert on the sampled experts.
Tolerances: max |err| <= 1e-2 * ||row||_inf and relative Frobenius <= 2e-3 (bf16 output).
"""
import numpy as np
import pytest
import torch

from oracle import sampled

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    yield _ops
    for key, val in (("gemm_pair", -1), ("gemm_path", 0), ("gemm_block_n", 0)):
        _ops.set_option(key, val)


def _check(ops, aq, a_s, bq, bs, c, seed, rows=None, n_cols=576):
    assert ops.device_status()[0] == 0
    m, n = c.shape
    rows = sampled.band_rows(m, 16, seed) if rows is None else rows
    cols = sampled.stratified(n, n_cols, seed + 1)
    row, fro = sampled.gemm_sample(aq, a_s, bq, bs, c, rows, cols)
    assert row <= sampled.ROW_TOL and fro <= sampled.FRO_TOL_16BIT, f"row {row:.3e} frobenius {fro:.3e}"
    return rows


# the N-sharded configuration (per-rank shards N/G for G = 1, 2, 4, 8) and the prefill shapes at M = 16384
@pytest.mark.parametrize("n,k", [(73728, 7168), (36864, 7168), (18432, 7168), (9216, 7168), (7168, 18432)])
def test_m16384_shapes_sampled_against_the_oracle(ops, n, k):
    from inference_b200 import synth
    m = 16384
    x = synth.activations(m, k, seed=0, outliers=True)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    bq, bs = synth.quantised_weights(n, k, seed=1 + n % 7)
    ops.set_option("gemm_pair", -1)
    c = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
    rows = _check(ops, aq, a_s, bq, bs, c, seed=n + k)
    assert sampled.quant_rows_exact(x, aq, a_s, rows)
    # the other large-tile kernel must produce the same bits everywhere (same sums in the same order)
    ops.set_option("gemm_pair", 0)
    ops.set_option("gemm_path", 1)
    try:
        c1 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
        ops.set_option("gemm_pair", 1)
        c2 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, torch.bfloat16)
    finally:
        ops.set_option("gemm_pair", -1)
        ops.set_option("gemm_path", 0)
    assert ops.device_status()[0] == 0
    assert torch.equal(c1, c2) and torch.equal(c, c2)


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (257, 300, 384), (300, 1000, 1536), (1000, 1536, 2048),
                                   (129, 257, 384), (4096, 2048, 1024), (513, 7168, 2048)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32, torch.float16])
def test_pair_kernel_equals_single_cta_kernel_and_oracle(ops, m, n, k, dt):
    """Ragged M and N, N * 2 not a multiple of 16 (no TMA store), a second CTA without rows."""
    from inference_b200 import synth
    x = synth.activations(m, k, seed=m + n, outliers=True)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    bq, bs = synth.quantised_weights(n, k, seed=3)
    canary = torch.full((m * n + 2048,), -5.0, dtype=dt, device="cuda")
    ops.set_option("gemm_path", 1)
    try:
        ops.set_option("gemm_pair", 0)
        c1 = ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, dt)
        ops.set_option("gemm_pair", 1)
        c2 = canary[:m * n].view(m, n)
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=c2)
    finally:
        ops.set_option("gemm_pair", -1)
        ops.set_option("gemm_path", 0)
    assert ops.device_status()[0] == 0
    assert bool((canary[m * n:] == -5.0).all()), "the pair kernel wrote past the output"
    assert torch.equal(c1, c2)
    rows = sampled.band_rows(m, 24, seed=m)
    cols = sampled.stratified(n, 256, seed=n)
    row, fro = sampled.gemm_sample(aq, a_s, bq, bs, c2, rows, cols)
    tol = sampled.FRO_TOL_F32 if dt == torch.float32 else sampled.FRO_TOL_16BIT
    assert row <= sampled.ROW_TOL and fro <= tol, f"row {row:.3e} frobenius {fro:.3e}"


def _expert_weights(synth, experts, n, k, seed):
    bq = torch.empty((experts, n, k), dtype=torch.uint8, device="cuda")
    bs = torch.empty((experts, n // 128, k // 128), dtype=torch.float32, device="cuda")
    step = 32
    for e0 in range(0, experts, step):
        q, s_ = synth.quantised_weights(step * n, k, seed=seed + e0)
        bq[e0:e0 + step] = q.view(step, n, k)
        bs[e0:e0 + step] = s_.view(step, n // 128, k // 128)
        del q, s_
    return bq, bs


@pytest.mark.parametrize("name,n,k", [("gate_up", 4096, 7168), ("down", 7168, 2048)])
def test_256_expert_grouped_launch_on_sampled_experts(ops, name, n, k):
    """The MoE configuration at full size: 256 experts, top-8 of 4096 tokens (32768 routed rows).
    Experts checked: the one with the fewest rows, the one with the most, the first, the last and
    two more; every row of theirs x 256 stratified columns against the oracle, and the whole
    block of rows bit for bit against a plain GEMM call on that expert."""
    from inference_b200 import synth
    experts, tokens, topk = 256, 4096, 8
    g = torch.Generator(device="cpu")
    g.manual_seed(11)
    logits = torch.randn((tokens, experts), generator=g, dtype=torch.float32)
    ids = torch.topk(torch.softmax(logits, dim=1), topk, dim=1).indices
    counts = torch.bincount(ids.flatten(), minlength=experts).tolist()
    m_total = tokens * topk
    x = synth.activations(m_total, k, seed=12, outliers=True)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    bq, bs = _expert_weights(synth, experts, n, k, seed=100 if name == "gate_up" else 500)
    canary = torch.full((m_total * n + 4096,), -9.0, dtype=torch.bfloat16, device="cuda")
    c = canary[:m_total * n].view(m_total, n)
    ops.w8a8_block_fp8_gemm_grouped(aq, a_s, bq, bs, counts, out=c)
    assert ops.device_status()[0] == 0
    assert bool((canary[m_total * n:] == -9.0).all())
    # the same through the device-side tile list
    lay = ops.moe_align(ids.to(torch.int32).cuda(), experts)
    c_dev = ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay, torch.bfloat16)
    assert ops.device_status()[0] == 0
    assert torch.equal(c, c_dev)
    offsets = np.concatenate([[0], np.cumsum(counts)])
    nonzero = [e for e in range(experts) if counts[e] > 0]
    picks = {min(nonzero, key=lambda e: counts[e]), max(nonzero, key=lambda e: counts[e]), nonzero[0], nonzero[-1],
             nonzero[len(nonzero) // 3], nonzero[2 * len(nonzero) // 3]}
    ops.set_option("gemm_path", 1)
    ops.set_option("gemm_pair", 0)
    try:
        for e in sorted(picks):
            r0, r1 = int(offsets[e]), int(offsets[e + 1])
            single = ops.w8a8_block_fp8_gemm(aq[r0:r1], a_s[r0:r1], bq[e], bs[e], torch.bfloat16)
            assert torch.equal(c[r0:r1], single), f"expert {e} ({r1 - r0} rows) differs from its own call"
            cols = sampled.stratified(n, 256, seed=e)
            row, fro = sampled.gemm_sample(aq[r0:r1], a_s[r0:r1], bq[e], bs[e], c[r0:r1], np.arange(r1 - r0), cols)
            assert row <= sampled.ROW_TOL and fro <= sampled.FRO_TOL_16BIT, f"expert {e}: row {row:.3e} fro {fro:.3e}"
    finally:
        ops.set_option("gemm_path", 0)
        ops.set_option("gemm_pair", -1)
