"""The mixture-of-experts kernels around the grouped GEMM, through the C ABI, against the oracle:
routing and SwiGLU follow the reference's CPU functions (reference/reference.cpp:152-181, :55-63);
the layout, scatter and combine kernels have no reference counterpart and are checked against the
oracle's restatement of what the reference's host loop over experts would do."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from inference_b200 import ops as _ops
    assert _ops.has_cuda() and _ops.device_sm_version(0) == 100, "needs a B200"
    _ops.set_option("gemm_path", 1)   # bit-for-bit comparisons between the large-tile GEMM's launch forms
    yield _ops
    _ops.set_option("gemm_path", 0)


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


# ------------------------------------------------------------------------------------ routing
@pytest.mark.parametrize("tokens,experts,topk", [(257, 256, 8), (3, 8, 2), (17, 1024, 16), (4096, 256, 8),
                                                 (33, 100, 3), (5, 32, 32), (64, 384, 6), (9, 600, 1)])
@pytest.mark.parametrize("renorm", [True, False])
def test_topk_softmax_matches_the_cpu_reference(ops, tokens, experts, topk, renorm):
    rng = np.random.default_rng(tokens * 31 + experts)
    logits = (2.0 * rng.standard_normal((tokens, experts))).astype(np.float32)   # the reference test's N(0, 2)
    want_ids, want_w = oracle.topk_softmax(logits, topk, renorm)
    ids, w = ops.topk_softmax(cuda(logits), topk, renorm)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    # tolerance of the reference's own GPU test (tests/test_topk.cpp:54-55)
    np.testing.assert_allclose(w.cpu().numpy(), want_w, rtol=1e-4, atol=1e-5)


def test_topk_softmax_and_swiglu_golden_vectors(ops):
    import os
    from conftest import GOLDEN
    g = np.load(os.path.join(GOLDEN, "moe_golden.npz"))
    for name, k in (("a", 8), ("b", 2), ("c", 16)):
        for renorm in (0, 1):
            ids, w = ops.topk_softmax(cuda(g[f"logits_{name}"]), k, bool(renorm))
            assert np.array_equal(ids.cpu().numpy(), g[f"ids_{name}{renorm}"])
            np.testing.assert_allclose(w.cpu().numpy(), g[f"w_{name}{renorm}"], rtol=1e-4, atol=1e-5)
    ids, w = ops.topk_softmax(cuda(g["logits_ties"]), 6, True)
    assert np.array_equal(ids.cpu().numpy(), g["ids_ties"])
    np.testing.assert_allclose(ops.silu_and_mul(cuda(g["gate_up"])).cpu().numpy(), g["silu"], rtol=2e-6, atol=1e-7)


def test_topk_softmax_breaks_ties_by_lower_index(ops):
    logits = np.zeros((4, 64), np.float32)
    logits[1, [5, 40, 41]] = 3.0
    logits[2, :] = np.arange(64)[::-1] // 8          # runs of 8 equal values
    logits[3, 63] = 1.0
    want_ids, want_w = oracle.topk_softmax(logits, 6, True)
    ids, w = ops.topk_softmax(cuda(logits), 6, True)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert ids[0].tolist() == [0, 1, 2, 3, 4, 5] and ids[1].tolist()[:3] == [5, 40, 41]
    np.testing.assert_allclose(w.cpu().numpy(), want_w, rtol=1e-4, atol=1e-5)


def test_topk_softmax_rejects_what_the_reference_ignores(ops):
    from inference_b200._capi import InferopError
    logits = torch.zeros((4, 2048), dtype=torch.float32, device="cuda")
    with pytest.raises(InferopError):
        ops.topk_softmax(logits, 4)                   # more than 1024 experts
    with pytest.raises(InferopError):
        ops.topk_softmax(logits[:, :8].contiguous(), 9)   # topk > experts


# ------------------------------------------------------------------------------------- SwiGLU
def test_silu_and_mul_fp32(ops):
    rng = np.random.default_rng(2)
    for (t, d) in [(64, 512), (7, 33), (1, 1)]:
        x = rng.standard_normal((t, 2 * d)).astype(np.float32) * 3
        want = oracle.silu_and_mul(x)
        got = ops.silu_and_mul(cuda(x)).cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("t,d", [(64, 2048), (5, 24), (3, 7)])
def test_silu_and_mul_16bit_is_the_rounded_fp32_result(ops, dt, t, d):
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.standard_normal((t, 2 * d)).astype(np.float32) * 3).to(dt)
    want = torch.from_numpy(oracle.silu_and_mul(x.float().numpy())).to(dt)
    got = ops.silu_and_mul(x.cuda()).cpu()
    # the exponential differs from the host's in the last bit now and then: allow one unit in
    # the last place of the 16-bit result on a small fraction of the elements
    diff = (got.view(torch.int16).int() - want.view(torch.int16).int()).abs()
    assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 5e-3


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_silu_and_mul_quant_equals_the_two_kernels_and_the_oracle(ops, dt):
    rng = np.random.default_rng(4)
    for (t, d) in [(300, 2048), (1, 128), (77, 384)]:
        x = torch.from_numpy(rng.standard_normal((t, 2 * d)).astype(np.float32) * 3).to(dt).cuda()
        x[0, :128] = 0          # a zero group: scale 1
        h = ops.silu_and_mul(x)
        q2, s2 = ops.quant_fp8_per_token_group(h)
        q1, s1 = ops.silu_and_mul_quant(x)
        assert torch.equal(q1, q2) and torch.equal(s1, s2)
        wq, ws = oracle.quant_fp8_per_token_group(h.float().cpu().numpy())
        assert np.array_equal(q1.cpu().numpy(), wq) and np.array_equal(s1.cpu().numpy(), ws)


# ------------------------------------------------------------------------------------- layout
@pytest.mark.parametrize("tokens,experts,topk", [(4096, 256, 8), (1, 8, 2), (100, 1024, 16), (513, 64, 4),
                                                 (40000, 16, 2), (31, 3, 1)])
def test_moe_align_matches_the_stable_sort(ops, tokens, experts, topk):
    rng = np.random.default_rng(tokens + experts)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    if tokens == 513:
        logits[:, 7] = -50.0         # an expert nobody picks
        logits[:, 3] += 4.0          # and a crowded one (several M-tiles)
    ids, _ = oracle.topk_softmax(logits, topk, True)
    counts, offsets, pos, src, row0, meta = oracle.moe_align(ids, experts)
    lay = ops.moe_align(cuda(ids), experts)
    torch.cuda.synchronize()
    assert np.array_equal(lay.counts.cpu().numpy(), counts)
    assert np.array_equal(lay.offsets.cpu().numpy(), offsets)
    assert np.array_equal(lay.pos.cpu().numpy(), pos)
    assert np.array_equal(lay.src_token.cpu().numpy(), src)
    n = int(lay.num_mtiles.item())
    assert n == len(row0) and n <= lay.max_mtiles
    assert np.array_equal(lay.tile_row0.cpu().numpy()[:n], row0)
    assert np.array_equal(lay.tile_meta.cpu().numpy()[:n], meta)


@pytest.mark.parametrize("tokens,experts,topk", [(4096, 256, 8), (700, 1024, 6), (9, 5, 2), (40000, 16, 2)])
def test_moe_align_layout_does_not_depend_on_the_cluster_size(ops, tokens, experts, topk):
    """The pairs are dealt to the warps of 1 to 8 CTAs; the stable order and the tile table must
    come out the same, also when some CTAs of the cluster get no pair at all."""
    rng = np.random.default_rng(tokens * 7 + experts)
    ids = rng.integers(0, experts, size=(tokens, topk)).astype(np.int32)
    ids[rng.random(ids.shape) < 0.02] = experts + 3          # ids another rank owns
    flat = ids.reshape(-1)
    own = np.nonzero(flat < experts)[0]
    order = own[np.argsort(flat[own], kind="stable")]
    rows = len(order)
    pos = np.full(flat.size, -1, np.int32)
    pos[order] = np.arange(rows, dtype=np.int32)
    src = (order // topk).astype(np.int32)
    counts = np.bincount(flat[own], minlength=experts).astype(np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    row0 = np.array([offsets[e] + r for e in range(experts) for r in range(0, counts[e], 128)], np.int32)
    meta = np.array([(e << 8) | (min(128, counts[e] - r) - 1) for e in range(experts)
                     for r in range(0, counts[e], 128)], np.int32)
    try:
        for ctas in (1, 2, 3, 8, 0):
            ops.set_option("align_ctas", ctas)
            lay = ops.moe_align(cuda(ids), experts)
            torch.cuda.synchronize()
            n = int(lay.num_mtiles.item())
            assert np.array_equal(lay.counts.cpu().numpy(), counts), ctas
            assert np.array_equal(lay.offsets.cpu().numpy(), offsets), ctas
            assert np.array_equal(lay.pos.cpu().numpy(), pos), ctas
            assert np.array_equal(lay.src_token.cpu().numpy()[:rows], src), ctas
            assert n == len(row0), ctas
            assert np.array_equal(lay.tile_row0.cpu().numpy()[:n], row0), ctas
            assert np.array_equal(lay.tile_meta.cpu().numpy()[:n], meta), ctas
    finally:
        ops.set_option("align_ctas", 0)


def test_moe_align_marks_ids_outside_the_expert_range(ops):
    ids = np.array([[0, 1], [9, 1], [-3, 0]], np.int32)
    lay = ops.moe_align(cuda(ids), 4)
    assert lay.pos.cpu().tolist() == [0, 2, -1, 3, -1, 1]
    assert lay.counts.cpu().tolist() == [2, 2, 0, 0]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_moe_scatter_quant_writes_the_quantised_row_to_every_copy(ops, dt):
    rng = np.random.default_rng(6)
    tokens, experts, topk, cols = 200, 16, 4, 512
    ids, _ = oracle.topk_softmax(rng.standard_normal((tokens, experts)).astype(np.float32), topk)
    x = torch.from_numpy(rng.standard_normal((tokens, cols)).astype(np.float32)).to(dt)
    x[3] = 0
    lay = ops.moe_align(cuda(ids), experts)
    q, s = ops.moe_scatter_quant(x.cuda(), lay)
    wq, ws = oracle.quant_fp8_per_token_group(x.float().numpy())
    src = lay.src_token.cpu().numpy()
    assert np.array_equal(q.cpu().numpy(), wq[src]) and np.array_equal(s.cpu().numpy(), ws[src])


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_moe_combine_is_the_ordered_fp32_sum(ops, dt):
    rng = np.random.default_rng(7)
    tokens, experts, topk, hidden = 150, 32, 8, 264
    ids, w = oracle.topk_softmax(rng.standard_normal((tokens, experts)).astype(np.float32), topk)
    y = torch.from_numpy(rng.standard_normal((tokens * topk, hidden)).astype(np.float32)).to(dt)
    lay = ops.moe_align(cuda(ids), experts)
    got = ops.moe_combine(y.cuda(), cuda(w), lay).cpu()
    want = torch.from_numpy(oracle.moe_combine(y.float().numpy(), w, lay.pos.cpu().numpy())).to(dt)
    assert torch.equal(got, want)


# ------------------------------------------------------------------- grouped GEMM, device tiles
def test_grouped_gemm_from_device_tiles_equals_the_host_count_form(ops):
    from inference_b200 import synth
    rng = np.random.default_rng(8)
    tokens, experts, topk, n, k = 700, 12, 3, 384, 512
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    logits[:, 5] = -60.0      # an empty expert
    ids, _ = oracle.topk_softmax(logits, topk)
    lay = ops.moe_align(cuda(ids), experts)
    x = synth.activations(tokens, k, seed=2)
    aq, a_s = ops.moe_scatter_quant(x, lay)
    bq, bs = synth.quantised_weights(experts * n, k, seed=3)
    bq, bs = bq.view(experts, n, k), bs.view(experts, n // 128, k // 128)
    got = ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay)
    want = ops.w8a8_block_fp8_gemm_grouped(aq, a_s, bq, bs, lay.counts.cpu().tolist())
    assert ops.device_status()[0] == 0
    assert torch.equal(got, want)


# ------------------------------------------------ SwiGLU + re-quantisation in the gate_up epilogue
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("tokens,experts,topk,inter,k", [(700, 12, 3, 384, 512), (64, 4, 2, 128, 256),
                                                          (4096, 64, 8, 2048, 1024)])
def test_swiglu_epilogue_equals_gemm_then_silu_and_mul_quant(ops, dt, tokens, experts, topk, inter, k):
    """One launch against the two it replaces (grouped GEMM with 16-bit output, then
    silu_and_mul_quant): bytes and scales must be identical; and against the oracle's chain
    (fp64 golden GEMM -> rounding -> SwiGLU -> quantisation) on one expert, where a 16-bit
    rounding of the GEMM result may differ by one unit in the last place."""
    from inference_b200 import synth
    rng = np.random.default_rng(tokens + inter)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    if experts > 4:
        logits[:, 1] = -60.0      # an empty expert
    ids, _ = oracle.topk_softmax(logits, topk)
    lay = ops.moe_align(cuda(ids), experts)
    x = synth.activations(tokens, k, seed=2).to(dt)
    aq, a_s = ops.moe_scatter_quant(x, lay)
    bq, bs = synth.quantised_weights(experts * 2 * inter, k, seed=3)
    bq, bs = bq.view(experts, 2 * inter, k), bs.view(experts, 2 * inter // 128, k // 128)
    pairs = tokens * topk
    gu = ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay, dt)
    q2, s2 = ops.silu_and_mul_quant(gu)
    canary = torch.full((pairs * inter + 4096,), 0xA5, dtype=torch.uint8, device="cuda")
    q1 = canary[:pairs * inter].view(pairs, inter)
    s1 = torch.full((pairs, inter // 128), -1.0, dtype=torch.float32, device="cuda")
    ops.w8a8_block_fp8_gemm_grouped_tiles_swiglu(aq, a_s, bq, bs, lay, dt, q1, s1)
    assert ops.device_status()[0] == 0
    assert bool((canary[pairs * inter:] == 0xA5).all())
    valid = int(lay.offsets.cpu()[-1].item())          # rows that belong to some expert
    assert torch.equal(q1[:valid], q2[:valid]) and torch.equal(s1[:valid], s2[:valid])


_SMALL_TILE_COUNTS = [1, 32, 33, 129, 160, 0, 5, 159, 31, 128, 290, 17]
_FORMS = [(1, 1), (0, 1), (1, 0), (0, 0)]    # (small tiles replicated, tiles claimed from a device counter)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_grouped_gemm_small_tiles_in_the_replicated_form_are_bit_equal(ops, dt):
    """M-tiles of at most 32 rows load their rows four times over and spread the columns over the
    four lane quarters; the arithmetic per element is that of the plain form, so toggling the form
    must not change a bit, and rows next to a small tile must stay untouched.  Nor may it matter
    whether the CTAs claim their tiles from the device counter or are dealt them round-robin."""
    from inference_b200 import synth
    experts, n, k = len(_SMALL_TILE_COUNTS), 640, 512            # 640 = two 256-wide tiles + half a tile
    ids = np.repeat(np.arange(experts, dtype=np.int32), _SMALL_TILE_COUNTS)
    ids = np.random.default_rng(21).permutation(ids).reshape(-1, 1)
    lay = ops.moe_align(cuda(ids), experts)
    x = synth.activations(ids.shape[0], k, seed=2)
    aq, a_s = ops.moe_scatter_quant(x, lay)
    bq, bs = synth.quantised_weights(experts * n, k, seed=3)
    bq, bs = bq.view(experts, n, k), bs.view(experts, n // 128, k // 128)
    outs = []
    try:
        for form, claimed in _FORMS:
            ops.set_option("grouped_rep", form)
            ops.set_option("grouped_dynamic", claimed)
            out = torch.full((ids.shape[0] + 8, n), 7.0, dtype=dt, device="cuda")
            ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay, out=out[:ids.shape[0]])
            assert ops.device_status()[0] == 0
            assert bool((out[ids.shape[0]:] == 7.0).all())
            outs.append(out)
    finally:
        ops.set_option("grouped_rep", 1)
        ops.set_option("grouped_dynamic", 1)
    for o in outs[1:]:
        assert torch.equal(outs[0], o)
    want = ops.w8a8_block_fp8_gemm_grouped(aq, a_s, bq, bs, _SMALL_TILE_COUNTS, dt)
    assert torch.equal(outs[0][:ids.shape[0]], want)
    # the one-row expert against the oracle
    r = int(lay.offsets.cpu()[0].item())
    gold = oracle.w8a8_block_fp8_gemm(aq[r:r + 1].cpu().numpy(), a_s[r:r + 1].cpu().numpy(),
                                      bq[0].cpu().numpy(), bs[0].cpu().numpy())
    got = outs[0][r:r + 1].float().cpu().numpy()
    assert np.linalg.norm(got - gold) <= 1e-2 * np.linalg.norm(gold)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_swiglu_epilogue_small_tiles_in_the_replicated_form_are_bit_equal(ops, dt):
    from inference_b200 import synth
    experts, inter, k = len(_SMALL_TILE_COUNTS), 256, 384
    ids = np.repeat(np.arange(experts, dtype=np.int32), _SMALL_TILE_COUNTS)
    ids = np.random.default_rng(22).permutation(ids).reshape(-1, 1)
    rows = ids.shape[0]
    lay = ops.moe_align(cuda(ids), experts)
    x = synth.activations(rows, k, seed=4).to(dt)
    aq, a_s = ops.moe_scatter_quant(x, lay)
    bq, bs = synth.quantised_weights(experts * 2 * inter, k, seed=5)
    bq, bs = bq.view(experts, 2 * inter, k), bs.view(experts, 2 * inter // 128, k // 128)
    res = []
    try:
        for form, claimed in _FORMS:
            ops.set_option("grouped_rep", form)
            ops.set_option("grouped_dynamic", claimed)
            canary = torch.full((rows * inter + 4096,), 0xA5, dtype=torch.uint8, device="cuda")
            q = canary[:rows * inter].view(rows, inter)
            s = torch.full((rows, inter // 128), -1.0, dtype=torch.float32, device="cuda")
            ops.w8a8_block_fp8_gemm_grouped_tiles_swiglu(aq, a_s, bq, bs, lay, dt, q, s)
            assert ops.device_status()[0] == 0
            assert bool((canary[rows * inter:] == 0xA5).all())
            res.append((q, s))
    finally:
        ops.set_option("grouped_rep", 1)
        ops.set_option("grouped_dynamic", 1)
    for q, sc in res[1:]:
        assert torch.equal(res[0][0], q) and torch.equal(res[0][1], sc)
    q2, s2 = ops.silu_and_mul_quant(ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay, dt))
    assert torch.equal(res[0][0], q2) and torch.equal(res[0][1], s2)


def test_grouped_gemm_claimed_tiles_wait_runs_out_cleanly(ops):
    """With the producers issuing nothing (a host-set test hook) no role of the grouped kernel can
    make progress from the start: the warps that wait for a claimed tile give up after the wait
    budget, the call reports where, and the next call is right."""
    from inference_b200 import _capi, synth
    import ctypes as C
    experts, n, k = 4, 256, 256
    ids = np.repeat(np.arange(experts, dtype=np.int32), [40, 130, 7, 128]).reshape(-1, 1)
    lay = ops.moe_align(cuda(ids), experts)
    x = synth.activations(ids.shape[0], k, seed=2)
    aq, a_s = ops.moe_scatter_quant(x, lay)
    bq, bs = synth.quantised_weights(experts * n, k, seed=3)
    bq, bs = bq.view(experts, n, k), bs.view(experts, n // 128, k // 128)
    want = ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay)
    assert ops.device_status()[0] == 0
    rec = (C.c_uint32 * 4)()
    try:
        ops.set_option("wait_budget_us", 1000)
        ops.set_option("debug_no_loads", 1)
        ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay)
        rc = _capi.lib.inferop_device_status(rec, 1)                 # synchronises
        assert rc == _capi.ERR_DEVICE_WAIT, f"status {rc}, record {[hex(v) for v in rec]}"
        assert rec[0] in {0x402, 0x201, 0x202, 0x301}, hex(rec[0])
        assert _capi.lib.inferop_device_status(rec, 0) == _capi.OK   # the record was reset
    finally:
        ops.set_option("debug_no_loads", 0)
        ops.set_option("wait_budget_us", 0)
    got = ops.w8a8_block_fp8_gemm_grouped_tiles(aq, a_s, bq, bs, lay)
    assert ops.device_status()[0] == 0
    assert torch.equal(got, want)


def test_swiglu_epilogue_rejects_bad_arguments(ops):
    from inference_b200 import _capi
    t = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    f = _capi.lib.inferop_w8a8_block_fp8_gemm_grouped_tiles_swiglu
    assert f(p, p, p, p, p, p, p, p, p, 4, 4, 2, 200, 128, 128, 128, 2, None) == _capi.ERR_SHAPE    # inter % 128
    assert f(p, p, p, p, p, p, p, p, p, 4, 4, 2, 256, 128, 128, 128, 0, None) == _capi.ERR_DTYPE    # fp32 middle type
    assert f(p + 8, p, p, p, p, p, p, p, p, 4, 4, 2, 256, 128, 128, 128, 2, None) == _capi.ERR_POINTER


# ------------------------------------------------------------------------------ the whole layer
@pytest.mark.parametrize("fused", [True, False])
def test_layer_equals_the_reference_style_composition(ops, fused):
    """Six (or seven) launches with no host step against the reference's way of composing its operators:
    routing, then per expert quant -> GEMM -> SwiGLU -> quant -> GEMM on that expert's tokens, then
    the weighted sum."""
    from inference_b200 import synth
    from inference_b200.moe import MoEFP8Layer
    tokens, experts, topk, hidden, inter = 300, 8, 2, 512, 256
    x = synth.activations(tokens, hidden, seed=5)
    g = torch.Generator(device="cpu").manual_seed(9)
    logits = torch.randn((tokens, experts), generator=g).cuda()
    wgu, sgu = synth.quantised_weights(experts * 2 * inter, hidden, seed=6)
    wd, sd = synth.quantised_weights(experts * hidden, inter, seed=7)
    wgu, sgu = wgu.view(experts, 2 * inter, hidden), sgu.view(experts, 2 * inter // 128, hidden // 128)
    wd, sd = wd.view(experts, hidden, inter), sd.view(experts, hidden // 128, inter // 128)
    layer = MoEFP8Layer(wgu, sgu, wd, sd, topk, tokens, fused_swiglu=fused)
    got = layer.forward(x, logits)
    assert ops.device_status()[0] == 0

    ids, w = ops.topk_softmax(logits, topk)
    ids_h, w_h = ids.cpu().numpy(), w.cpu().numpy()
    want_ids, want_w = oracle.topk_softmax(logits.cpu().numpy(), topk)
    assert np.array_equal(ids_h, want_ids)
    xq, xs = ops.quant_fp8_per_token_group(x)
    y = {}                                            # (token, k) -> expert output row
    for e in range(experts):
        t_idx, k_idx = np.nonzero(ids_h == e)
        if len(t_idx) == 0:
            continue
        sel = torch.from_numpy(t_idx).cuda()
        gu = ops.w8a8_block_fp8_gemm(xq[sel].contiguous(), xs[sel].contiguous(), wgu[e], sgu[e])
        hq, hs = ops.quant_fp8_per_token_group(ops.silu_and_mul(gu))
        ye = ops.w8a8_block_fp8_gemm(hq, hs, wd[e], sd[e]).float().cpu().numpy()
        for j, (t, k) in enumerate(zip(t_idx, k_idx)):
            y[(t, k)] = ye[j]
    acc = np.zeros((tokens, hidden), np.float32)
    for k in range(topk):
        yk = np.stack([y[(t, k)] for t in range(tokens)])
        acc = acc + (w_h[:, k:k + 1] * yk).astype(np.float32)
    want = torch.from_numpy(acc).to(torch.bfloat16)
    assert torch.equal(got.cpu(), want)
