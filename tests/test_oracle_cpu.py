"""CPU checks of the oracle: against the format definition, against the golden vectors
generated from the reference, and against the reference's compiled CPU code when present."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN, config1_inputs

needs_ref = pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built")


def spec_grid():
    """E4M3 values enumerated from the format definition (as tests/test_fp8.cpp:18-33 does)."""
    g = np.zeros(256, dtype=np.float64)
    for b in range(256):
        e, m = (b >> 3) & 15, b & 7
        if e == 15 and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1 + m / 8) * 2.0 ** (e - 7)
        g[b] = -v if b & 0x80 else v
    return g


def nearest_code(a: float, grid) -> int:
    """Nearest grid point, ties to the even code, saturating at 448 (tests/test_fp8.cpp:35-50)."""
    neg = np.signbit(a)
    a = abs(a)
    if a >= 448.0:
        return 0xFE if neg else 0x7E
    d = np.abs(grid[:0x7F] - a)
    best = int(np.argmin(d))
    ties = np.flatnonzero(d == d[best])
    if len(ties) > 1:
        best = int([t for t in ties if t % 2 == 0][0])
    return best | (0x80 if neg else 0)


def test_decode_all_256_against_format_definition():
    want = spec_grid()
    got = oracle.e4m3_decode(np.arange(256, dtype=np.uint8)).astype(np.float64)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan], want[~nan])
    assert np.array_equal(np.signbit(got[~nan]), np.signbit(want[~nan]))


def test_encode_against_nearest_grid_point():
    grid = spec_grid()
    rng = np.random.default_rng(3)
    mags = 10.0 ** rng.uniform(-9, 3, size=20000)
    f = (mags * rng.choice([-1.0, 1.0], size=mags.size)).astype(np.float32)
    pos = grid[:0x7F]
    mids = (pos[:-1] + pos[1:]) / 2
    f = np.concatenate([f, pos.astype(np.float32), mids.astype(np.float32),
                        -pos.astype(np.float32), -mids.astype(np.float32),
                        np.array([0.0, -0.0, 1e-45, -1e-45, 1e38, -1e38, np.inf, -np.inf, 464.0, 463.99],
                                 dtype=np.float32)])
    got = oracle.e4m3_encode(f)
    want = np.array([nearest_code(float(v), grid) for v in f], dtype=np.uint8)
    assert np.array_equal(got, want)


def test_round_trip_relative_error():
    # tests/test_fp8.cpp:108-118: |decode(encode(x)) - x| <= 2^-4 |x|; the bound holds on the
    # normal range [2^-6, 448) (the reference samples [0.01, 400], whose first 0.0056 is denormal)
    x = np.random.default_rng(5).uniform(2.0 ** -6, 400, 20000).astype(np.float32)
    back = oracle.e4m3_decode(oracle.e4m3_encode(x))
    assert np.all(np.abs(back - x) <= x / 16)


def test_codec_golden():
    g = np.load(os.path.join(GOLDEN, "codec_golden.npz"))
    assert np.array_equal(oracle.e4m3_decode(np.arange(256, dtype=np.uint8)).view(np.uint32),
                          g["decode_all"].view(np.uint32))
    assert np.array_equal(oracle.e4m3_encode(g["encode_in"]), g["encode_out"])


def test_bf16_round_to_nearest_even():
    f = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.3895314e38, 1e-40, 0.0, -0.0], np.float32)
    # 1 + 2^-8 is a tie -> even (1.0); 1 + 3*2^-8 is a tie -> even (1 + 2^-6)
    bits = oracle.bf16_narrow(f)
    assert bits[0] == 0x3F80 and bits[1] == 0x3F80 and bits[2] == 0x3F82 and bits[3] == 0xBF80
    assert np.array_equal(oracle.bf16_widen(bits)[[0, 6]], np.array([1.0, 0.0], np.float32))


def test_quant_golden_bf16_fp32_and_gs64():
    g = np.load(os.path.join(GOLDEN, "quant_golden.npz"))
    x = oracle.bf16_widen(g["x_bf16_bits"])
    q, s = oracle.quant_fp8_per_token_group(x, 128)
    assert np.array_equal(q, g["q"]) and np.array_equal(s.view(np.uint32), g["scales"].view(np.uint32))
    q, s = oracle.quant_fp8_per_token_group(x, 64)
    assert np.array_equal(q, g["q_gs64"]) and np.array_equal(s.view(np.uint32), g["scales_gs64"].view(np.uint32))
    q, s = oracle.quant_fp8_per_token_group(g["x_f32"], 128)
    assert np.array_equal(q, g["q_f32"]) and np.array_equal(s.view(np.uint32), g["scales_f32"].view(np.uint32))
    d = oracle.dequant_fp8_per_token_group(g["q"], g["scales"], 128)
    assert np.array_equal(d.view(np.uint32), g["dequant"].view(np.uint32))


def test_quant_zero_group_and_error_bound():
    # tests/test_quant.cpp:15-42
    x = np.random.default_rng(1).standard_normal((64, 768)).astype(np.float32)
    q, s = oracle.quant_fp8_per_token_group(x, 128)
    dq = oracle.dequant_fp8_per_token_group(q, s, 128)
    tol = np.maximum(np.abs(x) / 16, np.repeat(s, 128, axis=1) * 1.5e-3) + 1e-30
    assert np.all(np.abs(dq - x) <= tol)
    q, s = oracle.quant_fp8_per_token_group(np.zeros((1, 768), np.float32), 128)
    assert np.all(s == 1.0) and not q.any()


def test_quant_rejects_what_the_reference_ignores():
    with pytest.raises(ValueError):
        oracle.quant_fp8_per_token_group(np.zeros((2, 100), np.float32), 128)


def test_gemm_small_golden():
    g = np.load(os.path.join(GOLDEN, "gemm_small_golden.npz"))
    c = oracle.w8a8_block_fp8_gemm(g["aq"], g["a_scales"], g["bq"], g["b_scales"])
    assert np.array_equal(c.view(np.uint32), g["c"].view(np.uint32))
    sub = oracle.w8a8_block_fp8_gemm(g["aq"], g["a_scales"], g["bq"], g["b_scales"], rows=[0, 39],
                                     cols=[0, 127, 128, 199])
    assert np.array_equal(sub, g["c"][[0, 39]][:, [0, 127, 128, 199]])


def test_config1_golden_digests():
    with open(os.path.join(GOLDEN, "config1_golden.json")) as f:
        rec = json.load(f)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    a_bits, w_bits = config1_inputs()
    if sha(a_bits) != rec["sha256"]["a_bf16_bits"] or sha(w_bits) != rec["sha256"]["w_bf16_bits"]:
        pytest.skip("numpy's generator stream differs from the one the fixture was made with")
    aq, a_s = oracle.quant_fp8_per_token_group(oracle.bf16_widen(a_bits), 128)
    bq, bs = oracle.block_quant_weights(oracle.bf16_widen(w_bits))
    assert sha(aq) == rec["sha256"]["a_q"] and sha(a_s) == rec["sha256"]["a_scales"]
    assert sha(bq) == rec["sha256"]["b_q"] and sha(bs) == rec["sha256"]["b_scales"]
    c = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=4)
    assert sha(c) == rec["sha256"]["c_f32"]
    assert np.array_equal(c[:, :8], np.array(rec["c_first8cols"], dtype=np.float32))


def test_gemm_plausible_magnitude():
    # tests/test_gemm.cpp:52-60: N(0,1) x N(0,1) at 128^3 -> 1 < max|C| < 1e3
    rng = np.random.default_rng(11)
    a = rng.standard_normal((128, 128)).astype(np.float32)
    b = rng.standard_normal((128, 128)).astype(np.float32)
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(b)
    c = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    assert 1.0 < np.abs(c).max() < 1e3
    # and it is the dequantised product up to fp32 rounding
    ref = oracle.dequant_fp8_per_token_group(aq, a_s).astype(np.float64) @ \
        (oracle.e4m3_decode(bq).astype(np.float64) * bs[0, 0]).T
    assert np.allclose(c, ref, rtol=1e-5, atol=1e-4)


def test_topk_softmax_properties():
    lg = np.random.default_rng(2).standard_normal((100, 256)).astype(np.float32)
    ids, w = oracle.topk_softmax(lg, 8, True)
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-5)
    assert np.array_equal(ids[:, 0], lg.argmax(axis=1))
    assert all(len(set(r)) == 8 for r in ids)


def test_moe_golden_routing_and_swiglu():
    g = np.load(os.path.join(GOLDEN, "moe_golden.npz"))
    for name, k in (("a", 8), ("b", 2), ("c", 16)):
        for renorm in (0, 1):
            ids, w = oracle.topk_softmax(g[f"logits_{name}"], k, bool(renorm))
            assert np.array_equal(ids, g[f"ids_{name}{renorm}"])
            assert np.array_equal(w.view(np.uint32), g[f"w_{name}{renorm}"].view(np.uint32))
    ids, w = oracle.topk_softmax(g["logits_ties"], 6, True)
    assert np.array_equal(ids, g["ids_ties"]) and np.array_equal(w.view(np.uint32), g["w_ties"].view(np.uint32))
    assert np.array_equal(oracle.silu_and_mul(g["gate_up"]).view(np.uint32), g["silu"].view(np.uint32))


def test_moe_align_and_combine_restatements():
    rng = np.random.default_rng(3)
    ids, w = oracle.topk_softmax(rng.standard_normal((300, 16)).astype(np.float32), 4)
    counts, offsets, pos, src, row0, meta = oracle.moe_align(ids, 16)
    assert counts.sum() == 1200 and offsets[-1] == 1200 and sorted(pos.tolist()) == list(range(1200))
    flat = ids.reshape(-1)
    for e in range(16):          # every expert's rows: its pairs, in pair order
        rows = pos[flat == e]
        assert np.array_equal(rows, np.arange(offsets[e], offsets[e + 1]))
    assert np.array_equal(src[pos], np.arange(1200) // 4)
    assert sum((m & 0xFF) + 1 for m in meta) == 1200 and all((m >> 8) == flat[np.nonzero(pos == r)[0][0]]
                                                             for r, m in zip(row0, meta))
    y = rng.standard_normal((1200, 8)).astype(np.float32)
    out = oracle.moe_combine(y, w, pos)
    ref = np.einsum("tk,tkh->th", w.astype(np.float64), y[pos.reshape(300, 4)].astype(np.float64))
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------ against the reference itself
@needs_ref
def test_encoder_identical_to_reference_on_all_2_32_inputs():
    assert oracle.reference.encode_mismatches_vs_oracle() == 0


@needs_ref
def test_operators_identical_to_reference():
    R = oracle.reference
    rng = np.random.default_rng(9)
    x = oracle.bf16_widen(oracle.bf16_narrow((rng.standard_normal((96, 1024)) * rng.choice([1, 20], (1, 1024))).astype(np.float32)))
    q0, s0 = oracle.quant_fp8_per_token_group(x)
    q1, s1 = R.quant_fp8_per_token_group(x)
    assert np.array_equal(q0, q1) and np.array_equal(s0.view(np.uint32), s1.view(np.uint32))
    w = (0.02 * rng.standard_normal((200, 1024))).astype(np.float32)
    bq, bs = oracle.block_quant_weights(w)
    c0 = oracle.w8a8_block_fp8_gemm(q0, s0, bq, bs, threads=4)
    c1 = R.w8a8_block_fp8_gemm(q0, s0, bq, bs, threads=4)
    assert np.array_equal(c0.view(np.uint32), c1.view(np.uint32))
    d0 = oracle.dequant_fp8_per_token_group(q0, s0)
    d1 = R.dequant_fp8_per_token_group(q0, s0)
    assert np.array_equal(d0.view(np.uint32), d1.view(np.uint32))
    lg = rng.standard_normal((64, 256)).astype(np.float32)
    i0, w0 = oracle.topk_softmax(lg, 8)
    i1, w1 = R.topk_softmax(lg, 8)
    assert np.array_equal(i0, i1) and np.array_equal(w0.view(np.uint32), w1.view(np.uint32))
    assert np.array_equal(oracle.bf16_narrow(x[:4, :64] * 1.001), R.bf16_narrow(x[:4, :64] * 1.001))
    gu = (3 * rng.standard_normal((40, 256))).astype(np.float32)
    assert np.array_equal(oracle.silu_and_mul(gu).view(np.uint32), R.silu_and_mul(gu).view(np.uint32))


def test_sampled_checker_equals_the_full_oracle_on_the_sampled_entries():
    """oracle/sampled.py gathers the sampled operand rows and calls the oracle with one scale row
    per sampled column (block_n = 1): the same numbers as indexing the full golden result."""
    import torch
    from oracle import sampled
    rng = np.random.default_rng(3)
    m, n, k = 40, 700, 512
    a = oracle.bf16_widen(oracle.bf16_narrow(rng.standard_normal((m, k)).astype(np.float32)))
    w = oracle.bf16_widen(oracle.bf16_narrow((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = oracle.quant_fp8_per_token_group(a)
    bq, bs = oracle.block_quant_weights(w)
    full = oracle.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    rows = sampled.band_rows(m, 6, seed=1, band=16)
    cols = sampled.stratified(n, 37, seed=2)
    assert rows[0] == 0 and rows[-1] == m - 1 and len(np.unique(cols)) == len(cols) and cols.max() < n
    t = torch.from_numpy
    row, fro = sampled.gemm_sample(t(aq), t(a_s), t(bq), t(bs), t(full), rows, cols, threads=2)
    assert row == 0.0 and fro == 0.0
    noisy = full.copy()
    noisy[rows[1], cols[3]] *= 1.5
    assert sampled.gemm_sample(t(aq), t(a_s), t(bq), t(bs), t(noisy), rows, cols)[0] > 0
    x16 = t(oracle.bf16_narrow(a).view(np.int16)).view(torch.bfloat16)
    assert sampled.quant_rows_exact(x16, t(aq), t(a_s), rows)
    bad = aq.copy()
    bad[rows[2], 7] ^= 1
    assert not sampled.quant_rows_exact(x16, t(bad), t(a_s), rows)


# ------------------------------------------------------------------ rmsnorm / rope (the "next" operators)
def _norm_case(rows=33, cols=1024, seed=0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((rows, cols)).astype(np.float32),
            rng.uniform(0.5, 1.5, cols).astype(np.float32))


def test_rmsnorm_properties_of_the_reference_test():
    """tests/test_rmsnorm.cpp:12-43: unit weights give RMS 1; the fused form adds in place."""
    x, w = _norm_case()
    y1 = oracle.rmsnorm(x, np.ones_like(w))
    assert abs(np.sqrt(np.mean(y1.astype(np.float64) ** 2)) - 1.0) < 1e-3
    res, xr = _norm_case(seed=1)[0], _norm_case(seed=2)[0]
    new_res, out = oracle.fused_add_rmsnorm(res, xr, w)
    assert np.array_equal(new_res, res + xr)
    assert np.array_equal(out, oracle.rmsnorm(new_res, w))


def test_rope_properties_of_the_reference_test():
    """tests/test_rope.cpp:14-52: pair norms preserved, position 0 is the identity, the tail beyond
    rotary_dim is untouched."""
    rng = np.random.default_rng(3)
    tokens, heads, dim, rot = 64, 32, 128, 64
    q = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    pos = np.array([t * 17 + (t % 3) for t in range(tokens)], np.int64)
    r = oracle.rope_neox(q, pos, rot)
    half = rot // 2
    n0 = np.hypot(q[..., :half].astype(np.float64), q[..., half:rot])
    n1 = np.hypot(r[..., :half].astype(np.float64), r[..., half:rot])
    assert np.abs(n0 - n1).max() < 1e-4
    assert np.array_equal(r[..., rot:], q[..., rot:])
    ident = oracle.rope_neox(q, np.zeros(tokens, np.int64), rot)
    np.testing.assert_allclose(ident, q, rtol=1e-6, atol=1e-6)


@pytest.mark.skipif(not oracle.have_reference(), reason="reference tree not built here")
def test_rmsnorm_and_rope_restatements_equal_the_reference_bit_for_bit():
    R = oracle.reference
    for rows, cols, seed in ((33, 1024, 0), (1, 7168, 1), (7, 130, 2), (4, 1, 3)):
        x, w = _norm_case(rows, cols, seed)
        for eps in (1e-6, 1e-5):
            assert np.array_equal(oracle.rmsnorm(x, w, eps).view(np.uint32), R.rmsnorm(x, w, eps).view(np.uint32))
            res = _norm_case(rows, cols, seed + 10)[0]
            a, b = oracle.fused_add_rmsnorm(res, x, w, eps), R.fused_add_rmsnorm(res, x, w, eps)
            assert np.array_equal(a[0].view(np.uint32), b[0].view(np.uint32))
            assert np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))
    rng = np.random.default_rng(5)
    for tokens, heads, dim, rot, base, yarn in ((64, 32, 128, 64, 10000.0, 1.0), (5, 3, 64, 64, 500000.0, 0.25),
                                                (9, 1, 256, 2, 10000.0, 1.0), (3, 8, 96, 48, 10000.0, 1.0)):
        q = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
        pos = rng.integers(0, 131072, tokens).astype(np.int64)
        pos[0] = 0
        assert np.array_equal(oracle.rope_neox(q, pos, rot, base, yarn).view(np.uint32),
                              R.rope_neox(q, pos, rot, base, yarn).view(np.uint32))


def test_rmsnorm_and_rope_golden_vectors():
    """Vectors written by the reference's own CPU functions (tests/golden/make_golden.py: norm_rope)."""
    g = np.load(os.path.join(GOLDEN, "norm_rope_golden.npz"))
    assert np.array_equal(oracle.rmsnorm(g["x"], g["w"]).view(np.uint32), g["rms"].view(np.uint32))
    res, out = oracle.fused_add_rmsnorm(g["res"], g["x"], g["w"])
    assert np.array_equal(res.view(np.uint32), g["fused_res"].view(np.uint32))
    assert np.array_equal(out.view(np.uint32), g["fused_out"].view(np.uint32))
    assert np.array_equal(oracle.rope_neox(g["q"], g["pos"], 64).view(np.uint32), g["rope"].view(np.uint32))
    assert np.array_equal(oracle.rope_neox(g["q2"], g["pos2"], 64, 500000.0, 0.25).view(np.uint32),
                          g["rope2"].view(np.uint32))


# ------------------------------------------------------------------ paged attention decode
def attn_case(batch, heads, kv_heads, dim, block_size, lens, seed=0, shuffle=False):
    """The paged cache of the reference's test (tests/test_paged_attn.cpp:16-40): a shared first block,
    then disjoint blocks per sequence; `shuffle` permutes the physical blocks."""
    rng = np.random.default_rng(seed)
    per_seq = max((l + block_size - 1) // block_size for l in lens)
    blocks = 1 + batch * per_seq
    k = rng.standard_normal((blocks, block_size, kv_heads, dim)).astype(np.float32)
    v = rng.standard_normal((blocks, block_size, kv_heads, dim)).astype(np.float32)
    q = rng.standard_normal((batch, heads, dim)).astype(np.float32)
    tables = np.zeros((batch, per_seq), np.int32)
    for b in range(batch):
        for j in range(1, per_seq):
            tables[b, j] = 1 + b * per_seq + (j - 1)
    if shuffle:
        perm = rng.permutation(blocks).astype(np.int32)
        inv = np.argsort(perm)
        k, v = k[inv], v[inv]          # logical block i now lives at physical block perm[i]
        tables = perm[tables]
    return q, k, v, tables, np.array(lens, np.int32)


def test_paged_attention_properties_of_the_reference_test():
    """tests/test_paged_attn.cpp:42-76: outputs inside the range of V, a length-1 sequence returns its V row."""
    q, k, v, tables, lens = attn_case(3, 32, 8, 128, 16, [1, 17, 129])
    out = oracle.paged_attn_decode(q, k, v, tables, lens, 1.0 / np.sqrt(128.0))
    assert out.min() >= v.min() - 1e-3 and out.max() <= v.max() + 1e-3
    np.testing.assert_allclose(out[0, 0], v[tables[0, 0], 0, 0], atol=1e-4)
    empty = oracle.paged_attn_decode(q, k, v, tables, np.array([0, 17, 129], np.int32), 0.1)
    assert np.array_equal(empty[0], np.zeros_like(empty[0]))


@pytest.mark.skipif(not oracle.have_reference(), reason="reference tree not built here")
def test_paged_attention_restatement_equals_the_reference_bit_for_bit():
    R = oracle.reference
    for (b, h, kvh, d, bs, lens, shuf) in ((3, 32, 8, 128, 16, [1, 17, 129], False), (2, 16, 4, 64, 16, [5, 64], True),
                                           (2, 8, 8, 256, 16, [33, 200], True), (1, 4, 1, 128, 8, [77], True)):
        q, k, v, tables, sl = attn_case(b, h, kvh, d, bs, lens, seed=b + d, shuffle=shuf)
        scale = float(1.0 / np.sqrt(d))
        assert np.array_equal(oracle.paged_attn_decode(q, k, v, tables, sl, scale).view(np.uint32),
                              R.paged_attn_decode(q, k, v, tables, sl, scale).view(np.uint32))
