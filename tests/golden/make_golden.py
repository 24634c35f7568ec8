"""Generates the golden vectors in this directory from the reference's own CPU code.

Run where the reference tree is available (``make -C oracle`` builds
``oracle/_ref/libinferop_ref.so`` from the reference's reference/reference.cpp,
include/inferop/fp8.h and common.h):

    python tests/golden/make_golden.py

Every output below is produced by the unmodified reference functions
(``oracle.reference``), never by the in-tree restatement, so the committed files
pin the restatement and the CUDA kernels to the reference itself.
"""
import hashlib
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
R = oracle.reference
assert R is not None, "build oracle/_ref first (make -C oracle)"


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns using the reference's converter."""
    return R.bf16_narrow(x)


def codec():
    """Known-answer inputs of the reference's codec tests (tests/test_fp8.cpp:70-106,
    scripts/check_fp8.py:113-153): every grid point, every midpoint between neighbours,
    edge magnitudes, both signs; plus all 256 decodes."""
    grid = R.e4m3_decode(np.arange(0x7F, dtype=np.uint8)).astype(np.float64)
    pts = list(grid) + [(grid[i] + grid[i + 1]) / 2 for i in range(0x7E)]
    pts += [0.0, 2.0 ** -10, 2.0 ** -10 * 1.0000001, 2.0 ** -11, 447.9, 448.0, 463.9, 464.0, 464.1, 480.0,
            511.9, 512.0, 1e-45, 1e-30, 1e38, np.inf, 0.0009765624, 0.0029296875, 0.015625, 0.013671875]
    f = np.array(pts, dtype=np.float32)
    f = np.concatenate([f, -f, np.nextafter(f, np.float32(np.inf)), np.nextafter(f, np.float32(-np.inf))])
    f = np.concatenate([f, np.array([np.nan, -np.nan], dtype=np.float32)])
    np.savez_compressed(os.path.join(HERE, "codec_golden.npz"),
                        decode_all=R.e4m3_decode(np.arange(256, dtype=np.uint8)),
                        encode_in=f, encode_out=R.e4m3_encode(f))


def quant():
    """Quantiser vectors incl. the edge cases of tests/test_quant.cpp:34-41 (zero group)
    and inputs the reference handles implicitly (NaN, Inf, denormals, one huge outlier)."""
    rng = np.random.default_rng(20260101)
    x = rng.standard_normal((24, 512)).astype(np.float32)
    x[1, :128] = 0.0                       # all-zero group
    x[2, 130] = 1e4                        # outlier dominates its group
    x[3, 5] = np.nan                       # NaN is skipped by the maximum
    x[4, 7] = -np.nan
    x[5, 9] = np.inf                       # infinite maximum
    x[6, 11] = -np.inf
    x[7, :128] = (rng.standard_normal(128) * 1e-40).astype(np.float32)  # subnormal inputs
    x[8, 128:256] *= 1e-30
    x[9, 256:384] *= 1e30
    x[10, :128] = 0.0
    x[10, 3] = -0.0
    x[11, :128] = 448.0
    x[12, :] *= 20.0
    bits = bf16_round(x)
    xb = oracle.bf16_widen(bits)
    q, s = R.quant_fp8_per_token_group(xb, 128)
    q64, s64 = R.quant_fp8_per_token_group(xb, 64)
    qf, sf = R.quant_fp8_per_token_group(x, 128)   # fp32 input
    np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), x_bf16_bits=bits, q=q, scales=s,
                        q_gs64=q64, scales_gs64=s64, x_f32=x, q_f32=qf, scales_f32=sf,
                        dequant=R.dequant_fp8_per_token_group(q, s, 128))


def gemm_small():
    """A ragged GEMM small enough to store whole (M=40, N=200, K=384)."""
    rng = np.random.default_rng(7)
    m, n, k = 40, 200, 384
    a = oracle.bf16_widen(bf16_round(rng.standard_normal((m, k)).astype(np.float32)))
    w = oracle.bf16_widen(bf16_round((0.02 * rng.standard_normal((n, k))).astype(np.float32)))
    aq, a_s = R.quant_fp8_per_token_group(a, 128)
    bq, bs = oracle.block_quant_weights(w)  # test-helper semantics (tests/test_gemm.cpp:28-45)
    c = R.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
    np.savez_compressed(os.path.join(HERE, "gemm_small_golden.npz"), aq=aq, a_scales=a_s, bq=bq,
                        b_scales=bs, c=c)


def config1():
    """The CPU-runnable golden config: M=32, N=1024, K=1024, seed 0.  Inputs come from
    numpy's PCG64 stream (seed 0); the file keeps digests of every tensor plus the first
    8 columns of C so that a regenerated input set can be recognised and checked."""
    rng = np.random.default_rng(0)
    m, n, k = 32, 1024, 1024
    a_bits = bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    w_bits = bf16_round((0.02 * rng.standard_normal((n, k))).astype(np.float32))
    aq, a_s = R.quant_fp8_per_token_group(oracle.bf16_widen(a_bits), 128)
    bq, bs = oracle.block_quant_weights(oracle.bf16_widen(w_bits))
    c = R.w8a8_block_fp8_gemm(aq, a_s, bq, bs, threads=8)
    rec = {
        "shape": [m, n, k], "seed": 0,
        "sha256": {"a_bf16_bits": sha(a_bits), "w_bf16_bits": sha(w_bits), "a_q": sha(aq),
                   "a_scales": sha(a_s), "b_q": sha(bq), "b_scales": sha(bs), "c_f32": sha(c)},
        "c_first8cols": [[float(v) for v in row] for row in c[:, :8]],
        "c_frobenius": float(np.sqrt((c.astype(np.float64) ** 2).sum())),
    }
    with open(os.path.join(HERE, "config1_golden.json"), "w") as f:
        json.dump(rec, f, indent=1)


def moe():
    """Routing and SwiGLU vectors from the reference's CPU functions (reference.cpp:152-181,
    :55-63): the reference test's shapes (257 x 256 top-8, 3 x 8 top-2, 17 x 1024 top-16) with
    N(0, 2) logits, one set with repeated logits (tie-breaking), and a SwiGLU block."""
    rng = np.random.default_rng(21)
    out = {}
    for name, (t, e, k) in {"a": (257, 256, 8), "b": (3, 8, 2), "c": (17, 1024, 16)}.items():
        lg = (2.0 * rng.standard_normal((t, e))).astype(np.float32)
        for renorm in (0, 1):
            ids, w = R.topk_softmax(lg, k, bool(renorm))
            out[f"ids_{name}{renorm}"], out[f"w_{name}{renorm}"] = ids, w
        out[f"logits_{name}"] = lg
    ties = np.round(rng.standard_normal((40, 64)) * 2).astype(np.float32)   # many equal logits
    out["logits_ties"] = ties
    out["ids_ties"], out["w_ties"] = R.topk_softmax(ties, 6, True)
    gu = (3.0 * rng.standard_normal((48, 512))).astype(np.float32)
    out["gate_up"] = gu
    out["silu"] = R.silu_and_mul(gu)
    np.savez_compressed(os.path.join(HERE, "moe_golden.npz"), **out)


def norm_rope():
    """RMSNorm, residual add + RMSNorm and the NeoX rotary embedding from the reference's CPU
    functions (reference.cpp:11-53) on cut-down shapes of its own tests (tests/test_rmsnorm.cpp:8-10,
    tests/test_rope.cpp:8-11: fewer rows and heads, the same row length, head size, rotary size and
    positions) plus long positions and a scaled base."""
    rng = np.random.default_rng(33)
    out = {}
    x = rng.standard_normal((9, 1024)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 1024).astype(np.float32)
    res = rng.standard_normal((9, 1024)).astype(np.float32)
    out["x"], out["w"], out["res"] = x, w, res
    out["rms"] = R.rmsnorm(x, w, 1e-6)
    out["fused_res"], out["fused_out"] = R.fused_add_rmsnorm(res, x, w, 1e-6)
    q = rng.standard_normal((64, 3, 128)).astype(np.float32)
    pos = np.array([t * 17 + (t % 3) for t in range(64)], np.int64)
    out["q"], out["pos"] = q, pos
    out["rope"] = R.rope_neox(q, pos, 64, 10000.0, 1.0)
    q2 = rng.standard_normal((16, 4, 64)).astype(np.float32)
    pos2 = rng.integers(0, 131072, 16).astype(np.int64)
    out["q2"], out["pos2"] = q2, pos2
    out["rope2"] = R.rope_neox(q2, pos2, 64, 500000.0, 0.25)
    np.savez_compressed(os.path.join(HERE, "norm_rope_golden.npz"), **out)


if __name__ == "__main__":
    only = sys.argv[1:]
    if only == ["norm_rope"]:
        norm_rope()
        sys.exit(0)
    norm_rope()
    moe()
    codec()
    quant()
    gemm_small()
    config1()
    print("golden vectors written to", HERE)
