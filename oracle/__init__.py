"""CPU oracle for the blockwise-FP8 path.  TEST INFRASTRUCTURE ONLY.

numpy front end over ``oracle/oracle.c`` (the in-tree restatement of the
reference's CPU golden code) and, where it has been built, over
``oracle/_ref/libinferop_ref.so`` (the reference's own ``reference/reference.cpp``
compiled unmodified).  Nothing in the shipped package imports this module:
only the tests, the smoke check and the benchmark's CPU-baseline legs do, and
only as the checker or as the thing timed for the CPU baseline.

Function-by-function citations into the reference are in ``oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libinferop_ref.so")

_p = C.c_void_p
_i64 = C.c_int64
_int = C.c_int


def build(reference_root: str | None = None) -> None:
    """Compile the checker (and, when the reference tree is present, the reference's own CPU code
    and its CUDA kernels for this path: the two baselines of the benchmark)."""
    cmd = ["make", "-s", "-C", _HERE]
    if reference_root:
        cmd.append(f"REF={reference_root}")
    subprocess.run(cmd, check=True)


def _load(path):
    return C.CDLL(path) if os.path.exists(path) else None


_lib = _load(_LIB_PATH)
if _lib is None:
    build()
    _lib = C.CDLL(_LIB_PATH)
_ref = _load(_REF_PATH)


def have_reference() -> bool:
    """True when the reference's own compiled CPU code is available beside the oracle."""
    return _ref is not None


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


# ---------------------------------------------------------------- formats
def bf16_widen(h) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 (exact)."""
    h = np.ascontiguousarray(h, dtype=np.uint16)
    return (h.astype(np.uint32) << 16).view(np.float32)


def bf16_narrow(f) -> np.ndarray:
    """float32 -> uint16 bf16 bit patterns, round-to-nearest-even."""
    f = _f32(f)
    out = np.empty(f.shape, np.uint16)
    _lib.orc_bf16_narrow_array(_ptr(out), _ptr(f), _i64(f.size))
    return out


def e4m3_decode(b) -> np.ndarray:
    b = _u8(b)
    out = np.empty(b.shape, np.float32)
    _lib.orc_e4m3_decode_array(_ptr(out), _ptr(b), _i64(b.size))
    return out


def e4m3_encode(f) -> np.ndarray:
    f = _f32(f)
    out = np.empty(f.shape, np.uint8)
    _lib.orc_e4m3_encode_array(_ptr(out), _ptr(f), _i64(f.size))
    return out


# ---------------------------------------------------------------- operators
def quant_fp8_per_token_group(x, group_size: int = 128):
    """x float32 [rows, cols] -> (q uint8 [rows, cols], scales float32 [rows, cols/gs])."""
    x = _f32(x)
    rows, cols = x.shape
    q = np.zeros((rows, cols), np.uint8)
    s = np.zeros((rows, max(cols // max(group_size, 1), 0)), np.float32)
    rc = _lib.orc_quant_fp8_per_token_group(_ptr(q), _ptr(s), _ptr(x), _i64(rows), _i64(cols),
                                            _int(group_size))
    if rc != 0:
        raise ValueError("shape the reference treats as a no-op")
    return q, s


def dequant_fp8_per_token_group(q, scales, group_size: int = 128) -> np.ndarray:
    q = _u8(q)
    scales = _f32(scales)
    rows, cols = q.shape
    x = np.empty((rows, cols), np.float32)
    rc = _lib.orc_dequant_fp8_per_token_group(_ptr(x), _ptr(q), _ptr(scales), _i64(rows),
                                              _i64(cols), _int(group_size))
    if rc != 0:
        raise ValueError("bad shape")
    return x


def block_quant_weights(w, group_size: int = 128, block_n: int = 128):
    """W float32 [N, K] -> (bq uint8 [N, K], bs float32 [ceil(N/bn), K/gs])."""
    w = _f32(w)
    n, k = w.shape
    bq = np.zeros((n, k), np.uint8)
    bs = np.zeros(((n + block_n - 1) // block_n, k // group_size), np.float32)
    rc = _lib.orc_block_quant_weights(_ptr(bq), _ptr(bs), _ptr(w), _i64(n), _i64(k),
                                      _int(group_size), _int(block_n))
    if rc != 0:
        raise ValueError("bad shape")
    return bq, bs


def _gemm_call(aq, a_s, bq, bs, m, n, k, gs, bn, rows, cols):
    n_rows = m if rows is None else len(rows)
    n_cols = n if cols is None else len(cols)
    out = np.empty((n_rows, n_cols), np.float32)
    rc = _lib.orc_w8a8_block_fp8_gemm(_ptr(out), _ptr(aq), _ptr(a_s), _ptr(bq), _ptr(bs), _i64(m),
                                      _i64(n), _i64(k), _int(gs), _int(bn), _ptr(rows),
                                      _i64(n_rows), _ptr(cols), _i64(n_cols))
    if rc != 0:
        raise ValueError(f"oracle gemm rejected the call (rc={rc})")
    return out


def w8a8_block_fp8_gemm(aq, a_scales, bq, b_scales, group_size: int = 128, block_n: int = 128,
                        rows=None, cols=None, threads: int = 0) -> np.ndarray:
    """fp64-accumulated golden GEMM, narrowed to float32.

    ``rows`` / ``cols`` (int arrays) restrict the result to a sub-matrix
    ``C[rows][:, cols]``.  ``threads`` > 1 splits the rows over a thread pool
    (the C code holds no GIL), which changes nothing numerically.
    """
    aq, bq = _u8(aq), _u8(bq)
    a_s, bs = _f32(a_scales), _f32(b_scales)
    m, k = aq.shape
    n = bq.shape[0]
    assert bq.shape[1] == k
    if rows is not None:
        rows = np.ascontiguousarray(rows, dtype=np.int64)
    if cols is not None:
        cols = np.ascontiguousarray(cols, dtype=np.int64)
    sel = np.arange(m, dtype=np.int64) if rows is None else rows
    if threads <= 1 or len(sel) < 2:
        return _gemm_call(aq, a_s, bq, bs, m, n, k, group_size, block_n, rows, cols)
    parts = np.array_split(sel, min(threads, len(sel)))
    with ThreadPoolExecutor(len(parts)) as ex:
        outs = list(ex.map(lambda p: _gemm_call(aq, a_s, bq, bs, m, n, k, group_size, block_n,
                                                np.ascontiguousarray(p), cols), parts))
    return np.concatenate(outs, axis=0)


def topk_softmax(logits, topk: int, renormalize: bool = True):
    logits = _f32(logits)
    t, e = logits.shape
    ids = np.empty((t, topk), np.int32)
    w = np.empty((t, topk), np.float32)
    rc = _lib.orc_topk_softmax(_ptr(ids), _ptr(w), _ptr(logits), _i64(t), _int(e), _int(topk),
                               _int(1 if renormalize else 0))
    if rc != 0:
        raise ValueError("bad shape")
    return ids, w


def silu_and_mul(gate_up):
    """gate_up fp32 [tokens, 2d] -> fp32 [tokens, d] (reference/reference.cpp:55-63)."""
    gate_up = _f32(gate_up)
    t, d2 = gate_up.shape
    out = np.empty((t, d2 // 2), np.float32)
    if _lib.orc_silu_and_mul(_ptr(out), _ptr(gate_up), _i64(t), _i64(d2 // 2)) != 0:
        raise ValueError("bad shape")
    return out


def rmsnorm(x, weight, eps: float = 1e-6):
    """x fp32 [rows, cols], weight fp32 [cols] -> fp32 [rows, cols] (reference/reference.cpp:11-21)."""
    x, weight = _f32(x), _f32(weight)
    rows, cols = x.shape
    out = np.empty_like(x)
    if _lib.orc_rmsnorm(_ptr(out), _ptr(x), _ptr(weight), _i64(rows), _i64(cols), C.c_float(eps)) != 0:
        raise ValueError("bad shape")
    return out


def fused_add_rmsnorm(residual, x, weight, eps: float = 1e-6):
    """-> (residual + x, rmsnorm(residual + x)), both fp32 (reference/reference.cpp:23-35)."""
    res = _f32(residual).copy()
    x, weight = _f32(x), _f32(weight)
    rows, cols = x.shape
    out = np.empty_like(x)
    if _lib.orc_fused_add_rmsnorm(_ptr(res), _ptr(out), _ptr(x), _ptr(weight), _i64(rows), _i64(cols),
                                  C.c_float(eps)) != 0:
        raise ValueError("bad shape")
    return res, out


def rope_neox(qkv, positions, rotary_dim: int, base: float = 10000.0, yarn_factor: float = 1.0):
    """qkv fp32 [tokens, heads, head_dim], positions int64 [tokens] -> rotated copy
    (reference/reference.cpp:37-53)."""
    q = _f32(qkv).copy()
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    tokens, heads, head_dim = q.shape
    if _lib.orc_rope_neox(_ptr(q), _ptr(pos), _i64(tokens), _int(heads), _int(head_dim), _int(rotary_dim),
                          C.c_float(base), C.c_float(yarn_factor)) != 0:
        raise ValueError("bad shape")
    return q


def _attn_call(fn, q, k_cache, v_cache, block_tables, seq_lens, scale):
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    bt = np.ascontiguousarray(block_tables, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    batch, heads, dim = q.shape
    _, block_size, kv_heads, _ = k_cache.shape
    out = np.empty_like(q)
    rc = fn(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(bt), _ptr(sl), _int(batch), _int(heads),
            _int(kv_heads), _int(dim), _int(block_size), _int(bt.shape[1]), C.c_float(scale))
    return out, rc


def paged_attn_decode(q, k_cache, v_cache, block_tables, seq_lens, scale: float):
    """q fp32 [batch, heads, dim], caches fp32 [blocks, block_size, kv_heads, dim], block_tables int32
    [batch, max_blocks], seq_lens int32 [batch] -> fp32 [batch, heads, dim] (reference/reference.cpp:112-150)."""
    out, rc = _attn_call(_lib.orc_paged_attn_decode, q, k_cache, v_cache, block_tables, seq_lens, scale)
    if rc != 0:
        raise ValueError("bad shape")
    return out


def moe_align(topk_ids, experts: int, tile_rows: int = 128):
    """Expert-sorted layout of a routing: the checker of the device kernel that has no reference
    counterpart (the reference loops over experts on the host).  Pairs (token, k) are sorted by
    expert with a stable sort; returns counts, offsets, pos, src_token, tile_row0, tile_meta."""
    ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
    t, topk = ids.shape
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    pos = np.empty(t * topk, np.int32)
    pos[order] = np.arange(t * topk, dtype=np.int32)
    counts = np.bincount(flat, minlength=experts).astype(np.int32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    src_token = (order // topk).astype(np.int32)
    row0, meta = [], []
    for e in range(experts):
        for r in range(0, int(counts[e]), tile_rows):
            row0.append(int(offsets[e]) + r)
            meta.append((e << 8) | (min(tile_rows, int(counts[e]) - r) - 1))
    return counts, offsets, pos, src_token, np.array(row0, np.int32), np.array(meta, np.int32)


def moe_combine(y, weights, pos):
    """out[t] = sum_k w[t,k] * y[pos[t,k]] with every product and sum rounded to fp32, in the
    order of k (y fp32 [pairs, hidden], weights fp32 [tokens, topk], pos int [tokens*topk])."""
    y, weights = _f32(y), _f32(weights)
    t, topk = weights.shape
    p = np.asarray(pos).reshape(t, topk)
    acc = np.zeros((t, y.shape[1]), np.float32)
    for k in range(topk):
        acc = acc + (weights[:, k:k + 1] * y[p[:, k]]).astype(np.float32)
    return acc


# ---------------------------------------------------------------- the reference itself
class _Reference:
    """The reference's unmodified CPU functions (``oracle/_ref``), same signatures as above."""

    def __init__(self, lib):
        self.lib = lib
        lib.ref_e4m3_to_f32.restype = C.c_float
        lib.ref_e4m3_to_f32.argtypes = [C.c_uint8]
        lib.ref_f32_to_e4m3.restype = C.c_uint8
        lib.ref_f32_to_e4m3.argtypes = [C.c_float]
        lib.ref_f32_to_bf16.restype = C.c_uint16
        lib.ref_f32_to_bf16.argtypes = [C.c_float]

    def hardware_threads(self) -> int:
        return int(self.lib.ref_hardware_threads())

    def encode_mismatches_vs_oracle(self, lo: int = 0, hi: int = 1 << 32, threads: int = 0) -> int:
        """Number of fp32 bit patterns in [lo, hi) where oracle.c's encoder differs from the
        reference's.  Runs natively on all cores; the full range takes seconds."""
        fn = self.lib.ref_encode_mismatches
        fn.restype = C.c_uint64
        fn.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int]
        other = C.cast(_lib.orc_f32_to_e4m3, C.c_void_p)
        return int(fn(other, lo, hi, threads))

    def e4m3_decode(self, b):
        b = _u8(b)
        return np.array([self.lib.ref_e4m3_to_f32(int(v)) for v in b.ravel()],
                        np.float32).reshape(b.shape)

    def e4m3_encode(self, f):
        f = _f32(f)
        out = np.empty(f.shape, np.uint8)
        self.lib.ref_e4m3_encode_array(_ptr(out), _ptr(f), _i64(f.size))
        return out

    def bf16_narrow(self, f):
        f = _f32(f)
        return np.array([self.lib.ref_f32_to_bf16(float(v)) for v in f.ravel()],
                        np.uint16).reshape(f.shape)

    def quant_fp8_per_token_group(self, x, group_size=128, threads=1):
        x = _f32(x)
        rows, cols = x.shape
        q = np.zeros((rows, cols), np.uint8)
        s = np.zeros((rows, cols // group_size), np.float32)
        if threads == 1:
            self.lib.ref_quant_fp8_per_token_group(_ptr(q), _ptr(s), _ptr(x), _i64(rows),
                                                   _i64(cols), _int(group_size))
        else:
            self.lib.ref_quant_fp8_per_token_group_mt(_ptr(q), _ptr(s), _ptr(x), _i64(rows),
                                                      _i64(cols), _int(group_size), _int(threads))
        return q, s

    def dequant_fp8_per_token_group(self, q, scales, group_size=128):
        q, scales = _u8(q), _f32(scales)
        rows, cols = q.shape
        x = np.empty((rows, cols), np.float32)
        self.lib.ref_dequant_fp8_per_token_group(_ptr(x), _ptr(q), _ptr(scales), _i64(rows),
                                                 _i64(cols), _int(group_size))
        return x

    def w8a8_block_fp8_gemm(self, aq, a_scales, bq, b_scales, group_size=128, block_n=128,
                            threads=1):
        aq, bq = _u8(aq), _u8(bq)
        a_s, bs = _f32(a_scales), _f32(b_scales)
        m, k = aq.shape
        n = bq.shape[0]
        out = np.empty((m, n), np.float32)
        if threads == 1:
            self.lib.ref_w8a8_block_fp8_gemm(_ptr(out), _ptr(aq), _ptr(a_s), _ptr(bq), _ptr(bs),
                                             _i64(m), _i64(n), _i64(k), _int(group_size),
                                             _int(block_n))
        else:
            self.lib.ref_w8a8_block_fp8_gemm_mt(_ptr(out), _ptr(aq), _ptr(a_s), _ptr(bq),
                                                _ptr(bs), _i64(m), _i64(n), _i64(k),
                                                _int(group_size), _int(block_n), _int(threads))
        return out

    def rmsnorm(self, x, weight, eps=1e-6):
        x, weight = _f32(x), _f32(weight)
        out = np.empty_like(x)
        self.lib.ref_rmsnorm(_ptr(out), _ptr(x), _ptr(weight), _i64(x.shape[0]), _i64(x.shape[1]), C.c_float(eps))
        return out

    def fused_add_rmsnorm(self, residual, x, weight, eps=1e-6):
        res, x, weight = _f32(residual).copy(), _f32(x), _f32(weight)
        out = np.empty_like(x)
        self.lib.ref_fused_add_rmsnorm(_ptr(res), _ptr(out), _ptr(x), _ptr(weight), _i64(x.shape[0]),
                                       _i64(x.shape[1]), C.c_float(eps))
        return res, out

    def rope_neox(self, qkv, positions, rotary_dim, base=10000.0, yarn_factor=1.0):
        q = _f32(qkv).copy()
        pos = np.ascontiguousarray(positions, dtype=np.int64)
        t, h, d = q.shape
        self.lib.ref_rope_neox(_ptr(q), _ptr(pos), _i64(t), _int(h), _int(d), _int(rotary_dim), C.c_float(base),
                               C.c_float(yarn_factor))
        return q

    def paged_attn_decode(self, q, k_cache, v_cache, block_tables, seq_lens, scale):
        self.lib.ref_paged_attn_decode.restype = None
        return _attn_call(self.lib.ref_paged_attn_decode, q, k_cache, v_cache, block_tables, seq_lens, scale)[0]

    def silu_and_mul(self, gate_up):
        gate_up = _f32(gate_up)
        t, d2 = gate_up.shape
        out = np.empty((t, d2 // 2), np.float32)
        self.lib.ref_silu_and_mul(_ptr(out), _ptr(gate_up), _i64(t), _i64(d2 // 2))
        return out

    def topk_softmax(self, logits, topk, renormalize=True):
        logits = _f32(logits)
        t, e = logits.shape
        ids = np.empty((t, topk), np.int32)
        w = np.empty((t, topk), np.float32)
        self.lib.ref_topk_softmax(_ptr(ids), _ptr(w), _ptr(logits), _i64(t), _int(e), _int(topk),
                                  _int(1 if renormalize else 0))
        return ids, w


reference = _Reference(_ref) if _ref is not None else None
