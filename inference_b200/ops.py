"""Host-side mirror of the reference's operator interface for the blockwise-FP8 path.

Same operator names, argument meaning and contracts as the reference's
``include/inferop/ops.h`` (:64-70 quant / dequant, :81-84 GEMM), over torch
CUDA tensors instead of raw pointers.  torch is used for device memory and
streams only; all arithmetic happens in libinferop_b200.so, reached through its
C ABI.  Unlike the reference's ``void`` functions these raise ``InferopError``
on a rejected call instead of doing nothing.
"""
from __future__ import annotations

import ctypes as C
import enum

import torch

from . import _capi
from ._capi import InferopError, check, lib


class dtype(enum.IntEnum):
    """Element type codes of the C ABI (reference include/inferop/common.h:13)."""
    fp32 = 0
    fp16 = 1
    bf16 = 2
    fp8_e4m3 = 3


_TORCH2CODE = {torch.float32: dtype.fp32, torch.float16: dtype.fp16, torch.bfloat16: dtype.bf16}
_CODE2TORCH = {v: k for k, v in _TORCH2CODE.items()}


def _stream_ptr(stream=None) -> int:
    s = torch.cuda.current_stream() if stream is None else stream
    return int(s.cuda_stream)


def _dev_tensor(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _check_quantised(a_q, a_scales, b_q, b_scales, grouped: bool = False) -> None:
    """Types and exact shapes of a quantised operand set: a mis-shaped scale tensor would make a
    kernel read out of bounds on the device, so it is rejected here."""
    if a_q.dtype != torch.uint8 or b_q.dtype != torch.uint8:
        raise ValueError("a_q and b_q must be uint8 (E4M3 bytes)")
    if a_scales.dtype != torch.float32 or b_scales.dtype != torch.float32:
        raise ValueError("a_scales and b_scales must be fp32")
    if a_q.dim() != 2 or b_q.dim() != (3 if grouped else 2):
        raise ValueError("a_q must be [M, K] and b_q [N, K]" + (" per group: [G, N, K]" if grouped else ""))
    m, k = a_q.shape
    n = b_q.shape[-2]
    if b_q.shape[-1] != k:
        raise ValueError("a_q and b_q disagree on K")
    if k % 128 != 0:
        raise InferopError(_capi.ERR_SHAPE, "K must be a multiple of 128")
    if tuple(a_scales.shape) != (m, k // 128):
        raise ValueError(f"a_scales must be [M, K/128] = [{m}, {k // 128}], got {tuple(a_scales.shape)}")
    want = ((b_q.shape[0],) if grouped else ()) + ((n + 127) // 128, k // 128)
    if tuple(b_scales.shape) != want:
        raise ValueError(f"b_scales must be {list(want)}, got {list(b_scales.shape)}")


def has_cuda() -> bool:
    return bool(lib.inferop_has_cuda())


def device_count() -> int:
    return int(lib.inferop_device_count())


def device_name(ordinal: int = 0) -> str:
    return lib.inferop_device_name(ordinal).decode()


def device_sm_version(ordinal: int = 0) -> int:
    return int(lib.inferop_device_sm_version(ordinal))


def quant_fp8_per_token_group(x: torch.Tensor, group_size: int = 128, q: torch.Tensor | None = None,
                              scales: torch.Tensor | None = None, stream=None):
    """x [rows, cols] (fp32/fp16/bf16) -> (q uint8 [rows, cols], scales fp32 [rows, cols/gs])."""
    _dev_tensor(x, "x")
    if x.dim() != 2 or x.dtype not in _TORCH2CODE:
        raise ValueError("x must be a 2-D fp32/fp16/bf16 tensor")
    rows, cols = x.shape
    if group_size <= 0 or cols % group_size != 0 or rows == 0:
        raise InferopError(_capi.ERR_SHAPE, "quant_fp8_per_token_group")
    with torch.cuda.device(x.device):
        if q is None:
            q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
        if scales is None:
            scales = torch.empty((rows, cols // group_size), dtype=torch.float32, device=x.device)
        check(lib.inferop_quant_fp8_per_token_group(q.data_ptr(), scales.data_ptr(), x.data_ptr(),
                                                    int(_TORCH2CODE[x.dtype]), rows, cols, group_size,
                                                    _stream_ptr(stream)),
              "quant_fp8_per_token_group")
    return q, scales


def dequant_fp8_per_token_group(q: torch.Tensor, scales: torch.Tensor, out_dtype=torch.bfloat16,
                                group_size: int = 128, stream=None) -> torch.Tensor:
    _dev_tensor(q, "q")
    _dev_tensor(scales, "scales")
    if q.dim() != 2 or q.dtype != torch.uint8 or scales.dtype != torch.float32:
        raise ValueError("q must be a 2-D uint8 tensor and scales fp32")
    rows, cols = q.shape
    if group_size <= 0 or cols % group_size != 0 or tuple(scales.shape) != (rows, cols // group_size):
        raise ValueError("scales must be [rows, cols / group_size]")
    with torch.cuda.device(q.device):
        x = torch.empty((rows, cols), dtype=out_dtype, device=q.device)
        check(lib.inferop_dequant_fp8_per_token_group(x.data_ptr(), int(_TORCH2CODE[out_dtype]),
                                                      q.data_ptr(), scales.data_ptr(), rows, cols,
                                                      group_size, _stream_ptr(stream)),
              "dequant_fp8_per_token_group")
    return x


def w8a8_block_fp8_gemm(a_q: torch.Tensor, a_scales: torch.Tensor, b_q: torch.Tensor,
                        b_scales: torch.Tensor, out_dtype=torch.bfloat16, group_size: int = 128,
                        block_n: int = 128, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """C[M,N] = (A_q * sa) @ (B_q * sb)^T with fp32 accumulation.

    a_q [M,K] uint8 (E4M3), a_scales [M,K/128] fp32, b_q [N,K] uint8,
    b_scales [ceil(N/128), K/128] fp32.
    """
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    _check_quantised(a_q, a_scales, b_q, b_scales)
    m, k = a_q.shape
    n = b_q.shape[0]
    with torch.cuda.device(a_q.device):
        if out is None:
            out = torch.empty((m, n), dtype=out_dtype, device=a_q.device)
        elif tuple(out.shape) != (m, n) or not out.is_contiguous():
            raise ValueError("out must be a contiguous [M, N] tensor")
        check(lib.inferop_w8a8_block_fp8_gemm(out.data_ptr(), a_q.data_ptr(), a_scales.data_ptr(),
                                              b_q.data_ptr(), b_scales.data_ptr(), m, n, k, group_size,
                                              block_n, int(_TORCH2CODE[out.dtype]), _stream_ptr(stream)),
              "w8a8_block_fp8_gemm")
    return out


def w8a8_block_fp8_gemm_fused_quant(a: torch.Tensor, b_q: torch.Tensor, b_scales: torch.Tensor,
                                    out_dtype=torch.bfloat16, out: torch.Tensor | None = None,
                                    stream=None) -> torch.Tensor:
    """quant_fp8_per_token_group(a) followed by w8a8_block_fp8_gemm as one call (a in bf16 /
    fp16): one launch with the quantisation as the GEMM's A-operand prologue for M <= 32; for
    larger M the quantiser and the GEMM are chained by programmatic dependent launch through
    library-owned scratch.  Bit-identical to the two separate calls."""
    for t, name in ((a, "a"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    if a.dtype not in (torch.float16, torch.bfloat16) or a.dim() != 2:
        raise ValueError("a must be a 2-D fp16 or bf16 tensor")
    m, k = a.shape
    n = b_q.shape[0]
    if b_q.dtype != torch.uint8 or b_q.dim() != 2 or b_q.shape[1] != k or b_scales.dtype != torch.float32 or \
            k % 128 != 0 or tuple(b_scales.shape) != ((n + 127) // 128, k // 128):
        raise ValueError("b_q must be uint8 [N, K] and b_scales fp32 [ceil(N/128), K/128]")
    with torch.cuda.device(a.device):
        if out is None:
            out = torch.empty((m, n), dtype=out_dtype, device=a.device)
        check(lib.inferop_w8a8_block_fp8_gemm_fused_quant(out.data_ptr(), a.data_ptr(), int(_TORCH2CODE[a.dtype]),
                                                          b_q.data_ptr(), b_scales.data_ptr(), m, n, k, 128,
                                                          128, int(_TORCH2CODE[out.dtype]), _stream_ptr(stream)),
              "w8a8_block_fp8_gemm_fused_quant")
    return out


def w8a8_block_fp8_gemm_grouped(a_q: torch.Tensor, a_scales: torch.Tensor, b_q: torch.Tensor,
                                b_scales: torch.Tensor, m_per_group, out_dtype=torch.bfloat16,
                                out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """All groups' (MoE experts') GEMMs in one launch; same result as one call per group.

    a_q [sum(m_g), K], a_scales [sum(m_g), K/128]: the groups' rows stacked in group order;
    b_q [G, N, K], b_scales [G, N/128, K/128]; m_per_group: host sequence of G row counts.
    """
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    _check_quantised(a_q, a_scales, b_q, b_scales, grouped=True)
    groups, n, k = b_q.shape
    counts = (C.c_int64 * groups)(*[int(v) for v in m_per_group])
    m_total = int(sum(counts))
    if a_q.shape != (m_total, k):
        raise ValueError("a_q does not hold sum(m_per_group) rows of K bytes")
    with torch.cuda.device(a_q.device):
        if out is None:
            out = torch.empty((m_total, n), dtype=out_dtype, device=a_q.device)
        check(lib.inferop_w8a8_block_fp8_gemm_grouped(out.data_ptr(), a_q.data_ptr(), a_scales.data_ptr(),
                                                      b_q.data_ptr(), b_scales.data_ptr(), counts, groups,
                                                      n, k, 128, 128, int(_TORCH2CODE[out.dtype]),
                                                      _stream_ptr(stream)),
              "w8a8_block_fp8_gemm_grouped")
    return out


def w8a8_block_fp8_gemm_allgather(peer_ptrs, rank: int, a_q: torch.Tensor, a_scales: torch.Tensor,
                                  b_q: torch.Tensor, b_scales: torch.Tensor, out_dtype=torch.bfloat16,
                                  stream=None) -> None:
    """GEMM of this rank's column shard whose epilogue writes the result into every rank's buffer.

    peer_ptrs: one device address per rank (entry `rank` = the local buffer), each the base of
    that rank's row-major [M, N_shard * ranks] result in `out_dtype`; this call fills columns
    [rank * N_shard, (rank + 1) * N_shard) of all of them.  The ranks must meet after the call
    (``shard.PeerOutput.barrier``) before any of them reads its buffer.
    """
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    _check_quantised(a_q, a_scales, b_q, b_scales)
    m, k = a_q.shape
    n = b_q.shape[0]
    ptrs = (C.c_void_p * len(peer_ptrs))(*[int(p) for p in peer_ptrs])
    with torch.cuda.device(a_q.device):
        check(lib.inferop_w8a8_block_fp8_gemm_allgather(ptrs, len(peer_ptrs), int(rank), a_q.data_ptr(),
                                                        a_scales.data_ptr(), b_q.data_ptr(),
                                                        b_scales.data_ptr(), m, n, k, 128, 128,
                                                        int(_TORCH2CODE[out_dtype]), _stream_ptr(stream)),
              "w8a8_block_fp8_gemm_allgather")


def w8a8_block_fp8_gemm_scatter(slot_ptrs, rank: int, a_q: torch.Tensor, a_scales: torch.Tensor,
                                b_q: torch.Tensor, b_scales: torch.Tensor, stream=None) -> None:
    """GEMM of this rank's K shard; the fp32 partial result goes, tile by tile, into slot `rank`
    of the rank that owns the rows (slot_ptrs[d] = base of rank d's [G][M/G][N] fp32 slots)."""
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    _check_quantised(a_q, a_scales, b_q, b_scales)
    m, k = a_q.shape
    n = b_q.shape[0]
    ptrs = (C.c_void_p * len(slot_ptrs))(*[int(p) for p in slot_ptrs])
    with torch.cuda.device(a_q.device):
        check(lib.inferop_w8a8_block_fp8_gemm_scatter(ptrs, len(slot_ptrs), int(rank), a_q.data_ptr(),
                                                      a_scales.data_ptr(), b_q.data_ptr(), b_scales.data_ptr(),
                                                      m, n, k, 128, 128, _stream_ptr(stream)),
              "w8a8_block_fp8_gemm_scatter")


def w8a8_block_fp8_gemm_into(out: torch.Tensor, col0: int, a_q: torch.Tensor, a_scales: torch.Tensor,
                             b_q: torch.Tensor, b_scales: torch.Tensor, stream=None) -> torch.Tensor:
    """The GEMM with its [M, N] result written to columns [col0, col0 + N) of the wider row-major
    tensor `out` [M, ldc] (fp16 / bf16, rows contiguous)."""
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    if not out.is_cuda or out.dim() != 2 or out.stride(1) != 1:
        raise ValueError("out must be a 2-D CUDA tensor with contiguous rows")
    _check_quantised(a_q, a_scales, b_q, b_scales)
    m, k = a_q.shape
    n = b_q.shape[0]
    if out.shape[0] != m:
        raise ValueError("out does not have M rows")
    with torch.cuda.device(a_q.device):
        check(lib.inferop_w8a8_block_fp8_gemm_into(out.data_ptr(), out.stride(0), int(col0), a_q.data_ptr(),
                                                   a_scales.data_ptr(), b_q.data_ptr(), b_scales.data_ptr(), m, n, k,
                                                   128, 128, int(_TORCH2CODE[out.dtype]), _stream_ptr(stream)),
              "w8a8_block_fp8_gemm_into")
    return out


def copy_2d_async(dst_ptr: int, dst_pitch_bytes: int, src_ptr: int, src_pitch_bytes: int, width_bytes: int, rows: int,
                  device, stream=None) -> None:
    """`rows` rows of width_bytes from the device address src_ptr (row pitch src_pitch_bytes) to
    dst_ptr (row pitch dst_pitch_bytes), by the copy engines, on `stream`.  Either address may
    be peer-mapped."""
    with torch.cuda.device(device):
        check(lib.inferop_copy_2d_async(int(dst_ptr), int(dst_pitch_bytes), int(src_ptr), int(src_pitch_bytes),
                                        int(width_bytes), int(rows), _stream_ptr(stream)), "copy_2d_async")


def reduce_slots(slots: torch.Tensor, out_dtype=torch.bfloat16, out: torch.Tensor | None = None,
                 stream=None) -> torch.Tensor:
    """slots fp32 [G, rows, N] -> out [rows, N]: the sum over G in order, rounded once."""
    _dev_tensor(slots, "slots")
    g, rows, n = slots.shape
    with torch.cuda.device(slots.device):
        if out is None:
            out = torch.empty((rows, n), dtype=out_dtype, device=slots.device)
        check(lib.inferop_reduce_slots(out.data_ptr(), int(_TORCH2CODE[out.dtype]), slots.data_ptr(), g, rows, n,
                                       _stream_ptr(stream)), "reduce_slots")
    return out


# --------------------------------------------------------------------------- mixture of experts
def topk_softmax(logits: torch.Tensor, topk: int, renormalize: bool = True, ids: torch.Tensor | None = None,
                 weights: torch.Tensor | None = None, stream=None):
    """Routing: softmax over logits [tokens, experts] (fp32) + top-k -> (ids int32, weights fp32),
    both [tokens, topk] (reference include/inferop/ops.h:108-110)."""
    _dev_tensor(logits, "logits")
    if logits.dtype != torch.float32:
        raise ValueError("logits must be fp32")
    tokens, experts = logits.shape
    with torch.cuda.device(logits.device):
        if ids is None:
            ids = torch.empty((tokens, topk), dtype=torch.int32, device=logits.device)
        if weights is None:
            weights = torch.empty((tokens, topk), dtype=torch.float32, device=logits.device)
        check(lib.inferop_topk_softmax(ids.data_ptr(), weights.data_ptr(), logits.data_ptr(), tokens, experts,
                                       topk, 1 if renormalize else 0, _stream_ptr(stream)), "topk_softmax")
    return ids, weights


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None,
            stream=None) -> torch.Tensor:
    """out[r, c] = weight[c] * x[r, c] / sqrt(mean(x[r, :]^2) + eps); x [rows, cols], weight [cols], one dtype."""
    _dev_tensor(x, "x")
    _dev_tensor(weight, "weight")
    if x.dim() != 2 or x.dtype not in _TORCH2CODE or weight.dtype != x.dtype or tuple(weight.shape) != (x.shape[1],):
        raise ValueError("x must be [rows, cols] and weight [cols] of the same fp32/fp16/bf16 dtype")
    rows, cols = x.shape
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty_like(x)
        check(lib.inferop_rmsnorm(out.data_ptr(), x.data_ptr(), weight.data_ptr(), int(_TORCH2CODE[x.dtype]),
                                  rows, cols, float(eps), _stream_ptr(stream)), "rmsnorm")
    return out


def fused_add_rmsnorm(residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                      out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """residual += x in place; returns rmsnorm(residual)."""
    for t, name in ((residual, "residual"), (x, "x"), (weight, "weight")):
        _dev_tensor(t, name)
    if (x.dim() != 2 or x.dtype not in _TORCH2CODE or residual.shape != x.shape or residual.dtype != x.dtype
            or weight.dtype != x.dtype or tuple(weight.shape) != (x.shape[1],) or not residual.is_contiguous()):
        raise ValueError("residual and x must be contiguous [rows, cols], weight [cols], one fp32/fp16/bf16 dtype")
    rows, cols = x.shape
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty_like(x)
        check(lib.inferop_fused_add_rmsnorm(residual.data_ptr(), out.data_ptr(), x.data_ptr(), weight.data_ptr(),
                                            int(_TORCH2CODE[x.dtype]), rows, cols, float(eps),
                                            _stream_ptr(stream)), "fused_add_rmsnorm")
    return out


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None,
                  q: torch.Tensor | None = None, scales: torch.Tensor | None = None, stream=None):
    """quant_fp8_per_token_group(rmsnorm(x, weight)) in one pass (with `residual`: residual += x first, in
    place, then the norm of the sum).  x fp16 / bf16 [rows, cols], cols % 128 == 0 -> (q uint8, scales fp32)."""
    _dev_tensor(x, "x")
    _dev_tensor(weight, "weight")
    if x.dim() != 2 or x.dtype not in (torch.float16, torch.bfloat16) or weight.dtype != x.dtype or \
            tuple(weight.shape) != (x.shape[1],):
        raise ValueError("x must be fp16 / bf16 [rows, cols] and weight [cols] of the same dtype")
    if residual is not None:
        _dev_tensor(residual, "residual")
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("residual must match x")
    rows, cols = x.shape
    with torch.cuda.device(x.device):
        if q is None:
            q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
        if scales is None:
            scales = torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
        check(lib.inferop_rmsnorm_quant(q.data_ptr(), scales.data_ptr(), residual.data_ptr() if residual is not None else None,
                                        x.data_ptr(), weight.data_ptr(), int(_TORCH2CODE[x.dtype]), rows, cols, 128,
                                        float(eps), _stream_ptr(stream)), "rmsnorm_quant")
    return q, scales


def rope_neox(qkv: torch.Tensor, positions: torch.Tensor, rotary_dim: int, base: float = 10000.0,
              yarn_factor: float = 1.0, stream=None) -> torch.Tensor:
    """NeoX rotary embedding in place on qkv [tokens, heads, head_dim]; positions int64 [tokens]."""
    _dev_tensor(qkv, "qkv")
    _dev_tensor(positions, "positions")
    if qkv.dim() != 3 or qkv.dtype not in _TORCH2CODE or positions.dtype != torch.int64 or \
            positions.numel() != qkv.shape[0]:
        raise ValueError("qkv must be [tokens, heads, head_dim] (fp32/fp16/bf16) and positions int64 [tokens]")
    tokens, heads, head_dim = qkv.shape
    with torch.cuda.device(qkv.device):
        check(lib.inferop_rope_neox(qkv.data_ptr(), positions.data_ptr(), int(_TORCH2CODE[qkv.dtype]), tokens,
                                    heads, head_dim, int(rotary_dim), float(base), float(yarn_factor),
                                    _stream_ptr(stream)), "rope_neox")
    return qkv


def paged_attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                      seq_lens: torch.Tensor, scale: float, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """q [batch, heads, dim]; k_cache / v_cache [blocks, block_size, kv_heads, dim] (q's dtype); block_tables
    int32 [batch, max_blocks]; seq_lens int32 [batch] -> [batch, heads, dim]."""
    for t, name in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache"), (block_tables, "block_tables"),
                    (seq_lens, "seq_lens")):
        _dev_tensor(t, name)
    if q.dim() != 3 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape or q.dtype not in _TORCH2CODE or \
            k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or k_cache.shape[3] != q.shape[2]:
        raise ValueError("q must be [batch, heads, dim] and the caches [blocks, block_size, kv_heads, dim] of one dtype")
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32 or block_tables.dim() != 2 or \
            block_tables.shape[0] != q.shape[0] or seq_lens.numel() != q.shape[0]:
        raise ValueError("block_tables must be int32 [batch, max_blocks] and seq_lens int32 [batch]")
    batch, heads, dim = q.shape
    _, block_size, kv_heads, _ = k_cache.shape
    with torch.cuda.device(q.device):
        if out is None:
            out = torch.empty_like(q)
        check(lib.inferop_paged_attn_decode(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                            block_tables.data_ptr(), seq_lens.data_ptr(), int(_TORCH2CODE[q.dtype]),
                                            batch, heads, kv_heads, dim, block_size, block_tables.shape[1],
                                            float(scale), _stream_ptr(stream)), "paged_attn_decode")
    return out


def silu_and_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, d + i] (reference include/inferop/ops.h:54-55)."""
    _dev_tensor(gate_up, "gate_up")
    tokens, d2 = gate_up.shape
    with torch.cuda.device(gate_up.device):
        if out is None:
            out = torch.empty((tokens, d2 // 2), dtype=gate_up.dtype, device=gate_up.device)
        check(lib.inferop_silu_and_mul(out.data_ptr(), gate_up.data_ptr(), int(_TORCH2CODE[gate_up.dtype]),
                                       tokens, d2 // 2, _stream_ptr(stream)), "silu_and_mul")
    return out


def silu_and_mul_quant(gate_up: torch.Tensor, q: torch.Tensor | None = None,
                       scales: torch.Tensor | None = None, stream=None):
    """silu_and_mul followed by quant_fp8_per_token_group (group 128) in one pass, bit for bit."""
    _dev_tensor(gate_up, "gate_up")
    tokens, d2 = gate_up.shape
    d = d2 // 2
    with torch.cuda.device(gate_up.device):
        if q is None:
            q = torch.empty((tokens, d), dtype=torch.uint8, device=gate_up.device)
        if scales is None:
            scales = torch.empty((tokens, d // 128), dtype=torch.float32, device=gate_up.device)
        check(lib.inferop_silu_and_mul_quant(q.data_ptr(), scales.data_ptr(), gate_up.data_ptr(),
                                             int(_TORCH2CODE[gate_up.dtype]), tokens, d, 128,
                                             _stream_ptr(stream)), "silu_and_mul_quant")
    return q, scales


class MoeLayout:
    """Device arrays describing the expert-sorted order of a routing (see inferop_moe_align)."""

    def __init__(self, tokens: int, topk: int, experts: int, device):
        self.tokens, self.topk, self.experts = tokens, topk, experts
        self.pairs = tokens * topk
        self.max_mtiles = int(lib.inferop_moe_max_mtiles(tokens, topk, experts))
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.empty(experts, **i32)
        self.offsets = torch.empty(experts + 1, **i32)
        self.pos = torch.empty(self.pairs, **i32)
        self.src_token = torch.empty(self.pairs, **i32)
        self.tile_row0 = torch.empty(self.max_mtiles, **i32)
        self.tile_meta = torch.empty(self.max_mtiles, **i32)
        self.num_mtiles = torch.zeros(1, **i32)


def moe_align(topk_ids: torch.Tensor, experts: int, layout: MoeLayout | None = None, stream=None) -> MoeLayout:
    _dev_tensor(topk_ids, "topk_ids")
    tokens, topk = topk_ids.shape
    with torch.cuda.device(topk_ids.device):
        if layout is None:
            layout = MoeLayout(tokens, topk, experts, topk_ids.device)
        check(lib.inferop_moe_align(topk_ids.data_ptr(), tokens, topk, experts, layout.counts.data_ptr(),
                                    layout.offsets.data_ptr(), layout.pos.data_ptr(),
                                    layout.src_token.data_ptr(), layout.tile_row0.data_ptr(),
                                    layout.tile_meta.data_ptr(), layout.num_mtiles.data_ptr(),
                                    _stream_ptr(stream)), "moe_align")
    return layout


def moe_scatter_quant(x: torch.Tensor, layout: MoeLayout, q: torch.Tensor | None = None,
                      scales: torch.Tensor | None = None, stream=None):
    """Quantise every token row once and write it to its top-k expert-sorted rows."""
    _dev_tensor(x, "x")
    tokens, cols = x.shape
    with torch.cuda.device(x.device):
        if q is None:
            q = torch.empty((layout.pairs, cols), dtype=torch.uint8, device=x.device)
        if scales is None:
            scales = torch.empty((layout.pairs, cols // 128), dtype=torch.float32, device=x.device)
        check(lib.inferop_moe_scatter_quant(q.data_ptr(), scales.data_ptr(), x.data_ptr(),
                                            int(_TORCH2CODE[x.dtype]), layout.pos.data_ptr(), tokens, cols,
                                            layout.topk, 128, _stream_ptr(stream)), "moe_scatter_quant")
    return q, scales


def moe_permute_rows(src: torch.Tensor, perm: torch.Tensor, dst: torch.Tensor, gather: bool, stream=None) -> torch.Tensor:
    """gather: dst[i] = src[perm[i]]; else dst[perm[i]] = src[i] (rows with perm < 0 skipped).
    src / dst are 2-D with the same row size in bytes (a multiple of 16); perm int32 with one
    entry per row of the side that is walked in order (dst for gather, src for scatter)."""
    _dev_tensor(src, "src")
    _dev_tensor(dst, "dst")
    _dev_tensor(perm, "perm")
    row_bytes = src.shape[1] * src.element_size()
    if perm.dtype != torch.int32 or dst.shape[1] * dst.element_size() != row_bytes:
        raise ValueError("perm must be int32 and src / dst rows must have the same size")
    rows = perm.numel()
    with torch.cuda.device(src.device):
        check(lib.inferop_moe_permute_rows(dst.data_ptr(), src.data_ptr(), perm.data_ptr(), rows, row_bytes,
                                           1 if gather else 0, _stream_ptr(stream)), "moe_permute_rows")
    return dst


def moe_combine(y: torch.Tensor, weights: torch.Tensor, layout: MoeLayout, out: torch.Tensor | None = None,
                stream=None) -> torch.Tensor:
    """out[t] = sum_k weights[t, k] * y[pos[t, k]]."""
    _dev_tensor(y, "y")
    _dev_tensor(weights, "weights")
    hidden = y.shape[1]
    with torch.cuda.device(y.device):
        if out is None:
            out = torch.empty((layout.tokens, hidden), dtype=y.dtype, device=y.device)
        check(lib.inferop_moe_combine(out.data_ptr(), y.data_ptr(), weights.data_ptr(), layout.pos.data_ptr(),
                                      int(_TORCH2CODE[y.dtype]), layout.tokens, hidden, layout.topk,
                                      _stream_ptr(stream)), "moe_combine")
    return out


def w8a8_block_fp8_gemm_grouped_tiles(a_q: torch.Tensor, a_scales: torch.Tensor, b_q: torch.Tensor,
                                      b_scales: torch.Tensor, layout: MoeLayout, out_dtype=torch.bfloat16,
                                      out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """The grouped GEMM driven by the device-side tile list of a MoeLayout (no host round trip)."""
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    _check_quantised(a_q, a_scales, b_q, b_scales, grouped=True)
    groups, n, k = b_q.shape
    m_total = a_q.shape[0]
    with torch.cuda.device(a_q.device):
        if out is None:
            out = torch.empty((m_total, n), dtype=out_dtype, device=a_q.device)
        check(lib.inferop_w8a8_block_fp8_gemm_grouped_tiles(
            out.data_ptr(), a_q.data_ptr(), a_scales.data_ptr(), b_q.data_ptr(), b_scales.data_ptr(),
            layout.tile_row0.data_ptr(), layout.tile_meta.data_ptr(), layout.num_mtiles.data_ptr(),
            layout.max_mtiles, m_total, groups, n, k, 128, 128, int(_TORCH2CODE[out.dtype]),
            _stream_ptr(stream)), "w8a8_block_fp8_gemm_grouped_tiles")
    return out


def w8a8_block_fp8_gemm_grouped_tiles_swiglu(a_q: torch.Tensor, a_scales: torch.Tensor, b_q: torch.Tensor,
                                             b_scales: torch.Tensor, layout: MoeLayout, mid_dtype=torch.bfloat16,
                                             q: torch.Tensor | None = None, scales: torch.Tensor | None = None,
                                             stream=None):
    """gate_up projection + SwiGLU + 1x128 quantisation in one launch: the same (q, scales) as
    w8a8_block_fp8_gemm_grouped_tiles(out dtype mid_dtype) followed by silu_and_mul_quant.
    b_q [G, 2 * inter, K] (gate rows first), b_scales [G, 2 * inter / 128, K / 128]."""
    for t, name in ((a_q, "a_q"), (a_scales, "a_scales"), (b_q, "b_q"), (b_scales, "b_scales")):
        _dev_tensor(t, name)
    if mid_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("mid_dtype must be fp16 or bf16")
    _check_quantised(a_q, a_scales, b_q, b_scales, grouped=True)
    groups, n2, k = b_q.shape
    inter = n2 // 2
    m_total = a_q.shape[0]
    with torch.cuda.device(a_q.device):
        if q is None:
            q = torch.empty((m_total, inter), dtype=torch.uint8, device=a_q.device)
        if scales is None:
            scales = torch.empty((m_total, inter // 128), dtype=torch.float32, device=a_q.device)
        check(lib.inferop_w8a8_block_fp8_gemm_grouped_tiles_swiglu(
            q.data_ptr(), scales.data_ptr(), a_q.data_ptr(), a_scales.data_ptr(), b_q.data_ptr(), b_scales.data_ptr(),
            layout.tile_row0.data_ptr(), layout.tile_meta.data_ptr(), layout.num_mtiles.data_ptr(),
            layout.max_mtiles, m_total, groups, inter, k, 128, 128, int(_TORCH2CODE[mid_dtype]),
            _stream_ptr(stream)), "w8a8_block_fp8_gemm_grouped_tiles_swiglu")
    return q, scales


def device_status(reset: bool = True):
    """Synchronise and return the device-side status record (code, block, aux0, aux1)."""
    rec = (C.c_uint32 * 4)()
    rc = lib.inferop_device_status(rec, 1 if reset else 0)
    if rc not in (_capi.OK, _capi.ERR_DEVICE_WAIT):
        raise InferopError(rc, "device_status")
    return tuple(int(v) for v in rec)


def set_option(key: str, value: int) -> None:
    check(lib.inferop_set_option(key.encode(), int(value)), f"set_option({key})")
