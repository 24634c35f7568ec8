"""A mixture-of-experts feed-forward layer on the blockwise-FP8 kernels, entirely on the device.

The reference offers the pieces (``topk_softmax``, ``silu_and_mul``, ``quant_fp8_per_token_group``,
``w8a8_block_fp8_gemm``; include/inferop/ops.h:54-55, :64-65, :81-84, :108-110) and leaves their
composition to the caller: one GEMM call per expert from the host, which needs the experts' row
counts on the host.  This layer runs the same arithmetic as six launches on one stream with no
host synchronisation in between:

    topk_softmax -> moe_align -> moe_scatter_quant -> grouped GEMM (gate_up) with SwiGLU and the
    1x128 re-quantisation in its epilogue -> grouped GEMM (down) -> moe_combine

(seven with ``fused_swiglu=False``, which keeps silu_and_mul_quant as a kernel of its own).
"""
from __future__ import annotations

import torch

from . import ops


class MoEFP8Layer:
    """w_gate_up [E, 2*inter, hidden] and w_down [E, hidden, inter] as E4M3 bytes with 128x128
    block scales ([E, rows/128, cols/128]).  Buffers are sized once for `max_tokens`."""

    def __init__(self, w_gate_up, s_gate_up, w_down, s_down, topk: int, max_tokens: int,
                 renormalize: bool = True, dtype=torch.bfloat16, fused_swiglu: bool = True):
        """fused_swiglu: SwiGLU and the re-quantisation run in the gate_up GEMM's epilogue (six
        launches, no 16-bit gate_up matrix); False keeps the separate silu_and_mul_quant kernel
        (seven launches).  Both give the same bits."""
        self.fused_swiglu = fused_swiglu
        self.w_gate_up, self.s_gate_up, self.w_down, self.s_down = w_gate_up, s_gate_up, w_down, s_down
        self.experts, n_gu, self.hidden = w_gate_up.shape
        self.inter = n_gu // 2
        assert w_down.shape == (self.experts, self.hidden, self.inter)
        self.topk, self.renormalize, self.dtype = topk, renormalize, dtype
        dev = w_gate_up.device
        self._cap = 0
        self._dev = dev
        self._alloc(max_tokens)

    def _alloc(self, tokens: int) -> None:
        dev, pairs = self._dev, tokens * self.topk
        self._cap = tokens
        self.layout = ops.MoeLayout(tokens, self.topk, self.experts, dev)
        self.ids = torch.empty((tokens, self.topk), dtype=torch.int32, device=dev)
        self.weights = torch.empty((tokens, self.topk), dtype=torch.float32, device=dev)
        self.xq = torch.empty((pairs, self.hidden), dtype=torch.uint8, device=dev)
        self.xs = torch.empty((pairs, self.hidden // 128), dtype=torch.float32, device=dev)
        self.gate_up = torch.empty((pairs, 2 * self.inter), dtype=self.dtype, device=dev)
        self.hq = torch.empty((pairs, self.inter), dtype=torch.uint8, device=dev)
        self.hs = torch.empty((pairs, self.inter // 128), dtype=torch.float32, device=dev)
        self.y = torch.empty((pairs, self.hidden), dtype=self.dtype, device=dev)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [tokens, hidden] (bf16 / fp16), logits [tokens, E] fp32 -> [tokens, hidden]."""
        tokens = x.shape[0]
        if tokens != self._cap:
            # the layout arrays and the grouped GEMM's bounds are tied to the token count
            self._alloc(tokens)
        ops.topk_softmax(logits, self.topk, self.renormalize, self.ids, self.weights)
        ops.moe_align(self.ids, self.experts, self.layout)
        ops.moe_scatter_quant(x, self.layout, self.xq, self.xs)
        if self.fused_swiglu and self.inter % 128 == 0:
            ops.w8a8_block_fp8_gemm_grouped_tiles_swiglu(self.xq, self.xs, self.w_gate_up, self.s_gate_up, self.layout,
                                                         self.dtype, self.hq, self.hs)
        else:
            ops.w8a8_block_fp8_gemm_grouped_tiles(self.xq, self.xs, self.w_gate_up, self.s_gate_up, self.layout,
                                                  out=self.gate_up)
            ops.silu_and_mul_quant(self.gate_up, self.hq, self.hs)
        ops.w8a8_block_fp8_gemm_grouped_tiles(self.hq, self.hs, self.w_down, self.s_down, self.layout, out=self.y)
        return ops.moe_combine(self.y, self.weights, self.layout, out)
