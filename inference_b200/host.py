"""Host-buffer front end: y = quant(x) @ W^T for activations and results that live in host memory.

The operators of this library take device pointers (like the reference's).  A caller whose
activations arrive in host memory and whose results must return there pays for two PCIe
transfers per call; this module hides as much of them as the hardware allows by cutting the
rows into panels and running copy-in, quantise + GEMM and copy-out of successive panels on three
streams, so that the call is bounded by the slowest of the three instead of their sum.
Weights stay resident on the device.
"""
from __future__ import annotations

import torch

from . import ops


class HostLinearFP8:
    """A block-quantised weight matrix on the device, applied to host-resident activations.

    b_q [N, K] uint8 (E4M3), b_scales [N/128, K/128] fp32, both CUDA tensors.
    """

    def __init__(self, b_q: torch.Tensor, b_scales: torch.Tensor, max_rows: int, panel_rows: int = 2048,
                 in_dtype=torch.bfloat16, out_dtype=torch.bfloat16):
        self.b_q, self.b_scales = b_q, b_scales
        self.n, self.k = b_q.shape
        self.panel = min(panel_rows, max_rows)
        dev = b_q.device
        self.dev = dev
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        # two sets of device buffers: panel i+1 is copied in while panel i computes
        self.x = [torch.empty((self.panel, self.k), dtype=in_dtype, device=dev) for _ in range(2)]
        self.q = [torch.empty((self.panel, self.k), dtype=torch.uint8, device=dev) for _ in range(2)]
        self.s = [torch.empty((self.panel, self.k // 128), dtype=torch.float32, device=dev) for _ in range(2)]
        self.c = [torch.empty((self.panel, self.n), dtype=out_dtype, device=dev) for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_mm = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        # one small warm-up call per stream so that later calls allocate nothing
        with torch.cuda.stream(self.s_mm):
            ops.quant_fp8_per_token_group(self.x[0][:1], 128, self.q[0][:1], self.s[0][:1])
            ops.w8a8_block_fp8_gemm(self.q[0][:1], self.s[0][:1], b_q, b_scales, out=self.c[0][:1])
        torch.cuda.synchronize(dev)

    def __call__(self, x_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """x_host [M, K] and out_host [M, N] are pinned host tensors.  Returns out_host; the work
        is complete when the call returns."""
        m = x_host.shape[0]
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_mm, self.s_out):
            s.wait_stream(cur)
        for i, r0 in enumerate(range(0, m, self.panel)):
            rows = min(self.panel, m - r0)
            b = i & 1
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(self.ev_mm[b])       # buffers of panel i-2 are free again
                self.x[b][:rows].copy_(x_host[r0:r0 + rows], non_blocking=True)
                self.ev_in[b].record(self.s_in)
            with torch.cuda.stream(self.s_mm):
                self.s_mm.wait_event(self.ev_in[b])
                if i >= 2:
                    self.s_mm.wait_event(self.ev_out[b])      # c[b] has been copied out
                ops.quant_fp8_per_token_group(self.x[b][:rows], 128, self.q[b][:rows], self.s[b][:rows])
                ops.w8a8_block_fp8_gemm(self.q[b][:rows], self.s[b][:rows], self.b_q, self.b_scales,
                                        out=self.c[b][:rows])
                self.ev_mm[b].record(self.s_mm)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_mm[b])
                out_host[r0:r0 + rows].copy_(self.c[b][:rows], non_blocking=True)
                self.ev_out[b].record(self.s_out)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_mm)
        cur.synchronize()
        return out_host
