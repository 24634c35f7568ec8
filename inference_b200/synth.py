"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

Activations: bf16 ~ N(0, 1); optionally 1 % of the K channels are scaled by 20
(outlier channels).  Weights: bf16 ~ N(0, 0.02), block-quantised per 128 x 128
block to E4M3 with one fp32 scale per block, the way the reference's GEMM test
builds its weights (tests/test_gemm.cpp:28-45: scale = absmax * fl(1/448),
q = e4m3(w * fl(1/scale))).  This is input preparation, done with torch on
whatever device is asked for; it is not part of the measured path.
"""
from __future__ import annotations

import torch

E4M3_MAX_INV = 1.0 / 448.0


def activations(m: int, k: int, seed: int = 0, outliers: bool = True, device="cuda") -> torch.Tensor:
    """bf16 [m, k]."""
    g = torch.Generator(device=device)
    g.manual_seed(seed * 7919 + 1)
    a = torch.randn((m, k), generator=g, device=device, dtype=torch.float32)
    if outliers:
        gc = torch.Generator(device="cpu")
        gc.manual_seed(seed * 7919 + 2)
        n_out = max(1, k // 100)
        idx = torch.randperm(k, generator=gc)[:n_out].to(device)
        a[:, idx] *= 20.0
    return a.to(torch.bfloat16)


def weights_bf16(n: int, k: int, seed: int = 0, device="cuda", std: float = 0.02) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed * 7919 + 3)
    w = torch.randn((n, k), generator=g, device=device, dtype=torch.float32) * std
    return w.to(torch.bfloat16)


def block_quant_weights(w: torch.Tensor, block: int = 128):
    """w [N, K] (any float dtype) -> (b_q uint8 [N, K], b_scales fp32 [ceil(N/128), K/128])."""
    n, k = w.shape
    assert k % block == 0
    nb = (n + block - 1) // block
    wf = w.to(torch.float32)
    if nb * block != n:
        wf = torch.nn.functional.pad(wf, (0, 0, 0, nb * block - n))
    blocks = wf.view(nb, block, k // block, block)
    amax = blocks.abs().amax(dim=(1, 3))
    inv448 = torch.tensor(E4M3_MAX_INV, dtype=torch.float32, device=w.device)
    scale = torch.where(amax == 0, torch.ones_like(amax), amax * inv448)
    inv = (1.0 / scale)[:, None, :, None]
    q = (blocks * inv).to(torch.float8_e4m3fn).view(torch.uint8)
    q = q.reshape(nb * block, k)[:n].contiguous()
    return q, scale.contiguous()


def quantised_weights(n: int, k: int, seed: int = 0, device="cuda", chunk_rows: int = 8192):
    """Block-quantised weights generated chunk by chunk (keeps peak memory small for big N)."""
    qs, ss = [], []
    for r0 in range(0, n, chunk_rows):
        rows = min(chunk_rows, n - r0)
        w = weights_bf16(rows, k, seed=seed * 1000003 + r0, device=device)
        q, s = block_quant_weights(w)
        qs.append(q)
        ss.append(s)
    return torch.cat(qs, 0), torch.cat(ss, 0)
