"""Expert-parallel form of the mixture-of-experts layer: the experts are split over the ranks of a
group, every rank routes its own tokens, ships each (token, expert) pair's quantised row to the
rank that owns the expert, runs its local experts on what it received, ships the results back and
combines them on the token's owner.

The reference composes a layer from one GEMM call per expert on one device (its roadmap lists
"grouped GEMM + dispatch / combine" as future work, docs/ROADMAP.md:39; routing semantics
reference/reference.cpp:152-181).  Here:

    owner of the tokens                         owner of the experts
    -------------------                         --------------------
    topk_softmax, moe_align (all experts)
    moe_scatter_quant: rows sorted by expert,
      i.e. by destination rank, quantised once
    counts per destination  -- all-to-all -->   counts per source
    E4M3 rows, scales, ids  -- all-to-all -->   moe_align over the received ids (local experts),
                                                rows permuted into expert order,
                                                gate_up GEMM (+ SwiGLU + quantise), down GEMM,
                                                results permuted back into arrival order
    moe_combine             <-- all-to-all --   bf16 rows

Rank r owns experts [r E/G, (r + 1) E/G).  What crosses NVLink on the way out is FP8 (half the
bytes of the bf16 activations).  Every row's result depends only on that row and the expert's
weights, and the combine adds a token's k results in the order of k, so the output equals the
single-device layer bit for bit.  The row counts per rank pair are needed on the host to size
the exchange (one small device-to-host copy per call); everything else stays on the device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops


def expert_bounds(experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by `rank`: equal contiguous blocks."""
    if experts % world != 0:
        raise ValueError(f"{experts} experts do not split over {world} ranks")
    per = experts // world
    return rank * per, (rank + 1) * per


def rows_per_rank(counts: torch.Tensor, world: int) -> torch.Tensor:
    """Per-expert row counts [E] -> rows bound for each rank [G] (experts in contiguous blocks)."""
    return counts.view(world, -1).sum(dim=1)


def exchange_rows(send: torch.Tensor, send_rows, recv_rows, group=None) -> torch.Tensor:
    """All-to-all of row blocks.  `send` holds the rows for rank 0, then those for rank 1, ...
    (send_rows[d] rows each); the result holds the rows from rank 0, then from rank 1, ...
    (recv_rows[s] rows each).  NCCL's all_to_all_single where the backend has it; elsewhere (gloo
    on CPU ranks, which has no all-to-all) the same result from an all-gather of padded buffers."""
    send_rows = [int(v) for v in send_rows]
    recv_rows = [int(v) for v in recv_rows]
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    recv = torch.empty((sum(recv_rows),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(recv, send.contiguous(), recv_rows, send_rows, group=group)
        return recv
    # emulation: every rank publishes its whole send buffer (padded to the longest) and its split
    lens = torch.tensor([send.shape[0]], dtype=torch.int64)
    all_lens = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_lens, lens, group=group)
    longest = max(int(v.item()) for v in all_lens)
    padded = torch.zeros((max(longest, 1),) + tuple(send.shape[1:]), dtype=send.dtype)
    padded[:send.shape[0]] = send
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded, group=group)
    splits = torch.tensor(send_rows, dtype=torch.int64)
    all_splits = [torch.zeros(world, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_splits, splits, group=group)
    at = 0
    for s in range(world):
        first = int(all_splits[s][:rank].sum().item())
        n = int(all_splits[s][rank].item())
        assert n == recv_rows[s]
        recv[at:at + n] = bufs[s][first:first + n]
        at += n
    return recv


class RoutedTokens:
    """What the owner of the tokens keeps between dispatch and combine."""

    def __init__(self, ids, weights, layout, xq, xs, sorted_ids, send_counts):
        self.ids, self.weights, self.layout = ids, weights, layout
        self.xq, self.xs, self.sorted_ids, self.send_counts = xq, xs, sorted_ids, send_counts


class ExpertParallelMoE:
    """One rank's share of an expert-parallel MoE layer.

    w_gate_up [E/G, 2*inter, hidden], w_down [E/G, hidden, inter] (E4M3 bytes) with their
    128 x 128 block scales: the weights of THIS rank's experts only."""

    def __init__(self, w_gate_up, s_gate_up, w_down, s_down, experts_total: int, topk: int, world: int, rank: int,
                 group=None, renormalize: bool = True, dtype=torch.bfloat16):
        self.w_gate_up, self.s_gate_up, self.w_down, self.s_down = w_gate_up, s_gate_up, w_down, s_down
        self.experts_total, self.topk, self.world, self.rank, self.group = experts_total, topk, world, rank, group
        self.lo, self.hi = expert_bounds(experts_total, world, rank)
        self.local_experts, n_gu, self.hidden = w_gate_up.shape
        assert self.local_experts == self.hi - self.lo
        self.inter = n_gu // 2
        self.renormalize, self.dtype = renormalize, dtype

    # ---- owner of the tokens, before the exchange
    def route(self, x: torch.Tensor, logits: torch.Tensor) -> RoutedTokens:
        ids, weights = ops.topk_softmax(logits, self.topk, self.renormalize)
        layout = ops.moe_align(ids, self.experts_total)
        xq, xs = ops.moe_scatter_quant(x, layout)                 # rows in expert order = destination order
        sorted_ids = torch.full((layout.pairs,), -1, dtype=torch.int32, device=x.device)
        sorted_ids[layout.pos.long()] = ids.flatten()             # the expert of every sorted row
        return RoutedTokens(ids, weights, layout, xq, xs, sorted_ids, rows_per_rank(layout.counts, self.world))

    # ---- owner of the experts
    def run_experts(self, rq: torch.Tensor, rs: torch.Tensor, expert_ids: torch.Tensor) -> torch.Tensor:
        """rq [R, hidden] E4M3 rows, rs their scales, expert_ids [R] (global ids, all owned by this
        rank), in arrival order -> the experts' outputs [R, hidden] in the same order."""
        rows = rq.shape[0]
        dev = rq.device
        if rows == 0:
            return torch.empty((0, self.hidden), dtype=self.dtype, device=dev)
        local = (expert_ids - self.lo).to(torch.int32).view(rows, 1).contiguous()
        lay = ops.moe_align(local, self.local_experts)
        q = ops.moe_permute_rows(rq, lay.pos, torch.empty_like(rq), gather=False)
        if (rs.shape[1] * 4) % 16 == 0:
            s = ops.moe_permute_rows(rs, lay.pos, torch.empty_like(rs), gather=False)
        else:   # scale rows shorter than the kernel's 16-byte unit (hidden < 512): a small indexed copy
            s = torch.empty_like(rs)
            s[lay.pos.long()] = rs
        if self.inter % 128 == 0:
            hq, hs = ops.w8a8_block_fp8_gemm_grouped_tiles_swiglu(q, s, self.w_gate_up, self.s_gate_up, lay, self.dtype)
        else:
            gu = ops.w8a8_block_fp8_gemm_grouped_tiles(q, s, self.w_gate_up, self.s_gate_up, lay, self.dtype)
            hq, hs = ops.silu_and_mul_quant(gu)
        y = ops.w8a8_block_fp8_gemm_grouped_tiles(hq, hs, self.w_down, self.s_down, lay, self.dtype)
        return ops.moe_permute_rows(y, lay.pos, torch.empty_like(y), gather=True)

    # ---- owner of the tokens, after the way back
    def combine(self, y_back: torch.Tensor, routed: RoutedTokens, out: torch.Tensor | None = None) -> torch.Tensor:
        return ops.moe_combine(y_back, routed.weights, routed.layout, out)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [tokens of this rank, hidden], logits [tokens, experts_total] -> [tokens, hidden]."""
        routed = self.route(x, logits)
        recv_counts = torch.empty_like(routed.send_counts)
        dist.all_to_all_single(recv_counts, routed.send_counts, group=self.group)
        send_h, recv_h = routed.send_counts.cpu().tolist(), recv_counts.cpu().tolist()   # sizes the exchange
        rq = exchange_rows(routed.xq, send_h, recv_h, self.group)
        rs = exchange_rows(routed.xs, send_h, recv_h, self.group)
        rid = exchange_rows(routed.sorted_ids, send_h, recv_h, self.group)
        y = self.run_experts(rq, rs, rid)
        y_back = exchange_rows(y, recv_h, send_h, self.group)
        return self.combine(y_back, routed, out)
