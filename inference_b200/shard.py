"""Column-parallel (N-sharded) use of the blockwise-FP8 GEMM across the GPUs of one box.

The reference has no multi-GPU code; this is the partition the benchmark configuration asks
for: rank g of G owns weight rows [g*N/G, (g+1)*N/G) of ``b_q`` and the matching rows of
``b_scales``; activations are replicated and quantised by every rank; each rank produces
``C_g [M, N/G]``.  Output columns depend only on their own weight rows, so there is no data
exchange on the compute path; the one optional collective is an all-gather of the outputs.

Everything here is plain index arithmetic plus ``torch.distributed`` calls, so it runs on
CPU ranks (gloo) as well as on GPUs (nccl).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

BLOCK = 128


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of the weight matrix owned by `rank`.  N must split into whole 128-row
    scale blocks per rank so that no scale block straddles two ranks."""
    if n % (BLOCK * world) != 0:
        raise ValueError(f"N={n} does not split into {world} shards of whole {BLOCK}-row blocks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weights(b_q: torch.Tensor, b_scales: torch.Tensor, world: int, rank: int):
    """This rank's slice of a full (b_q [N, K], b_scales [N/128, K/128]) pair."""
    lo, hi = shard_bounds(b_q.shape[0], world, rank)
    return b_q[lo:hi].contiguous(), b_scales[lo // BLOCK:hi // BLOCK].contiguous()


def gather_outputs(c_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the per-rank outputs into the rank-blocked layout [G, M, N/G]
    (each rank's panel contiguous, which is what one all-gather produces without a copy)."""
    world = dist.get_world_size(group)
    m, n_loc = c_local.shape
    out = torch.empty((world * m, n_loc), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(out, c_local.contiguous(), group=group)
    return out.view(world, m, n_loc)


def blocked_to_row_major(c_blocked: torch.Tensor) -> torch.Tensor:
    """[G, M, N/G] -> [M, N] (a strided copy; only for consumers that need the flat layout)."""
    g, m, n_loc = c_blocked.shape
    return c_blocked.permute(1, 0, 2).reshape(m, g * n_loc)


def peer_columns(n_shard: int, rank: int) -> tuple[int, int]:
    """Columns [lo, hi) of the full [M, N_shard * G] result that `rank`'s GEMM epilogue fills
    in every rank's buffer (the all-gather variant of the GEMM)."""
    return rank * n_shard, (rank + 1) * n_shard


class PeerOutput:
    """The full [M, N] result buffer of this rank, mapped into every rank of the group, and the
    other ranks' buffers mapped into this one.

    `ptrs[d]` is the address of rank d's buffer in this process: what the all-gather variant of
    the GEMM takes as its destinations.  The mapping uses torch's symmetric memory (CUDA virtual
    memory handles exchanged over the process group's store); multicast binding is switched off
    because only plain peer stores are used.  Without an initialised process group the object
    degrades to a single local buffer (one destination).
    """

    def __init__(self, m: int, n_total: int, dtype=torch.bfloat16, device=None, group=None):
        import os
        self.m, self.n_total = m, n_total
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            self.group = group if group is not None else dist.group.WORLD
            self.local = symm.empty((m, n_total), dtype=dtype, device=device)
            self._handle = symm.rendezvous(self.local, self.group)
            self.rank = self._handle.rank
            self.world = self._handle.world_size
            self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
            self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        else:
            self.group = None
            self.local = torch.empty((m, n_total), dtype=dtype, device=device)
            self._handle = None
            self.rank, self.world = 0, 1
            self.ptrs = [self.local.data_ptr()]
            self._flag = None

    def barrier(self) -> None:
        """Stream-ordered meeting point of the ranks: enqueued after a rank's GEMM, it completes
        only when every rank's GEMM (and with it every store into this rank's buffer) has."""
        if self._flag is not None:
            dist.all_reduce(self._flag, group=self.group)


class PanelGather:
    """Column-parallel GEMM whose result reaches every rank's row-major [M, N] buffer through the
    copy engines: the GEMM runs in row panels and writes each panel straight into its place in
    this rank's own buffer (columns [rank N/G, (rank + 1) N/G)); as soon as a panel is complete,
    one 2-D copy per other rank (a stream per destination, destinations rotated so that the ranks
    do not all target the same GPU at once) pushes it over NVLink into the same place of that
    rank's buffer while the tensor cores work on the next panel.  Peer STORES by DMA only: no SM and no epilogue time of the GEMM is spent on the
    transfer, and nothing is loaded from another GPU.  The ranks meet once at the end."""

    def __init__(self, m: int, n_total: int, dtype=torch.bfloat16, device=None, group=None, panels: int = 8):
        self.out = PeerOutput(m, n_total, dtype, device, group)
        self.world, self.rank = self.out.world, self.out.rank
        self.m, self.n_total = m, n_total
        self.n_loc = n_total // self.world
        while panels > 1 and m % (panels * BLOCK) != 0:
            panels //= 2
        self.panels = panels
        self.rows = m // panels
        self.device = self.out.local.device
        self.streams = [torch.cuda.Stream(self.device) for _ in range(max(self.world - 1, 0))]
        self.events = [torch.cuda.Event() for _ in range(panels)]
        self.elem = self.out.local.element_size()

    def __call__(self, a_q, a_scales, b_q, b_scales) -> torch.Tensor:
        """Enqueue GEMM + gather; returns this rank's full [M, N] buffer (complete on the current
        stream once the call's last enqueued operation, the meeting of the ranks, has run)."""
        from . import ops
        cur = torch.cuda.current_stream()
        pitch = self.n_total * self.elem
        for st in self.streams:
            st.wait_stream(cur)          # the previous step's readers of the destination buffers are done
        col0 = self.rank * self.n_loc
        for p in range(self.panels):
            r0, r1 = p * self.rows, (p + 1) * self.rows
            ops.w8a8_block_fp8_gemm_into(self.out.local[r0:r1], col0, a_q[r0:r1], a_scales[r0:r1], b_q, b_scales)
            self.events[p].record(cur)
            offset = (r0 * self.n_total + col0) * self.elem
            for i, st in enumerate(self.streams):
                d = (self.rank + 1 + i) % self.world
                st.wait_event(self.events[p])
                ops.copy_2d_async(self.out.ptrs[d] + offset, pitch, self.out.ptrs[self.rank] + offset, pitch,
                                  self.n_loc * self.elem, r1 - r0, self.device, stream=st)
        for st in self.streams:
            cur.wait_stream(st)
        self.out.barrier()
        return self.out.local


# ----------------------------------------------------------------------------- row-parallel (K shards)
def k_shard_bounds(k: int, world: int, rank: int) -> tuple[int, int]:
    """Columns [lo, hi) of A_q / B_q owned by `rank` when K is split; whole 128-wide scale groups."""
    if k % (BLOCK * world) != 0:
        raise ValueError(f"K={k} does not split into {world} shards of whole {BLOCK}-column groups")
    per = k // world
    return rank * per, (rank + 1) * per


def shard_k(a_q: torch.Tensor, a_scales: torch.Tensor, b_q: torch.Tensor, b_scales: torch.Tensor,
            world: int, rank: int):
    """This rank's K range of a full (a_q [M, K], a_scales [M, K/128], b_q [N, K], b_scales
    [N/128, K/128]) set, each made contiguous."""
    lo, hi = k_shard_bounds(a_q.shape[1], world, rank)
    return (a_q[:, lo:hi].contiguous(), a_scales[:, lo // BLOCK:hi // BLOCK].contiguous(),
            b_q[:, lo:hi].contiguous(), b_scales[:, lo // BLOCK:hi // BLOCK].contiguous())


def owner_rows(m: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of the reduce-scattered result that `rank` owns."""
    if m % (BLOCK * world) != 0:
        raise ValueError(f"M={m} does not split into {world} blocks of whole {BLOCK}-row tiles")
    per = m // world
    return rank * per, (rank + 1) * per


class PeerSlots:
    """This rank's fp32 slots [G][M/G][N] for the partial results of its rows, mapped into every
    rank, and the other ranks' slots mapped into this one (`ptrs[d]` = rank d's slots here): the
    destinations of the scatter GEMM.  Same mapping mechanism and degradation as PeerOutput."""

    def __init__(self, m: int, n: int, device=None, group=None):
        import os
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            self.group = group if group is not None else dist.group.WORLD
            self.world = dist.get_world_size(self.group)
            self.rank = dist.get_rank(self.group)
            rows = owner_rows(m, self.world, self.rank)
            self.local = symm.empty((self.world, rows[1] - rows[0], n), dtype=torch.float32, device=device)
            self._handle = symm.rendezvous(self.local, self.group)
            self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
            self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        else:
            self.group, self.world, self.rank = None, 1, 0
            self.local = torch.empty((1, m, n), dtype=torch.float32, device=device)
            self.ptrs = [self.local.data_ptr()]
            self._flag = None

    def barrier(self) -> None:
        if self._flag is not None:
            dist.all_reduce(self._flag, group=self.group)
