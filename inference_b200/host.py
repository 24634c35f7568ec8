"""Host-buffer front end: y = quant(x) @ W^T for activations and results that live in host memory.

The operators of this library take device pointers (like the reference's).  A caller whose
activations arrive in host memory and whose results must return there pays for two PCIe
transfers per call; this module hides as much of them as the hardware allows by cutting the
rows into panels and running copy-in, quantise + GEMM and copy-out of successive panels on three
streams, so that the call is bounded by the slowest of the three instead of their sum.
Weights stay resident on the device.

With several ranks (column-parallel weights, one process per GPU) every rank needs the whole
quantised activation panel but there is no reason for every rank to upload and quantise all of
it: rank r copies in and quantises rows [r P/G, (r+1) P/G) of each P-row panel, and the ranks
all-gather the E4M3 bytes and the scales over NVLink (half the bytes of the bf16 input, and the
host link of every GPU carries 1/G of the activations instead of all of them).  The gathered
panel is byte-identical to quantising the whole panel on one rank, because the quantisation
works on rows independently.
"""
from __future__ import annotations

import torch

from . import ops


def bind_to_device_numa_node(pci_bus_id: str, sysfs_root: str = "/sys/bus/pci/devices") -> dict | None:
    """Restrict this process to the CPUs next to the GPU with PCI address `pci_bus_id`
    ("0000:1b:00.0" or the 8-digit-domain form nvidia-smi prints), so that host buffers pinned
    afterwards land in that NUMA node's memory (first touch) and the copies between them and the
    GPU do not cross the socket interconnect.  One process per GPU, called before the pinned
    buffers are allocated.  Returns {"node", "cpus"} or None when the topology is not exposed
    (nothing is changed then)."""
    import os
    try:
        dom, bus, rest = pci_bus_id.strip().lower().split(":")
        path = os.path.join(sysfs_root, f"{dom[-4:]}:{bus}:{rest}")
        with open(os.path.join(path, "numa_node")) as f:
            node = int(f.read().strip())
        with open(os.path.join(path, "local_cpulist")) as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            if not part:
                continue
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)          # never widen what the container allows
        if node < 0 or not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return {"node": node, "cpus": len(cpus)}
    except (OSError, ValueError):
        return None


def rank_rows(rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of a `rows`-row panel that `rank` uploads and quantises: equal contiguous
    chunks in rank order (what an all-gather into one tensor reassembles in row order).  `rows`
    must be a multiple of `world`."""
    if rows % world != 0:
        raise ValueError(f"a panel of {rows} rows does not split over {world} ranks")
    per = rows // world
    return rank * per, (rank + 1) * per


class HostLinearFP8:
    """A block-quantised weight matrix on the device, applied to host-resident activations.

    b_q [N, K] uint8 (E4M3), b_scales [N/128, K/128] fp32, both CUDA tensors.
    """

    def __init__(self, b_q: torch.Tensor, b_scales: torch.Tensor, max_rows: int, panel_rows: int = 2048,
                 in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, group=None):
        """`group`: a torch.distributed process group whose ranks hold the column shards of one
        weight matrix and are all given the same activations; None = this rank works alone."""
        import torch.distributed as dist
        self.b_q, self.b_scales = b_q, b_scales
        self.n, self.k = b_q.shape
        self.panel = min(panel_rows, max_rows)
        dev = b_q.device
        self.dev = dev
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if self.world > 1 and (self.panel % self.world or max_rows % self.panel):
            raise ValueError("with several ranks the rows must be whole panels and a panel must split over the ranks")
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        # two sets of device buffers: panel i+1 is copied in while panel i computes
        self.x = [torch.empty((self.panel, self.k), dtype=in_dtype, device=dev) for _ in range(2)]
        self.q = [torch.empty((self.panel, self.k), dtype=torch.uint8, device=dev) for _ in range(2)]
        self.s = [torch.empty((self.panel, self.k // 128), dtype=torch.float32, device=dev) for _ in range(2)]
        self.c = [torch.empty((self.panel, self.n), dtype=out_dtype, device=dev) for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_mm = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        if self.world > 1:
            # this rank's chunk of a panel before the all-gather
            per = self.panel // self.world
            self.q_part = [torch.empty((per, self.k), dtype=torch.uint8, device=dev) for _ in range(2)]
            self.s_part = [torch.empty((per, self.k // 128), dtype=torch.float32, device=dev) for _ in range(2)]
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
        if self.world > 1 and m % self.panel:
            raise ValueError("with several ranks the rows must be whole panels")
        for i, r0 in enumerate(range(0, m, self.panel)):
            rows = min(self.panel, m - r0)
            b = i & 1
            lo, hi = rank_rows(rows, self.world, self.rank) if self.world > 1 else (0, rows)
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(self.ev_mm[b])       # buffers of panel i-2 are free again
                self.x[b][lo:hi].copy_(x_host[r0 + lo:r0 + hi], non_blocking=True)
                self.ev_in[b].record(self.s_in)
            with torch.cuda.stream(self.s_mm):
                self.s_mm.wait_event(self.ev_in[b])
                if i >= 2:
                    self.s_mm.wait_event(self.ev_out[b])      # c[b] has been copied out
                if self.world > 1:
                    import torch.distributed as dist
                    ops.quant_fp8_per_token_group(self.x[b][lo:hi], 128, self.q_part[b], self.s_part[b])
                    dist.all_gather_into_tensor(self.q[b], self.q_part[b], group=self.group)
                    dist.all_gather_into_tensor(self.s[b], self.s_part[b], group=self.group)
                else:
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
