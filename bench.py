#!/usr/bin/env python
"""Benchmark of the blockwise-FP8 W8A8 path: quant_fp8_per_token_group -> w8a8_block_fp8_gemm.

    python bench.py --gpus N --steps K --warmup W            # this library, N ranks (torchrun for N>1)
    python bench.py --impl reference --gpus N ...            # the reference's CPU code on the host cores

Workload (the N-sharded configuration): A bf16 [16384, 7168] replicated, W E4M3 [73728, 7168]
with 128x128 block scales, column-parallel over the ranks (each rank owns N/G weight rows and
their scales), C bf16 [16384, N/G] per rank.  One step = quantise A, then the GEMM.  The total
problem is fixed while G grows ("strong" scaling); no data-path collective is involved unless
--gather is given, which adds an all-gather of C (by NCCL, and by the GEMM's own epilogue
over peer-mapped buffers) and reports both separately.

Prints ONE JSON line on stdout (rank 0).  Synthetic seeded inputs; see inference_b200/synth.py.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "block-FP8 GEMM TFLOPS (quant incl.) & % of B200 FP8 peak / HBM BW, 1-8 GPU"
M_FULL, N_FULL, K_FULL = 16384, 73728, 7168
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
GEMM_TRAFFIC_MEASURED_OVER_MODEL = 0.99   # (299.5 / 313 + 642 / 625) / 2, from the two ncu captures


print_result = print


_REAL_STDOUT_FD = None


def emit_now(text: str) -> None:
    """Write a result line straight to the process's real stdout (used when the run is cut short)."""
    fd = _REAL_STDOUT_FD if _REAL_STDOUT_FD is not None else 1
    os.write(fd, (text + "\n").encode())


def progress(msg: str) -> None:
    """One line on stderr: where a multi-GPU run is (stdout carries only the result line)."""
    print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def run_with_deadline(fn, seconds, on_timeout):
    import threading
    done = threading.Event()

    def watch():
        if not done.wait(seconds):
            on_timeout()

    threading.Thread(target=watch, daemon=True).start()
    try:
        return fn()
    finally:
        done.set()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=M_FULL)
    ap.add_argument("--n", type=int, default=N_FULL)
    ap.add_argument("--k", type=int, default=K_FULL)
    ap.add_argument("--gather", action="store_true",
                    help="(default for N > 1) also time the all-gather of C: NCCL, and the GEMM's own epilogue")
    ap.add_argument("--no-gather", action="store_true", help="skip the all-gather measurements")
    ap.add_argument("--collective-seconds", type=int, default=300,
                    help="deadline for the collective sections (N > 1); the main result is printed without them after it")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="end-to-end section: do not restrict the process to the CPUs next to its GPU")
    ap.add_argument("--no-sweep", action="store_true", help="skip the decode / prefill shape sweep (N=1 only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU-baseline sample budget")
    ap.add_argument("--moe-only", action="store_true",
                    help="run only the MoE section (grouped GEMMs and the expert layer) and print it")
    ap.add_argument("--refcuda-only", action="store_true", help="run only the secondary GPU baseline (the reference's CUDA kernels)")
    ap.add_argument("--block-ops-only", action="store_true", help="run only the RMSNorm / rotary-embedding timings")
    ap.add_argument("--sweep-only", action="store_true", help="run only the decode / prefill shape sweep and print it")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE",
                    help="library tuning option (inferop_set_option), e.g. --set gemm_pair=0; may be repeated")
    ap.add_argument("--moe-experts", type=int, default=256)
    ap.add_argument("--moe-tokens", type=int, default=4096)
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                "source": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.error = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {
                getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
                getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
            }
            while not self._stop.is_set():
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    for bit, name in names.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report it, do not guess
            self.error = repr(e)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "error": self.error}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ----------------------------------------------------------------------------- CPU arms
class CpuSample:
    """A bounded sample of the workload for the reference's CPU path: quantise `rows`
    activation rows, then the GEMM against `cols` weight rows (inputs prepared once, untimed)."""

    def __init__(self, rows: int, cols: int, k: int, seed: int = 0):
        import numpy as np
        import oracle
        self.oracle = oracle
        rng = np.random.default_rng(seed)
        a = rng.standard_normal((rows, k)).astype(np.float32)
        a[:, rng.choice(k, max(1, k // 100), replace=False)] *= 20.0
        self.a = oracle.bf16_widen(oracle.bf16_narrow(a))
        w = (0.02 * rng.standard_normal((cols, k))).astype(np.float32)
        self.bq, self.bs = oracle.block_quant_weights(w)
        self.rows, self.cols, self.k = rows, cols, k
        self.flops = 2.0 * rows * cols * k
        self.kind = "reference" if oracle.have_reference() else "port"

    def run(self, threads: int) -> float:
        """Seconds for one pass (quant + GEMM) on `threads` host threads."""
        o = self.oracle
        t0 = time.perf_counter()
        if self.kind == "reference":
            aq, a_s = o.reference.quant_fp8_per_token_group(self.a, 128, threads=threads)
            o.reference.w8a8_block_fp8_gemm(aq, a_s, self.bq, self.bs, threads=threads)
        else:
            aq, a_s = o.quant_fp8_per_token_group(self.a, 128)
            o.w8a8_block_fp8_gemm(aq, a_s, self.bq, self.bs, threads=threads)
        return time.perf_counter() - t0

    def describe(self) -> str:
        return f"{self.rows} activation rows x {self.cols} weight rows x K={self.k} (quant + GEMM)"


def sized_cpu_sample(k: int, threads: int, budget_s: float) -> CpuSample:
    """A sample costing about budget_s on this host: probe the rate, then scale the rows."""
    probe = CpuSample(max(threads, 8), 256, k)
    rate = probe.flops / max(probe.run(threads), 1e-6)
    cols = 2048
    rows = int(rate * budget_s / (2.0 * cols * k))
    rows = max(threads, (rows // threads) * threads)
    return CpuSample(rows, cols, k)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    k = args.k
    per_step = max(0.5, min(8.0, 120.0 / (args.steps + args.warmup)))
    smp = sized_cpu_sample(k, threads, per_step)
    for _ in range(args.warmup):
        smp.run(threads)
    t_total = sum(smp.run(threads) for _ in range(args.steps))
    flops_total = smp.flops * args.steps
    kind, used = smp.kind, min(threads, smp.rows)
    val = flops_total / t_total / 1e12
    sample = smp.describe() + " per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": {"workload": f"N-sharded W8A8 block-FP8 GEMM M={args.m} N={args.n} K={k}, quant incl.",
                   "note": "CPU arm: each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": used, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print_result(json.dumps(line))


# ----------------------------------------------------------------------------- parity gates
def parity_gate(x, aq, a_s, bq, bs, c, seed=0, rows_per_band=16, n_cols=512, b_rows=None):
    """The result of a timed section against the CPU oracle (the checker, outside every timed
    region): quantised bytes and scales of sampled rows byte for byte, and C on a sampled
    sub-matrix (rows from every 4096-row band x columns stratified over the whole width) within
    max|err| <= 1e-2 * ||row||_inf and relative Frobenius <= 2e-3.  Raises when out of tolerance."""
    from oracle import sampled
    m, n = c.shape
    rows = sampled.band_rows(m, rows_per_band, seed)
    cols = sampled.stratified(n, n_cols, seed + 1)
    quant_exact = sampled.quant_rows_exact(x, aq, a_s, rows) if x is not None else None
    row, fro = sampled.gemm_sample(aq, a_s, bq, bs, c, rows, cols, threads=min(16, os.cpu_count() or 1))
    ok = row <= sampled.ROW_TOL and fro <= sampled.FRO_TOL_16BIT and quant_exact is not False
    rec = {"row": row, "fro": fro, "quant_exact": quant_exact, "rows": int(len(rows)), "cols": int(len(cols)), "ok": bool(ok)}
    if not ok:
        raise AssertionError(f"parity gate failed: {rec}")
    return rec


# ----------------------------------------------------------------------------- secondary GPU baseline
def reference_cuda_baseline(m=4096, n=18432, k=7168, iters=3):
    """The reference's own CUDA kernels for this path (kernels/quant.cu + kernels/gemm/w8a8_block_fp8.cu,
    compiled unmodified for sm_100 into oracle/_ref/libinferop_ref_cuda.so) timed on this GPU through
    the same operator arguments, beside this library on the same inputs; their results are compared."""
    import ctypes as C
    import torch
    from inference_b200 import ops, synth
    path = os.path.join(ROOT, "oracle", "_ref", "libinferop_ref_cuda.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libinferop_ref_cuda.so has not been built (needs the reference tree)"}
    ref = C.CDLL(path)
    vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int32
    ref.refcuda_quant_fp8_per_token_group.argtypes = [vp, vp, vp, i32, i64, i64, i32, vp]
    ref.refcuda_quant_fp8_per_token_group.restype = None
    ref.refcuda_w8a8_block_fp8_gemm.argtypes = [vp] * 5 + [i64] * 3 + [i32] * 3 + [vp]
    ref.refcuda_w8a8_block_fp8_gemm.restype = None
    x = synth.activations(m, k, seed=0)
    bq, bs = synth.quantised_weights(n, k, seed=1)
    aq = torch.empty((m, k), dtype=torch.uint8, device="cuda")
    a_s = torch.empty((m, k // 128), dtype=torch.float32, device="cuda")
    c_ref = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def ref_step():
        ref.refcuda_quant_fp8_per_token_group(aq.data_ptr(), a_s.data_ptr(), x.data_ptr(), 2, m, k, 128, stream)
        ref.refcuda_w8a8_block_fp8_gemm(c_ref.data_ptr(), aq.data_ptr(), a_s.data_ptr(), bq.data_ptr(), bs.data_ptr(),
                                        m, n, k, 128, 128, 2, stream)

    aq2, a_s2 = torch.empty_like(aq), torch.empty_like(a_s)
    c_ours = torch.empty_like(c_ref)

    def our_step():
        ops.quant_fp8_per_token_group(x, 128, aq2, a_s2)
        ops.w8a8_block_fp8_gemm(aq2, a_s2, bq, bs, out=c_ours)

    out = {"m": m, "n": n, "k": k}
    for name, fn, reps in (("reference_cuda", ref_step, iters), ("this_library", our_step, 10)):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) * 1e-3 / reps
        out[name] = {"ms": round(t * 1e3, 3), "tflops": round(2.0 * m * n * k / t / 1e12, 1)}
    out["speedup"] = round(out["reference_cuda"]["ms"] / out["this_library"]["ms"], 1)
    # the reference multiplies by a reciprocal scale, the oracle (and this library) divide: bytes may
    # differ by a rounding step on a few elements, so quantisation is compared as a mismatch rate
    out["quant_bytes_differing"] = float((aq != aq2).float().mean().item())
    out["quant_scales_equal"] = bool(torch.equal(a_s, a_s2))
    # GEMM against GEMM on identical quantised inputs
    ref.refcuda_w8a8_block_fp8_gemm(c_ref.data_ptr(), aq2.data_ptr(), a_s2.data_ptr(), bq.data_ptr(), bs.data_ptr(),
                                    m, n, k, 128, 128, 2, stream)
    torch.cuda.synchronize()
    d = (c_ref.float() - c_ours.float())
    out["gemm_rel_frobenius_vs_reference_cuda"] = float((d.norm() / c_ref.float().norm()).item())
    out["what"] = "quant + GEMM, bf16 out; the reference's CUDA-core kernels (software E4M3 decode, 128x64 tiles) on the same B200"
    return out


# ----------------------------------------------------------------------------- shape sweep
def reference_cuda_lib():
    """oracle/_ref/libinferop_ref_cuda.so (the reference's own CUDA kernels built for sm_100) or None."""
    import ctypes as C
    path = os.path.join(ROOT, "oracle", "_ref", "libinferop_ref_cuda.so")
    if not os.path.exists(path):
        return None
    ref = C.CDLL(path)
    vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int32, C.c_float
    try:
        ref.refcuda_rmsnorm.argtypes = [vp, vp, vp, i32, i64, i64, f32, vp]
        ref.refcuda_rope_neox.argtypes = [vp, vp, i32, i64, i32, i32, i32, f32, f32, vp]
        ref.refcuda_paged_attn_decode.argtypes = [vp] * 6 + [i32] * 7 + [f32, vp]
        for fn in (ref.refcuda_rmsnorm, ref.refcuda_rope_neox, ref.refcuda_paged_attn_decode):
            fn.restype = None
    except AttributeError:
        return None          # an older build of the baseline library without these operators
    return ref


def block_ops(peaks, rows=16384, cols=7168, heads=32, head_dim=128, rotary=64):
    """The operators in front of the quantise + GEMM path in a transformer block (RMSNorm, residual add +
    RMSNorm, NeoX rotary embedding), bf16, device-timed on tensors larger than L2, each checked against
    the oracle on sampled rows after the timing."""
    import numpy as np
    import torch
    import oracle
    from inference_b200 import ops, synth
    x = synth.activations(rows, cols, seed=41, outliers=False)
    res = synth.activations(rows, cols, seed=42, outliers=False)
    w = (0.5 + torch.rand(cols, device="cuda")).to(torch.bfloat16)
    out = torch.empty_like(x)
    qkv = synth.activations(rows, heads * head_dim, seed=43, outliers=False).view(rows, heads, head_dim)
    pos = torch.arange(rows, dtype=torch.int64, device="cuda") * 7 % 131072

    def timed(fn, iters=10):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / iters

    rec = {}
    ref = reference_cuda_lib()
    cur = torch.cuda.current_stream().cuda_stream
    rows_s = np.array([0, 1, rows // 2, rows - 1])
    t = timed(lambda: ops.rmsnorm(x, w, 1e-6, out=out))
    want = oracle.rmsnorm(x[rows_s].float().cpu().numpy(), w.float().cpu().numpy())
    err = float(np.abs(out[rows_s].float().cpu().numpy() - want).max())
    assert err <= 2e-2 * (1 + float(np.abs(want).max())), f"rmsnorm off by {err}"
    byt = 4 * rows * cols
    rec["rmsnorm"] = {"us": round(t * 1e6, 1), "gbs": round(byt / t / 1e9, 1),
                      "frac_of_measured_hbm": round(byt / t / 1e9 / peaks["hbm_gbs"], 3), "max_abs_err": err}
    if ref is not None:
        # the reference's own kernel (one block per row, two passes over memory) on the same tensors
        out_r = torch.empty_like(out)
        tr = timed(lambda: ref.refcuda_rmsnorm(out_r.data_ptr(), x.data_ptr(), w.data_ptr(), 2, rows, cols, 1e-6, cur), iters=5)
        rec["rmsnorm"]["reference_cuda_us"] = round(tr * 1e6, 1)
        rec["rmsnorm"]["max_abs_diff_vs_reference_cuda"] = float((out.float() - out_r.float()).abs().max().item())
        del out_r
    res0 = res.clone()
    t = timed(lambda: ops.fused_add_rmsnorm(res, x, w, 1e-6, out=out))
    r1 = res0.clone()
    ops.fused_add_rmsnorm(r1, x, w, 1e-6, out=out)
    want_res, want_out = oracle.fused_add_rmsnorm(res0[rows_s].float().cpu().numpy(), x[rows_s].float().cpu().numpy(),
                                                  w.float().cpu().numpy())
    err = float(np.abs(out[rows_s].float().cpu().numpy() - want_out).max())
    assert err <= 3e-2 * (1 + float(np.abs(want_out).max())), f"fused_add_rmsnorm off by {err}"
    byt = 8 * rows * cols
    rec["fused_add_rmsnorm"] = {"us": round(t * 1e6, 1), "gbs": round(byt / t / 1e9, 1),
                                "frac_of_measured_hbm": round(byt / t / 1e9 / peaks["hbm_gbs"], 3), "max_abs_err": err}
    # RMSNorm + 1x128 FP8 quantisation in one pass against the two kernels (same bytes and scales)
    qq = torch.empty((rows, cols), dtype=torch.uint8, device="cuda")
    qs = torch.empty((rows, cols // 128), dtype=torch.float32, device="cuda")
    t1 = timed(lambda: ops.rmsnorm_quant(x, w, 1e-6, q=qq, scales=qs))
    q2 = torch.empty_like(qq)
    s2 = torch.empty_like(qs)

    def two_calls():
        ops.rmsnorm(x, w, 1e-6, out=out)
        ops.quant_fp8_per_token_group(out, 128, q2, s2)

    t2 = timed(two_calls)
    byt = 3 * rows * cols + 4 * rows * (cols // 128)
    rec["rmsnorm_quant"] = {"us": round(t1 * 1e6, 1), "gbs": round(byt / t1 / 1e9, 1),
                            "frac_of_measured_hbm": round(byt / t1 / 1e9 / peaks["hbm_gbs"], 3),
                            "two_kernels_us": round(t2 * 1e6, 1),
                            "same_bits": bool(torch.equal(qq, q2) and torch.equal(qs, s2))}
    assert rec["rmsnorm_quant"]["same_bits"]
    q0 = qkv.clone()
    t = timed(lambda: ops.rope_neox(qkv, pos, rotary))
    q1 = q0.clone()
    ops.rope_neox(q1, pos, rotary)
    want = oracle.rope_neox(q0[rows_s].float().cpu().numpy(), pos[rows_s].cpu().numpy(), rotary)
    err = float(np.abs(q1[rows_s].float().cpu().numpy() - want).max())
    assert err <= 2e-2 * (1 + float(np.abs(want).max())), f"rope off by {err}"
    byt = 4 * rows * heads * rotary   # only the rotated part of every head is read and written
    rec["rope_neox"] = {"us": round(t * 1e6, 1), "gbs": round(byt / t / 1e9, 1),
                        "frac_of_measured_hbm": round(byt / t / 1e9 / peaks["hbm_gbs"], 3), "max_abs_err": err,
                        "shape": [rows, heads, head_dim], "rotary_dim": rotary}
    if ref is not None:
        q2 = q0.clone()
        tr = timed(lambda: ref.refcuda_rope_neox(q2.data_ptr(), pos.data_ptr(), 2, rows, heads, head_dim, rotary,
                                                 10000.0, 1.0, cur), iters=5)
        rec["rope_neox"]["reference_cuda_us"] = round(tr * 1e6, 1)
        q2.copy_(q0)
        ref.refcuda_rope_neox(q2.data_ptr(), pos.data_ptr(), 2, rows, heads, head_dim, rotary, 10000.0, 1.0, cur)
        rec["rope_neox"]["max_abs_diff_vs_reference_cuda"] = float((q1.float() - q2.float()).abs().max().item())
        del q2
    rec["shape"] = [rows, cols]
    rec["dtype"] = "bf16"
    rec["paged_attn_decode"] = attention_bench(peaks, ref)
    return rec


def attention_bench(peaks, ref=None):
    """Paged attention decode, bf16, 32 query heads over 8 KV heads of 128: a batch of 64 sequences of 4096
    tokens and one sequence of 65536 tokens; bytes = the K and V rows of the sequences (read once)."""
    import numpy as np
    import torch
    import oracle
    from inference_b200 import ops
    heads, kvh, dim, bs = 32, 8, 128, 16
    out = []
    for batch, length in ((64, 4096), (1, 65536), (8, 1024)):
        per_seq = length // bs
        blocks = batch * per_seq
        g = torch.Generator(device="cuda")
        g.manual_seed(batch)
        k = torch.randn((blocks, bs, kvh, dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        v = torch.randn((blocks, bs, kvh, dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        q = torch.randn((batch, heads, dim), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        tables = torch.randperm(blocks, generator=g, device="cuda").to(torch.int32).view(batch, per_seq)
        lens = torch.full((batch,), length, dtype=torch.int32, device="cuda")
        o = torch.empty_like(q)
        scale = float(1.0 / np.sqrt(dim))
        for _ in range(2):
            ops.paged_attn_decode(q, k, v, tables, lens, scale, out=o)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 10
        e0.record()
        for _ in range(iters):
            ops.paged_attn_decode(q, k, v, tables, lens, scale, out=o)
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) * 1e-3 / iters
        # parity of one sequence against the oracle (its blocks only)
        b0 = batch - 1
        tb = tables[b0].long()
        want = oracle.paged_attn_decode(q[b0:b0 + 1].float().cpu().numpy(), k[tb].float().cpu().numpy(),
                                        v[tb].float().cpu().numpy(), np.arange(per_seq, dtype=np.int32)[None, :],
                                        np.array([length], np.int32), scale)
        err = float(np.abs(o[b0:b0 + 1].float().cpu().numpy() - want).max())
        assert err <= 2e-2, f"paged attention off by {err}"
        byt = 2 * batch * length * kvh * dim * 2
        one = {"batch": batch, "seq_len": length, "heads": heads, "kv_heads": kvh, "head_dim": dim,
               "us": round(t * 1e6, 1), "gbs": round(byt / t / 1e9, 1),
               "frac_of_measured_hbm": round(byt / t / 1e9 / peaks["hbm_gbs"], 3), "max_abs_err": err}
        if ref is not None:
            # the reference's own kernel: one block per (sequence, query head), the cache read once per query head
            o_r = torch.empty_like(o)
            cur = torch.cuda.current_stream().cuda_stream

            def ref_call():
                ref.refcuda_paged_attn_decode(o_r.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(),
                                              lens.data_ptr(), 2, batch, heads, kvh, dim, bs, per_seq, scale, cur)

            ref_call()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(3):
                ref_call()
            e1.record()
            torch.cuda.synchronize()
            one["reference_cuda_us"] = round(e0.elapsed_time(e1) * 1e3 / 3, 1)
            one["max_abs_diff_vs_reference_cuda"] = float((o.float() - o_r.float()).abs().max().item())
        out.append(one)
        del k, v
        torch.cuda.empty_cache()
    return out


def shape_sweep(peaks):
    """Decode (HBM-bound) and prefill (tensor-bound) shapes of the benchmark configs, quant + GEMM,
    device-timed.  Small shapes are replayed from a CUDA graph of 10 steps so that host launch cost
    does not enter; weights (>= 38 MB, up to 132 MB) are larger than or comparable to L2 and every
    step re-reads them after the other tensors of the step went through the cache."""
    import torch
    from inference_b200 import ops, synth
    out = []
    shapes = [(m, n, k) for (n, k) in ((18432, 7168), (7168, 18432), (24576, 1536)) for m in (1, 4, 16, 64)]
    shapes += [(m, n, k) for (n, k) in ((18432, 7168), (7168, 18432)) for m in (1024, 4096, 16384)]
    weights = {}
    for (m, n, k) in shapes:
        if (n, k) not in weights:
            weights.clear()
            weights[(n, k)] = synth.quantised_weights(n, k, seed=5)
        bq, bs = weights[(n, k)]
        x = synth.activations(m, k, seed=6)
        aq = torch.empty((m, k), dtype=torch.uint8, device="cuda")
        a_s = torch.empty((m, k // 128), dtype=torch.float32, device="cuda")
        c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

        def step():
            ops.quant_fp8_per_token_group(x, 128, aq, a_s)
            ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=c)

        side = torch.cuda.Stream()
        reps = 10 if m <= 64 else 3

        def graph_time(fn):
            """Seconds per call of fn, replayed from a CUDA graph of `reps` calls on the side stream."""
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()         # warm-up; also creates this stream's GEMM scratch before capture
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for _ in range(reps):
                        fn()
                g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(side)
                for _ in range(3):
                    g.replay()
                e1.record(side)
                torch.cuda.synchronize()
            del g
            return e0.elapsed_time(e1) * 1e-3 / (3 * reps)

        t = graph_time(step)
        flops = 2.0 * m * n * k
        byt = 3 * m * k + 4 * m * (k // 128) + m * k + 4 * m * (k // 128) + n * k + 4 * (n // 128) * (k // 128) + 2 * m * n
        rec = {"m": m, "n": n, "k": k, "us": round(t * 1e6, 2), "tflops": round(flops / t / 1e12, 1),
               "gbs": round(byt / t / 1e9, 1)}
        t_roof = max(flops / (NOMINAL_FP8_TFLOPS * 1e12), byt / (NOMINAL_HBM_GBS * 1e9))
        rec["frac_of_nominal_roofline"] = round(t_roof / t, 3)
        if m <= 64:
            rec["frac_of_measured_hbm"] = round(byt / t / 1e9 / peaks["hbm_gbs"], 3)
            rec["frac_of_nominal_hbm"] = round(byt / t / 1e9 / NOMINAL_HBM_GBS, 3)
        else:
            rec["frac_of_nominal_fp8_peak"] = round(flops / t / 1e12 / NOMINAL_FP8_TFLOPS, 3)
        rec["parity"] = parity_gate(x, aq, a_s, bq, bs, c, seed=m + n)
        # the same step through the one-call entry point (quantisation as the GEMM's A prologue): the
        # quantiser and the GEMM chained by programmatic dependent launch
        if m <= 16 or m >= 1024:
            c2 = torch.empty_like(c)
            t2 = graph_time(lambda: ops.w8a8_block_fp8_gemm_fused_quant(x, bq, bs, out=c2))
            rec["fused_prologue_us"] = round(t2 * 1e6, 2)
            rec["fused_equals_separate"] = bool(torch.equal(c, c2))
            if m <= 16:
                # and with the quantisation inside the small-M kernel (one launch; option fused_prologue)
                ops.set_option("fused_prologue", 1)
                try:
                    t3 = graph_time(lambda: ops.w8a8_block_fp8_gemm_fused_quant(x, bq, bs, out=c2))
                finally:
                    ops.set_option("fused_prologue", 0)
                rec["in_kernel_prologue_us"] = round(t3 * 1e6, 2)
                rec["in_kernel_equals_separate"] = bool(torch.equal(c, c2))
            del c2
        out.append(rec)
    return out


def moe_config(peaks, experts=256, hidden=7168, inter=2048, tokens=4096, topk=8):
    """MoE expert GEMMs (256 experts, top-8 of 4096 tokens): gate_up [4096 x 7168] and down
    [7168 x 2048] per expert, variable rows per expert from a seeded softmax + top-k routing.
    Times one grouped launch per projection against one GEMM call per expert (the reference's way)."""
    import numpy as np
    import torch
    from inference_b200 import ops, synth
    g = torch.Generator(device="cpu")
    g.manual_seed(11)
    logits = torch.randn((tokens, experts), generator=g, dtype=torch.float32)
    ids = torch.topk(torch.softmax(logits, dim=1), topk, dim=1).indices   # routing: softmax + top-k
    counts = torch.bincount(ids.flatten(), minlength=experts).tolist()
    order = torch.argsort(ids.flatten(), stable=True)                      # token copies grouped by expert
    token_of = (order // topk).cuda()
    m_total = tokens * topk
    out = {"experts": experts, "rows_total": m_total, "rows_per_expert_min_max": [min(counts), max(counts)]}
    x = synth.activations(tokens, hidden, seed=12)
    for name, n, k, a_src in (("gate_up", 2 * inter, hidden, x[token_of]),
                              ("down", hidden, inter, synth.activations(m_total, inter, seed=13))):
        aq, a_s = ops.quant_fp8_per_token_group(a_src.contiguous())
        bq = torch.empty((experts, n, k), dtype=torch.uint8, device="cuda")
        bs = torch.empty((experts, n // 128, k // 128), dtype=torch.float32, device="cuda")
        for e0 in range(0, experts, 32):   # generate in chunks: all experts share one distribution
            q, s_ = synth.quantised_weights(32 * n, k, seed=100 + e0)
            bq[e0:e0 + 32] = q.view(32, n, k)
            bs[e0:e0 + 32] = s_.view(32, n // 128, k // 128)
            del q, s_
        c = torch.empty((m_total, n), dtype=torch.bfloat16, device="cuda")

        def grouped():
            ops.w8a8_block_fp8_gemm_grouped(aq, a_s, bq, bs, counts, out=c)

        def looped():
            r = 0
            for e, me in enumerate(counts):
                if me:
                    ops.w8a8_block_fp8_gemm(aq[r:r + me], a_s[r:r + me], bq[e], bs[e], out=c[r:r + me])
                r += me

        res = {}
        for label, fn, iters in (("grouped", grouped, 5), ("per_expert_calls", looped, 2)):
            fn()
            torch.cuda.synchronize()
            e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0_.record()
            for _ in range(iters):
                fn()
            e1_.record()
            torch.cuda.synchronize()
            res[label + "_ms"] = round(e0_.elapsed_time(e1_) / iters, 3)
        # parity gate: the experts with the fewest and the most rows and one in between, all their rows
        from oracle import sampled
        import numpy as np
        offs = np.concatenate([[0], np.cumsum(counts)])
        nz = [e for e in range(experts) if counts[e] > 0]
        grouped()
        worst = [0.0, 0.0]
        for e in {min(nz, key=lambda i: counts[i]), max(nz, key=lambda i: counts[i]), nz[len(nz) // 2]}:
            r0, r1 = int(offs[e]), int(offs[e + 1])
            row, fro = sampled.gemm_sample(aq[r0:r1], a_s[r0:r1], bq[e], bs[e], c[r0:r1], np.arange(r1 - r0),
                                           sampled.stratified(n, 128, seed=e))
            assert row <= sampled.ROW_TOL and fro <= sampled.FRO_TOL_16BIT, f"MoE {name} expert {e}: row {row} fro {fro}"
            worst = [max(worst[0], row), max(worst[1], fro)]
        res["parity"] = {"row": worst[0], "fro": worst[1], "experts_checked": 3, "ok": True}
        flops = 2.0 * m_total * n * k
        byt = experts * n * k + m_total * k + 2 * m_total * n
        t = res["grouped_ms"] * 1e-3
        res.update({"n": n, "k": k, "tflops": round(flops / t / 1e12, 1), "gbs": round(byt / t / 1e9, 1),
                    "frac_of_measured_hbm": round(byt / t / 1e9 / peaks["hbm_gbs"], 3)})
        out[name] = res
        del bq, bs, c, aq, a_s
        torch.cuda.empty_cache()
    out["layer"] = moe_layer(peaks, experts, hidden, inter, tokens, topk, logits.cuda(), x)
    return out


def moe_layer(peaks, experts, hidden, inter, tokens, topk, logits, x):
    """The whole expert layer as six launches with no host step (routing -> layout ->
    scatter-quantise -> gate_up with SwiGLU + quantisation in its epilogue -> down -> combine),
    beside the seven-launch form with a separate SwiGLU kernel: per-kernel device times
    and, for the HBM-bound ones, achieved bandwidth against the measured copy rate."""
    import torch
    from inference_b200 import ops, synth
    from inference_b200.moe import MoEFP8Layer

    def weights(n, k, seed):
        bq = torch.empty((experts, n, k), dtype=torch.uint8, device="cuda")
        bs = torch.empty((experts, n // 128, k // 128), dtype=torch.float32, device="cuda")
        for e0 in range(0, experts, 32):
            q, s_ = synth.quantised_weights(32 * n, k, seed=seed + e0)
            bq[e0:e0 + 32] = q.view(32, n, k)
            bs[e0:e0 + 32] = s_.view(32, n // 128, k // 128)
        return bq, bs

    wgu, sgu = weights(2 * inter, hidden, 300)
    wd, sd = weights(hidden, inter, 700)
    layer = MoEFP8Layer(wgu, sgu, wd, sd, topk, tokens)
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    pairs = tokens * topk
    lay = layer.layout
    steps = [
        ("topk_softmax", lambda: ops.topk_softmax(logits, topk, True, layer.ids, layer.weights),
         4 * tokens * experts + 8 * pairs),
        ("moe_align", lambda: ops.moe_align(layer.ids, experts, lay), None),
        ("moe_scatter_quant", lambda: ops.moe_scatter_quant(x, lay, layer.xq, layer.xs),
         2 * tokens * hidden + pairs * hidden * (1 + 4 / 128)),
        ("gate_up_gemm_swiglu_quant", lambda: ops.w8a8_block_fp8_gemm_grouped_tiles_swiglu(
            layer.xq, layer.xs, wgu, sgu, lay, torch.bfloat16, layer.hq, layer.hs),
         experts * 2 * inter * hidden + pairs * hidden + pairs * inter * (1 + 4 / 128)),
        ("down_gemm", lambda: ops.w8a8_block_fp8_gemm_grouped_tiles(layer.hq, layer.hs, wd, sd, lay, out=layer.y),
         experts * hidden * inter + pairs * inter + 2 * pairs * hidden),
        ("moe_combine", lambda: ops.moe_combine(layer.y, layer.weights, lay, out),
         2 * pairs * hidden + 2 * tokens * hidden),
    ]
    for _ in range(2):
        layer.forward(x, logits, out)
    torch.cuda.synchronize()
    iters = 5
    res = {"kernels": {}}
    for name, fn, byt in steps:
        fn()
        e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0_.record()
        for _ in range(iters):
            fn()
        e1_.record()
        torch.cuda.synchronize()
        us = e0_.elapsed_time(e1_) / iters * 1e3
        rec = {"us": round(us, 1)}
        if byt:
            rec["gbs"] = round(byt / us / 1e3, 1)
            rec["frac_of_measured_hbm"] = round(byt / us / 1e3 / peaks["hbm_gbs"], 3)
        res["kernels"][name] = rec
    e0_, e1_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0_.record()
    for _ in range(iters):
        layer.forward(x, logits, out)
    e1_.record()
    torch.cuda.synchronize()
    ms = e0_.elapsed_time(e1_) / iters
    flops = 2.0 * pairs * hidden * (2 * inter) + 2.0 * pairs * inter * hidden
    res.update({"layer_ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1), "launches": len(steps),
                "host_synchronisations": 0})
    # the same layer with the separate SwiGLU + quantisation kernel (bit-identical output)
    out7 = torch.empty_like(out)
    layer7 = MoEFP8Layer(wgu, sgu, wd, sd, topk, tokens, fused_swiglu=False)
    for _ in range(2):
        layer7.forward(x, logits, out7)
    e0_.record()
    for _ in range(iters):
        layer7.forward(x, logits, out7)
    e1_.record()
    torch.cuda.synchronize()
    res["seven_launch_form"] = {"layer_ms": round(e0_.elapsed_time(e1_) / iters, 3), "same_bits": bool(torch.equal(out, out7))}
    assert ops.device_status()[0] == 0
    return res


def row_parallel_bench(args, world, rank, dev, max_over_ranks, sync_all, m=M_FULL, n=7168, k=18432):
    """The layer that follows a column-parallel one: activations and weights sharded over K, so
    every rank's GEMM yields a partial [M, N] sum and the ranks reduce-scatter it over the rows.
    Times (a) GEMM with fp32 output + NCCL reduce_scatter and (b) the GEMM whose epilogue stores
    its fp32 partial tiles into the row owners' slots + an ordered sum on the owner."""
    import torch
    import torch.distributed as dist
    from inference_b200 import ops, shard, synth
    if m % (128 * world) or k % (128 * world):
        return {"unavailable": "shape does not split over the ranks"}
    k_loc = k // world
    x = synth.activations(m, k_loc, seed=20 + rank, outliers=True, device=dev)     # this rank's K range
    bq, bs = synth.quantised_weights(n, k_loc, seed=40 + rank, device=dev)
    aq, a_s = ops.quant_fp8_per_token_group(x)
    part = torch.empty((m, n), dtype=torch.float32, device=dev)
    rs_out = torch.empty((m // world, n), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream()
    flops = 2.0 * m * n * k
    res = {"m": m, "n": n, "k": k, "k_per_gpu": k_loc,
           "bytes_sent_per_rank": 4 * (m // world) * n * (world - 1)}

    def timed(fn):
        for _ in range(2):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) * 1e-3 / args.steps)

    def gemm_only():
        ops.quant_fp8_per_token_group(x, 128, aq, a_s)
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=part)

    def nccl():
        gemm_only()
        dist.reduce_scatter_tensor(rs_out, part)

    progress("row-parallel: GEMM alone")
    t0 = timed(gemm_only)
    res["gemm_only"] = {"ms_per_step": t0 * 1e3, "value": flops / t0 / 1e12}
    progress("row-parallel: NCCL reduce_scatter")
    t1 = timed(nccl)
    res["nccl_reduce_scatter"] = {"ms_per_step": t1 * 1e3, "value": flops / t1 / 1e12, "sum": "fp32, NCCL's order"}
    progress("row-parallel: mapping the peers' slots")
    try:
        slots = shard.PeerSlots(m, n, dev)
        err = None
    except Exception as exc:
        slots, err = None, f"{type(exc).__name__}: {exc}"
    flag = torch.tensor([0 if slots is None else 1], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 0:
        res["fused"] = {"unavailable": err or "peer mapping failed on another rank"}
        return res
    out = torch.empty((m // world, n), dtype=torch.bfloat16, device=dev)

    def fused():
        ops.quant_fp8_per_token_group(x, 128, aq, a_s)
        ops.w8a8_block_fp8_gemm_scatter(slots.ptrs, rank, aq, a_s, bq, bs)
        slots.barrier()
        ops.reduce_slots(slots.local, out=out)
        slots.barrier()      # nobody overwrites slots that their owner is still adding

    progress("row-parallel: scatter epilogue + ordered sum")
    t2 = timed(fused)
    close = torch.allclose(out.float(), rs_out, rtol=2e-2, atol=1e-2)
    res["fused"] = {"ms_per_step": t2 * 1e3, "value": flops / t2 / 1e12, "sum": "fp32, rank order",
                    "agrees_with_nccl_within_bf16_rounding": bool(close),
                    "link_gbs_out_per_rank": res["bytes_sent_per_rank"] / t2 / 1e9}
    status = ops.device_status()
    assert status[0] == 0, f"device-side wait ran out: {status}"
    return res


def moe_ep_bench(args, world, rank, dev, max_over_ranks, sync_all, experts=256, hidden=7168, inter=2048,
                 tokens_total=4096, topk=8):
    """The MoE configuration sharded expert-parallel: every rank owns experts / G experts and
    tokens_total / G tokens; FP8 rows travel to the experts' owners and bf16 results back over
    NCCL all-to-all.  Timed: the whole layer per rank (max over ranks); checked: rank 0's output
    against the single-device layer on the same tokens (bit for bit)."""
    import torch
    import torch.distributed as dist
    from inference_b200 import synth
    from inference_b200.expert_parallel import ExpertParallelMoE, expert_bounds
    from inference_b200.moe import MoEFP8Layer
    if experts % (32 * world) or tokens_total % world:
        return {"unavailable": "experts / tokens do not split over the ranks"}
    lo, hi = expert_bounds(experts, world, rank)
    tokens = tokens_total // world

    def weights(e0, e1, n, k, seed):
        bq = torch.empty((e1 - e0, n, k), dtype=torch.uint8, device=dev)
        bs = torch.empty((e1 - e0, n // 128, k // 128), dtype=torch.float32, device=dev)
        for c0 in range(e0, e1, 32):     # chunks of 32 experts, seeded by the first expert of the chunk
            q, s_ = synth.quantised_weights(32 * n, k, seed=seed + c0, device=dev)
            bq[c0 - e0:c0 - e0 + 32] = q.view(32, n, k)
            bs[c0 - e0:c0 - e0 + 32] = s_.view(32, n // 128, k // 128)
            del q, s_
        return bq, bs

    wgu, sgu = weights(lo, hi, 2 * inter, hidden, 300)
    wd, sd = weights(lo, hi, hidden, inter, 700)
    layer = ExpertParallelMoE(wgu, sgu, wd, sd, experts, topk, world, rank)
    x = synth.activations(tokens, hidden, seed=50 + rank, device=dev)
    g = torch.Generator(device="cpu").manual_seed(60 + rank)
    logits = torch.randn((tokens, experts), generator=g).to(dev)
    out = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
    for _ in range(5):     # the first calls also set up NCCL's all-to-all connections
        layer.forward(x, logits, out)
    sync_all()
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = max(3, min(args.steps, 10))
    e0.record(stream)
    for _ in range(iters):
        layer.forward(x, logits, out)
    e1.record(stream)
    torch.cuda.synchronize()
    t = max_over_ranks(e0.elapsed_time(e1) * 1e-3 / iters)
    pairs = tokens_total * topk
    flops = 2.0 * pairs * hidden * (2 * inter) + 2.0 * pairs * inter * hidden
    res = {"experts": experts, "experts_per_rank": hi - lo, "tokens_total": tokens_total, "tokens_per_rank": tokens, "topk": topk,
           "layer_ms": t * 1e3, "tflops": flops / t / 1e12,
           "bytes_sent_per_rank_estimate": tokens * topk * (world - 1) // world * (hidden + hidden // 32 + 4 + 2 * hidden),
           "exchange": "NCCL all_to_all_single: FP8 rows + scales + ids out, bf16 rows back; one host copy of the row counts per call"}
    del wgu, sgu, wd, sd, layer
    torch.cuda.empty_cache()
    if rank == 0:
        # the single-device layer with all experts on rank 0's tokens: the expert-parallel result must equal it
        fgu, fsgu = weights(0, experts, 2 * inter, hidden, 300)
        fd, fsd = weights(0, experts, hidden, inter, 700)
        want = MoEFP8Layer(fgu, fsgu, fd, fsd, topk, tokens).forward(x, logits)
        res["equals_single_device_layer"] = bool(torch.equal(out, want))
        del fgu, fsgu, fd, fsd, want
        torch.cuda.empty_cache()
    return res


# ----------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    from inference_b200 import ops, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert ops.has_cuda() and ops.device_sm_version(local) == 100, "needs B200 (sm_100); no fallback"
    for kv in args.set:
        key, val = kv.split("=")
        ops.set_option(key, int(val))

    m, n, k = args.m, args.n, args.k
    assert n % (128 * world) == 0, "N must split into 128-row blocks per rank"
    n_loc = n // world
    dev = torch.device("cuda", local)

    # inputs: A replicated (same seed on every rank), this rank's weight shard
    x = synth.activations(m, k, seed=0, outliers=True, device=dev)
    bq, bs = synth.quantised_weights(n_loc, k, seed=1 + rank, device=dev)
    aq = torch.empty((m, k), dtype=torch.uint8, device=dev)
    a_s = torch.empty((m, k // 128), dtype=torch.float32, device=dev)
    c = torch.empty((m, n_loc), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream()

    def step():
        ops.quant_fp8_per_token_group(x, 128, aq, a_s)
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=c)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()

    # ---- device-timed region: exactly `steps` steps, per-kernel events inside
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        e0.record(stream)
        for i in range(args.steps):
            ev[i][0].record(stream)
            ops.quant_fp8_per_token_group(x, 128, aq, a_s)
            ev[i][1].record(stream)
            ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs, out=c)
            ev[i][2].record(stream)
        e1.record(stream)
        torch.cuda.synchronize()
    t_region = e0.elapsed_time(e1) * 1e-3
    t_quant = sum(e[0].elapsed_time(e[1]) for e in ev) * 1e-3 / args.steps
    t_gemm = sum(e[1].elapsed_time(e[2]) for e in ev) * 1e-3 / args.steps
    status = ops.device_status()
    assert status[0] == 0, f"device-side wait ran out: {status}"

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # parity of what was just timed: every rank checks its own shard against the oracle
    par = parity_gate(x, aq, a_s, bq, bs, c, seed=17 + rank)
    par["row"], par["fro"] = max_over_ranks(par["row"]), max_over_ranks(par["fro"])
    par["checked_by"] = f"every rank on its own [M, N/{world}] shard; worst rank shown"

    t_region = max_over_ranks(t_region)
    t_gemm_max = max_over_ranks(t_gemm)
    t_quant_max = max_over_ranks(t_quant)
    flops_total = 2.0 * m * n * k
    t_step = t_region / args.steps
    value = flops_total / t_step / 1e12

    # ---- end-to-end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        from inference_b200.host import HostLinearFP8, bind_to_device_numa_node
        # one process per GPU: keep the pinned buffers (allocated next) in the memory next to this GPU
        numa = None
        cpus_before = os.sched_getaffinity(0)
        if not args.no_numa_bind:
            try:
                bus_id = subprocess.run(["nvidia-smi", "-i", str(physical_gpu_index(local)), "--query-gpu=pci.bus_id",
                                         "--format=csv,noheader"], capture_output=True, text=True, timeout=20).stdout
                numa = bind_to_device_numa_node(bus_id)
            except Exception:
                numa = None
        x_host = x.cpu().pin_memory()
        c_host = torch.empty((m, n_loc), dtype=torch.bfloat16).pin_memory()
        lin = HostLinearFP8(bq, bs, max_rows=m, panel_rows=2048,   # the public host-buffer call
                            group=dist.group.WORLD if world > 1 else None)

        for _ in range(2):
            lin(x_host, c_host)
        sync_all()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 10))
        h0.record(stream)
        for _ in range(n_e2e):
            lin(x_host, c_host)
        h1.record(stream)
        torch.cuda.synchronize()
        te = max_over_ranks(h0.elapsed_time(h1) * 1e-3 / n_e2e)
        # parity of the end-to-end result (host buffer) on this rank's shard
        e2e_par = parity_gate(None, aq, a_s, bq, bs, c_host.to(dev), seed=23 + rank, rows_per_band=4, n_cols=128)
        e2e = {"value": flops_total / te / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": x_host.numel() * 2 // world, "d2h_bytes_per_step": c_host.numel() * 2,
               "bytes_are": "per rank (every rank uploads 1/G of the activation rows and reads back its [M, N/G] result)",
               "ms_per_step": te * 1e3, "steps": n_e2e, "host_numa_binding": numa, "parity": {"row": e2e_par["row"], "fro": e2e_par["fro"], "ok": True},
               "api": "inference_b200.host.HostLinearFP8: 2048-row panels, copy-in / quant (+ all-gather of the FP8 rows "
                      "at N > 1) + GEMM / copy-out on three streams"}
        del x_host, c_host, lin
        os.sched_setaffinity(0, cpus_before)   # the CPU baseline below uses every core it is allowed

    peaks = measured_peaks()
    # No FP8 figure was measured on this pool: the denominator is twice a measured bf16 cuBLAS
    # figure.  The sustained one was taken at a 1290 MHz median SM clock; when this run's sampled
    # clock is above that, the clock-comparable figure is the burst one.
    clk = clocks.summary().get("sm_mhz") or 0
    burst_basis = clk > 1350
    fp8_peak = 2.0 * (peaks["bf16_tflops"] if burst_basis else peaks["bf16_tflops_sustained"])
    gemm_flops = 2.0 * m * n_loc * k
    gemm_bytes = m * k + n_loc * k + 4 * m * (k // 128) + 4 * (n_loc // 128) * (k // 128) + 2 * m * n_loc
    quant_bytes = 3 * m * k + 4 * m * (k // 128)
    achieved = gemm_flops / t_gemm_max / 1e12
    roofline = {
        "bound": "tensor", "kernel": "w8a8_pair_gemm_kernel", "achieved": achieved, "peak": fp8_peak,
        "unit": "TFLOP/s", "frac": achieved / fp8_peak,
        "peak_source": f"2 x bf16_tflops{'' if burst_basis else '_sustained'} of {peaks['source']} peaks (no measured FP8 figure; "
                       f"sampled SM clock {clk} MHz {'above' if burst_basis else 'at or below'} the sustained figure's 1290 MHz)",
        "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
        "traffic": None,
        "avg_launch_ms": t_gemm_max * 1e3,
        "quant_kernel": {"bound": "hbm", "achieved": quant_bytes / t_quant_max / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": quant_bytes / t_quant_max / 1e9 / peaks["hbm_gbs"],
                         "avg_launch_ms": t_quant_max * 1e3},
        "gemm_algorithmic_bytes": gemm_bytes,
    }
    # DRAM traffic of one GEMM launch.  The kernel walks C in bands of 4096 rows; a band's
    # activations stay in L2 and the weights stream past once per band, so the traffic is
    # bands * N*K + M*K + M*N*2 (+ scales).  Two ncu captures of smaller cases (M=4096: 299.5 MB
    # measured against 313 MB modelled, M=8192: 642 MB against 625 MB; summaries under profiles/)
    # put measured / model at 0.99 on average; the bench shape itself holds too much device
    # memory for a multi-pass capture, so the model times that ratio is reported.
    bands = -(-m // 4096)
    model = bands * n_loc * k + m * k + 2 * m * n_loc + 4 * m * (k // 128) + 4 * (n_loc // 128) * (k // 128)
    ratio = GEMM_TRAFFIC_MEASURED_OVER_MODEL
    roofline["traffic"] = model * ratio
    roofline["traffic_note"] = "model bands*N*K + M*K + 2*M*N, checked against ncu at M=4096 and M=8192"

    # ---- the collective forms (all-gather of C, row-parallel partner): measured after the main
    # figures are complete and under a deadline, so that a box on which the peer mapping or a
    # collective stalls still yields the main result
    def collective_sections():
        # ---- optional all-gather of C (reported separately)
        gather = None
        if world > 1 and not args.no_gather:
            progress("all-gather by NCCL")
            c_all = torch.empty((world * m, n_loc), dtype=torch.bfloat16, device=dev)  # [G][M][N/G] rank-blocked
            for _ in range(2):
                dist.all_gather_into_tensor(c_all, c)
            sync_all()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(stream)
            for _ in range(args.steps):
                step()
                dist.all_gather_into_tensor(c_all, c)
            g1.record(stream)
            torch.cuda.synchronize()
            tg = max_over_ranks(g0.elapsed_time(g1) * 1e-3 / args.steps)
            gather = {"ms_per_step_with_gather": tg * 1e3, "value_with_gather": flops_total / tg / 1e12,
                      "bytes_received_per_rank": 2 * m * n_loc * (world - 1), "layout": "[G][M][N/G] rank-blocked"}
            # the same with the GEMM cut into row panels and each panel's all-gather issued on a
            # second stream as soon as the panel is done, so that NCCL moves panel p while the
            # tensor cores work on panel p + 1 (layout [P][G][M/P][N/G])
            progress("all-gather by NCCL, panel-pipelined")
            panels = 8 if m % (8 * 128) == 0 else 1
            rows_p = m // panels
            side = torch.cuda.Stream(device=dev)
            c_pan = torch.empty((panels, world * rows_p, n_loc), dtype=torch.bfloat16, device=dev)
            evs = [torch.cuda.Event() for _ in range(panels)]

            def panel_step():
                ops.quant_fp8_per_token_group(x, 128, aq, a_s)
                for pi in range(panels):
                    r0, r1 = pi * rows_p, (pi + 1) * rows_p
                    ops.w8a8_block_fp8_gemm(aq[r0:r1], a_s[r0:r1], bq, bs, out=c[r0:r1])
                    evs[pi].record(stream)
                    with torch.cuda.stream(side):
                        side.wait_event(evs[pi])
                        dist.all_gather_into_tensor(c_pan[pi], c[r0:r1])
                stream.wait_stream(side)

            for _ in range(2):
                panel_step()
            sync_all()
            g0.record(stream)
            for _ in range(args.steps):
                panel_step()
            g1.record(stream)
            torch.cuda.synchronize()
            tp = max_over_ranks(g0.elapsed_time(g1) * 1e-3 / args.steps)
            same_p = all(torch.equal(c_pan[pi].view(world, rows_p, n_loc)[r],
                                     c_all.view(world, m, n_loc)[r, pi * rows_p:(pi + 1) * rows_p])
                         for pi in range(panels) for r in range(world))
            gather["panel_pipelined"] = {"ms_per_step": tp * 1e3, "value": flops_total / tp / 1e12, "panels": panels,
                                         "layout": "[P][G][M/P][N/G]", "equals_nccl_gather": bool(same_p)}
            del c_pan
            # the same step with the gather done by the GEMM's own epilogue (peer stores into every
            # rank's row-major [M, N] buffer), then a stream-ordered meeting of the ranks
            from inference_b200 import shard
            progress("mapping the peers' output buffers")
            try:
                po = shard.PeerOutput(m, n, torch.bfloat16, dev)
                peer_error = None
            except Exception as exc:   # no peer mapping on this box: report it, keep the NCCL figures
                po, peer_error = None, f"{type(exc).__name__}: {exc}"
            # every rank must take the same branch
            flag = torch.tensor([0 if po is None else 1], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 1:
                progress("all-gather by the GEMM epilogue")

                def fused_step():
                    ops.quant_fp8_per_token_group(x, 128, aq, a_s)
                    ops.w8a8_block_fp8_gemm_allgather(po.ptrs, rank, aq, a_s, bq, bs)
                    po.barrier()

                for _ in range(2):
                    fused_step()
                sync_all()
                g0.record(stream)
                for _ in range(args.steps):
                    fused_step()
                g1.record(stream)
                torch.cuda.synchronize()
                tf = max_over_ranks(g0.elapsed_time(g1) * 1e-3 / args.steps)
                blocked = c_all.view(world, m, n_loc)
                same = all(torch.equal(po.local[:, r * n_loc:(r + 1) * n_loc], blocked[r]) for r in range(world))
                gpar = None
                if rank == 0:
                    # rank 0 checks its gathered [M, N] buffer against the oracle, every rank's column range
                    # with that rank's weights (regenerated here from the rank's seed)
                    worst = [0.0, 0.0]
                    for r in range(world):
                        bq_r, bs_r = (bq, bs) if r == 0 else synth.quantised_weights(n_loc, k, seed=1 + r, device=dev)
                        rec = parity_gate(None, aq, a_s, bq_r, bs_r, po.local[:, r * n_loc:(r + 1) * n_loc], seed=31 + r,
                                          rows_per_band=4, n_cols=64)
                        worst = [max(worst[0], rec["row"]), max(worst[1], rec["fro"])]
                        del bq_r, bs_r
                    gpar = {"row": worst[0], "fro": worst[1], "ok": True,
                            "checked_by": "rank 0 on its gathered [M, N] buffer, all ranks' column ranges"}
                gather["fused"] = {"ms_per_step": tf * 1e3, "value": flops_total / tf / 1e12,
                                   "layout": "[M][N] row-major on every rank",
                                   "equals_nccl_gather": bool(same), "parity": gpar,
                                   "link_gbs_out_per_rank": 2 * m * n_loc * (world - 1) / tf / 1e9}
                status = ops.device_status()
                assert status[0] == 0, f"device-side wait ran out: {status}"
                # the same gather by the copy engines: the GEMM in row panels, each finished panel pushed
                # into every rank's [M, N] buffer by one 2-D DMA copy per destination
                progress("all-gather by the copy engines, panel by panel")
                del po
                pg = shard.PanelGather(m, n, torch.bfloat16, dev, panels=8)

                def ce_step():
                    ops.quant_fp8_per_token_group(x, 128, aq, a_s)
                    pg(aq, a_s, bq, bs)

                for _ in range(2):
                    ce_step()
                sync_all()
                g0.record(stream)
                for _ in range(args.steps):
                    ce_step()
                g1.record(stream)
                torch.cuda.synchronize()
                tc = max_over_ranks(g0.elapsed_time(g1) * 1e-3 / args.steps)
                same_ce = all(torch.equal(pg.out.local[:, r * n_loc:(r + 1) * n_loc], blocked[r]) for r in range(world))
                gather["copy_engine_panels"] = {"ms_per_step": tc * 1e3, "value": flops_total / tc / 1e12, "panels": pg.panels,
                                                "layout": "[M][N] row-major on every rank", "equals_nccl_gather": bool(same_ce),
                                                "link_gbs_out_per_rank": 2 * m * n_loc * (world - 1) / tc / 1e9}
                best = min((("nccl_after_gemm", tg), ("nccl_panel_pipelined", tp), ("gemm_epilogue_peer_stores", tf),
                            ("copy_engine_panels", tc)), key=lambda kv: kv[1])
                gather["fastest_form"] = best[0]
                del pg
                po = None
            else:
                gather["fused"] = {"unavailable": peer_error or "peer mapping failed on another rank"}
            del c_all, po

        # ---- the row-parallel partner layer (K sharded), reduce-scattered: reported separately
        row_parallel = None
        if world > 1 and not args.no_gather:
            progress("row-parallel partner")
            row_parallel = row_parallel_bench(args, world, rank, dev, max_over_ranks, sync_all)
            progress("expert-parallel MoE layer")
            row_parallel = {"row_parallel": row_parallel, "moe_ep": moe_ep_bench(args, world, rank, dev, max_over_ranks, sync_all)}
            progress("collective sections done")
        return gather, row_parallel

    if rank != 0:
        # the other ranks take part in the collective sections and print nothing
        if not args.no_gather:
            # a rank whose collective section stalls leaves with a failure code: the stall must be visible
            run_with_deadline(collective_sections, args.collective_seconds, lambda: os._exit(3))
        dist.destroy_process_group()
        return

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": f"N-sharded W8A8 block-FP8 GEMM M={m} N={n} K={k}, quant incl.",
                   "m": m, "n": n, "k": k, "n_per_gpu": n_loc, "parallelism": f"column-parallel x{world}",
                   "out": "bf16", "l2": "inputs larger than L2 (no flush needed)",
                   "a": "bf16 N(0,1), 1% outlier channels x20", "w": "bf16 N(0,0.02) block-quantised 128x128"},
        "roofline": roofline, "parity": par, "gpu_launches": 2 * args.steps,
        "clocks": clocks.summary(),
        "frac_of_nominal_fp8_peak": value / (NOMINAL_FP8_TFLOPS * world),
    }
    if e2e:
        line["e2e"] = e2e
    if world > 1 and not args.no_gather:
        def give_up():
            if rank == 0:
                line["gather"] = {"unavailable": f"the collective sections did not finish within {args.collective_seconds} s"}
                emit_now(json.dumps(line))
            os._exit(3)   # the main figures are printed, the stalled collective is still a failure
        gather, row_parallel = run_with_deadline(collective_sections, args.collective_seconds, give_up)
        if gather:
            line["gather"] = gather
        if row_parallel:
            line["row_parallel"] = row_parallel["row_parallel"]
            line["moe_ep"] = row_parallel["moe_ep"]
    if world == 1 and not args.no_sweep:
        del x, bq, bs, aq, a_s, c
        torch.cuda.empty_cache()
        line["sweep"] = {"what": "quant + GEMM per shape, device-timed (CUDA graph replay), bf16 out",
                         "shapes": shape_sweep(peaks)}
        torch.cuda.empty_cache()
        line["moe"] = moe_config(peaks, experts=args.moe_experts, tokens=args.moe_tokens)
        torch.cuda.empty_cache()
        line["extra"] = {"reference_cuda": reference_cuda_baseline(), "block_ops": block_ops(peaks)}
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        smp = sized_cpu_sample(k, threads, args.cpu_seconds)
        dt = smp.run(threads)
        line["cpu_baseline"] = {"value": smp.flops / dt / 1e12, "unit": "TFLOP/s",
                                "cores": min(threads, smp.rows), "kind": smp.kind,
                                "sample": smp.describe() + f", {dt:.1f} s"}
    print_result(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    # Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line
    # there.  Everything else goes to stderr: fd 1 is pointed at fd 2 for the duration of the run
    # and the result line is written to the saved descriptor.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    global _REAL_STDOUT_FD
    _REAL_STDOUT_FD = real_stdout
    os.dup2(2, 1)
    captured = []
    global print_result
    print_result = lambda text: captured.append(text)
    try:
        if args.impl == "reference":
            run_reference(args)
        elif args.refcuda_only:
            print_result(json.dumps({"reference_cuda": reference_cuda_baseline()}))
        elif args.block_ops_only:
            print_result(json.dumps({"block_ops": block_ops(measured_peaks())}))
        elif args.moe_only or args.sweep_only:
            from inference_b200 import ops
            for kv in args.set:
                key, val = kv.split("=")
                ops.set_option(key, int(val))
            if args.moe_only:
                res = moe_config(measured_peaks(), experts=args.moe_experts, tokens=args.moe_tokens)
                print_result(json.dumps({"moe": res}))
            else:
                print_result(json.dumps({"sweep": shape_sweep(measured_peaks()), "options": args.set}))
        else:
            run_ours(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    for text in captured:
        print(text, flush=True)


if __name__ == "__main__":
    main()
