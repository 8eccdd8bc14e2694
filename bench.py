#!/usr/bin/env python
"""Benchmark of the selective-scan path.  Prints ONE JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Workloads (a "step" is one forward+backward pass of the scan over one synthetic batch):
  scan_130m  (default) fused selective scan fwd+bwd on the Mamba-130m layer shape
             (B=8 per GPU, L=2048, ED=1536, N=16, bf16 I/O, float32 state).  With N GPUs every
             rank scans its own batch (the path shards over batch with no communication).
  pscan      the PScan operator fwd+bwd, float32, (16, 2048, 1536, 16) per GPU.
  decode     one Mamba-2.8b-shaped layer-step (B=256, ED=5120) repeated; state traffic bound.
  lshard     the long sequence (1, 131072, 5120, 16) bf16 split over the N GPUs along L, with
             the carry all-gather between the local scans (strong scaling).

`--impl reference` times the reference's own algorithm (the CPU restatement under oracle/,
PyTorch ops on the host cores) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.samples, self.period, self._stop = [], period_s, threading.Event()
        self.thread, self.ok = None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.ok:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def stop(self):
        if self.thread:
            self._stop.set()
            self.thread.join()

    def summary(self, t_lo=None, t_hi=None):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        sel = [s for s in self.samples if (t_lo is None or s[0] >= t_lo) and (t_hi is None or s[0] <= t_hi)]
        window = "timed region"
        if len(sel) < 3:
            sel, window = self.samples, "whole measurement (timed region shorter than 3 samples)"
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        seen = set()
        for _, _, r in sel:
            for bit, nm in names.items():
                if r & bit:
                    seen.add(nm)
        return {"sm_mhz": statistics.median(s[1] for s in sel), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(seen), "samples": len(sel), "window": window}


# ------------------------------------------------------------------------ device timing
def time_region(fn, steps, world, finish=None):
    """barrier + sync, K calls of fn bracketed by CUDA events, sync + barrier; max over ranks (ms).

    `finish` (optional) runs before the closing event; a step that uses side streams joins them there."""
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_lo = time.perf_counter()
    e0.record()
    for _ in range(steps):
        fn()
    if finish is not None:
        finish()
    e1.record()
    torch.cuda.synchronize()
    t_hi = time.perf_counter()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = t.item()
    return ms, t_lo, t_hi


def time_kernel(fn, iters=10):
    """Average device time (ms) of one launch, each launch timed by its own event pair."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) for a, b in evs]
    return sum(ts) / len(ts), min(ts)


# ------------------------------------------------------------------------- CPU baseline
def cpu_reference_scan_fwd_bwd(Bsz, L, ED, N, seed, threads):
    """One fwd+bwd of the reference's selective_scan + gate (parallel-scan route) on the host."""
    from oracle import scan_oracle as O
    import torch.nn.functional as F
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Bsz, L, ED, generator=g).requires_grad_()
    delta = F.softplus(torch.randn(Bsz, L, ED, generator=g) * 0.5 - 4.6).requires_grad_()
    A = (-torch.arange(1, N + 1, dtype=torch.float32).repeat(ED, 1)).requires_grad_()
    Bm = torch.randn(Bsz, L, N, generator=g).requires_grad_()
    Cm = torch.randn(Bsz, L, N, generator=g).requires_grad_()
    D = torch.ones(ED, requires_grad=True)
    z = torch.randn(Bsz, L, ED, generator=g).requires_grad_()
    gy = torch.randn(Bsz, L, ED, generator=g)

    def step():
        for t in (x, delta, A, Bm, Cm, D, z):
            t.grad = None
        y = O.gate(O.selective_scan(x, delta, A, Bm, Cm, D), z)
        y.backward(gy)
    return step


def cpu_reference_pscan_fwd_bwd(Bsz, L, D, N, seed, threads):
    from oracle import scan_oracle as O
    import torch.nn.functional as F
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    A = torch.exp(-F.softplus(torch.randn(Bsz, L, D, N, generator=g))).requires_grad_()
    X = torch.randn(Bsz, L, D, N, generator=g).requires_grad_()
    G = torch.randn(Bsz, L, D, N, generator=g)

    def step():
        A.grad = None
        X.grad = None
        O.pscan(A, X).backward(G)
    return step


CPU_SAMPLES = {
    # workload: (builder, kwargs of the bounded sample, tokens in the sample, description)
    "scan_130m": (cpu_reference_scan_fwd_bwd, dict(Bsz=1, L=2048, ED=1536, N=16), 2048,
                  "1 of the 8 batch rows (B=1, L=2048, ED=1536, N=16), float32, selective_scan+gate fwd+bwd"),
    "lshard": (cpu_reference_scan_fwd_bwd, dict(Bsz=1, L=1024, ED=5120, N=16), 1024,
               "first 1024 of 131072 timesteps (B=1, ED=5120, N=16), float32, selective_scan+gate fwd+bwd"),
    "pscan": (cpu_reference_pscan_fwd_bwd, dict(Bsz=1, L=2048, D=1536, N=16), 2048,
              "1 of the 16 batch rows (B=1, L=2048, D=1536, N=16), float32, pscan fwd+bwd"),
}


def cpu_baseline(workload, repeats=3):
    threads = os.cpu_count() or 1
    builder, kw, tokens, desc = CPU_SAMPLES[workload]
    step = builder(seed=1002, threads=threads, **kw)
    step()                                            # warm-up
    ts = []
    for _ in range(repeats):
        t = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t)
    return {"value": tokens / statistics.median(ts), "unit": "tokens/s", "cores": threads,
            "kind": "port", "sample": desc, "s_per_sample": statistics.median(ts)}


def run_reference(args, rank):
    """The reference arm: the reference's own CPU algorithm on the host cores, rank 0 only."""
    if rank != 0:
        return
    wl = args.workload if args.workload in CPU_SAMPLES else "scan_130m"
    threads = os.cpu_count() or 1
    builder, kw, tokens, desc = CPU_SAMPLES[wl]
    step = builder(seed=1002, threads=threads, **kw)
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    v = tokens * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC[wl], "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": SCALING[wl], "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(wl, args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


METRIC = {"scan_130m": "selective_scan_fwd_bwd_tokens_per_s", "lshard": "selective_scan_fwd_bwd_tokens_per_s",
          "pscan": "pscan_fwd_bwd_tokens_per_s", "decode": "decode_layer_steps_tokens_per_s",
          "layer": "mamba_layer_fwd_bwd_tokens_per_s"}
SCALING = {"scan_130m": "weak", "pscan": "weak", "decode": "weak", "lshard": "strong", "layer": "weak"}


def workload_config(wl, n):
    if wl == "scan_130m":
        return {"workload": "fused selective scan fwd+bwd, Mamba-130m layer shape, gated, softplus(delta+bias) inside",
                "B_per_gpu": 8, "global_batch": 8 * n, "seq_len": 2048, "ED": 1536, "N": 16,
                "io_dtype": "bf16", "state_dtype": "f32", "parallelism": f"batch-sharded x{n}, no collective",
                "l2": "inputs+outputs of one step are 0.56 GB, larger than the 126 MB L2; no flush needed"}
    if wl == "pscan":
        return {"workload": "PScan fwd+bwd, float32", "B_per_gpu": 16, "global_batch": 16 * n, "seq_len": 2048,
                "D": 1536, "N": 16, "io_dtype": "f32", "parallelism": f"batch-sharded x{n}, no collective",
                "l2": "25.8 GB touched per step, larger than L2"}
    if wl == "decode":
        return {"workload": "one Mamba-2.8b-shaped layer-step (conv window + SSM state update + gate)",
                "B_per_gpu": 256, "global_batch": 256 * n, "ED": 5120, "N": 16, "io_dtype": "bf16",
                "state_dtype": "f32", "parallelism": f"batch-sharded x{n}, no collective",
                "l2": "8 layers' states (0.67 GB) are cycled so every step misses L2"}
    if wl == "layer":
        return {"workload": "one whole Mamba-130m-shaped residual layer fwd+bwd (projections by the GEMM library; RMSNorm, "
                            "conv1d+SiLU and gated scan by this library), bf16 autocast, float32 scan state",
                "B_per_gpu": 8, "global_batch": 8 * n, "seq_len": 2048, "d_model": 768, "ED": 1536, "N": 16,
                "io_dtype": "bf16", "state_dtype": "f32", "parallelism": f"batch-sharded x{n}, no collective",
                "l2": "activations of one step exceed the 126 MB L2; no flush needed"}
    return {"workload": "L-sharded fused selective scan fwd+bwd, long sequence", "global_batch": 1,
            "seq_len": 131072, "ED": 5120, "N": 16, "io_dtype": "bf16", "state_dtype": "f32",
            "parallelism": f"sequence split over {n} GPU(s), carry all-gather over NCCL",
            "l2": "14.8 GB touched per step, larger than L2"}


# ------------------------------------------------------------------------- GPU workloads
def bench_scan_130m(args, rank, world, dev):
    import mamba_b200
    from mamba_b200 import workloads
    from mamba_b200.mamba import sscan_fwd_raw, sscan_bwd_raw
    Bsz, L, ED, N = 8, 2048, 1536, 16
    w = workloads.layer_130m_scan_inputs(1002 + rank, dev, Bsz=Bsz, L=L)
    leaves = {k: w[k].clone().requires_grad_() for k in ("x", "delta_raw", "z", "B", "C", "A", "D", "delta_bias")}

    def step():
        for t in leaves.values():
            t.grad = None
        y = mamba_b200.selective_scan_fn(leaves["x"], leaves["delta_raw"], leaves["A"], leaves["B"], leaves["C"],
                                         leaves["D"], z=leaves["z"], delta_bias=leaves["delta_bias"])
        y.backward(w["dy"])

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms, t_lo, t_hi = time_region(step, args.steps, world)
    tokens = Bsz * L * world
    res = {"value": tokens * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
           "gpu_launches": 2 * args.steps}

    # per-kernel device time, raw launches on the same inputs (live, same process)
    A32, D32, b32 = w["A"], w["D"], w["delta_bias"]
    keep = {}

    def fwd():
        keep["out"] = sscan_fwd_raw(w["x"], w["delta_raw"], A32, w["B"], w["C"], D32, w["z"], b32, want_carries=True)

    fwd()
    carries = keep["out"][2]

    def bwd():
        keep["g"] = sscan_bwd_raw(w["x"], w["delta_raw"], A32, w["B"], w["C"], D32, w["z"], b32, w["dy"], carries)

    for f in (fwd, bwd, fwd, bwd, fwd, bwd):
        f()
    fwd_ms, fwd_min = time_kernel(fwd, 20)
    bwd_ms, bwd_min = time_kernel(bwd, 20)
    s = 2                                              # bytes per bf16 element
    fwd_bytes = (4 * ED + 2 * N) * s * Bsz * L
    bwd_bytes = (7 * ED + 4 * N) * s * Bsz * L
    res["kernels"] = {
        "sscan_fwd_kernel": {"ms": fwd_ms, "ms_min": fwd_min, "algorithmic_bytes": fwd_bytes,
                             "GBps": fwd_bytes / fwd_ms / 1e6},
        "sscan_bwd_kernel": {"ms": bwd_ms, "ms_min": bwd_min, "algorithmic_bytes": bwd_bytes,
                             "GBps": bwd_bytes / bwd_ms / 1e6},
    }
    res["dominant"] = ("sscan_bwd_kernel", bwd_bytes, bwd_ms)
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of that kernel on this exact workload,
    # from the ncu capture summarised in profiles/sscan_bwd_kernel__scan_130m.md (406.6 MB + 132.0 MB;
    # 354.4 MB algorithmic plus 201 MB of saved scan states read back)
    res["traffic"] = 538.6e6
    # why the HBM fraction is small: what the same capture shows to be busy instead (static figures of
    # that capture, not re-measured here)
    res["roofline_note"] = ("the fused backward is not HBM-bound: ncu shows DRAM at 9 % of peak while the "
                            "shared-memory pipe is at 72 %, instruction issue at 60 %, FMA 41 %, MUFU 33 % "
                            "(profiles/sscan_bwd_kernel__scan_130m.md)")

    if args.skip_e2e:
        sampler.stop()
        res["clocks"] = sampler.summary(t_lo, t_hi)
        return res
    # end to end through the public API with host buffers: every step copies its own inputs from pinned
    # host memory and its own results back; copies run on their own streams with two device slots, so the
    # copies of one step overlap the compute of its neighbours (nothing is skipped or reused).
    host_in = {k: w[k].detach().cpu().pin_memory() for k in ("x", "delta_raw", "z", "B", "C", "dy")}
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    slots = [{"dev": {k: torch.empty_like(w[k]) for k in host_in}, "ev_in": torch.cuda.Event(),
              "ev_done": torch.cuda.Event(), "ev_out": torch.cuda.Event(), "outs": None, "host": None}
             for _ in range(2)]
    state = {"i": 0}
    pA, pD, pb = leaves["A"].detach(), leaves["D"].detach(), leaves["delta_bias"].detach()

    def e2e_step():
        sl = slots[state["i"] % 2]
        state["i"] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(sl["ev_done"])                     # the slot's previous step has read its inputs
            for k in host_in:
                sl["dev"][k].copy_(host_in[k], non_blocking=True)
            sl["ev_in"].record(s_in)
        cur.wait_event(sl["ev_in"])
        cur.wait_event(sl["ev_out"])                          # previous results of this slot are on the host
        lv = {k: sl["dev"][k].requires_grad_() for k in ("x", "delta_raw", "z", "B", "C")}
        for t in lv.values():
            t.grad = None
        y = mamba_b200.selective_scan_fn(lv["x"], lv["delta_raw"], pA, lv["B"], lv["C"], pD, z=lv["z"], delta_bias=pb)
        y.backward(sl["dev"]["dy"])
        sl["outs"] = [y.detach()] + [lv[k].grad for k in ("x", "delta_raw", "z", "B", "C")]
        for k in lv:
            sl["dev"][k].requires_grad_(False)
        sl["ev_done"].record(cur)
        if sl["host"] is None:
            sl["host"] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in sl["outs"]]
        with torch.cuda.stream(s_out):
            s_out.wait_event(sl["ev_done"])
            for h, o in zip(sl["host"], sl["outs"]):
                h.copy_(o, non_blocking=True)
            sl["ev_out"].record(s_out)

    def e2e_finish():
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    for _ in range(3):
        e2e_step()
    e2e_finish()
    k_e2e = max(8, min(args.steps, 12))          # enough steps for the two-slot pipeline to reach its steady state
    ems, _, _ = time_region(e2e_step, k_e2e, world, finish=e2e_finish)
    sampler.stop()
    host_out = slots[0]["host"]
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    res["e2e"] = {"value": tokens * k_e2e / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                  "d2h_bytes_per_step": d2h, "steps": k_e2e, "ms_per_step": ems / k_e2e}
    res["clocks"] = sampler.summary(t_lo, t_hi)
    return res


def bench_pscan(args, rank, world, dev):
    import mamba_b200
    from mamba_b200 import workloads
    from mamba_b200.pscan import pscan_fwd_raw, pscan_bwd_raw
    Bsz, L, D, N = 16, 2048, 1536, 16
    A, X, G = workloads.pscan_inputs(1001 + rank, dev, Bsz, L, D, N)
    A.requires_grad_()
    X.requires_grad_()

    def step():
        A.grad = None
        X.grad = None
        mamba_b200.pscan(A, X).backward(G)

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms, t_lo, t_hi = time_region(step, args.steps, world)
    tokens = Bsz * L * world
    res = {"value": tokens * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
           "gpu_launches": 2 * args.steps}
    Ad, Xd = A.detach(), X.detach()
    keep = {}

    def fwd():
        keep["H"] = pscan_fwd_raw(Ad, Xd)[0]

    fwd()

    def bwd():
        keep["g"] = pscan_bwd_raw(Ad, keep["H"], G)

    for f in (fwd, bwd, fwd, bwd):
        f()
    fwd_ms, fwd_min = time_kernel(fwd, 10)
    bwd_ms, bwd_min = time_kernel(bwd, 10)
    sampler.stop()
    elems = Bsz * L * D * N
    res["kernels"] = {
        "pscan_fwd_kernel": {"ms": fwd_ms, "ms_min": fwd_min, "algorithmic_bytes": 3 * elems * 4,
                             "GBps": 3 * elems * 4 / fwd_ms / 1e6},
        "pscan_bwd_kernel": {"ms": bwd_ms, "ms_min": bwd_min, "algorithmic_bytes": 5 * elems * 4,
                             "GBps": 5 * elems * 4 / bwd_ms / 1e6},
    }
    res["dominant"] = ("pscan_bwd_kernel", 5 * elems * 4, bwd_ms)
    # end to end with host buffers would move 12.9 GB per step over PCIe; measured on one batch row
    hA, hX, hG = (t[:1].detach().cpu().pin_memory() for t in (A, X, G))
    dA, dX, dG = (torch.empty_like(t[:1]) for t in (A, X, G))
    hout = [torch.empty(hA.shape).pin_memory() for _ in range(3)]

    def e2e_step():
        dA.copy_(hA, non_blocking=True); dX.copy_(hX, non_blocking=True); dG.copy_(hG, non_blocking=True)
        a, x = dA.requires_grad_(), dX.requires_grad_()
        a.grad = None; x.grad = None
        H = mamba_b200.pscan(a, x)
        H.backward(dG)
        for h, o in zip(hout, (H.detach(), a.grad, x.grad)):
            h.copy_(o, non_blocking=True)
        dA.requires_grad_(False); dX.requires_grad_(False)

    for _ in range(2):
        e2e_step()
    k_e2e = 3
    ems, _, _ = time_region(e2e_step, k_e2e, world)
    per = L * D * N * 4
    res["e2e"] = {"value": L * world * k_e2e / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 3 * per,
                  "d2h_bytes_per_step": 3 * per, "steps": k_e2e, "ms_per_step": ems / k_e2e,
                  "note": "one batch row per step (B=1 of 16): the full batch would move 12.9 GB over PCIe"}
    res["clocks"] = sampler.summary(t_lo, t_hi)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="scan_130m", choices=["scan_130m", "pscan", "decode", "lshard", "layer"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave out the host-buffer leg")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback "
                         "(use --impl reference for the host-CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    wl = args.workload
    if wl == "scan_130m":
        res = bench_scan_130m(args, rank, world, dev)
    elif wl == "pscan":
        res = bench_pscan(args, rank, world, dev)
    elif wl == "decode":
        from mamba_b200.benchmarks import bench_decode
        res = bench_decode(args, rank, world, dev, ClockSampler, time_region, time_kernel)
    elif wl == "layer":
        from mamba_b200.benchmarks import bench_layer
        res = bench_layer(args, rank, world, dev, ClockSampler, time_region, time_kernel)
    else:
        from mamba_b200.benchmarks import bench_lshard
        res = bench_lshard(args, rank, world, dev, ClockSampler, time_region, time_kernel)

    peaks, peak_kind = measured_peaks()
    name, abytes, kms = res["dominant"]
    achieved = abytes / kms / 1e6
    roof = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} copy bandwidth",
            "frac_of_nominal_8TBps": achieved / 8000.0, "traffic": res.get("traffic"),
            **({"note": res["roofline_note"]} if "roofline_note" in res else {}),
            "algorithmic_bytes_per_launch": abytes, "kernel_ms": kms}
    line = {
        "metric": METRIC[wl], "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": SCALING[wl], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(wl, world), **({"seq_len": res["seq_len"]} if "seq_len" in res else {}),
                       **({"subshards_per_gpu": res["subshards"]} if "subshards" in res else {})),
        "roofline": roof, "kernels": res.get("kernels"),
        "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"], "clocks": res.get("clocks"),
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and wl in CPU_SAMPLES:
            line["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(line))
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
