#!/usr/bin/env python
"""Benchmark of the selective-scan path.  Prints ONE JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A "step" is one forward+backward pass of the scan over one synthetic batch.  The headline (`value`,
`ms_per_step`, `roofline`, `e2e`) is always the fused selective scan on the Mamba-130m layer shape
(B=8 per GPU, L=2048, ED=1536, N=16, bf16 I/O, float32 state, softplus(delta+bias) and gate inside);
with N GPUs every rank scans its own batch (the path shards over batch with no communication).
The timed region of K steps is repeated `--regions` times; `ms_per_step` is the median region.

The default workload `all` adds, in the same line:
  "lshard"   the long sequence (1, 131072, 5120, 16) bf16 split along L over the N GPUs (strong
             scaling; N=1 runs it sub-sharded on one GPU), with the time of each pass and of the
             collectives, preceded by a parity self-check of the sharded scan against the single
             launch on a short sequence ("lshard_parity");
  "pscan", "decode", "b1_long"   (N=1 only) the PScan operator (16, 2048, 1536, 16) float32, the
             Mamba-2.8b-shaped 64-layer decode step (B=256), and the batch-1 shapes the reference
             publishes, each with its dominant kernel's roofline fraction;
  "reference_on_gpu"   (N=1 only) the reference's own parallel-scan path run with PyTorch on this
             same GPU, as a second comparison (the contract baseline is the CPU arm).
`--workload scan_130m|pscan|decode|lshard|layer` runs that one workload as the headline instead.

`--impl reference` times the reference's own implementation on the host cores on a bounded sample
of the headline workload: the unmodified reference from oracle/_ref when it has been made
(kind "reference"), else the CPU restatement under oracle/ (kind "port").
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


def time_regions(fn, steps, world, regions, finish=None):
    """`regions` timed regions of exactly `steps` steps each.  Returns (median region ms, every
    region's ms, host time of the first region's start, of the last region's end)."""
    out, lo, hi = [], None, None
    for _ in range(max(1, regions)):
        ms, t_lo, t_hi = time_region(fn, steps, world, finish)
        out.append(ms)
        lo = t_lo if lo is None else lo
        hi = t_hi
    return statistics.median(out), out, lo, hi


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


class Timing:
    """What the GPU legs (bench_legs.py) get from this file: one definition of "timed region"."""
    ClockSampler = ClockSampler
    time_region = staticmethod(time_region)
    time_regions = staticmethod(time_regions)
    time_kernel = staticmethod(time_kernel)


# ------------------------------------------------------------------------- CPU baseline
def reference_functions():
    """(kind, selective_scan(x, delta, A, B, C, D), pscan(A, X)) of the reference's own code: the
    unmodified reference package from oracle/_ref when it has been made there ("reference"), else the
    CPU restatement under oracle/ ("port").  Both run on whatever device their tensors are on."""
    from oracle.make_ref import ref_path
    p = ref_path()
    if p is not None:
        if p not in sys.path:
            sys.path.insert(0, p)
        import mambapy.mamba as rm
        import mambapy.pscan as rp
        return "reference", (lambda x, d, A, B, C, D: rm.MambaBlock.selective_scan(None, x, d, A, B, C, D)), rp.pscan
    from oracle import scan_oracle as O
    return "port", O.selective_scan, O.pscan


def reference_scan_fwd_bwd(Bsz, L, ED, N, seed, device="cpu"):
    """One fwd+bwd of the reference's selective_scan + gate (mambapy/mamba.py:274-295, :229-231),
    float32, on `device`.  Returns (step function, kind)."""
    import torch.nn.functional as F
    kind, scan, _ = reference_functions()
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g)
    x = mk(Bsz, L, ED).to(device).requires_grad_()
    delta = F.softplus(mk(Bsz, L, ED) * 0.5 - 4.6).to(device).requires_grad_()
    A = (-torch.arange(1, N + 1, dtype=torch.float32).repeat(ED, 1)).to(device).requires_grad_()
    Bm = mk(Bsz, L, N).to(device).requires_grad_()
    Cm = mk(Bsz, L, N).to(device).requires_grad_()
    D = torch.ones(ED, device=device, requires_grad=True)
    z = mk(Bsz, L, ED).to(device).requires_grad_()
    gy = mk(Bsz, L, ED).to(device)

    def step():
        for t in (x, delta, A, Bm, Cm, D, z):
            t.grad = None
        y = scan(x, delta, A, Bm, Cm, D) * F.silu(z)
        y.backward(gy)
    return step, kind


def reference_pscan_fwd_bwd(Bsz, L, D, N, seed, device="cpu"):
    import torch.nn.functional as F
    kind, _, pscan = reference_functions()
    g = torch.Generator().manual_seed(seed)
    A = torch.exp(-F.softplus(torch.randn(Bsz, L, D, N, generator=g))).to(device).requires_grad_()
    X = torch.randn(Bsz, L, D, N, generator=g).to(device).requires_grad_()
    G = torch.randn(Bsz, L, D, N, generator=g).to(device)

    def step():
        A.grad = None
        X.grad = None
        pscan(A, X).backward(G)
    return step, kind


CPU_SAMPLES = {
    # workload: (builder, kwargs of the bounded sample, tokens in the sample, description)
    "scan_130m": (reference_scan_fwd_bwd, dict(Bsz=1, L=2048, ED=1536, N=16), 2048,
                  "1 of the 8 batch rows (B=1, L=2048, ED=1536, N=16), float32, selective_scan+gate fwd+bwd"),
    "lshard": (reference_scan_fwd_bwd, dict(Bsz=1, L=1024, ED=5120, N=16), 1024,
               "first 1024 of 131072 timesteps (B=1, ED=5120, N=16), float32, selective_scan+gate fwd+bwd"),
    "pscan": (reference_pscan_fwd_bwd, dict(Bsz=1, L=2048, D=1536, N=16), 2048,
              "1 of the 16 batch rows (B=1, L=2048, D=1536, N=16), float32, pscan fwd+bwd"),
}


def cpu_baseline(workload, repeats=3):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    builder, kw, tokens, desc = CPU_SAMPLES[workload]
    step, kind = builder(seed=1002, **kw)
    step()                                            # warm-up
    ts = []
    for _ in range(repeats):
        t = time.perf_counter()
        step()
        ts.append(time.perf_counter() - t)
    return {"value": tokens / statistics.median(ts), "unit": "tokens/s", "cores": threads,
            "kind": kind, "sample": desc, "s_per_sample": statistics.median(ts)}


def run_reference(args, rank):
    """The reference arm: the reference's own CPU implementation on the host cores, rank 0 only."""
    if rank != 0:
        return
    wl = args.workload if args.workload in CPU_SAMPLES else "scan_130m"
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    builder, kw, tokens, desc = CPU_SAMPLES[wl]
    step, kind = builder(seed=1002, **kw)
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
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


METRIC = {"scan_130m": "selective_scan_fwd_bwd_tokens_per_s", "lshard": "selective_scan_fwd_bwd_tokens_per_s",
          "pscan": "pscan_fwd_bwd_tokens_per_s", "decode": "decode_layer_steps_tokens_per_s",
          "layer": "mamba_layer_fwd_bwd_tokens_per_s"}
SCALING = {"scan_130m": "weak", "pscan": "weak", "decode": "weak", "lshard": "strong", "layer": "weak"}
DTYPE = {"scan_130m": "bf16", "pscan": "f32", "decode": "bf16", "lshard": "bf16", "layer": "bf16"}


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
        return {"workload": "Mamba-2.8b-shaped decode step, 64 layers (conv window + SSM state update + gate per layer)",
                "B_per_gpu": 256, "global_batch": 256 * n, "ED": 5120, "N": 16, "io_dtype": "bf16",
                "state_dtype": "f32", "parallelism": f"batch-sharded x{n}, no collective",
                "l2": "the 64 layers' states (5.4 GB) are walked in turn so every layer-step misses L2"}
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


def roofline_of(res, peaks, peak_kind):
    name, abytes, kms = res["dominant"]
    achieved = abytes / kms / 1e6
    roof = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} copy bandwidth",
            "frac_of_nominal_8TBps": achieved / 8000.0, "traffic": res.get("traffic"),
            "algorithmic_bytes_per_launch": abytes, "kernel_ms": kms}
    if res.get("traffic") is not None:
        roof["traffic_source"] = res.get("traffic_source", "static")
    for k in ("binding", "mufu", "note"):
        if k in res.get("roofline_extra", {}):
            roof[k] = res["roofline_extra"][k]
    return roof


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--regions", type=int, default=5, help="how many times the timed region of --steps steps is repeated")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "scan_130m", "pscan", "decode", "lshard", "layer"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave out the host-buffer leg")
    ap.add_argument("--decode-layers", type=int, default=64, help="layers of the decode workload")
    ap.add_argument("--pscan-batch", type=int, default=16, help="batch rows of the pscan workload (16 = the configuration; smaller for profiler captures)")
    ap.add_argument("--lshard-len", type=int, default=131072, help="sequence length of the lshard workload")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    extras = args.workload == "all"
    if extras:
        args.workload = "scan_130m"

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback "
                         "(use --impl reference for the host-CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import bench_legs as legs
    from mamba_b200 import _lib
    wl = args.workload
    res = getattr(legs, "bench_" + wl)(args, rank, world, dev, Timing)
    peaks, peak_kind = measured_peaks()
    line = {
        "metric": METRIC[wl], "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": SCALING[wl], "vs_baseline": None, "dtype": DTYPE[wl], "reference_dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(wl, world), **({"seq_len": res["seq_len"]} if "seq_len" in res else {}),
                       **({"subshards_per_gpu": res["subshards"]} if "subshards" in res else {})),
        "regions": res.get("regions"),
        "roofline": roofline_of(res, peaks, peak_kind), "kernels": res.get("kernels"),
        "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"], "clocks": res.get("clocks"),
    }
    if wl == "pscan" and args.pscan_batch != 16:
        line["config"].update(B_per_gpu=args.pscan_batch, global_batch=args.pscan_batch * world,
                              l2="reduced batch (profiler capture), still larger than L2")
    if extras:
        # the sequence-sharded scan at every N (its parity self-check first), then the single-GPU summaries
        line["lshard_parity"] = legs.lshard_parity(rank, world, dev)
        ls = legs.bench_lshard(args, rank, world, dev, Timing, summary=True)
        line["lshard"] = {k: ls[k] for k in ("value", "ms_per_step", "regions", "passes_ms", "collective_ms",
                                             "subshards", "seq_len", "kernels") if k in ls}
        line["lshard"].update(unit="tokens/s", scaling="strong",
                              roofline_frac=roofline_of(ls, peaks, peak_kind)["frac"])
        if world == 1:
            for name in ("pscan", "decode"):
                r = getattr(legs, "bench_" + name)(args, rank, world, dev, Timing, summary=True)
                roof = roofline_of(r, peaks, peak_kind)
                line[name] = {"value": r["value"], "unit": "tokens/s", "ms_per_step": r["ms_per_step"],
                              "dtype": DTYPE[name], "kernels": r.get("kernels"),
                              "roofline": {k: roof[k] for k in ("kernel", "achieved", "peak", "frac")}}
            line["b1_long"] = legs.bench_b1_long(args, dev, Timing)
            line["reference_on_gpu"] = legs.reference_on_gpu(dev, reference_scan_fwd_bwd, Timing)
    # a bounded wait that gave up inside a kernel leaves wrong outputs behind without any host-side error:
    # the status word is read here, after the last synchronisation, and a non-zero word fails the run
    status = _lib.device_status(dev)
    line["device_status"] = status
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and wl in CPU_SAMPLES:
            line["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(line))
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    bad = status != 0 or (extras and line["lshard_parity"].get("status") != "ok")
    if bad:
        raise SystemExit(f"bench.py: device status {status}, lshard parity {line.get('lshard_parity')}")


if __name__ == "__main__":
    main()
