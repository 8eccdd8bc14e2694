"""GPU legs of bench.py: one function per workload, each returning a dict of results.

bench.py owns the command line, the JSON line and the timing helpers (passed in as `T`, so there is one
definition of "timed region"); this file owns what is launched.  With `summary=True` a leg skips its
host-buffer (end-to-end) part: bench.py's default run uses that for the secondary workloads.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

import bench_workloads as workloads
from mamba_b200.mamba import ssm_step_fn, conv_step_fn, sscan_fwd_raw, sscan_bwd_raw, rms_norm

MUFU_PER_CLK_PER_SM = 16          # ex2 results per clock and SM on sm_100
BWD_TRAFFIC_BYTES_130M = 538.6e6  # DRAM read + write bytes of one backward launch on the 130m workload (ncu)


def _sm_count_and_clock(dev):
    p = torch.cuda.get_device_properties(dev)
    return p.multi_processor_count, p.clock_rate * 1e3 if hasattr(p, "clock_rate") else 1.965e9


def mufu_floor_ms(elements, ex2_per_element, dev):
    """Time the ex2 evaluations of a scan over `elements` (b, t, e, n) items need on the MUFU pipe alone
    (16 results per clock and SM) at the device's maximum SM clock."""
    sms, hz = _sm_count_and_clock(dev)
    return elements * ex2_per_element / (sms * MUFU_PER_CLK_PER_SM * hz) * 1e3

# ----------------------------------------------------------------------------------- decode
def decode_layer_step(W, x, h, win):
    """One ResidualBlock.step (mambapy/mamba.py:114-125, :351-382) on explicit weights, with the
    caches updated in place.  x: (B, D); h: (B, ED, N) f32; win: (B, ED, d_conv-1)."""
    R = W["dt_w"].shape[1]
    N = W["A"].shape[1]
    xz = F.linear(rms_norm(x, W["norm_w"], 1e-5), W["in_proj"])
    xs, z = xz.chunk(2, dim=1)
    xc, _ = conv_step_fn(xs, win, W["conv_w"], W["conv_b"], inplace=True)
    dbc = F.linear(xc, W["x_proj"])
    dlt, Bm, Cm = torch.split(dbc, [R, N, N], dim=-1)
    dlt = F.linear(dlt, W["dt_w"])
    y, _ = ssm_step_fn(xc, h, dlt, W["A"], Bm, Cm, W["D"], z=z, delta_bias=W["dt_b"], inplace=True)
    return F.linear(y, W["out_proj"]) + x


def bench_decode(args, rank, world, dev, T, summary=False):
    """Batched decode, Mamba-2.8b shape: 64 layers, B = 256 single-token inputs per step.

    A "step" is one token for the whole batch through all 64 layers (the reference's Mamba.step),
    replayed from one CUDA graph; tokens/s = 256 * steps / time."""
    n_layers = args.decode_layers
    Bsz, Dm, ED, N, K = 256, 2560, 5120, 16, 4
    Ws = [workloads.decode_layer_weights(1003 + i, dev) for i in range(n_layers)]
    gen = torch.Generator(device=dev).manual_seed(1003 + 1000 * rank)
    hs = [torch.randn(Bsz, ED, N, generator=gen, device=dev) for _ in range(n_layers)]
    wins = [torch.randn(Bsz, ED, K - 1, generator=gen, device=dev).bfloat16() for _ in range(n_layers)]
    x_in = torch.randn(Bsz, Dm, generator=gen, device=dev).bfloat16()
    out = torch.empty_like(x_in)

    def model_step():
        x = x_in
        for W, h, win in zip(Ws, hs, wins):
            x = decode_layer_step(W, x, h, win)
        out.copy_(x)

    with torch.no_grad():
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                model_step()
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            model_step()

        for _ in range(max(args.warmup, 3)):
            graph.replay()
        sampler = T.ClockSampler(dev.index or 0)
        sampler.start()
        steps = min(args.steps, 20) if summary else args.steps
        ms, t_lo, t_hi = T.time_region(graph.replay, steps, world)
        res = {"value": Bsz * world * steps / (ms * 1e-3), "ms_per_step": ms / steps,
               "gpu_launches": 2 * n_layers * steps}

        # the state-update kernel alone, cycling over the layers' states so every launch misses L2
        W0 = Ws[0]
        xc = torch.randn(Bsz, ED, generator=gen, device=dev).bfloat16()
        dlt = torch.randn(Bsz, ED, generator=gen, device=dev).bfloat16()
        zz = torch.randn(Bsz, ED, generator=gen, device=dev).bfloat16()
        Bm = torch.randn(Bsz, N, generator=gen, device=dev).bfloat16()
        Cm = torch.randn(Bsz, N, generator=gen, device=dev).bfloat16()
        it = {"i": 0}

        def one():
            i = it["i"] = (it["i"] + 1) % n_layers
            ssm_step_fn(xc, hs[i], dlt, W0["A"], Bm, Cm, W0["D"], z=zz, delta_bias=W0["dt_b"], inplace=True)

        xs_raw = torch.randn(Bsz, ED, generator=gen, device=dev).bfloat16()

        def conv_one():
            i = it["i"] = (it["i"] + 1) % n_layers
            conv_step_fn(xs_raw, wins[i], W0["conv_w"], W0["conv_b"], inplace=True)

        for _ in range(4):
            one()
            conv_one()

        def graph_time(fn, launches):
            """Device time per launch with the host out of the way: `launches` calls in one CUDA graph."""
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                fn()
            torch.cuda.current_stream().wait_stream(st)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(launches):
                    fn()
            g.replay()
            ms, mn = T.time_kernel(g.replay, 8)
            return ms / launches, mn / launches

        k_ms, k_min = graph_time(one, n_layers)
        c_ms, c_min = graph_time(conv_one, n_layers)
        state_bytes = 2 * Bsz * ED * N * 4 + 4 * Bsz * ED * 2 + 2 * Bsz * N * 2
        conv_bytes = 2 * Bsz * ED * (K - 1) * 2 + 2 * Bsz * ED * 2
        res["kernels"] = {
            "ssm_step_kernel": {"ms": k_ms, "ms_min": k_min, "algorithmic_bytes": state_bytes,
                                "GBps": state_bytes / k_ms / 1e6},
            "conv_step_kernel": {"ms": c_ms, "ms_min": c_min, "algorithmic_bytes": conv_bytes,
                                 "GBps": conv_bytes / c_ms / 1e6},
        }
        res["dominant"] = ("ssm_step_kernel", state_bytes, k_ms)
        res["n_layers"] = n_layers
        if summary:
            sampler.stop()
            res["clocks"] = sampler.summary(t_lo, t_hi)
            return res

        # end to end: the token batch comes from pinned host memory, the hidden output goes back
        hx = x_in.cpu().pin_memory()
        hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()

        def e2e_step():
            x_in.copy_(hx, non_blocking=True)
            graph.replay()
            hout.copy_(out, non_blocking=True)

        for _ in range(2):
            e2e_step()
        k_e2e = max(3, min(args.steps, 20))
        ems, _, _ = T.time_region(e2e_step, k_e2e, world)
        sampler.stop()
        nbytes = x_in.numel() * x_in.element_size()
        res["e2e"] = {"value": Bsz * world * k_e2e / (ems * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "steps": k_e2e,
                      "ms_per_step": ems / k_e2e}
        res["clocks"] = sampler.summary(t_lo, t_hi)
    return res


# ---------------------------------------------------------------------------- sequence sharding
def _lshard_pass_times(step, n):
    """Run `step` n times with every shard-local pass (methods of split.CudaOps) and every collective
    of the sequence-sharded scan bracketed by its own CUDA events.  Returns ({pass: ms per step},
    ms per step spent in collectives); this rank's numbers, taken outside the timed regions."""
    import torch.distributed as dist
    from mamba_b200 import split
    rec = []

    def timed(name, fn):
        def wrapped(*a, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **k)
            e1.record()
            rec.append((name, e0, e1))
            return out
        return wrapped

    saved = []
    for name, attr in list(vars(split.CudaOps).items()):
        if isinstance(attr, staticmethod):
            saved.append((split.CudaOps, name, attr))
            setattr(split.CudaOps, name, staticmethod(timed(name, attr.__func__)))
    saved.append((split, "_gather", split._gather))
    split._gather = timed("all_gather", split._gather)
    saved.append((dist, "all_reduce", dist.all_reduce))
    dist.all_reduce = timed("all_reduce", dist.all_reduce)
    try:
        for _ in range(n):
            step()
        torch.cuda.synchronize()
    finally:
        for obj, name, old in saved:
            setattr(obj, name, old)
    tot = {}
    for name, e0, e1 in rec:
        tot[name] = tot.get(name, 0.0) + e0.elapsed_time(e1) / n
    coll = sum(v for k, v in tot.items() if k in ("all_gather", "all_reduce"))
    return {k: v for k, v in tot.items() if k not in ("all_gather", "all_reduce")}, coll


def lshard_parity(rank, world, dev):
    """Self-check run before the sequence-sharded benchmark, at every N: a short sequence (L = 4096,
    ED = 256, bf16) through the SAME sharded code path (NCCL collectives when N > 1, sub-shards when
    N = 1) against the single-launch scan of the whole sequence on rank 0.  Returns the largest
    deviations and "ok" / "MISMATCH"; bench.py fails the run on a mismatch."""
    import torch.distributed as dist
    import mamba_b200
    from mamba_b200.lshard import selective_scan_lsharded
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    L, ED, N = 4096, 256, 16
    Ls = L // world
    full = workloads.long_scan_inputs(77, dev, 1, L, ED, N)
    sl = lambda k: full[k][:, rank * Ls:(rank + 1) * Ls].contiguous()
    lv = {k: sl(k).requires_grad_() for k in ("x", "delta", "z", "B", "C")}
    A, D = full["A"].clone().requires_grad_(), full["D"].clone().requires_grad_()
    y = selective_scan_lsharded(lv["x"], lv["delta"], A, lv["B"], lv["C"], D, z=lv["z"])
    y.backward(sl("dy"))

    def gathered(t):
        if world == 1:
            return t
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t.contiguous())
        return torch.cat(out, dim=1)

    got = {"y": gathered(y.detach()), "dx": gathered(lv["x"].grad), "ddelta": gathered(lv["delta"].grad),
           "dz": gathered(lv["z"].grad), "dB": gathered(lv["B"].grad), "dC": gathered(lv["C"].grad),
           "dA": A.grad, "dD": D.grad}
    out = {"status": "ok", "L": L, "ED": ED, "ranks": world}
    if rank == 0:
        rl = {k: full[k].clone().requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}
        yr = mamba_b200.selective_scan_fn(rl["x"], rl["delta"], rl["A"], rl["B"], rl["C"], rl["D"], z=rl["z"])
        yr.backward(full["dy"])
        want = {"y": yr.detach(), "dx": rl["x"].grad, "ddelta": rl["delta"].grad, "dz": rl["z"].grad,
                "dB": rl["B"].grad, "dC": rl["C"].grad, "dA": rl["A"].grad, "dD": rl["D"].grad}
        errs = {}
        for k, wv in want.items():
            g, wv = got[k].float(), wv.float()
            scale = max(1.0, wv.abs().max().item())
            errs[k] = ((g - wv).abs() / (2e-2 * wv.abs() + 2e-2 * scale)).max().item()   # 1.0 = at tolerance
        out["max_error_over_tolerance"] = errs
        if not all(v <= 1.0 for v in errs.values()):
            out["status"] = "MISMATCH"
    if world > 1:
        flag = torch.tensor([1.0 if out["status"] == "ok" else 0.0], device=dev)
        dist.broadcast(flag, 0)
        if flag.item() == 0.0:
            out["status"] = "MISMATCH"
    return out


def bench_b1_long(args, dev, T):
    """Batch 1, d_model 1024 (ED 2048, N 16), L = 2048 and 65536: the shapes the reference publishes its
    own fwd+bwd times for.  Fused scan (gated, bf16 I/O) forward + backward through the public API."""
    import mamba_b200
    out = {}
    for L in (2048, 65536):
        w = workloads.long_scan_inputs(1005, dev, 1, L, 2048, 16)
        lv = {k: w[k].requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}

        def step():
            for t in lv.values():
                t.grad = None
            y = mamba_b200.selective_scan_fn(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"])
            y.backward(w["dy"])

        for _ in range(3):
            step()
        steps = 20 if L == 2048 else 5
        ms, _, _ = T.time_region(step, steps, 1)
        out[f"L{L}"] = {"ms_per_step": ms / steps, "value": L * steps / (ms * 1e-3), "unit": "tokens/s",
                        "shape": f"B=1, L={L}, ED=2048, N=16, bf16, gated, fwd+bwd"}
    return out


def reference_on_gpu(dev, builder, T):
    """The reference's own parallel-scan path (float32, PyTorch ops) on this same GPU, on the headline
    shape (B = 8, L = 2048, ED = 1536, N = 16).  A second comparison; the contract baseline is the CPU arm."""
    try:
        step, kind = builder(Bsz=8, L=2048, ED=1536, N=16, seed=1002, device=dev)
        for _ in range(2):
            step()
        ms, _, _ = T.time_region(step, 3, 1)
        out = {"value": 8 * 2048 * 3 / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms / 3, "kind": kind,
               "dtype": "f32", "what": "selective_scan (pscan route) + gate, fwd+bwd, torch ops on the GPU"}
    except torch.cuda.OutOfMemoryError as e:                      # the reference materialises (B, L, ED, N) tensors
        out = {"unavailable": f"out of memory: {str(e)[:80]}"}
    torch.cuda.empty_cache()
    return out


def bench_lshard(args, rank, world, dev, T, summary=False):
    """Long sequence split over the ranks along L; fwd+bwd with the carry exchange (strong scaling)."""
    import torch.distributed as dist
    from mamba_b200.lshard import selective_scan_lsharded, pick_subshards, _split
    L = args.lshard_len
    Bsz, ED, N = 1, 5120, 16
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    Ls = L // world
    w = workloads.long_scan_inputs(1004, dev, Bsz, L, ED, N, t0=rank * Ls, t1=(rank + 1) * Ls)
    leaves = {k: w[k].requires_grad_() for k in ("x", "delta", "z", "B", "C", "A", "D")}

    def step():
        for t in leaves.values():
            t.grad = None
        y = selective_scan_lsharded(leaves["x"], leaves["delta"], leaves["A"], leaves["B"], leaves["C"],
                                    leaves["D"], z=leaves["z"])
        y.backward(w["dy"])

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = T.ClockSampler(dev.index or 0)
    sampler.start()
    steps = min(args.steps, 10) if summary else args.steps
    ms, all_ms, t_lo, t_hi = T.time_regions(step, steps, world, 3 if summary else args.regions)
    res = {"value": Bsz * L * steps / (ms * 1e-3), "ms_per_step": ms / steps,
           "gpu_launches": 8 * steps * len(all_ms), "seq_len": L,
           "regions": {"n": len(all_ms), "steps_each": steps, "ms_per_step_median": ms / steps,
                       "ms_per_step_min": min(all_ms) / steps, "ms_per_step_max": max(all_ms) / steps}}
    # where the step goes: every pass and every collective of three more steps, timed with events
    passes, coll = _lshard_pass_times(step, 3)
    res["passes_ms"], res["collective_ms"] = passes, coll

    # the two big kernels alone, on the sub-sharded view the sharded scan really launches
    S = pick_subshards(Bsz, Ls, ED, world)
    d = {k: w[k].detach() for k in ("A", "D")}
    d.update({k: _split(w[k].detach(), S) for k in ("x", "delta", "z", "B", "C", "dy")})
    res["subshards"] = S
    keep = {}

    def fwd():
        keep["o"] = sscan_fwd_raw(d["x"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["z"], want_carries=True)

    fwd()

    def bwd():
        keep["g"] = sscan_bwd_raw(d["x"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["z"], None, d["dy"],
                                  keep["o"][2])

    for f in (fwd, bwd, fwd, bwd):
        f()
    fwd_ms, fwd_min = T.time_kernel(fwd, 5)
    bwd_ms, bwd_min = T.time_kernel(bwd, 5)
    sampler.stop()
    fwd_bytes = (4 * ED + 2 * N) * 2 * Bsz * Ls
    bwd_bytes = (7 * ED + 4 * N) * 2 * Bsz * Ls
    res["kernels"] = {
        "sscan_fwd_kernel": {"ms": fwd_ms, "ms_min": fwd_min, "algorithmic_bytes": fwd_bytes,
                             "GBps": fwd_bytes / fwd_ms / 1e6},
        "sscan_bwd_kernel": {"ms": bwd_ms, "ms_min": bwd_min, "algorithmic_bytes": bwd_bytes,
                             "GBps": bwd_bytes / bwd_ms / 1e6},
    }
    res["dominant"] = ("sscan_bwd_kernel", bwd_bytes, bwd_ms)
    res["clocks"] = sampler.summary(t_lo, t_hi)

    if not (args.skip_e2e or summary):
        # end to end on a bounded slice of the shard (the whole shard would pin > 10 GB of host memory)
        n = min(Ls, 16384)
        host_in = {k: w[k].detach()[:, :n].cpu().pin_memory() for k in ("x", "delta", "z", "B", "C", "dy")}
        dev_in = {k: torch.empty_like(w[k].detach()[:, :n]) for k in host_in}
        host_out = []

        def e2e_step():
            for k in host_in:
                dev_in[k].copy_(host_in[k], non_blocking=True)
            lv = {k: dev_in[k].requires_grad_() for k in ("x", "delta", "z", "B", "C")}
            for t in lv.values():
                t.grad = None
            y = selective_scan_lsharded(lv["x"], lv["delta"], d["A"], lv["B"], lv["C"], d["D"], z=lv["z"])
            y.backward(dev_in["dy"])
            outs = [y.detach()] + [lv[k].grad for k in ("x", "delta", "z", "B", "C")]
            if not host_out:
                host_out.extend(torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs)
            for h, o in zip(host_out, outs):
                h.copy_(o, non_blocking=True)
            for k in lv:
                dev_in[k].requires_grad_(False)

        for _ in range(2):
            e2e_step()
        ems, _, _ = T.time_region(e2e_step, 3, world)
        res["e2e"] = {"value": n * world * 3 / (ems * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in.values()),
                      "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in host_out),
                      "steps": 3, "ms_per_step": ems / 3,
                      "note": f"first {n} timesteps of each rank's shard per step"}
    return res


def bench_layer(args, rank, world, dev, T, summary=False):
    """One whole Mamba-130m-shaped residual layer (mambapy/mamba.py:111), forward + backward, bf16 autocast
    with float32 scan state: RMSNorm kernel, in_proj, conv1d+SiLU kernel, x_proj, dt_proj, fused scan
    (softplus, gate inside), out_proj, residual add.  The four projections are library GEMMs; the line
    reports how the step splits."""
    from mamba_b200 import mamba as M
    Bsz, L, d_model = 8, 2048, 768
    layer = workloads.LayerParams(1002 + rank, dev, d_model=d_model)
    gen = torch.Generator(device=dev).manual_seed(77 + rank)
    x = torch.randn(Bsz, L, d_model, generator=gen, device=dev).requires_grad_()
    dy = torch.randn(Bsz, L, d_model, generator=gen, device=dev)
    params = list(layer.parameters())

    def step():
        x.grad = None
        for q in params:
            q.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = M.forward(layer, M.rms_norm(x, layer.norm_weight, 1e-5)) + x
        y.backward(dy.to(y.dtype))

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = T.ClockSampler(dev.index or 0)
    sampler.start()
    ms, t_lo, t_hi = T.time_region(step, args.steps, world)
    res = {"value": Bsz * L * world * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
           "gpu_launches": 4 * args.steps}

    # the library's own kernels alone, on the tensors the layer really feeds them
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        xz = layer.in_proj(M.rms_norm(x, layer.norm_weight, 1e-5))
        xs, z = xz.chunk(2, dim=-1)
        xc = M.causal_conv1d_silu(xs, layer.conv1d.weight, layer.conv1d.bias)
        dlt, Bm, Cm = M._project(layer, xc)
        draw = torch.nn.functional.linear(dlt, layer.dt_proj.weight)
    A = -torch.exp(layer.A_log.detach().float())
    D, bias = layer.D.detach().float(), layer.dt_proj.bias.detach().float()
    gy = torch.randn(Bsz, L, 2 * d_model, generator=gen, device=dev).to(torch.bfloat16)
    keep = {}

    def fwd():
        keep["o"] = M.sscan_fwd_raw(xc, draw, A, Bm, Cm, D, z, bias, want_carries=True)

    fwd()

    def bwd():
        keep["g"] = M.sscan_bwd_raw(xc, draw, A, Bm, Cm, D, z, bias, gy, keep["o"][2])

    xs_leaf = xs.detach().requires_grad_()

    def conv_fb():
        xs_leaf.grad = None
        M.causal_conv1d_silu(xs_leaf, layer.conv1d.weight.detach(), layer.conv1d.bias.detach()).backward(gy)

    for f in (fwd, bwd, conv_fb, fwd, bwd, conv_fb):
        f()
    fwd_ms, fwd_min = T.time_kernel(fwd, 20)
    bwd_ms, bwd_min = T.time_kernel(bwd, 20)
    conv_ms, conv_min = T.time_kernel(conv_fb, 20)
    sampler.stop()
    ED, N = 2 * d_model, 16
    fwd_bytes = (4 * ED + 2 * N) * 2 * Bsz * L
    bwd_bytes = (7 * ED + 4 * N) * 2 * Bsz * L
    res["kernels"] = {
        "sscan_fwd_kernel": {"ms": fwd_ms, "ms_min": fwd_min, "algorithmic_bytes": fwd_bytes,
                             "GBps": fwd_bytes / fwd_ms / 1e6},
        "sscan_bwd_kernel": {"ms": bwd_ms, "ms_min": bwd_min, "algorithmic_bytes": bwd_bytes,
                             "GBps": bwd_bytes / bwd_ms / 1e6},
        "conv1d_silu_fwd+bwd": {"ms": conv_ms, "ms_min": conv_min},
        # what is left of the step once the library's own kernels are taken out (their fastest timings:
        # a median can be inflated by host-side stalls between launches)
        "projections_and_glue": {"ms": ms / args.steps - fwd_min - bwd_min - conv_min},
    }
    res["dominant"] = ("sscan_bwd_kernel", bwd_bytes, bwd_ms)
    res["clocks"] = sampler.summary(t_lo, t_hi)
    return res


# ----------------------------------------------------------------------------------- fused scan, PScan
def bench_scan_130m(args, rank, world, dev, T, summary=False):
    import mamba_b200
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
    sampler = T.ClockSampler(dev.index or 0)
    sampler.start()
    ms, all_ms, t_lo, t_hi = T.time_regions(step, args.steps, world, args.regions)
    tokens = Bsz * L * world
    # launches of this library's kernels per step: forward, zero-fill of the gradient accumulators, backward
    res = {"value": tokens * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
           "gpu_launches": 2 * args.steps * len(all_ms),
           "regions": {"n": len(all_ms), "steps_each": args.steps, "ms_per_step_median": ms / args.steps,
                       "ms_per_step_min": min(all_ms) / args.steps, "ms_per_step_max": max(all_ms) / args.steps}}

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
    fwd_ms, fwd_min = T.time_kernel(fwd, 20)
    bwd_ms, bwd_min = T.time_kernel(bwd, 20)
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
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of that kernel on this exact workload: a
    # figure from an ncu capture of the same kernel, typed in here (the run that prints it does not measure it)
    res["traffic"] = BWD_TRAFFIC_BYTES_130M
    res["traffic_source"] = "static: ncu capture of one launch of this kernel on this workload"
    # The fused kernels are bound by arithmetic, not HBM: one ex2 per (b, t, e, n) element forward, two
    # backward (the decay is evaluated again in the reverse walk), plus 4 resp. 6 per (b, t, e) for
    # softplus and the gate.  The second entry is the time those evaluations alone need.
    elems = Bsz * L * ED * N
    fl_f = mufu_floor_ms(elems, 1 + 4 / N, dev)
    fl_b = mufu_floor_ms(elems, 2 + 6 / N, dev)
    res["roofline_extra"] = {
        "binding": "shared-memory pipe, then MUFU (ex2); DRAM is under 15 % busy in the ncu captures",
        "mufu": {"bound": "mufu", "unit": "ms", "floor_ms": {"fwd": fl_f, "bwd": fl_b, "step": fl_f + fl_b},
                 "frac": {"fwd": fl_f / fwd_ms, "bwd": fl_b / bwd_ms, "step": (fl_f + fl_b) / (fwd_ms + bwd_ms)},
                 "how": "ex2 evaluations / (SMs * 16 per clock * max SM clock)"}}

    if args.skip_e2e or summary:
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
    ems, _, _ = T.time_region(e2e_step, k_e2e, world, finish=e2e_finish)
    sampler.stop()
    host_out = slots[0]["host"]
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    res["e2e"] = {"value": tokens * k_e2e / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                  "d2h_bytes_per_step": d2h, "steps": k_e2e, "ms_per_step": ems / k_e2e}
    res["clocks"] = sampler.summary(t_lo, t_hi)
    return res


def bench_pscan(args, rank, world, dev, T, summary=False):
    import mamba_b200
    from mamba_b200.pscan import pscan_fwd_raw, pscan_bwd_raw
    Bsz, L, D, N = getattr(args, "pscan_batch", 16), 2048, 1536, 16
    A, X, G = workloads.pscan_inputs(1001 + rank, dev, Bsz, L, D, N)
    A.requires_grad_()
    X.requires_grad_()

    def step():
        A.grad = None
        X.grad = None
        mamba_b200.pscan(A, X).backward(G)

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = T.ClockSampler(dev.index or 0)
    sampler.start()
    steps = min(args.steps, 10) if summary else args.steps          # one step moves 25.8 GB
    ms, t_lo, t_hi = T.time_region(step, steps, world)
    tokens = Bsz * L * world
    res = {"value": tokens * steps / (ms * 1e-3), "ms_per_step": ms / steps, "gpu_launches": 2 * steps}
    Ad, Xd = A.detach(), X.detach()
    keep = {}

    def fwd():
        keep["H"] = pscan_fwd_raw(Ad, Xd)[0]

    fwd()

    def bwd():
        keep["g"] = pscan_bwd_raw(Ad, keep["H"], G)

    for f in (fwd, bwd, fwd, bwd):
        f()
    fwd_ms, fwd_min = T.time_kernel(fwd, 10)
    bwd_ms, bwd_min = T.time_kernel(bwd, 10)
    sampler.stop()
    elems = Bsz * L * D * N
    res["kernels"] = {
        "pscan_fwd_kernel": {"ms": fwd_ms, "ms_min": fwd_min, "algorithmic_bytes": 3 * elems * 4,
                             "GBps": 3 * elems * 4 / fwd_ms / 1e6},
        "pscan_bwd_kernel": {"ms": bwd_ms, "ms_min": bwd_min, "algorithmic_bytes": 5 * elems * 4,
                             "GBps": 5 * elems * 4 / bwd_ms / 1e6},
    }
    res["dominant"] = ("pscan_bwd_kernel", 5 * elems * 4, bwd_ms)
    if summary:
        res["clocks"] = sampler.summary(t_lo, t_hi)
        return res
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
    ems, _, _ = T.time_region(e2e_step, k_e2e, world)
    per = L * D * N * 4
    res["e2e"] = {"value": L * world * k_e2e / (ems * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 3 * per,
                  "d2h_bytes_per_step": 3 * per, "steps": k_e2e, "ms_per_step": ems / k_e2e,
                  "note": "one batch row per step (B=1 of 16): the full batch would move 12.9 GB over PCIe"}
    res["clocks"] = sampler.summary(t_lo, t_hi)
    return res


