"""GPU legs of bench.py for the decode and the sequence-sharded workloads.

Kept inside the package so that bench.py stays a thin driver; the timing helpers are passed in by
bench.py (one definition of "timed region" for every workload).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import workloads
from .mamba import ssm_step_fn, conv_step_fn, sscan_fwd_raw, sscan_bwd_raw, rms_norm


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


def bench_decode(args, rank, world, dev, ClockSampler, time_region, time_kernel):
    """Batched decode, Mamba-2.8b shape: 64 layers, B = 256 single-token inputs per step.

    A "step" is one token for the whole batch through all 64 layers (the reference's Mamba.step),
    replayed from one CUDA graph; tokens/s = 256 * steps / time."""
    n_layers = int(os.environ.get("MB200_DECODE_LAYERS", "64"))
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
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        ms, t_lo, t_hi = time_region(graph.replay, args.steps, world)
        res = {"value": Bsz * world * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
               "gpu_launches": 2 * n_layers * args.steps}

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
            ms, mn = time_kernel(g.replay, 8)
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
        ems, _, _ = time_region(e2e_step, k_e2e, world)
        sampler.stop()
        nbytes = x_in.numel() * x_in.element_size()
        res["e2e"] = {"value": Bsz * world * k_e2e / (ems * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "steps": k_e2e,
                      "ms_per_step": ems / k_e2e}
        res["clocks"] = sampler.summary(t_lo, t_hi)
        res["n_layers"] = n_layers
    return res


# ---------------------------------------------------------------------------- sequence sharding
def bench_lshard(args, rank, world, dev, ClockSampler, time_region, time_kernel):
    """Long sequence split over the ranks along L; fwd+bwd with the carry exchange (strong scaling)."""
    import torch.distributed as dist
    from .lshard import selective_scan_lsharded, pick_subshards, _split
    L = int(os.environ.get("MB200_LSHARD_L", "131072"))
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
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms, t_lo, t_hi = time_region(step, args.steps, world)
    res = {"value": Bsz * L * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
           "gpu_launches": 8 * args.steps, "seq_len": L}

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
    fwd_ms, fwd_min = time_kernel(fwd, 5)
    bwd_ms, bwd_min = time_kernel(bwd, 5)
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

    if not args.skip_e2e:
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
        ems, _, _ = time_region(e2e_step, 3, world)
        res["e2e"] = {"value": n * world * 3 / (ems * 1e-3), "unit": "tokens/s",
                      "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in.values()),
                      "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in host_out),
                      "steps": 3, "ms_per_step": ems / 3,
                      "note": f"first {n} timesteps of each rank's shard per step"}
    return res


def bench_layer(args, rank, world, dev, ClockSampler, time_region, time_kernel):
    """One whole Mamba-130m-shaped residual layer (mambapy/mamba.py:111), forward + backward, bf16 autocast
    with float32 scan state: RMSNorm kernel, in_proj, conv1d+SiLU kernel, x_proj, dt_proj, fused scan
    (softplus, gate inside), out_proj, residual add.  The four projections are library GEMMs; the line
    reports how the step splits."""
    from . import mamba as M
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
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms, t_lo, t_hi = time_region(step, args.steps, world)
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
    fwd_ms, fwd_min = time_kernel(fwd, 20)
    bwd_ms, bwd_min = time_kernel(bwd, 20)
    conv_ms, conv_min = time_kernel(conv_fb, 20)
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
