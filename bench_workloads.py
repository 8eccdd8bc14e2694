"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

No dataset or checkpoint is involved anywhere on this path: the reference's own performance
charts use random tensors.  Every generator takes a seed and a device and returns plain tensors.

  layer_130m_scan_inputs   the tensors a Mamba-130m-shaped layer (d_model 768, ED 1536, N 16,
                           dt_rank 48, d_conv 4) feeds its selective scan, obtained by pushing
                           x ~ N(0,1) of shape (B, L, 768) through randomly initialised
                           in_proj / conv1d / SiLU / x_proj / dt_proj (the reference's init,
                           mambapy/mamba.py:127-172) in bf16
  pscan_inputs             A_in = exp(-softplus(N(0,1))) in (0,1), X_in ~ N(0,1), grad ~ N(0,1)
  long_scan_inputs         the long-sequence config: delta = softplus(N(0,1)*0.5 - 4.6), the rest N(0,1)
  decode_layer_weights     weights and caches of one Mamba-2.8b-shaped layer for step()
  LayerParams              the parameters of one MambaBlock-shaped layer under the reference's
                           attribute names, for timing the whole layer (projections included)
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def s4d_real_A(ED: int, N: int, device) -> torch.Tensor:
    """A = -exp(A_log) with A_log = log(1..N) per channel (mambapy/mamba.py:168-169, :241)."""
    A_log = torch.log(torch.arange(1, N + 1, dtype=torch.float32, device=device)).repeat(ED, 1)
    return -torch.exp(A_log)


def dt_bias_init(ED: int, gen, device, dt_min=1e-3, dt_max=1e-1, floor=1e-4) -> torch.Tensor:
    """Inverse-softplus of dt ~ log-uniform[dt_min, dt_max] (mambapy/mamba.py:158-163)."""
    dt = torch.exp(torch.rand(ED, generator=gen, device=device) * (math.log(dt_max) - math.log(dt_min))
                   + math.log(dt_min)).clamp(min=floor)
    return dt + torch.log(-torch.expm1(-dt))


def layer_130m_scan_inputs(seed: int, device, Bsz=8, L=2048, d_model=768, N=16, d_conv=4,
                           dtype=torch.bfloat16):
    """dict(x, delta_raw, z, B, C, A, D, delta_bias, dy) for the fused scan of one 130m-shaped layer.

    delta_raw is the dt_proj output WITHOUT bias and softplus; the kernel applies
    softplus(delta_raw + delta_bias) itself.  x is post-conv, post-SiLU."""
    gen = torch.Generator(device=device).manual_seed(seed)
    ED, R = 2 * d_model, math.ceil(d_model / 16)
    u = lambda shape, bound: (torch.rand(shape, generator=gen, device=device) * 2 - 1) * bound
    w_in = u((2 * ED, d_model), 1 / math.sqrt(d_model))           # nn.Linear default init range
    w_conv = u((ED, 1, d_conv), 1 / math.sqrt(d_conv))
    b_conv = u((ED,), 1 / math.sqrt(d_conv))
    w_x = u((R + 2 * N, ED), 1 / math.sqrt(ED))
    w_dt = u((ED, R), R ** -0.5)
    bias = dt_bias_init(ED, gen, device)
    inp = torch.randn(Bsz, L, d_model, generator=gen, device=device)
    with torch.no_grad():
        xz = F.linear(inp.to(dtype), w_in.to(dtype))
        x, z = xz.chunk(2, dim=-1)
        x = F.conv1d(x.transpose(1, 2), w_conv.to(dtype), b_conv.to(dtype), padding=d_conv - 1,
                     groups=ED)[:, :, :L].transpose(1, 2)
        x = F.silu(x).contiguous()
        dbc = F.linear(x, w_x.to(dtype))
        dlt, Bm, Cm = torch.split(dbc, [R, N, N], dim=-1)
        delta_raw = F.linear(dlt, w_dt.to(dtype)).contiguous()
        dy = torch.randn(Bsz, L, ED, generator=gen, device=device).to(dtype)
    return dict(x=x, delta_raw=delta_raw, z=z.contiguous(), B=Bm.contiguous(), C=Cm.contiguous(),
                A=s4d_real_A(ED, N, device), D=torch.ones(ED, device=device), delta_bias=bias, dy=dy)


def pscan_inputs(seed: int, device, Bsz=16, L=2048, D=1536, N=16, dtype=torch.float32):
    gen = torch.Generator(device=device).manual_seed(seed)
    shape = (Bsz, L, D, N)
    A = torch.exp(-F.softplus(torch.randn(shape, generator=gen, device=device))).to(dtype)
    X = torch.randn(shape, generator=gen, device=device).to(dtype)
    G = torch.randn(shape, generator=gen, device=device).to(dtype)
    return A, X, G


def long_scan_inputs(seed: int, device, Bsz=1, L=131072, ED=5120, N=16, dtype=torch.bfloat16,
                     t0: int = 0, t1: int | None = None):
    """The long-sequence config, optionally only timesteps [t0, t1) of it.

    Every timestep is generated from its own position-keyed seed block, so a shard produced
    alone is bit-identical to the same rows of the full tensor."""
    t1 = L if t1 is None else t1
    block = 4096
    outs = {k: [] for k in ("x", "delta", "z", "dy", "B", "C")}
    for s in range((t0 // block) * block, t1, block):
        gen = torch.Generator(device=device).manual_seed(seed * 1000003 + s // block)
        n = min(block, L - s)
        x = torch.randn(Bsz, n, ED, generator=gen, device=device)
        d = F.softplus(torch.randn(Bsz, n, ED, generator=gen, device=device) * 0.5 - 4.6)
        z = torch.randn(Bsz, n, ED, generator=gen, device=device)
        dy = torch.randn(Bsz, n, ED, generator=gen, device=device)
        Bm = torch.randn(Bsz, n, N, generator=gen, device=device)
        Cm = torch.randn(Bsz, n, N, generator=gen, device=device)
        lo, hi = max(t0 - s, 0), min(t1 - s, n)
        for k, v in zip(("x", "delta", "z", "dy", "B", "C"), (x, d, z, dy, Bm, Cm)):
            outs[k].append(v[:, lo:hi].to(dtype))
    res = {k: torch.cat(v, dim=1).contiguous() for k, v in outs.items()}
    res["A"] = s4d_real_A(ED, N, device)
    res["D"] = torch.ones(ED, device=device)
    return res


def decode_layer_weights(seed: int, device, d_model=2560, N=16, d_conv=4, dtype=torch.bfloat16):
    """Weights of one Mamba-2.8b-shaped layer (ED 5120, dt_rank 160) with the reference's init."""
    gen = torch.Generator(device=device).manual_seed(seed)
    ED, R = 2 * d_model, math.ceil(d_model / 16)
    u = lambda shape, bound: ((torch.rand(shape, generator=gen, device=device) * 2 - 1) * bound)
    return dict(
        norm_w=torch.ones(d_model, device=device),             # RMSNorm gain, float32 like the kernel takes it
        in_proj=u((2 * ED, d_model), 1 / math.sqrt(d_model)).to(dtype),
        conv_w=u((ED, 1, d_conv), 1 / math.sqrt(d_conv)),      # the kernel takes the filter in float32
        conv_b=u((ED,), 1 / math.sqrt(d_conv)),
        x_proj=u((R + 2 * N, ED), 1 / math.sqrt(ED)).to(dtype),
        dt_w=u((ED, R), R ** -0.5).to(dtype),
        dt_b=dt_bias_init(ED, gen, device),
        A=s4d_real_A(ED, N, device),
        D=torch.ones(ED, device=device),
        out_proj=u((d_model, ED), 1 / math.sqrt(ED)).to(dtype),
    )


class LayerParams(torch.nn.Module):
    """The parameters of one Mamba layer under the attribute names of the reference's MambaBlock
    (mambapy/mamba.py:127-172: in_proj, conv1d, x_proj, dt_proj, A_log, D, out_proj, config), with its
    initialisation (dt bias inverse-softplus of log-uniform dt, S4D-real A).  It holds parameters only;
    `mamba_b200.mamba.forward(params, x)` runs the layer."""

    def __init__(self, seed: int, device, d_model=768, N=16, d_conv=4, expand=2):
        super().__init__()
        import types
        nn = torch.nn
        ED, R = expand * d_model, math.ceil(d_model / 16)
        self.config = types.SimpleNamespace(d_model=d_model, d_inner=ED, dt_rank=R, d_state=N, d_conv=d_conv)
        gen = torch.Generator(device=device).manual_seed(seed)
        u = lambda shape, bound: (torch.rand(shape, generator=gen, device=device) * 2 - 1) * bound
        self.in_proj = nn.Linear(d_model, 2 * ED, bias=False, device=device)
        self.conv1d = nn.Conv1d(ED, ED, d_conv, groups=ED, padding=d_conv - 1, bias=True, device=device)
        self.x_proj = nn.Linear(ED, R + 2 * N, bias=False, device=device)
        self.dt_proj = nn.Linear(R, ED, bias=True, device=device)
        self.out_proj = nn.Linear(ED, d_model, bias=False, device=device)
        with torch.no_grad():
            self.in_proj.weight.copy_(u((2 * ED, d_model), 1 / math.sqrt(d_model)))
            self.conv1d.weight.copy_(u((ED, 1, d_conv), 1 / math.sqrt(d_conv)))
            self.conv1d.bias.copy_(u((ED,), 1 / math.sqrt(d_conv)))
            self.x_proj.weight.copy_(u((R + 2 * N, ED), 1 / math.sqrt(ED)))
            self.dt_proj.weight.copy_(u((ED, R), R ** -0.5))
            self.dt_proj.bias.copy_(dt_bias_init(ED, gen, device))
            self.out_proj.weight.copy_(u((d_model, ED), 1 / math.sqrt(ED)))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, N + 1, dtype=torch.float32, device=device)).repeat(ED, 1))
        self.D = nn.Parameter(torch.ones(ED, device=device))
        self.norm_weight = nn.Parameter(torch.ones(d_model, device=device))     # RMSNorm in front of the block

    def _apply_layernorms(self, dt, B, C):
        return dt, B, C
