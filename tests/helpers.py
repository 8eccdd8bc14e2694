"""Shared helpers of the test-suite: golden loading, seeded inputs, a reference-shaped block."""
import math
import os
import types

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def golden(name):
    return {k: v for k, v in np.load(os.path.join(GOLDEN, name)).items()}


def scan_inputs(seed, Bsz, L, ED, N, dtype=torch.float32, structured_A=True, big_delta=False):
    """Seeded selective-scan inputs with the value distributions of the small CPU config."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Bsz, L, ED, generator=g)
    delta = F.softplus(torch.randn(Bsz, L, ED, generator=g) * 0.5 - (1.0 if big_delta else 4.6))
    if structured_A:
        A = -torch.exp(torch.log(torch.arange(1, N + 1, dtype=torch.float32))).repeat(ED, 1)
    else:
        A = -torch.exp(torch.randn(ED, N, generator=g))
    Bm = torch.randn(Bsz, L, N, generator=g)
    Cm = torch.randn(Bsz, L, N, generator=g)
    D = torch.randn(ED, generator=g)
    z = torch.randn(Bsz, L, ED, generator=g)
    gy = torch.randn(Bsz, L, ED, generator=g)
    cast = lambda t: t.to(dtype).float()          # what the kernel will actually see
    return dict(x=cast(x), delta=cast(delta), A=A, B=cast(Bm), C=cast(Cm), D=D, z=cast(z), gy=cast(gy))


class RefShapedBlock(nn.Module):
    """A module with the attribute names of the reference's MambaBlock (mambapy/mamba.py:127-195),
    so the drop-in `step` / `ssm_step` / `forward` can be bound to it without the reference."""

    def __init__(self, d_model, d_state=16, expand=2, d_conv=4):
        super().__init__()
        ED = expand * d_model
        R = math.ceil(d_model / 16)
        self.config = types.SimpleNamespace(d_model=d_model, d_inner=ED, d_state=d_state,
                                            dt_rank=R, d_conv=d_conv)
        self.in_proj = nn.Linear(d_model, 2 * ED, bias=False)
        self.conv1d = nn.Conv1d(ED, ED, d_conv, bias=True, groups=ED, padding=d_conv - 1)
        self.x_proj = nn.Linear(ED, R + 2 * d_state, bias=False)
        self.dt_proj = nn.Linear(R, ED, bias=True)
        self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32).repeat(ED, 1)))
        self.D = nn.Parameter(torch.ones(ED))
        self.out_proj = nn.Linear(ED, d_model, bias=False)

    def _apply_layernorms(self, dt, B, C):
        return dt, B, C

    def load_golden(self, g, li):
        with torch.no_grad():
            self.in_proj.weight.copy_(torch.from_numpy(g[f"l{li}_in_proj"]))
            self.conv1d.weight.copy_(torch.from_numpy(g[f"l{li}_conv_w"]))
            self.conv1d.bias.copy_(torch.from_numpy(g[f"l{li}_conv_b"]))
            self.x_proj.weight.copy_(torch.from_numpy(g[f"l{li}_x_proj"]))
            self.dt_proj.weight.copy_(torch.from_numpy(g[f"l{li}_dt_w"]))
            self.dt_proj.bias.copy_(torch.from_numpy(g[f"l{li}_dt_b"]))
            self.A_log.copy_(torch.from_numpy(g[f"l{li}_A_log"]))
            self.D.copy_(torch.from_numpy(g[f"l{li}_D"]))
            self.out_proj.weight.copy_(torch.from_numpy(g[f"l{li}_out_proj"]))
        return self

    def weights(self):
        return {"in_proj": self.in_proj.weight, "conv_w": self.conv1d.weight, "conv_b": self.conv1d.bias,
                "x_proj": self.x_proj.weight, "dt_w": self.dt_proj.weight, "dt_b": self.dt_proj.bias,
                "A_log": self.A_log, "D": self.D, "out_proj": self.out_proj.weight}


def assert_close(got, want, rtol, atol, msg=""):
    got = got.detach().float().cpu().numpy() if torch.is_tensor(got) else got
    want = want.detach().float().cpu().numpy() if torch.is_tensor(want) else want
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol, err_msg=msg)


def oracle_f64_blocked(inp, gated=True, bias=None, block=512):
    """Float64 oracle (outputs and every gradient) for WIDE problems: the closed-form forward/backward
    of the oracle, run `block` channels at a time (oracle.selective_scan_fwd_bwd_f64).

    inp: dict of float tensors x, delta, z, gy (B, L, ED), B, C (B, L, N), A (ED, N), D (ED);
    bias (ED) optional: delta is then raw and softplus(delta + bias) is applied by the oracle.
    Returns (y, grads) with grads keyed x, delta, B, C, A, D (and z, bias)."""
    from oracle import scan_oracle as O
    y, _, grads = O.selective_scan_fwd_bwd_f64(inp["x"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"],
                                               inp["gy"], z=inp["z"] if gated else None, delta_bias=bias,
                                               block=block)
    return y, grads
