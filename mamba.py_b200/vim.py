"""Drop-in for the bidirectional block of the reference's Vision Mamba (mambapy/vim.py:205-261).

The reference runs its second direction as flip(xz) -> conv -> projections -> scan -> flip(y).  Here
the second scan walks the ORIGINAL sequence from its last timestep to its first inside the kernels
(`selective_scan_fn(..., reverse=True)`), gated by the un-flipped z, so only the convolution input is
flipped (the convolution kernel is causal); delta, B, C, z and y are never flipped or copied.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .mamba import causal_conv1d_silu, selective_scan_fn


def _conv_silu(conv, xs, L):
    if conv.weight.shape[-1] == 4:
        return causal_conv1d_silu(xs, conv.weight, conv.bias)
    return F.silu(conv(xs.transpose(1, 2))[:, :, :L].transpose(1, 2))


def _ssm(self, x, z, A_log, D, x_proj, dt_proj, reverse):
    """mambapy/vim.py:263-299 with softplus(delta + bias), the scan and the gate in one kernel."""
    cfg = self.config
    A = -torch.exp(A_log.float())
    delta, B, C = torch.split(x_proj(x), [cfg.dt_rank, cfg.d_state, cfg.d_state], dim=-1)
    delta, B, C = self._apply_layernorms(delta, B, C)
    delta = F.linear(delta, dt_proj.weight)
    return selective_scan_fn(x, delta, A, B, C, D, z=z, delta_bias=dt_proj.bias, reverse=reverse)


def forward(self, x):
    """mambapy/vim.py:205-261; x: (B, L, D) -> (B, L, D)."""
    _, L, _ = x.shape
    xz = self.in_proj(x)
    xs, z = xz.chunk(2, dim=-1)
    y = _ssm(self, _conv_silu(self.conv1d, xs, L), z, self.A_log, self.D, self.x_proj, self.dt_proj, False)
    if not self.config.bidirectional:
        return self.out_proj(y)
    # second direction: the reference convolves the flipped sequence; in original time order that is
    # flip(conv(flip(x))).  Everything after it is per-timestep, and the scan runs right to left.
    xb = _conv_silu(self.conv1d_b, xs.flip(1), L).flip(1)
    yb = _ssm(self, xb, z, self.A_log_b, self.D_b, self.x_proj_b, self.dt_proj_b, True)
    s = y + yb
    return self.out_proj(s / 2 if self.config.divide_output else s)
