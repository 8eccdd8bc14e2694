"""Selective scan with the SEQUENCE split over the ranks of a process group (one GPU each).

The reference is single-device; this is the sequence-sharded form of MambaBlock.selective_scan
(mambapy/mamba.py:274-295) plus its gate, and must reproduce the single-device result on the
concatenated sequence.  Rank r holds timesteps [r*L/R, (r+1)*L/R) of every (B, L, .) tensor.
The protocol (carry pass, all_gather of the carries, fold, full pass; mirrored in the backward, then an
all_reduce of the parameter gradients) is split.py's; this file binds it to a process group and autograd.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .kernels import _rows, _f32, _act_dtype, _require_cuda
from .split import (CudaOps, _gather, _split, _merge, pick_subshards,     # noqa: F401  (re-exported)
                    split_forward as sharded_forward, split_backward as sharded_backward)


class LShardSelectiveScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, A, Bm, Cm, D, z, delta_bias, group):
        _require_cuda(x, delta, A, Bm, Cm, D, z, delta_bias)
        dt = _act_dtype(x, delta, z, Bm, Cm)
        xs, ds, zs = _rows(x, dt), _rows(delta, dt), _rows(z, dt)
        Bs, Cs = _rows(Bm, dt), _rows(Cm, dt)
        A32, D32, b32 = _f32(A), _f32(D), _f32(delta_bias)
        needs_grad = any(t is not None and t.requires_grad for t in (x, delta, A, Bm, Cm, D, z, delta_bias))
        S = pick_subshards(xs.shape[0], xs.shape[1], xs.shape[2], dist.get_world_size(group))
        y, h_in, P_all, carries, _ = sharded_forward(CudaOps, group, xs, ds, A32, Bs, Cs, D32, zs, b32,
                                                     want_carries=needs_grad, subshards=S)
        ctx.group, ctx.subshards = group, S
        ctx.save_for_backward(xs, ds, A32, Bs, Cs, D32, zs, b32, carries, P_all)
        ctx.in_dtypes = tuple(None if t is None else t.dtype for t in (x, delta, A, Bm, Cm, D, z, delta_bias))
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, ds, A32, Bs, Cs, D32, zs, b32, carries, P_all = ctx.saved_tensors
        dy = _rows(dy, xs.dtype)
        dx, dd, dz, dB, dC, dA, dD, dbias, _ = sharded_backward(
            CudaOps, ctx.group, xs, ds, A32, Bs, Cs, D32, zs, b32, dy, carries, P_all, subshards=ctx.subshards)
        tx, td, tA, tB, tC, tD, tz, tb = ctx.in_dtypes
        cast = lambda g, t: None if (g is None or t is None) else g.to(t)
        return (cast(dx, tx), cast(dd, td), cast(dA, tA), cast(dB, tB), cast(dC, tC), cast(dD, tD),
                cast(dz, tz), cast(dbias, tb), None)


def selective_scan_lsharded(x, delta, A, B, C, D=None, z=None, delta_bias=None, group=None):
    """Fused selective scan of THIS RANK'S slice of the sequence; ranks hold consecutive slices.

    Same arguments as `selective_scan_fn`, each (B, L/R, .) tensor being the local slice.  The
    parameter gradients (A, D, delta_bias) come back summed over all ranks."""
    if group is None:
        group = dist.group.WORLD
    return LShardSelectiveScanFn.apply(x, delta, A, B, C, D, z, delta_bias, group)
