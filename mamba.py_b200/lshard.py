"""Selective scan with the SEQUENCE split over the ranks of a process group (one GPU each).

The reference is single-device; this is the sequence-sharded form of MambaBlock.selective_scan
(mambapy/mamba.py:274-295) plus its gate, and must reproduce the single-device result on the
concatenated sequence.  Rank r holds timesteps [r*L/R, (r+1)*L/R) of every (B, L, .) tensor.

Forward on rank r:
  1. carry pass      S_r = state the shard reaches from a zero state          (no outputs written)
  2. decay product   P_r = exp(A * sum_t delta_t) over the shard
  3. all_gather of (P_r, S_r): 2*B*ED*N floats per rank, the only forward exchange
  4. fold            h_in = state entering shard r = fold of shards 0..r-1 (h <- P_q*h + S_q)
  5. full pass from h_in: y_r and the chunk carries for the backward
Backward on rank r:
  1. reverse carry pass  G_r = gradient carry leaving the shard when none enters it
  2. all_gather of G_r (the P_r of the forward are reused)
  3. fold            g_in = carry entering shard r from the right = fold of shards R-1..r+1
  4. full backward with the saved chunk carries and g_in
  5. all_reduce of the parameter gradients (dA, dD, d delta_bias)
The backward cannot be patched additively because da[t] = g[t]*h[t-1] is bilinear in the two
carries, hence the two-phase form in both directions.

The arithmetic is behind a small `ops` object so the collective protocol can be exercised on CPU
ranks (gloo) with stand-in arithmetic; the product always uses `CudaOps` (libmamba_b200.so).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .mamba import sscan_fwd_raw, sscan_bwd_raw, _rows, _f32, _act_dtype, _require_cuda


class CudaOps:
    """The shard-local arithmetic, every method one kernel launch of libmamba_b200.so."""

    @staticmethod
    def carry_pass(x, delta, A, Bm, Cm, delta_bias):
        _, hT, _ = sscan_fwd_raw(x, delta, A, Bm, Cm, None, None, delta_bias, None,
                                 want_last=True, want_carries=False, want_y=False)
        return hT

    @staticmethod
    def decay_prod(delta, A, delta_bias):
        lib = _lib.load()
        Bsz, L, ED = delta.shape
        N = A.shape[1]
        P = torch.empty((Bsz, ED, N), dtype=torch.float32, device=delta.device)
        flags = _lib.DELTA_SOFTPLUS if delta_bias is not None else 0
        with torch.cuda.device(delta.device):
            rc = lib.mb200_decay_prod(delta.data_ptr(), A.data_ptr(), _lib.ptr(delta_bias), P.data_ptr(),
                                      Bsz, L, ED, N, delta.stride(0), delta.stride(1),
                                      _lib.dtype_code(delta.dtype), flags, _lib.current_stream(delta.device))
        _lib.check(rc, "mb200_decay_prod")
        return P

    @staticmethod
    def fold(P_all, S_all, rank, reverse):
        """P_all, S_all: (R, B, ED, N) float32 contiguous.  Returns (B, ED, N)."""
        lib = _lib.load()
        R = P_all.shape[0]
        out = torch.empty(P_all.shape[1:], dtype=torch.float32, device=P_all.device)
        with torch.cuda.device(P_all.device):
            rc = lib.mb200_carry_fold(P_all.data_ptr(), S_all.data_ptr(), out.data_ptr(), R, out.numel(),
                                      rank, int(reverse), _lib.current_stream(P_all.device))
        _lib.check(rc, "mb200_carry_fold")
        return out

    @staticmethod
    def full_fwd(x, delta, A, Bm, Cm, D, z, delta_bias, h_in, want_carries):
        y, hT, carries = sscan_fwd_raw(x, delta, A, Bm, Cm, D, z, delta_bias, h_in,
                                       want_last=True, want_carries=want_carries)
        return y, hT, carries

    @staticmethod
    def rev_carry_pass(delta, z, dy, Cm, A, delta_bias):
        lib = _lib.load()
        Bsz, L, ED = delta.shape
        N = A.shape[1]
        g = torch.empty((Bsz, ED, N), dtype=torch.float32, device=delta.device)
        flags = _lib.DELTA_SOFTPLUS if delta_bias is not None else 0
        zs = (z.stride(0), z.stride(1)) if z is not None else (0, 0)
        with torch.cuda.device(delta.device):
            rc = lib.mb200_sscan_bwd_carry(
                delta.data_ptr(), _lib.ptr(z), dy.data_ptr(), Cm.data_ptr(), A.data_ptr(),
                _lib.ptr(delta_bias), g.data_ptr(), Bsz, L, ED, N, delta.stride(0), delta.stride(1),
                zs[0], zs[1], dy.stride(0), dy.stride(1), Cm.stride(0), Cm.stride(1),
                _lib.dtype_code(delta.dtype), flags, _lib.current_stream(delta.device))
        _lib.check(rc, "mb200_sscan_bwd_carry")
        return g

    @staticmethod
    def full_bwd(x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, g_in):
        return sscan_bwd_raw(x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, g_in=g_in,
                             want_g_out=True)


def _gather(t: torch.Tensor, group) -> torch.Tensor:
    """all_gather of equal-shaped tensors into one (R, ...) tensor."""
    R = dist.get_world_size(group)
    out = torch.empty((R,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather(list(out.unbind(0)), t.contiguous(), group=group)
    return out


def _split(t, S):
    """(B, L, C) -> (B*S, L/S, C): every batch row cut into S consecutive sub-shards (a view when
    the batch stride allows it)."""
    if t is None or S == 1:
        return t
    return t.unflatten(1, (S, t.shape[1] // S)).flatten(0, 1)


def _merge(t, S):
    """Inverse of _split for outputs: (B*S, L/S, C) -> (B, L, C)."""
    if t is None or S == 1:
        return t
    return t.unflatten(0, (t.shape[0] // S, S)).flatten(1, 2)


def pick_subshards(Bsz, L_local, ED, world):
    """How many sub-shards to cut each rank's slice into so that one GPU has enough independent
    (batch row, channel tile) work items.  Each CTA owns 32 channels of one row and about 444 CTAs
    are resident on a B200; with fewer items most SMs idle.  On a single rank sub-sharding costs
    an extra carry pass, so it is only chosen when the GPU would otherwise be under half full."""
    items = Bsz * ((ED + 31) // 32)
    best, best_eff = 1, None
    for S in (1, 2, 4, 8):
        if L_local % (16 * S):
            continue
        n = items * S
        eff = n / (-(-n // 444) * 444)
        if world == 1 and S > 1:
            eff *= 0.7                                   # the extra carry passes
        if best_eff is None or eff > best_eff + 1e-9:
            best, best_eff = S, eff
    return best


def sharded_forward(ops, group, x, delta, A, Bm, Cm, D, z, delta_bias, want_carries=True, subshards=1):
    """Steps 1-5 of the forward.  Returns (y, h_in, P_all, carries, hT).

    With subshards = S > 1 every rank's slice is itself cut into S consecutive pieces that are
    scanned as extra batch rows; the fold then runs over the R*S pieces in sequence order.
    h_in is (B*S, ED, N): the state entering each piece.  P_all is (R*S, B, ED, N)."""
    rank, R, S = dist.get_rank(group), dist.get_world_size(group), subshards
    Bsz = x.shape[0]
    xs, ds, zs, Bs, Cs = (_split(t, S) for t in (x, delta, z, Bm, Cm))
    if R * S == 1:
        y, hT, carries = ops.full_fwd(xs, ds, A, Bs, Cs, D, zs, delta_bias, None, want_carries)
        return y, None, None, carries, hT
    Sl = ops.carry_pass(xs, ds, A, Bs, Cs, delta_bias)                     # (B*S, ED, N)
    P = ops.decay_prod(ds, A, delta_bias)
    PS = torch.stack([P, Sl]).unflatten(1, (Bsz, S))                       # (2, B, S, ED, N)
    PS = _gather(PS, group) if R > 1 else PS.unsqueeze(0)                  # (R, 2, B, S, ED, N)
    PS = PS.permute(1, 0, 3, 2, 4, 5).reshape(2, R * S, Bsz, *P.shape[1:]).contiguous()
    P_all, S_all = PS[0], PS[1]                                            # (R*S, B, ED, N)
    h_in = torch.stack([ops.fold(P_all, S_all, rank * S + s, False) for s in range(S)], dim=1)
    h_in = h_in.flatten(0, 1).contiguous()                                 # (B*S, ED, N)
    y, hT, carries = ops.full_fwd(xs, ds, A, Bs, Cs, D, zs, delta_bias, h_in, want_carries)
    hT = hT.unflatten(0, (Bsz, S))[:, -1]
    return _merge(y, S), h_in, P_all, carries, hT


def sharded_backward(ops, group, x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, P_all, subshards=1):
    """Steps 1-5 of the backward.  Returns what `full_bwd` returns (per-token gradients merged back
    to (B, L/R, .), parameter gradients all-reduced; the last entry is the carry leaving the slice)."""
    rank, R, S = dist.get_rank(group), dist.get_world_size(group), subshards
    Bsz = x.shape[0]
    xs, ds, zs, Bs, Cs, dys = (_split(t, S) for t in (x, delta, z, Bm, Cm, dy))
    if R * S == 1:
        g_in = None
    else:
        G = ops.rev_carry_pass(ds, zs, dys, Cs, A, delta_bias).unflatten(0, (Bsz, S))   # (B, S, ED, N)
        G = _gather(G, group) if R > 1 else G.unsqueeze(0)                               # (R, B, S, ED, N)
        G_all = G.permute(0, 2, 1, 3, 4).reshape(R * S, Bsz, *G.shape[3:]).contiguous()
        g_in = torch.stack([ops.fold(P_all, G_all, rank * S + s, True) for s in range(S)], dim=1)
        g_in = g_in.flatten(0, 1).contiguous()
    outs = list(ops.full_bwd(xs, ds, A, Bs, Cs, D, zs, delta_bias, dys, carries, g_in))
    for i in range(5):
        outs[i] = _merge(outs[i], S)
    if outs[8] is not None and S > 1:
        outs[8] = outs[8].unflatten(0, (Bsz, S))[:, 0]
    if R > 1:
        # dA, dD, d(delta_bias) are sums over all timesteps: one flat all-reduce
        parts = [outs[5].reshape(-1), outs[6].reshape(-1)] + ([outs[7].reshape(-1)] if outs[7] is not None else [])
        flat = torch.cat(parts)
        dist.all_reduce(flat, group=group)
        nA, nD = outs[5].numel(), outs[6].numel()
        outs[5] = flat[:nA].view_as(outs[5])
        outs[6] = flat[nA:nA + nD].view_as(outs[6])
        if outs[7] is not None:
            outs[7] = flat[nA + nD:].view_as(outs[7])
    return tuple(outs)


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
