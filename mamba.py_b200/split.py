"""Selective scan of a sequence cut into consecutive pieces that are scanned side by side.

Two uses, one protocol:
  * one GPU, few batch rows: a (B, L, .) problem has only B * ceil(ED / 32) independent work items for
    the fused kernels, which leaves most of a B200 idle when B is small (the reference's own published
    timings are all batch 1).  Every row is cut into S consecutive sub-shards that run as extra batch rows.
  * several GPUs, one long sequence (lshard.py): rank r holds timesteps [r*L/R, (r+1)*L/R) and may cut its
    slice into sub-shards as well.
The reference is single-device and has neither (mambapy/mamba.py:274-295 scans the whole sequence);
whatever the cut, the result must equal the scan of the concatenated sequence.

Forward:   1. carry pass over every piece: state reached from a zero state, and the piece's decay product
              P = exp(A * sum_t delta_t)                                     (one kernel, no outputs written)
           2. (ranks > 1) all_gather of (P, S): 2*B*S*ED*N floats per rank, the only forward exchange
           3. fold: state entering every local piece, h <- P_q*h + S_q over the pieces before it (one kernel)
           4. full pass of all local pieces from those states: y and the saved states for the backward
Backward:  1. reverse carry pass: gradient carry leaving every piece when none enters it
           2. (ranks > 1) all_gather of these; the P of the forward are reused
           3. fold from the right: carry entering every local piece
           4. full backward with the saved states and those carries
           5. (ranks > 1) all_reduce of the parameter gradients (dA, dD, d delta_bias)
The backward cannot be patched additively because da[t] = g[t]*h[t-1] is bilinear in the two carries,
hence the two-phase form in both directions.

The arithmetic is behind a small `ops` object so the protocol can be exercised on CPU ranks (gloo) with
stand-in arithmetic; the product always uses `CudaOps` (libmamba_b200.so).
"""
from __future__ import annotations

import torch

from .kernels import sscan_fwd_raw, sscan_bwd_raw, sscan_fwd_carry_raw, sscan_bwd_carry_raw, carry_fold_range

RESIDENT_CTAS = 444          # 148 SMs x 3 CTAs of the fused kernels


class CudaOps:
    """The piece-local arithmetic, every method one kernel launch of libmamba_b200.so."""

    @staticmethod
    def carry_pass(x, delta, A, Bm, Cm, delta_bias, skip_last=0):
        """-> one (2, rows, ED, N) tensor: [0] the decay product of every row's span, [1] the state it reaches
        from a zero state.  The last `skip_last` rows are left out (zeros)."""
        return sscan_fwd_carry_raw(x, delta, A, Bm, delta_bias, skip_last=skip_last)

    @staticmethod
    def fold_range(P_all, S_all, init, first, num, reverse):
        """P_all, S_all: (B, pieces, ED, N); init (B, ED, N) or None -> (B, num, ED, N)."""
        return carry_fold_range(P_all, S_all, init, first, num, reverse)

    @staticmethod
    def full_fwd(x, delta, A, Bm, Cm, D, z, delta_bias, h_in, want_carries):
        return sscan_fwd_raw(x, delta, A, Bm, Cm, D, z, delta_bias, h_in, want_last=True, want_carries=want_carries)

    @staticmethod
    def rev_carry_pass(delta, z, dy, Cm, A, delta_bias, skip_first=0):
        return sscan_bwd_carry_raw(delta, z, dy, Cm, A, delta_bias, skip_first=skip_first)

    @staticmethod
    def full_bwd(x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, g_in):
        return sscan_bwd_raw(x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, g_in=g_in, want_g_out=True)


def _group_info(group):
    if group is None:
        return 0, 1
    import torch.distributed as dist
    return dist.get_rank(group), dist.get_world_size(group)


def _gather(t: torch.Tensor, group) -> torch.Tensor:
    """all_gather of equal-shaped tensors into one (R, ...) tensor."""
    import torch.distributed as dist
    R = dist.get_world_size(group)
    out = torch.empty((R,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather(list(out.unbind(0)), t.contiguous(), group=group)
    return out


def _split(t, S):
    """(B, L, C) -> (B*S, L/S, C): every batch row cut into S consecutive sub-shards (a view when the batch
    stride allows it)."""
    if t is None or S == 1:
        return t
    return t.unflatten(1, (S, t.shape[1] // S)).flatten(0, 1)


def _merge(t, S):
    """Inverse of _split for outputs: (B*S, L/S, C) -> (B, L, C)."""
    if t is None or S == 1:
        return t
    return t.unflatten(0, (t.shape[0] // S, S)).flatten(1, 2)


def pick_subshards(Bsz, L_local, ED, world=1):
    """How many sub-shards to cut each row of this device's slice into.

    The fused kernels have Bsz * ceil(ED / 32) independent work items (a CTA owns one) and 148 SMs hold three
    CTAs each.  Measured on B200, forward + backward of one row (ms): ED 2048, L 65536: 12.0 uncut, 7.8 / 5.8 /
    5.8 / 4.8 in 2 / 4 / 8 / 16 pieces; ED 2048, L 8192: 1.53 uncut, 0.68 in 16; ED 5120, L 131072: 35.5 uncut,
    27.0 / 23.9 / 23.7 in 4 / 8 / 16.  So: cut until there are about two waves of CTAs (the pieces' tails then
    overlap), keep pieces at least 512 timesteps long, and leave alone what already fills half the GPU (on a
    single rank a cut costs two extra carry passes) or is so short that the extra launches eat the gain."""
    items = Bsz * ((ED + 31) // 32)
    if world == 1 and (L_local < 4096 or 2 * items >= RESIDENT_CTAS):
        return 1
    best = 1
    for S in (2, 4, 8, 16):
        if L_local % (16 * S) or L_local // S < 512:
            break
        best = S
        if items * S >= 2 * RESIDENT_CTAS:
            break
    return best


def split_forward(ops, group, x, delta, A, Bm, Cm, D, z, delta_bias, h0=None, want_carries=True, subshards=1):
    """Steps 1-4 of the forward.  Returns (y, h_in, P_all, carries, hT).

    Every rank's slice is cut into S = subshards consecutive pieces that are scanned as extra batch rows;
    the fold runs over the R*S pieces in sequence order.  h_in is (B*S, ED, N), the state entering each local
    piece; P_all is (B, R*S, ED, N); hT (B, ED, N) is the state leaving this rank's last piece.
    `h0` (B, ED, N), the state entering the very first piece, is honoured on a single rank."""
    rank, R = _group_info(group)
    S, Bsz = subshards, x.shape[0]
    xs, ds, zs, Bs, Cs = (_split(t, S) for t in (x, delta, z, Bm, Cm))
    if R * S == 1:
        y, hT, carries = ops.full_fwd(xs, ds, A, Bs, Cs, D, zs, delta_bias, h0, want_carries)
        return y, None, None, carries, hT
    # one row on one rank: its last piece's carry feeds nothing, so that piece is left out of the pass
    skip = 1 if (R == 1 and Bsz == 1) else 0
    PS = ops.carry_pass(xs, ds, A, Bs, Cs, delta_bias, **({"skip_last": 1} if skip else {}))
    PS = PS.unflatten(1, (Bsz, S))                                          # (2, B, S, ED, N): decay product, state
    if R > 1:
        PS = _gather(PS, group).permute(1, 2, 0, 3, 4, 5).reshape(2, Bsz, R * S, *PS.shape[3:]).contiguous()
    P_all, S_all = PS[0], PS[1]                                              # (B, R*S, ED, N)
    h_in = ops.fold_range(P_all, S_all, h0, rank * S, S, False).flatten(0, 1)   # (B*S, ED, N)
    y, hT, carries = ops.full_fwd(xs, ds, A, Bs, Cs, D, zs, delta_bias, h_in, want_carries)
    hT = hT.unflatten(0, (Bsz, S))[:, -1]
    return _merge(y, S), h_in, P_all, carries, hT


def split_backward(ops, group, x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, P_all, subshards=1):
    """Steps 1-5 of the backward.  Returns what `full_bwd` returns (per-token gradients merged back to
    (B, L/R, .), parameter gradients all-reduced; the last entry is the carry leaving this rank's slice to
    the left, which on rank 0 is the gradient of the initial state)."""
    rank, R = _group_info(group)
    S, Bsz = subshards, x.shape[0]
    xs, ds, zs, Bs, Cs, dys = (_split(t, S) for t in (x, delta, z, Bm, Cm, dy))
    if R * S == 1:
        g_in = None
    else:
        skip = 1 if (R == 1 and Bsz == 1) else 0                    # the first piece's carry feeds nothing
        G = ops.rev_carry_pass(ds, zs, dys, Cs, A, delta_bias, **({"skip_first": 1} if skip else {}))
        G = G.unflatten(0, (Bsz, S))                                                      # (B, S, ED, N)
        if R > 1:
            G = _gather(G, group).permute(1, 0, 2, 3, 4).reshape(Bsz, R * S, *G.shape[2:])
        g_in = ops.fold_range(P_all, G.contiguous(), None, rank * S, S, True).flatten(0, 1)
    outs = list(ops.full_bwd(xs, ds, A, Bs, Cs, D, zs, delta_bias, dys, carries, g_in))
    for i in range(5):
        outs[i] = _merge(outs[i], S)
    if outs[8] is not None and S > 1:
        outs[8] = outs[8].unflatten(0, (Bsz, S))[:, 0]
    if R > 1:
        import torch.distributed as dist
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
