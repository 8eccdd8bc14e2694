"""Raw launchers of the fused-scan kernels in libmamba_b200.so: tensors in, tensors out, no autograd.

Callers prepare the tensors (activation dtype, unit-stride last dimension, float32 parameters); every
function here allocates the outputs, passes pointers and strides through the C ABI and raises on a
non-zero return code.  The autograd wrappers (mamba.py), the split-sequence scan (split.py, lshard.py)
and bench.py's per-kernel timings all go through these.
"""
from __future__ import annotations

import torch

from . import _lib


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mamba_b200 runs on CUDA tensors only (there is no CPU path)")


def _rows(t: torch.Tensor | None, dtype) -> torch.Tensor | None:
    """Cast to the activation dtype and make the last dim unit-stride (copy only if needed)."""
    if t is None:
        return None
    if t.dtype != dtype:
        t = t.to(dtype)
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


def _act_dtype(x: torch.Tensor, *others):
    """Activation dtype the kernel runs in: bfloat16 only when EVERY activation tensor is bfloat16,
    float32 as soon as one of them is (under autocast the reference keeps delta in float32 while x, B
    and C are bfloat16, mambapy/mamba.py:264-265; rounding delta to bfloat16 would change the decay)."""
    dts = {t.dtype for t in (x,) + others if t is not None}
    for d in dts:
        if d not in (torch.float32, torch.bfloat16):
            raise TypeError(f"mamba_b200 kernels take float32 or bfloat16 activations, got {d}")
    return torch.bfloat16 if dts == {torch.bfloat16} else torch.float32


def _tensor_map_ok(t: torch.Tensor) -> bool:
    """16-byte aligned base and byte strides: what a tiled tensor map of a (B, L, C) tensor needs."""
    es = t.element_size()
    return t.data_ptr() % 16 == 0 and (t.stride(0) * es) % 16 == 0 and (t.stride(1) * es) % 16 == 0


def _f32(t):
    return None if t is None else t.detach().float().contiguous()


def sscan_fwd_raw(x, delta, A, Bm, Cm, D, z=None, delta_bias=None, h0=None,
                  want_last=False, want_carries=False, want_y=True, reverse=False, general_decay=False):
    """Launch the fused forward.  Tensors must already be prepared by the caller.

    Returns (y, hT, carries); entries not asked for are None.  With `reverse` the scan runs from the
    last timestep to the first; None is returned when the kernels cannot do that for these tensors
    (the caller then flips them itself).  `general_decay` switches off the kernels' own shortcut for an
    A with the S4D-real structure (every decay then gets its own exponential)."""
    lib = _lib.load()
    Bsz, L, ED = x.shape
    N = A.shape[1]
    dev = x.device
    y = torch.empty((Bsz, L, ED), dtype=x.dtype, device=dev) if want_y else None
    hT = torch.empty((Bsz, ED, N), dtype=torch.float32, device=dev) if want_last else None
    chunk = lib.mb200_sscan_chunk()
    carries = (torch.empty((Bsz, (L + chunk - 1) // chunk, ED, N), dtype=torch.float32, device=dev)
               if want_carries else None)
    flags = ((_lib.DELTA_SOFTPLUS if delta_bias is not None else 0) | (_lib.REVERSE if reverse else 0)
             | (_lib.GENERAL_DECAY if general_decay else 0))
    zs = (z.stride(0), z.stride(1)) if z is not None else (0, 0)
    ys = (y.stride(0), y.stride(1)) if y is not None else (0, 0)
    with torch.cuda.device(dev):
        rc = lib.mb200_sscan_fwd(
            x.data_ptr(), delta.data_ptr(), _lib.ptr(z), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(),
            _lib.ptr(D), _lib.ptr(delta_bias), _lib.ptr(h0), _lib.ptr(y), _lib.ptr(hT),
            _lib.ptr(carries), Bsz, L, ED, N,
            x.stride(0), x.stride(1), delta.stride(0), delta.stride(1), zs[0], zs[1],
            Bm.stride(0), Bm.stride(1), Cm.stride(0), Cm.stride(1), ys[0], ys[1],
            _lib.dtype_code(x.dtype), flags, _lib.current_stream(dev))
    if reverse and rc == _lib.EUNSUPPORTED:
        return None
    _lib.check(rc, "mb200_sscan_fwd")
    _lib.check_status(dev, "mb200_sscan_fwd")
    return y, hT, carries


def sscan_bwd_raw(x, delta, A, Bm, Cm, D, z, delta_bias, dy, carries, g_in=None, want_g_out=False,
                  reverse=False, general_decay=False, out_dz=None):
    """Launch the fused backward.  Returns (dx, ddelta, dz, dB, dC, dA, dD, dbias, g_out).

    `reverse` must be what the forward that produced `carries` ran with."""
    lib = _lib.load()
    Bsz, L, ED = x.shape
    N = A.shape[1]
    dev = x.device
    dx = torch.empty((Bsz, L, ED), dtype=x.dtype, device=dev)
    dd = torch.empty_like(dx)
    # dz may be written straight into a caller's (strided) view, e.g. the second half of d(xz)
    dz = (out_dz if out_dz is not None else torch.empty_like(dx)) if z is not None else None
    # every buffer the kernel accumulates into comes out of ONE zero-filled allocation (one fill launch)
    nBC, nA = Bsz * L * N, ED * N
    acc = torch.zeros(2 * nBC + nA + 2 * ED, dtype=torch.float32, device=dev)
    dB = acc[:nBC].view(Bsz, L, N)
    dC = acc[nBC:2 * nBC].view(Bsz, L, N)
    dA = acc[2 * nBC:2 * nBC + nA].view(ED, N)
    dD = acc[2 * nBC + nA:2 * nBC + nA + ED]
    dbias = acc[2 * nBC + nA + ED:] if delta_bias is not None else None
    g_out = torch.empty((Bsz, ED, N), dtype=torch.float32, device=dev) if want_g_out else None
    flags = ((_lib.DELTA_SOFTPLUS if delta_bias is not None else 0) | (_lib.REVERSE if reverse else 0)
             | (_lib.GENERAL_DECAY if general_decay else 0))
    zs = (z.stride(0), z.stride(1)) if z is not None else (0, 0)
    dzs = (dz.stride(0), dz.stride(1)) if dz is not None else (0, 0)
    with torch.cuda.device(dev):
        rc = lib.mb200_sscan_bwd(
            x.data_ptr(), delta.data_ptr(), _lib.ptr(z), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(),
            _lib.ptr(D), _lib.ptr(delta_bias), dy.data_ptr(), carries.data_ptr(), _lib.ptr(g_in),
            dx.data_ptr(), dd.data_ptr(), _lib.ptr(dz), dB.data_ptr(), dC.data_ptr(), dA.data_ptr(),
            dD.data_ptr(), _lib.ptr(dbias), _lib.ptr(g_out), Bsz, L, ED, N,
            x.stride(0), x.stride(1), delta.stride(0), delta.stride(1), zs[0], zs[1],
            Bm.stride(0), Bm.stride(1), Cm.stride(0), Cm.stride(1), dy.stride(0), dy.stride(1),
            dx.stride(0), dx.stride(1), dd.stride(0), dd.stride(1), dzs[0], dzs[1],
            _lib.dtype_code(x.dtype), flags, _lib.current_stream(dev))
    _lib.check(rc, "mb200_sscan_bwd")
    _lib.check_status(dev, "mb200_sscan_bwd")
    return dx, dd, dz, dB, dC, dA, dD, dbias, g_out



def sscan_fwd_carry_raw(x, delta, A, Bm, delta_bias=None, skip_last=0):
    """Forward carry pass of a span, one pass over x, delta, B.  Returns one (2, B, ED, N) float32 tensor:
    [0] the span's decay product exp(A * sum_t delta), [1] the state reached from a zero state.
    The last `skip_last` rows are not scanned (their entries are zero): nothing follows the last piece of
    a sequence, so its carry is never used."""
    lib = _lib.load()
    rows, L, ED = x.shape
    Bsz = rows - skip_last
    N = A.shape[1]
    dev = x.device
    out = torch.empty((2, rows, ED, N), dtype=torch.float32, device=dev)
    if skip_last:
        out[:, Bsz:].zero_()
    flags = _lib.DELTA_SOFTPLUS if delta_bias is not None else 0
    with torch.cuda.device(dev):
        rc = lib.mb200_sscan_fwd_carry(x.data_ptr(), delta.data_ptr(), A.data_ptr(), Bm.data_ptr(), _lib.ptr(delta_bias),
                                       out[1].data_ptr(), out[0].data_ptr(), Bsz, L, ED, N, x.stride(0), x.stride(1),
                                       delta.stride(0), delta.stride(1), Bm.stride(0), Bm.stride(1),
                                       _lib.dtype_code(x.dtype), flags, _lib.current_stream(dev))
    _lib.check(rc, "mb200_sscan_fwd_carry")
    _lib.check_status(dev, "mb200_sscan_fwd_carry")
    return out


def sscan_bwd_carry_raw(delta, z, dy, Cm, A, delta_bias=None, skip_first=0):
    """Reverse carry pass of a span: the gradient carry (B, ED, N) float32 that leaves its first timestep
    when none enters its last one.  The first `skip_first` rows are not scanned (entries zero): nothing
    precedes the first piece of a sequence."""
    lib = _lib.load()
    rows, L, ED = delta.shape
    N = A.shape[1]
    g_all = torch.empty((rows, ED, N), dtype=torch.float32, device=delta.device)
    if skip_first:
        g_all[:skip_first].zero_()
        delta, dy, Cm = delta[skip_first:], dy[skip_first:], Cm[skip_first:]
        z = z[skip_first:] if z is not None else None
    g = g_all[skip_first:]
    Bsz = rows - skip_first
    flags = _lib.DELTA_SOFTPLUS if delta_bias is not None else 0
    zs = (z.stride(0), z.stride(1)) if z is not None else (0, 0)
    with torch.cuda.device(delta.device):
        rc = lib.mb200_sscan_bwd_carry(
            delta.data_ptr(), _lib.ptr(z), dy.data_ptr(), Cm.data_ptr(), A.data_ptr(),
            _lib.ptr(delta_bias), g.data_ptr(), Bsz, L, ED, N, delta.stride(0), delta.stride(1),
            zs[0], zs[1], dy.stride(0), dy.stride(1), Cm.stride(0), Cm.stride(1),
            _lib.dtype_code(delta.dtype), flags, _lib.current_stream(delta.device))
    _lib.check(rc, "mb200_sscan_bwd_carry")
    _lib.check_status(delta.device, "mb200_sscan_bwd_carry")
    return g_all


def carry_fold_range(P_all, S_all, init, first, num, reverse):
    """P_all, S_all: (batch, R, ...) float32 contiguous; init: (batch, ...) or None.  Returns (batch, num, ...):
    entry i is the state entering piece first+i (forward), or the gradient carry entering it from the right
    (reverse), folded over the R pieces in ONE launch."""
    lib = _lib.load()
    batch, R = P_all.shape[0], P_all.shape[1]
    M = P_all[0, 0].numel()
    out = torch.empty((batch, num) + tuple(P_all.shape[2:]), dtype=torch.float32, device=P_all.device)
    with torch.cuda.device(P_all.device):
        rc = lib.mb200_carry_fold_range(P_all.data_ptr(), S_all.data_ptr(), _lib.ptr(init), out.data_ptr(), batch, R, M,
                                        first, num, int(reverse), _lib.current_stream(P_all.device))
    _lib.check(rc, "mb200_carry_fold_range")
    return out


def conv1d_silu_fwd_raw(xs, w32, b32):
    """silu(depthwise causal conv1d(x)), d_conv 4, on (B, L, ED) with any batch / row strides."""
    lib = _lib.load()
    Bsz, L, ED = xs.shape
    y = torch.empty((Bsz, L, ED), dtype=xs.dtype, device=xs.device)
    with torch.cuda.device(xs.device):
        rc = lib.mb200_conv1d_silu_fwd(xs.data_ptr(), w32.data_ptr(), _lib.ptr(b32), y.data_ptr(), Bsz, L, ED,
                                       w32.shape[1], xs.stride(0), xs.stride(1), y.stride(0), y.stride(1),
                                       _lib.dtype_code(xs.dtype), _lib.current_stream(xs.device))
    _lib.check(rc, "mb200_conv1d_silu_fwd")
    return y


def conv1d_silu_bwd_raw(xs, w32, b32, dy, out_dx=None):
    """Backward of conv1d_silu_fwd_raw.  Returns (dx, dw (ED, K) float32, db (ED) float32 or None); dx may be a
    caller's (strided) view."""
    lib = _lib.load()
    Bsz, L, ED = xs.shape
    dx = out_dx if out_dx is not None else torch.empty_like(xs)
    dw = torch.zeros_like(w32)
    db = torch.zeros(ED, dtype=torch.float32, device=xs.device) if b32 is not None else None
    with torch.cuda.device(xs.device):
        rc = lib.mb200_conv1d_silu_bwd(xs.data_ptr(), w32.data_ptr(), _lib.ptr(b32), dy.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), _lib.ptr(db), Bsz, L, ED, w32.shape[1], xs.stride(0), xs.stride(1),
                                       dy.stride(0), dy.stride(1), dx.stride(0), dx.stride(1),
                                       _lib.dtype_code(xs.dtype), _lib.current_stream(xs.device))
    _lib.check(rc, "mb200_conv1d_silu_bwd")
    return dx, dw, db
