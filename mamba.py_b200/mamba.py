"""Drop-ins for the scan methods of the reference's MambaBlock (mambapy/mamba.py).

The functions below take `self` first so they can be bound onto the reference's MambaBlock
(see `mamba_b200.install`) or onto any object with the same attribute names:

    selective_scan(self, x, delta, A, B, C, D)      mambapy/mamba.py:274-295
    selective_scan_seq(self, x, delta, A, B, C, D)  mambapy/mamba.py:297-327 (same kernel)
    ssm_step(self, x, h)                            mambapy/mamba.py:384-414
    step(self, x, cache)                            mambapy/mamba.py:351-382
    ssm(self, x, z) / forward(self, x)              mambapy/mamba.py:236-272 / :205-234 with the
                                                    softplus, the scan and the gate in one kernel

`selective_scan_fn` is the functional form with the optional gate `z`, the fused
`softplus(delta + delta_bias)`, an incoming state `h0` and the outgoing state.
Everything runs in libmamba_b200.so on CUDA tensors; there is no CPU path.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


from .kernels import (_require_cuda, _rows, _act_dtype, _tensor_map_ok, _f32, sscan_fwd_raw, sscan_bwd_raw,
                      sscan_fwd_carry_raw, sscan_bwd_carry_raw, carry_fold_range, conv1d_silu_fwd_raw,
                      conv1d_silu_bwd_raw)
from .split import CudaOps, pick_subshards, split_forward, split_backward


class SelectiveScanFn(torch.autograd.Function):
    """y (and optionally the last state) of the fused scan; gradients for every input."""

    @staticmethod
    def forward(ctx, x, delta, A, Bm, Cm, D, z, delta_bias, h0, return_last_state, reverse=False, subshards=None):
        _require_cuda(x, delta, A, Bm, Cm, D, z, delta_bias, h0)
        dt = _act_dtype(x, delta, z, Bm, Cm)
        xs, ds, zs = _rows(x, dt), _rows(delta, dt), _rows(z, dt)
        Bs, Cs = _rows(Bm, dt), _rows(Cm, dt)
        A32, D32, b32, h032 = _f32(A), _f32(D), _f32(delta_bias), _f32(h0)
        needs_grad = any(t is not None and t.requires_grad
                         for t in (x, delta, A, Bm, Cm, D, z, delta_bias, h0))
        out = None
        ctx.flipped = False
        P_all = None
        # Few batch rows: cut every row into S consecutive pieces that run side by side (split.py); the
        # reference's own published shapes are all batch 1, i.e. 64 work items for a 148-SM GPU.
        S = subshards if subshards else pick_subshards(xs.shape[0], xs.shape[1], xs.shape[2], 1)
        if reverse or S < 1 or xs.shape[1] % (16 * S) or xs.shape[1] == 0:
            S = 1
        if S > 1:
            y, _, P_all, carries, hT = split_forward(CudaOps, None, xs, ds, A32, Bs, Cs, D32, zs, b32, h0=h032,
                                                     want_carries=needs_grad, subshards=S)
            out = (y, hT if return_last_state else None, carries)
        if out is None and reverse and not (needs_grad and A32.shape[1] != 16):    # the reverse backward exists for d_state 16
            out = sscan_fwd_raw(xs, ds, A32, Bs, Cs, D32, zs, b32, h032, want_last=return_last_state,
                                want_carries=needs_grad, reverse=True)
        if reverse and out is None:
            # what the reference does (mambapy/vim.py:228-261): scan the flipped sequence, flip back
            xs, ds, zs, Bs, Cs = (None if t is None else t.flip(1) for t in (xs, ds, zs, Bs, Cs))
            ctx.flipped = True
        if out is None:
            out = sscan_fwd_raw(xs, ds, A32, Bs, Cs, D32, zs, b32, h032,
                                want_last=return_last_state, want_carries=needs_grad)
        y, hT, carries = out
        if ctx.flipped:
            y = y.flip(1)
        ctx.reverse = reverse and not ctx.flipped
        ctx.subshards = S
        ctx.save_for_backward(xs, ds, A32, Bs, Cs, D32, zs, b32, carries, P_all)
        ctx.in_dtypes = tuple(None if t is None else t.dtype
                              for t in (x, delta, A, Bm, Cm, D, z, delta_bias, h0))
        ctx.has_h0 = h0 is not None
        if return_last_state:
            ctx.mark_non_differentiable(hT)
            return y, hT
        return y

    @staticmethod
    def backward(ctx, dy, *unused):
        xs, ds, A32, Bs, Cs, D32, zs, b32, carries, P_all = ctx.saved_tensors
        dy = _rows(dy.flip(1) if ctx.flipped else dy, xs.dtype)
        if ctx.subshards > 1:
            dx, dd, dz, dB, dC, dA, dD, dbias, g_out = split_backward(
                CudaOps, None, xs, ds, A32, Bs, Cs, D32, zs, b32, dy, carries, P_all, subshards=ctx.subshards)
            tx, td, tA, tB, tC, tD, tz, tb, th = ctx.in_dtypes
            cast = lambda g, t: None if (g is None or t is None) else g.to(t)
            return (cast(dx, tx), cast(dd, td), cast(dA, tA), cast(dB, tB), cast(dC, tC), cast(dD, tD),
                    cast(dz, tz), cast(dbias, tb), cast(g_out if ctx.has_h0 else None, th), None, None, None)
        if ctx.reverse and not _tensor_map_ok(dy):
            # the in-kernel reverse backward exists on the tensor-map path only; an upstream gradient
            # that is an offset or narrow view of something wider is copied to a dense tensor first
            dy = dy.contiguous()
        dx, dd, dz, dB, dC, dA, dD, dbias, g_out = sscan_bwd_raw(
            xs, ds, A32, Bs, Cs, D32, zs, b32, dy, carries, want_g_out=ctx.has_h0, reverse=ctx.reverse)
        if ctx.flipped:
            dx, dd, dz, dB, dC = (None if t is None else t.flip(1) for t in (dx, dd, dz, dB, dC))
        tx, td, tA, tB, tC, tD, tz, tb, th = ctx.in_dtypes
        cast = lambda g, t: None if (g is None or t is None) else g.to(t)
        return (cast(dx, tx), cast(dd, td), cast(dA, tA), cast(dB, tB), cast(dC, tC),
                cast(dD, tD), cast(dz, tz), cast(dbias, tb), cast(g_out, th), None, None, None)


def selective_scan_fn(x, delta, A, B, C, D=None, z=None, delta_bias=None, h0=None,
                      return_last_state=False, reverse=False, subshards=None):
    """Fused selective scan.

    x, delta, z : (B, L, ED)   B, C : (B, L, N)   A : (ED, N)   D : (ED)
    With `delta_bias` the kernel applies delta = softplus(delta + delta_bias) itself (the
    contract of the fused seam at mambapy/mamba.py:260); with `z` it also applies the
    y * silu(z) gate (mambapy/mamba.py:229-231).  Returns y (B, L, ED), plus the final state
    (B, ED, N) float32 when `return_last_state`.

    `reverse=True` scans from the last timestep to the first (h0 enters at t = L-1, the returned state
    leaves t = 0): the second direction of the reference's bidirectional model, which flips the
    sequence, scans and flips back (mambapy/vim.py:228-261).  The kernels do it in place when the
    tensors meet the tensor-map alignment rules (and d_state is 16 if gradients are needed);
    otherwise this function flips, as the reference does.

    With few batch rows the sequence is cut into `subshards` consecutive pieces that are scanned side by
    side (two extra carry passes, see split.py): None picks the number from the shape, 1 never cuts, any
    other value is used if L is a multiple of 16 * subshards.
    """
    return SelectiveScanFn.apply(x, delta, A, B, C, D, z, delta_bias, h0, return_last_state, reverse, subshards)


# ----------------------------------------------------------------- MambaBlock method drop-ins

def selective_scan(self, x, delta, A, B, C, D):
    """mambapy/mamba.py:274-295.  x, delta: (B, L, ED); A: (ED, N); B, C: (B, L, N); D: (ED)."""
    return selective_scan_fn(x, delta, A, B, C, D)


def selective_scan_seq(self, x, delta, A, B, C, D):
    """mambapy/mamba.py:297-327.  The sequential variant computes the same y; same kernel."""
    return selective_scan_fn(x, delta, A, B, C, D)


def ssm_step_fn(x, h, delta, A, B, C, D=None, z=None, delta_bias=None, inplace=False):
    """One decode step on projected inputs.  x, delta, z: (B, ED); B, C: (B, N); h: (B, ED, N) or None.

    Returns (y, h_new); h_new is a fresh float32 tensor (the reference also returns a new one,
    mambapy/mamba.py:408).  `inplace=True` (opt-in, for decode loops that own their cache)
    overwrites a float32 contiguous `h` instead and returns it."""
    _require_cuda(x, delta, A, B, C, D, z, delta_bias, h)
    lib = _lib.load()
    dt = _act_dtype(x, delta, z, B, C)
    xs, ds, zs, Bs, Cs = (_rows(t, dt) for t in (x, delta, z, B, C))
    A32, D32, b32 = _f32(A), _f32(D), _f32(delta_bias)
    h32 = None if h is None else h.float().contiguous()
    Bsz, ED = xs.shape
    N = A32.shape[1]
    if inplace:
        if h is None or h32.data_ptr() != h.data_ptr():
            raise ValueError("inplace=True needs a float32 contiguous state tensor")
        h_new = h
    else:
        h_new = torch.empty((Bsz, ED, N), dtype=torch.float32, device=xs.device)
    y = torch.empty((Bsz, ED), dtype=dt, device=xs.device)
    flags = _lib.DELTA_SOFTPLUS if b32 is not None else 0
    with torch.cuda.device(xs.device):
        rc = lib.mb200_ssm_step(
            xs.data_ptr(), ds.data_ptr(), _lib.ptr(zs), A32.data_ptr(), Bs.data_ptr(), Cs.data_ptr(),
            _lib.ptr(D32), _lib.ptr(b32), _lib.ptr(h32), h_new.data_ptr(), y.data_ptr(), Bsz, ED, N,
            xs.stride(0), ds.stride(0), zs.stride(0) if zs is not None else 0, Bs.stride(0),
            Cs.stride(0), y.stride(0), _lib.dtype_code(dt), flags, _lib.current_stream(xs.device))
    _lib.check(rc, "mb200_ssm_step")
    return y, h_new


def conv_step_fn(x, inputs, weight, bias, inplace=False):
    """Conv-window part of a decode step (mambapy/mamba.py:366-369, :379).

    x: (B, ED) new pre-conv input; inputs: (B, ED, d_conv-1) cached window;
    weight: (ED, 1, d_conv) depthwise filter; bias: (ED) or None.
    Returns (silu(conv(x)), new window).  The window is a fresh tensor unless `inplace=True`
    (opt-in), which shifts a contiguous window of the activation dtype in place."""
    _require_cuda(x, inputs, weight, bias)
    lib = _lib.load()
    dt = _act_dtype(x)
    xs = _rows(x, dt)
    win = inputs.to(dt).contiguous()
    Bsz, ED = xs.shape
    K = weight.shape[-1]
    w32 = weight.detach().reshape(ED, K).float().contiguous()
    b32 = _f32(bias)
    xc = torch.empty((Bsz, ED), dtype=dt, device=xs.device)
    if inplace:
        if win.data_ptr() != inputs.data_ptr():
            raise ValueError("inplace=True needs a contiguous window of the activation dtype")
        new_win = inputs
    else:
        new_win = torch.empty_like(win)
    with torch.cuda.device(xs.device):
        rc = lib.mb200_conv_step(xs.data_ptr(), win.data_ptr(), w32.data_ptr(), _lib.ptr(b32),
                                 xc.data_ptr(), new_win.data_ptr(), Bsz, ED, K, xs.stride(0),
                                 _lib.dtype_code(dt), _lib.current_stream(xs.device))
    _lib.check(rc, "mb200_conv_step")
    return xc, new_win


class CausalConv1dSiluFn(torch.autograd.Function):
    """silu(depthwise causal conv1d(x)) on (B, L, ED) tensors, d_conv = 4."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        _require_cuda(x, weight, bias)
        lib = _lib.load()
        dt = _act_dtype(x)
        xs = _rows(x, dt)
        Bsz, L, ED = xs.shape
        K = weight.shape[-1]
        w32 = weight.detach().reshape(ED, K).float().contiguous()
        b32 = _f32(bias)
        y = torch.empty((Bsz, L, ED), dtype=dt, device=xs.device)
        with torch.cuda.device(xs.device):
            rc = lib.mb200_conv1d_silu_fwd(xs.data_ptr(), w32.data_ptr(), _lib.ptr(b32), y.data_ptr(), Bsz, L, ED, K,
                                           xs.stride(0), xs.stride(1), y.stride(0), y.stride(1),
                                           _lib.dtype_code(dt), _lib.current_stream(xs.device))
        _lib.check(rc, "mb200_conv1d_silu_fwd")
        ctx.save_for_backward(xs, w32, b32)
        ctx.meta = (x.dtype, weight.dtype, weight.shape, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xs, w32, b32 = ctx.saved_tensors
        lib = _lib.load()
        dy = _rows(dy, xs.dtype)
        Bsz, L, ED = xs.shape
        K = w32.shape[1]
        dx = torch.empty_like(xs)
        dw = torch.zeros_like(w32)
        db = torch.zeros(ED, dtype=torch.float32, device=xs.device) if b32 is not None else None
        with torch.cuda.device(xs.device):
            rc = lib.mb200_conv1d_silu_bwd(xs.data_ptr(), w32.data_ptr(), _lib.ptr(b32), dy.data_ptr(), dx.data_ptr(),
                                           dw.data_ptr(), _lib.ptr(db), Bsz, L, ED, K, xs.stride(0), xs.stride(1),
                                           dy.stride(0), dy.stride(1), dx.stride(0), dx.stride(1),
                                           _lib.dtype_code(xs.dtype), _lib.current_stream(xs.device))
        _lib.check(rc, "mb200_conv1d_silu_bwd")
        tx, tw, wshape, tb = ctx.meta
        return dx.to(tx), dw.to(tw).reshape(wshape), None if db is None else db.to(tb)


def causal_conv1d_silu(x, weight, bias=None):
    """silu(conv1d(x)) of MambaBlock.forward (mambapy/mamba.py:217-221) without the transposes.

    x: (B, L, ED); weight: (ED, 1, 4) as nn.Conv1d(groups=ED) holds it; bias: (ED) or None."""
    return CausalConv1dSiluFn.apply(x, weight, bias)


class RMSNormFn(torch.autograd.Function):
    """y = x * rsqrt(mean(x^2, -1) + eps) * weight in one pass over x (mambapy/mamba.py:416-433)."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        lib = _lib.load()
        dt = _act_dtype(x)
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if x2.dtype != dt or x2.stride(-1) != 1:
            x2 = x2.to(dt).contiguous()
        rows = x2.shape[0]
        w32 = None if weight is None else _f32(weight)
        y = torch.empty((rows, D), dtype=dt, device=x.device)
        rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            rc = lib.mb200_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(w32), y.data_ptr(), rstd.data_ptr(), rows, D,
                                       x2.stride(0), y.stride(0), float(eps), _lib.dtype_code(dt),
                                       _lib.current_stream(x.device))
        _lib.check(rc, "mb200_rmsnorm_fwd")
        ctx.save_for_backward(x2, w32, rstd)
        ctx.meta = (x.shape, x.dtype, None if weight is None else weight.dtype)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w32, rstd = ctx.saved_tensors
        shape, tx, tw = ctx.meta
        lib = _lib.load()
        rows, D = x2.shape
        dy2 = dy.reshape(rows, D)
        if dy2.dtype != x2.dtype or dy2.stride(-1) != 1:
            dy2 = dy2.to(x2.dtype).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.zeros(D, dtype=torch.float32, device=x2.device) if w32 is not None else None
        with torch.cuda.device(x2.device):
            rc = lib.mb200_rmsnorm_bwd(x2.data_ptr(), _lib.ptr(w32), rstd.data_ptr(), dy2.data_ptr(), dx.data_ptr(),
                                       _lib.ptr(dw), rows, D, x2.stride(0), dy2.stride(0), dx.stride(0),
                                       _lib.dtype_code(x2.dtype), _lib.current_stream(x2.device))
        _lib.check(rc, "mb200_rmsnorm_bwd")
        return dx.view(shape).to(tx), None if dw is None else dw.to(tw), None


def rms_norm(x, weight=None, eps=1e-5):
    """RMSNorm over the last dimension; weight None is the reference's muP variant (no gain)."""
    if not x.is_cuda:
        raise RuntimeError("mamba_b200 kernels need CUDA tensors; there is no CPU path")
    return RMSNormFn.apply(x, weight, eps)


class AddRMSNormFn(torch.autograd.Function):
    """(y, s) with s = x + residual and y = RMSNorm(s), one pass (mb200_add_rmsnorm_fwd)."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps, y_dtype):
        lib = _lib.load()
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        r2 = None
        res_dtype = x.dtype
        if residual is not None:
            r2 = residual.reshape(-1, D)
            if r2.stride(-1) != 1:
                r2 = r2.contiguous()
            res_dtype = torch.promote_types(x.dtype, residual.dtype)       # what `x + residual` would give
            if r2.dtype != res_dtype:
                r2 = r2.to(res_dtype)
        rows = x2.shape[0]
        w32 = None if weight is None else _f32(weight)
        s = torch.empty((rows, D), dtype=res_dtype, device=x.device)
        y = torch.empty((rows, D), dtype=y_dtype, device=x.device)
        rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            rc = lib.mb200_add_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(r2), _lib.ptr(w32), s.data_ptr(), y.data_ptr(),
                                           rstd.data_ptr(), rows, D, x2.stride(0), 0 if r2 is None else r2.stride(0),
                                           s.stride(0), y.stride(0), float(eps), _lib.dtype_code(x2.dtype),
                                           _lib.dtype_code(res_dtype), _lib.dtype_code(y_dtype),
                                           _lib.current_stream(x.device))
        _lib.check(rc, "mb200_add_rmsnorm_fwd")
        ctx.save_for_backward(s, w32, rstd)
        ctx.meta = (x.shape, x.dtype, None if residual is None else residual.dtype,
                    None if weight is None else weight.dtype)
        return y.view(x.shape), s.view(x.shape)

    @staticmethod
    def backward(ctx, dy, ds_out):
        s, w32, rstd = ctx.saved_tensors
        shape, tx, tr, tw = ctx.meta
        lib = _lib.load()
        rows, D = s.shape
        y_dtype = dy.dtype if dy.dtype in (torch.float32, torch.bfloat16) else torch.float32
        dy2 = dy.reshape(rows, D)
        if dy2.dtype != y_dtype or dy2.stride(-1) != 1:
            dy2 = dy2.to(y_dtype).contiguous()
        if s.dtype == torch.bfloat16 and y_dtype != torch.bfloat16:
            dy2, y_dtype = dy2.to(torch.bfloat16), torch.bfloat16
        dr2 = None
        if ds_out is not None:
            dr2 = ds_out.reshape(rows, D)
            if dr2.dtype != s.dtype or dr2.stride(-1) != 1:
                dr2 = dr2.to(s.dtype).contiguous()
        ds = torch.empty_like(s)
        dw = torch.zeros(D, dtype=torch.float32, device=s.device) if w32 is not None else None
        with torch.cuda.device(s.device):
            rc = lib.mb200_add_rmsnorm_bwd(s.data_ptr(), _lib.ptr(w32), rstd.data_ptr(), dy2.data_ptr(), _lib.ptr(dr2),
                                           ds.data_ptr(), _lib.ptr(dw), rows, D, s.stride(0), dy2.stride(0),
                                           0 if dr2 is None else dr2.stride(0), ds.stride(0),
                                           _lib.dtype_code(s.dtype), _lib.dtype_code(y_dtype),
                                           _lib.current_stream(s.device))
        _lib.check(rc, "mb200_add_rmsnorm_bwd")
        ds = ds.view(shape)
        return ds.to(tx), None if tr is None else ds.to(tr), None if dw is None else dw.to(tw), None, None


def add_rms_norm(x, residual=None, weight=None, eps=1e-5):
    """s = x + residual (residual None: s = x); y = RMSNorm(s).  Returns (y, s) from ONE pass over the data:
    the residual add of one layer fused with the normalisation in front of the next
    (mambapy/mamba.py:106-112).  Under autocast y comes out in the autocast dtype, which is what the
    projection that consumes it would cast it to anyway."""
    if not x.is_cuda:
        raise RuntimeError("mamba_b200 kernels need CUDA tensors; there is no CPU path")
    y_dtype = x.dtype if residual is None else torch.promote_types(x.dtype, residual.dtype)
    if torch.is_autocast_enabled():
        y_dtype = torch.get_autocast_gpu_dtype()
    if y_dtype not in (torch.float32, torch.bfloat16):
        y_dtype = torch.float32
    return AddRMSNormFn.apply(x, residual, weight, eps, y_dtype)


def stack_forward(self, x):
    """Drop-in for Mamba.forward (mambapy/mamba.py:77-85): the loop over ResidualBlocks
    (`x = mixer(norm(x)) + x`, mambapy/mamba.py:106-112) with each layer's residual add fused into the
    next layer's RMSNorm; the last add stays an ordinary add."""
    h, res = x, None
    for layer in self.layers:
        norm = layer.norm
        normed, res = add_rms_norm(h, res, None if getattr(norm, "use_mup", False) else norm.weight, norm.eps)
        h = layer.mixer(normed)
    return h + res if res is not None else h


def rmsnorm_forward(self, x):
    """Drop-in for RMSNorm.forward (mambapy/mamba.py:427-433)."""
    return rms_norm(x, None if getattr(self, "use_mup", False) else self.weight, self.eps)


def _project(self, x):
    """delta (pre-softplus, without bias), B, C from x as in mambapy/mamba.py:393-396."""
    cfg = self.config
    deltaBC = self.x_proj(x)
    delta, B, C = torch.split(deltaBC, [cfg.dt_rank, cfg.d_state, cfg.d_state], dim=-1)
    delta, B, C = self._apply_layernorms(delta, B, C)
    return delta, B, C


def ssm_step(self, x, h):
    """mambapy/mamba.py:384-414.  x: (B, ED); h: (B, ED, N) or None.  Returns (y, h)."""
    A = -torch.exp(self.A_log.float())
    delta, B, C = _project(self, x)
    delta = F.linear(delta, self.dt_proj.weight)          # bias and softplus happen in the kernel
    return ssm_step_fn(x, h, delta, A, B, C, self.D, delta_bias=self.dt_proj.bias)


def step(self, x, cache):
    """mambapy/mamba.py:351-382.  x: (B, D); cache = (h (B, ED, N) or None, inputs (B, ED, d_conv-1)).

    Returns (output (B, D), (h, inputs)) with fresh cache tensors."""
    h, inputs = cache
    xz = self.in_proj(x)
    xs, z = xz.chunk(2, dim=1)
    xc, inputs = conv_step_fn(xs, inputs, self.conv1d.weight, self.conv1d.bias)
    A = -torch.exp(self.A_log.float())
    delta, B, C = _project(self, xc)
    delta = F.linear(delta, self.dt_proj.weight)
    y, h = ssm_step_fn(xc, h, delta, A, B, C, self.D, z=z, delta_bias=self.dt_proj.bias)
    return self.out_proj(y), (h, inputs)


class FusedInnerFn(torch.autograd.Function):
    """Everything between in_proj and out_proj of MambaBlock.forward (mambapy/mamba.py:214-231) as ONE autograd
    node: conv1d + SiLU, x_proj, dt_proj, and the fused scan with softplus(delta + bias) and the gate inside.

    Written as separate nodes, autograd glues the backward together with copies: a `cat` of the gradients of
    the two halves of xz (the whole (B, L, 2*ED) tensor again), a `cat` for the split of the x_proj output, an
    add of the two gradients that reach the conv output, and casts of dB, dC.  Here the backward writes dz and
    the conv's dx straight into the two halves of d(xz), dB and dC straight into d(x_proj output), and adds
    the second gradient of the conv output in the epilogue of the GEMM that produces it."""

    @staticmethod
    def forward(ctx, xz, conv_w, conv_b, xproj_w, dt_w, dt_b, A_log, D, dt_rank, d_state):
        dt = xz.dtype
        ED = xz.shape[-1] // 2
        R, N = dt_rank, d_state
        xs, z = xz[..., :ED], xz[..., ED:]
        cw32 = conv_w.detach().reshape(ED, conv_w.shape[-1]).float().contiguous()
        cb32 = _f32(conv_b)
        xc = conv1d_silu_fwd_raw(xs, cw32, cb32)
        Wx, Wdt = xproj_w.detach().to(dt), dt_w.detach().to(dt)
        dbc = F.linear(xc, Wx)                                   # (B, L, R + 2N)
        delta_r = F.linear(dbc[..., :R], Wdt)                    # (B, L, ED); bias and softplus happen in the kernel
        A = -torch.exp(A_log.detach().float())
        D32, b32 = _f32(D), _f32(dt_b)
        needs_grad = any(ctx.needs_input_grad)
        y, _, carries = sscan_fwd_raw(xc, delta_r, A, dbc[..., R:R + N], dbc[..., R + N:], D32, z, b32,
                                      want_carries=needs_grad)
        ctx.save_for_backward(xz, xc, dbc, delta_r, A, D32, b32, carries, cw32, cb32, Wx, Wdt)
        ctx.meta = (R, N, conv_w.shape, conv_w.dtype, None if conv_b is None else conv_b.dtype, xproj_w.dtype,
                    dt_w.dtype, dt_b.dtype, A_log.dtype, D.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xz, xc, dbc, delta_r, A, D32, b32, carries, cw32, cb32, Wx, Wdt = ctx.saved_tensors
        R, N, cw_shape, t_cw, t_cb, t_wx, t_wdt, t_bdt, t_A, t_D = ctx.meta
        ED = xc.shape[-1]
        dy = _rows(dy, xc.dtype)
        dxz = torch.empty_like(xz, memory_format=torch.contiguous_format)
        dx_s, dd, _, dB, dC, dA, dD, dbias, _ = sscan_bwd_raw(
            xc, delta_r, A, dbc[..., R:R + N], dbc[..., R + N:], D32, xz[..., ED:], b32, dy, carries,
            out_dz=dxz[..., ED:])
        d_dbc = torch.empty_like(dbc)
        dd2 = dd.flatten(0, 1)
        d_dbc[..., :R] = F.linear(dd, Wdt.t())                   # through dt_proj
        d_dbc[..., R:R + N].copy_(dB)                            # float32 accumulators -> activation dtype, in place
        d_dbc[..., R + N:].copy_(dC)
        d2 = d_dbc.flatten(0, 1)
        dWdt = dd2.t() @ dbc[..., :R].flatten(0, 1)              # (ED, R)
        dWx = d2.t() @ xc.flatten(0, 1)                          # (R + 2N, ED)
        dx_s.flatten(0, 1).addmm_(d2, Wx)                        # + gradient through x_proj, in the GEMM's epilogue
        _, dcw, dcb = conv1d_silu_bwd_raw(xz[..., :ED], cw32, cb32, dx_s, out_dx=dxz[..., :ED])
        return (dxz, dcw.reshape(cw_shape).to(t_cw), None if dcb is None else dcb.to(t_cb), dWx.to(t_wx), dWdt.to(t_wdt),
                dbias.to(t_bdt), (dA * A).to(t_A), dD.to(t_D), None, None)


def _fusable(self, xz):
    cfg = self.config
    return (xz.is_cuda and xz.dtype in (torch.float32, torch.bfloat16) and self.conv1d.weight.shape[-1] == 4
            and getattr(self, "dt_layernorm", None) is None and getattr(self, "B_layernorm", None) is None
            and getattr(self, "C_layernorm", None) is None and cfg.d_state in (8, 16, 32, 64))


def ssm(self, x, z):
    """mambapy/mamba.py:236-272 with softplus(delta + dt_bias), the scan and the gate fused.

    Like the reference's own fused branch (mambapy/mamba.py:252-261) this returns the GATED y,
    so the matching `forward` below skips the z branch."""
    A = -torch.exp(self.A_log.float())
    delta, B, C = _project(self, x)
    delta = F.linear(delta, self.dt_proj.weight)          # (B, L, ED), no transposes needed
    return selective_scan_fn(x, delta, A, B, C, self.D, z=z, delta_bias=self.dt_proj.bias)


def forward(self, x):
    """mambapy/mamba.py:205-234 with the scan path fused; x: (B, L, D) -> (B, L, D)."""
    _, L, _ = x.shape
    xz = self.in_proj(x)
    if _fusable(self, xz):
        cfg = self.config
        y = FusedInnerFn.apply(xz, self.conv1d.weight, self.conv1d.bias, self.x_proj.weight, self.dt_proj.weight,
                               self.dt_proj.bias, self.A_log, self.D, cfg.dt_rank, cfg.d_state)
        return self.out_proj(y)
    xs, z = xz.chunk(2, dim=-1)
    if self.conv1d.weight.shape[-1] == 4:
        xs = causal_conv1d_silu(xs, self.conv1d.weight, self.conv1d.bias)
    else:
        xs = F.silu(self.conv1d(xs.transpose(1, 2))[:, :, :L].transpose(1, 2))
    y = ssm(self, xs, z)
    return self.out_proj(y)
