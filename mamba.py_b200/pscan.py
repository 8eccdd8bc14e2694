"""Drop-in for the reference's mambapy/pscan.py: `PScan`, `pscan`, `npo2`, `pad_npo2`.

`pscan(A_in, X_in)` returns H with H[t] = A[t]*H[t-1] + X[t] along dim 1 of (B, L, D, N)
tensors and is differentiable w.r.t. both inputs, exactly as mambapy/pscan.py:151-226.
Differences that a caller cannot observe through the values: L is not padded to a power of
two, nothing is cloned (the inputs are only read), and the result is a fresh contiguous
tensor.  The work happens in libmamba_b200.so; CPU tensors are rejected.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib


def npo2(len):
    """Next power of two above len (mambapy/pscan.py:13-18); kept for API compatibility."""
    return 2 ** math.ceil(math.log2(len))


def pad_npo2(X):
    """Zero-pad dim 1 of (B, L, D, N) to a power of two (mambapy/pscan.py:20-33).

    The kernels take any L, so nothing in this package calls it."""
    return F.pad(X, (0, 0, 0, 0, 0, npo2(X.size(1)) - X.size(1)), "constant", 0)


def _dense_dn(t: torch.Tensor) -> torch.Tensor:
    """(B, L, D, N) view whose (D, N) block is dense; copies only if it is not."""
    N, D = t.size(3), t.size(2)
    if t.stride(3) == 1 and (D == 1 or t.stride(2) == N):
        return t
    return t.contiguous()


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mamba_b200 runs on CUDA tensors only (there is no CPU path)")


def pscan_fwd_raw(A, X, h0=None, want_last=False):
    """Launch the forward kernel.  Returns (H, hT or None)."""
    _require_cuda(A, X, h0)
    if A.shape != X.shape or A.dim() != 4:
        raise ValueError(f"pscan expects two (B, L, D, N) tensors, got {tuple(A.shape)} and {tuple(X.shape)}")
    if A.dtype != X.dtype:
        raise TypeError("A_in and X_in must have the same dtype")
    code = _lib.dtype_code(X.dtype)
    lib = _lib.load()
    B, L, D, N = X.shape
    A, X = _dense_dn(A), _dense_dn(X)
    H = torch.empty((B, L, D, N), dtype=X.dtype, device=X.device)
    hT = torch.empty((B, D * N), dtype=torch.float32, device=X.device) if want_last else None
    if h0 is not None:
        h0 = h0.reshape(B, D * N).float().contiguous()
    nseg = lib.mb200_pscan_segments(B, L, D * N) if L > 0 else 1
    ws = torch.empty(2 * B * nseg * D * N, dtype=torch.float32, device=X.device) if nseg > 1 else None
    with torch.cuda.device(X.device):
        rc = lib.mb200_pscan_fwd(A.data_ptr(), X.data_ptr(), H.data_ptr(), B, L, D * N,
                                 A.stride(0), A.stride(1), X.stride(0), X.stride(1),
                                 H.stride(0), H.stride(1), _lib.ptr(h0), _lib.ptr(hT), _lib.ptr(ws),
                                 nseg, code, _lib.current_stream(X.device))
    _lib.check(rc, "mb200_pscan_fwd")
    return H, hT


def pscan_bwd_raw(A, H, G, h0=None):
    """Launch the backward kernel.  Returns (gradA, gradX)."""
    _require_cuda(A, H, G)
    code = _lib.dtype_code(H.dtype)
    lib = _lib.load()
    B, L, D, N = H.shape
    A, H, G = _dense_dn(A), _dense_dn(H), _dense_dn(G.to(H.dtype))
    gA = torch.empty((B, L, D, N), dtype=H.dtype, device=H.device)
    gX = torch.empty_like(gA)
    nseg = lib.mb200_pscan_segments(B, L, D * N) if L > 0 else 1
    ws = torch.empty(2 * B * nseg * D * N, dtype=torch.float32, device=H.device) if nseg > 1 else None
    with torch.cuda.device(H.device):
        rc = lib.mb200_pscan_bwd(A.data_ptr(), H.data_ptr(), G.data_ptr(), gA.data_ptr(), gX.data_ptr(),
                                 B, L, D * N, A.stride(0), A.stride(1), H.stride(0), H.stride(1),
                                 G.stride(0), G.stride(1), gA.stride(0), gA.stride(1),
                                 gX.stride(0), gX.stride(1), _lib.ptr(h0), _lib.ptr(ws), nseg, code,
                                 _lib.current_stream(H.device))
    _lib.check(rc, "mb200_pscan_bwd")
    return gA, gX


class PScan(torch.autograd.Function):
    """Same call contract as mambapy/pscan.py:35-224 (`PScan.apply(A_in, X_in)`)."""

    @staticmethod
    def forward(ctx, A_in, X_in):
        """
        Args:
            A_in : (B, L, D, N)
            X_in : (B, L, D, N)
        Returns:
            H : (B, L, D, N)
        """
        H, _ = pscan_fwd_raw(A_in, X_in)
        ctx.save_for_backward(A_in, H)
        return H

    @staticmethod
    def backward(ctx, grad_output_in):
        """Returns gradA, gradX, both (B, L, D, N) (mambapy/pscan.py:188-224)."""
        A_in, H = ctx.saved_tensors
        gA, gX = pscan_bwd_raw(A_in, H, grad_output_in)
        return gA, gX


pscan = PScan.apply
