"""CPU oracle for the selective-scan path of mamba.py.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic that the reference
performs on its scan path.  It exists so the CUDA kernels can be checked against it
and so the reference's own algorithm can be timed on host cores.  Nothing in the
shipped package imports it; the product path never routes through it.

Parity status: PINNED.  The functions below are checked (tests/test_oracle.py)
against golden vectors produced by importing and running the unmodified reference
(tests/golden/make_golden.py wrote them), and against the one known-answer vector
the reference's own docs hold (docs/tests.ipynb cell 1).

What follows which reference lines (paths inside the reference project):
  blelloch_scan_         mambapy/pscan.py:36-92    (PScan.pscan, in-place up/down sweep)
  blelloch_scan_rev_     mambapy/pscan.py:94-149   (PScan.pscan_rev)
  pscan_forward          mambapy/pscan.py:151-186  (PScan.forward: pad to 2^k, clone, sweep)
  pscan_backward         mambapy/pscan.py:188-224  (PScan.backward)
  selective_scan         mambapy/mamba.py:274-295  (discretise, scan, C-contraction, D skip)
  selective_scan_seq     mambapy/mamba.py:297-327  (same with a loop over t)
  gate                   mambapy/mamba.py:229-231  (y * silu(z))
  ssm_step               mambapy/mamba.py:384-414  (one decode step of the SSM)
  block_step             mambapy/mamba.py:351-382  (conv window, silu, ssm_step, gate, cache)
  selective_scan_f64     mambapy/mamba.py:297-327 in float64, the arbiter for 1e-6 disputes
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- pscan

def next_pow2(n: int) -> int:
    """Smallest power of two >= n (mambapy/pscan.py:13-18)."""
    return 1 << max(0, math.ceil(math.log2(n))) if n > 0 else 1


def _pad_len_pow2(T: torch.Tensor) -> torch.Tensor:
    """Zero-pad dim 1 of a (B, L, D, N) tensor up to a power of two (pscan.py:20-33)."""
    L = T.size(1)
    return F.pad(T, (0, 0, 0, 0, 0, next_pow2(L) - L))


def blelloch_scan_(A: torch.Tensor, X: torch.Tensor) -> None:
    """In-place inclusive scan of H[t] = A[t]*H[t-1] + X[t] over dim 2 of (B, D, L, N).

    L must be a power of two.  Both A and X are overwritten.  The combine order is the
    reference's: an up-sweep over node pairs down to four nodes, a hand-unrolled
    4-node (or 2-node) root, then a down-sweep (pscan.py:52-92).  Nodes of level k
    live at positions 2^k - 1 + j*2^k, so each level is a pair of strided slices.
    """
    L = A.size(2)
    levels = int(math.log2(L))
    for k in range(levels - 2):                      # up-sweep, pscan.py:54-63
        s = 1 << k
        lo = slice(s - 1, L, 2 * s)
        hi = slice(2 * s - 1, L, 2 * s)
        X[:, :, hi].add_(A[:, :, hi].mul(X[:, :, lo]))
        A[:, :, hi].mul_(A[:, :, lo])
    nodes = L if levels < 2 else 4
    s = L // nodes
    n = [i * s + s - 1 for i in range(nodes)]        # surviving node positions
    if nodes == 4:                                    # pscan.py:66-70
        X[:, :, n[1]].add_(A[:, :, n[1]].mul(X[:, :, n[0]]))
        A[:, :, n[1]].mul_(A[:, :, n[0]])
        X[:, :, n[3]].add_(A[:, :, n[3]].mul(X[:, :, n[2]] + A[:, :, n[2]].mul(X[:, :, n[1]])))
    elif nodes == 2:                                  # pscan.py:71-73
        X[:, :, n[1]].add_(A[:, :, n[1]].mul(X[:, :, n[0]]))
        return
    else:
        return
    X[:, :, n[2]].add_(A[:, :, n[2]].mul(X[:, :, n[1]]))   # pscan.py:78-81
    A[:, :, n[2]].mul_(A[:, :, n[1]])
    for k in range(levels - 3, -1, -1):              # down-sweep, pscan.py:83-92
        s = 1 << k
        tgt = slice(3 * s - 1, L, 2 * s)             # even nodes from the second pair on
        src = slice(2 * s - 1, L - s, 2 * s)         # the odd node just before each
        X[:, :, tgt].add_(A[:, :, tgt].mul(X[:, :, src]))
        A[:, :, tgt].mul_(A[:, :, src])


def blelloch_scan_rev_(A: torch.Tensor, X: torch.Tensor) -> None:
    """Mirror image of blelloch_scan_: G[t] = X[t] + A[t]*G[t+1] (pscan.py:94-149)."""
    L = A.size(2)
    levels = int(math.log2(L))
    for k in range(levels - 2):                      # pscan.py:108-119
        s = 1 << k
        lo = slice(0, L, 2 * s)
        hi = slice(s, L, 2 * s)
        X[:, :, lo].add_(A[:, :, lo].mul(X[:, :, hi]))
        A[:, :, lo].mul_(A[:, :, hi])
    nodes = L if levels < 2 else 4
    s = L // nodes
    n = [i * s for i in range(nodes)]
    if nodes == 4:                                    # pscan.py:122-126
        X[:, :, n[2]].add_(A[:, :, n[2]].mul(X[:, :, n[3]]))
        A[:, :, n[2]].mul_(A[:, :, n[3]])
        X[:, :, n[0]].add_(A[:, :, n[0]].mul(X[:, :, n[1]].add(A[:, :, n[1]].mul(X[:, :, n[2]]))))
    elif nodes == 2:                                  # pscan.py:127-129
        X[:, :, n[0]].add_(A[:, :, n[0]].mul(X[:, :, n[1]]))
        return
    else:
        return
    X[:, :, n[1]].add_(A[:, :, n[1]].mul(X[:, :, n[2]]))   # pscan.py:134-137
    A[:, :, n[1]].mul_(A[:, :, n[2]])
    for k in range(levels - 3, -1, -1):              # pscan.py:139-149
        s = 1 << k
        tgt = slice(s, L - s, 2 * s)                 # odd nodes except the last
        src = slice(2 * s, L, 2 * s)                 # the even node just after each
        X[:, :, tgt].add_(A[:, :, tgt].mul(X[:, :, src]))
        A[:, :, tgt].mul_(A[:, :, src])


def pscan_forward(A_in: torch.Tensor, X_in: torch.Tensor):
    """H of shape (B, L, D, N) plus what the reference saves for backward.

    Inputs are left untouched (the reference clones or pads them, pscan.py:168-174).
    Returns (H, saved) where saved = (A_in, Hpad) and Hpad is the padded (B, D, Lp, N)
    view the reference keeps (pscan.py:183).
    """
    L = X_in.size(1)
    if L == next_pow2(L):
        A = A_in.clone()
        X = X_in.clone()
    else:
        A = _pad_len_pow2(A_in)
        X = _pad_len_pow2(X_in)
    A = A.transpose(2, 1)
    X = X.transpose(2, 1)
    blelloch_scan_(A, X)
    return X.transpose(2, 1)[:, :L], (A_in, X)


def pscan_backward(saved, grad_out: torch.Tensor):
    """(gradA, gradX) for pscan_forward (pscan.py:188-224).

    gradX is the reverse scan of grad_out with A shifted one step left; gradA[t] is
    H[t-1] * gradX[t] with gradA[0] = 0.
    """
    A_in, H = saved
    L = grad_out.size(1)
    if L == next_pow2(L):
        G = grad_out.clone()
    else:
        G = _pad_len_pow2(grad_out)
        A_in = _pad_len_pow2(A_in)
    G = G.transpose(2, 1)
    A_in = A_in.transpose(2, 1)
    A = F.pad(A_in[:, :, 1:], (0, 0, 0, 1))
    blelloch_scan_rev_(A, G)
    Q = torch.zeros_like(H)
    Q[:, :, 1:].add_(H[:, :, :-1] * G[:, :, 1:])
    return Q.transpose(2, 1)[:, :L], G.transpose(2, 1)[:, :L]


class _PScanOracle(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A_in, X_in):
        H, saved = pscan_forward(A_in, X_in)
        ctx.save_for_backward(*saved)
        return H

    @staticmethod
    def backward(ctx, g):
        return pscan_backward(ctx.saved_tensors, g)


pscan = _PScanOracle.apply


def scan_sequential(A: torch.Tensor, X: torch.Tensor, h0: torch.Tensor | None = None) -> torch.Tensor:
    """Plain loop over t for H[t] = A[t]*H[t-1] + X[t]; inputs (B, L, D, N)."""
    h = torch.zeros_like(X[:, 0]) if h0 is None else h0
    out = []
    for t in range(X.size(1)):
        h = A[:, t] * h + X[:, t]
        out.append(h)
    return torch.stack(out, dim=1)


# ------------------------------------------------------------------- selective scan

def selective_scan(x, delta, A, B, C, D, scan=pscan):
    """y of shape (B, L, ED) by the reference's parallel-scan route (mamba.py:274-295)."""
    dA = torch.exp(delta.unsqueeze(-1) * A)
    dBx = (delta.unsqueeze(-1) * B.unsqueeze(2)) * x.unsqueeze(-1)
    hs = scan(dA, dBx)
    y = (hs @ C.unsqueeze(-1)).squeeze(3)
    return y + D * x


def selective_scan_seq(x, delta, A, B, C, D, h0=None, return_last_state=False):
    """Same result with an explicit loop over t (mamba.py:297-327)."""
    dA = torch.exp(delta.unsqueeze(-1) * A)
    dBx = (delta.unsqueeze(-1) * B.unsqueeze(2)) * x.unsqueeze(-1)
    h = torch.zeros(x.size(0), x.size(2), A.size(1), dtype=dA.dtype) if h0 is None else h0
    hs = []
    for t in range(x.size(1)):
        h = dA[:, t] * h + dBx[:, t]
        hs.append(h)
    hs = torch.stack(hs, dim=1)
    y = (hs @ C.unsqueeze(-1)).squeeze(3) + D * x
    return (y, h) if return_last_state else y


def gate(y, z):
    """The z branch of MambaBlock.forward (mamba.py:229-231)."""
    return y * F.silu(z)


def selective_scan_f64(x, delta, A, B, C, D, z=None, h0=None, return_last_state=False):
    """Float64 sequential arbiter; differentiable, so autograd gives reference gradients.

    Inputs of any float dtype are promoted to float64 first; the optional gate and an
    optional incoming state h0 (B, ED, N) are included so that sharded and chunked
    variants of the kernels have a single-sequence answer to be compared with.
    """
    f = lambda t: None if t is None else t.double()
    x, delta, A, B, C, D, z, h0 = map(f, (x, delta, A, B, C, D, z, h0))
    out = selective_scan_seq(x, delta, A, B, C, D, h0=h0, return_last_state=True)
    y, h = out
    if z is not None:
        y = gate(y, z)
    return (y, h) if return_last_state else y


# --------------------------------------------------------------------------- decode

def ssm_step(x, h, delta, A, B, C, D):
    """One recurrent step given the already-projected delta (post-softplus), B, C.

    mamba.py:400-412: h' = exp(delta*A)*h + delta*B*x ; y = h'.C + D*x.  h may be None.
    """
    dA = torch.exp(delta.unsqueeze(-1) * A)
    dBx = (delta.unsqueeze(-1) * B.unsqueeze(1)) * x.unsqueeze(-1)
    if h is None:
        h = torch.zeros(x.size(0), x.size(1), A.size(1), dtype=dA.dtype)
    h = dA * h + dBx
    y = (h @ C.unsqueeze(-1)).squeeze(2) + D * x
    return y, h


def block_step(x, cache, W):
    """MambaBlock.step on explicit weights (mamba.py:351-382).

    W is a dict of tensors: in_proj (2ED, D), conv_w (ED, 1, K), conv_b (ED),
    x_proj (R+2N, ED), dt_w (ED, R), dt_b (ED), A_log (ED, N), D (ED), out_proj (D, ED).
    cache = (h or None, inputs (B, ED, K-1)).  Returns (out, (h', inputs')).
    """
    h, inputs = cache
    ED, N = W["A_log"].shape
    R = W["dt_w"].shape[1]
    K = W["conv_w"].shape[2]
    xz = x @ W["in_proj"].t()
    xs, z = xz.chunk(2, dim=1)
    x_cache = xs.unsqueeze(2)
    win = torch.cat([inputs, x_cache], dim=2)                       # (B, ED, K)
    xc = F.conv1d(win, W["conv_w"], W["conv_b"], padding=K - 1, groups=ED)[:, :, K - 1]
    xc = F.silu(xc)
    A = -torch.exp(W["A_log"].float())
    dBC = xc @ W["x_proj"].t()
    dlt, Bm, Cm = torch.split(dBC, [R, N, N], dim=-1)
    dlt = F.softplus(dlt @ W["dt_w"].t() + W["dt_b"])
    y, h = ssm_step(xc, h, dlt, A, Bm, Cm, W["D"].float())
    out = (y * F.silu(z)) @ W["out_proj"].t()
    inputs = torch.cat([inputs[:, :, 1:], x_cache], dim=2)
    return out, (h, inputs)


# ------------------------------------------------- closed-form float64 forward + backward, for wide problems

def selective_scan_fwd_bwd_f64(x, delta, A, B, C, D, gy, z=None, delta_bias=None, h0=None, block=512):
    """y, last state and EVERY gradient of the gated selective scan in float64, without autograd.

    The forward is the sequential loop of mamba.py:297-327 (plus the gate, mamba.py:229-231, and
    softplus(delta + delta_bias), mamba.py:264-265, when `delta_bias` is given); the backward is the
    hand-derived adjoint of exactly those lines (the reference gets it from autograd and, for the
    scan, from PScan.backward, pscan.py:188-224):
        dy' = gy*silu(z);  g[t] = dy'[t] C[t] + a[t+1] g[t+1];  da[t] = g[t] h[t-1]
        dx = dy' D + delta sum_n g B        ddelta = sum_n (g B x + da a A)
        dB = sum_e g delta x                dC = sum_e dy' h
        dA = sum_{b,t} da a delta           dD = sum_{b,t} dy' x
        dz = gy y_ungated silu'(z)          d(delta_raw) = ddelta*sigmoid(raw+bias) = d(bias) summed
    Only the two recurrences loop over t; everything else is one vectorised pass, and channels are
    processed `block` at a time (they are independent; dB and dC add up over blocks), so that a row of
    the 130m layer (L 2048, ED 1536) takes seconds where the autograd tape of the loop takes minutes.
    tests/test_oracle.py checks it against autograd of selective_scan_seq.

    Returns (y, hT, grads) with grads keyed x, delta, A, B, C, D and, when given, z, bias, h0.
    """
    f = lambda t: None if t is None else t.detach().double()
    x, delta, A, B, C, D, gy, z, delta_bias, h0 = map(f, (x, delta, A, B, C, D, gy, z, delta_bias, h0))
    Bsz, L, ED = x.shape
    N = A.shape[1]
    ys, hTs = [], []
    per = {k: [] for k in ("x", "delta", "A", "D", "z", "bias", "h0")}
    gB = torch.zeros(Bsz, L, N, dtype=torch.float64)
    gC = torch.zeros(Bsz, L, N, dtype=torch.float64)
    for e0 in range(0, ED, block):
        sl = slice(e0, min(ED, e0 + block))
        xb, rawb, Ab, Db, gyb = x[..., sl], delta[..., sl], A[sl], D[sl], gy[..., sl]
        db = F.softplus(rawb + delta_bias[sl]) if delta_bias is not None else rawb
        a = torch.exp(db.unsqueeze(-1) * Ab)                                  # (B, L, E, N)
        u = (db * xb).unsqueeze(-1) * B.unsqueeze(2)
        hs = torch.empty_like(a)
        h = torch.zeros(Bsz, xb.shape[2], N, dtype=torch.float64) if h0 is None else h0[:, sl].clone()
        h_first = h.clone()
        for t in range(L):
            h = torch.addcmul(u[:, t], a[:, t], h)
            hs[:, t] = h
        y_ssm = (hs * C.unsqueeze(2)).sum(-1) + Db * xb
        if z is not None:
            zb = z[..., sl]
            sg = torch.sigmoid(zb)
            silu = zb * sg
            ys.append(y_ssm * silu)
            dyp = gyb * silu
            per["z"].append(gyb * y_ssm * sg * (1 + zb * (1 - sg)))
        else:
            ys.append(y_ssm)
            dyp = gyb
        hTs.append(h)
        g = torch.empty_like(a)
        inj = dyp.unsqueeze(-1) * C.unsqueeze(2)
        acc = torch.zeros_like(h)
        for t in range(L - 1, -1, -1):
            acc = inj[:, t] + (a[:, t + 1] * acc if t + 1 < L else 0)
            g[:, t] = acc
        hprev = torch.cat([h_first.unsqueeze(1), hs[:, :-1]], dim=1)
        daa = g * hprev * a                                                  # da * a
        gBsum = (g * B.unsqueeze(2)).sum(-1)                                 # sum_n g B   (B, L, E)
        per["x"].append(dyp * Db + db * gBsum)
        ddelta = xb * gBsum + (daa * Ab).sum(-1)
        if delta_bias is not None:
            ddelta = ddelta * torch.sigmoid(rawb + delta_bias[sl])
            per["bias"].append(ddelta.sum((0, 1)))
        per["delta"].append(ddelta)
        per["A"].append((daa * db.unsqueeze(-1)).sum((0, 1)))
        per["D"].append((dyp * xb).sum((0, 1)))
        per["h0"].append(a[:, 0] * g[:, 0])
        gB += (g * (db * xb).unsqueeze(-1)).sum(2)
        gC += (hs * dyp.unsqueeze(-1)).sum(2)
    grads = {"x": torch.cat(per["x"], -1), "delta": torch.cat(per["delta"], -1), "A": torch.cat(per["A"], 0),
             "D": torch.cat(per["D"], 0), "B": gB, "C": gC}
    if z is not None:
        grads["z"] = torch.cat(per["z"], -1)
    if delta_bias is not None:
        grads["bias"] = torch.cat(per["bias"], 0)
    if h0 is not None:
        grads["h0"] = torch.cat(per["h0"], 1)
    return torch.cat(ys, -1), torch.cat(hTs, 1), grads
