"""Fused selective-scan kernels against the reference's golden vectors and the float64 oracle."""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as O
from tests.helpers import golden, scan_inputs, assert_close

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5          # float32 contract
BF_RTOL, BF_ATOL = 2e-2, 2e-2    # bf16 I/O with float32 state

DEV = "cuda:0"


def _oracle(inp, gated=True, h0=None, bias=None):
    leaves = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")}
    delta = leaves["delta"]
    bleaf = None
    if bias is not None:
        bleaf = bias.double().requires_grad_()
        delta = torch.nn.functional.softplus(delta + bleaf)
    h0l = None if h0 is None else h0.double().requires_grad_()
    y, hT = O.selective_scan_f64(leaves["x"], delta, leaves["A"], leaves["B"], leaves["C"], leaves["D"],
                                 z=leaves["z"] if gated else None, h0=h0l, return_last_state=True)
    y.backward(inp["gy"].double())
    grads = {k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in leaves.items()}
    if bleaf is not None:
        grads["bias"] = bleaf.grad
    if h0l is not None:
        grads["h0"] = h0l.grad
    return y.detach(), hT.detach(), grads


def _kernel(inp, dtype, gated=True, h0=None, bias=None, subshards=None):
    import mamba_b200
    act = lambda k: inp[k].to(DEV).to(dtype).requires_grad_()
    par = lambda k: inp[k].to(DEV).requires_grad_()
    leaves = dict(x=act("x"), delta=act("delta"), A=par("A"), B=act("B"), C=act("C"), D=par("D"), z=act("z"))
    bl = None if bias is None else bias.to(DEV).requires_grad_()
    h0l = None if h0 is None else h0.to(DEV).requires_grad_()
    y, hT = mamba_b200.selective_scan_fn(leaves["x"], leaves["delta"], leaves["A"], leaves["B"], leaves["C"],
                                         leaves["D"], z=leaves["z"] if gated else None, delta_bias=bl,
                                         h0=h0l, return_last_state=True, subshards=subshards)
    y.backward(inp["gy"].to(DEV).to(dtype))
    grads = {k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in leaves.items()}
    if bl is not None:
        grads["bias"] = bl.grad
    if h0l is not None:
        grads["h0"] = h0l.grad
    return y.detach(), hT.detach(), grads


def _compare(inp, dtype, rtol, atol, subshards=None, **kw):
    yo, ho, go = _oracle(inp, **kw)
    yk, hk, gk = _kernel(inp, dtype, subshards=subshards, **kw)
    assert yk.dtype == dtype
    assert_close(yk, yo.float(), rtol, atol, "y")
    assert_close(hk, ho.float(), rtol, atol, "last state")
    for k in go:
        if k == "z" and not kw.get("gated", True):
            continue
        # sums over many terms (dA, dD, dB, dC, bias) carry accumulated rounding: scale atol
        scale = go[k].abs().max().item() + 1e-30
        assert_close(gk[k], go[k].float(), rtol, max(atol, atol * scale * 4), f"grad {k}")


def test_golden_small_config():
    """The small CPU config of the reference: outputs and every gradient, gated and un-gated."""
    import mamba_b200
    g = golden("selective_scan.npz")
    t = lambda k: torch.from_numpy(g[k]).to(DEV)
    for gated in (False, True):
        leaves = [t(k).requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")]
        x, dl, A, Bm, Cm, D, z = leaves
        y = mamba_b200.selective_scan_fn(x, dl, A, Bm, Cm, D, z=z if gated else None)
        y.backward(t("gy"))
        for route in ("pscan", "seq"):
            assert_close(y, g[f"{route}_yg" if gated else f"{route}_y"], RTOL, ATOL, f"y {route}")
            names = ("x", "delta", "A", "B", "C", "D") + (("z",) if gated else ())
            for nm, leaf in zip(names, leaves):
                key = f"{route}_g{nm}" if gated else f"{route}_ung_g{nm}"
                scale = float(np.abs(g[key]).max())
                assert_close(leaf.grad, g[key], RTOL, max(ATOL, ATOL * scale * 4), f"grad {nm} {route} gated={gated}")


def test_method_dropins_match_golden():
    """selective_scan / selective_scan_seq with the reference's method signature."""
    from mamba_b200 import selective_scan, selective_scan_seq
    g = golden("selective_scan.npz")
    t = lambda k: torch.from_numpy(g[k]).to(DEV)
    for fn in (selective_scan, selective_scan_seq):
        y = fn(None, t("x"), t("delta"), t("A"), t("B"), t("C"), t("D"))
        assert_close(y, g["pscan_y"], RTOL, ATOL)
        assert_close(y, g["seq_y"], RTOL, ATOL)


@pytest.mark.parametrize("Bsz,L,ED,N", [(2, 64, 32, 16), (1, 1, 8, 16), (3, 17, 40, 16), (2, 100, 33, 16),
                                          (1, 250, 64, 8), (2, 77, 24, 32), (1, 50, 16, 64), (2, 31, 5, 8)])
@pytest.mark.parametrize("gated", [True, False])
def test_f32_vs_f64_oracle(Bsz, L, ED, N, gated):
    inp = scan_inputs(100 + L + ED + N, Bsz, L, ED, N, structured_A=(N == 16))
    _compare(inp, torch.float32, RTOL, ATOL, gated=gated)


def test_f32_with_state_and_softplus():
    inp = scan_inputs(42, 2, 90, 48, 16, structured_A=False, big_delta=True)
    g = torch.Generator().manual_seed(43)
    h0 = torch.randn(2, 48, 16, generator=g)
    bias = torch.randn(48, generator=g) * 0.5 - 3.0
    inp["delta"] = torch.randn(2, 90, 48, generator=g)           # raw delta, softplus inside
    _compare(inp, torch.float32, RTOL, ATOL, gated=True, h0=h0, bias=bias)


@pytest.mark.parametrize("Bsz,L,ED,N", [(2, 64, 32, 16), (2, 130, 72, 16), (1, 45, 20, 16), (1, 64, 32, 64)])
def test_bf16_io_fp32_state(Bsz, L, ED, N):
    """bf16 activations, float32 state; the oracle sees the same bf16-rounded inputs."""
    inp = scan_inputs(7 + L, Bsz, L, ED, N, dtype=torch.bfloat16)
    yo, ho, go = _oracle(inp)
    yk, hk, gk = _kernel(inp, torch.bfloat16)
    assert yk.dtype == torch.bfloat16
    assert_close(yk, yo.float(), BF_RTOL, BF_ATOL, "y")
    assert_close(hk, ho.float(), RTOL, ATOL, "state stays float32")
    for k in ("x", "delta", "z", "B", "C", "A", "D"):
        scale = go[k].abs().max().item()
        assert_close(gk[k], go[k].float(), BF_RTOL, BF_ATOL * max(1.0, scale), f"grad {k}")


def test_strided_views_like_the_block_feeds():
    """x and z as chunk() views of one tensor, B and C as split() views (mambapy/mamba.py:214,245)."""
    import mamba_b200
    inp = scan_inputs(9, 2, 70, 32, 16)
    xz = torch.cat([inp["x"], inp["z"]], -1).to(DEV)
    dbc = torch.cat([torch.zeros(2, 70, 2), inp["B"], inp["C"]], -1).to(DEV)
    x, z = xz.chunk(2, dim=-1)
    _, Bm, Cm = torch.split(dbc, [2, 16, 16], dim=-1)
    y = mamba_b200.selective_scan_fn(x, inp["delta"].to(DEV), inp["A"].to(DEV), Bm, Cm, inp["D"].to(DEV), z=z)
    yo, _, _ = _oracle(inp)
    assert_close(y, yo.float(), RTOL, ATOL)


def test_split_sequence_consistency_full_width():
    """At the benchmark layer width: forward over L equals two halves chained through the state,
    and the backward of the halves chained through the gradient carry equals the whole."""
    from mamba_b200.mamba import sscan_fwd_raw, sscan_bwd_raw
    Bsz, L, ED, N = 2, 2048, 1536, 16
    g = torch.Generator(device="cuda").manual_seed(3)
    r = lambda *s: torch.randn(*s, generator=g, device=DEV)
    x, z, dy = r(Bsz, L, ED), r(Bsz, L, ED), r(Bsz, L, ED)
    delta = torch.nn.functional.softplus(r(Bsz, L, ED) * 0.5 - 4.6)
    A = -torch.arange(1, N + 1, device=DEV, dtype=torch.float32).repeat(ED, 1)
    Bm, Cm, D = r(Bsz, L, N), r(Bsz, L, N), torch.ones(ED, device=DEV)
    y, hT, car = sscan_fwd_raw(x, delta, A, Bm, Cm, D, z, want_last=True, want_carries=True)
    full = sscan_bwd_raw(x, delta, A, Bm, Cm, D, z, None, dy, car, want_g_out=True)
    m = 1024                                  # a multiple of the carry spacing
    sl = lambda t, a, b: t[:, a:b]
    y0, h0, c0 = sscan_fwd_raw(sl(x, 0, m), sl(delta, 0, m), A, sl(Bm, 0, m), sl(Cm, 0, m), D, sl(z, 0, m),
                               want_last=True, want_carries=True)
    y1, h1, c1 = sscan_fwd_raw(sl(x, m, L), sl(delta, m, L), A, sl(Bm, m, L), sl(Cm, m, L), D, sl(z, m, L),
                               h0=h0, want_last=True, want_carries=True)
    assert torch.allclose(torch.cat([y0, y1], 1), y, rtol=1e-5, atol=1e-6)
    assert torch.allclose(h1, hT, rtol=1e-5, atol=1e-6)
    b1 = sscan_bwd_raw(sl(x, m, L), sl(delta, m, L), A, sl(Bm, m, L), sl(Cm, m, L), D, sl(z, m, L), None,
                       sl(dy, m, L), c1, want_g_out=True)
    b0 = sscan_bwd_raw(sl(x, 0, m), sl(delta, 0, m), A, sl(Bm, 0, m), sl(Cm, 0, m), D, sl(z, 0, m), None,
                       sl(dy, 0, m), c0, g_in=b1[8], want_g_out=True)
    for i, nm in enumerate(("dx", "ddelta", "dz", "dB", "dC")):
        assert torch.allclose(torch.cat([b0[i], b1[i]], 1), full[i], rtol=1e-4, atol=1e-5), nm
    assert torch.allclose(b0[5] + b1[5], full[5], rtol=1e-3, atol=1e-3), "dA"
    assert torch.allclose(b0[6] + b1[6], full[6], rtol=1e-3, atol=1e-3), "dD"
    assert torch.allclose(b0[8], full[8], rtol=1e-4, atol=1e-6), "carry leaving t=0"


def test_linearity_in_x_full_width():
    """y is linear in x for fixed delta, A, B, C (D included): y(2x) == 2 y(x) at full width."""
    from mamba_b200.mamba import sscan_fwd_raw
    Bsz, L, ED, N = 1, 2048, 1536, 16
    g = torch.Generator(device="cuda").manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=g, device=DEV)
    x = r(Bsz, L, ED)
    delta = torch.nn.functional.softplus(r(Bsz, L, ED) * 0.5 - 4.6)
    A = -torch.arange(1, N + 1, device=DEV, dtype=torch.float32).repeat(ED, 1)
    Bm, Cm, D = r(Bsz, L, N), r(Bsz, L, N), torch.ones(ED, device=DEV)
    y1, _, _ = sscan_fwd_raw(x, delta, A, Bm, Cm, D)
    y2, _, _ = sscan_fwd_raw(2 * x, delta, A, Bm, Cm, D)
    assert torch.allclose(y2, 2 * y1, rtol=1e-6, atol=1e-6)


def test_mixed_dtypes_run_in_float32():
    """bf16 x, B, C with a float32 delta (what autocast gives the reference): nothing is rounded to
    bf16 behind the caller's back; the kernel runs in float32 and returns float32 like the reference."""
    import mamba_b200
    inp = scan_inputs(21, 2, 40, 32, 16, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    inp["delta"] = torch.nn.functional.softplus(torch.randn(2, 40, 32, generator=g) * 0.5 - 3.0)   # full float32
    y = mamba_b200.selective_scan_fn(inp["x"].to(DEV).bfloat16(), inp["delta"].to(DEV), inp["A"].to(DEV),
                                     inp["B"].to(DEV).bfloat16(), inp["C"].to(DEV).bfloat16(), inp["D"].to(DEV))
    assert y.dtype == torch.float32
    yo = O.selective_scan_f64(inp["x"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"])
    assert_close(y, yo.float(), RTOL, ATOL)


def test_empty_and_errors():
    import mamba_b200
    z = lambda *s: torch.zeros(*s, device=DEV)
    y = mamba_b200.selective_scan_fn(z(2, 0, 8), z(2, 0, 8), -torch.ones(8, 16, device=DEV), z(2, 0, 16), z(2, 0, 16), z(8))
    assert y.shape == (2, 0, 8)
    with pytest.raises(RuntimeError):            # d_state the kernels are not compiled for
        mamba_b200.selective_scan_fn(z(1, 4, 8), z(1, 4, 8), -torch.ones(8, 12, device=DEV), z(1, 4, 12), z(1, 4, 12), z(8))
    with pytest.raises(TypeError):
        mamba_b200.selective_scan_fn(z(1, 4, 8).double(), z(1, 4, 8).double(), -torch.ones(8, 16, device=DEV),
                                     z(1, 4, 16).double(), z(1, 4, 16).double(), z(8))
    with pytest.raises(RuntimeError):            # CPU tensors: no fallback
        mamba_b200.selective_scan_fn(torch.zeros(1, 4, 8), torch.zeros(1, 4, 8), -torch.ones(8, 16),
                                     torch.zeros(1, 4, 16), torch.zeros(1, 4, 16), torch.zeros(8))


@pytest.mark.parametrize("Bsz,L,ED,S,use_h0,use_bias", [(1, 4096, 64, None, False, False), (2, 512, 40, 4, True, True),
                                                       (1, 2048, 96, 16, True, False), (3, 256, 32, 2, False, True)])
def test_rows_cut_into_pieces_match_the_oracle(Bsz, L, ED, S, use_h0, use_bias):
    """Few batch rows: every row is cut into S pieces scanned side by side (carry pass, fold, full pass, and
    the mirror image in the backward).  Same answer as the scan of the whole row, including the incoming
    state, its gradient and the outgoing state; S = None lets the library choose (and it must choose > 1)."""
    from mamba_b200.split import pick_subshards
    inp = scan_inputs(600 + L + ED, Bsz, L, ED, 16, structured_A=False, big_delta=True)
    g = torch.Generator().manual_seed(L)
    h0 = torch.randn(Bsz, ED, 16, generator=g) if use_h0 else None
    bias = None
    if use_bias:
        bias = torch.randn(ED, generator=g) * 0.5 - 3.0
        inp["delta"] = torch.randn(Bsz, L, ED, generator=g)
    if S is None:
        assert pick_subshards(Bsz, L, ED, 1) > 1
    _compare(inp, torch.float32, RTOL, ATOL, subshards=S, gated=True, h0=h0, bias=bias)


def test_rows_cut_into_pieces_bf16_long():
    inp = scan_inputs(77, 1, 4096, 128, 16, dtype=torch.bfloat16)
    yo, ho, go = _oracle(inp)
    yk, hk, gk = _kernel(inp, torch.bfloat16, subshards=8)
    assert_close(yk, yo.float(), BF_RTOL, BF_ATOL, "y")
    assert_close(hk, ho.float(), 1e-3, 1e-4, "last state")
    for k in ("x", "delta", "z", "B", "C", "A", "D"):
        scale = max(1.0, go[k].abs().max().item())
        assert_close(gk[k], go[k].float(), BF_RTOL, BF_ATOL * scale, f"grad {k}")
