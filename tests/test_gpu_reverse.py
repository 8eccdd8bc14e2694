"""Reverse-direction scan (MB200_REVERSE) against the oracle run on the flipped sequence, which is how
the reference's bidirectional model obtains it (mambapy/vim.py:228-261)."""
import pytest
import torch

from oracle import scan_oracle as O
from tests.helpers import scan_inputs, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACT = ("x", "delta", "B", "C", "z", "gy")


def _oracle_reversed(inp, gated, h0, bias):
    f = {k: (v.flip(1) if k in ACT else v) for k, v in inp.items()}
    leaves = {k: f[k].double().requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")}
    delta = leaves["delta"]
    bl = None
    if bias is not None:
        bl = bias.double().requires_grad_()
        delta = torch.nn.functional.softplus(delta + bl)
    h0l = None if h0 is None else h0.double().requires_grad_()
    y, hT = O.selective_scan_f64(leaves["x"], delta, leaves["A"], leaves["B"], leaves["C"], leaves["D"],
                                 z=leaves["z"] if gated else None, h0=h0l, return_last_state=True)
    y.backward(f["gy"].double())
    g = {k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in leaves.items()}
    g = {k: (v.flip(1) if k in ACT else v) for k, v in g.items()}
    if bl is not None:
        g["bias"] = bl.grad
    if h0l is not None:
        g["h0"] = h0l.grad
    return y.detach().flip(1), hT.detach(), g


def _kernel_reversed(inp, dtype, gated, h0, bias):
    import mamba_b200
    act = lambda k: inp[k].to(DEV).to(dtype).requires_grad_()
    par = lambda k: inp[k].to(DEV).requires_grad_()
    lv = dict(x=act("x"), delta=act("delta"), A=par("A"), B=act("B"), C=act("C"), D=par("D"), z=act("z"))
    bl = None if bias is None else bias.to(DEV).requires_grad_()
    h0l = None if h0 is None else h0.to(DEV).requires_grad_()
    y, hT = mamba_b200.selective_scan_fn(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"],
                                         z=lv["z"] if gated else None, delta_bias=bl, h0=h0l,
                                         return_last_state=True, reverse=True)
    y.backward(inp["gy"].to(DEV).to(dtype))
    g = {k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in lv.items()}
    if bl is not None:
        g["bias"] = bl.grad
    if h0l is not None:
        g["h0"] = h0l.grad
    return y.detach(), hT.detach(), g


def _compare(inp, dtype, rtol, atol, gated=True, h0=None, bias=None):
    yo, ho, go = _oracle_reversed(inp, gated, h0, bias)
    yk, hk, gk = _kernel_reversed(inp, dtype, gated, h0, bias)
    assert_close(yk, yo.float(), rtol, atol, "y")
    assert_close(hk, ho.float(), rtol, atol, "last state")
    for k in go:
        if k == "z" and not gated:
            continue
        scale = go[k].abs().max().item() + 1e-30
        assert_close(gk[k], go[k].float(), rtol, max(atol, atol * scale * 4), f"grad {k}")


@pytest.mark.parametrize("Bsz,L,ED,N", [(2, 64, 32, 16), (1, 1, 8, 16), (2, 37, 40, 16), (1, 100, 64, 16),
                                        (2, 8, 32, 16), (1, 9, 32, 16), (1, 17, 16, 16), (2, 129, 96, 16)])
@pytest.mark.parametrize("gated", [True, False])
def test_reverse_in_place_f32(Bsz, L, ED, N, gated):
    """Aligned float32 tensors with d_state 16: the kernels walk the sequence backwards themselves."""
    import mamba_b200
    from mamba_b200.mamba import sscan_fwd_raw
    inp = scan_inputs(500 + L + ED, Bsz, L, ED, N)
    d = {k: inp[k].to(DEV) for k in ("x", "delta", "A", "B", "C", "D", "z")}
    assert sscan_fwd_raw(d["x"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["z"], reverse=True) is not None
    _compare(inp, torch.float32, 1e-4, 1e-5, gated=gated)
    assert mamba_b200._lib.load().mb200_device_status() == 0


def test_reverse_with_state_and_softplus():
    inp = scan_inputs(77, 2, 77, 48, 16)
    g = torch.Generator().manual_seed(5)
    inp["delta"] = torch.randn(2, 77, 48, generator=g) * 0.5 - 4.0      # raw: softplus happens in the kernel
    _compare(inp, torch.float32, 1e-4, 1e-5, h0=torch.randn(2, 48, 16, generator=g),
             bias=torch.randn(48, generator=g) * 0.1)


@pytest.mark.parametrize("Bsz,L,ED,N", [(2, 200, 64, 16), (1, 515, 128, 16)])
def test_reverse_bf16(Bsz, L, ED, N):
    inp = scan_inputs(900 + L, Bsz, L, ED, N, dtype=torch.bfloat16)
    _compare(inp, torch.bfloat16, 2e-2, 2e-2)


@pytest.mark.parametrize("Bsz,L,ED,N", [(2, 50, 32, 8), (1, 33, 20, 16), (2, 40, 24, 32)])
def test_reverse_falls_back_to_flipping(Bsz, L, ED, N):
    """Other d_state (with gradients) or tensors the tensor-map path cannot take: same answer by flipping."""
    inp = scan_inputs(300 + L + N, Bsz, L, ED, N)
    _compare(inp, torch.float32, 1e-4, 1e-5)
