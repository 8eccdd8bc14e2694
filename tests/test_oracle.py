"""The CPU oracle against the golden vectors the unmodified reference produced."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import scan_oracle as O


def _load(golden_dir, name):
    return {k: v for k, v in np.load(os.path.join(golden_dir, name)).items()}


def test_known_answer_cumsum(golden_dir):
    g = _load(golden_dir, "pscan_kat.npz")
    expect = np.array([5, 6, 8, 11, 15, 20, 26, 33, 41, 41, 41, 41, 41, 41, 41, 41], dtype=np.float32)
    assert np.array_equal(g["H"], expect)          # what the reference's docs store
    X = torch.from_numpy(g["X"]).view(1, 16, 1, 1)
    H = O.pscan(torch.ones_like(X), X)
    assert np.array_equal(H.reshape(-1).numpy(), expect)
    Hs = O.scan_sequential(torch.ones_like(X), X)
    assert np.array_equal(Hs.reshape(-1).numpy(), expect)


def test_pscan_restatement_is_bit_exact(golden_dir):
    """Same combine tree as the reference, so float32 results agree bit for bit."""
    g = _load(golden_dir, "pscan_cases.npz")
    for L in g["Ls"]:
        A = torch.from_numpy(g[f"L{L}_A"]).requires_grad_()
        X = torch.from_numpy(g[f"L{L}_X"]).requires_grad_()
        A0, X0 = A.detach().clone(), X.detach().clone()
        H = O.pscan(A, X)
        H.backward(torch.from_numpy(g[f"L{L}_G"]))
        assert np.array_equal(H.detach().numpy(), g[f"L{L}_H"]), L
        assert np.array_equal(A.grad.numpy(), g[f"L{L}_gA"]), L
        assert np.array_equal(X.grad.numpy(), g[f"L{L}_gX"]), L
        assert torch.equal(A.detach(), A0) and torch.equal(X.detach(), X0)   # inputs untouched


def test_pscan_matches_sequential(golden_dir):
    g = _load(golden_dir, "pscan_cases.npz")
    for L in g["Ls"]:
        A = torch.from_numpy(g[f"L{L}_A"])
        X = torch.from_numpy(g[f"L{L}_X"])
        Hs = O.scan_sequential(A.double(), X.double())
        np.testing.assert_allclose(g[f"L{L}_H"], Hs.numpy(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("route", ["pscan", "seq"])
def test_selective_scan_golden(golden_dir, route):
    g = _load(golden_dir, "selective_scan.npz")
    t = lambda k: torch.from_numpy(g[k]).clone()
    leaves = [t(k).requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")]
    x, dl, A, Bm, Cm, D, z = leaves
    fn = O.selective_scan if route == "pscan" else O.selective_scan_seq
    y = fn(x, dl, A, Bm, Cm, D)
    out = O.gate(y, z)
    out.backward(t("gy"))
    # identical op sequence => identical bits
    assert np.array_equal(y.detach().numpy(), g[f"{route}_y"])
    assert np.array_equal(out.detach().numpy(), g[f"{route}_yg"])
    for nm, leaf in zip(("x", "delta", "A", "B", "C", "D", "z"), leaves):
        np.testing.assert_allclose(leaf.grad.numpy(), g[f"{route}_g{nm}"], rtol=1e-6, atol=1e-7, err_msg=nm)


def test_f64_arbiter_agrees_with_reference(golden_dir):
    g = _load(golden_dir, "selective_scan.npz")
    t = lambda k: torch.from_numpy(g[k]).clone()
    leaves = [t(k).double().requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")]
    x, dl, A, Bm, Cm, D, z = leaves
    out = O.selective_scan_f64(x, dl, A, Bm, Cm, D, z=z)
    out.backward(t("gy").double())
    np.testing.assert_allclose(out.detach().numpy(), g["pscan_yg"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(out.detach().numpy(), g["seq_yg"], rtol=1e-4, atol=1e-5)
    for nm, leaf in zip(("x", "delta", "A", "B", "C", "D", "z"), leaves):
        np.testing.assert_allclose(leaf.grad.numpy(), g[f"pscan_g{nm}"], rtol=1e-4, atol=2e-5, err_msg=nm)


def test_f64_state_carry_splits_sequence(golden_dir):
    """Scanning two halves with the carried state equals scanning the whole."""
    g = _load(golden_dir, "selective_scan.npz")
    t = lambda k: torch.from_numpy(g[k])
    x, dl, A, Bm, Cm, D = (t(k) for k in ("x", "delta", "A", "B", "C", "D"))
    y, h = O.selective_scan_f64(x, dl, A, Bm, Cm, D, return_last_state=True)
    m = 29
    y0, h0 = O.selective_scan_f64(x[:, :m], dl[:, :m], A, Bm[:, :m], Cm[:, :m], D, return_last_state=True)
    y1, h1 = O.selective_scan_f64(x[:, m:], dl[:, m:], A, Bm[:, m:], Cm[:, m:], D, h0=h0, return_last_state=True)
    np.testing.assert_allclose(torch.cat([y0, y1], 1).numpy(), y.numpy(), rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(h1.numpy(), h.numpy(), rtol=1e-12, atol=1e-13)


def test_block_step_golden(golden_dir):
    """Mamba.step unrolled over the sequence: outputs, states and conv windows."""
    g = _load(golden_dir, "block_step.npz")
    xs = torch.from_numpy(g["xs"])
    Bsz, L, Dm = xs.shape
    n_layers = 2
    Ws = []
    for li in range(n_layers):
        W = {k: torch.from_numpy(g[f"l{li}_{k}"]) for k in
             ("in_proj", "conv_w", "conv_b", "x_proj", "dt_w", "dt_b", "A_log", "D", "out_proj")}
        W["norm_w"] = torch.from_numpy(g[f"l{li}_norm_w"])
        Ws.append(W)
    ED = Ws[0]["A_log"].shape[0]
    caches = [(None, torch.zeros(Bsz, ED, 3)) for _ in range(n_layers)]
    outs = []
    for t in range(L):
        x = xs[:, t]
        for li, W in enumerate(Ws):
            xn = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * W["norm_w"]
            o, caches[li] = O.block_step(xn, caches[li], W)
            x = o + x
        outs.append(x)
        hs = torch.stack([c[0] for c in caches])
        np.testing.assert_allclose(hs.numpy(), g["h_after"][t], rtol=1e-5, atol=1e-6)
    outs = torch.stack(outs, 1)
    np.testing.assert_allclose(outs.numpy(), g["steps"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(outs.numpy(), g["forward"], rtol=1e-4, atol=1e-5)   # step == forward
    np.testing.assert_allclose(torch.stack([c[1] for c in caches]).numpy(), g["conv_after"], rtol=0, atol=0)


@pytest.mark.parametrize("Bsz,L,ED,N,gated,use_bias,use_h0",
                         [(2, 64, 32, 16, True, True, True), (1, 37, 20, 8, False, False, False),
                          (2, 50, 24, 16, True, False, True)])
def test_closed_form_f64_matches_autograd_of_the_sequential_loop(Bsz, L, ED, N, gated, use_bias, use_h0):
    """The hand-derived float64 backward used for wide problems equals autograd of the sequential
    restatement (itself pinned by the golden vectors above), block-wise over channels."""
    from tests.helpers import scan_inputs
    inp = scan_inputs(5 + L, Bsz, L, ED, N, structured_A=False, big_delta=True)
    g = torch.Generator().manual_seed(1)
    bias = torch.randn(ED, generator=g) * 0.5 - 2 if use_bias else None
    h0 = torch.randn(Bsz, ED, N, generator=g) if use_h0 else None
    lv = {k: inp[k].double().requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")}
    extra = {}
    if use_bias:
        extra["bias"] = bias.double().requires_grad_()
    if use_h0:
        extra["h0"] = h0.double().requires_grad_()
    d = torch.nn.functional.softplus(lv["delta"] + extra["bias"]) if use_bias else lv["delta"]
    y, hT = O.selective_scan_f64(lv["x"], d, lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"] if gated else None,
                                 h0=extra.get("h0"), return_last_state=True)
    y.backward(inp["gy"].double())
    y2, hT2, gr = O.selective_scan_fwd_bwd_f64(inp["x"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"],
                                               inp["gy"], z=inp["z"] if gated else None, delta_bias=bias, h0=h0,
                                               block=7)
    assert torch.allclose(y2, y.detach(), rtol=1e-12, atol=1e-12)
    assert torch.allclose(hT2, hT.detach(), rtol=1e-12, atol=1e-12)
    for k, v in gr.items():
        want = (extra[k] if k in extra else lv[k]).grad
        assert torch.allclose(v, want, rtol=1e-10, atol=1e-11), k


def test_closed_form_f64_matches_reference_golden(golden_dir):
    """... and the reference's own outputs and gradients on the small config (float32 golden)."""
    import numpy as np
    g = {k: torch.from_numpy(v) for k, v in np.load(f"{golden_dir}/selective_scan.npz").items()}
    y, _, gr = O.selective_scan_fwd_bwd_f64(g["x"], g["delta"], g["A"], g["B"], g["C"], g["D"], g["gy"], z=g["z"])
    assert torch.allclose(y.float(), g["pscan_yg"], rtol=1e-4, atol=1e-5)
    for k in ("x", "delta", "A", "B", "C", "D", "z"):
        want = g[f"pscan_g{k}"]
        assert torch.allclose(gr[k].float(), want, rtol=1e-4, atol=1e-5 * max(1.0, want.abs().max().item()) * 4), k
