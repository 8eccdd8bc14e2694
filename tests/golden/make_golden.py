"""Writes the golden fixtures in this folder by running the UNMODIFIED reference.

Usage (only where the reference checkout is present):

    python tests/golden/make_golden.py /path/to/reference

The reference is pure Python on top of torch, so it is imported from its checkout
and executed on the CPU in float32.  Every fixture stores the seeded inputs and the
reference's outputs, so the tests never need the reference itself.  Fixtures are
small (.npz, float32) and are committed; this script is the record of how they were
made.

Files written:
  pscan_cases.npz       PScan.apply forward + backward for several L (powers of two and not)
  pscan_kat.npz         the integer known-answer vector from the reference's docs/tests.ipynb
  selective_scan.npz    MambaBlock.selective_scan / selective_scan_seq on the small config,
                        outputs and gradients of x, delta, A, B, C, D (and z through the gate)
  block_step.npz        Mamba.step unrolled for a 2-layer model, with the matching forward
"""
import sys
import os

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def small_config_inputs(seed=1000, Bsz=2, L=64, ED=32, N=16):
    """Seeded inputs of the small CPU config: x, delta, A, B, C, D, z, upstream grad."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(Bsz, L, ED, generator=g)
    delta = F.softplus(torch.randn(Bsz, L, ED, generator=g) * 0.5 - 4.6)
    A = -torch.exp(torch.log(torch.arange(1, N + 1, dtype=torch.float32))).repeat(ED, 1)
    Bm = torch.randn(Bsz, L, N, generator=g)
    Cm = torch.randn(Bsz, L, N, generator=g)
    D = torch.ones(ED)
    z = torch.randn(Bsz, L, ED, generator=g)
    gy = torch.randn(Bsz, L, ED, generator=g)
    return x, delta, A, Bm, Cm, D, z, gy


def main(ref_root):
    sys.path.insert(0, ref_root)
    from mambapy.pscan import pscan
    from mambapy.mamba import Mamba, MambaBlock, MambaConfig

    torch.set_num_threads(4)

    # ---- pscan forward/backward, assorted L ------------------------------------
    out = {}
    Ls = [1, 2, 3, 4, 5, 7, 8, 16, 31, 37, 64, 100]
    for i, L in enumerate(Ls):
        g = torch.Generator().manual_seed(2000 + i)
        A = torch.exp(-F.softplus(torch.randn(2, L, 6, 16, generator=g))).requires_grad_()
        X = torch.randn(2, L, 6, 16, generator=g).requires_grad_()
        G = torch.randn(2, L, 6, 16, generator=g)
        H = pscan(A, X)
        H.backward(G)
        out[f"L{L}_A"] = A.detach().numpy()
        out[f"L{L}_X"] = X.detach().numpy()
        out[f"L{L}_G"] = G.numpy()
        out[f"L{L}_H"] = H.detach().contiguous().numpy()
        out[f"L{L}_gA"] = A.grad.numpy()
        out[f"L{L}_gX"] = X.grad.numpy()
    out["Ls"] = np.array(Ls)
    np.savez_compressed(os.path.join(HERE, "pscan_cases.npz"), **out)

    # ---- integer known-answer vector (A == 1 gives a cumulative sum) ------------
    v = torch.tensor([5, 1, 2, 3, 4, 5, 6, 7, 8, 0, 0, 0, 0, 0, 0, 0], dtype=torch.float32)
    Xk = v.view(1, 16, 1, 1).clone()
    Hk = pscan(torch.ones_like(Xk), Xk)
    np.savez_compressed(os.path.join(HERE, "pscan_kat.npz"), X=v.numpy(), H=Hk.reshape(-1).numpy())

    # ---- selective_scan on the small config --------------------------------------
    x, delta, A, Bm, Cm, D, z, gy = small_config_inputs()
    blk = MambaBlock(MambaConfig(d_model=16, n_layers=0))
    res = dict(x=x, delta=delta, A=A, B=Bm, C=Cm, D=D, z=z, gy=gy)
    for name, fn in (("pscan", blk.selective_scan), ("seq", blk.selective_scan_seq)):
        leaves = [t.clone().requires_grad_() for t in (x, delta, A, Bm, Cm, D, z)]
        xx, dd, AA, BB, CC, DD, zz = leaves
        y = fn(xx, dd, AA, BB, CC, DD)
        res[f"{name}_y"] = y.detach()
        out_g = y * F.silu(zz)                      # the gate of MambaBlock.forward
        res[f"{name}_yg"] = out_g.detach()
        out_g.backward(gy)
        for nm, t in zip(("x", "delta", "A", "B", "C", "D", "z"), leaves):
            res[f"{name}_g{nm}"] = t.grad
        # un-gated gradients as well
        leaves = [t.clone().requires_grad_() for t in (x, delta, A, Bm, Cm, D)]
        y = fn(*leaves)
        y.backward(gy)
        for nm, t in zip(("x", "delta", "A", "B", "C", "D"), leaves):
            res[f"{name}_ung_g{nm}"] = t.grad
    np.savez_compressed(os.path.join(HERE, "selective_scan.npz"),
                        **{k: v.detach().numpy() for k, v in res.items()})

    # ---- Mamba.step unrolled vs forward (2 layers, d_model 16, L = 11) -------------
    torch.manual_seed(1003)
    cfg = MambaConfig(d_model=16, n_layers=2)
    model = Mamba(cfg).eval()
    Bsz, L = 3, 11
    xs = torch.randn(Bsz, L, 16)
    with torch.no_grad():
        full = model(xs)
        caches = [(None, torch.zeros(Bsz, cfg.d_inner, cfg.d_conv - 1)) for _ in range(cfg.n_layers)]
        steps, hs = [], []
        for t in range(L):
            o, caches = model.step(xs[:, t], caches)
            steps.append(o)
            hs.append(torch.stack([c[0] for c in caches]))
        steps = torch.stack(steps, dim=1)
    st = {"xs": xs.numpy(), "forward": full.numpy(), "steps": steps.numpy(),
          "h_after": torch.stack(hs).numpy(),
          "conv_after": torch.stack([c[1] for c in caches]).numpy()}
    for li, layer in enumerate(model.layers):
        m = layer.mixer
        st[f"l{li}_norm_w"] = layer.norm.weight.detach().numpy()
        st[f"l{li}_in_proj"] = m.in_proj.weight.detach().numpy()
        st[f"l{li}_conv_w"] = m.conv1d.weight.detach().numpy()
        st[f"l{li}_conv_b"] = m.conv1d.bias.detach().numpy()
        st[f"l{li}_x_proj"] = m.x_proj.weight.detach().numpy()
        st[f"l{li}_dt_w"] = m.dt_proj.weight.detach().numpy()
        st[f"l{li}_dt_b"] = m.dt_proj.bias.detach().numpy()
        st[f"l{li}_A_log"] = m.A_log.detach().numpy()
        st[f"l{li}_D"] = m.D.detach().numpy()
        st[f"l{li}_out_proj"] = m.out_proj.weight.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "block_step.npz"), **st)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
