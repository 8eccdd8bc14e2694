"""The drop-in on the reference's OWN classes, on the GPU, against the unpatched reference on the CPU.

oracle/_ref/ holds an unmodified copy of the reference package (oracle/make_ref.py puts it there; it is
git-ignored and travels with the working tree).  Each test builds a reference model twice with the
same weights: one stays on the CPU and runs the reference's code, the other goes to the GPU and runs
under `mamba_b200.install()` / `install(fuse_block=True)`.  Outputs, input gradients, every parameter
gradient and the decode caches are compared in float32 (rtol 1e-4, atol 1e-5 scaled by magnitude)."""
import copy
import os
import sys

import pytest
import torch

from oracle.make_ref import ref_path
from tests.helpers import assert_close

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(ref_path() is None, reason="oracle/_ref not made (python oracle/make_ref.py)")]
DEV = "cuda:0"
RTOL, ATOL = 1e-4, 1e-5


@pytest.fixture()
def ref():
    import mamba_b200
    sys.path.insert(0, ref_path())
    try:
        import mambapy.mamba as rm
        import mambapy.vim as rv
        import mambapy.jamba as rj
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        yield rm, rv, rj
    finally:
        mamba_b200.uninstall()
        sys.path.remove(ref_path())


def _fwd_bwd(model, x, gy):
    x = x.clone().requires_grad_()
    for p in model.parameters():
        p.grad = None
    y = model(x)
    y.backward(gy)
    return y.detach(), x.grad, {n: p.grad for n, p in model.named_parameters()}


def _check(got, want, ctx):
    yk, gxk, gpk = got
    yr, gxr, gpr = want
    assert_close(yk, yr, RTOL, ATOL * max(1.0, yr.abs().max().item()), f"output {ctx}")
    assert_close(gxk, gxr, RTOL, ATOL * max(1.0, gxr.abs().max().item()) * 4, f"input grad {ctx}")
    assert set(gpk) == set(gpr)
    for n, g in gpr.items():
        assert gpk[n] is not None, f"{n} got no gradient {ctx}"
        assert_close(gpk[n], g, RTOL, ATOL * max(1.0, g.abs().max().item()) * 4, f"grad {n} {ctx}")


@pytest.mark.parametrize("fuse_block", [False, True])
@pytest.mark.parametrize("L", [37, 64])
def test_mamba_forward_backward_and_steps(ref, fuse_block, L):
    """Mamba (2 layers, d_model 64): forward + backward, then 8 decode steps from an empty cache."""
    import mamba_b200
    rm, _, _ = ref
    torch.manual_seed(1)
    cfg = rm.MambaConfig(d_model=64, n_layers=2)
    cpu = rm.Mamba(cfg)
    gpu = copy.deepcopy(cpu).to(DEV)
    x, gy = torch.randn(2, L, 64), torch.randn(2, L, 64)
    want = _fwd_bwd(cpu, x, gy)
    mamba_b200.install(fuse_block=fuse_block)
    assert mamba_b200.installed()
    if fuse_block:                                   # the layer loop with the residual adds fused into the norms
        assert rm.Mamba.forward is mamba_b200.mamba.stack_forward
    got = _fwd_bwd(gpu, x.to(DEV), gy.to(DEV))
    _check(got, want, f"fuse_block={fuse_block} L={L}")
    # decode: Mamba.step from (None, zeros) caches (mambapy/mamba.py:87-97, :351-382)
    def caches(dev):
        return [(None, torch.zeros(2, cfg.d_inner, cfg.d_conv - 1, device=dev)) for _ in range(cfg.n_layers)]
    cg = caches(DEV)
    outs_g = []
    with torch.no_grad():
        for t in range(8):
            o, cg = gpu.step(x[:, t].to(DEV), cg)
            outs_g.append(o)
    mamba_b200.uninstall()
    cc = caches("cpu")
    with torch.no_grad():
        for t in range(8):
            o, cc = cpu.step(x[:, t], cc)
            assert_close(outs_g[t], o, RTOL, ATOL * max(1.0, o.abs().max().item()), f"step {t}")
        for (hg, wg), (hc, wc) in zip(cg, cc):
            assert_close(hg, hc, RTOL, ATOL, "state after 8 steps")
            assert_close(wg, wc, RTOL, ATOL, "conv window after 8 steps")
        # and the steps equal the forward on the same prefix, as in the reference
        assert_close(torch.stack(outs_g, 1), want[0][:, :8], 1e-3, 1e-4, "step == forward")


def test_mamba_sequential_route_and_state_dict(ref):
    """config.pscan=False sends the block through selective_scan_seq (mambapy/mamba.py:267-270); the
    patched model keeps the reference's parameter names, so its state_dict loads into a fresh one."""
    import mamba_b200
    rm, _, _ = ref
    torch.manual_seed(2)
    cfg = rm.MambaConfig(d_model=32, n_layers=1, pscan=False, d_state=16)
    cpu = rm.Mamba(cfg)
    gpu = copy.deepcopy(cpu).to(DEV)
    x, gy = torch.randn(1, 50, 32), torch.randn(1, 50, 32)
    want = _fwd_bwd(cpu, x, gy)
    mamba_b200.install()
    got = _fwd_bwd(gpu, x.to(DEV), gy.to(DEV))
    _check(got, want, "pscan=False")
    fresh = rm.Mamba(cfg)
    fresh.load_state_dict(gpu.state_dict())


@pytest.mark.parametrize("fuse_block", [False, True])
def test_vim_bidirectional_block(ref, fuse_block):
    """The bidirectional block of mambapy/vim.py:205-261.  With fuse_block its forward scans the second
    direction right-to-left inside the kernels instead of flipping the sequence."""
    import mamba_b200
    _, rv, _ = ref
    torch.manual_seed(3)
    cfg = rv.MambaConfig(d_model=32, n_layers=2, bidirectional=True)
    cpu = rv.VMamba(cfg)
    gpu = copy.deepcopy(cpu).to(DEV)
    x, gy = torch.randn(2, 48, 32), torch.randn(2, 48, 32)
    want = _fwd_bwd(cpu, x, gy)
    mamba_b200.install(fuse_block=fuse_block)
    assert rv.VMambaBlock.selective_scan is mamba_b200.selective_scan        # the scan itself is always swapped
    if fuse_block:
        from mamba_b200 import vim as kernel_vim
        assert rv.VMambaBlock.forward is kernel_vim.forward
    got = _fwd_bwd(gpu, x.to(DEV), gy.to(DEV))
    _check(got, want, f"vim fuse_block={fuse_block}")


def test_jamba_mamba_layer_forward_and_decode(ref):
    """Jamba's MambaLayer (mambapy/jamba.py:404-443) calls MambaBlock.forward without a cache and
    MambaBlock.step with one, with the inner RMSNorms on delta, B, C switched on."""
    import mamba_b200
    _, _, rj = ref
    torch.manual_seed(4)
    cfg = rj.JambaLMConfig(d_model=32, n_layers=2, mlp_size=64, num_attention_heads=4, num_key_value_heads=2,
                           num_experts=2, num_experts_per_tok=1)
    cpu = rj.MambaLayer(cfg, num_experts=1)
    gpu = copy.deepcopy(cpu).to(DEV)
    x = torch.randn(2, 20, 32)
    with torch.no_grad():
        (yr, _), _ = cpu(x)
        cache_c = (None, torch.zeros(2, 64, 3))
        steps_c = []
        for t in range(6):
            (o, _), cache_c = cpu(x[:, t:t + 1], cache_c)
            steps_c.append(o)
        mamba_b200.install()
        (yg, _), _ = gpu(x.to(DEV))
        cache_g = (None, torch.zeros(2, 64, 3, device=DEV))
        for t in range(6):
            (o, _), cache_g = gpu(x[:, t:t + 1].to(DEV), cache_g)
            assert_close(o, steps_c[t], RTOL, ATOL * max(1.0, steps_c[t].abs().max().item()), f"jamba step {t}")
    assert_close(yg, yr, RTOL, ATOL * max(1.0, yr.abs().max().item()), "jamba MambaLayer forward")
    assert_close(cache_g[0], cache_c[0], RTOL, ATOL, "jamba state")
