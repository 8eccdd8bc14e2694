"""One-pass RMSNorm kernel against the reference's formula (mambapy/mamba.py:427-433) in float64."""
import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference(x, w, eps):
    out = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return out if w is None else out * w


@pytest.mark.parametrize("shape", [(2, 64, 768), (1, 1, 16), (3, 37, 100), (5, 2560), (2, 9, 4104)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gain", [True, False])
def test_rms_norm_forward_backward(shape, dtype, gain):
    import mamba_b200
    g = torch.Generator().manual_seed(sum(shape))
    D = shape[-1]
    x = (torch.randn(*shape, generator=g) * 2).to(dtype).float()
    w = torch.randn(D, generator=g) if gain else None
    gy = torch.randn(*shape, generator=g).to(dtype).float()
    xr = x.double().requires_grad_()
    wr = None if w is None else w.double().requires_grad_()
    yr = _reference(xr, wr, 1e-5)
    yr.backward(gy.double())
    xc = x.to(DEV).to(dtype).requires_grad_()
    wc = None if w is None else w.to(DEV).requires_grad_()
    y = mamba_b200.rms_norm(xc, wc, 1e-5)
    y.backward(gy.to(DEV).to(dtype))
    tol = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 2e-2)
    assert y.dtype == dtype and y.shape == tuple(shape)
    assert_close(y, yr.float(), *tol, "y")
    assert_close(xc.grad, xr.grad.float(), *tol, "dx")
    if gain:
        scale = max(1.0, wr.grad.abs().max().item())
        assert_close(wc.grad, wr.grad.float(), tol[0] * 10, tol[1] * scale * 4, "dweight")


def test_rms_norm_takes_strided_rows_and_rejects_cpu():
    import mamba_b200
    g = torch.Generator().manual_seed(3)
    xz = torch.randn(4, 33, 2 * 64, generator=g).to(DEV)
    x = xz[..., :64]                                   # a chunk() view: row stride 128
    w = torch.randn(64, generator=g).to(DEV)
    y = mamba_b200.rms_norm(x, w, 1e-5)
    assert_close(y, _reference(x.double().cpu(), w.double().cpu(), 1e-5).float(), 1e-4, 1e-5, "y")
    with pytest.raises(RuntimeError):
        mamba_b200.rms_norm(torch.randn(2, 8), torch.ones(8))


@pytest.mark.parametrize("shape", [(2, 64, 768), (3, 37, 100), (5, 2560)])
@pytest.mark.parametrize("dx,dres", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.bfloat16), (torch.float32, None)])
def test_residual_add_fused_with_rms_norm(shape, dx, dres):
    """(y, s) = (RMSNorm(x + res), x + res) from one kernel, forward and backward, against float64 autograd of
    the reference's two separate steps (mambapy/mamba.py:111 and :427-433)."""
    import mamba_b200
    g = torch.Generator().manual_seed(sum(shape) + 1)
    D = shape[-1]
    x = torch.randn(*shape, generator=g).to(dx).float()
    res = None if dres is None else (torch.randn(*shape, generator=g) * 2).to(dres).float()
    w = torch.randn(D, generator=g)
    gy, gs = torch.randn(*shape, generator=g), torch.randn(*shape, generator=g)
    xr, wr = x.double().requires_grad_(), w.double().requires_grad_()
    rr = None if res is None else res.double().requires_grad_()
    sr = xr if rr is None else xr + rr
    if dres == torch.bfloat16:                                     # the stream itself is bfloat16: the sum is rounded
        sr = sr + (sr.detach().bfloat16().double() - sr.detach())
    yr = _reference(sr, wr, 1e-5)
    (yr * gy.double()).sum().backward(retain_graph=True)
    (sr * gs.double()).sum().backward()
    xc = x.to(DEV).to(dx).requires_grad_()
    rc = None if res is None else res.to(DEV).to(dres).requires_grad_()
    wc = w.to(DEV).requires_grad_()
    y, s = mamba_b200.add_rms_norm(xc, rc, wc, 1e-5)
    ((y.float() * gy.to(DEV)).sum() + (s.float() * gs.to(DEV)).sum()).backward()
    low = torch.bfloat16 in (dx, dres)
    tol = (2e-2, 2e-2) if low else (1e-4, 1e-5)
    assert s.dtype == (dx if dres is None else torch.promote_types(dx, dres))
    assert_close(s, sr.float(), *tol, "sum")
    assert_close(y, yr.float(), tol[0], tol[1] * 4, "y")
    assert_close(xc.grad, xr.grad.float(), tol[0], tol[1] * 4, "dx")
    if rc is not None:
        assert_close(rc.grad, rr.grad.float(), tol[0], tol[1] * 4, "dres")
    assert_close(wc.grad, wr.grad.float(), tol[0] * 10, tol[1] * max(1.0, wr.grad.abs().max().item()) * 4, "dweight")
