"""Fused depthwise causal conv1d + SiLU against the reference's own op sequence run on the CPU."""
import pytest
import torch
import torch.nn.functional as F

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference(x, w, b):
    """mambapy/mamba.py:217-221 in float64: transpose, Conv1d(padding=3, groups=ED), slice, transpose, silu."""
    L = x.shape[1]
    y = F.conv1d(x.transpose(1, 2), w, b, padding=w.shape[-1] - 1, groups=w.shape[0])[:, :, :L].transpose(1, 2)
    return F.silu(y)


@pytest.mark.parametrize("Bsz,L,ED", [(2, 64, 32), (1, 1, 8), (3, 130, 40), (2, 257, 33), (1, 3, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_conv1d_silu_forward_backward(Bsz, L, ED, dtype):
    import mamba_b200
    g = torch.Generator().manual_seed(L + ED)
    x = torch.randn(Bsz, L, ED, generator=g).to(dtype).float()
    w = torch.randn(ED, 1, 4, generator=g) * 0.5
    b = torch.randn(ED, generator=g) * 0.1
    gy = torch.randn(Bsz, L, ED, generator=g).to(dtype).float()
    xr, wr, br = (t.double().requires_grad_() for t in (x, w, b))
    yr = _reference(xr, wr, br)
    yr.backward(gy.double())
    xc, wc, bc = x.to(DEV).to(dtype).requires_grad_(), w.to(DEV).requires_grad_(), b.to(DEV).requires_grad_()
    y = mamba_b200.causal_conv1d_silu(xc, wc, bc)
    y.backward(gy.to(DEV).to(dtype))
    tol = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 2e-2)
    assert y.dtype == dtype and y.shape == (Bsz, L, ED)
    assert_close(y, yr.float(), *tol, "y")
    assert_close(xc.grad, xr.grad.float(), *tol, "dx")
    scale = max(1.0, wr.grad.abs().max().item())
    assert_close(wc.grad, wr.grad.float(), tol[0] * 10, tol[1] * scale * 4, "dw")
    assert_close(bc.grad, br.grad.float(), tol[0] * 10, tol[1] * scale * 4, "dbias")


def test_conv1d_silu_on_a_chunk_view():
    """x as the first half of the in_proj output (a strided view), as MambaBlock.forward has it."""
    import mamba_b200
    g = torch.Generator().manual_seed(5)
    xz = torch.randn(2, 100, 64, generator=g).to(DEV)
    x, _ = xz.chunk(2, dim=-1)
    w = torch.randn(32, 1, 4, generator=g).to(DEV)
    y = mamba_b200.causal_conv1d_silu(x, w, None)
    yr = _reference(x.cpu().double(), w.cpu().double(), None)
    assert_close(y, yr.float(), 1e-4, 1e-5)
