"""PScan kernels against the golden vectors of the reference and the CPU oracle (needs a GPU)."""
import numpy as np
import pytest
import torch

from oracle import scan_oracle as O
from tests.helpers import golden, assert_close

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5          # float32 tolerance of the parity contract


def _dev():
    return torch.device("cuda:0")


def test_golden_forward_backward():
    import mamba_b200
    g = golden("pscan_cases.npz")
    for L in g["Ls"]:
        A = torch.from_numpy(g[f"L{L}_A"]).to(_dev()).requires_grad_()
        X = torch.from_numpy(g[f"L{L}_X"]).to(_dev()).requires_grad_()
        A0, X0 = A.detach().clone(), X.detach().clone()
        H = mamba_b200.pscan(A, X)
        H.backward(torch.from_numpy(g[f"L{L}_G"]).to(_dev()))
        assert_close(H, g[f"L{L}_H"], RTOL, ATOL, f"H L={L}")
        assert_close(A.grad, g[f"L{L}_gA"], RTOL, ATOL, f"gradA L={L}")
        assert_close(X.grad, g[f"L{L}_gX"], RTOL, ATOL, f"gradX L={L}")
        assert torch.equal(A.detach(), A0) and torch.equal(X.detach(), X0), "inputs were modified"
        assert H.shape == X.shape and H.dtype == X.dtype


def test_known_answer_vector():
    import mamba_b200
    g = golden("pscan_kat.npz")
    X = torch.from_numpy(g["X"]).view(1, 16, 1, 1).to(_dev())
    H = mamba_b200.pscan(torch.ones_like(X), X)
    assert np.array_equal(H.reshape(-1).cpu().numpy(), g["H"])      # integers: exact


@pytest.mark.parametrize("shape", [(1, 4096, 3, 16), (2, 1000, 5, 8), (3, 129, 7, 4), (1, 65, 1, 1),
                                   (2, 300, 33, 16)])
def test_against_sequential_oracle(shape):
    """Shapes that take the segmented (low-parallelism) and the scalar (unaligned) paths."""
    import mamba_b200
    g = torch.Generator().manual_seed(sum(shape))
    A = torch.exp(-torch.nn.functional.softplus(torch.randn(shape, generator=g)))
    X = torch.randn(shape, generator=g)
    G = torch.randn(shape, generator=g)
    Ad, Xd = A.double().requires_grad_(), X.double().requires_grad_()
    Hs = O.scan_sequential(Ad, Xd)
    Hs.backward(G.double())
    Ac, Xc = A.to(_dev()).requires_grad_(), X.to(_dev()).requires_grad_()
    H = mamba_b200.pscan(Ac, Xc)
    H.backward(G.to(_dev()))
    assert_close(H, Hs.float(), RTOL, ATOL)
    assert_close(Ac.grad, Ad.grad.float(), RTOL, 5 * ATOL)
    assert_close(Xc.grad, Xd.grad.float(), RTOL, 5 * ATOL)


def test_strided_inputs_and_empty():
    import mamba_b200
    g = torch.Generator().manual_seed(7)
    big = torch.rand(2, 50, 6, 32, generator=g).to(_dev())
    A, X = big[..., :16], big[..., 16:]                       # last-dim slices: (D, N) block not dense
    H = mamba_b200.pscan(A, X)
    Hs = O.scan_sequential(A.cpu().double(), X.cpu().double())
    assert_close(H, Hs.float(), RTOL, ATOL)
    At, Xt = big.transpose(0, 1)[:, :, :, :16], big.transpose(0, 1)[:, :, :, 16:]   # (50, 2, 6, 16)
    H2 = mamba_b200.pscan(At, Xt)
    Hs2 = O.scan_sequential(At.cpu().double(), Xt.cpu().double())
    assert_close(H2, Hs2.float(), RTOL, ATOL)
    E = torch.empty(2, 0, 3, 16, device=_dev())
    assert mamba_b200.pscan(E, E).shape == (2, 0, 3, 16)


def test_bf16_io_fp32_state():
    import mamba_b200
    g = torch.Generator().manual_seed(11)
    shape = (2, 257, 8, 16)
    A = torch.exp(-torch.nn.functional.softplus(torch.randn(shape, generator=g))).bfloat16()
    X = torch.randn(shape, generator=g).bfloat16()
    H = mamba_b200.pscan(A.to(_dev()), X.to(_dev()))
    assert H.dtype == torch.bfloat16
    Hs = O.scan_sequential(A.double(), X.double())
    assert_close(H, Hs.float(), 2e-2, 2e-2)                   # bf16 output rounding


def test_full_size_split_consistency():
    """At the benchmark's per-row size: scanning a sequence equals scanning its two halves with
    the state carried over (a size-independent property, no oracle needed)."""
    from mamba_b200.pscan import pscan_fwd_raw
    g = torch.Generator(device="cuda").manual_seed(5)
    shape = (2, 2048, 1536, 16)
    A = torch.exp(-torch.nn.functional.softplus(torch.randn(shape, generator=g, device=_dev())))
    X = torch.randn(shape, generator=g, device=_dev())
    H, hT = pscan_fwd_raw(A, X, want_last=True)
    m = 1000
    H0, h0 = pscan_fwd_raw(A[:, :m], X[:, :m], want_last=True)
    H1, h1 = pscan_fwd_raw(A[:, m:], X[:, m:], h0=h0, want_last=True)
    assert torch.allclose(torch.cat([H0, H1], 1), H, rtol=1e-5, atol=1e-6)
    assert torch.allclose(h1, hT, rtol=1e-5, atol=1e-6)
    assert torch.allclose(hT.view(2, 1536, 16), H[:, -1], rtol=0, atol=0)
