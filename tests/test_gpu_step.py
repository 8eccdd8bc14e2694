"""Decode-step kernels against the reference's golden step trace and the CPU oracle."""
import pytest
import torch

from oracle import scan_oracle as O
from tests.helpers import golden, RefShapedBlock, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL, ATOL = 1e-4, 1e-5


def _rms(x, w):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w


def test_step_unrolled_matches_reference_trace():
    """Mamba.step unrolled over 11 tokens, 2 layers: outputs, states and conv windows."""
    from mamba_b200 import step
    g = golden("block_step.npz")
    xs = torch.from_numpy(g["xs"]).to(DEV)
    Bsz, L, Dm = xs.shape
    blocks = [RefShapedBlock(16).load_golden(g, li).to(DEV) for li in range(2)]
    norms = [torch.from_numpy(g[f"l{li}_norm_w"]).to(DEV) for li in range(2)]
    caches = [(None, torch.zeros(Bsz, 32, 3, device=DEV)) for _ in range(2)]
    outs = []
    with torch.no_grad():
        for t in range(L):
            x = xs[:, t]
            for li, blk in enumerate(blocks):
                old_inputs = caches[li][1]
                o, caches[li] = step(blk, _rms(x, norms[li]), caches[li])
                assert caches[li][1] is not old_inputs          # fresh cache tensors
                x = o + x
            outs.append(x)
            hs = torch.stack([c[0] for c in caches])
            assert_close(hs, g["h_after"][t], RTOL, ATOL, f"h after token {t}")
    outs = torch.stack(outs, 1)
    assert_close(outs, g["steps"], RTOL, ATOL)
    assert_close(outs, g["forward"], RTOL, ATOL)               # step == forward
    assert_close(torch.stack([c[1] for c in caches]), g["conv_after"], RTOL, ATOL)


@pytest.mark.parametrize("N", [8, 16, 32, 64])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ssm_step_fn_vs_oracle(N, dtype):
    from mamba_b200 import ssm_step_fn
    g = torch.Generator().manual_seed(N)
    Bsz, ED = 5, 72
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype).float()
    x, z, Bm, Cm = rnd(Bsz, ED), rnd(Bsz, ED), rnd(Bsz, N), rnd(Bsz, N)
    delta = torch.nn.functional.softplus(rnd(Bsz, ED) - 2).to(dtype).float()
    A = -torch.exp(torch.randn(ED, N, generator=g))
    D = torch.randn(ED, generator=g)
    h = torch.randn(Bsz, ED, N, generator=g)
    yo, ho = O.ssm_step(x.double(), h.double(), delta.double(), A.double(), Bm.double(), Cm.double(), D.double())
    yo = O.gate(yo, z.double())
    c = lambda t: t.to(DEV).to(dtype)
    yk, hk = ssm_step_fn(c(x), h.to(DEV), c(delta), A.to(DEV), c(Bm), c(Cm), D.to(DEV), z=c(z))
    tol = (RTOL, ATOL) if dtype == torch.float32 else (2e-2, 2e-2)
    assert_close(yk, yo.float(), *tol)
    assert_close(hk, ho.float(), RTOL, ATOL)
    y0, h0 = ssm_step_fn(c(x), None, c(delta), A.to(DEV), c(Bm), c(Cm), D.to(DEV))     # h = None -> zeros
    yo0, ho0 = O.ssm_step(x.double(), None, delta.double(), A.double(), Bm.double(), Cm.double(), D.double())
    assert_close(h0, ho0.float(), RTOL, ATOL)
    assert_close(y0, yo0.float(), *tol)


def test_fused_block_forward_matches_step_and_oracle():
    """forward() with softplus+scan+gate fused equals the step trace of the same weights."""
    from mamba_b200.mamba import forward, step
    g = golden("block_step.npz")
    blk = RefShapedBlock(16).load_golden(g, 0).to(DEV)
    x = torch.randn(3, 29, 16, generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.no_grad():
        yf = forward(blk, x)
        cache = (None, torch.zeros(3, 32, 3, device=DEV))
        ys = []
        for t in range(x.shape[1]):
            o, cache = step(blk, x[:, t], cache)
            ys.append(o)
    assert_close(yf, torch.stack(ys, 1), RTOL, ATOL)
    # and against the CPU oracle run on the same weights
    W = {k: v.detach().cpu() for k, v in blk.weights().items()}
    cache = (None, torch.zeros(3, 32, 3))
    outs = []
    for t in range(x.shape[1]):
        o, cache = O.block_step(x[:, t].cpu(), cache, W)
        outs.append(o)
    assert_close(yf, torch.stack(outs, 1), RTOL, ATOL)
