"""Randomised shapes through the fused scan (tensor-map path, generic path, ragged tails, every
option) against the float64 oracle."""
import random

import pytest
import torch

from tests.helpers import scan_inputs
from tests.test_gpu_sscan import _oracle, _kernel, RTOL, ATOL, BF_RTOL, BF_ATOL
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(24))
def test_random_configuration(seed):
    rng = random.Random(seed)
    Bsz = rng.randint(1, 3)
    L = rng.choice([1, 2, 15, 16, 17, 31, 33, 47, 64, 95, 129, 200])
    ED = rng.choice([4, 8, 12, 24, 32, 36, 40, 64, 68, 96, 100, 132])
    N = rng.choice([16, 16, 16, 8, 32, 64])
    dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16])
    gated = rng.random() < 0.7
    use_bias = rng.random() < 0.5
    use_h0 = rng.random() < 0.4
    inp = scan_inputs(1000 + seed, Bsz, L, ED, N, dtype=dtype, structured_A=rng.random() < 0.5,
                      big_delta=rng.random() < 0.5)
    g = torch.Generator().manual_seed(seed)
    bias = h0 = None
    if use_bias:
        bias = torch.randn(ED, generator=g) * 0.5 - 2.5
        inp["delta"] = torch.randn(Bsz, L, ED, generator=g).to(dtype).float()
    if use_h0:
        h0 = torch.randn(Bsz, ED, N, generator=g)
    yo, ho, go = _oracle(inp, gated=gated, h0=h0, bias=bias)
    yk, hk, gk = _kernel(inp, dtype, gated=gated, h0=h0, bias=bias)
    rt, at = (RTOL, ATOL) if dtype == torch.float32 else (BF_RTOL, BF_ATOL)
    ctx = f"B={Bsz} L={L} ED={ED} N={N} {dtype} gated={gated} bias={use_bias} h0={use_h0}"
    assert_close(yk, yo.float(), rt, at * max(1.0, yo.abs().max().item()), "y " + ctx)
    assert_close(hk, ho.float(), RTOL, ATOL * max(1.0, ho.abs().max().item()), "state " + ctx)
    for k in go:
        if k == "z" and not gated:
            continue
        scale = max(1.0, go[k].abs().max().item())
        assert_close(gk[k], go[k].float(), rt, at * scale * 4, f"grad {k} " + ctx)


@pytest.mark.parametrize("seed", range(100, 112))
def test_random_configuration_reversed(seed):
    """The same, scanning from the last timestep to the first (in the kernels or through the flip
    fallback, whichever the shape gets)."""
    from tests.test_gpu_reverse import _oracle_reversed, _kernel_reversed
    rng = random.Random(seed)
    Bsz = rng.randint(1, 3)
    L = rng.choice([1, 7, 8, 9, 16, 23, 33, 64, 95, 129, 200])
    ED = rng.choice([8, 24, 32, 40, 64, 68, 96, 128])
    N = rng.choice([16, 16, 16, 8, 32])
    dtype = rng.choice([torch.float32, torch.float32, torch.bfloat16])
    gated = rng.random() < 0.7
    use_bias = rng.random() < 0.5
    use_h0 = rng.random() < 0.4
    inp = scan_inputs(2000 + seed, Bsz, L, ED, N, dtype=dtype, structured_A=rng.random() < 0.5,
                      big_delta=rng.random() < 0.5)
    g = torch.Generator().manual_seed(seed)
    bias = h0 = None
    if use_bias:
        bias = torch.randn(ED, generator=g) * 0.5 - 2.5
        inp["delta"] = torch.randn(Bsz, L, ED, generator=g).to(dtype).float()
    if use_h0:
        h0 = torch.randn(Bsz, ED, N, generator=g)
    yo, ho, go = _oracle_reversed(inp, gated, h0, bias)
    yk, hk, gk = _kernel_reversed(inp, dtype, gated, h0, bias)
    rt, at = (RTOL, ATOL) if dtype == torch.float32 else (BF_RTOL, BF_ATOL)
    ctx = f"reverse B={Bsz} L={L} ED={ED} N={N} {dtype} gated={gated} bias={use_bias} h0={use_h0}"
    assert_close(yk, yo.float(), rt, at * max(1.0, yo.abs().max().item()), "y " + ctx)
    assert_close(hk, ho.float(), RTOL, ATOL * max(1.0, ho.abs().max().item()), "state " + ctx)
    for k in go:
        if k == "z" and not gated:
            continue
        scale = max(1.0, go[k].abs().max().item())
        assert_close(gk[k], go[k].float(), rt, at * scale * 4, f"grad {k} " + ctx)
