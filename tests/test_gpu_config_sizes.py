"""Parity at the SIZES of the benchmark configurations, against the CPU oracle (not kernel against
kernel): the fused scan exactly as bench.py instantiates it, PScan at the layer's D*N, the decode
step at the 2.8b widths, and the sequence-sharded scan at ED = 5120.

One batch row of each configuration is checked: rows are independent, and a row already crosses
every tile, ring-stage and barrier-phase boundary the full batch does (L = 2048 is 128 tiles)."""
import math

import pytest
import torch
import torch.nn.functional as F

from oracle import scan_oracle as O
from tests.helpers import assert_close, oracle_f64_blocked, scan_inputs, RefShapedBlock

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL, ATOL = 1e-4, 1e-5          # float32 contract
BF_RTOL, BF_ATOL = 2e-2, 2e-2    # bf16 I/O with float32 state


def _grad_check(got, want, rtol, atol, ctx):
    for k, w in want.items():
        scale = max(1.0, w.abs().max().item())
        assert_close(got[k], w.float(), rtol, atol * scale * 4, f"grad {k} {ctx}")


@pytest.mark.parametrize("dtype,subshards", [(torch.bfloat16, 1), (torch.float32, 1), (torch.bfloat16, None)])
def test_layer_130m_scan_as_benchmarked(dtype, subshards):
    """The instantiation bench.py times: L = 2048, ED = 1536, N = 16, softplus(delta + bias) inside,
    gated, the reference's dt-bias and S4D-real initialisation; bf16 I/O (and once in float32).  With
    subshards = 1 the row goes through one launch per direction, as the rows of the benchmark's batch of 8
    do; with None the library cuts the lone row into pieces, as it does for any batch-1 call."""
    import bench_workloads
    import mamba_b200
    w = bench_workloads.layer_130m_scan_inputs(1002, torch.device(DEV), Bsz=1, L=2048, dtype=dtype)
    names = ("x", "delta_raw", "z", "B", "C", "A", "D", "delta_bias")
    lv = {k: w[k].clone().requires_grad_() for k in names}
    y = mamba_b200.selective_scan_fn(lv["x"], lv["delta_raw"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"],
                                     delta_bias=lv["delta_bias"], subshards=subshards)
    y.backward(w["dy"])
    assert y.dtype == dtype
    inp = dict(x=w["x"], delta=w["delta_raw"], z=w["z"], B=w["B"], C=w["C"], A=w["A"], D=w["D"], gy=w["dy"])
    inp = {k: v.detach().float().cpu() for k, v in inp.items()}          # what the kernel saw, exactly
    yo, go = oracle_f64_blocked(inp, gated=True, bias=w["delta_bias"].detach().cpu())
    got = dict(x=lv["x"].grad, delta=lv["delta_raw"].grad, z=lv["z"].grad, B=lv["B"].grad, C=lv["C"].grad,
               A=lv["A"].grad, D=lv["D"].grad, bias=lv["delta_bias"].grad)
    if dtype == torch.float32:
        assert_close(y, yo.float(), RTOL, ATOL * max(1.0, yo.abs().max().item()), "y f32")
        _grad_check(got, go, RTOL, ATOL, "f32")
    else:
        assert_close(y, yo.float(), BF_RTOL, BF_ATOL * max(1.0, yo.abs().max().item()), "y bf16")
        _grad_check(got, go, BF_RTOL, BF_ATOL, "bf16")


def test_pscan_at_layer_width_one_row():
    """PScan at D*N = 1536*16, L = 2048, one batch row: H, gradA, gradX against the sequential loop."""
    import mamba_b200
    g = torch.Generator().manual_seed(1001)
    shape = (1, 2048, 1536, 16)
    A = torch.exp(-F.softplus(torch.randn(shape, generator=g)))
    X = torch.randn(shape, generator=g)
    G = torch.randn(shape, generator=g)
    Ad, Xd = A.to(DEV).requires_grad_(), X.to(DEV).requires_grad_()
    H = mamba_b200.pscan(Ad, Xd)
    H.backward(G.to(DEV))
    # closed form of the sequential loop and of its gradients, float64 (mambapy/pscan.py:188-224)
    A64, X64, G64 = A.double(), X.double(), G.double()
    Hs = O.scan_sequential(A64, X64)
    gX = torch.empty_like(G64)
    acc = torch.zeros_like(G64[:, 0])
    for t in range(shape[1] - 1, -1, -1):
        acc = G64[:, t] + (A64[:, t + 1] * acc if t + 1 < shape[1] else 0)
        gX[:, t] = acc
    gA = torch.zeros_like(G64)
    gA[:, 1:] = Hs[:, :-1] * gX[:, 1:]
    assert_close(H, Hs.float(), RTOL, ATOL * max(1.0, Hs.abs().max().item()), "H")
    assert_close(Xd.grad, gX.float(), RTOL, ATOL * max(1.0, gX.abs().max().item()), "gradX")
    assert_close(Ad.grad, gA.float(), RTOL, ATOL * max(1.0, gA.abs().max().item()) * 4, "gradA")


def test_step_at_2_8b_widths():
    """MambaBlock.step at d_model = 2560 (ED 5120, dt_rank 160), 2 layers x 8 steps, batch 4, from the
    cache (None, window): outputs, states and windows against the oracle's block_step."""
    from mamba_b200 import step
    torch.manual_seed(1003)
    d_model, Bsz, steps, n_layers = 2560, 4, 8, 2
    blocks = [RefShapedBlock(d_model) for _ in range(n_layers)]
    for blk in blocks:                        # the reference's dt-bias init (mambapy/mamba.py:158-163)
        with torch.no_grad():
            dt = torch.exp(torch.rand(2 * d_model) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
            blk.dt_proj.bias.copy_(dt + torch.log(-torch.expm1(-dt)))
    cuda_blocks = [RefShapedBlock(d_model).to(DEV) for _ in range(n_layers)]
    for cb, blk in zip(cuda_blocks, blocks):
        cb.load_state_dict(blk.state_dict())
    xs = torch.randn(steps, Bsz, d_model)
    ref_caches = [(None, torch.randn(Bsz, 2 * d_model, 3)) for _ in range(n_layers)]
    cu_caches = [(None, c[1].to(DEV)) for c in ref_caches]
    with torch.no_grad():
        for t in range(steps):
            xr, xc = xs[t].double(), xs[t].to(DEV)
            for li in range(n_layers):
                Wd = {k: v.detach().double() for k, v in blocks[li].weights().items()}
                h, win = ref_caches[li]
                out_r, ref_caches[li] = O.block_step(xr, (None if h is None else h.double(), win.double()), Wd)
                out_c, cu_caches[li] = step(cuda_blocks[li], xc, cu_caches[li])
                # TF32 is off by default for float32 matmuls: the projections are float32 GEMMs
                assert_close(out_c, out_r.float(), 1e-3, 1e-4 * max(1.0, out_r.abs().max().item()), f"out t={t} l={li}")
                assert_close(cu_caches[li][0], ref_caches[li][0].float(), 1e-3, 1e-4, f"h t={t} l={li}")
                assert_close(cu_caches[li][1], ref_caches[li][1].float(), 1e-5, 1e-6, f"window t={t} l={li}")
                xr, xc = out_r + xr, out_c + xc


def test_lshard_emulation_at_long_config_width():
    """ED = 5120, L = 4096 cut into 8 shards chained on one GPU (carry pass, decay product, fold, full
    pass; reverse carry pass, fold, full backward) against the float64 oracle on the whole sequence."""
    from tests.test_gpu_lshard import _emulate
    inp = scan_inputs(1004, 1, 4096, 5120, 16, dtype=torch.bfloat16)
    got = _emulate(inp, 8, torch.bfloat16)
    yo, go = oracle_f64_blocked(inp, gated=True, block=512)
    assert_close(got["y"], yo.float(), BF_RTOL, BF_ATOL * max(1.0, yo.abs().max().item()), "y")
    _grad_check({k: got[k] for k in go}, go, BF_RTOL, BF_ATOL, "lshard bf16")


@pytest.mark.parametrize("Bsz,L,ED,reverse", [(1, 640, 64, False), (2, 1100, 40, False), (1, 700, 32, True)])
def test_bf16_long_enough_to_wrap_the_ring_twice(Bsz, L, ED, reverse):
    """bf16 rings have 8 (forward) and 6 (backward) stages of 16 timesteps: a stage's barrier parity
    flips for the second time at timestep 256 (forward) / 192 (backward).  These lengths go past it."""
    from tests.test_gpu_sscan import _oracle, _kernel
    from tests.test_gpu_reverse import _oracle_reversed, _kernel_reversed
    inp = scan_inputs(4000 + L, Bsz, L, ED, 16, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(L)
    bias = torch.randn(ED, generator=g) * 0.5 - 2.5
    inp["delta"] = torch.randn(Bsz, L, ED, generator=g).bfloat16().float()
    if reverse:
        yo, ho, go = _oracle_reversed(inp, True, None, bias)
        yk, hk, gk = _kernel_reversed(inp, torch.bfloat16, True, None, bias)
    else:
        yo, ho, go = _oracle(inp, gated=True, bias=bias)
        yk, hk, gk = _kernel(inp, torch.bfloat16, gated=True, bias=bias, subshards=1)     # one launch over all of L
    assert_close(yk, yo.float(), BF_RTOL, BF_ATOL * max(1.0, yo.abs().max().item()), "y")
    assert_close(hk, ho.float(), RTOL, ATOL * max(1.0, ho.abs().max().item()), "state")
    _grad_check(gk, go, BF_RTOL, BF_ATOL, f"L={L}")
