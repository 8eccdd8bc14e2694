"""Stand-ins for a memory checker and a race detector on the fused scan: canary rows around every
output, run-twice agreement, the bounded-wait give-up path, and layouts the backward must survive."""
import pytest
import torch

from tests.helpers import scan_inputs, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _padded(shape, dtype, pad=3, fill=12345.0):
    """A (B, L + 2*pad, ED + 16) buffer filled with a canary; returns (buffer, interior view).  The view's
    row stride stays a multiple of 16 bytes so the tensor-map path takes it."""
    Bsz, L, ED = shape
    buf = torch.full((Bsz, L + 2 * pad, ED + 16), fill, dtype=dtype, device=DEV)
    return buf, buf[:, pad:pad + L, 8:8 + ED]


@pytest.mark.parametrize("Bsz,L,ED,dtype", [(2, 100, 40, torch.float32), (1, 33, 72, torch.bfloat16),
                                            (2, 130, 64, torch.bfloat16)])
def test_outputs_stay_inside_their_rows(Bsz, L, ED, dtype):
    """y, dx, ddelta, dz are written into views with canary rows and columns around them: ragged L and
    ragged channel tiles must not spill a single element outside the (L, ED) interior."""
    from mamba_b200 import _lib
    from mamba_b200.mamba import sscan_fwd_raw
    lib = _lib.load()
    N = 16
    inp = scan_inputs(70 + L, Bsz, L, ED, N, dtype=dtype)
    d = {k: inp[k].to(DEV).to(dtype).contiguous() for k in ("x", "delta", "z", "B", "C", "gy")}
    A, D = inp["A"].to(DEV), inp["D"].to(DEV)
    ybuf, y = _padded((Bsz, L, ED), dtype)
    _, _, car = sscan_fwd_raw(d["x"], d["delta"], A, d["B"], d["C"], D, d["z"], want_carries=True)
    args = lambda t: (t.stride(0), t.stride(1))
    with torch.cuda.device(0):
        rc = lib.mb200_sscan_fwd(d["x"].data_ptr(), d["delta"].data_ptr(), d["z"].data_ptr(), A.data_ptr(),
                                 d["B"].data_ptr(), d["C"].data_ptr(), D.data_ptr(), None, None, y.data_ptr(),
                                 None, None, Bsz, L, ED, N, *args(d["x"]), *args(d["delta"]), *args(d["z"]),
                                 *args(d["B"]), *args(d["C"]), *args(y), _lib.dtype_code(dtype), 0,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    bufs = {k: _padded((Bsz, L, ED), dtype) for k in ("dx", "dd", "dz")}
    acc = torch.zeros(2 * Bsz * L * N + ED * N + ED, dtype=torch.float32, device=DEV)
    dB, dC = acc[:Bsz * L * N], acc[Bsz * L * N:2 * Bsz * L * N]
    dA, dD = acc[2 * Bsz * L * N:2 * Bsz * L * N + ED * N], acc[2 * Bsz * L * N + ED * N:]
    with torch.cuda.device(0):
        rc = lib.mb200_sscan_bwd(d["x"].data_ptr(), d["delta"].data_ptr(), d["z"].data_ptr(), A.data_ptr(),
                                 d["B"].data_ptr(), d["C"].data_ptr(), D.data_ptr(), None, d["gy"].data_ptr(),
                                 car.data_ptr(), None, bufs["dx"][1].data_ptr(), bufs["dd"][1].data_ptr(),
                                 bufs["dz"][1].data_ptr(), dB.data_ptr(), dC.data_ptr(), dA.data_ptr(), dD.data_ptr(),
                                 None, None, Bsz, L, ED, N, *args(d["x"]), *args(d["delta"]), *args(d["z"]),
                                 *args(d["B"]), *args(d["C"]), *args(d["gy"]), *args(bufs["dx"][1]),
                                 *args(bufs["dd"][1]), *args(bufs["dz"][1]), _lib.dtype_code(dtype), 0,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    for name, (buf, view) in dict(y=(ybuf, y), **bufs).items():
        mask = torch.ones_like(buf, dtype=torch.bool)
        mask[:, 3:3 + L, 8:8 + ED] = False
        assert bool((buf[mask] == 12345.0).all()), f"{name}: a write landed outside the output's rows"
        assert bool(torch.isfinite(view.float()).all()) and not bool((view == 12345.0).all()), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_run_twice_agreement(dtype):
    """Two launches on the same inputs: everything written with plain stores (y, last state, saved
    states, dx, ddelta, dz) is bitwise identical; the sums accumulated with floating-point atomics
    (dA, dD, dB, dC, d bias) agree to rounding (their order of addition is not fixed)."""
    from mamba_b200.mamba import sscan_fwd_raw, sscan_bwd_raw
    Bsz, L, ED, N = 3, 300, 96, 16
    inp = scan_inputs(11, Bsz, L, ED, N, dtype=dtype)
    d = {k: inp[k].to(DEV).to(dtype).contiguous() for k in ("x", "delta", "z", "B", "C", "gy")}
    A, D = inp["A"].to(DEV), inp["D"].to(DEV)
    runs = []
    for _ in range(2):
        y, hT, car = sscan_fwd_raw(d["x"], d["delta"], A, d["B"], d["C"], D, d["z"], want_last=True, want_carries=True)
        g = sscan_bwd_raw(d["x"], d["delta"], A, d["B"], d["C"], D, d["z"], None, d["gy"], car, want_g_out=True)
        runs.append((y, hT, car) + tuple(g))
    torch.cuda.synchronize()
    a, b = runs
    for i, nm in enumerate(("y", "hT", "carries", "dx", "ddelta", "dz")):
        assert torch.equal(a[i], b[i]), f"{nm} differs between two identical launches"
    assert torch.equal(a[11], b[11]), "g_out"
    for i, nm in ((6, "dB"), (7, "dC"), (8, "dA"), (9, "dD")):
        assert_close(a[i], b[i], 1e-5, 1e-5 * max(1.0, a[i].abs().max().item()), nm)


@pytest.mark.expects_wait_timeout
def test_bounded_wait_gives_up_and_reports():
    """A warp waits (a few hundred polls) on a barrier nothing arrives at: the kernel returns normally,
    the status word says so, reading it clears it, and the context stays usable."""
    from mamba_b200 import _lib
    lib = _lib.load()
    assert _lib.device_status(0) == 0
    with torch.cuda.device(0):
        assert lib.mb200_selftest_wait_timeout(500, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 1            # MB200_DEV_WAIT_TIMEOUT
    assert _lib.device_status(0) == 0            # cleared by the read
    assert lib.mb200_selftest_wait_timeout(0, None) != 0          # out-of-range limit is refused
    t = torch.ones(1024, device=DEV)
    assert float(t.sum()) == 1024.0              # the context is alive


def test_reverse_backward_with_a_misaligned_upstream_gradient():
    """reverse=True forward on aligned tensors, backward fed a gradient that is an offset slice of a
    wider tensor (row stride and base not 16-byte aligned): the backward must still run."""
    import mamba_b200
    from tests.test_gpu_reverse import _oracle_reversed
    Bsz, L, ED, N = 2, 40, 32, 16
    inp = scan_inputs(321, Bsz, L, ED, N)
    lv = {k: inp[k].to(DEV).requires_grad_() for k in ("x", "delta", "A", "B", "C", "D", "z")}
    y = mamba_b200.selective_scan_fn(lv["x"], lv["delta"], lv["A"], lv["B"], lv["C"], lv["D"], z=lv["z"], reverse=True)
    wide = torch.zeros(Bsz, L, ED + 3, device=DEV)
    wide[..., 1:1 + ED] = inp["gy"].to(DEV)
    y.backward(wide[..., 1:1 + ED])
    yo, _, go = _oracle_reversed(inp, True, None, None)
    assert_close(y, yo.float(), 1e-4, 1e-5)
    for k in ("x", "delta", "z", "B", "C", "A", "D"):
        scale = max(1.0, go[k].abs().max().item())
        assert_close(lv[k].grad, go[k].float(), 1e-4, 1e-5 * scale * 4, k)
