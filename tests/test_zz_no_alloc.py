"""The allocation-free PScan forward (mb200_pscan_fwd_noalloc), called through the C ABI.

Some hosts of the library cannot allocate device memory when they call it (a server with a
pre-planned arena, a loop that must not hit cudaMalloc's synchronisation, a foreign runtime with
no allocator to offer), so this entry point keeps its scratch in a fixed array inside the
library.  The test drives it with ctypes on a shape that needs the scratch (a segmented launch)
and checks that it returns exactly what the ordinary entry point returns, twice in a row, since
the shared array still holds the first call's aggregates when the second call starts.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import pytest
import torch

from mamba_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, shape):
    g = torch.Generator().manual_seed(seed)
    A = torch.exp(-torch.nn.functional.softplus(torch.randn(shape, generator=g))).to(DEV)
    X = torch.randn(shape, generator=g).to(DEV)
    return A, X


def _call_noalloc(lib, A, X, H, hT, nseg):
    B, L, D, N = X.shape
    with torch.cuda.device(X.device):
        return lib.mb200_pscan_fwd_noalloc(
            A.data_ptr(), X.data_ptr(), H.data_ptr(), B, L, D * N, A.stride(0), A.stride(1),
            X.stride(0), X.stride(1), H.stride(0), H.stride(1), None, hT.data_ptr(), nseg,
            _lib.F32, torch.cuda.current_stream(X.device).cuda_stream)


def _call_plain(lib, A, X, H, hT, nseg):
    B, L, D, N = X.shape
    ws = torch.empty(2 * B * nseg * D * N, dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        rc = lib.mb200_pscan_fwd(
            A.data_ptr(), X.data_ptr(), H.data_ptr(), B, L, D * N, A.stride(0), A.stride(1),
            X.stride(0), X.stride(1), H.stride(0), H.stride(1), None, hT.data_ptr(), ws.data_ptr(),
            nseg, _lib.F32, torch.cuda.current_stream(X.device).cuda_stream)
    torch.cuda.synchronize()
    return rc


def test_noalloc_matches_plain_entry_point_twice():
    lib = _lib.load()
    shape = (2, 3000, 4, 16)                     # few channels, long L: the segmented path
    nseg = lib.mb200_pscan_segments(shape[0], shape[1], shape[2] * shape[3])
    assert nseg > 1, "this shape is meant to need scratch"
    assert 2 * shape[0] * nseg * shape[2] * shape[3] <= lib.mb200_pscan_noalloc_max_ws_floats()
    for seed in (1, 2):                          # second call finds the first call's leftovers
        A, X = _inputs(seed, shape)
        H_ref, hT_ref = torch.empty_like(X), torch.empty(shape[0], shape[2] * shape[3], device=DEV)
        assert _call_plain(lib, A, X, H_ref, hT_ref, nseg) == 0
        H, hT = torch.full_like(X, float("nan")), torch.full_like(hT_ref, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, A, X, H, hT, nseg)
        torch.cuda.synchronize()
        assert rc == 0, lib.mb200_strerror(rc)
        assert torch.cuda.memory_allocated() == before        # torch's allocator was not touched
        # same kernels, same launch geometry: float32 tolerance of the other parity tests
        assert torch.allclose(H, H_ref, rtol=1e-4, atol=1e-5)
        assert torch.allclose(hT, hT_ref, rtol=1e-4, atol=1e-5)
        # and against an independent answer: the un-segmented launch
        H1, h1 = torch.empty_like(X), torch.empty_like(hT_ref)
        assert _call_plain(lib, A, X, H1, h1, 1) == 0
        assert torch.allclose(H, H1, rtol=1e-4, atol=1e-5)
        # and against the CPU oracle's sequential loop, so this file stands on its own
        from oracle import scan_oracle as O
        Hs = O.scan_sequential(A.cpu().double(), X.cpu().double())
        assert torch.allclose(H.cpu().double(), Hs, rtol=1e-4, atol=1e-5)
        assert torch.allclose(hT.cpu().double(), Hs[:, -1].reshape(shape[0], -1), rtol=1e-4, atol=1e-5)


def test_noalloc_library_choice_and_limit():
    lib = _lib.load()
    A, X = _inputs(3, (1, 2000, 2, 16))
    H, hT = torch.empty_like(X), torch.empty(1, 32, device=DEV)
    assert _call_noalloc(lib, A, X, H, hT, 0) == 0            # nseg = 0: the library chooses
    H1, h1 = torch.empty_like(X), torch.empty_like(hT)
    assert _call_plain(lib, A, X, H1, h1, 1) == 0
    torch.cuda.synchronize()
    assert torch.allclose(H, H1, rtol=1e-4, atol=1e-5)
    # a request whose aggregates cannot fit the fixed array is refused and nothing is launched.  The
    # buffers are real and large enough for the call, so that a regression of the limit check would
    # show up as a wrong return code, not as an out-of-bounds access.
    big = (1, 64, 1024, 16)                                   # nseg 65: 2*1*65*16384 floats > 2^21
    Ab, Xb = _inputs(4, big)
    Hb, hb = torch.empty_like(Xb), torch.empty(1, big[2] * big[3], device=DEV)
    assert 2 * big[0] * 65 * big[2] * big[3] > lib.mb200_pscan_noalloc_max_ws_floats()
    rc = _call_noalloc(lib, Ab, Xb, Hb, hb, 65)
    torch.cuda.synchronize()
    assert rc == -6 and b"limit" in lib.mb200_strerror(rc)
