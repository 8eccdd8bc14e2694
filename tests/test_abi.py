"""CPU-side checks of the boundary: the library loads, exports what the header declares, refuses
bad arguments without touching a GPU, and install()/uninstall() rebind the reference's names."""
import os
import re
import sys

import pytest
import torch

from tests.helpers import ROOT


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "mamba_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mb200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mamba_b200 import _lib
    lib = _lib.load()
    declared = _header_symbols()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    for name in _lib.exported_symbols():
        assert name in declared, f"{name} bound in Python but not declared in the header"
    assert lib.mb200_version() >= 100
    assert lib.mb200_sscan_chunk() == 8


def test_error_codes_without_a_gpu():
    from mamba_b200 import _lib
    lib = _lib.load()
    assert lib.mb200_strerror(0) == b"ok"
    # argument validation happens before any CUDA call
    assert lib.mb200_carry_fold(None, None, None, 0, 4, 0, 0, None) == -1
    assert lib.mb200_sscan_fwd(*([None] * 12), 1, 4, 8, 12, *([0] * 12), 0, 0, None) == -3      # N = 12
    assert lib.mb200_sscan_fwd(*([None] * 12), 1, 4, 8, 16, *([0] * 12), 7, 0, None) == -2      # dtype
    assert lib.mb200_sscan_fwd(*([None] * 12), 1, 4, 8, 16, *([0] * 12), 0, 0, None) == -1      # null x
    assert lib.mb200_pscan_fwd(None, None, None, -1, 4, 8, *([0] * 6), None, None, None, 1, 0, None) == -1
    assert lib.mb200_conv_step(*([None] * 6), 1, 8, 9, 8, 0, None) == -6                         # K > 8
    with pytest.raises(RuntimeError):
        _lib.check(-3, "probe")
    with pytest.raises(TypeError):
        _lib.dtype_code(torch.float64)


def test_cpu_tensors_are_rejected_loudly():
    import mamba_b200
    t = torch.zeros(1, 4, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mamba_b200.selective_scan_fn(t, t, -torch.ones(8, 16), torch.zeros(1, 4, 16), torch.zeros(1, 4, 16), torch.zeros(8))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mamba_b200.pscan(torch.ones(1, 4, 2, 16), torch.ones(1, 4, 2, 16))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mamba_b200.ssm_step_fn(torch.zeros(1, 8), None, torch.zeros(1, 8), -torch.ones(8, 16),
                               torch.zeros(1, 16), torch.zeros(1, 16))


def test_npo2_helpers_keep_reference_semantics():
    from mamba_b200 import npo2, pad_npo2
    assert [npo2(n) for n in (1, 2, 3, 5, 64, 65)] == [1, 2, 4, 8, 64, 128]
    X = torch.arange(2 * 5 * 3 * 4, dtype=torch.float32).view(2, 5, 3, 4)
    Y = pad_npo2(X)
    assert Y.shape == (2, 8, 3, 4) and torch.equal(Y[:, :5], X) and Y[:, 5:].abs().sum() == 0


REF = os.environ.get("MAMBAPY_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "mambapy")), reason="reference checkout not present")
def test_install_rebinds_reference_names_and_uninstall_restores():
    sys.path.insert(0, REF)
    try:
        import mambapy.pscan as rp
        import mambapy.mamba as rm
        import mamba_b200
        orig = (rp.pscan, rp.PScan, rm.pscan, rm.MambaBlock.selective_scan, rm.MambaBlock.step,
                rm.MambaBlock.ssm_step, rm.MambaBlock.selective_scan_seq, rm.MambaBlock.forward)
        sd_keys = list(rm.Mamba(rm.MambaConfig(d_model=16, n_layers=1)).state_dict().keys())
        mamba_b200.install()
        assert mamba_b200.installed()
        assert rp.pscan is mamba_b200.pscan and rm.pscan is mamba_b200.pscan and rp.PScan is mamba_b200.PScan
        assert rm.MambaBlock.selective_scan is mamba_b200.selective_scan
        assert rm.MambaBlock.step is mamba_b200.step and rm.MambaBlock.forward is orig[7]
        model = rm.Mamba(rm.MambaConfig(d_model=16, n_layers=1))
        assert list(model.state_dict().keys()) == sd_keys            # no new parameters or buffers
        with pytest.raises(RuntimeError, match="CUDA tensors only"):  # no silent CPU route
            model(torch.zeros(1, 8, 16))
        mamba_b200.uninstall()
        mamba_b200.install(fuse_block=True)
        assert rm.MambaBlock.forward is not orig[7]
        norm_fwd = rm.RMSNorm.forward
        assert norm_fwd.__name__ == "rmsnorm_forward"
        mamba_b200.uninstall()
        assert rm.RMSNorm.forward is not norm_fwd
        now = (rp.pscan, rp.PScan, rm.pscan, rm.MambaBlock.selective_scan, rm.MambaBlock.step,
               rm.MambaBlock.ssm_step, rm.MambaBlock.selective_scan_seq, rm.MambaBlock.forward)
        assert all(a is b for a, b in zip(orig, now)) and not mamba_b200.installed()
        y = model(torch.zeros(1, 8, 16))                              # the reference runs again on CPU
        assert y.shape == (1, 8, 16)
    finally:
        sys.path.remove(REF)
