"""mamba_b200: the selective-scan path of mamba.py as hand-written sm_100a CUDA kernels.

Public surface (mirrors the reference's names):

    from mamba_b200 import pscan, PScan                      # mambapy.pscan
    from mamba_b200 import selective_scan_fn                 # fused scan (+gate, +softplus)
    from mamba_b200.mamba import selective_scan, selective_scan_seq, ssm_step, step
    mamba_b200.install()      # rebind the reference's own names to these kernels
    mamba_b200.uninstall()    # put the reference's code back

The package is importable as `mamba_b200`; its directory carries the project name.
"""
from .pscan import PScan, pscan, npo2, pad_npo2
from .mamba import (selective_scan_fn, selective_scan, selective_scan_seq, ssm_step, step,
                    ssm_step_fn, conv_step_fn, causal_conv1d_silu, rms_norm, add_rms_norm)
from .patch import install, uninstall, installed
from ._lib import device_status

__all__ = ["PScan", "pscan", "npo2", "pad_npo2", "selective_scan_fn", "selective_scan",
           "selective_scan_seq", "ssm_step", "step", "ssm_step_fn", "conv_step_fn", "causal_conv1d_silu", "rms_norm", "add_rms_norm",
           "install", "uninstall", "installed", "device_status"]
