"""install() / uninstall(): rebind the reference's scan entry points to the CUDA kernels.

The reference has no plugin registry; its seams are Python names.  `pscan` is imported BY NAME
into mambapy.mamba, mambapy.vim and mambapy.onnx.mamba_onnx (mambapy/mamba.py:9), so replacing
mambapy.pscan.pscan alone would not reach them; every importer is rebound, and the MambaBlock
methods of the scan path are replaced.  Nothing is added to any module's parameters or
buffers, so reference state_dicts keep loading unchanged.
"""
from __future__ import annotations

import importlib
import sys

from . import mamba as _m
from . import vim as _v
from .pscan import PScan as _PScan, pscan as _pscan

_saved: list[tuple[object, str, object]] = []

_PSCAN_IMPORTERS = ("mambapy.mamba", "mambapy.vim", "mambapy.onnx.mamba_onnx", "mambapy.jamba")
_BLOCK_METHODS = ("selective_scan", "selective_scan_seq", "ssm_step", "step")


def _swap(obj, name, new):
    _saved.append((obj, name, getattr(obj, name)))
    setattr(obj, name, new)


def installed() -> bool:
    return bool(_saved)


def install(fuse_block: bool = False) -> None:
    """Patch an importable `mambapy`.

    fuse_block=False keeps MambaBlock.forward/ssm as they are and swaps only the methods whose
    signatures the reference defines (selective_scan, selective_scan_seq, ssm_step, step) plus
    pscan/PScan.  fuse_block=True also swaps MambaBlock.ssm and MambaBlock.forward for the
    variants that run softplus, scan and gate in one kernel, Mamba.forward for a loop that fuses each
    layer's residual add into the next layer's RMSNorm, RMSNorm.forward for the one-pass kernel,
    and (when mambapy.vim has been imported) the bidirectional block's forward (mambapy/vim.py:205-261)
    for one that scans the second direction in place instead of flipping the sequence.
    """
    if _saved:
        return
    ref_pscan = importlib.import_module("mambapy.pscan")
    _swap(ref_pscan, "pscan", _pscan)
    _swap(ref_pscan, "PScan", _PScan)
    for modname in _PSCAN_IMPORTERS:
        mod = sys.modules.get(modname)
        if mod is None and modname == "mambapy.mamba":
            mod = importlib.import_module(modname)
        if mod is not None and hasattr(mod, "pscan"):
            _swap(mod, "pscan", _pscan)
    blocks = [sys.modules["mambapy.mamba"].MambaBlock]
    for modname, cls in (("mambapy.vim", "VMambaBlock"), ("mambapy.onnx.mamba_onnx", "MambaBlock")):
        mod = sys.modules.get(modname)
        if mod is not None and hasattr(mod, cls):
            blocks.append(getattr(mod, cls))
    for i, blk in enumerate(blocks):
        for name in _BLOCK_METHODS:
            # the ONNX variant's step() has another signature; only same-signature methods move
            if hasattr(blk, name) and (i == 0 or name in ("selective_scan", "selective_scan_seq")):
                _swap(blk, name, getattr(_m, name))
    if fuse_block:
        _swap(blocks[0], "ssm", _m.ssm)
        _swap(blocks[0], "forward", _m.forward)
        stack = getattr(sys.modules["mambapy.mamba"], "Mamba", None)
        if stack is not None:
            _swap(stack, "forward", _m.stack_forward)     # residual adds fused into the following RMSNorm
        for modname in ("mambapy.mamba", "mambapy.vim"):
            norm = getattr(sys.modules.get(modname), "RMSNorm", None)
            if norm is not None:
                _swap(norm, "forward", _m.rmsnorm_forward)
        vim = sys.modules.get("mambapy.vim")
        if vim is not None and hasattr(vim, "VMambaBlock"):
            # the bidirectional block: second direction scanned right-to-left inside the kernels
            _swap(vim.VMambaBlock, "forward", _v.forward)


def uninstall() -> None:
    """Undo install(); the reference's own code runs again."""
    while _saved:
        obj, name, old = _saved.pop()
        setattr(obj, name, old)
