"""Puts an UNMODIFIED copy of the reference's `mambapy` package under oracle/_ref/.  TEST INFRASTRUCTURE.

    python oracle/make_ref.py [/path/to/reference]

The reference is pure Python on top of torch, so "building" it is an offline pip install of its own
setup.py into a target folder (a plain copy of the package directory if pip cannot run).  The result
is git-ignored: no reference source enters the history, but the folder travels with the working tree
to machines that do not have the reference checkout, so that
  * the GPU tests can run the reference's own classes (Mamba, MambaBlock, the bidirectional block of
    vim.py) with and without `mamba_b200.install()` and compare the two, and
  * bench.py's reference arm can time the reference's own code (cpu_baseline.kind = "reference").
Nothing in the shipped package imports it.  `ref_path()` returns the folder to put on sys.path, or
None when it has not been made.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
DEFAULT_REFERENCE = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def ref_path() -> str | None:
    return TARGET if os.path.isfile(os.path.join(TARGET, "mambapy", "pscan.py")) else None


def make_ref(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Install the reference into oracle/_ref/.  Returns the folder, or None if there is no checkout."""
    if not os.path.isdir(os.path.join(reference, "mambapy")):
        return ref_path()
    if ref_path() and not force:
        return TARGET
    shutil.rmtree(TARGET, ignore_errors=True)
    os.makedirs(TARGET, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")                 # the checkout is read-only; pip builds in-tree
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns("assets", "docs", "examples", "mlx", ".git"))
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--target", TARGET, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or not ref_path():
            shutil.rmtree(TARGET, ignore_errors=True)
            os.makedirs(TARGET, exist_ok=True)
            shutil.copytree(os.path.join(src, "mambapy"), os.path.join(TARGET, "mambapy"))
            how = "copied (pip install failed: %s)" % (r.stderr.strip().splitlines() or ["?"])[-1]
        else:
            how = "pip install --no-index --no-deps --target"
    with open(os.path.join(TARGET, "HOW.txt"), "w") as f:
        f.write(how + "\n")
    return TARGET


if __name__ == "__main__":
    print(make_ref(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE, force=True))
