"""Reference arm of the benchmark: run the UNMODIFIED reference from ``baseline/_ref`` if it can run here.

The reference (QuantTrio/cubic-serve) pins ``torch==2.13.0``, ``triton==3.7.1`` and requires a CUDA 13.0
``nvcc`` at start-up to compile its kernels, and it serves only its own ``qwen3_5`` / ``qwen3_5_moe`` /
``qwen4_exp`` model families.  ``probe()`` checks, without running any of its GPU code, whether those
preconditions hold on this machine; if not, the arm reports why in one line.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import subprocess
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def probe() -> str | None:
    """Return None if the reference can be launched here, else a one-line reason."""
    if not os.path.isdir(os.path.join(REF_DIR, "cubic_serve")):
        return "reference not installed under baseline/_ref (offline pip install did not produce the package)"
    try:
        import torch
        import triton
    except ImportError as exc:  # pragma: no cover
        return f"missing dependency: {exc}"
    if not torch.__version__.startswith("2.13"):
        return (f"reference pins torch==2.13.0 (cu130) and triton==3.7.1; this image has torch {torch.__version__}, "
                f"triton {triton.__version__} and no network to install them")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    try:
        out = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.TimeoutExpired):
        return "no nvcc on this machine (the reference compiles its kernels at start-up)"
    if "release 13." not in out:
        return "reference requires CUDA 13.0 nvcc at start-up; this image has CUDA 12.9"
    return None


def run(args) -> dict:
    """The reference's engine cannot start on this image (``probe``).  Below the engine, its operator layer was tried
    on a B200 of this pool through its own public API (``baseline/reference_ops.py``): the stock Marlin path raises
    "Native CUDA compilation requires the CUDA 13.0 baseline", its Triton path fails to compile under Triton 3.6
    ("PassManager::run failed") or to launch ("function takes exactly 38 arguments (24 given)"); the record is
    ``profiles/reference_ops_same_box.md``.  So there is nothing of the reference that produces the metric here."""
    reason = probe()
    if reason is None:
        reason = ("reference serves only qwen3_5/qwen3_5_moe/qwen4_exp checkpoints; the dense 8B GQA benchmark config "
                  "has no model family in it")
    return {"impl": "reference", "unavailable": reason}
