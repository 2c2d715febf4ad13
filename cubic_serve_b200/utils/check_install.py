"""Installation check (``cubic check-install``): what is needed to serve, one line per item, exit code 0 when all
required items are present.  Nothing here launches a kernel; ``cubic qualify`` does that.

Reference counterpart: ``tools/check_install.py``, ``tools/build_cuda.py`` (build step), ``tools/cuda/check_graphs.py``.
"""
from __future__ import annotations

import ctypes
import importlib
import shutil
from pathlib import Path

REQUIRED_MODULES = ("torch", "numpy", "safetensors")
OPTIONAL_MODULES = ("transformers", "uvicorn", "xgrammar", "gguf", "prometheus_client", "PIL")   # PIL: image parts
REQUIRED_SYMBOLS = ("cb_wq_gemm", "cb_wq_gemm_sk", "cb_wq_gemm_act", "cb_wq_gemm_grouped", "cb_paged_attn",
                    "cb_rope_kv_write", "cb_rmsnorm", "cb_sample", "cb_tp_reduce_norm", "cb_ep_dispatch", "cb_moe_route",
                    "cb_gdn_conv", "cb_gdn_delta", "cb_hadamard", "cb_reasoning_budget")


def run_checks(build: bool = False) -> dict:
    items: list[dict] = []

    def add(name: str, ok: bool, detail: str, required: bool = True) -> None:
        items.append({"item": name, "ok": bool(ok), "required": required, "detail": detail})

    for mod in REQUIRED_MODULES + OPTIONAL_MODULES:
        required = mod in REQUIRED_MODULES
        try:
            m = importlib.import_module(mod)
            add(f"python module {mod}", True, str(getattr(m, "__version__", "present")), required)
        except Exception as exc:  # noqa: BLE001 - any import failure is the finding
            add(f"python module {mod}", False, f"{type(exc).__name__}: {exc}", required)
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if Path("/usr/local/cuda/bin/nvcc").exists() else None)
    add("nvcc (needed to build the kernels)", nvcc is not None, nvcc or "not found", required=False)

    from ..ops import native
    lib_path = native.CSRC.parent / "libcubic_b200.so"
    if build and nvcc:
        try:
            native.build()
        except Exception as exc:  # noqa: BLE001
            add("build of csrc/*.cu for sm_100a", False, f"{type(exc).__name__}: {exc}")
    add("native library", lib_path.exists(), str(lib_path) if lib_path.exists() else "missing: run `python __graft_entry__.py`")
    if lib_path.exists():
        try:
            lib = ctypes.CDLL(str(lib_path))
            missing = [s for s in REQUIRED_SYMBOLS if not hasattr(lib, s)]
            add("native entry points", not missing, "all present" if not missing else f"missing {missing}")
        except OSError as exc:
            add("native entry points", False, f"cannot load: {exc}")
        problems = native.verify_bundle()
        add("native library matches its sources (bundle manifest)", not problems,
            "source digests, flags and library digest agree" if not problems else "rebuild: " + "; ".join(problems[:4]),
            required=False)
        from ..contracts.implementation import identity
        add("implementation identity", True, identity().short(), required=False)
    try:
        import torch
        if torch.cuda.is_available():
            n = torch.cuda.device_count()
            caps = sorted({torch.cuda.get_device_capability(i) for i in range(n)})
            add("CUDA devices", True, f"{n} x {torch.cuda.get_device_name(0)}")
            add("compute capability 10.0 (sm_100a kernels)", caps == [(10, 0)], f"found {caps}")
            if n > 1:
                p2p = all(torch.cuda.can_device_access_peer(0, i) for i in range(1, n))
                add("peer access between GPUs (fused tensor / expert parallelism)", p2p, "yes" if p2p else "no", required=False)
        else:
            add("CUDA devices", False, "none visible: only the CPU reference path (--execution-mode eager) can run", required=False)
    except Exception as exc:  # noqa: BLE001
        add("CUDA devices", False, f"{type(exc).__name__}: {exc}", required=False)
    ok = all(i["ok"] for i in items if i["required"])
    return {"ok": ok, "items": items}


def format_report(report: dict) -> str:
    lines = []
    for i in report["items"]:
        mark = "ok  " if i["ok"] else ("FAIL" if i["required"] else "warn")
        lines.append(f"[{mark}] {i['item']}: {i['detail']}")
    lines.append("installation is complete" if report["ok"] else "installation is NOT complete")
    return "\n".join(lines)
