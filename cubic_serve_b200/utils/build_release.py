"""Build a release: the sm_100a kernel library, its bundle manifest, a wheel that carries both, and a release record.

``python -m cubic_serve_b200.utils.build_release --out dist`` compiles ``csrc/*.cu`` (when stale or ``--rebuild``),
checks that the library is the one its manifest and the sources describe, builds the wheel without network access
(``pip wheel --no-deps --no-build-isolation``), checks the wheel's contents, and writes ``release.json`` beside it:
wheel name and SHA-256, implementation digest, compiler, per-source digests.  Folders that the wheel build
creates in the source tree (``build/``, ``*.egg-info``) are removed afterwards.

Reference counterpart: ``tools/build_release.py`` and ``tools/build_cuda.py`` (release and kernel builds).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import shutil
import subprocess
import sys
import zipfile
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parent.parent.parent
REQUIRED_IN_WHEEL = ("cubic_serve_b200/libcubic_b200.so", "cubic_serve_b200/libcubic_b200.manifest.json",
                     "cubic_serve_b200/cli.py", "cubic_serve_b200/csrc/cubic_b200.h")


def check_wheel(path: Path) -> list[str]:
    """Problems of a built wheel: a required file missing, test or scratch files inside, a library that is not the one
    its manifest names."""
    problems = []
    with zipfile.ZipFile(path) as z:
        names = set(z.namelist())
        for need in REQUIRED_IN_WHEEL:
            if need not in names:
                problems.append(f"{need} is not in the wheel")
        top = {n.split("/", 1)[0] for n in names if "/" in n}
        allowed = {"cubic_serve_b200"} | {t for t in top if t.endswith((".dist-info", ".data"))}
        stray = sorted(n for n in names if ("/" in n and n.split("/", 1)[0] not in allowed) or n.endswith(".o"))
        if stray:
            problems.append(f"files that do not belong in a wheel: {stray[:4]}")
        if not any(n.endswith("entry_points.txt") for n in names):
            problems.append("no console script entry point")
        if not problems:
            manifest = json.loads(z.read("cubic_serve_b200/libcubic_b200.manifest.json"))
            digest = hashlib.sha256(z.read("cubic_serve_b200/libcubic_b200.so")).hexdigest()
            if manifest.get("library_sha256") != digest:
                problems.append("the library in the wheel is not the one its manifest describes")
    return problems


def build_release(out: Path, rebuild: bool = False, root: Path = REPO_ROOT) -> dict:
    from ..contracts.implementation import identity
    from ..ops import native
    if rebuild or native.needs_build():
        native.build(force=True)
    problems = native.verify_bundle()
    if problems:
        raise RuntimeError("native bundle does not match its sources: " + "; ".join(problems))
    out = Path(out).resolve()
    out.mkdir(parents=True, exist_ok=True)
    leftovers = [p for p in (root / "build", root / "cubic_serve_b200.egg-info") if not p.exists()]
    cmd = [sys.executable, "-m", "pip", "wheel", str(root), "--no-deps", "--no-build-isolation", "-w", str(out)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    for p in leftovers:                       # folders this build created in the source tree
        shutil.rmtree(p, ignore_errors=True)
    if res.returncode != 0:
        raise RuntimeError(f"wheel build failed:\n{res.stdout[-2000:]}")
    wheels = sorted(out.glob("cubic_serve_b200-*.whl"), key=lambda p: p.stat().st_mtime)
    if not wheels:
        raise RuntimeError("pip reported success but wrote no wheel")
    wheel = wheels[-1]
    problems = check_wheel(wheel)
    if problems:
        raise RuntimeError("the wheel is not releasable: " + "; ".join(problems))
    manifest = native.read_manifest() or {}
    record = {"wheel": wheel.name, "wheel_sha256": hashlib.sha256(wheel.read_bytes()).hexdigest(),
              "implementation": identity().digest, "arch": manifest.get("arch"), "nvcc": manifest.get("nvcc"),
              "library_sha256": manifest.get("library_sha256"), "sources": manifest.get("sources", {})}
    (out / "release.json").write_text(json.dumps(record, indent=1, sort_keys=True) + "\n")
    return record


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="build the kernel library, a wheel that carries it, and a release record")
    ap.add_argument("--out", default="dist")
    ap.add_argument("--rebuild", action="store_true", help="recompile the kernels even when the bundle is up to date")
    a = ap.parse_args(argv)
    record = build_release(Path(a.out), a.rebuild)
    print(json.dumps({k: v for k, v in record.items() if k != "sources"}, indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
