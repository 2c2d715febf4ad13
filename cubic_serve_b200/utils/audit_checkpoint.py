"""Audit of a quantized checkpoint: inventory, shard digests, per-weight decode statistics, error against a source.

``cubic audit-checkpoint DIR [--reference BF16_DIR] [--json]`` admits the checkpoint (closed inventory: every tensor
owned by a logical weight, every logical weight present), hashes the shards, decodes every logical weight through its
quantization extension and checks what a loader silently assumes: the decoded shape, finite values, scales that are
positive and finite, no all-zero rows or groups of rows.  With ``--reference`` (the unquantized checkpoint the
quantized one was made from) it also reports the relative error of every weight and flags outliers against the
format's expected quantization noise.

Reference counterpart: ``tools/quantization/audit_checkpoint.py``.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

# relative L2 error a healthy quantization of Gaussian-like weights stays under (bits -> bound); a weight above it
# was quantized from other data than the reference, or its metadata is damaged
EXPECTED_REL_ERROR = {2: 0.60, 3: 0.35, 4: 0.18, 5: 0.10, 6: 0.06, 8: 0.02, 16: 0.005}


def _sha256(path: Path) -> str:
    h = hashlib.sha256()
    with path.open("rb") as f:
        for block in iter(lambda: f.read(1 << 22), b""):
            h.update(block)
    return h.hexdigest()


def _scale_findings(module: str, payload: dict) -> list[str]:
    out = []
    for suffix, t in payload.items():
        if "scale" in suffix and t.is_floating_point():
            v = t.float()
            if not torch.isfinite(v).all():
                out.append(f"{module}.{suffix}: non-finite scale values")
            elif (v < 0).any():
                out.append(f"{module}.{suffix}: negative scale values")
            elif (v == 0).all():
                out.append(f"{module}.{suffix}: all scales are zero")
    return out


def audit_checkpoint(path: str | Path, reference: str | Path | None = None, digests: bool = True,
                     max_weights: int | None = None) -> dict:
    from ..models.checkpoint import CheckpointError, SafetensorsDirectory, admit_checkpoint, logical_inventory
    from ..quantization import registry
    path = Path(path)
    findings: list[str] = []
    try:
        ck = admit_checkpoint(path)
    except (CheckpointError, OSError, ValueError) as exc:
        return {"ok": False, "path": str(path), "findings": [f"admission failed: {exc}"], "weights": [], "shards": {}}
    cfg, q = ck.cfg, ck.cfg.quant
    ext = registry.get(q.method)
    shards = {f: _sha256(path / f) for f in sorted({t.file for t in ck.store.tensors.values()})} if digests else {}
    ref_store = SafetensorsDirectory(reference) if reference else None
    linears, _plain = logical_inventory(cfg)
    bound = EXPECTED_REL_ERROR.get(q.bits, 0.2)
    weights = []
    for i, (module, shape) in enumerate(linears.items()):
        if max_weights is not None and i >= max_weights:
            break
        payload = ck.payload(module)
        findings += _scale_findings(module, payload)
        try:
            dense = ext.dense(payload, shape, q).float()
        except Exception as exc:  # noqa: BLE001 - any decode failure is the finding
            findings.append(f"{module}: decode failed: {type(exc).__name__}: {exc}")
            continue
        row = {"module": module, "shape": list(dense.shape), "quantized": q.method != "none" and set(payload) != {"weight"},
               "rms": float(dense.pow(2).mean().sqrt()), "max_abs": float(dense.abs().max())}
        if tuple(dense.shape) != tuple(shape):
            findings.append(f"{module}: decodes to {tuple(dense.shape)}, the architecture needs {tuple(shape)}")
        if not torch.isfinite(dense).all():
            findings.append(f"{module}: non-finite decoded values")
        else:
            dead = int((dense.abs().amax(dim=1) == 0).sum())
            row["zero_rows"] = dead
            if dead:
                findings.append(f"{module}: {dead} output rows decode to all zeros")
        if ref_store is not None:
            name = f"{module}.weight"
            if name not in ref_store:
                findings.append(f"{module}: the reference checkpoint has no {name}")
            else:
                w = ref_store.get(name).float()
                if w.shape != dense.shape:
                    findings.append(f"{module}: reference shape {tuple(w.shape)} differs from {tuple(dense.shape)}")
                else:
                    rel = float((dense - w).norm() / w.norm().clamp_min(1e-20))
                    row["rel_error"] = rel
                    limit = bound if row["quantized"] else EXPECTED_REL_ERROR[16]
                    if rel > limit:
                        findings.append(f"{module}: relative error {rel:.3f} exceeds the {q.bits}-bit bound {limit}")
        weights.append(row)
    for name in ck.plain.values():
        t = ck.store.get(name)
        if t.is_floating_point() and not torch.isfinite(t.float()).all():
            findings.append(f"{name}: non-finite values")
    errs = [w["rel_error"] for w in weights if "rel_error" in w]
    summary = {"weights": len(weights), "quantized": sum(w["quantized"] for w in weights)}
    if errs:
        summary.update(rel_error_mean=sum(errs) / len(errs), rel_error_max=max(errs))
    return {"ok": not findings, "path": str(path), "model": cfg.name, "format": f"{q.method} {q.bits}-bit group {q.group_size}",
            "findings": findings, "summary": summary, "shards": shards, "weights": weights}


def format_report(report: dict, verbose: bool = False) -> str:
    lines = [f"checkpoint {report['path']}: {report.get('model', '?')} ({report.get('format', '?')})"]
    for f, d in report.get("shards", {}).items():
        lines.append(f"  shard {f} sha256 {d}")
    if "summary" in report:
        s = report["summary"]
        lines.append(f"  {s['weights']} logical weights decoded, {s['quantized']} quantized" +
                     (f", relative error mean {s['rel_error_mean']:.4f} max {s['rel_error_max']:.4f}" if "rel_error_max" in s else ""))
    if verbose:
        for w in report["weights"]:
            lines.append(f"    {w['module']} {w['shape']} rms {w['rms']:.4g}" + (f" rel {w['rel_error']:.4f}" if "rel_error" in w else ""))
    for f in report["findings"]:
        lines.append(f"  FINDING: {f}")
    lines.append("audit passed" if report["ok"] else f"audit FAILED with {len(report['findings'])} findings")
    return "\n".join(lines)


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="audit a quantized checkpoint")
    ap.add_argument("checkpoint")
    ap.add_argument("--reference", help="the unquantized checkpoint this one was made from")
    ap.add_argument("--no-digests", action="store_true")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    report = audit_checkpoint(a.checkpoint, a.reference, digests=not a.no_digests)
    print(json.dumps(report, indent=1) if a.json else format_report(report, a.verbose))
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
