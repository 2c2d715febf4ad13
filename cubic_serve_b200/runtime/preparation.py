"""Start-up evidence: qualification receipts, cached launch plans and the cross-rank agreement on them.

Three things happen between "weights loaded" and "ready to serve" that depend only on *which code* runs on *which
device* with *which operands*, not on the requests that follow:

* the numerical qualification of the kernels (``guardrail.qualify``) -- seconds, and identical on every start;
* launch plans: decisions derived from device queries and search (K splits per GEMM shape, persistent-kernel use,
  resident cluster counts, the KV page plan);
* under several ranks, the agreement that all of them run the same implementation on the same model with the same
  plan (and the smallest KV page count any of them can hold).

Receipts and plans are JSON files in an evidence directory, addressed by the SHA-256 of (kind, implementation digest,
device description, operand digest).  An entry is used only when all four recorded values equal the ones asked for,
so a change of any source file in the implementation's closure, of the build flags, of the GPU model or of the model
configuration invalidates it without any bookkeeping.  A failed qualification is recorded but never reused.

Reference counterpart: ``runtime/quantized_qualification.py:75`` (``StartupQualification``: receipts keyed by source
and operand digests), ``runtime/preparation.py:25`` (``StartupPreparation``: plan caches), cross-rank consensus via
``all_gather_object``.
"""
from __future__ import annotations

import json
import os
import tempfile
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from ..contracts.implementation import ImplementationIdentity, digest_of

RECEIPT_VERSION = 1


class StartupDisagreement(RuntimeError):
    """The ranks of a deployment do not agree on what they are about to run."""


def default_evidence_dir() -> Path:
    env = os.environ.get("CUBIC_EVIDENCE_DIR")
    if env:
        return Path(env)
    return Path(os.environ.get("XDG_CACHE_HOME", Path.home() / ".cache")) / "cubic_serve_b200" / "evidence"


def device_description(device: int = 0) -> dict:
    """What a plan or receipt depends on of the GPU: model name, SM count, memory size, compute capability and the
    driver's CUDA version.  Not the device index, not its UUID: eight equal GPUs share their evidence."""
    import torch
    if not torch.cuda.is_available():
        return {"name": "cpu", "sms": 0, "memory_gib": 0, "capability": [0, 0], "cuda": None}
    p = torch.cuda.get_device_properties(device)
    return {"name": p.name, "sms": p.multi_processor_count, "memory_gib": round(p.total_memory / 2 ** 30),
            "capability": [p.major, p.minor], "cuda": torch.version.cuda}


@dataclass(frozen=True)
class EvidenceKey:
    kind: str                 # "qualification", "plan:<name>"
    implementation: str       # ImplementationIdentity.digest
    device: str               # digest of the device description
    operands: str             # digest of the operand description (model configuration, runner options, shapes)

    def address(self) -> str:
        return digest_of([RECEIPT_VERSION, self.kind, self.implementation, self.device, self.operands])


class EvidenceStore:
    """Directory of JSON entries addressed by ``EvidenceKey``.  Writes are atomic (temporary file + rename), so ranks
    that start together and write the same entry cannot leave a torn file; unreadable or foreign entries read as
    absent."""

    def __init__(self, root: str | Path | None = None) -> None:
        self.root = Path(root) if root else default_evidence_dir()

    def _path(self, key: EvidenceKey) -> Path:
        return self.root / f"{key.kind.replace(':', '_').replace('/', '_')}-{key.address()[:32]}.json"

    def load(self, key: EvidenceKey) -> dict | None:
        try:
            entry = json.loads(self._path(key).read_text())
        except (OSError, ValueError):
            return None
        recorded = entry.get("key", {})
        if entry.get("version") != RECEIPT_VERSION or any(recorded.get(f) != getattr(key, f) for f in
                                                          ("kind", "implementation", "device", "operands")):
            return None
        return entry

    def save(self, key: EvidenceKey, payload: dict, ok: bool = True) -> Path:
        self.root.mkdir(parents=True, exist_ok=True)
        entry = {"version": RECEIPT_VERSION, "key": {"kind": key.kind, "implementation": key.implementation,
                                                      "device": key.device, "operands": key.operands},
                 "ok": bool(ok), "created": time.time(), "payload": payload}
        path = self._path(key)
        fd, tmp = tempfile.mkstemp(dir=self.root, prefix=path.stem, suffix=".tmp")
        try:
            with os.fdopen(fd, "w") as f:
                json.dump(entry, f, sort_keys=True)
            os.replace(tmp, path)
        except BaseException:
            try:
                os.unlink(tmp)
            except OSError:
                pass
            raise
        return path

    def entries(self) -> list[dict]:
        out = []
        for p in sorted(self.root.glob("*.json")) if self.root.exists() else []:
            try:
                out.append(json.loads(p.read_text()))
            except (OSError, ValueError):
                continue
        return out


class StartupQualification:
    """Runs the kernel qualification once per (implementation, device, operands) and keeps the receipt."""

    def __init__(self, store: EvidenceStore, identity: ImplementationIdentity, device: dict) -> None:
        self.store, self.identity, self.device = store, identity, device

    def key(self, operands) -> EvidenceKey:
        return EvidenceKey("qualification", self.identity.digest, digest_of(self.device), digest_of(operands))

    def ensure(self, run: Callable[[], dict], operands=None, force: bool = False) -> tuple[dict, bool]:
        """Returns ``(report, reused)``.  ``run`` is called unless a passing receipt exists; its report (a dict with
        an ``ok`` field) is recorded either way, and a failing one raises nothing here: the caller decides."""
        key = self.key(operands)
        if not force:
            entry = self.store.load(key)
            if entry is not None and entry["ok"] and entry["payload"].get("ok"):
                return entry["payload"], True
        report = run()
        self.store.save(key, report, ok=bool(report.get("ok")))
        return report, False


class StartupPreparation:
    """Cache of launch plans.  ``plan(name, operands, compute)`` returns the stored plan made under the same
    implementation, device and operands, or computes, stores and returns it.  Plans are JSON values."""

    def __init__(self, store: EvidenceStore, identity: ImplementationIdentity, device: dict) -> None:
        self.store, self.identity, self.device = store, identity, device
        self.hits = 0
        self.misses = 0

    def plan(self, name: str, operands, compute: Callable[[], object]):
        key = EvidenceKey(f"plan:{name}", self.identity.digest, digest_of(self.device), digest_of(operands))
        entry = self.store.load(key)
        if entry is not None and entry["ok"]:
            self.hits += 1
            return entry["payload"]["plan"]
        self.misses += 1
        value = compute()
        self.store.save(key, {"plan": value, "operands": operands})
        return value


def consensus(local: dict, minimum: tuple[str, ...] = (), group=None) -> dict:
    """Agreement of all ranks on ``local`` (a flat dict of JSON values).

    Every field must be equal on all ranks, except those named in ``minimum``: they are replaced by the smallest
    value any rank reported (the KV page count every rank can hold).  Raises ``StartupDisagreement`` naming the
    field and the ranks' values otherwise.  Without an initialised process group the local values are returned.
    """
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(local)
    gathered: list = [None] * dist.get_world_size(group)
    dist.all_gather_object(gathered, local, group=group)
    agreed = dict(local)
    for field in sorted(set().union(*[set(g) for g in gathered])):
        values = [g.get(field) for g in gathered]
        if field in minimum:
            agreed[field] = min(values)
        elif any(v != values[0] for v in values):
            raise StartupDisagreement(f"ranks disagree on {field!r}: " +
                                      ", ".join(f"rank {r}: {v!r}" for r, v in enumerate(values)))
    return agreed
