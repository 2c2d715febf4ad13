"""Start-up evidence: implementation identity, the native bundle manifest, receipts, plan caches, rank consensus."""
import datetime
import json
import multiprocessing as mp
import os
import socket

import pytest

from cubic_serve_b200.contracts import implementation as impl
from cubic_serve_b200.runtime.preparation import (EvidenceKey, EvidenceStore, StartupDisagreement, StartupPreparation,
                                                  StartupQualification, consensus)


def test_source_closure_follows_imports_without_importing():
    files = {str(p.relative_to(impl.PACKAGE_ROOT)) for p in impl.source_closure((f"{impl.PACKAGE_NAME}.runtime.engine",))}
    assert "runtime/engine.py" in files and "runtime/scheduler.py" in files and "runtime/__init__.py" in files
    assert "api/server.py" not in files                       # the engine does not reach the HTTP layer
    serving = {str(p.relative_to(impl.PACKAGE_ROOT)) for p in impl.source_closure((f"{impl.PACKAGE_NAME}.runtime.serving",))}
    assert {"api/server.py", "models/decoder.py", "ops/kernels.py", "executor/gpu_executor.py"} <= serving
    with pytest.raises(ValueError):
        impl.source_closure(("json",))


def test_identity_changes_with_content_and_extras(tmp_path, monkeypatch):
    pkg = tmp_path / "toy"
    (pkg / "sub").mkdir(parents=True)
    (pkg / "__init__.py").write_text("")
    (pkg / "sub" / "__init__.py").write_text("")
    (pkg / "a.py").write_text("from .sub import b\nfrom . import c\nimport json\n")
    (pkg / "sub" / "b.py").write_text("from ..c import f\n")
    (pkg / "c.py").write_text("def f():\n    return 1\n")
    (pkg / "unused.py").write_text("x = 1\n")
    monkeypatch.setattr(impl, "PACKAGE_ROOT", pkg)
    monkeypatch.setattr(impl, "PACKAGE_NAME", "toy")
    impl.identity.cache_clear()
    one = impl.identity("t", ("toy.a",), native=False)
    assert [f for f, _ in one.files] == ["__init__.py", "a.py", "c.py", "sub/__init__.py", "sub/b.py"]
    (pkg / "unused.py").write_text("x = 2\n")
    impl.identity.cache_clear()
    assert impl.identity("t", ("toy.a",), native=False).digest == one.digest      # outside the closure
    (pkg / "c.py").write_text("def f():\n    return 2\n")
    impl.identity.cache_clear()
    two = impl.identity("t", ("toy.a",), native=False)
    assert two.digest != one.digest
    assert impl.identity("t", ("toy.a",), native=False, extras=("-O2",)).digest != two.digest
    impl.identity.cache_clear()


def test_native_bundle_manifest_detects_changed_sources(tmp_path, monkeypatch):
    from cubic_serve_b200.ops import native
    csrc = tmp_path / "csrc"
    csrc.mkdir()
    (csrc / "k.cu").write_text("// kernel\n")
    (csrc / "k.cuh").write_text("// header\n")
    lib = tmp_path / "lib.so"
    lib.write_bytes(b"\x7fELF-not-really")
    monkeypatch.setattr(native, "CSRC", csrc)
    monkeypatch.setattr(native, "LIB_PATH", lib)
    monkeypatch.setattr(native, "MANIFEST_PATH", tmp_path / "lib.manifest.json")
    assert native.verify_bundle() == ["lib.manifest.json is missing or unreadable"]
    manifest = {"library_sha256": native._sha(lib), "flags": list(native.NVCC_FLAGS), "sources": native._source_digests()}
    native.MANIFEST_PATH.write_text(json.dumps(manifest))
    assert native.verify_bundle() == [] and not native.needs_build()
    os.utime(csrc / "k.cu", (4e9, 4e9))                       # a newer file time alone does not make the bundle stale
    assert not native.needs_build()
    (csrc / "k.cuh").write_text("// header, edited\n")
    (csrc / "new.cu").write_text("// another\n")
    assert native.verify_bundle() == ["k.cuh changed after the build", "new.cu was added after the build"]
    assert native.needs_build()
    lib.write_bytes(b"other")
    assert "lib.so is not the file the manifest describes" in native.verify_bundle()


def _ident(digest="d" * 64):
    return impl.ImplementationIdentity("t", digest, ())


def test_receipts_are_reused_only_under_the_same_digests(tmp_path):
    store = EvidenceStore(tmp_path / "ev")
    dev = {"name": "B200", "sms": 148}
    calls = []

    def run(ok=True):
        calls.append(1)
        return {"ok": ok, "results": [{"kernel": "k", "class": "exact"}]}

    sq = StartupQualification(store, _ident(), dev)
    report, reused = sq.ensure(run, {"quick": True})
    assert report["ok"] and not reused and len(calls) == 1
    report, reused = sq.ensure(run, {"quick": True})
    assert reused and len(calls) == 1
    assert sq.ensure(run, {"quick": True}, force=True)[1] is False and len(calls) == 2
    assert StartupQualification(store, _ident("e" * 64), dev).ensure(run, {"quick": True})[1] is False     # other code
    assert StartupQualification(store, _ident(), {"name": "H100", "sms": 132}).ensure(run, {"quick": True})[1] is False
    assert sq.ensure(run, {"quick": False})[1] is False                                                    # other operands
    # a failing report is recorded but never reused
    bad = StartupQualification(store, _ident("f" * 64), dev)
    assert bad.ensure(lambda: run(False))[0]["ok"] is False
    n = len(calls)
    assert bad.ensure(lambda: run(False))[1] is False and len(calls) == n + 1
    assert any(not e["ok"] for e in store.entries())
    # a torn or foreign file reads as absent
    key = sq.key({"quick": True})
    store._path(key).write_text("{not json")
    assert store.load(key) is None
    other = EvidenceKey("qualification", "x", "y", "z")
    store._path(key).write_text(json.dumps({"version": 1, "key": other.__dict__, "ok": True, "payload": {}}))
    assert store.load(key) is None


def test_plan_cache_computes_once(tmp_path):
    store = EvidenceStore(tmp_path)
    prep = StartupPreparation(store, _ident(), {"name": "B200"})
    n = []
    plan = prep.plan("gemm_splits", {"m": 256, "n": 4096, "k": 4096}, lambda: n.append(1) or {"splits": 2, "stream_k": False})
    again = StartupPreparation(store, _ident(), {"name": "B200"}).plan("gemm_splits", {"k": 4096, "n": 4096, "m": 256},
                                                                        lambda: n.append(1) or {"splits": 9})
    assert plan == again == {"splits": 2, "stream_k": False} and len(n) == 1
    assert prep.plan("gemm_splits", {"m": 16, "n": 4096, "k": 4096}, lambda: {"splits": 4}) == {"splits": 4}
    assert (prep.hits, prep.misses) == (0, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _consensus_rank(rank, port, q, disagree):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=30))
    local = {"implementation": "abc" if not (disagree and rank) else "abd", "model": "m", "tp": 2, "pages": 1000 - 100 * rank}
    try:
        q.put((rank, "ok", consensus(local, minimum=("pages",))))
    except StartupDisagreement as exc:
        q.put((rank, "disagree", str(exc)))
    dist.destroy_process_group()


@pytest.mark.parametrize("disagree", [False, True])
def test_rank_consensus_over_gloo(disagree):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_consensus_rank, args=(r, port, q, disagree)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    if disagree:
        assert all(kind == "disagree" and "'implementation'" in msg and "rank 1: 'abd'" in msg for _, kind, msg in got)
    else:
        assert all(kind == "ok" and val["pages"] == 900 and val["implementation"] == "abc" for _, kind, val in got)


def test_consensus_without_process_group_is_local():
    assert consensus({"pages": 7}, minimum=("pages",)) == {"pages": 7}


def test_qualify_with_receipt_runs_once(tmp_path):
    from cubic_serve_b200.guardrail.qualify import qualify_with_receipt
    calls = []
    run = lambda: calls.append(1) or {"ok": True, "results": []}
    assert qualify_with_receipt(0, quick=True, evidence_dir=tmp_path, run=run)[1] is False
    assert qualify_with_receipt(0, quick=True, evidence_dir=tmp_path, run=run)[1] is True
    assert len(calls) == 1
