"""Release and checkpoint tools: ``audit-checkpoint`` and the wheel check of ``build_release``."""
import dataclasses
import hashlib
import json
import zipfile

import torch

from cubic_serve_b200.models.checkpoint import write_random_checkpoint
from cubic_serve_b200.models.config import ModelConfig, QuantSpec
from cubic_serve_b200.utils.audit_checkpoint import audit_checkpoint, format_report


def _cfg(quant):
    return ModelConfig(name="toy", family="gqa_decoder", num_layers=2, hidden_size=256, num_q_heads=4, num_kv_heads=2,
                       head_dim=64, intermediate_size=512, vocab_size=512, rope_theta=1e6, quant=quant)


def _rewrite(path, edit):
    from safetensors.torch import load_file, save_file
    f = path / "model.safetensors"
    tensors = load_file(str(f))
    edit(tensors)
    save_file(tensors, str(f))


def test_audit_passes_and_measures_error_against_the_source(tmp_path):
    q = write_random_checkpoint(tmp_path / "q", _cfg(QuantSpec("cubic", 4, 128)), seed=3)
    ref = write_random_checkpoint(tmp_path / "ref", _cfg(QuantSpec("none", 16, 0)), seed=3)
    r = audit_checkpoint(q, ref)
    assert r["ok"] and r["summary"]["weights"] == 14 and r["summary"]["quantized"] == 14
    assert 0.05 < r["summary"]["rel_error_max"] < 0.18
    assert len(r["shards"]) == 1 and len(next(iter(r["shards"].values()))) == 64
    assert "audit passed" in format_report(r, verbose=True)
    # a reference the checkpoint was NOT made from: every weight is flagged
    other = write_random_checkpoint(tmp_path / "other", _cfg(QuantSpec("none", 16, 0)), seed=4)
    bad = audit_checkpoint(q, other, digests=False)
    assert not bad["ok"] and len(bad["findings"]) == 14 and "exceeds the 4-bit bound" in bad["findings"][0]
    # an unquantized checkpoint audits against itself with (almost) no error
    same = audit_checkpoint(ref, ref, digests=False)
    assert same["ok"] and same["summary"]["quantized"] == 0 and same["summary"]["rel_error_max"] < 1e-6


def test_audit_reports_damaged_metadata_and_foreign_tensors(tmp_path):
    q = write_random_checkpoint(tmp_path / "q", _cfg(QuantSpec("int", 4, 128)), seed=1)

    def damage(t):
        s = t["model.layers.0.mlp.down_proj.weight_scale"].clone()
        s[3] = float("nan")
        t["model.layers.0.mlp.down_proj.weight_scale"] = s
        z = t["model.layers.1.self_attn.k_proj.weight_scale"].clone()
        z[5] = 0
        t["model.layers.1.self_attn.k_proj.weight_scale"] = z
    _rewrite(q, damage)
    r = audit_checkpoint(q, digests=False)
    text = "\n".join(r["findings"])
    assert not r["ok"]
    assert "down_proj.weight_scale: non-finite scale values" in text and "down_proj: non-finite decoded values" in text
    assert "k_proj: 1 output rows decode to all zeros" in text
    assert "audit FAILED" in format_report(r)
    _rewrite(q, lambda t: t.__setitem__("model.layers.0.extra.weight", torch.zeros(2)))
    closed = audit_checkpoint(q, digests=False)
    assert not closed["ok"] and "admission failed" in closed["findings"][0] and "no logical weight owns" in closed["findings"][0]


def test_audit_cli(tmp_path, capsys):
    from cubic_serve_b200.cli import main
    q = write_random_checkpoint(tmp_path / "q", _cfg(QuantSpec("cubic", 4, 128)), seed=3)
    assert main(["audit-checkpoint", str(q), "--no-digests", "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["summary"]["weights"] == 14


def test_wheel_check(tmp_path):
    from cubic_serve_b200.utils.build_release import check_wheel
    lib = b"\x7fELF-library"
    manifest = {"library_sha256": hashlib.sha256(lib).hexdigest()}

    def wheel(name, files):
        p = tmp_path / name
        with zipfile.ZipFile(p, "w") as z:
            for n, data in files.items():
                z.writestr(n, data)
        return p
    good = {"cubic_serve_b200/libcubic_b200.so": lib, "cubic_serve_b200/libcubic_b200.manifest.json": json.dumps(manifest),
            "cubic_serve_b200/cli.py": "", "cubic_serve_b200/csrc/cubic_b200.h": "",
            "cubic_serve_b200-0.1.0.dist-info/entry_points.txt": "[console_scripts]\ncubic = cubic_serve_b200.cli:main\n"}
    assert check_wheel(wheel("good.whl", good)) == []
    assert check_wheel(wheel("other_lib.whl", {**good, "cubic_serve_b200/libcubic_b200.so": b"another"})) == [
        "the library in the wheel is not the one its manifest describes"]
    missing = {k: v for k, v in good.items() if not k.endswith(".so")}
    problems = check_wheel(wheel("missing.whl", {**missing, "tests/test_x.py": ""}))
    assert "cubic_serve_b200/libcubic_b200.so is not in the wheel" in problems and any("do not belong" in p for p in problems)


def test_quantize_then_audit_then_load(tmp_path, capsys):
    """bf16 checkpoint -> ``cubic quantize`` -> the audit against the source passes, the loader takes it, shards
    and index are written when the shard limit is small."""
    from cubic_serve_b200.cli import main
    from cubic_serve_b200.models.checkpoint import admit_checkpoint, load_decoder_weights
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.utils.quantize_checkpoint import quantize_checkpoint
    src = write_random_checkpoint(tmp_path / "src", _cfg(QuantSpec("none", 16, 0)), seed=9)
    (src / "tokenizer_config.json").write_text("{}")
    assert main(["quantize", str(src), str(tmp_path / "q4"), "--format", "cubic", "--bits", "4", "--group-size", "128"]) == 0
    stats = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert stats["quantized"] == 14 and stats["shards"] == 1 and stats["compression"] > 1.5
    assert (tmp_path / "q4" / "model.safetensors").exists() and (tmp_path / "q4" / "tokenizer_config.json").exists()
    audit = audit_checkpoint(tmp_path / "q4", src, digests=False)
    assert audit["ok"] and audit["summary"]["quantized"] == 14 and audit["summary"]["rel_error_max"] < 0.18
    ck = admit_checkpoint(tmp_path / "q4")
    assert ck.cfg.quant.method == "cubic" and load_decoder_weights(ck, "cpu").layers[0].qkv.fmt == wq_pack.FMT_CUBIC4
    sharded = quantize_checkpoint(src, tmp_path / "i8", "int", 8, 128, shard_bytes=200_000)
    assert sharded["shards"] > 1 and (tmp_path / "i8" / "model.safetensors.index.json").exists()
    a8 = audit_checkpoint(tmp_path / "i8", src, digests=False)
    assert a8["ok"] and a8["summary"]["rel_error_max"] < 0.02
    import pytest
    from cubic_serve_b200.models.checkpoint import CheckpointError
    with pytest.raises(CheckpointError, match="already quantized"):
        quantize_checkpoint(tmp_path / "q4", tmp_path / "again", "cubic", 4, 128)
    with pytest.raises(ValueError):
        quantize_checkpoint(src, tmp_path / "x", "no-such-format", 4, 128)


def test_every_module_of_the_package_imports_without_a_gpu():
    """Import smoke of the whole package (rarely used entry points included): no module may need CUDA, a network or
    an optional dependency at import time."""
    import importlib
    import pkgutil

    import cubic_serve_b200
    failed = {}
    # the kernel library sits in the package directory but is a plain shared object (ctypes), not a Python module
    names = [m.name for m in pkgutil.walk_packages(cubic_serve_b200.__path__, "cubic_serve_b200.")
             if not m.name.endswith(".libcubic_b200")]
    assert len(names) > 60
    for name in names:
        try:
            importlib.import_module(name)
        except Exception as exc:  # noqa: BLE001 - collected and reported together
            failed[name] = f"{type(exc).__name__}: {exc}"
    assert not failed, failed
