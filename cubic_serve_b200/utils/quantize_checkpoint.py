"""Quantize an unquantized checkpoint into one of the registered weight formats.

``cubic quantize SRC DST --format cubic --bits 4 --group-size 128`` reads a HuggingFace-style directory with bf16 /
fp16 / fp32 weights, quantizes every logical linear weight of the architecture through the format's quantization
extension (round-to-nearest on the format's grid; no calibration data), copies the other tensors (embeddings, norms,
router, small control projections) unchanged, and writes ``DST`` with the format's ``quantization_config``.  The
result is what ``cubic audit-checkpoint DST --reference SRC`` checks and what ``cubic serve DST`` loads.  Shards are
written one source shard at a time, so peak memory is one shard plus one weight.

Reference counterpart: the quantized-checkpoint schema of ``models/quantized.py`` (payload naming
``<module>.<suffix>``); the reference ships no quantizer of its own.
"""
from __future__ import annotations

import json
import shutil
from pathlib import Path

import torch

KEEP_UNQUANTIZED = ("in_proj_ba",)           # few-row control projections stay in bf16 (as in published checkpoints)


def quantize_checkpoint(src: str | Path, dst: str | Path, method: str, bits: int, group_size: int,
                        shard_bytes: int = 4 << 30) -> dict:
    from safetensors.torch import save_file

    from ..models.checkpoint import CheckpointError, SafetensorsDirectory, _quant_config_json, logical_inventory, quantize_payload
    from ..models.config import ModelConfig, QuantSpec
    from ..quantization import registry
    src, dst = Path(src), Path(dst)
    cfg = ModelConfig.from_hf_config(src / "config.json")
    if cfg.quant.method != "none":
        raise CheckpointError(f"{src} is already quantized ({cfg.quant.method})")
    q = QuantSpec(method, bits, group_size)
    registry.get(method)                                   # unknown formats fail before anything is written
    store = SafetensorsDirectory(src)
    linears, plain = logical_inventory(cfg)
    expected = {f"{m}.weight" for m in linears} | set(plain)
    missing, extra = sorted(expected - set(store.tensors)), sorted(set(store.tensors) - expected)
    if missing or extra:
        raise CheckpointError(f"source inventory does not match the architecture: missing {missing[:3]}, unowned {extra[:3]}")
    dst.mkdir(parents=True, exist_ok=True)
    shard: dict[str, torch.Tensor] = {}
    weight_map: dict[str, str] = {}
    files: list[str] = []
    size = 0
    stats = {"quantized": 0, "copied": 0, "source_bytes": 0, "written_bytes": 0}

    def flush() -> None:
        nonlocal shard, size
        if not shard:
            return
        name = f"model-{len(files) + 1:05d}.safetensors"
        save_file(shard, str(dst / name))
        files.append(name)
        for k in shard:
            weight_map[k] = name
        shard, size = {}, 0

    def put(name: str, t: torch.Tensor) -> None:
        nonlocal size
        t = t.contiguous()
        nbytes = t.numel() * t.element_size()
        if size and size + nbytes > shard_bytes:
            flush()
        shard[name] = t
        size += nbytes
        stats["written_bytes"] += nbytes

    for module, shape in linears.items():
        w = store.get(f"{module}.weight")
        stats["source_bytes"] += w.numel() * w.element_size()
        if tuple(w.shape) != tuple(shape):
            raise CheckpointError(f"{module}.weight has shape {tuple(w.shape)}, the architecture needs {tuple(shape)}")
        if module.endswith(KEEP_UNQUANTIZED):
            put(f"{module}.weight", w.to(torch.bfloat16))
            stats["copied"] += 1
            continue
        for suffix, t in quantize_payload(w.float(), q).items():
            put(f"{module}.{suffix}", t)
        stats["quantized"] += 1
    for name in plain:
        t = store.get(name)
        stats["source_bytes"] += t.numel() * t.element_size()
        put(name, t)
        stats["copied"] += 1
    flush()
    # single shard: the conventional file name and no index
    if len(files) == 1:
        (dst / files[0]).rename(dst / "model.safetensors")
    else:
        final = {f: f"model-{i + 1:05d}-of-{len(files):05d}.safetensors" for i, f in enumerate(files)}
        for old, new in final.items():
            (dst / old).rename(dst / new)
        (dst / "model.safetensors.index.json").write_text(json.dumps(
            {"metadata": {"total_size": stats["written_bytes"]}, "weight_map": {k: final[v] for k, v in weight_map.items()}}, indent=1))
    hf = json.loads((src / "config.json").read_text())
    qc = _quant_config_json(q)
    if qc:
        hf["quantization_config"] = qc
    (dst / "config.json").write_text(json.dumps(hf, indent=1))
    for extra_file in ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "generation_config.json",
                       "vocab.json", "merges.txt", "tokenizer.model", "chat_template.jinja"):
        if (src / extra_file).exists():
            shutil.copy2(src / extra_file, dst / extra_file)
    stats.update(format=f"{method} {bits}-bit group {group_size}", shards=len(files),
                 compression=round(stats["source_bytes"] / max(stats["written_bytes"], 1), 2))
    return stats


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="quantize an unquantized checkpoint into a registered weight format")
    ap.add_argument("source")
    ap.add_argument("destination")
    ap.add_argument("--format", default="cubic")
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--shard-gib", type=float, default=4.0)
    a = ap.parse_args(argv)
    print(json.dumps(quantize_checkpoint(a.source, a.destination, a.format, a.bits, a.group_size, int(a.shard_gib * 2 ** 30))))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
