"""Operator configuration: the few launch-policy numbers of the native kernels, overridable from a JSON file.

Role of the reference's immutable operator config (``ops/strategies.py:276`` ``OperatorConfig`` with families
``launch``, ``linear``, ``moe``, ``collective``): one validated object that every launch policy reads, so that a
deployment can pin or change a policy without touching code.  Here the families are:

``gemm``       which weight-GEMM kernel serves a shape (``ops/kernels.py::use_stream_k``), the split-K bounds of
               the per-tile kernel, a forced run length for the persistent kernel
``attention``  how many KV splits a decode step uses for a given number of row blocks
``moe``        rows per work item of the grouped expert GEMMs

``load_operator_config(path)`` reads ``{"gemm": {...}, "attention": {...}, "moe": {...}, "profiles": [...]}``; unknown
families or keys are errors (a typo must not silently keep the default).  Profiles override the base by device name,
model name, SM count and tensor-parallel size (reference: profiles by device / model / shape).  ``CUBIC_OPERATOR_CONFIG=/path.json`` or
``cubic serve --operator-config`` installs it process-wide before any kernel is launched.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields, replace


@dataclass(frozen=True)
class GemmPolicy:
    stream_k_max_rows: int = 256        # persistent kernel for quantized weights only up to this many batch rows ...
    stream_k_min_tile_ratio: float = 1.0   # ... and only when tiles > ratio * SMs (wave quantisation is what it removes)
    stream_k_bf16: bool = True          # bf16 weights (lm_head): persistent kernel whenever tiles > SMs
    stream_k_min_units: int = 0         # 0 = the kernel's own cost model
    split_k_max: int = 8                # per-tile kernel: largest split-K factor
    split_k_min_blocks: int = 8         # ... and the fewest k-blocks a split may get
    fuse_swiglu: bool = True            # SwiGLU in the epilogue of the gate/up GEMM (weight rows re-ordered at load)
    cta_pairs: bool = True              # persistent kernel on CTA pairs (cta_group::2) above stream_k_max_rows ...
    pair_min_blocks: int = 80           # ... when every pair gets at least this many k-blocks (else one CTA per tile)


@dataclass(frozen=True)
class AttentionPolicy:
    target_ctas: int = 296              # KV splits are chosen so that row blocks x kv heads x splits reaches this
    max_splits: int = 32


@dataclass(frozen=True)
class MoePolicy:
    rows_per_item_small: int = 32       # rows per grouped-GEMM work item while routes < threshold x experts
    rows_per_item_large: int = 64
    large_routes_per_expert: int = 32


@dataclass(frozen=True)
class OperatorConfig:
    gemm: GemmPolicy = field(default_factory=GemmPolicy)
    attention: AttentionPolicy = field(default_factory=AttentionPolicy)
    moe: MoePolicy = field(default_factory=MoePolicy)

    def validate(self) -> None:
        g, a, m = self.gemm, self.attention, self.moe
        if g.stream_k_max_rows < 0 or g.stream_k_min_units < 0 or not 1 <= g.split_k_max <= 64 or g.split_k_min_blocks < 1:
            raise ValueError("gemm policy out of range")
        if g.stream_k_min_tile_ratio <= 0:
            raise ValueError("gemm.stream_k_min_tile_ratio must be positive")
        if a.target_ctas < 1 or not 1 <= a.max_splits <= 64:
            raise ValueError("attention policy out of range")
        for v in (m.rows_per_item_small, m.rows_per_item_large):
            if v < 16 or v > 256 or v % 16:
                raise ValueError("moe rows per item must be a multiple of 16 in [16, 256]")
        if m.large_routes_per_expert < 1:
            raise ValueError("moe.large_routes_per_expert must be positive")


def _family(cls, data: object, name: str):
    if not isinstance(data, dict):
        raise ValueError(f"operator config: family {name!r} must be an object")
    known = {f.name: f.type for f in fields(cls)}
    unknown = sorted(set(data) - set(known))
    if unknown:
        raise ValueError(f"operator config: unknown key(s) {unknown} in family {name!r}")
    base = cls()
    typed = {}
    for k, v in data.items():
        want = type(getattr(base, k))
        if want is bool:
            if not isinstance(v, bool):
                raise ValueError(f"operator config: {name}.{k} must be true or false")
        elif isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ValueError(f"operator config: {name}.{k} must be a number")
        typed[k] = want(v)
    return replace(base, **typed)


_FAMILIES = {"gemm": GemmPolicy, "attention": AttentionPolicy, "moe": MoePolicy}
_MATCH_KEYS = ("device", "model", "sms", "tp")


def _profile_matches(match: object, context: dict) -> bool:
    """``match``: ``{"device": "NVIDIA B200*", "model": "dense-*", "sms": 148, "tp": 8}`` -- strings are shell patterns
    (case-insensitive), numbers compare equal; a key the context does not provide does not match."""
    import fnmatch
    if not isinstance(match, dict) or not match:
        raise ValueError("operator config: a profile needs a non-empty 'match' object")
    unknown = sorted(set(match) - set(_MATCH_KEYS))
    if unknown:
        raise ValueError(f"operator config: unknown match key(s) {unknown} (known: {list(_MATCH_KEYS)})")
    for key, want in match.items():
        have = context.get(key)
        if have is None:
            return False
        if isinstance(want, str):
            if not fnmatch.fnmatchcase(str(have).lower(), want.lower()):
                return False
        elif have != want:
            return False
    return True


def operator_config_from_dict(data: object, context: dict | None = None) -> OperatorConfig:
    """Top-level families are the base; ``"profiles": [{"match": {...}, "gemm": {...}, ...}, ...]`` are overrides by
    device name, model name, SM count and tensor-parallel size: every profile that matches ``context`` is applied in
    file order, a later one winning key by key.  Profiles are validated even when they do not match."""
    if not isinstance(data, dict):
        raise ValueError("operator config must be a JSON object")
    unknown = sorted(set(data) - set(_FAMILIES) - {"profiles"})
    if unknown:
        raise ValueError(f"operator config: unknown family {unknown}")
    merged = {name: dict(data.get(name, {})) if isinstance(data.get(name, {}), dict) else data.get(name) for name in _FAMILIES}
    profiles = data.get("profiles", [])
    if not isinstance(profiles, list):
        raise ValueError("operator config: 'profiles' must be a list")
    for i, prof in enumerate(profiles):
        if not isinstance(prof, dict):
            raise ValueError(f"operator config: profile {i} must be an object")
        bad = sorted(set(prof) - set(_FAMILIES) - {"match", "name"})
        if bad:
            raise ValueError(f"operator config: unknown key(s) {bad} in profile {i}")
        for name, cls in _FAMILIES.items():
            _family(cls, prof.get(name, {}), f"profiles[{i}].{name}")          # a typo is an error in any profile
        if _profile_matches(prof.get("match"), context or {}):
            for name in _FAMILIES:
                if isinstance(merged[name], dict):
                    merged[name].update(prof.get(name, {}))
    cfg = OperatorConfig(**{name: _family(cls, merged[name], name) for name, cls in _FAMILIES.items()})
    cfg.validate()
    return cfg


def load_operator_config(path: str, context: dict | None = None) -> OperatorConfig:
    with open(path, "r", encoding="utf-8") as f:
        return operator_config_from_dict(json.load(f), context)


def launch_context(model: str | None = None, tp: int = 1, device: int = 0) -> dict:
    """What profiles can match on, for the current process: GPU name and SM count (when a GPU is visible), the model
    name and the tensor-parallel size."""
    ctx: dict = {"tp": int(tp)}
    if model:
        ctx["model"] = model.split(":", 1)[1] if model.startswith("random:") else os.path.basename(model.rstrip("/"))
    try:
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(device)
            ctx.update(device=p.name, sms=p.multi_processor_count)
    except Exception:  # noqa: BLE001 - no GPU: device keys stay absent and device-specific profiles do not match
        pass
    return ctx


_active: OperatorConfig | None = None


def active() -> OperatorConfig:
    """The process-wide configuration (defaults, or the file named by ``CUBIC_OPERATOR_CONFIG``)."""
    global _active
    if _active is None:
        path = os.environ.get("CUBIC_OPERATOR_CONFIG")
        ctx = json.loads(os.environ.get("CUBIC_OPERATOR_CONTEXT") or "null")      # set by the process that chose profiles
        _active = load_operator_config(path, ctx if ctx is not None else launch_context()) if path else OperatorConfig()
    return _active


def install(cfg: OperatorConfig) -> None:
    global _active
    cfg.validate()
    _active = cfg
