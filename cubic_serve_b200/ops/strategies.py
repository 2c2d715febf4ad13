"""Operator configuration: the few launch-policy numbers of the native kernels, overridable from a JSON file.

Role of the reference's immutable operator config (``ops/strategies.py:276`` ``OperatorConfig`` with families
``launch``, ``linear``, ``moe``, ``collective``): one validated object that every launch policy reads, so that a
deployment can pin or change a policy without touching code.  Here the families are:

``gemm``       which weight-GEMM kernel serves a shape (``ops/kernels.py::use_stream_k``), the split-K bounds of
               the per-tile kernel, a forced run length for the persistent kernel
``attention``  how many KV splits a decode step uses for a given number of row blocks
``moe``        rows per work item of the grouped expert GEMMs

``load_operator_config(path)`` reads ``{"gemm": {...}, "attention": {...}, "moe": {...}}``; unknown families or keys
are errors (a typo must not silently keep the default).  ``CUBIC_OPERATOR_CONFIG=/path.json`` or
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


def operator_config_from_dict(data: object) -> OperatorConfig:
    if not isinstance(data, dict):
        raise ValueError("operator config must be a JSON object")
    families = {"gemm": GemmPolicy, "attention": AttentionPolicy, "moe": MoePolicy}
    unknown = sorted(set(data) - set(families))
    if unknown:
        raise ValueError(f"operator config: unknown family {unknown}")
    cfg = OperatorConfig(**{name: _family(cls, data.get(name, {}), name) for name, cls in families.items()})
    cfg.validate()
    return cfg


def load_operator_config(path: str) -> OperatorConfig:
    with open(path, "r", encoding="utf-8") as f:
        return operator_config_from_dict(json.load(f))


_active: OperatorConfig | None = None


def active() -> OperatorConfig:
    """The process-wide configuration (defaults, or the file named by ``CUBIC_OPERATOR_CONFIG``)."""
    global _active
    if _active is None:
        path = os.environ.get("CUBIC_OPERATOR_CONFIG")
        _active = load_operator_config(path) if path else OperatorConfig()
    return _active


def install(cfg: OperatorConfig) -> None:
    global _active
    cfg.validate()
    _active = cfg
