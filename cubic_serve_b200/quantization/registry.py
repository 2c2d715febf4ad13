"""Quantization extensions: one descriptor per weight format and the registry that resolves them.

A format is described once -- how its ``quantization_config`` block is recognised, which payload tensors a logical
weight owns on disk, how a payload decodes to a dense matrix, how a dense matrix is quantized into a payload (random
checkpoints, tests), which packed layout the tensor-core GEMM consumes natively and which compute modes it offers --
and everything else (checkpoint admission, loaders, the random-checkpoint writer, ``cubic inspect-model``) asks the
registry.  Out-of-tree formats register through the ``cubic_serve_b200.quantization`` entry-point group or by
calling ``register`` before a checkpoint is admitted.

Reference counterpart: ``quantization/api.py`` (extension descriptor), ``quantization/registry.py:36-85`` (builtins
``awq, fp8, nvfp4, cubic, int, ggml``, entry-point discovery, compute-mode checks).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

ENTRY_POINT_GROUP = "cubic_serve_b200.quantization"


class QuantizationRegistryError(ValueError):
    pass


@dataclass(frozen=True)
class QuantizationExtension:
    name: str                                    # ``QuantSpec.method`` this extension serves
    payload_suffixes: tuple[str, ...]            # ``<module>.<suffix>`` tensors a logical weight may own
    compute_modes: tuple[str, ...]               # offered modes, the first is the default (e.g. ``w4a16``)
    native_format: int | None                    # ``ops.wq_pack`` layout the GEMM decodes in its main loop; None = bf16 at load
    detect: Callable[[dict], object | None]      # quantization_config block -> QuantSpec, or None when it is another format
    dense: Callable[[dict, tuple, object], object]       # (payload, (N, K), QuantSpec) -> fp32 [N, K]
    quantize: Callable[[object, object], dict]           # (fp32 [N, K], QuantSpec) -> payload
    config_json: Callable[[object], dict | None]         # QuantSpec -> quantization_config block (None = unquantized)
    description: str = ""


_extensions: dict[str, QuantizationExtension] = {}
_builtins_loaded = False
_entry_points_loaded = False


def register(ext: QuantizationExtension, replace: bool = False) -> None:
    if not ext.name or not ext.compute_modes:
        raise QuantizationRegistryError("an extension needs a name and at least one compute mode")
    if ext.name in _extensions and not replace:
        raise QuantizationRegistryError(f"quantization extension {ext.name!r} is already registered")
    _extensions[ext.name] = ext


def _ensure_builtins() -> None:
    global _builtins_loaded
    if not _builtins_loaded:
        _builtins_loaded = True
        from . import builtin
        for ext in builtin.extensions():
            if ext.name not in _extensions:
                register(ext)


def discover_entry_points() -> list[str]:
    """Load extensions published by installed distributions; returns the names added.  An entry point is a callable
    that returns one extension or an iterable of them.  A broken plug-in is an error, not a silent skip."""
    global _entry_points_loaded
    _ensure_builtins()
    added: list[str] = []
    if _entry_points_loaded:
        return added
    _entry_points_loaded = True
    from importlib import metadata
    try:
        eps = metadata.entry_points(group=ENTRY_POINT_GROUP)
    except TypeError:                      # importlib.metadata of older interpreters
        eps = metadata.entry_points().get(ENTRY_POINT_GROUP, [])
    for ep in eps:
        made = ep.load()()
        for ext in ([made] if isinstance(made, QuantizationExtension) else list(made)):
            if not isinstance(ext, QuantizationExtension):
                raise QuantizationRegistryError(f"entry point {ep.name!r} did not return a QuantizationExtension")
            register(ext)
            added.append(ext.name)
    return added


def get(name: str) -> QuantizationExtension:
    _ensure_builtins()
    ext = _extensions.get(name)
    if ext is None:
        discover_entry_points()
        ext = _extensions.get(name)
    if ext is None:
        raise QuantizationRegistryError(f"no quantization extension for weight format {name!r}; known: {sorted(_extensions)}")
    return ext


def names() -> list[str]:
    _ensure_builtins()
    return sorted(_extensions)


def detect(quantization_config: dict):
    """``quantization_config`` block of a checkpoint -> QuantSpec of the extension that recognises it."""
    _ensure_builtins()
    if not quantization_config:
        return get("none").detect({})
    for attempt in range(2):
        for ext in _extensions.values():
            if ext.name == "none":
                continue
            spec = ext.detect(quantization_config)
            if spec is not None:
                return spec
        if attempt == 0 and not discover_entry_points():
            break
    method = quantization_config.get("quant_method") or quantization_config.get("format")
    raise ValueError(f"unsupported quantization_config: {method!r}")


def resolve_compute_mode(name: str, requested: str | None = None) -> str:
    """The compute mode a format runs in: its default, or ``requested`` when the format offers it."""
    ext = get(name)
    if requested is None or requested == "auto":
        return ext.compute_modes[0]
    if requested not in ext.compute_modes:
        raise QuantizationRegistryError(f"format {name!r} offers compute modes {list(ext.compute_modes)}, not {requested!r}")
    return requested
