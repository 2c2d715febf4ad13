"""Model definitions: the built-in decoder families and externally supplied adapters.

A ``ModelDefinition`` names a family, the HuggingFace architectures it serves and the callables the runtime needs
(configuration parser, random-init and checkpoint weight loaders, runner factory).  The built-in families are the
plain GQA decoder, the GQA mixture-of-experts decoder and the hybrid Gated DeltaNet decoder, all executed by
``models.decoder.DecoderRunner``.

An adapter is a single Python file that defines ``MODEL_DEFINITION``.  It is loaded only after a source audit: the
file is parsed (never imported first) and rejected when it imports anything outside an allow-list or names a
facility that reaches outside the process (files, sockets, subprocesses, dynamic code).  The audit is a policy check
of what the adapter *says*, not a sandbox.

Reference counterpart: ``models/builtin.py:35-248`` (built-in definitions), ``models/loader.py:120-783`` (isolated
adapter loader with AST source-policy audit), ``models/adapter.py:78`` (``ModelDefinition``).
"""
from __future__ import annotations

import ast
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .config import ModelConfig


class ModelRegistryError(ValueError):
    pass


@dataclass(frozen=True)
class ModelDefinition:
    family: str
    architectures: tuple[str, ...]                      # HuggingFace ``architectures`` entries served by the family
    parse_config: Callable[[Path], ModelConfig]         # checkpoint directory's config.json -> ModelConfig
    random_weights: Callable[..., object]               # (cfg, device, seed, tp_rank, tp_size, ...) -> weights
    load_weights: Callable[..., object]                 # (admitted checkpoint, device, tp_rank, tp_size, ...) -> weights
    build_runner: Callable[..., object]                 # (cfg, weights, **runner options) -> runner
    description: str = ""


_definitions: dict[str, ModelDefinition] = {}


def register(defn: ModelDefinition, replace: bool = False) -> None:
    if defn.family in _definitions and not replace:
        raise ModelRegistryError(f"model family {defn.family!r} is already registered")
    _definitions[defn.family] = defn


def _builtin() -> None:
    if _definitions:
        return
    from .checkpoint import load_decoder_weights
    from .decoder import DecoderRunner, random_decoder_weights

    def parse(path: Path) -> ModelConfig:
        return ModelConfig.from_hf_config(Path(path) / "config.json" if Path(path).is_dir() else path)

    def runner(cfg, weights, **kw):
        return DecoderRunner(cfg, weights, **kw)

    common = dict(parse_config=parse, random_weights=random_decoder_weights, load_weights=load_decoder_weights,
                  build_runner=runner)
    register(ModelDefinition("gqa_decoder", ("LlamaForCausalLM", "Qwen2ForCausalLM", "Qwen3ForCausalLM", "MistralForCausalLM"),
                             description="grouped-query attention decoder with a SwiGLU feed-forward", **common))
    register(ModelDefinition("gqa_moe", ("Qwen3MoeForCausalLM", "Qwen2MoeForCausalLM", "MixtralForCausalLM"),
                             description="grouped-query attention decoder with routed experts", **common))
    register(ModelDefinition("qwen3_5", ("Qwen3NextForCausalLM", "Qwen3_5ForCausalLM"),
                             description="hybrid decoder: Gated DeltaNet layers with periodic gated full attention", **common))
    register(ModelDefinition("qwen3_5_moe", ("Qwen3_5MoeForCausalLM",),
                             description="hybrid decoder with routed experts", **common))

    def parse_q4(path: Path):
        from .qwen4_exp import parse_qwen4_exp_config_json
        p = Path(path)
        return parse_qwen4_exp_config_json((p / "config.json" if p.is_dir() else p).read_bytes())

    def random_q4(cfg, device="cpu", seed=0, *a, **kw):
        from .qwen4_exp import random_qwen4_exp_weights
        return random_qwen4_exp_weights(cfg, seed)

    def load_q4(ck, device="cpu", *a, **kw):
        from .qwen4_exp import qwen4_exp_tensor_shapes
        return {n: ck.store.get(n) for n in qwen4_exp_tensor_shapes(ck.cfg)}

    def runner_q4(cfg, weights, **kw):
        from .qwen4_exp import Qwen4ExpEagerExecutor
        return Qwen4ExpEagerExecutor(cfg, weights)

    register(ModelDefinition("qwen4_exp", ("Qwen4ExpForConditionalGeneration", "Qwen4ExpForCausalLM"),
                             parse_config=parse_q4, random_weights=random_q4, load_weights=load_q4, build_runner=runner_q4,
                             description="multi-stream residual decoder: Gated DeltaNet and block-selective attention "
                                         "layers, n-gram lexical embeddings, routed experts (eager executor)"))


def get(family: str) -> ModelDefinition:
    _builtin()
    if family not in _definitions:
        raise ModelRegistryError(f"unknown model family {family!r}; known: {sorted(_definitions)}")
    return _definitions[family]


def families() -> list[str]:
    _builtin()
    return sorted(_definitions)


def for_architecture(arch: str) -> ModelDefinition:
    """The definition that lists ``arch`` among its HuggingFace architectures."""
    _builtin()
    for d in _definitions.values():
        if arch in d.architectures:
            return d
    raise ModelRegistryError(f"no model definition serves architecture {arch!r}")


# ------------------------------------------------------------------ adapters
ALLOWED_IMPORT_ROOTS = ("torch", "numpy", "math", "dataclasses", "typing", "functools", "itertools", "collections",
                        "enum", "json", "cubic_serve_b200", "__future__")
FORBIDDEN_NAMES = ("exec", "eval", "compile", "__import__", "open", "input", "breakpoint", "globals", "vars", "getattr",
                   "setattr", "delattr")
FORBIDDEN_ATTRIBUTES = ("system", "popen", "spawn", "fork", "remove", "unlink", "rmtree", "__subclasses__", "__globals__",
                        "__builtins__", "__code__")


@dataclass(frozen=True)
class PolicyViolation:
    line: int
    what: str


def audit_source(text: str, filename: str = "<adapter>") -> list[PolicyViolation]:
    """Source-policy audit of an adapter: every import must start from an allowed root; no dynamic code, file, process
    or introspection facilities; no dunder attribute access except ``__name__`` / ``__doc__``."""
    try:
        tree = ast.parse(text, filename)
    except SyntaxError as exc:
        return [PolicyViolation(exc.lineno or 0, f"syntax error: {exc.msg}")]
    found: list[PolicyViolation] = []
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                if a.name.split(".")[0] not in ALLOWED_IMPORT_ROOTS:
                    found.append(PolicyViolation(node.lineno, f"import of {a.name!r} is not allowed"))
        elif isinstance(node, ast.ImportFrom):
            root = (node.module or "").split(".")[0]
            if node.level or root not in ALLOWED_IMPORT_ROOTS:
                found.append(PolicyViolation(node.lineno, f"import from {'.' * node.level}{node.module or ''!s} is not allowed"))
        elif isinstance(node, ast.Name) and node.id in FORBIDDEN_NAMES:
            found.append(PolicyViolation(node.lineno, f"use of {node.id!r} is not allowed"))
        elif isinstance(node, ast.Attribute):
            if node.attr in FORBIDDEN_ATTRIBUTES or (node.attr.startswith("__") and node.attr.endswith("__")
                                                     and node.attr not in ("__name__", "__doc__", "__init__", "__post_init__")):
                found.append(PolicyViolation(node.lineno, f"attribute {node.attr!r} is not allowed"))
        elif isinstance(node, (ast.Global, ast.Nonlocal)):
            found.append(PolicyViolation(node.lineno, "global / nonlocal statements are not allowed"))
    return sorted(found, key=lambda v: v.line)


def load_adapter(path: str | Path, register_it: bool = True) -> ModelDefinition:
    """Audit, then execute an adapter file and return (and register) its ``MODEL_DEFINITION``."""
    path = Path(path)
    text = path.read_text()
    violations = audit_source(text, str(path))
    if violations:
        lines = "; ".join(f"line {v.line}: {v.what}" for v in violations[:5])
        raise ModelRegistryError(f"adapter {path.name} violates the source policy: {lines}")
    namespace: dict = {"__name__": f"cubic_adapter_{path.stem}"}
    code = compile(text, str(path), "exec")
    exec(code, namespace)  # noqa: S102 - the source passed the audit above
    defn = namespace.get("MODEL_DEFINITION")
    if not isinstance(defn, ModelDefinition):
        raise ModelRegistryError(f"adapter {path.name} does not define MODEL_DEFINITION (a ModelDefinition)")
    if register_it:
        register(defn, replace=True)
    return defn
