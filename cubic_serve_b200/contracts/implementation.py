"""Implementation identity: a digest over everything whose change can change what a model computes.

Start-up evidence (qualification receipts, cached launch plans) is only valid for the code that produced it.  The
identity of an implementation is therefore a SHA-256 over the *source closure* of its entry modules: the Python files
of this package that the entry modules import, directly or through other package modules (found by parsing the
import statements, nothing is imported or executed), plus the native sources and build flags of the kernel library.
A cached plan or receipt names the digest it was made under and is ignored under any other.

Reference counterpart: ``contracts/implementation.py:88`` (source-closure hashing of implementation modules).
"""
from __future__ import annotations

import ast
import hashlib
import json
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parent.parent
PACKAGE_NAME = PACKAGE_ROOT.name


@dataclass(frozen=True)
class ImplementationIdentity:
    name: str
    digest: str                       # hex SHA-256 over the sorted (relative path, file digest) pairs and the extras
    files: tuple[tuple[str, str], ...]

    def short(self) -> str:
        return self.digest[:16]

    def to_json(self) -> str:
        return json.dumps({"name": self.name, "digest": self.digest, "files": list(self.files)})


def file_digest(path: Path) -> str:
    h = hashlib.sha256()
    with Path(path).open("rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _module_file(module: str) -> Path | None:
    """``cubic_serve_b200.a.b`` -> its source file inside the package, or None for anything outside it."""
    parts = module.split(".")
    if parts[0] != PACKAGE_NAME:
        return None
    base = PACKAGE_ROOT.joinpath(*parts[1:])
    if base.is_dir() and (base / "__init__.py").exists():
        return base / "__init__.py"
    f = base.with_suffix(".py")
    return f if f.exists() else None


def _module_name(path: Path) -> str:
    rel = path.relative_to(PACKAGE_ROOT).with_suffix("")
    parts = [PACKAGE_NAME, *rel.parts]
    if parts[-1] == "__init__":
        parts.pop()
    return ".".join(parts)


def imported_package_modules(path: Path) -> set[Path]:
    """Package files named by the import statements of ``path`` (absolute and relative forms, any nesting level:
    imports inside functions count, they run too)."""
    tree = ast.parse(path.read_text(), str(path))
    me = _module_name(path).split(".")
    is_pkg = path.name == "__init__.py"
    found: set[Path] = set()

    def add(module: str) -> bool:
        f = _module_file(module)
        if f is not None:
            found.add(f)
        return f is not None

    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                add(a.name)
        elif isinstance(node, ast.ImportFrom):
            if node.level:
                base = me if is_pkg else me[:-1]
                base = base[:len(base) - (node.level - 1)] if node.level > 1 else base
                module = ".".join(base + ([node.module] if node.module else []))
            else:
                module = node.module or ""
            if not module.startswith(PACKAGE_NAME):
                continue
            add(module)
            for a in node.names:            # ``from .ops import kernels`` names a module, ``from .x import f`` does not
                add(f"{module}.{a.name}")
    found.discard(path)
    return found


def source_closure(entry_modules: tuple[str, ...]) -> list[Path]:
    """Every package file reachable from the entry modules through import statements, sorted."""
    todo = []
    for m in entry_modules:
        f = _module_file(m)
        if f is None:
            raise ValueError(f"{m!r} is not a module of {PACKAGE_NAME}")
        todo.append(f)
    seen: set[Path] = set()
    while todo:
        f = todo.pop()
        if f in seen:
            continue
        seen.add(f)
        # a package's __init__ runs before any of its modules
        for parent in f.relative_to(PACKAGE_ROOT).parents:
            init = PACKAGE_ROOT / parent / "__init__.py"
            if init.exists() and init not in seen:
                todo.append(init)
        todo.extend(imported_package_modules(f) - seen)
    return sorted(seen)


def native_sources() -> list[Path]:
    csrc = PACKAGE_ROOT / "csrc"
    return sorted(p for pat in ("*.cu", "*.cuh", "*.h") for p in csrc.glob(pat))


@lru_cache(maxsize=16)
def identity(name: str = "serving", entry_modules: tuple[str, ...] = (f"{PACKAGE_NAME}.runtime.serving",),
             native: bool = True, extras: tuple[str, ...] = ()) -> ImplementationIdentity:
    """Identity of the implementation reached from ``entry_modules`` (default: the serving path).  ``extras`` are
    further strings that take part in the digest (build flags, a format version)."""
    files = source_closure(entry_modules) + (native_sources() if native else [])
    pairs = tuple((str(p.relative_to(PACKAGE_ROOT)), file_digest(p)) for p in files)
    if native:
        from ..ops import native as native_lib
        extras = extras + tuple(native_lib.NVCC_FLAGS)
    h = hashlib.sha256()
    for rel, d in pairs:
        h.update(rel.encode() + b"\0" + d.encode() + b"\n")
    for e in extras:
        h.update(b"extra\0" + e.encode() + b"\n")
    return ImplementationIdentity(name, h.hexdigest(), pairs)


def digest_of(obj) -> str:
    """Digest of a JSON-serialisable description (a model configuration, runner options, a device description)."""
    return hashlib.sha256(json.dumps(obj, sort_keys=True, default=str).encode()).hexdigest()
