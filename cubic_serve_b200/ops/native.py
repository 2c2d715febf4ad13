"""Build and load the sm_100a native library (``libcubic_b200.so``).

The kernels are plain CUDA C++ with ``extern "C"`` launchers; Python reaches
them through ``ctypes`` with raw device pointers and the current CUDA stream,
the same split the reference uses (driver-API launches, no CPython extension:
``ops/cuda/native.py:101-255`` there).  The library is compiled ahead of time
into the package directory so that it ships with a source snapshot.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import subprocess
import threading
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_PATH = Path(__file__).resolve().parent.parent / "libcubic_b200.so"
MANIFEST_PATH = LIB_PATH.with_suffix(".manifest.json")
SOURCES = ("wq_gemm.cu", "elementwise.cu", "kv_cache.cu", "paged_attn.cu", "sampling.cu", "tp_comm.cu", "moe.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
)

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class NativeLibraryError(RuntimeError):
    """The native library is missing, failed to build, or a launch failed."""


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()] + sorted(
        p for p in CSRC.glob("*.cu") if p.name not in SOURCES
    )


def _sha(path: Path) -> str:
    h = hashlib.sha256()
    with path.open("rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _source_digests() -> dict[str, str]:
    deps = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    return {p.name: _sha(p) for p in deps}


def read_manifest() -> dict | None:
    """The bundle manifest written beside the library by ``build``: source digests, flags, compiler, library digest."""
    try:
        return json.loads(MANIFEST_PATH.read_text())
    except (OSError, ValueError):
        return None


def verify_bundle(check_library: bool = True) -> list[str]:
    """Problems of the built bundle against the sources in the tree (empty = the library is what the sources build):
    missing library or manifest, a source whose content differs from the one compiled, other flags, a library file
    that is not the one the manifest describes."""
    if not LIB_PATH.exists():
        return [f"{LIB_PATH.name} is missing"]
    man = read_manifest()
    if man is None:
        return [f"{MANIFEST_PATH.name} is missing or unreadable"]
    problems = []
    now = _source_digests()
    built = man.get("sources", {})
    for name in sorted(set(now) | set(built)):
        if name not in built:
            problems.append(f"{name} was added after the build")
        elif name not in now:
            problems.append(f"{name} was compiled but is gone")
        elif now[name] != built[name]:
            problems.append(f"{name} changed after the build")
    if list(man.get("flags", [])) != list(NVCC_FLAGS):
        problems.append("the compiler flags changed after the build")
    if check_library and man.get("library_sha256") != _sha(LIB_PATH):
        problems.append(f"{LIB_PATH.name} is not the file the manifest describes")
    return problems


def needs_build() -> bool:
    """Content-addressed staleness check: file times do not survive a copy of the tree to another machine, the
    digests in the manifest do.  A library without a manifest falls back to comparing file times."""
    if not LIB_PATH.exists():
        return True
    if read_manifest() is None:
        built = LIB_PATH.stat().st_mtime
        deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
        return any(p.stat().st_mtime > built for p in deps)
    return bool(verify_bundle(check_library=False))


def _nvcc_version() -> str:
    try:
        out = subprocess.run([_nvcc(), "--version"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True).stdout
        return out.strip().splitlines()[-1] if out.strip() else ""
    except OSError:
        return ""


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libcubic_b200.so``."""
    if not force and not needs_build():
        return LIB_PATH
    objdir = CSRC / "build"
    objdir.mkdir(exist_ok=True)
    procs = []
    objs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        objs.append(str(obj))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise NativeLibraryError(f"nvcc failed for {src.name}:\n{out}")
        if verbose and out:
            print(out)
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [_nvcc(), "-shared", "-o", str(tmp), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise NativeLibraryError(f"link failed:\n{res.stdout}")
    os.replace(tmp, LIB_PATH)
    manifest = {"library": LIB_PATH.name, "library_sha256": _sha(LIB_PATH), "arch": "sm_100a", "flags": list(NVCC_FLAGS),
                "nvcc": _nvcc_version(), "sources": _source_digests()}
    MANIFEST_PATH.write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    return LIB_PATH


def lib() -> ctypes.CDLL:
    """Return the loaded library; build it first if a compiler is available and it is stale."""
    global _lib
    with _lock:
        if _lib is None:
            if needs_build():
                try:
                    build()
                except (OSError, NativeLibraryError) as exc:
                    if not LIB_PATH.exists():
                        raise NativeLibraryError(
                            f"{LIB_PATH.name} is missing and could not be built: {exc}"
                        ) from exc
            _lib = ctypes.CDLL(str(LIB_PATH))
            _declare(_lib)
            if os.environ.get("CUBIC_SERVE_PDL", "1") == "0":
                _lib.cb_set_pdl(0)       # programmatic dependent launch of the kernels off (csrc/launch.cuh)
        return _lib


def _declare(l: ctypes.CDLL) -> None:
    vp, i, f, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    l.cb_wq_gemm.argtypes = [i, vp, i, vp, vp, vp, i, vp, f, i, i, i, i, i, vp, vp, vp, vp]
    l.cb_wq_gemm.restype = i
    l.cb_wq_gemm_workspace_bytes.argtypes = [i, i, i]
    l.cb_wq_gemm_workspace_bytes.restype = ll
    l.cb_rmsnorm.argtypes = [vp, vp, vp, vp, vp, i, i, f, i, vp]
    l.cb_rmsnorm.restype = i
    l.cb_rmsnorm_rows.argtypes = [vp, vp, vp, vp, i, i, f, i, vp]
    l.cb_rmsnorm_rows.restype = i
    l.cb_set_pdl.argtypes = [i]
    l.cb_set_pdl.restype = None
    l.cb_pdl_enabled.argtypes = []
    l.cb_pdl_enabled.restype = i
    l.cb_swiglu.argtypes = [vp, vp, i, i, vp]
    l.cb_swiglu.restype = i
    l.cb_embedding.argtypes = [vp, vp, vp, i, i, i, i, vp]
    l.cb_embedding.restype = i
    l.cb_kv_blob_bytes.argtypes = [i, i, i]
    l.cb_kv_blob_bytes.restype = i
    l.cb_rope_kv_write.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, f, i, i, i, vp]
    l.cb_hadamard.argtypes = [vp, i, vp, i, i, i, vp]
    l.cb_hadamard.restype = i
    l.cb_rope_kv_write.restype = i
    l.cb_rope_kv_write_axes.argtypes = [vp, vp, vp, vp, vp, vp, i, i, vp, vp, vp, vp, vp, i, i, i, i, i, f, i, i, i, vp]
    l.cb_rope_kv_write_axes.restype = i
    l.cb_copy_pages.argtypes = [vp, vp, vp, i, ll, vp]
    l.cb_copy_pages.restype = i
    l.cb_paged_attn_partial_floats.argtypes = [i, i, i]
    l.cb_paged_attn_partial_floats.restype = ll
    l.cb_paged_attn.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, i, vp, vp, vp, vp]
    l.cb_paged_attn.restype = i
    l.cb_sample.argtypes = [vp, i, vp, i, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
    l.cb_sample.restype = i
    l.cb_verify_greedy.argtypes = [vp, vp, vp, i, vp, vp, vp, i, vp]
    l.cb_verify_greedy.restype = i
    l.cb_sample_candidates.argtypes = [vp, i, vp, i, vp, vp, vp, vp, i, i, i, vp]
    l.cb_sample_candidates.restype = i
    l.cb_sample_merge.argtypes = [vp, vp, i, ll, i, vp, vp, vp, vp, vp, vp, vp, vp]
    l.cb_sample_merge.restype = i
    l.cb_tp_exchange.argtypes = [vp, vp]
    l.cb_tp_exchange.restype = i
    l.cb_wq_gemm_tp.argtypes = [i, vp, i, vp, vp, vp, i, vp, f, i, i, i, i, i, vp, vp, vp, vp, vp]
    l.cb_wq_gemm_tp.restype = i
    l.cb_wq_gemm_sk.argtypes = [i, vp, i, vp, vp, vp, i, vp, f, i, i, i, i, i, vp, ll, vp, vp, vp, vp]
    l.cb_wq_gemm_sk.restype = i
    l.cb_wq_gemm_act.argtypes = [i, vp, i, vp, vp, vp, i, f, i, i, i, i, i, i, i, vp, ll, vp, vp, vp, vp]
    l.cb_wq_gemm_act.restype = i
    l.cb_tp_reduce_norm.argtypes = [vp, vp]
    l.cb_tp_reduce_norm.restype = i
    l.cb_tp_wait.argtypes = [vp, vp, ctypes.c_uint, i, vp, vp]
    l.cb_tp_wait.restype = i
    l.cb_tp_argmax_merge.argtypes = [vp, vp]
    l.cb_tp_argmax_merge.restype = i
    l.cb_moe_route.argtypes = [vp, i, vp, i, i, i, i, i, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    l.cb_moe_route.restype = i
    l.cb_moe_combine.argtypes = [vp, vp, vp, i, i, i, vp, vp, vp]
    l.cb_moe_combine.restype = i
    l.cb_wq_gemm_grouped_mode.argtypes = [i]
    l.cb_wq_gemm_grouped_mode.restype = None
    l.cb_reasoning_budget.argtypes = [vp, vp, vp, vp, vp, i, i, ctypes.POINTER(ctypes.c_int), i, vp]
    l.cb_reasoning_budget.restype = i
    l.cb_gdn_conv.argtypes = [vp, i, vp, i, vp, vp, vp, vp, i, i, vp]
    l.cb_gdn_conv.restype = i
    l.cb_gdn_delta.argtypes = [vp, vp, vp]
    l.cb_gdn_delta.restype = i
    l.cb_sigmoid_gate.argtypes = [vp, i, vp, i, vp, i, i, i, vp]
    l.cb_sigmoid_gate.restype = i
    l.cb_wq_gemm_pair_mode.argtypes = [i]
    l.cb_wq_gemm_pair_mode.restype = None
    l.cb_wq_gemm_cluster_splitk.argtypes = [i]
    l.cb_wq_gemm_cluster_splitk.restype = None
    l.cb_wq_gemm_resident_clusters.argtypes = [i, i]
    l.cb_wq_gemm_resident_clusters.restype = i
    l.cb_wq_gemm_resident_pairs.argtypes = [i]
    l.cb_wq_gemm_resident_pairs.restype = i
    l.cb_moe_permute.argtypes = [vp, vp, i, i, i, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp]
    l.cb_moe_permute.restype = i
    l.cb_ep_dispatch.argtypes = [vp, vp]
    l.cb_ep_dispatch.restype = i
    l.cb_ep_unpack.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, vp, vp, vp, vp, vp]
    l.cb_ep_unpack.restype = i
    l.cb_ep_combine_push.argtypes = [vp, vp]
    l.cb_ep_combine_push.restype = i
    l.cb_ep_finish.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, vp, vp]
    l.cb_ep_finish.restype = i
    l.cb_wq_gemm_grouped.argtypes = [i, vp, i, vp, vp, vp, i, f, i, i, i, i, vp, i, i, i, ll, ll, vp, vp]
    l.cb_wq_gemm_grouped.restype = i
    l.cb_wq_gemm_grouped_act.argtypes = l.cb_wq_gemm_grouped.argtypes
    l.cb_wq_gemm_grouped_act.restype = i
    l.cb_verify_sampled.argtypes = [vp, vp, vp, vp, vp, vp, i, vp, vp, vp, vp, vp, vp, vp, vp, i, vp]
    l.cb_verify_sampled.restype = i
    l.cb_canary_fill.argtypes = [vp, ll, ctypes.c_uint, vp]
    l.cb_canary_fill.restype = i
    l.cb_canary_check.argtypes = [vp, ll, ctypes.c_uint, i, vp, vp]
    l.cb_canary_check.restype = i
    # fp8 (e4m3 x e4m3) tensor path: activation quantizers and the GEMM entries
    l.cb_fp8_quantize_rows.argtypes = [vp, i, vp, i, vp, i, i, vp]
    l.cb_fp8_quantize_rows.restype = i
    l.cb_fp8_quantize_rows_phase.argtypes = [vp, i, vp, i, vp, i, i, i, vp]
    l.cb_fp8_quantize_rows_phase.restype = i
    l.cb_rmsnorm_fp8.argtypes = [vp, vp, vp, vp, vp, i, vp, i, i, f, i, vp]
    l.cb_rmsnorm_fp8.restype = i
    l.cb_swiglu_fp8.argtypes = [vp, vp, i, vp, i, i, vp]
    l.cb_swiglu_fp8.restype = i
    l.cb_wq_gemm_fp8.argtypes = [vp, i, vp, vp, vp, i, vp, i, vp, i, i, i, i, i, i, i, vp, ll, vp, vp, vp, vp]
    l.cb_wq_gemm_fp8.restype = i
    l.cb_wq_gemm_fp8_grouped.argtypes = [vp, i, vp, vp, vp, i, vp, i, i, i, i, vp, i, i, i, i, vp, vp]
    l.cb_wq_gemm_fp8_grouped.restype = i


class TpLinkStruct(ctypes.Structure):
    """Mirror of ``CbTpLink`` in ``csrc/wq_gemm.cu``."""
    _fields_ = [("mode", ctypes.c_int), ("rank", ctypes.c_int), ("size", ctypes.c_int),
                ("rows_per_rank", ctypes.c_int), ("recv", ctypes.c_void_p * 8), ("rs_flag", ctypes.c_void_p * 8),
                ("ag_flag", ctypes.c_void_p), ("ag_state", ctypes.c_void_p), ("ag_expected", ctypes.c_uint)]


class GdnSegmentsStruct(ctypes.Structure):
    """Mirror of ``CbGdnSegments`` in ``csrc/gdn.cu``."""
    _fields_ = [("row0", ctypes.c_void_p), ("count", ctypes.c_void_p), ("slot", ctypes.c_void_p),
                ("pos0", ctypes.c_void_p), ("num", ctypes.c_int)]


class GdnDeltaStruct(ctypes.Structure):
    """Mirror of ``CbGdnDelta`` in ``csrc/gdn.cu``."""
    _fields_ = [("qkv", ctypes.c_void_p), ("ldqkv", ctypes.c_int), ("z", ctypes.c_void_p), ("ldz", ctypes.c_int),
                ("ba", ctypes.c_void_p), ("ldba", ctypes.c_int), ("a_log", ctypes.c_void_p),
                ("dt_bias", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("state", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("ldo", ctypes.c_int), ("Hk", ctypes.c_int), ("Hv", ctypes.c_int),
                ("eps_norm", ctypes.c_float), ("eps_l2", ctypes.c_float), ("commit", ctypes.c_int)]


class ReduceNormStruct(ctypes.Structure):
    """Mirror of ``CbReduceNorm`` in ``csrc/tp_comm.cu``."""
    _fields_ = [("recv", ctypes.c_void_p), ("rs_flag", ctypes.c_void_p), ("rs_state", ctypes.c_void_p),
                ("rs_expected", ctypes.c_uint), ("h", ctypes.c_void_p), ("norm_w", ctypes.c_void_p),
                ("x_peer", ctypes.c_void_p * 8), ("ag_flag_peer", ctypes.c_void_p * 8), ("status", ctypes.c_void_p),
                ("rank", ctypes.c_int), ("size", ctypes.c_int), ("rows_per_rank", ctypes.c_int), ("H", ctypes.c_int),
                ("M", ctypes.c_int), ("eps", ctypes.c_float), ("zero_centered", ctypes.c_int),
                ("local_only", ctypes.c_int), ("recv_mc", ctypes.c_void_p), ("x_mc", ctypes.c_void_p)]


class ExchangeStruct(ctypes.Structure):
    """Mirror of ``CbExchange`` in ``csrc/tp_comm.cu``."""
    _fields_ = [("local", ctypes.c_void_p), ("area_peer", ctypes.c_void_p * 8), ("flag_peer", ctypes.c_void_p * 8),
                ("my_flag", ctypes.c_void_p), ("my_state", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("rank", ctypes.c_int), ("size", ctypes.c_int), ("segments", ctypes.c_int), ("seg_words", ctypes.c_int),
                ("seg_stride", ctypes.c_int), ("area_words", ctypes.c_int)]


class EpDispatchStruct(ctypes.Structure):
    """Mirror of ``CbEpDispatch`` in ``csrc/ep_comm.cu``."""
    _fields_ = [("logits", ctypes.c_void_p), ("x", ctypes.c_void_p), ("ld", ctypes.c_int), ("cnt", ctypes.c_int),
                ("E", ctypes.c_int), ("k", ctypes.c_int), ("H", ctypes.c_int), ("normalize", ctypes.c_int),
                ("experts_per_rank", ctypes.c_int), ("rank", ctypes.c_int), ("size", ctypes.c_int),
                ("cap", ctypes.c_int), ("xin_peer", ctypes.c_void_p * 8), ("ids_peer", ctypes.c_void_p * 8),
                ("w_peer", ctypes.c_void_p * 8), ("cnt_peer", ctypes.c_void_p * 8), ("flag_peer", ctypes.c_void_p * 8),
                ("local_cnt", ctypes.c_void_p), ("sent", ctypes.c_void_p), ("done", ctypes.c_void_p)]


class EpCombineStruct(ctypes.Structure):
    """Mirror of ``CbEpCombine`` in ``csrc/ep_comm.cu``."""
    _fields_ = [("y", ctypes.c_void_p), ("route_pos", ctypes.c_void_p), ("topk_w", ctypes.c_void_p),
                ("cnt_in", ctypes.c_void_p), ("size", ctypes.c_int), ("cap", ctypes.c_int), ("k", ctypes.c_int),
                ("H", ctypes.c_int), ("rank", ctypes.c_int), ("yin_peer", ctypes.c_void_p * 8),
                ("flag_peer", ctypes.c_void_p * 8), ("done", ctypes.c_void_p)]


class ArgmaxMergeStruct(ctypes.Structure):
    """Mirror of ``CbArgmaxMerge`` in ``csrc/tp_comm.cu``."""
    _fields_ = [("local_val", ctypes.c_void_p), ("local_id", ctypes.c_void_p), ("slot_val", ctypes.c_void_p * 8),
                ("slot_id", ctypes.c_void_p * 8), ("flag_peer", ctypes.c_void_p * 8), ("my_val", ctypes.c_void_p),
                ("my_id", ctypes.c_void_p), ("my_flag", ctypes.c_void_p), ("my_state", ctypes.c_void_p),
                ("out_id", ctypes.c_void_p), ("status", ctypes.c_void_p), ("rank", ctypes.c_int),
                ("size", ctypes.c_int), ("rows", ctypes.c_int), ("rows_max", ctypes.c_int)]


def check(code: int, what: str) -> None:
    if code != 0:
        raise NativeLibraryError(f"{what} failed with code {code}")
