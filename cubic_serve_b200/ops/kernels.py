"""Tensor-level wrappers over the native sm_100a kernels.

Every wrapper takes CUDA tensors, launches on the current stream and raises
``NativeLibraryError`` on a non-zero launch code.  There is deliberately no
PyTorch fallback on the GPU path: a missing library is an error.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import native
from .wq_pack import FMT_BF16, FMT_CUBIC4, FMT_FP8, FMT_FP8_BLOCK, PackedWeight

PAGE_TOKENS = 16


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Workspace:
    """Per-device scratch shared by split-K GEMMs and split-KV attention.

    ``counters`` must stay zero between launches (the kernels restore it);
    ``status`` collects device-side error codes and is polled by ``check_status``.
    """

    def __init__(self, device: torch.device, gemm_bytes: int = 64 << 20, attn_floats: int = 4 << 20,
                 counters: int = 1 << 16) -> None:
        self.device = device
        self.gemm = torch.empty(gemm_bytes, dtype=torch.uint8, device=device)
        self.attn = torch.empty(max(attn_floats, 1), dtype=torch.float32, device=device)
        self.gemm_counters = torch.zeros(counters, dtype=torch.int32, device=device)
        self.attn_counters = torch.zeros(counters, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._retired: list[torch.Tensor] = []
        # e4m3 activation operand of the fp8 GEMMs (codes and per-token scales), grown on demand
        self.fp8_q = torch.empty(0, dtype=torch.uint8, device=device)
        self.fp8_scale = torch.empty(0, dtype=torch.float32, device=device)

    def ensure_fp8(self, rows: int, k: int) -> None:
        if rows * k > self.fp8_q.numel():
            self._retired.append(self.fp8_q)          # captured graphs may hold the old address: retire, never free
            self.fp8_q = torch.empty(max(rows * k, 256 * 16384), dtype=torch.uint8, device=self.device)
        if rows > self.fp8_scale.numel():
            self._retired.append(self.fp8_scale)
            self.fp8_scale = torch.empty(max(rows, 8192), dtype=torch.float32, device=self.device)

    def ensure_attn(self, floats: int) -> None:
        if floats > self.attn.numel():
            # captured graphs may hold the old address: retire, never free
            self._retired.append(self.attn)
            self.attn = torch.empty(floats, dtype=torch.float32, device=self.device)

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise native.NativeLibraryError(f"device kernel reported status {code} (bounded wait ran out)")


_workspaces: dict[int, Workspace] = {}


def workspace(device: torch.device) -> Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = _workspaces[idx] = Workspace(torch.device("cuda", idx))
    return ws


def sm_count(device: torch.device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


_CLUSTER_CAPACITY_GUESS = {2: 72, 3: 40, 4: 32, 5: 24, 6: 16, 7: 16, 8: 16}      # 8 GPCs of 16-18 usable SMs
_cluster_capacity: dict[tuple[int, int], int] = {}


def resident_clusters(fmt: int, size: int) -> int:
    """Clusters of ``size`` K splits of the per-tile GEMM that fit on the device at once (its CTAs share a GPC)."""
    key = (fmt, size)
    if key not in _cluster_capacity:
        n = 0
        if torch.cuda.is_available():
            n = native.lib().cb_wq_gemm_resident_clusters(fmt, size)
        _cluster_capacity[key] = n if n > 0 else _CLUSTER_CAPACITY_GUESS.get(size, 0)
    return _cluster_capacity[key]


# Measured launch plans (``ops/autotune.py``): "fmt:m:n:k:act" -> (use the persistent kernel, split-K factor of the
# per-tile kernel).  Consulted before the rules below when the caller forces nothing; empty unless a plan was installed.
TUNED_PLANS: dict[str, tuple[bool, int]] = {}


def choose_splits(m: int, n: int, k: int, sms: int = 148, fmt: int = FMT_CUBIC4, cluster: bool = True) -> int:
    """Split-K factor: fill the SMs when the (n-tile x m-tile) grid is small.

    The splits of a tile form a thread-block cluster and sum their partial tiles through distributed shared
    memory; that only works when all clusters of the launch are resident at once, so the largest factor whose
    clusters fit is taken (48 tiles: 2, because only ~40 clusters of 3 fit on 8 GPCs).  ``cluster`` False (partials
    through the workspace, the last split sums them) keeps the plain rule.  A split pays off while each CTA still
    has >= 8 k-blocks of work.
    """
    from .strategies import active
    g = active().gemm
    n_tiles = -(-n // 128)
    m_tiles = -(-m // 256)
    tiles = n_tiles * m_tiles
    k_blocks = k // 64
    if tiles * 2 > sms or k_blocks < 2 * g.split_k_min_blocks:
        return 1
    base = max(1, min(sms // tiles, k_blocks // g.split_k_min_blocks, g.split_k_max))
    if cluster:
        for s in range(min(base, 8), 1, -1):
            if tiles <= resident_clusters(fmt, s):
                return s
    return base


def use_stream_k(m: int, n: int, fmt: int, sms: int = 148, k: int = 4096) -> bool:
    """Which GEMM kernel serves a shape when the caller does not say.

    Measured on a B200 inside CUDA graphs (cubic4, K = 4096): the persistent stream-K kernel wins when there are
    more weight tiles than SMs, because it removes the second, partly empty wave: N = 24576 runs 69 -> 45 us at
    16-64 batch rows, 70 -> 54 us at 128 and 80 -> 69 us at 256 (the fix-up of a streamed tile is deferred to the
    end of its CTA and done by 640 threads), and the bf16 lm_head is 5 % faster.  With fewer tiles than SMs its
    fixed costs (start-up, fp32 partial tiles summed by the last CTA) make it 10-25 % slower than one CTA per
    (tile, split).  Above 256 rows (prefill chunks, several row tiles) the persistent kernel runs on CTA pairs
    (cta_group::2, half an activation tile per SM): 4096 x 24576 x 4096 takes 700 us against 778 us, 4096 x 4096 x
    12288 342 against 425; it is chosen when every pair gets enough k-blocks to amortise its start-up
    (512 x 6144 x 4096, 41 k-blocks per pair, is 48 us against 41 us on the per-tile kernel).
    The thresholds live in the operator configuration (``ops/strategies.py``).
    """
    from .strategies import active
    g = active().gemm
    n_tiles = -(-n // 128)
    m_tiles = -(-m // 256)
    if m > max(g.stream_k_max_rows, 256) and fmt != FMT_BF16:
        pairs = sms // 2
        return (g.cta_pairs and n_tiles % 2 == 0 and pairs > 0
                and (n_tiles // 2) * m_tiles * (k // 64) >= g.pair_min_blocks * pairs)
    if n_tiles * m_tiles <= g.stream_k_min_tile_ratio * sms:
        return False
    return m <= g.stream_k_max_rows or (fmt == FMT_BF16 and g.stream_k_bf16)


@dataclass
class Fp8Act:
    """Activations quantized per token for the fp8 GEMMs: e4m3 bytes ``q [M, K]`` and fp32 scales ``scale [M]``."""
    q: torch.Tensor
    scale: torch.Tensor

    @property
    def shape(self):
        return self.q.shape

    @property
    def device(self):
        return self.q.device


def fp8_quantize(x: torch.Tensor, ws: Workspace | None = None, out: Fp8Act | None = None, scale_max=None) -> Fp8Act:
    """Dynamic per-token e4m3 quantization of ``x [M, K]`` (bf16): ``scale = max(amax / 448, 1 / (448 * 512))``,
    ``q = e4m3(x / scale)`` (the reference's rule, ``quantization/extensions/fp8/reference.py:47-59`` there).  Without
    ``out`` the result lives in the workspace's fp8 buffers until the next quantization.

    ``scale_max``: a callable that reduces the fp32 scale vector in place with MAX over the tensor-parallel ranks; given
    for operands whose K dimension is sharded, so that every rank quantizes with the scale of the whole row."""
    m, k = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    if out is None:
        ws = ws or workspace(x.device)
        ws.ensure_fp8(m, k)
        out = Fp8Act(ws.fp8_q[:m * k].view(m, k), ws.fp8_scale[:m])
    if scale_max is not None:
        for phase in (1, 2):
            code = native.lib().cb_fp8_quantize_rows_phase(x.data_ptr(), x.stride(0), out.q.data_ptr(), out.q.stride(0),
                                                           out.scale.data_ptr(), m, k, phase, _stream())
            native.check(code, "cb_fp8_quantize_rows_phase")
            if phase == 1:
                scale_max(out.scale)
        return out
    code = native.lib().cb_fp8_quantize_rows(x.data_ptr(), x.stride(0), out.q.data_ptr(), out.q.stride(0),
                                             out.scale.data_ptr(), m, k, _stream())
    native.check(code, "cb_fp8_quantize_rows")
    return out


def rmsnorm_fp8(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                zero_centered: bool = False, ws: Workspace | None = None) -> Fp8Act:
    """RMSNorm whose output leaves as e4m3 + per-token scales (the bf16-rounded norm output is what gets quantized,
    so the result equals ``fp8_quantize(rmsnorm(...))``)."""
    m, h = x.shape
    ws = ws or workspace(x.device)
    ws.ensure_fp8(m, h)
    out = Fp8Act(ws.fp8_q[:m * h].view(m, h), ws.fp8_scale[:m])
    code = native.lib().cb_rmsnorm_fp8(x.data_ptr(), _ptr(residual), _ptr(residual), weight.data_ptr(), out.q.data_ptr(), h,
                                       out.scale.data_ptr(), m, h, float(eps), int(zero_centered), _stream())
    native.check(code, "cb_rmsnorm_fp8")
    return out


def swiglu_fp8(gate_up: torch.Tensor, ws: Workspace | None = None) -> Fp8Act:
    """SwiGLU of ``[gate | up]`` whose output leaves as e4m3 + per-token scales."""
    m, two_i = gate_up.shape
    i = two_i // 2
    ws = ws or workspace(gate_up.device)
    ws.ensure_fp8(m, i)
    out = Fp8Act(ws.fp8_q[:m * i].view(m, i), ws.fp8_scale[:m])
    code = native.lib().cb_swiglu_fp8(gate_up.data_ptr(), out.q.data_ptr(), i, out.scale.data_ptr(), m, i, _stream())
    native.check(code, "cb_swiglu_fp8")
    return out


def _wq_gemm_fp8(x, w: PackedWeight, out, residual, splits, ws: Workspace, link, swiglu: bool,
                 min_units: int | None = None) -> torch.Tensor:
    """The fp8 branch of ``wq_gemm`` / ``wq_gemm_act``: quantize the activations per token unless the caller already
    holds them as ``Fp8Act``, then e4m3 x e4m3 on the tensor cores with both scales applied in the epilogue."""
    if link is not None and (link.mode & 1) and not isinstance(x, Fp8Act):
        raise ValueError("an fp8 GEMM cannot wait for gathered rows: its quantizer would read them before they arrive")
    a = x if isinstance(x, Fp8Act) else fp8_quantize(x, ws)
    m, k = a.q.shape
    push = link is not None and (link.mode & 2)
    l = native.lib()
    # the persistent kernel (stream-K at decode sizes with more tiles than SMs, CTA pairs above 256 rows) serves row
    # scales; block scales and explicit split factors stay on the per-tile kernel
    # (measured: the fp8 loop is bound by the L2 -> SM operand feed in both kernels; CTA pairs pay off for deep K at
    # prefill sizes -- 4096 x 4096 x 12288: 153 us against 176 us -- and nowhere else, stream-K at decode sizes ties)
    stream_k = (splits is None and w.fmt == FMT_FP8 and link is None
                and (min_units is not None or (m >= 2048 and k >= 8192 and (-(-w.n // 128)) % 2 == 0)))
    if stream_k and min_units is None:
        from .strategies import active
        min_units = active().gemm.stream_k_min_units
    min_units = min_units or 0
    if not stream_k:
        if splits is None:
            splits = choose_splits(m, w.n, k, fmt=w.fmt)
        if splits > 1 and l.cb_wq_gemm_workspace_bytes(m, w.n, splits) > ws.gemm.numel():
            splits = 1
    code = l.cb_wq_gemm_fp8(a.q.data_ptr(), a.q.stride(0), a.scale.data_ptr(), w.codes.data_ptr(), w.meta.data_ptr(),
                            int(w.fmt == FMT_FP8_BLOCK), None if push else out.data_ptr(), w.n if push else out.stride(0),
                            _ptr(residual), m, w.n, k, int(splits or 1), int(swiglu), int(stream_k), int(min_units),
                            ws.gemm.data_ptr(), ws.gemm.numel(), ws.gemm_counters.data_ptr(), ws.status.data_ptr(),
                            _stream(), None if link is None else ctypes.byref(link))
    native.check(code, "cb_wq_gemm_fp8")
    return out


def wq_gemm(x: torch.Tensor, w: PackedWeight, out: torch.Tensor | None = None,
            residual: torch.Tensor | None = None, splits: int | None = None,
            ws: Workspace | None = None, link=None, min_units: int | None = None) -> torch.Tensor:
    """``out[M, N] = x[M, K] @ W[N, K]^T * alpha (+ residual)`` with W in packed form.

    Two kernels: one CTA per (weight tile, K split) (``csrc/wq_gemm.cu``) and the persistent stream-K kernel
    (``csrc/wq_gemm_sk.cu``).  With neither ``splits`` nor ``min_units`` given the faster one for the shape is
    used (``use_stream_k``).  ``splits`` forces the first with that split-K factor; ``min_units`` forces the
    second (0 = its own schedule, > 0 = the smallest run of k-blocks a CTA is dealt).
    """
    assert isinstance(x, Fp8Act) or (x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1)
    m, k = x.shape
    assert k == w.k, (k, w.k)
    push = link is not None and (link.mode & 2)
    if out is None and not push:
        out = torch.empty((m, w.n), dtype=torch.bfloat16, device=x.device)
    assert push or (out.stride(1) == 1 and out.shape == (m, w.n))
    if residual is not None:
        assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
    ws = ws or workspace(x.device)
    if w.fmt in (FMT_FP8, FMT_FP8_BLOCK):
        return _wq_gemm_fp8(x, w, out, residual, splits, ws, link, False, min_units)
    l = native.lib()
    if splits is None and min_units is None and link is None and TUNED_PLANS:
        tuned = TUNED_PLANS.get(f"{w.fmt}:{m}:{w.n}:{k}:0")
        if tuned is not None:
            splits, min_units = (None, 0) if tuned[0] else (tuned[1], None)
    if splits is None and min_units is None and use_stream_k(m, w.n, w.fmt, sm_count(x.device), k):
        from .strategies import active
        min_units = active().gemm.stream_k_min_units
    if splits is None and min_units is not None:
        code = l.cb_wq_gemm_sk(w.fmt, x.data_ptr(), x.stride(0), w.codes.data_ptr(), _ptr(w.meta),
                               None if push else out.data_ptr(), w.n if push else out.stride(0), _ptr(residual),
                               float(w.alpha), m, w.n, k, w.group_k, int(min_units), ws.gemm.data_ptr(),
                               ws.gemm.numel(), ws.gemm_counters.data_ptr(), ws.status.data_ptr(), _stream(),
                               None if link is None else ctypes.byref(link))
        native.check(code, "cb_wq_gemm_sk")
        return out
    if splits is None:
        splits = choose_splits(m, w.n, k, fmt=w.fmt)
    if splits > 1:
        need = l.cb_wq_gemm_workspace_bytes(m, w.n, splits)
        if need > ws.gemm.numel():
            splits = 1
    code = l.cb_wq_gemm_tp(w.fmt, x.data_ptr(), x.stride(0), w.codes.data_ptr(), _ptr(w.meta),
                           None if push else out.data_ptr(), w.n if push else out.stride(0), _ptr(residual),
                           float(w.alpha), m, w.n, k, w.group_k, splits, ws.gemm.data_ptr(),
                           ws.gemm_counters.data_ptr(), ws.status.data_ptr(), _stream(),
                           None if link is None else ctypes.byref(link))
    native.check(code, "cb_wq_gemm")
    return out


def wq_gemm_act(x: torch.Tensor, w: PackedWeight, out: torch.Tensor | None = None, splits: int | None = None,
                ws: Workspace | None = None, min_units: int | None = None, link=None) -> torch.Tensor:
    """Gate/up projection with SwiGLU in the GEMM epilogue: ``out[M, N/2] = silu(x Wg^T) * (x Wu^T)``.

    ``w`` is the ``[gate; up]`` matrix in the interleaved row order (``wq_pack.swiglu_interleave``).  The projection
    ``link`` (gather-wait only) as in ``wq_gemm``.  The projection is rounded to bf16 before the activation, as when ``wq_gemm`` and ``swiglu`` run as two kernels, so both paths
    give the same values; the ``[M, N]`` intermediate is never written.  Kernel choice as in ``wq_gemm``.
    """
    assert w.act_interleaved, "weight rows are not in the SwiGLU order"
    assert isinstance(x, Fp8Act) or (x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1)
    m, k = x.shape
    assert k == w.k, (k, w.k)
    if out is None:
        out = torch.empty((m, w.n // 2), dtype=torch.bfloat16, device=x.device)
    assert out.stride(1) == 1 and out.shape == (m, w.n // 2)
    ws = ws or workspace(x.device)
    if w.fmt in (FMT_FP8, FMT_FP8_BLOCK):
        return _wq_gemm_fp8(x, w, out, None, splits, ws, link, True, min_units)
    l = native.lib()
    if splits is None and min_units is None and link is None and TUNED_PLANS:
        tuned = TUNED_PLANS.get(f"{w.fmt}:{m}:{w.n}:{k}:1")
        if tuned is not None:
            splits, min_units = (None, 0) if tuned[0] else (tuned[1], None)
    stream_k = splits is None and (min_units is not None or use_stream_k(m, w.n, w.fmt, sm_count(x.device), k))
    if stream_k and min_units is None:
        from .strategies import active
        min_units = active().gemm.stream_k_min_units
    if not stream_k:
        if splits is None:
            splits = choose_splits(m, w.n, k, fmt=w.fmt)
        if splits > 1 and l.cb_wq_gemm_workspace_bytes(m, w.n, splits) > ws.gemm.numel():
            splits = 1
    code = l.cb_wq_gemm_act(w.fmt, x.data_ptr(), x.stride(0), w.codes.data_ptr(), _ptr(w.meta), out.data_ptr(),
                            out.stride(0), float(w.alpha), m, w.n, k, w.group_k, int(stream_k), int(splits or 1),
                            int(min_units or 0), ws.gemm.data_ptr(), ws.gemm.numel(), ws.gemm_counters.data_ptr(),
                            ws.status.data_ptr(), _stream(), None if link is None else ctypes.byref(link))
    native.check(code, "cb_wq_gemm_act")
    return out


def gate_up_act(x: torch.Tensor, w: PackedWeight, gu: torch.Tensor, act: torch.Tensor, ws: Workspace | None = None,
                link=None) -> int:
    """``act = swiglu(x @ W^T)`` for a ``[gate; up]`` projection: one launch when the rows of ``w`` are interleaved
    for the fused epilogue, else the GEMM into ``gu`` followed by the activation kernel.  Returns the launch count."""
    if w.act_interleaved:
        wq_gemm_act(x, w, out=act, ws=ws, link=link)
        return 1
    wq_gemm(x, w, out=gu, ws=ws, link=link)
    swiglu(gu, out=act)
    return 2


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor | None = None,
            residual: torch.Tensor | None = None, zero_centered: bool = False) -> torch.Tensor:
    """RMSNorm; with ``residual`` the sum ``x + residual`` is written back into ``residual`` first."""
    rows, h = x.shape
    if out is None:
        out = torch.empty_like(x)
    code = native.lib().cb_rmsnorm(x.data_ptr(), _ptr(residual), _ptr(residual), weight.data_ptr(), out.data_ptr(),
                                   rows, h, float(eps), int(zero_centered), _stream())
    native.check(code, "cb_rmsnorm")
    return out


def rmsnorm_rows(x: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor | None = None,
                 zero_centered: bool = False) -> torch.Tensor:
    """``out[i] = rmsnorm(x[rows[i]])`` (``rows`` int64): the final norm over the rows whose logits are wanted, with the
    row gather done by the kernel's own loads."""
    assert rows.dtype == torch.int64 and x.stride(1) == 1 and x.stride(0) == x.shape[1]
    n, h = rows.numel(), x.shape[1]
    if out is None:
        out = torch.empty((n, h), dtype=x.dtype, device=x.device)
    code = native.lib().cb_rmsnorm_rows(x.data_ptr(), rows.data_ptr(), weight.data_ptr(), out.data_ptr(), n, h,
                                        float(eps), int(zero_centered), _stream())
    native.check(code, "cb_rmsnorm_rows")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    rows, two_i = gate_up.shape
    i = two_i // 2
    if out is None:
        out = torch.empty((rows, i), dtype=gate_up.dtype, device=gate_up.device)
    native.check(native.lib().cb_swiglu(gate_up.data_ptr(), out.data_ptr(), rows, i, _stream()), "cb_swiglu")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None, vocab_start: int = 0) -> torch.Tensor:
    t = ids.numel()
    h = table.shape[1]
    if out is None:
        out = torch.empty((t, h), dtype=table.dtype, device=table.device)
    code = native.lib().cb_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), t, h, vocab_start,
                                     table.shape[0], _stream())
    native.check(code, "cb_embedding")
    return out


def kv_blob_bytes(head_dim: int, k_bits: int, v_bits: int) -> int:
    d = head_dim
    scale = PAGE_TOKENS * (d // 32) * 4
    return PAGE_TOKENS * d * k_bits // 8 + PAGE_TOKENS * d * v_bits // 8 + 2 * scale


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                  slots: torch.Tensor, inv_freq: torch.Tensor, hq: int, hkv: int, head_dim: int,
                  k_bits: int, v_bits: int, q_norm: torch.Tensor | None = None,
                  k_norm: torch.Tensor | None = None, eps: float = 1e-6, rotary_dim: int | None = None,
                  rotate: bool = False, positions_hw: tuple[torch.Tensor, torch.Tensor] | None = None,
                  mrope_section: tuple[int, int, int] | None = None, qkv_bias: torch.Tensor | None = None) -> None:
    """``rotate``: every q / k / v head vector is Walsh-Hadamard transformed (after RoPE) before it is written, which
    spreads outlier channels over the 32-channel quantization groups; ``q . k`` is unchanged and the attention
    output is transformed back with ``hadamard`` (reference: ``ops/cuda/cache_rotation_native.cu:12``).
    ``positions_hw``: int32 row- and column-axis positions ``[T]`` each; with them ``positions`` is the temporal axis
    and ``mrope_section`` says how many frequency slots follow each axis (interleaved layout; reference:
    ``ops/cuda/position/qwen_mrope.py:25``).  ``qkv_bias``: bf16 ``[(hq + 2 hkv) head_dim]`` added to the rows as they
    are read (projection biases of the Qwen2 family)."""
    t = qkv.shape[0]
    rot = head_dim if rotary_dim is None else rotary_dim
    if qkv_bias is not None:
        assert qkv_bias.dtype == torch.bfloat16 and qkv_bias.numel() == (hq + 2 * hkv) * head_dim and qkv_bias.is_contiguous()
    if positions_hw is None and qkv_bias is None:
        code = native.lib().cb_rope_kv_write(qkv.data_ptr(), q_out.data_ptr(), cache.data_ptr(), positions.data_ptr(),
                                             slots.data_ptr(), _ptr(q_norm), _ptr(k_norm), inv_freq.data_ptr(), t, hq,
                                             hkv, head_dim, rot, float(eps), k_bits, v_bits, int(rotate), _stream())
        native.check(code, "cb_rope_kv_write")
        return
    ph = pw = None
    sec = (0, 0, 0)
    if positions_hw is not None:
        if mrope_section is None or sum(mrope_section) != rot // 2:
            raise ValueError("three-axis positions need the section counts of the rotary width")
        ph, pw = positions_hw
        sec = mrope_section
        assert ph.dtype == pw.dtype == torch.int32 and ph.numel() >= t and pw.numel() >= t
    code = native.lib().cb_rope_kv_write_axes(qkv.data_ptr(), q_out.data_ptr(), cache.data_ptr(), positions.data_ptr(),
                                              _ptr(ph), _ptr(pw), int(sec[1]), int(sec[2]), _ptr(qkv_bias),
                                              slots.data_ptr(), _ptr(q_norm), _ptr(k_norm), inv_freq.data_ptr(), t, hq,
                                              hkv, head_dim, rot, float(eps), k_bits, v_bits, int(rotate), _stream())
    native.check(code, "cb_rope_kv_write_axes")


def hadamard(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform of every consecutive 128-vector of the rows of ``x`` (bf16; its own inverse)."""
    rows, cols = x.shape
    assert cols % 128 == 0 and x.stride(1) == 1 and x.dtype == torch.bfloat16
    out = x if out is None else out
    native.check(native.lib().cb_hadamard(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), cols // 128, rows,
                                          _stream()), "cb_hadamard")
    return out


def copy_pages(cache: torch.Tensor, src: torch.Tensor, dst: torch.Tensor) -> None:
    page_bytes = cache.stride(0) * cache.element_size()
    native.check(native.lib().cb_copy_pages(cache.data_ptr(), src.data_ptr(), dst.data_ptr(), src.numel(),
                                            page_bytes, _stream()), "cb_copy_pages")


def copy_rows(t: torch.Tensor, src: torch.Tensor, dst: torch.Tensor) -> None:
    """``t[dst[i]] = t[src[i]]`` for whole leading-axis rows of a contiguous tensor (bit-preserving; the page-copy
    kernel with a row as the page).  A row must be a multiple of 16 bytes."""
    if not t.is_contiguous() or (t.stride(0) * t.element_size()) % 16:
        raise ValueError("copy_rows: rows must be contiguous multiples of 16 bytes")
    copy_pages(t, src, dst)


def paged_attention(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor,
                    rb_req: torch.Tensor, rb_qstart: torch.Tensor, rb_qcount: torch.Tensor, rb_ctx: torch.Tensor,
                    hq: int, hkv: int, head_dim: int, k_bits: int, v_bits: int, scale: float | None = None,
                    splits: int = 1, ws: Workspace | None = None) -> torch.Tensor:
    """Attention of row blocks over the paged quantized cache (see ``csrc/paged_attn.cu``)."""
    rbs = rb_req.numel()
    ws = ws or workspace(q.device)
    l = native.lib()
    if splits > 1:
        ws.ensure_attn(l.cb_paged_attn_partial_floats(rbs, hkv, splits))
        assert rbs * hkv <= ws.attn_counters.numel()
    code = l.cb_paged_attn(q.data_ptr(), out.data_ptr(), cache.data_ptr(), page_table.data_ptr(), rb_req.data_ptr(),
                           rb_qstart.data_ptr(), rb_qcount.data_ptr(), rb_ctx.data_ptr(), rbs, hq, hkv, head_dim,
                           page_table.shape[1], k_bits, v_bits,
                           float(scale if scale is not None else 1.0 / math.sqrt(head_dim)), splits,
                           ws.attn.data_ptr(), ws.attn_counters.data_ptr(), ws.status.data_ptr(), _stream())
    native.check(code, "cb_paged_attn")
    return out


def sample(logits: torch.Tensor, out_ids: torch.Tensor, temperature: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, top_k: torch.Tensor | None = None,
           seeds: torch.Tensor | None = None, counters: torch.Tensor | None = None,
           mask: torch.Tensor | None = None, out_logprob: torch.Tensor | None = None,
           vocab: int | None = None, out_value: torch.Tensor | None = None, id_offset: int = 0) -> torch.Tensor:
    rows = logits.shape[0]
    code = native.lib().cb_sample(logits.data_ptr(), logits.stride(0), _ptr(mask),
                                  0 if mask is None else mask.stride(0), _ptr(temperature), _ptr(top_p), _ptr(top_k),
                                  _ptr(seeds), _ptr(counters), out_ids.data_ptr(), _ptr(out_logprob),
                                  _ptr(out_value), int(id_offset), rows, vocab or logits.shape[1], _stream())
    native.check(code, "cb_sample")
    return out_ids


SAMPLE_CANDIDATES = 20      # candidate slots per row of vocab-sharded sampling (= the largest top-k)


def sample_candidates(logits: torch.Tensor, cand_val: torch.Tensor, cand_id: torch.Tensor,
                      temperature: torch.Tensor | None = None, top_k: torch.Tensor | None = None,
                      mask: torch.Tensor | None = None, vocab: int | None = None, id_offset: int = 0) -> None:
    """Rank-local half of vocab-sharded sampling: the best (logit, global id) pairs of every row, ``[rows, 20]``."""
    rows = logits.shape[0]
    code = native.lib().cb_sample_candidates(logits.data_ptr(), logits.stride(0), _ptr(mask),
                                             0 if mask is None else mask.stride(0), _ptr(temperature), _ptr(top_k),
                                             cand_val.data_ptr(), cand_id.data_ptr(), int(id_offset), rows,
                                             vocab or logits.shape[1], _stream())
    native.check(code, "cb_sample_candidates")


def sample_merge(cand_val: torch.Tensor, cand_id: torch.Tensor, sources: int, source_stride: int, rows: int,
                 out_ids: torch.Tensor, temperature: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
                 top_k: torch.Tensor | None = None, seeds: torch.Tensor | None = None,
                 counters: torch.Tensor | None = None, out_logprob: torch.Tensor | None = None) -> torch.Tensor:
    """Draw every row's token from the union of ``sources`` candidate sets (same result on every rank)."""
    code = native.lib().cb_sample_merge(cand_val.data_ptr(), cand_id.data_ptr(), sources, source_stride, rows,
                                        _ptr(temperature), _ptr(top_p), _ptr(top_k), _ptr(seeds), _ptr(counters),
                                        out_ids.data_ptr(), _ptr(out_logprob), _stream())
    native.check(code, "cb_sample_merge")
    return out_ids


def verify_greedy(target_ids: torch.Tensor, draft_ids: torch.Tensor, depth: torch.Tensor, max_depth: int,
                  accepted: torch.Tensor, bonus: torch.Tensor, forced_reject_at: torch.Tensor | None = None) -> None:
    code = native.lib().cb_verify_greedy(target_ids.data_ptr(), draft_ids.data_ptr(), depth.data_ptr(), max_depth,
                                         _ptr(forced_reject_at), accepted.data_ptr(), bonus.data_ptr(),
                                         depth.numel(), _stream())
    native.check(code, "cb_verify_greedy")


def verify_sampled(q_val: torch.Tensor, q_id: torch.Tensor, p_val: torch.Tensor, p_id: torch.Tensor,
                   draft_ids: torch.Tensor, depth: torch.Tensor, max_depth: int, temperature: torch.Tensor,
                   top_p: torch.Tensor, top_k: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
                   accepted: torch.Tensor, bonus: torch.Tensor, emitted: torch.Tensor) -> None:
    """p / q rejection sampling of a speculative round over sparse candidate distributions (``[R, D, 20]`` draft
    candidates, ``[R, D + 1, 20]`` target candidates as written by ``sample_candidates``); ``emitted [R, D + 1]``
    receives every request's accepted drafts followed by its next token.  See ``csrc/sampling.cu``."""
    code = native.lib().cb_verify_sampled(q_val.data_ptr(), q_id.data_ptr(), p_val.data_ptr(), p_id.data_ptr(),
                                          draft_ids.data_ptr(), depth.data_ptr(), int(max_depth), temperature.data_ptr(),
                                          top_p.data_ptr(), top_k.data_ptr(), seeds.data_ptr(), counters.data_ptr(),
                                          accepted.data_ptr(), bonus.data_ptr(), emitted.data_ptr(), depth.numel(),
                                          _stream())
    native.check(code, "cb_verify_sampled")


# ------------------------------------------------------------------ mixture of experts
class MoeScratch:
    """Fixed-address routing buffers for up to ``max_tokens`` tokens (graph-capturable)."""

    def __init__(self, max_tokens: int, top_k: int, hidden: int, inter2: int, local_experts: int, mb: int, device) -> None:
        routes = max_tokens * top_k
        self.mb = mb
        self.max_items = -(-routes // mb) + local_experts
        i32 = dict(dtype=torch.int32, device=device)
        self.topk_ids = torch.empty(max_tokens, top_k, **i32)
        self.topk_w = torch.empty(max_tokens, top_k, dtype=torch.float32, device=device)
        self.counts = torch.zeros(local_experts, **i32)
        self.offsets = torch.zeros(local_experts, **i32)
        self.cursors = torch.zeros(local_experts, **i32)
        self.total = torch.zeros(1, **i32)
        self.tiles = torch.zeros(1 + 3 * self.max_items, **i32)
        self.route_pos = torch.empty(max_tokens, top_k, **i32)
        bf = dict(dtype=torch.bfloat16, device=device)
        # + mb rows of slack: a work item's TMA tile may run past the last route (those rows are never stored)
        self.xs = torch.zeros(routes + mb, hidden, **bf)
        self.gu = torch.zeros(routes + mb, inter2, **bf)
        self.act = torch.zeros(routes + mb, inter2 // 2, **bf)
        self.y = torch.zeros(routes + mb, hidden, **bf)


def moe_route(router_logits: torch.Tensor, x: torch.Tensor, top_k: int, sc: MoeScratch, normalize: bool = True,
              expert_lo: int = 0, expert_count: int | None = None) -> None:
    t, e = router_logits.shape
    cnt = e if expert_count is None else expert_count
    code = native.lib().cb_moe_route(router_logits.data_ptr(), router_logits.stride(0), x.data_ptr(), t, e, top_k,
                                     x.shape[1], int(normalize), expert_lo, cnt, sc.mb, sc.topk_ids.data_ptr(),
                                     sc.topk_w.data_ptr(), sc.counts.data_ptr(), sc.offsets.data_ptr(),
                                     sc.cursors.data_ptr(), sc.total.data_ptr(), sc.tiles.data_ptr(),
                                     sc.route_pos.data_ptr(), sc.xs.data_ptr(), _stream())
    native.check(code, "cb_moe_route")


def wq_gemm_grouped(x: torch.Tensor, w: PackedWeight, out: torch.Tensor, rows: int, sc: MoeScratch,
                    code_stride: int, meta_stride: int, ws: Workspace | None = None, swiglu: bool = False) -> torch.Tensor:
    """Per-expert ``out[rows of e] = x[rows of e] @ W_e^T`` over the work list in ``sc.tiles``; ``w`` stacks the experts.

    ``swiglu``: every expert's ``[gate; up]`` rows are interleaved and ``out`` (``N / 2`` columns) gets the activation.
    """
    ws = ws or workspace(x.device)
    assert swiglu == w.act_interleaved
    if w.fmt in (FMT_FP8, FMT_FP8_BLOCK):
        # the routed rows (plus the slack rows a work item's tile may touch) are quantized per token, then one grouped
        # launch over the stacked e4m3 experts
        a = fp8_quantize(x[:min(x.shape[0], rows + sc.mb)], ws)
        code = native.lib().cb_wq_gemm_fp8_grouped(a.q.data_ptr(), a.q.stride(0), a.scale.data_ptr(), w.codes.data_ptr(),
                                                   w.meta.data_ptr(), int(w.fmt == FMT_FP8_BLOCK), out.data_ptr(),
                                                   out.stride(0), rows, w.n, w.k,
                                                   sc.tiles.data_ptr(), sc.max_items, sc.mb, w.codes.shape[0], int(swiglu),
                                                   ws.status.data_ptr(), _stream())
        native.check(code, "cb_wq_gemm_fp8_grouped")
        return out
    entry = native.lib().cb_wq_gemm_grouped_act if swiglu else native.lib().cb_wq_gemm_grouped
    code = entry(w.fmt, x.data_ptr(), x.stride(0), w.codes.data_ptr(), _ptr(w.meta),
                                           out.data_ptr(), out.stride(0), float(w.alpha), rows, w.n, w.k, w.group_k,
                                           sc.tiles.data_ptr(), sc.max_items, sc.mb, w.codes.shape[0], code_stride, meta_stride,
                                           ws.status.data_ptr(), _stream())
    native.check(code, "cb_wq_gemm_grouped")
    return out


def moe_combine(y: torch.Tensor, sc: MoeScratch, tokens: int, out: torch.Tensor,
                residual: torch.Tensor | None = None) -> torch.Tensor:
    code = native.lib().cb_moe_combine(y.data_ptr(), sc.route_pos.data_ptr(), sc.topk_w.data_ptr(), tokens,
                                       sc.topk_ids.shape[1], y.shape[1], _ptr(residual), out.data_ptr(), _stream())
    native.check(code, "cb_moe_combine")
    return out


# ------------------------------------------------------------------ gated delta net (hybrid family)
@dataclass
class GdnSegments:
    """A step's token rows grouped by request: rows ``[row0, row0 + count)`` of state slot ``slot``, the first at
    absolute position ``pos0`` (0 = the request starts here, from zero state).  int32 device tensors of length >= num."""
    row0: torch.Tensor
    count: torch.Tensor
    slot: torch.Tensor
    pos0: torch.Tensor
    num: int

    def struct(self) -> "native.GdnSegmentsStruct":
        s = native.GdnSegmentsStruct()
        s.row0, s.count, s.slot, s.pos0 = self.row0.data_ptr(), self.count.data_ptr(), self.slot.data_ptr(), self.pos0.data_ptr()
        s.num = int(self.num)
        return s


def gdn_conv(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, seg: GdnSegments, out: torch.Tensor,
             bias: torch.Tensor | None = None, commit: bool = True) -> torch.Tensor:
    """Depthwise causal conv1d (kernel 4) + SiLU over ``x[T, C]`` per request segment; ``state[slots, 3, C]`` holds
    every request's last three inputs and is updated unless ``commit`` is False (speculative review pass).
    ``w``: fp32 ``[C, 4]`` (tap 3 multiplies the current input)."""
    c = w.shape[0]
    assert w.dtype == torch.float32 and w.shape[1] == 4 and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and out.stride(1) == 1 and x.shape[1] >= c
    assert state.dtype == torch.bfloat16 and state.shape[1:] == (3, c) and state.is_contiguous()
    st = seg.struct()
    code = native.lib().cb_gdn_conv(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), w.data_ptr(), _ptr(bias),
                                    state.data_ptr(), ctypes.byref(st), c, int(commit), _stream())
    native.check(code, "cb_gdn_conv")
    return out


def gdn_delta(qkv: torch.Tensor, z: torch.Tensor, ba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
              norm_w: torch.Tensor, state: torch.Tensor, seg: GdnSegments, out: torch.Tensor, hk: int, hv: int,
              eps_norm: float = 1e-6, eps_l2: float = 1e-6, commit: bool = True) -> torch.Tensor:
    """Gated delta rule + gated RMSNorm per (segment, value head); ``state[slots, Hv, 128, 128]`` fp32 is updated
    unless ``commit`` is False (speculative review pass: the state is read, the outputs are written, nothing else).

    ``qkv[T, 2 Hk 128 + Hv 128]`` (after ``gdn_conv``), ``z[T, Hv 128]``, ``ba[T, 2 Hv]`` = ``[b | a]``.
    """
    assert state.dtype == torch.float32 and state.shape[1:] == (hv, 128, 128) and state.is_contiguous()
    for t in (a_log, dt_bias, norm_w):
        assert t.dtype == torch.float32 and t.is_contiguous()
    d = native.GdnDeltaStruct()
    d.qkv, d.ldqkv, d.z, d.ldz, d.ba, d.ldba = qkv.data_ptr(), qkv.stride(0), z.data_ptr(), z.stride(0), ba.data_ptr(), ba.stride(0)
    d.a_log, d.dt_bias, d.norm_w, d.state = a_log.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr(), state.data_ptr()
    d.out, d.ldo, d.Hk, d.Hv, d.eps_norm, d.eps_l2 = out.data_ptr(), out.stride(0), hk, hv, eps_norm, eps_l2
    d.commit = int(commit)
    st = seg.struct()
    native.check(native.lib().cb_gdn_delta(ctypes.byref(d), ctypes.byref(st), _stream()), "cb_gdn_delta")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out = x * sigmoid(gate)`` (bf16; the output gate of the hybrid family's full-attention layers)."""
    rows, cols = x.shape
    out = x if out is None else out
    code = native.lib().cb_sigmoid_gate(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), out.data_ptr(),
                                        out.stride(0), rows, cols, _stream())
    native.check(code, "cb_sigmoid_gate")
    return out


# ------------------------------------------------------------------ thinking-token budgets
class ReasoningBudget:
    """Device state of the thinking-token budgets: one counter per request slot (see ``csrc/sampling.cu``)."""

    def __init__(self, slots: int, end_token_id: int, forced_tokens: list[int], device) -> None:
        if not 1 <= len(forced_tokens) <= 4 or end_token_id not in forced_tokens:
            raise ValueError("the forced end sequence has 1 to 4 tokens and contains the closing token")
        self.end_token_id = int(end_token_id)
        self.forced = [int(t) for t in forced_tokens]
        self._seq = (ctypes.c_int * len(self.forced))(*self.forced)
        self.left = torch.full((slots,), -1, dtype=torch.int32, device=device)
        self.fpos = torch.zeros(slots, dtype=torch.int32, device=device)

    def apply(self, ids: torch.Tensor, row_slot: torch.Tensor, init: torch.Tensor, rows: int) -> None:
        """Run the state machine on the step's ``rows`` sampled ids in place."""
        code = native.lib().cb_reasoning_budget(ids.data_ptr(), row_slot.data_ptr(), init.data_ptr(), self.left.data_ptr(),
                                                self.fpos.data_ptr(), rows, self.end_token_id, self._seq,
                                                len(self.forced), _stream())
        native.check(code, "cb_reasoning_budget")
