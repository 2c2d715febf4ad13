"""GGUF / GGML block formats: Q4_K native decode (to the 4-bit affine GEMM operand) and a library-backed path.

The reference admits ``Q8_0, Q6_K, IQ3_S, IQ4_NL, IQ4_XS`` plus plain float tensors
(``quantization/extensions/ggml/checkpoint.py:17`` there) and decodes original GGML blocks inside its kernels
(``ggml/decode.cuh:41-81``).  Here:

* **Q4_K** (super-blocks of 256 with 6-bit sub-block scales and mins; ``block_q4_K`` of ggml-common.h: fp16 ``d``,
  fp16 ``dmin``, 12 bytes of packed 6-bit scales/mins, 128 bytes of nibbles) is decoded to 4-bit codes plus a
  per-32-column ``(scale, offset)`` pair, exactly what the affine 4-bit GEMM path streams -- so Q4_K weights stay
  4-bit in HBM and are expanded inside the GEMM main loop;
* the other admitted block types are expanded to bf16 at load time with the ``gguf`` package's reference
  dequantizers (the runtime then treats them as plain bf16 weights).
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import wq_pack

QK_K = 256
Q4K_BLOCK_BYTES = 144
ADMITTED = ("F32", "F16", "BF16", "Q8_0", "Q4_K", "Q6_K", "IQ3_S", "IQ4_NL", "IQ4_XS")


class GGUFFormatError(ValueError):
    pass


def _scale_min_k4(scales: np.ndarray):
    """12 packed bytes per block -> (sc[8], m[8]) 6-bit values (llama.cpp ``get_scale_min_k4``)."""
    q = scales.astype(np.int32)
    sc = np.empty(q.shape[:-1] + (8,), dtype=np.int32)
    mn = np.empty_like(sc)
    for j in range(4):
        sc[..., j] = q[..., j] & 63
        mn[..., j] = q[..., j + 4] & 63
    for j in range(4, 8):
        sc[..., j] = (q[..., j + 4] & 0xF) | ((q[..., j - 4] >> 6) << 4)
        mn[..., j] = (q[..., j + 4] >> 4) | ((q[..., j] >> 6) << 4)
    return sc, mn


def q4k_decode(raw: np.ndarray):
    """``uint8 [rows, blocks * 144]`` -> codes ``uint8 [rows, K]``, scale and offset ``float32 [rows, K / 32]``.

    ``w = code * scale + offset`` with ``scale = d * sc`` and ``offset = -dmin * m`` per 32-column sub-block.
    """
    rows = raw.shape[0]
    blk = raw.reshape(rows, -1, Q4K_BLOCK_BYTES)
    d = blk[..., 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    dmin = blk[..., 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    sc, mn = _scale_min_k4(blk[..., 4:16])
    qs = blk[..., 16:144].reshape(rows, -1, 4, 32)                       # 4 groups of 32 bytes = 64 values each
    lo, hi = qs & 0xF, qs >> 4
    codes = np.stack([lo, hi], axis=3).reshape(rows, -1)                 # sub-block 2i = low nibbles, 2i+1 = high
    scale = (d[..., None] * sc).reshape(rows, -1).astype(np.float32)
    offset = (-dmin[..., None] * mn).reshape(rows, -1).astype(np.float32)
    return codes.astype(np.uint8), scale, offset


def q4k_dense(raw: np.ndarray) -> np.ndarray:
    codes, scale, offset = q4k_decode(raw)
    return codes.astype(np.float32) * np.repeat(scale, 32, 1) + np.repeat(offset, 32, 1)


def q4k_quantize(w: np.ndarray) -> np.ndarray:
    """Simple Q4_K encoder for tests / random checkpoints (min-max per sub-block, 6-bit scales and mins)."""
    rows, k = w.shape
    if k % QK_K:
        raise GGUFFormatError("Q4_K rows must be a multiple of 256 columns")
    b = w.astype(np.float32).reshape(rows, k // QK_K, 8, 32)
    mn = np.minimum(b.min(-1), 0.0)
    mx = b.max(-1)
    sub_scale = np.maximum((mx - mn) / 15.0, 1e-12)
    sub_min = -mn
    d = np.maximum(sub_scale.max(-1) / 63.0, 1e-12).astype(np.float16)
    dmin = np.maximum(sub_min.max(-1) / 63.0, 1e-12).astype(np.float16)
    sc = np.clip(np.rint(sub_scale / d.astype(np.float32)[..., None]), 0, 63).astype(np.int32)
    m6 = np.clip(np.rint(sub_min / dmin.astype(np.float32)[..., None]), 0, 63).astype(np.int32)
    eff_s = np.maximum(d.astype(np.float32)[..., None] * sc, 1e-12)
    eff_m = dmin.astype(np.float32)[..., None] * m6
    q = np.clip(np.rint((b + eff_m[..., None]) / eff_s[..., None]), 0, 15).astype(np.uint8)
    out = np.zeros((rows, k // QK_K, Q4K_BLOCK_BYTES), dtype=np.uint8)
    out[..., 0:2] = d[..., None].view(np.uint8)
    out[..., 2:4] = dmin[..., None].view(np.uint8)
    s = out[..., 4:16]
    for j in range(4):
        s[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        s[..., j + 4] = (m6[..., j] & 63) | ((m6[..., j + 4] >> 4) << 6)
        s[..., j + 8] = (sc[..., j + 4] & 0xF) | ((m6[..., j + 4] & 0xF) << 4)
    qg = q.reshape(rows, k // QK_K, 4, 2, 32)
    out[..., 16:144] = (qg[..., 0, :] | (qg[..., 1, :] << 4)).reshape(rows, k // QK_K, 128)
    return out.reshape(rows, -1)


def to_packed_weight(type_name: str, raw: np.ndarray, shape: tuple[int, int]) -> wq_pack.PackedWeight:
    """One GGUF tensor (logical ``[N, K]``) -> GEMM operand."""
    n, k = shape
    if type_name not in ADMITTED:
        raise GGUFFormatError(f"GGML type {type_name} is not admitted (admitted: {', '.join(ADMITTED)})")
    if type_name == "Q4_K":
        codes, scale, offset = q4k_decode(np.ascontiguousarray(raw).reshape(n, -1))
        return wq_pack.pack_affine4(torch.from_numpy(codes), torch.from_numpy(scale), torch.from_numpy(offset), 32)
    return wq_pack.pack_bf16(torch.from_numpy(dense(type_name, raw, shape)))


def dense(type_name: str, raw: np.ndarray, shape: tuple[int, int]) -> np.ndarray:
    n, k = shape
    if type_name == "F32":
        return np.asarray(raw, dtype=np.float32).reshape(n, k)
    if type_name == "F16":
        return np.asarray(raw).view(np.float16).astype(np.float32).reshape(n, k)
    if type_name == "BF16":
        u = np.asarray(raw).view(np.uint16).astype(np.uint32) << 16
        return u.view(np.float32).reshape(n, k)
    if type_name == "Q4_K":
        return q4k_dense(np.ascontiguousarray(raw).reshape(n, -1))
    import gguf
    qtype = getattr(gguf.GGMLQuantizationType, type_name)
    return gguf.quants.dequantize(np.ascontiguousarray(raw).reshape(n, -1), qtype).astype(np.float32).reshape(n, k)
