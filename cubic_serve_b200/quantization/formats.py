"""Checkpoint weight formats other than CubicQuant: decode rules, offline quantizers, GEMM packing.

On-disk layouts follow the reference's format table (``quantization/extensions/*/checkpoint.py`` and
``layout.py`` there); logical matrices are ``[N, K]`` (out, in):

* INT (compressed-tensors ``pack-quantized``): ``weight_packed int32 [N, words(K)]`` offset-binary codes,
  ``floor(32/b)`` codes per word (LSB first), ``weight_scale [N, K/G]``, optional ``weight_zero_point int32
  [words(N), K/G]`` packed the same way along N; ``w = (q - z) * s`` (symmetric: ``z = 2^(b-1)``).
* AWQ GEMM: ``qweight int32 [K, N/8]`` with nibble order ``[0, 4, 1, 5, 2, 6, 3, 7]``, ``qzeros int32 [K/G, N/8]``,
  ``scales fp16 [K/G, N]``; ``w = (q - z) * s``.
* FP8: ``weight float8_e4m3fn [N, K]`` with ``weight_scale fp32 [N, 1]`` (per channel) or
  ``weight_scale_inv fp32 [N/128, K/128]`` (128 x 128 blocks); ``w = q * s``.
* NVFP4: ``weight_packed uint8 [N, K/2]`` (low nibble first, e2m1 with bit 3 = sign), ``weight_scale
  float8_e4m3fn [N, K/16]``, ``weight_global_scale fp32 [1]`` (compressed-tensors: divide) or ``weight_scale_2``
  (ModelOpt: multiply).

``to_packed_weight`` maps each format to what the tcgen05 GEMM consumes (4-bit formats natively, the rest as
bf16 after a load-time decode).
"""
from __future__ import annotations

import math

import torch

from ..ops import wq_pack

AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)
NVFP4_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


class FormatError(ValueError):
    pass


# ----------------------------------------------------------------------- INT
def int_unpack(packed: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    """``int32 [R, words]`` -> unsigned codes ``[R, count]`` (legacy layout: floor(32/bits) codes per word)."""
    if packed.dtype != torch.int32:
        raise FormatError("INT payload must be int32 words")
    per = 32 // bits
    shifts = torch.arange(per, device=packed.device, dtype=torch.int32) * bits
    vals = (packed.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return vals.reshape(packed.shape[0], -1)[:, :count]


def int_pack(codes: torch.Tensor, bits: int) -> torch.Tensor:
    per = 32 // bits
    r, c = codes.shape
    pad = (-c) % per
    v = torch.nn.functional.pad(codes.to(torch.int64), (0, pad)).reshape(r, -1, per)
    shifts = torch.arange(per, device=codes.device, dtype=torch.int64) * bits
    words = (v << shifts).sum(-1)
    return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)


def int_decode(payload: dict, bits: int, group: int, shape: tuple[int, int]):
    """Return unsigned codes ``[N, K]``, fp32 scale and zero point ``[N, K/G]`` (``group <= 0`` = per channel)."""
    n, k = shape
    g = group if group and group > 0 else k
    q = int_unpack(payload["weight_packed"], bits, k)
    if q.shape[0] != n:
        raise FormatError("INT packed rows differ from N")
    scale = payload["weight_scale"].float().reshape(n, -1)
    groups = math.ceil(k / g)
    if scale.shape[1] != groups:
        raise FormatError("INT scale shape does not match the group size")
    if "weight_zero_point" in payload:
        zp = int_unpack(payload["weight_zero_point"].t().contiguous(), bits, n).t().float()
    else:
        zp = torch.full((n, groups), float(1 << (bits - 1)), device=q.device)
    return q, scale, zp


def int_dense(payload: dict, bits: int, group: int, shape: tuple[int, int]) -> torch.Tensor:
    q, s, z = int_decode(payload, bits, group, shape)
    g = group if group and group > 0 else shape[1]
    col = torch.arange(shape[1], device=q.device) // g
    return (q.float() - z[:, col]) * s[:, col]


def int_quantize(w: torch.Tensor, bits: int = 4, group: int = 128, symmetric: bool = True) -> dict:
    n, k = w.shape
    wg = w.float().reshape(n, k // group, group)
    if symmetric:
        qmax = (1 << (bits - 1)) - 1
        scale = (wg.abs().amax(-1) / qmax).clamp_min(1e-10)
        q = (torch.round(wg / scale[..., None]).clamp(-qmax - 1, qmax) + (1 << (bits - 1))).reshape(n, k)
        return {"weight_packed": int_pack(q, bits), "weight_scale": scale.half(),
                "weight_shape": torch.tensor([n, k], dtype=torch.int64)}
    lo, hi = wg.amin(-1), wg.amax(-1)
    scale = ((hi - lo) / ((1 << bits) - 1)).clamp_min(1e-10)
    zp = torch.round(-lo / scale).clamp(0, (1 << bits) - 1)
    q = torch.round(wg / scale[..., None] + zp[..., None]).clamp(0, (1 << bits) - 1).reshape(n, k)
    return {"weight_packed": int_pack(q, bits), "weight_scale": scale.half(),
            "weight_zero_point": int_pack(zp.t().contiguous(), bits).t().contiguous(),
            "weight_shape": torch.tensor([n, k], dtype=torch.int64)}


# ----------------------------------------------------------------------- AWQ
def awq_unpack(words: torch.Tensor) -> torch.Tensor:
    """``int32 [R, C/8]`` -> 4-bit values ``[R, C]`` undoing the AWQ nibble interleave."""
    shifts = torch.tensor([4 * AWQ_ORDER.index(i) for i in range(8)], device=words.device, dtype=torch.int32)
    return ((words.unsqueeze(-1) >> shifts) & 15).reshape(words.shape[0], -1)


def awq_pack(vals: torch.Tensor) -> torch.Tensor:
    r, c = vals.shape
    v = vals.to(torch.int64).reshape(r, c // 8, 8)
    shifts = torch.tensor([4 * AWQ_ORDER.index(i) for i in range(8)], device=vals.device, dtype=torch.int64)
    words = (v << shifts).sum(-1)
    return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)


def awq_decode(payload: dict, group: int):
    """Return codes ``[N, K]``, scale and zero ``[N, K/G]`` (transposed to the logical orientation)."""
    q = awq_unpack(payload["qweight"]).t().contiguous()              # [N, K]
    z = awq_unpack(payload["qzeros"]).t().contiguous().float()       # [N, K/G]
    s = payload["scales"].float().t().contiguous()                   # [N, K/G]
    if q.shape[1] != s.shape[1] * group:
        raise FormatError("AWQ group size does not match the scales")
    return q, s, z


def awq_dense(payload: dict, group: int) -> torch.Tensor:
    q, s, z = awq_decode(payload, group)
    col = torch.arange(q.shape[1], device=q.device) // group
    return (q.float() - z[:, col]) * s[:, col]


# ----------------------------------------------------------------------- FP8
def fp8_dense(payload: dict) -> torch.Tensor:
    w = payload["weight"].float()
    if "weight_scale_inv" in payload or ("weight_scale" in payload and payload["weight_scale"].dim() == 2
                                         and payload["weight_scale"].shape[1] > 1):
        s = payload.get("weight_scale_inv", payload.get("weight_scale")).float()
        n, k = w.shape
        s = s.repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
        return w * s
    return w * payload["weight_scale"].float().reshape(-1, 1)


def fp8_quantize(w: torch.Tensor, block: bool = False) -> dict:
    wf = w.float()
    if not block:
        s = (wf.abs().amax(1, keepdim=True) / 448.0).clamp_min(1e-12)
        return {"weight": (wf / s).to(torch.float8_e4m3fn), "weight_scale": s}
    n, k = wf.shape
    nb, kb = math.ceil(n / 128), math.ceil(k / 128)
    pad = torch.nn.functional.pad(wf, (0, kb * 128 - k, 0, nb * 128 - n)).reshape(nb, 128, kb, 128)
    s = (pad.abs().amax((1, 3)) / 448.0).clamp_min(1e-12)
    q = (pad / s[:, None, :, None]).reshape(nb * 128, kb * 128)[:n, :k].to(torch.float8_e4m3fn)
    return {"weight": q, "weight_scale_inv": s}


def fp8_activation_quantize(x: torch.Tensor):
    """Dynamic per-token e4m3 activation quantisation (scale floored at 1 / (448 * 512), as the reference does).  The
    divisions are carried out in double and rounded once to fp32, i.e. correctly rounded fp32 divisions (a CUDA
    tensor divided by a Python scalar is multiplied by the scalar's reciprocal, which is one ulp off now and then)."""
    xf = x.float()
    s = (xf.abs().amax(-1, keepdim=True).double() / 448.0).float().clamp_min(1.0 / (448.0 * 512.0))
    q = (xf.double() / s.double()).float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, s


# --------------------------------------------------------------------- NVFP4
def nvfp4_dense(payload: dict) -> torch.Tensor:
    packed = payload["weight_packed"] if "weight_packed" in payload else payload["weight"]
    p = packed.to(torch.int32)
    nib = torch.stack([p & 15, p >> 4], -1).reshape(p.shape[0], -1)
    lut = torch.tensor(NVFP4_LEVELS + tuple(-v for v in NVFP4_LEVELS), device=p.device)
    scale = payload["weight_scale"].float().repeat_interleave(16, 1)
    if "weight_global_scale" in payload:
        return lut[nib.long()] * scale / payload["weight_global_scale"].float().reshape(())
    return lut[nib.long()] * scale * payload["weight_scale_2"].float().reshape(())


def nvfp4_global_multiplier(payload: dict) -> float:
    if "weight_global_scale" in payload:
        return 1.0 / float(payload["weight_global_scale"].float().reshape(()))
    return float(payload["weight_scale_2"].float().reshape(()))


def nvfp4_quantize(w: torch.Tensor, amax: float | None = None) -> dict:
    """Compressed-tensors convention: block scale = e4m3(amax * g / 6), codes ties-to-even on the level grid.

    ``amax``: largest magnitude that sets the global scale (default: of ``w`` itself); a shard quantized with the
    whole matrix's value gets exactly the codes and scales the whole matrix would have in its rows / columns."""
    wf = w.float()
    n, k = wf.shape
    amax = (wf.abs().amax() if amax is None else torch.as_tensor(float(amax), device=wf.device)).clamp_min(1e-12)
    g = (448.0 * 6.0) / amax                                   # global scale (stored inverse: decode divides by it)
    blocks = wf.reshape(n, k // 16, 16)
    bs = (blocks.abs().amax(-1) * g / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    denom = (bs.float() / g).clamp_min(1e-30)
    u = (blocks.abs() / denom[..., None]).clamp(max=6.0)
    levels = torch.tensor(NVFP4_LEVELS, device=w.device)
    idx = (u[..., None] - levels).abs().argmin(-1)
    nib = (idx + torch.where(blocks < 0, 8, 0)).reshape(n, k).to(torch.int32)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).to(torch.uint8)
    return {"weight_packed": packed, "weight_scale": bs, "weight_global_scale": g.reshape(1).float()}


def nvfp4_activation_quantize(x: torch.Tensor, global_scale: float):
    """Group-16 FP4 activation quantisation used by the native block-scaled path (returns codes-as-values, scales)."""
    xf = x.float()
    b = xf.reshape(*xf.shape[:-1], xf.shape[-1] // 16, 16)
    s = (b.abs().amax(-1) * global_scale / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn).float()
    denom = (s / global_scale).clamp_min(1e-30)
    u = (b.abs() / denom[..., None]).clamp(max=6.0)
    levels = torch.tensor(NVFP4_LEVELS, device=x.device)
    q = levels[(u[..., None] - levels).abs().argmin(-1)] * b.sign()
    return q.reshape(xf.shape), s


# ------------------------------------------------------------ GEMM packing
def to_packed_weight(method: str, payload: dict, shape: tuple[int, int], bits: int = 4, group: int = 128) -> wq_pack.PackedWeight:
    """Checkpoint payload of one logical matrix -> the operand form the sm_100a GEMM streams."""
    n, k = shape
    if method == "int":
        if bits == 4 and (group <= 0 or group % 32 == 0):
            q, s, z = int_decode(payload, 4, group, shape)
            g = group if group > 0 else k
            return wq_pack.pack_affine4(q.to(torch.uint8), s, -z * s, g)
        return wq_pack.pack_bf16(int_dense(payload, bits, group, shape))
    if method == "awq":
        q, s, z = awq_decode(payload, group)
        return wq_pack.pack_affine4(q.to(torch.uint8), s, -z * s, group)
    if method == "fp8" and payload["weight"].dtype == torch.float8_e4m3fn and payload["weight_scale"].numel() == n \
            and k % 64 == 0:
        return wq_pack.pack_fp8(payload["weight"], payload["weight_scale"])
    if method in ("fp8", "fp8_block") and payload["weight"].dtype == torch.float8_e4m3fn and k % 64 == 0:
        bs = payload.get("weight_scale_inv", payload.get("weight_scale"))
        if bs is not None and bs.dim() == 2 and tuple(bs.shape) == (-(-n // 128), -(-k // 128)) and bs.shape[1] > 1:
            return wq_pack.pack_fp8_block(payload["weight"], bs)
    if method in ("fp8", "fp8_block"):
        return wq_pack.pack_bf16(fp8_dense(payload))
    if method == "nvfp4":
        packed = payload["weight_packed"] if "weight_packed" in payload else payload["weight"]
        return wq_pack.pack_nvfp4(packed, payload["weight_scale"].float(), nvfp4_global_multiplier(payload))
    if method == "none":
        return wq_pack.pack_bf16(payload["weight"])
    raise FormatError(f"unknown weight format {method!r}")
