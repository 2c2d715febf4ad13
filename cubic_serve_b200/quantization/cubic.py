"""CubicQuant codec: bitstream codes + per-group cubic level curve.

On-disk layout (must match the reference checkpoint format, see
``quantization/extensions/cubic/layout.py:22-55`` and ``reference.py:31-122``
there): ``weight_packed`` is ``uint8 [N, ceil(K*b/8)]``, a little-endian
bitstream of signed two's-complement ``b``-bit codes; the most-negative code is
reserved and decodes to zero (``b == 1``: codes are +-1).  Metadata variant A
(``float32-scale-float16-ab``) carries ``weight_scale`` fp32, ``weight_a`` and
``weight_b`` fp16, each ``[N/GO, ceil(K/GI)]``.  Variant B
(``int8-scale-int4-ab-global-fp32``) and variant C
(``e5m9-scale-curve2-tensor-fp16``) are decoded to the same (scale, a, b) triple.

Decode rule for a code ``c`` with ``t = |c| / (2^(b-1) - 1)``::

    w = sign(c) * s * t * (a + t * (b + t * (1 - a - b)))

This module is the CPU/PyTorch oracle and the offline quantizer used for
random-init benchmark checkpoints; the GPU path consumes the same payload after
``ops.wq_pack`` re-tiles it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

METADATA_A = "float32-scale-float16-ab"
METADATA_B = "int8-scale-int4-ab-global-fp32"
METADATA_C = "e5m9-scale-curve2-tensor-fp16"


class CubicFormatError(ValueError):
    pass


@dataclass(frozen=True)
class CubicScheme:
    bits: int = 4
    group_in: int = 128
    group_out: int = 1
    metadata: str = METADATA_A

    def __post_init__(self) -> None:
        if not 1 <= self.bits <= 8:
            raise CubicFormatError("Cubic supports 1..8 bit codes")
        if self.metadata not in (METADATA_A, METADATA_B, METADATA_C):
            raise CubicFormatError(f"unknown Cubic metadata format {self.metadata!r}")
        if self.group_in <= 0 or self.group_out <= 0:
            raise CubicFormatError("group sizes must be positive")


def packed_row_bytes(k: int, bits: int) -> int:
    return math.ceil(k * bits / 8)


def unpack_codes(packed: torch.Tensor, bits: int, k: int) -> torch.Tensor:
    """Bitstream -> signed int8 codes ``[N, K]`` with the reserved code mapped to 0."""
    if packed.dtype != torch.uint8 or packed.ndim != 2:
        raise CubicFormatError("weight_packed must be a 2-D uint8 tensor")
    if packed.shape[1] != packed_row_bytes(k, bits):
        raise CubicFormatError("packed row length does not match K")
    n = packed.shape[0]
    # expand to a bit matrix [N, bytes*8] (little endian inside each byte), then regroup
    bit_idx = torch.arange(8, device=packed.device, dtype=torch.int32)
    bit_mat = ((packed.to(torch.int32).unsqueeze(-1) >> bit_idx) & 1).reshape(n, -1)[:, : k * bits]
    weights = (1 << torch.arange(bits, device=packed.device, dtype=torch.int32))
    raw = (bit_mat.reshape(n, k, bits) * weights).sum(-1)
    if bits == 1:
        return (raw * 2 - 1).to(torch.int8)
    sign = 1 << (bits - 1)
    signed = torch.where(raw >= sign, raw - (1 << bits), raw)
    signed = torch.where(signed == -sign, torch.zeros_like(signed), signed)
    return signed.to(torch.int8)


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Signed codes ``[N, K]`` -> little-endian bitstream ``uint8 [N, ceil(K*b/8)]``."""
    n, k = codes.shape
    if bits == 1:
        raw = ((codes.to(torch.int32) + 1) // 2) & 1
    else:
        raw = codes.to(torch.int32) & ((1 << bits) - 1)
    bit_idx = torch.arange(bits, device=codes.device, dtype=torch.int32)
    bit_mat = ((raw.unsqueeze(-1) >> bit_idx) & 1).reshape(n, k * bits)
    pad = (-bit_mat.shape[1]) % 8
    if pad:
        bit_mat = torch.nn.functional.pad(bit_mat, (0, pad))
    weights = (1 << torch.arange(8, device=codes.device, dtype=torch.int32))
    return (bit_mat.reshape(n, -1, 8) * weights).sum(-1).to(torch.uint8)


def metadata_triple(payload: dict, scheme: CubicScheme, shape: tuple[int, int],
                    partitions: tuple[int, ...] | None = None):
    """Return fp32 ``scale`` and fp16 ``a``, ``b`` of shape ``[N/GO, ceil(K/GI)]`` for any variant."""
    n, k = shape
    go, gi = scheme.group_out, scheme.group_in
    parts = partitions or (n,)
    if sum(parts) != n or any(p <= 0 or p % go for p in parts):
        raise CubicFormatError("output partitions must close output groups")
    groups = (n // go, math.ceil(k / gi))

    def take(name: str, dtype: torch.dtype, shp: tuple[int, ...]) -> torch.Tensor:
        t = payload.get(name)
        if t is None:
            raise CubicFormatError(f"missing payload tensor {name}")
        if t.dtype != dtype or tuple(t.shape) != tuple(shp):
            raise CubicFormatError(f"{name}: expected {dtype} {shp}, got {t.dtype} {tuple(t.shape)}")
        return t

    if scheme.metadata == METADATA_A:
        return (take("weight_scale", torch.float32, groups), take("weight_a", torch.float16, groups),
                take("weight_b", torch.float16, groups))
    rows_per_part = torch.tensor([p // go for p in parts])
    if scheme.metadata == METADATA_B:
        scale = take("weight_scale", torch.int8, groups)
        ab = take("weight_ab", torch.uint8, groups).to(torch.int32)

        def glob(name: str) -> torch.Tensor:
            v = take(name, torch.float32, (len(parts),))
            if not bool(torch.isfinite(v).all()):
                raise CubicFormatError("global metadata must be finite")
            return torch.repeat_interleave(v, rows_per_part.to(v.device))[:, None]

        lo, hi = ab & 15, ab >> 4
        a4 = torch.where(lo >= 8, lo - 16, lo).float()
        b4 = torch.where(hi >= 8, hi - 16, hi).float()
        return (scale.float() * glob("weight_scale_global"),
                (1.0 + a4 * glob("weight_a_global")).half(),
                (b4 * glob("weight_b_global")).half())
    meta = take("weight_metadata", torch.uint16, groups).to(torch.int32)
    ca = take("weight_curve_a", torch.float16, (len(parts), 4))
    cb = take("weight_curve_b", torch.float16, (len(parts), 4))
    scale = ((meta & 0x3FFF) << 1).to(torch.int16).view(torch.float16).float()
    part = torch.repeat_interleave(torch.arange(len(parts)), rows_per_part)[:, None].to(meta.device)
    curve = (meta >> 14).long()
    return scale, ca[part, curve], cb[part, curve]


def level_curve(t: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return t * (a + t * (b + t * (1.0 - a - b)))


def decode(payload: dict, scheme: CubicScheme, shape: tuple[int, int],
           partitions: tuple[int, ...] | None = None) -> torch.Tensor:
    """Dequantize to fp32 ``[N, K]`` (the independent oracle)."""
    n, k = shape
    codes = unpack_codes(payload["weight_packed"], scheme.bits, k)
    if codes.shape[0] != n:
        raise CubicFormatError("packed rows differ from N")
    scale, a, b = metadata_triple(payload, scheme, shape, partitions)
    if not bool(torch.isfinite(scale).all()) or bool((scale < 0).any()):
        raise CubicFormatError("scale must be finite and non-negative")
    rows = torch.arange(n, device=codes.device) // scheme.group_out
    cols = torch.arange(k, device=codes.device) // scheme.group_in
    s = scale[rows[:, None], cols[None, :]]
    values = codes.float()
    if scheme.bits == 1:
        return values * s
    aa = a[rows[:, None], cols[None, :]].float()
    bb = b[rows[:, None], cols[None, :]].float()
    t = (values.abs().double() / ((1 << (scheme.bits - 1)) - 1)).float()
    return values.sign() * (s * level_curve(t, aa, bb))


# candidate curves tried by the offline quantizer: (a, b); (1, 0) is the uniform grid
_CURVES = ((1.0, 0.0), (0.75, 0.25), (0.5, 0.5), (0.6, 0.9), (1.25, -0.25))


def quantize(weight: torch.Tensor, scheme: CubicScheme = CubicScheme()) -> dict:
    """Quantize ``[N, K]`` to a variant-A payload (``group_out`` must be 1).

    Per group: scale = max|w|; among a few fixed level curves pick the one with
    the least squared error; codes are the nearest level with the sign of ``w``.
    """
    if scheme.metadata != METADATA_A or scheme.group_out != 1:
        raise CubicFormatError("the offline quantizer writes variant A with group_out == 1")
    if scheme.bits < 2:
        raise CubicFormatError("the offline quantizer needs >= 2 bits")
    n, k = weight.shape
    gi = scheme.group_in
    groups = math.ceil(k / gi)
    pad = groups * gi - k
    w = weight.float()
    if pad:
        w = torch.nn.functional.pad(w, (0, pad))
    wg = w.reshape(n, groups, gi)
    scale = wg.abs().amax(-1)  # [N, G]
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    u = (wg.abs() / safe[..., None]).clamp(max=1.0)
    qmax = (1 << (scheme.bits - 1)) - 1
    t = torch.arange(qmax + 1, device=w.device, dtype=torch.float32) / qmax
    best_err = None
    best_idx = None
    best_a = torch.empty_like(scale)
    best_b = torch.empty_like(scale)
    for a, b in _CURVES:
        levels = level_curve(t, torch.tensor(a), torch.tensor(b)).to(w.device)  # monotone for these curves
        idx = (u[..., None] - levels).abs().argmin(-1)
        err = ((levels[idx] - u) ** 2).sum(-1)
        if best_err is None:
            best_err, best_idx = err, idx
            best_a.fill_(a)
            best_b.fill_(b)
        else:
            better = err < best_err
            best_err = torch.where(better, err, best_err)
            best_idx = torch.where(better[..., None], idx, best_idx)
            best_a = torch.where(better, torch.full_like(best_a, a), best_a)
            best_b = torch.where(better, torch.full_like(best_b, b), best_b)
    codes = (best_idx * wg.sign().long()).reshape(n, groups * gi)[:, :k].to(torch.int8)
    return {
        "weight_packed": pack_codes(codes, scheme.bits),
        "weight_scale": scale.float().contiguous(),
        "weight_a": best_a.half().contiguous(),
        "weight_b": best_b.half().contiguous(),
    }
