"""Re-tile checkpoint payloads into the layout the tcgen05 GEMM streams.

The reference repacks every format into Marlin tiles at load time
(``quantization/common/marlin/repack.py:149-280``); this is the same step for
the sm_100a kernel in ``csrc/wq_gemm.cu``:

* ``codes``: ``uint8 [n_tiles, k_blocks, 2, 128, 16]`` -- per (128-row tile,
  64-column k-block) one contiguous 4 KiB block that a single bulk copy moves;
  32-bit word ``j`` of row ``r``, half ``h`` covers columns ``64*kb + 32*h + 8*j .. +7``.
  Affine / NVFP4: nibble ``i`` (``i < 4``) is column ``2i`` of those, nibble ``i + 4`` is column
  ``2i + 1`` (an adjacent column pair comes out with one mask), offset-binary.
  Cubic: sign-magnitude, nibble ``i`` holds ``|c|`` of column ``i`` in its low three bits, the sign of column
  ``i < 4`` is bit ``8i + 7`` of the word and that of column ``4 + i`` bit ``8i + 3`` (``cubic_lut8`` in
  ``csrc/wq_gemm_common.cuh`` turns such a word into eight bf16 weights with byte permutes);
* ``meta``: affine / NVFP4 ``uint8 [n_tiles, meta_blocks, 2, 128, 4]`` -- 1 KiB per block; Cubic
  ``uint8 [n_tiles, groups, 1, 128, 16]`` -- 2 KiB per K group: per row the eight levels
  ``s t (a + t (b + t (1 - a - b)))``, ``t = m / 7``, evaluated in fp32 and rounded ONCE to bf16 (the reference's
  decode contract), stored as low bytes of levels 0..3, 4..7, then high bytes of levels 0..3, 4..7.

All functions are pure tensor code and run on CPU or GPU.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

FMT_CUBIC4 = 0
FMT_AFFINE4 = 1
FMT_NVFP4 = 2
FMT_BF16 = 3
FMT_FP8 = 4          # e4m3 weights [N, K] as stored in the checkpoint + one fp32 scale per row; W8A8 on the fp8 tensor path
FMT_FP8_BLOCK = 5    # the same with one fp32 scale per 128 x 128 block ([ceil(N / 128), ceil(K / 128)])

TILE_N = 128
BLOCK_K = 64


@dataclass
class PackedWeight:
    fmt: int
    n: int
    k: int
    group_k: int
    codes: torch.Tensor          # uint8 (or bf16 [N, K] for FMT_BF16)
    meta: torch.Tensor | None    # uint8 (fp32 row scales for FMT_FP8)
    alpha: float = 1.0
    act_interleaved: bool = False   # gate / up rows interleaved for the fused SwiGLU epilogue (swiglu_interleave)

    def to(self, device) -> "PackedWeight":
        return PackedWeight(self.fmt, self.n, self.k, self.group_k, self.codes.to(device),
                            None if self.meta is None else self.meta.to(device), self.alpha, self.act_interleaved)

    @property
    def nbytes(self) -> int:
        return self.codes.numel() * self.codes.element_size() + (0 if self.meta is None else self.meta.numel() * self.meta.element_size())


def _tile_nibbles(nib: torch.Tensor) -> torch.Tensor:
    """``uint8 [N, K]`` values 0..15 -> tiled code bytes (N padded to 128 with `pad` already applied)."""
    n, k = nib.shape
    nt, kb = n // TILE_N, k // BLOCK_K
    v = nib.reshape(nt, TILE_N, kb, 2, 4, 4, 2).to(torch.int32)   # [nt, r, kb, h, j, pair p, even/odd e]
    # nibble index inside the word = p + 4*e  ->  byte (p + 4e) // 2, low/high nibble (p + 4e) % 2
    nibs = v.permute(0, 1, 2, 3, 4, 6, 5).reshape(nt, TILE_N, kb, 2, 4, 4, 2)  # [.., nibble index // 2, nibble index % 2]
    byts = (nibs[..., 0] | (nibs[..., 1] << 4)).to(torch.uint8)    # [nt, r, kb, h, j, byte]
    return byts.permute(0, 2, 3, 1, 4, 5).contiguous().reshape(nt, kb, 2, TILE_N, 16)


def _untile_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """Inverse of ``_tile_nibbles``: tiled bytes -> ``float [N_pad, K]`` nibble values."""
    nt, kb = codes.shape[0], codes.shape[1]
    byts = codes.reshape(nt, kb, 2, TILE_N, 4, 4).permute(0, 3, 1, 2, 4, 5).to(torch.int32)  # [nt, r, kb, h, j, byte]
    nibs = torch.stack([byts & 15, byts >> 4], -1).reshape(nt, TILE_N, kb, 2, 4, 2, 4)        # [.., e, p]
    return nibs.permute(0, 1, 2, 3, 4, 6, 5).reshape(nt * TILE_N, kb * BLOCK_K).float()


def _bf16_pair_words(lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    """Two fp32 tensors -> int32 words holding bf16(lo) in bits 0..15 and bf16(hi) in bits 16..31."""
    pair = torch.stack([lo.float().to(torch.bfloat16), hi.float().to(torch.bfloat16)], -1).contiguous()
    return pair.view(torch.int32).reshape(lo.shape)


def _pad_rows(t: torch.Tensor, rows: int, value) -> torch.Tensor:
    if t.shape[0] == rows:
        return t
    pad = torch.full((rows - t.shape[0], *t.shape[1:]), value, dtype=t.dtype, device=t.device)
    return torch.cat([t, pad], 0)


def _tile_words(words: torch.Tensor) -> torch.Tensor:
    """``int32 [N_pad, K / 8]`` code words (eight columns each) -> tiled bytes ``[nt, kb, 2, 128, 16]``."""
    n, w = words.shape
    nt, kb = n // TILE_N, w // 8
    v = words.reshape(nt, TILE_N, kb, 2, 4).permute(0, 2, 3, 1, 4).contiguous()      # [nt, kb, h, r, j]
    return v.view(torch.uint8).reshape(nt, kb, 2, TILE_N, 16)


def _untile_words(codes: torch.Tensor) -> torch.Tensor:
    """Inverse of ``_tile_words``: tiled bytes -> ``int32 [N_pad, K / 8]`` code words."""
    nt, kb = codes.shape[0], codes.shape[1]
    v = codes.contiguous().view(torch.int32).reshape(nt, kb, 2, TILE_N, 4).permute(0, 3, 1, 2, 4)
    return v.reshape(nt * TILE_N, kb * 8)


def cubic_code_words(codes: torch.Tensor) -> torch.Tensor:
    """Signed 4-bit codes ``[N, K]`` (reserved most-negative code already 0) -> sign-magnitude words ``int32 [N, K/8]``."""
    n, k = codes.shape
    c = codes.to(torch.int64).reshape(n, k // 8, 8)
    mag = c.abs().clamp(max=7)
    neg = (c < 0).to(torch.int64)
    i = torch.arange(8, device=codes.device)
    sign_bit = torch.where(i < 4, 8 * i + 7, 8 * (i - 4) + 3)
    words = ((mag << (4 * i)) | (neg << sign_bit)).sum(-1)
    return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)


def cubic_codes_from_words(words: torch.Tensor) -> torch.Tensor:
    """Inverse of ``cubic_code_words``: ``int32 [N, K/8]`` -> signed codes ``int64 [N, K]``."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    i = torch.arange(8, device=words.device)
    sign_bit = torch.where(i < 4, 8 * i + 7, 8 * (i - 4) + 3)
    mag = (w.unsqueeze(-1) >> (4 * i)) & 7
    neg = (w.unsqueeze(-1) >> sign_bit) & 1
    return (mag * (1 - 2 * neg)).reshape(words.shape[0], -1)


def cubic_levels(scale: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The eight non-negative levels of every (row, group): fp32 curve rounded once to bf16, ``[..., 8]``."""
    t = (torch.arange(8, device=scale.device, dtype=torch.float32) / 7.0)
    s, a, b = scale.float().unsqueeze(-1), a.float().unsqueeze(-1), b.float().unsqueeze(-1)
    return (s * t * (a + t * (b + t * (1.0 - a - b)))).to(torch.bfloat16)


def pack_cubic4(codes: torch.Tensor, scale: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
                group_k: int) -> PackedWeight:
    """Signed 4-bit Cubic codes ``int8 [N, K]`` (reserved code already 0) + variant-A metadata."""
    n, k = codes.shape
    if k % BLOCK_K or group_k % BLOCK_K:
        raise ValueError("K and the Cubic group must be multiples of 64")
    n_pad = -(-n // TILE_N) * TILE_N
    words = cubic_code_words(_pad_rows(codes.to(torch.int16), n_pad, 0))
    groups = -(-k // group_k)
    sc = _pad_rows(scale.float().reshape(n, groups), n_pad, 0.0)
    af = _pad_rows(a.float().reshape(n, groups), n_pad, 0.0)
    bf = _pad_rows(b.float().reshape(n, groups), n_pad, 0.0)
    lv = cubic_levels(sc, af, bf).contiguous().view(torch.uint8).reshape(n_pad, groups, 8, 2)   # [.., level, lo / hi byte]
    table = torch.cat([lv[..., 0], lv[..., 1]], -1)                                 # [N, G, 16]: 8 low bytes, 8 high bytes
    nt = n_pad // TILE_N
    meta = table.reshape(nt, TILE_N, groups, 16).permute(0, 2, 1, 3).contiguous().reshape(nt, groups, 1, TILE_N, 16)
    return PackedWeight(FMT_CUBIC4, n, k, group_k, _tile_words(words), meta)


def pack_affine4(q: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, group_k: int) -> PackedWeight:
    """Unsigned 4-bit codes ``uint8 [N, K]`` with ``w = q * scale + offset`` per (row, K-group).

    Covers INT pack-quantized (``offset = -zero_point * scale``), AWQ and GGUF
    Q4_K (``scale = d * sc``, ``offset = -dmin * m`` per 32-column sub-block).
    ``group_k`` must be a multiple of 32 (or the whole K).
    """
    n, k = q.shape
    if k % BLOCK_K or group_k % 32:
        raise ValueError("K must be a multiple of 64 and the group a multiple of 32")
    n_pad = -(-n // TILE_N) * TILE_N
    nib = _pad_rows(q.to(torch.uint8), n_pad, 0)
    groups = -(-k // group_k)
    reps = group_k // 32
    sc = _pad_rows(scale.float().reshape(n, groups), n_pad, 0.0)
    of = _pad_rows(offset.float().reshape(n, groups), n_pad, 0.0)
    words = _bf16_pair_words(sc, of + 8.0 * sc).repeat_interleave(reps, dim=1)[:, : k // 32].contiguous()
    nt, kb = n_pad // TILE_N, k // BLOCK_K
    meta = words.reshape(nt, TILE_N, kb, 2).permute(0, 2, 3, 1).contiguous()  # [nt, kb, h, 128]
    return PackedWeight(FMT_AFFINE4, n, k, group_k, _tile_nibbles(nib), meta.view(torch.uint8).reshape(nt, kb, 2, TILE_N, 4))


NVFP4_META_SHIFT = 118      # block scales are stored times 2**118 (and alpha times 2**8): see pack_nvfp4


def pack_nvfp4(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: float) -> PackedWeight:
    """NVFP4 ``weight_packed uint8 [N, K/2]`` (low nibble first), e4m3 block scales ``[N, K/16]``.

    ``global_scale`` multiplies the result (pass ``1 / weight_global_scale`` for
    compressed-tensors checkpoints, ``weight_scale_2`` for ModelOpt).

    Kernel form: the codes are re-tiled into the sign-magnitude words of the Cubic path (a nibble's low three bits,
    exponent and mantissa of the e2m1 value, are a byte-permute selector), so eight codes become four bf16 pairs
    ``magnitude x 2**-126`` through one constant table in 13 integer instructions, and ONE packed multiply per pair by
    the block scale finishes them.  For that the metadata holds ``scale x 2**118`` (exact in bf16: e4m3 scales reach
    448, so ``x 2**126`` would overflow) and ``alpha`` carries the remaining ``2**8``.
    """
    n, k2 = packed.shape
    k = k2 * 2
    if k % BLOCK_K:
        raise ValueError("K must be a multiple of 64")
    n_pad = -(-n // TILE_N) * TILE_N
    p32 = packed.to(torch.int32)
    nib = torch.stack([p32 & 15, p32 >> 4], -1).reshape(n, k)
    nib = _pad_rows(nib, n_pad, 0)
    signed = (nib & 7) * (1 - 2 * (nib >> 3))                 # -0 becomes 0: the same value
    bs = _pad_rows(block_scale.float().reshape(n, k // 16), n_pad, 0.0).reshape(n_pad, k // 32, 2) * float(2 ** NVFP4_META_SHIFT)
    words = _bf16_pair_words(bs[..., 0], bs[..., 1])
    nt, kb = n_pad // TILE_N, k // BLOCK_K
    meta = words.reshape(nt, TILE_N, kb, 2).permute(0, 2, 3, 1).contiguous()
    return PackedWeight(FMT_NVFP4, n, k, 16, _tile_words(cubic_code_words(signed)),
                        meta.view(torch.uint8).reshape(nt, kb, 2, TILE_N, 4), alpha=float(global_scale) * 256.0)


def pack_bf16(weight: torch.Tensor) -> PackedWeight:
    n, k = weight.shape
    if k % BLOCK_K:
        raise ValueError("K must be a multiple of 64")
    return PackedWeight(FMT_BF16, n, k, k, weight.to(torch.bfloat16).contiguous(), None)


def pack_fp8(weight: torch.Tensor, scale: torch.Tensor) -> PackedWeight:
    """Channel-scaled e4m3 weights for the fp8 tensor-core GEMM (``tcgen05.mma.kind::f8f6f4``): the checkpoint's bytes
    are the operand (TMA fetches 128 x 128-byte tiles of the row-major matrix), ``meta`` holds the fp32 row scales.
    ``weight``: ``torch.float8_e4m3fn`` or its bytes, ``[N, K]``; ``scale``: ``[N]`` or ``[N, 1]``."""
    n, k = weight.shape
    if k % BLOCK_K:
        raise ValueError("K must be a multiple of 64")
    codes = weight.contiguous().view(torch.uint8)
    meta = scale.to(torch.float32).reshape(-1).contiguous()
    if meta.numel() != n:
        raise ValueError("fp8 weights need one scale per output row")
    return PackedWeight(FMT_FP8, n, k, k, codes, meta)


def pack_fp8_block(weight: torch.Tensor, block_scale: torch.Tensor) -> PackedWeight:
    """Block-scaled e4m3 weights (``weight_scale_inv`` of block-quantized checkpoints: one fp32 scale per 128 x 128
    block) for the fp8 tensor-core GEMM, whose weight tile is one block row and whose pipeline stage is one block
    column.  ``weight``: ``[N, K]`` e4m3 (or its bytes); ``block_scale``: ``[ceil(N / 128), ceil(K / 128)]``."""
    n, k = weight.shape
    if k % BLOCK_K:
        raise ValueError("K must be a multiple of 64")
    meta = block_scale.to(torch.float32).contiguous()
    if tuple(meta.shape) != (-(-n // 128), -(-k // 128)):
        raise ValueError(f"block scales of a {n} x {k} matrix have shape {(-(-n // 128), -(-k // 128))}, not {tuple(meta.shape)}")
    return PackedWeight(FMT_FP8_BLOCK, n, k, 128, weight.contiguous().view(torch.uint8), meta)


def swiglu_row_order(inter: int) -> torch.Tensor:
    """Row order of a ``[gate; up]`` matrix (``2 * inter`` rows) for the fused SwiGLU epilogue of the GEMM.

    A 128-row weight tile then holds 64 output features as four blocks of {16 gate rows, 16 up rows}: the four
    epilogue warps of a tile (one TMEM lane quadrant each) find a feature's gate and up accumulators 16 lanes
    apart.  ``order[i]`` is the source row of new row ``i``.
    """
    if inter % 16:
        raise ValueError("the fused SwiGLU epilogue needs an intermediate size that is a multiple of 16")
    i = torch.arange(2 * inter)
    feature = (i // 32) * 16 + i % 16
    return feature + ((i % 32) // 16) * inter


def permute_rows(pw: PackedWeight, order: torch.Tensor) -> PackedWeight:
    """Reorder the output rows of a packed matrix (new row ``i`` = old row ``order[i]``) without re-quantizing."""
    if order.numel() != pw.n:
        raise ValueError("row order must cover every row")
    if pw.fmt == FMT_BF16:
        return PackedWeight(pw.fmt, pw.n, pw.k, pw.group_k, pw.codes[order.to(pw.codes.device)].contiguous(), None, pw.alpha)
    if pw.fmt == FMT_FP8_BLOCK:
        raise ValueError("rows of block-scaled weights cannot be reordered across scale blocks")
    if pw.fmt == FMT_FP8:
        o = order.to(pw.codes.device)
        return PackedWeight(pw.fmt, pw.n, pw.k, pw.group_k, pw.codes[o].contiguous(), pw.meta[o].contiguous(), pw.alpha)
    nt = pw.codes.shape[0]
    full = torch.cat([order, torch.arange(pw.n, nt * TILE_N)]).to(pw.codes.device)

    def rows(t: torch.Tensor) -> torch.Tensor:       # [nt, x, y, 128, w]: the row index is (dim 0, dim 3)
        shape = t.shape
        flat = t.permute(0, 3, 1, 2, 4).reshape(nt * TILE_N, -1)[full]
        return flat.reshape(nt, TILE_N, shape[1], shape[2], shape[4]).permute(0, 2, 3, 1, 4).contiguous()

    return PackedWeight(pw.fmt, pw.n, pw.k, pw.group_k, rows(pw.codes), rows(pw.meta), pw.alpha)


def swiglu_interleave(pw: PackedWeight, stacked: bool = False) -> PackedWeight:
    """``[gate; up]`` projection re-ordered for the fused SwiGLU epilogue (``kernels.wq_gemm_act``).

    ``stacked``: ``codes`` / ``meta`` carry a leading expert dimension and every expert is re-ordered.
    """
    if pw.act_interleaved:
        return pw
    if pw.fmt == FMT_FP8_BLOCK:
        # a 128-row tile of the interleaved order would mix gate and up rows of different scale blocks: block-scaled
        # weights keep their row order and the activation runs as a kernel of its own
        return pw
    order = swiglu_row_order(pw.n // 2)
    if not stacked:
        out = permute_rows(pw, order)
    else:
        per = [permute_rows(PackedWeight(pw.fmt, pw.n, pw.k, pw.group_k, pw.codes[e],
                                         None if pw.meta is None else pw.meta[e], pw.alpha), order)
               for e in range(pw.codes.shape[0])]
        out = PackedWeight(pw.fmt, pw.n, pw.k, pw.group_k, torch.stack([q.codes for q in per]),
                           None if pw.meta is None else torch.stack([q.meta for q in per]), pw.alpha)
    out.act_interleaved = True
    return out


def unpack_to_dense(pw: PackedWeight) -> torch.Tensor:
    """Oracle: rebuild the fp32 ``[N, K]`` matrix a PackedWeight represents, from its packed bytes (CPU or GPU).

    Cubic weights are exactly the bf16 levels the kernel looks up; for the other formats the bf16-rounded metadata
    is used as stored but evaluated in fp32, i.e. the value the kernel approximates with packed bf16 arithmetic.
    """
    if pw.fmt == FMT_BF16:
        return pw.codes.float()
    if pw.fmt == FMT_FP8:
        return pw.codes.view(torch.float8_e4m3fn).float() * pw.meta.reshape(-1, 1)
    if pw.fmt == FMT_FP8_BLOCK:
        s = pw.meta.repeat_interleave(128, 0)[:pw.n].repeat_interleave(128, 1)[:, :pw.k]
        return pw.codes.view(torch.float8_e4m3fn).float() * s
    nt = pw.codes.shape[0]
    if pw.fmt == FMT_CUBIC4:
        c = cubic_codes_from_words(_untile_words(pw.codes))                        # [N_pad, K]
        n_pad, k = c.shape
        g = pw.meta.shape[1]
        table = pw.meta.reshape(nt, g, TILE_N, 16).permute(0, 2, 1, 3).reshape(n_pad, g, 16)
        lv = torch.stack([table[..., :8], table[..., 8:]], -1).contiguous().view(torch.bfloat16).reshape(n_pad, g, 8).float()
        col = (torch.arange(k, device=c.device) // pw.group_k).expand(n_pad, k)
        mag = lv[torch.arange(n_pad, device=c.device).unsqueeze(1), col, c.abs()]
        return (mag * torch.sign(c).float())[: pw.n]
    if pw.fmt == FMT_NVFP4:
        c = cubic_codes_from_words(_untile_words(pw.codes))                        # signed magnitude indices [N_pad, K]
        nib = (c.abs() + 8 * (c < 0)).float()
    else:
        nib = _untile_nibbles(pw.codes)
    n_pad, k = nib.shape
    words = pw.meta.reshape(nt, -1, 2, TILE_N, 4).view(torch.int32).reshape(nt, -1, 2, TILE_N)

    def halves(w):  # int32 words -> (lo, hi) fp32 from bf16 halves
        pair = w.contiguous().view(torch.bfloat16).reshape(*w.shape, 2).float()
        return pair[..., 0], pair[..., 1]

    lo, hi = halves(words.permute(0, 3, 1, 2).reshape(n_pad, -1))   # [N, K/32] each
    if pw.fmt == FMT_AFFINE4:
        col = torch.arange(k, device=nib.device) // 32
        return ((nib - 8.0) * lo[:, col] + hi[:, col])[: pw.n]
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device=nib.device)
    bs = torch.stack([lo, hi], -1).reshape(n_pad, k // 16)
    col = torch.arange(k, device=nib.device) // 16
    # stored scales carry 2**118 and alpha 2**8 (see pack_nvfp4); the table values stand for magnitude x 2**-126
    return (lut[nib.long()] * (bs[:, col] * float(2.0 ** -126)) * pw.alpha)[: pw.n]
