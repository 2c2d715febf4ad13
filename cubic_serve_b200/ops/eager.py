"""Independent PyTorch oracles for the native kernels (fp32 math, CPU or GPU).

These never call the native library.  They follow the reference's eager
oracles in spirit (``ops/eager/attention.py``, ``ops/eager/kv_cache.py``): a
candidate kernel is always compared against code that shares nothing with it.
"""
from __future__ import annotations

import math

import torch

PAGE_TOKENS = 16
KV_GROUP = 32


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, zero_centered: bool = False) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    ww = w.float() + (1.0 if zero_centered else 0.0)
    return xf * inv * ww


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return torch.nn.functional.silu(g) * u


def rope_inv_freq(rotary_dim: int, theta: float, device=None, scaling: tuple | None = None) -> torch.Tensor:
    """Rotary frequencies.  ``scaling`` (``ModelConfig.rope_scaling``): ``("linear", factor)`` divides every frequency;
    ``("llama3", factor, low_freq_factor, high_freq_factor, original_max_position)`` keeps wavelengths below
    ``original / high`` as they are, divides those above ``original / low`` by ``factor`` and blends in between;
    ``("yarn", factor, original_max_position, beta_fast, beta_slow, attention_factor)`` blends by slot index (its
    attention factor is a softmax scale, ``ModelConfig.attention_scale``).  All are static, so the kernels see them only
    as another frequency table."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, device=device, dtype=torch.float32) / rotary_dim))
    if scaling is None:
        return inv
    if scaling[0] == "linear":
        return inv / float(scaling[1])
    if scaling[0] == "llama3":
        _, factor, low, high, original = scaling
        wavelen = 2 * torch.pi / inv
        smooth = ((original / wavelen - low) / (high - low)).clamp(0, 1)
        blended = (1 - smooth) * inv / factor + smooth * inv
        return torch.where(wavelen < original / high, inv, torch.where(wavelen > original / low, inv / factor, blended))
    if scaling[0] == "factors":                # one divisor per slot, as stored by GGUF exporters (``rope_freqs.weight``)
        div = torch.tensor(scaling[1], device=device, dtype=torch.float32)
        if div.numel() != inv.numel():
            raise ValueError("the rotary divisor table does not match the rotary width")
        return inv / div
    if scaling[0] == "yarn":
        # wavelengths that turn more than ``beta_fast`` times inside the trained context keep their frequency, those
        # that turn less than ``beta_slow`` times are stretched by ``factor``, a linear ramp over the slot index between
        _, factor, original, beta_fast, beta_slow, _ = scaling

        def slot(turns: float) -> float:
            return rotary_dim * math.log(original / (turns * 2 * math.pi)) / (2 * math.log(theta))
        low, high = max(math.floor(slot(beta_fast)), 0), min(math.ceil(slot(beta_slow)), rotary_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rotary_dim // 2, device=device, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
        return inv / factor * ramp + inv * (1 - ramp)
    raise ValueError(f"unknown rotary scaling {scaling[0]!r}")


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on ``[T, H, D]`` over the first ``2 * len(inv_freq)`` channels."""
    half = inv_freq.numel()
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    a, b, rest = xf[..., :half], xf[..., half:2 * half], xf[..., 2 * half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1)


def mrope_axes(section, half: int) -> list[int]:
    """Axis (0 temporal, 1 row, 2 column) of every frequency slot under the interleaved three-axis layout: the row axis
    takes slots 1, 4, 7, ... and the column axis 2, 5, 8, ... as far as their counts reach, the rest is temporal
    (reference: ``ops/eager/hybrid.py:112-193``)."""
    t, h, w = (int(v) for v in section)
    if t + h + w != half or min(t, h, w) <= 0:
        raise ValueError("the three section counts are positive and sum to half the rotary width")
    if max(3 * h - 2, 3 * w - 1) >= half:
        raise ValueError("the section counts do not fit the interleaved layout")
    axes = [0] * half
    for i in range(1, 3 * h, 3):
        axes[i] = 1
    for i in range(2, 3 * w, 3):
        axes[i] = 2
    return axes


def rope3(x: torch.Tensor, positions3: torch.Tensor, inv_freq: torch.Tensor, section) -> torch.Tensor:
    """Rotate-half RoPE on ``[T, H, D]`` with ``positions3 [3, T]``: frequency slot ``j`` turns by the position on axis
    ``mrope_axes(section)[j]``.  Equal rows of ``positions3`` give ``rope``."""
    half = inv_freq.numel()
    axes = torch.tensor(mrope_axes(section, half), device=positions3.device)
    pos = positions3.float()[axes, :].t()                      # [T, half]: the position each slot uses
    ang = pos * inv_freq[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    a, b, rest = xf[..., :half], xf[..., half:2 * half], xf[..., 2 * half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], -1)


def kv_quantize(x: torch.Tensor, bits: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-(token, head, 32-channel group) quantization.

    ``x``: ``[..., D]`` -> integer codes (float tensor) and fp32 scales ``[..., D/32]``.
    Range +-127 (8 bit), +-31 (6 bit), +-7 (4 bit); round-to-nearest-even.
    """
    qmax = float((1 << (bits - 1)) - 1)
    g = x.float().reshape(*x.shape[:-1], x.shape[-1] // KV_GROUP, KV_GROUP)
    amax = g.abs().amax(-1)
    scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    codes = torch.round(g / scale[..., None]).clamp(-qmax, qmax)
    return codes.reshape(x.shape), scale


def kv_quantize_token_groups(k: torch.Tensor, bits: int, tokens_per_group: int = 32) -> torch.Tensor:
    """Quantize-dequantize of keys ``[S, H, D]`` with ONE scale per (head, channel, block of ``tokens_per_group``
    tokens); the incomplete last block stays in its native precision until it fills (the "tail").  This is the
    token-grouped K form of the reference's cache ABI (``runtime/cache/quantization.py:113-286`` there); the native cache of
    this build groups 32 CHANNELS of one token instead (``kv_quantize``).  Oracle for accuracy comparisons only."""
    S = k.shape[0]
    full = S // tokens_per_group * tokens_per_group
    qmax = float((1 << (bits - 1)) - 1)
    out = k.float().clone()
    if full:
        blk = out[:full].view(full // tokens_per_group, tokens_per_group, *k.shape[1:])
        amax = blk.abs().amax(1, keepdim=True)
        scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
        out[:full] = (torch.round(blk / scale).clamp(-qmax, qmax) * scale).view(full, *k.shape[1:])
    return out


def kv_dequantize(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    g = codes.reshape(*codes.shape[:-1], codes.shape[-1] // KV_GROUP, KV_GROUP)
    return (g * scale[..., None]).reshape(codes.shape)


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, visible: torch.Tensor,
                   scale: float | None = None) -> torch.Tensor:
    """GQA attention of query rows of ONE request against its dense K/V.

    ``q``: ``[R, Hq, D]``; ``k``/``v``: ``[S, Hkv, D]``; ``visible[r]`` = number of
    leading tokens row ``r`` may see.  Returns fp32 ``[R, Hq, D]``.
    """
    r, hq, d = q.shape
    s, hkv, _ = k.shape
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    logits = torch.einsum("rhd,shd->rhs", q.float(), kf) * scale
    mask = torch.arange(s, device=q.device)[None, :] >= visible[:, None]
    logits = logits.masked_fill(mask[:, None, :], float("-inf"))
    p = torch.softmax(logits, -1)
    return torch.einsum("rhs,shd->rhd", p, vf)


# ---------------------------------------------------------------- cache blob codec
def _k_pos(bits: int, tok: torch.Tensor, ch: torch.Tensor):
    if bits == 8:
        return (ch >> 4) * 256 + tok * 16 + (ch & 15), torch.zeros_like(ch)
    c = ch & 31
    return (ch >> 5) * 256 + tok * 16 + (c & 15), torch.where(c >= 16, 4, 0)


def _v_pos(bits: int, d: int, tok: torch.Tensor, ch: torch.Tensor):
    p = tok >> 1
    chunk = (ch >> 2) ^ ((p & 3) << 2)
    if bits == 8:
        return p * (d * 2) + chunk * 8 + (ch & 3) * 2 + (tok & 1), torch.zeros_like(ch)
    return p * d + chunk * 4 + (ch & 3), torch.where((tok & 1) == 1, 4, 0)


def _k_hi_pos(d: int, tok: torch.Tensor, ch: torch.Tensor):
    """6-bit K: byte offset of the 32-bit word of high bits (from the start of the code region) and bit shift."""
    c = ch & 31
    shift = 8 * (c & 3) + torch.where(tok >= 8, 0, 4) + torch.where(c >= 16, 2, 0)
    return PAGE_TOKENS * d // 2 + (ch >> 5) * 128 + (tok & 7) * 16 + ((c & 15) >> 2) * 4, shift


def _v_hi_pos(d: int, tok: torch.Tensor, ch: torch.Tensor):
    p = tok >> 1
    chunk = (ch >> 2) ^ ((p & 3) << 2)
    shift = 8 * (ch & 3) + torch.where(p >= 4, 0, 4) + torch.where((tok & 1) == 1, 2, 0)
    return PAGE_TOKENS * d // 2 + (p & 3) * d + chunk * 4, shift


def blob_layout(d: int, k_bits: int, v_bits: int) -> dict:
    kc = PAGE_TOKENS * d * k_bits // 8
    vc = PAGE_TOKENS * d * v_bits // 8
    sc = PAGE_TOKENS * (d // KV_GROUP) * 4
    return {"k_scale": kc, "v_code": kc + sc, "v_scale": kc + sc + vc, "bytes": kc + 2 * sc + vc}


def decode_cache_page(blob: torch.Tensor, d: int, k_bits: int, v_bits: int):
    """One (page, head) blob ``uint8 [blob_bytes]`` -> dequantized fp32 K, V ``[16, D]``."""
    lay = blob_layout(d, k_bits, v_bits)
    tok = torch.arange(PAGE_TOKENS, device=blob.device)[:, None].expand(PAGE_TOKENS, d)
    ch = torch.arange(d, device=blob.device)[None, :].expand(PAGE_TOKENS, d)
    b32 = blob.to(torch.int32)

    def codes(region_off: int, pos, shift, bits, hi=None):
        if bits == 6:
            # nibble plane (4-bit layout) + plane of the two high bits, read as little-endian 32-bit words
            low = (b32[region_off + pos] >> shift) & 15
            hpos, hshift = hi
            word = (b32[region_off + hpos].long() | (b32[region_off + hpos + 1].long() << 8)
                    | (b32[region_off + hpos + 2].long() << 16) | (b32[region_off + hpos + 3].long() << 24))
            raw = (low.long() | (((word >> hshift) & 3) << 4)).to(torch.int32)
        else:
            raw = (b32[region_off + pos] >> shift) & ((1 << bits) - 1 if bits < 8 else 255)
        return (raw - (1 << (bits - 1))).float()

    kp, ks = _k_pos(k_bits, tok, ch)
    vp, vs = _v_pos(v_bits, d, tok, ch)
    kcodes = codes(0, kp, ks, k_bits, _k_hi_pos(d, tok, ch))
    vcodes = codes(lay["v_code"], vp, vs, v_bits, _v_hi_pos(d, tok, ch))
    ksc = blob[lay["k_scale"]:lay["v_code"]].contiguous().view(torch.float32).reshape(PAGE_TOKENS, d // KV_GROUP)
    vsc = blob[lay["v_scale"]:lay["bytes"]].contiguous().view(torch.float32).reshape(PAGE_TOKENS, d // KV_GROUP)
    return kv_dequantize(kcodes, ksc), kv_dequantize(vcodes, vsc)


# ------------------------------------------------------------------ gated delta net (hybrid family) oracles
def gdn_conv(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor | None, bias: torch.Tensor | None = None,
             exact: bool = False):
    """Depthwise causal conv1d (kernel 4) + SiLU over ONE request's rows ``x[n, C]`` (bf16); ``state[3, C]`` = its
    previous three inputs (None = zeros).  Returns ``(y[n, C] bf16, new state[3, C] bf16)``.  fp32 arithmetic, the
    order of ``csrc/gdn.cu`` (reference oracle: ``ops/eager/hybrid.py:255``)."""
    n, c = x.shape
    hist = torch.zeros(3, c) if state is None else state.float().cpu()
    seq = torch.cat([hist, x.float().cpu()], 0)
    wf = w.float().cpu()
    y = torch.empty(n, c)
    for t in range(n):
        win = seq[t:t + 4]                                  # inputs t-3 .. t
        a = wf[:, 0] * win[0] + wf[:, 1] * win[1] + wf[:, 2] * win[2] + wf[:, 3] * win[3]
        if bias is not None:
            a = a + bias.float().cpu()
        y[t] = a / (1 + torch.exp(-a))
    if exact:                                   # fp32 throughout: the arithmetic without the kernels' storage roundings
        return y, seq[-3:]
    return y.to(torch.bfloat16), seq[-3:].to(torch.bfloat16)


def gdn_delta(qkv: torch.Tensor, z: torch.Tensor, ba: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
              norm_w: torch.Tensor, state: torch.Tensor | None, hk: int, hv: int, eps_norm: float = 1e-6,
              eps_l2: float = 1e-6, d: int = 128, gate: str = "silu", exact: bool = False):
    """Gated delta rule + gated RMSNorm over ONE request's rows (fp32 recurrence; reference oracle:
    ``ops/eager/hybrid.py:340-548``).  ``state[Hv, d, d]`` fp32 or None; ``gate``: activation of the output gate
    (``silu`` or ``sigmoid``).  Returns ``(out[n, Hv d] bf16, state)``."""
    n = qkv.shape[0]
    bf = torch.float32 if exact else torch.bfloat16      # ``exact``: no storage roundings between the steps
    q = qkv[:, :hk * d].float().cpu().view(n, hk, d)
    k = qkv[:, hk * d:2 * hk * d].float().cpu().view(n, hk, d)
    v = qkv[:, 2 * hk * d:2 * hk * d + hv * d].float().cpu().view(n, hv, d)
    zz = z.float().cpu().view(n, hv, d)
    b, a = ba[:, :hv].float().cpu(), ba[:, hv:2 * hv].float().cpu()
    S = torch.zeros(hv, d, d) if state is None else state.float().cpu().clone()
    rep = hv // hk
    out = torch.empty(n, hv, d)
    for t in range(n):
        qn = (q[t] * torch.rsqrt((q[t] * q[t]).sum(-1, keepdim=True) + eps_l2)).to(bf).float() * (d ** -0.5)
        kn = (k[t] * torch.rsqrt((k[t] * k[t]).sum(-1, keepdim=True) + eps_l2)).to(bf).float()
        qn, kn = qn.repeat_interleave(rep, 0), kn.repeat_interleave(rep, 0)          # [Hv, d]
        beta = torch.sigmoid(b[t])
        decay = torch.exp(-torch.exp(a_log.float().cpu()) * torch.nn.functional.softplus(a[t] + dt_bias.float().cpu()))
        S = S * decay[:, None, None]
        mem = (S * kn[:, None, :]).sum(-1)                                           # [Hv, d_v]
        delta = (v[t] - mem) * beta[:, None]
        S = S + delta[:, :, None] * kn[:, None, :]
        o = (S * qn[:, None, :]).sum(-1).to(bf).float()
        normed = (o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps_norm)).to(bf).float()
        act = 1 / (1 + torch.exp(-zz[t]))
        out[t] = normed * norm_w.float().cpu()[None, :] * (act if gate == "sigmoid" else zz[t] * act)
    return out.reshape(n, hv * d).to(bf), S
