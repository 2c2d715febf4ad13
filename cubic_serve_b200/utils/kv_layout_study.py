"""Accuracy of the two K-cache grouping schemes on keys with outlier channels (CPU, eager oracles).

    python -m cubic_serve_b200.utils.kv_layout_study

Keys of real decoders carry a few channels whose magnitude is many times the rest (rotary pairs of low frequency).  The
native cache quantizes 32 consecutive CHANNELS of one token with one scale: an outlier channel sets the scale of its 31
neighbours.  The reference's cache ABI gives every channel its own scale over a block of 32 TOKENS (and keeps the
incomplete block unquantized): outliers stay in their own groups, at the price of a write path that needs a tail.
The native cache's answer to outliers is its rotation option (``--enable-kv-cache-rotation``): q and k are
Walsh-Hadamard transformed before the keys are quantized, which spreads an outlier over the whole head.
The script measures, for the three schemes and INT8 / INT6 / INT4 codes, the relative error of the attention logits
``q . k`` and of the attention output on synthetic keys with a controllable outlier ratio, and prints one JSON object.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import eager


def hadamard(n: int) -> torch.Tensor:
    """Normalised Walsh-Hadamard matrix of a power-of-two size (symmetric, its own inverse)."""
    h = torch.ones(1, 1)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    if h.shape[0] != n:
        raise ValueError("the head width is a power of two")
    return h / n ** 0.5


def study(seq: int = 512, heads: int = 4, dim: int = 128, outlier_channels: int = 4, ratio: float = 20.0, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(seq, heads, dim, generator=g)
    idx = torch.randperm(dim, generator=g)[:outlier_channels]
    k[..., idx] *= ratio
    v = torch.randn(seq, heads, dim, generator=g)
    q = torch.randn(16, heads, dim, generator=g)
    q[..., idx] /= ratio ** 0.5                                    # queries are small where keys are large, as in trained models

    def logits(keys):
        return torch.einsum("thd,shd->ths", q, keys) / dim ** 0.5

    def output(keys):
        return torch.einsum("ths,shd->thd", torch.softmax(logits(keys), -1), v)
    ref_l, ref_o = logits(k), output(k)
    rel = lambda a, b: float((a - b).norm() / b.norm())            # noqa: E731
    rows = {}
    had = hadamard(dim)
    for bits in (8, 6, 4):
        per_token = eager.kv_dequantize(*eager.kv_quantize(k, bits))
        per_channel = eager.kv_quantize_token_groups(k, bits)
        # the native cache's rotation option: q and k are Walsh-Hadamard transformed (q . k is unchanged), the transformed
        # keys are quantized; an outlier channel is spread over all channels of the head
        rotated = eager.kv_dequantize(*eager.kv_quantize(k @ had, bits))
        rot_l = torch.einsum("thd,shd->ths", q @ had, rotated) / dim ** 0.5
        rot_o = torch.einsum("ths,shd->thd", torch.softmax(rot_l, -1), v)
        rows[f"int{bits}"] = {
            "channel_groups_of_a_token": {"logits": round(rel(logits(per_token), ref_l), 5), "output": round(rel(output(per_token), ref_o), 5)},
            "channel_groups_after_rotation": {"logits": round(rel(rot_l, ref_l), 5), "output": round(rel(rot_o, ref_o), 5)},
            "token_groups_of_a_channel": {"logits": round(rel(logits(per_channel), ref_l), 5), "output": round(rel(output(per_channel), ref_o), 5)}}
    return {"seq": seq, "heads": heads, "dim": dim, "outlier_channels": outlier_channels, "outlier_ratio": ratio, "errors": rows}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ratio", type=float, nargs="*", default=[1.0, 5.0, 20.0, 50.0])
    ap.add_argument("--outlier-channels", type=int, default=4)
    args = ap.parse_args(argv)
    print(json.dumps([study(outlier_channels=args.outlier_channels, ratio=r) for r in args.ratio], indent=1))


if __name__ == "__main__":
    main()
