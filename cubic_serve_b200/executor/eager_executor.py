"""Eager (PyTorch, CPU or GPU) executor with a paged fp32 KV store.

``--execution-mode eager``: the same ``execute(segments)`` contract as the
native executor, implemented with the independent oracle math in
``models/reference.py``.  It keeps K/V per physical page so prefix sharing and
copy-on-write behave exactly as on the GPU path; the quantized cache is
simulated by quantize -> dequantize at write time.
"""
from __future__ import annotations

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.reference import DenseWeights, EagerDecoder
from ..ops import eager
from .gpu_executor import Segment

PAGE = 16


def sample_row(logits: torch.Tensor, s: Segment) -> int:
    """The sampled token of one row of fp32 logits under the segment's mask and sampling parameters."""
    if getattr(s, "mask", None) is not None:                  # structured output: disallowed tokens cannot win
        bits = np.unpackbits(np.asarray(s.mask, dtype=np.uint32).view(np.uint8), bitorder="little")
        allowed = torch.from_numpy(bits[:logits.numel()].astype(bool))
        logits = logits.masked_fill(~allowed, float("-inf"))
    if s.temperature <= 0:
        return int(logits.argmax())
    k = s.top_k if 0 < s.top_k <= 20 else 20
    vals, idx = logits.topk(k)
    p = torch.softmax(vals / s.temperature, -1)
    if s.top_p < 1:
        keep = int((p.cumsum(0) < s.top_p).sum()) + 1
        p = p[:keep] / p[:keep].sum()
    g = torch.Generator().manual_seed((s.seed * 1000003 + s.draw) & 0x7FFFFFFF)
    return int(idx[torch.multinomial(p, 1, generator=g)])


class EagerPagedExecutor:
    accepts_features = True          # segments may carry encoder feature rows and three-axis positions
    accepts_deepstack = True         # ... and additions after the first decoder layers

    def __init__(self, cfg: ModelConfig, weights: DenseWeights, num_pages: int,
                 kv_bits: tuple[int, int] | None = None) -> None:
        self.cfg = cfg
        self.dec = EagerDecoder(cfg, weights, kv_bits)
        shape = (num_pages, PAGE, cfg.num_kv_heads, cfg.head_dim)
        self.k = [torch.zeros(shape) for _ in range(cfg.num_layers)]
        self.v = [torch.zeros(shape) for _ in range(cfg.num_layers)]
        self.h2d_bytes_last = self.d2h_bytes_last = self.kernel_launches_last = 0

    def copy_pages(self, pairs) -> None:
        for src, dst in pairs:
            for li in range(self.cfg.num_layers):
                self.k[li][dst] = self.k[li][src]
                self.v[li][dst] = self.v[li][src]

    @torch.no_grad()
    def execute(self, segs: list[Segment]) -> np.ndarray:
        out = []
        for s in segs:
            logits = self._run_segment(s)
            if s.sample:
                out.append(sample_row(logits, s))
        return np.asarray(out, dtype=np.int32)

    def _run_segment(self, s: Segment) -> torch.Tensor:
        cfg, w, dec = self.cfg, self.dec.w, self.dec
        n = len(s.token_ids)
        pages = torch.as_tensor(np.asarray(s.pages), dtype=torch.long)
        pos = torch.arange(s.start, s.start + n)
        total = s.start + n
        h = w.embed[torch.as_tensor(np.asarray(s.token_ids), dtype=torch.long)].float()
        for off, rows in (s.embeds or ()):                        # encoder features take the place of the embedding
            h[off:off + rows.shape[0]] = rows.float()
        pos3 = None
        if s.positions3 is not None and cfg.mrope_section is not None:
            pos3 = torch.as_tensor(np.asarray(s.positions3), dtype=torch.long)
        rot = (lambda t: eager.rope(t, pos, dec.inv_freq)) if pos3 is None else \
            (lambda t: eager.rope3(t, pos3, dec.inv_freq, cfg.mrope_section))
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        for li, l in enumerate(w.layers):
            x = eager.rmsnorm(h, l.ln1, cfg.rms_eps, cfg.zero_centered_norm)
            q = (x @ l.wq.t()).view(n, Hq, D)
            k = (x @ l.wk.t()).view(n, Hkv, D)
            v = (x @ l.wv.t()).view(n, Hkv, D)
            if l.q_norm is not None:
                q, k = eager.rmsnorm(q, l.q_norm, cfg.rms_eps), eager.rmsnorm(k, l.k_norm, cfg.rms_eps)
            q, k = rot(q), rot(k)
            if dec.kv_bits is not None:
                k, v = dec._kvq(k, dec.kv_bits[0]), dec._kvq(v, dec.kv_bits[1])
            self.k[li][pages[pos // PAGE], pos % PAGE] = k
            self.v[li][pages[pos // PAGE], pos % PAGE] = v
            np_ = -(-total // PAGE)
            kk = self.k[li][pages[:np_]].reshape(np_ * PAGE, Hkv, D)[:total]
            vv = self.v[li][pages[:np_]].reshape(np_ * PAGE, Hkv, D)[:total]
            attn = eager.attention_rows(q, kk, vv, pos + 1, cfg.attention_scale)
            h = h + attn.reshape(n, Hq * D) @ l.wo.t()
            x = eager.rmsnorm(h, l.ln2, cfg.rms_eps, cfg.zero_centered_norm)
            h = h + (torch.nn.functional.silu(x @ l.w_gate.t()) * (x @ l.w_up.t())) @ l.w_down.t()
            for off, rows in (getattr(s, "deep_embeds", None) or ()):
                if li < rows.shape[1]:
                    h[off:off + rows.shape[0]] += rows[:, li].float()
        last = eager.rmsnorm(h[-1:], w.final_norm, cfg.rms_eps, cfg.zero_centered_norm)
        return (last @ w.lm_head.t())[0]
