"""Multi-token-prediction (MTP) draft head on the native kernels.

Structure of the reference's MTP head (``models/qwen3_5/model.py:1512-1644``, ``executor/mtp_runner.py:152``):

    u = fc([ rmsnorm_e(embed(token)) ; rmsnorm_h(previous hidden) ])      # 2H -> H
    u = one full-attention decoder layer (own KV pages)                  # same layer code as the target
    logits = lm_head(rmsnorm(u))                                          # embeddings and lm_head are SHARED

Depth 1 consumes the target's hidden state of the last verified position, deeper proposals chain the head's
own output hidden.  The head writes its KV into its own one-layer cache at the same page ids / slots as the
target, so no extra page accounting is needed.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import kernels as K
from ..ops import wq_pack
from .config import ModelConfig
from .decoder import DecoderRunner, LayerWeights, StepBatch, quantize_linear


@dataclass
class MtpWeights:
    enorm: torch.Tensor
    hnorm: torch.Tensor
    fc: wq_pack.PackedWeight          # [H, 2H]
    layer: LayerWeights
    norm: torch.Tensor


def random_mtp_weights(cfg: ModelConfig, device, seed: int = 1, std: float = 0.02, tp_rank: int = 0,
                       tp_size: int = 1) -> MtpWeights:
    """Random head weights.  Under tensor parallelism every rank draws the FULL matrices from the same seed and keeps
    its rows (QKV: whole heads, gate / up features) or columns (o, down), like ``random_decoder_weights``; the
    2H -> H input projection and the norms are replicated."""
    gen = torch.Generator(device=device).manual_seed(seed * 7919)
    H, D = cfg.hidden_size, cfg.head_dim
    from .config import kv_heads_of_rank
    kv_first, hkv = kv_heads_of_rank(cfg.num_kv_heads, tp_rank, tp_size)
    hq, inter = cfg.num_q_heads // tp_size, cfg.intermediate_size // tp_size
    r = tp_rank

    def rnd(n, k):
        return torch.randn(n, k, device=device, generator=gen) * std

    def sections(full, widths):
        out, base = [], 0
        for w in widths:
            out.append(full[base + r * w:base + (r + 1) * w])
            base += w * tp_size
        return torch.cat(out).contiguous()

    def cols(full, width):
        return full[:, r * width:(r + 1) * width].contiguous()

    ones = lambda n: torch.ones(n, device=device, dtype=torch.bfloat16)  # noqa: E731
    qkv = rnd((cfg.num_q_heads + 2 * cfg.num_kv_heads) * D, H)
    o = rnd(H, cfg.q_size)
    gate_up = rnd(2 * cfg.intermediate_size, H)
    down = rnd(H, cfg.intermediate_size)
    kb, vb = cfg.num_q_heads * D, (cfg.num_q_heads + cfg.num_kv_heads) * D
    qkv_local = torch.cat([qkv[r * hq * D:(r + 1) * hq * D], qkv[kb + kv_first * D:kb + (kv_first + hkv) * D],
                           qkv[vb + kv_first * D:vb + (kv_first + hkv) * D]]).contiguous()
    layer = LayerWeights(ln1=ones(H), ln2=ones(H), qkv=quantize_linear(qkv_local, cfg),
                         o=quantize_linear(cols(o, hq * D), cfg),
                         gate_up=quantize_linear(sections(gate_up, [inter, inter]), cfg),
                         down=quantize_linear(cols(down, inter), cfg))
    return MtpWeights(ones(H), ones(H), quantize_linear(rnd(H, 2 * H), cfg), layer, ones(H))


class MtpRunner:
    """Runs the draft head for a batch of rows; shares buffers, embeddings and lm_head with the target runner."""

    def __init__(self, target: DecoderRunner, weights: MtpWeights) -> None:
        self.t = target
        self.w = weights
        cfg, dev = target.cfg, target.device
        if target.tp is not None and target.tp.fused is not None:
            raise ValueError("the MTP head runs with the NCCL tensor-parallel collectives (tp mode 'nccl')")
        self.part = (torch.empty(target.max_tokens, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
                     if target.tp is not None else None)
        blob = K.kv_blob_bytes(target.D, target.k_bits, target.v_bits)
        self.kv = torch.zeros(target.num_pages, target.hkv, blob, dtype=torch.uint8, device=dev)
        T, H = target.max_tokens, cfg.hidden_size
        bf = torch.bfloat16
        self.cat = torch.empty(T, 2 * H, dtype=bf, device=dev)
        self.emb = torch.empty(T, H, dtype=bf, device=dev)
        self.h = torch.empty(T, H, dtype=bf, device=dev)
        self.launches = 0
        from ..ops.strategies import active
        lw = weights.layer
        if active().gemm.fuse_swiglu and torch.device(dev).type == "cuda" and (lw.gate_up.n // 2) % 16 == 0:
            lw.gate_up = wq_pack.swiglu_interleave(lw.gate_up)

    def forward(self, b: StepBatch, prev_hidden: torch.Tensor) -> torch.Tensor:
        """One pass over ``b.num_tokens`` rows.  ``prev_hidden[i]`` is the hidden state that precedes row i.

        Returns the head's output hidden ``[T, H]`` (the residual stream after its decoder layer).
        """
        t, w, cfg = self.t, self.w, self.t.cfg
        T, H = b.num_tokens, cfg.hidden_size
        emb, cat, h = self.emb[:T], self.cat[:T], self.h[:T]
        tp = t.tp
        K.embedding(b.token_ids[:T], t.w.embed, out=emb, vocab_start=t.w.vocab_start)
        if tp is not None:
            tp.all_reduce(emb)                      # vocabulary-sharded table: the owner contributes the row, the others zeros
        # the two normalised halves sit side by side in `cat` (row stride 2H); the norm kernel writes dense
        # rows, so it goes through dense temporaries and the halves are copied in
        e_n = K.rmsnorm(emb, w.enorm, cfg.rms_eps)
        h_n = K.rmsnorm(prev_hidden[:T], w.hnorm, cfg.rms_eps)
        cat[:, :H].copy_(e_n)
        cat[:, H:].copy_(h_n)
        K.wq_gemm(cat, w.fc, out=h, ws=t.ws)
        lw = w.layer
        x, qkv, q, attn = t.x[:T], t.qkv[:T], t.q[:T], t.attn[:T]
        K.rmsnorm(h, lw.ln1, cfg.rms_eps, out=x)
        K.wq_gemm(x, lw.qkv, out=qkv, ws=t.ws)
        K.rope_kv_write(qkv, q, self.kv, b.positions, b.slots, t.inv_freq, t.hq, t.hkv, t.D, t.k_bits, t.v_bits,
                        q_norm=lw.q_norm, k_norm=lw.k_norm, eps=cfg.rms_eps, rotary_dim=cfg.rotary_dim,
                        rotate=t.kv_rotation)
        K.paged_attention(q.view(T, t.hq, t.D), attn.view(T, t.hq, t.D), self.kv, b.page_table,
                          b.rb_req[:b.num_row_blocks], b.rb_qstart, b.rb_qcount, b.rb_ctx, t.hq, t.hkv, t.D, t.k_bits,
                          t.v_bits, scale=t.cfg.attention_scale, splits=b.attn_splits, ws=t.ws)
        if t.kv_rotation:
            K.hadamard(attn)
        if tp is None:
            K.wq_gemm(attn, lw.o, out=h, residual=h, ws=t.ws)
            K.rmsnorm(h, lw.ln2, cfg.rms_eps, out=x)
        else:
            part = self.part[:T]
            K.wq_gemm(attn, lw.o, out=part, ws=t.ws)
            tp.all_reduce(part)
            K.rmsnorm(part, lw.ln2, cfg.rms_eps, out=x, residual=h)      # h += sum of the ranks' partial rows
        gu, act = t.gu[:T], t.act[:T]
        fused = 2 - K.gate_up_act(x, lw.gate_up, gu, act, ws=t.ws)
        if tp is None:
            K.wq_gemm(act, lw.down, out=h, residual=h, ws=t.ws)
        else:
            part = self.part[:T]
            K.wq_gemm(act, lw.down, out=part, ws=t.ws)
            tp.all_reduce(part)
            h.add_(part)
        self.launches = 16 - fused + (4 if tp is not None else 0)
        return h

    def logits(self, hidden: torch.Tensor, rows: int, out: torch.Tensor) -> torch.Tensor:
        xn = K.rmsnorm(hidden[:rows], self.w.norm, self.t.cfg.rms_eps)
        return K.wq_gemm(xn, self.t.w.lm_head, out=out[:rows], ws=self.t.ws)
