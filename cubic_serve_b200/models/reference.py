"""Eager fp32 reference decoder (CPU or GPU, no native kernels).

The oracle for end-to-end tests and the ``--execution-mode eager`` path, in the
role of the reference's ``Qwen3_5ReferenceModel.forward``
(``models/qwen3_5/model.py:1646``) and ``examples/toy_adapter.py``: plain
PyTorch, one request at a time or a padded batch, dense weights (optionally
the dequantized form of a quantized checkpoint) and an optional simulated
quantized KV cache that follows the serving cache ABI (symmetric codes, one
fp32 scale per token / head / 32-channel group).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import eager
from ..quantization import cubic
from .config import ModelConfig


@dataclass
class DenseLayer:
    ln1: torch.Tensor
    ln2: torch.Tensor
    wq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor
    w_gate: torch.Tensor
    w_up: torch.Tensor
    w_down: torch.Tensor
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None


@dataclass
class DenseWeights:
    embed: torch.Tensor
    layers: list[DenseLayer]
    final_norm: torch.Tensor
    lm_head: torch.Tensor


def random_dense_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> DenseWeights:
    g = torch.Generator().manual_seed(seed)
    H, D = cfg.hidden_size, cfg.head_dim

    def rnd(n, k):
        return torch.randn(n, k, generator=g) * std

    layers = []
    for _ in range(cfg.num_layers):
        layers.append(DenseLayer(
            ln1=torch.ones(H), ln2=torch.ones(H),
            wq=rnd(cfg.q_size, H), wk=rnd(cfg.kv_size, H), wv=rnd(cfg.kv_size, H), wo=rnd(H, cfg.q_size),
            w_gate=rnd(cfg.intermediate_size, H), w_up=rnd(cfg.intermediate_size, H),
            w_down=rnd(H, cfg.intermediate_size),
            q_norm=torch.ones(D) if cfg.qk_norm else None, k_norm=torch.ones(D) if cfg.qk_norm else None))
    embed = rnd(cfg.vocab_size, H)
    head = embed if cfg.tie_embeddings else rnd(cfg.vocab_size, H)
    return DenseWeights(embed, layers, torch.ones(H), head)


def dense_weights_from_checkpoint(ck) -> DenseWeights:
    """fp32 weights of a dense full-attention decoder checkpoint, every linear decoded by its quantization extension
    (the values the packed kernels approximate): what the eager reference engine and ``cubic reference`` run on."""
    from .checkpoint import CheckpointError, _dense_of, _layer_modules, logical_inventory
    cfg = ck.cfg
    if cfg.is_moe or cfg.is_hybrid:
        raise CheckpointError("the eager reference decoder covers dense full-attention decoders")
    shapes, _ = logical_inventory(cfg)
    method, q = cfg.quant.method, cfg.quant

    def lin(module):
        p = ck.payload(module)
        if len(p) == 1 and "weight" in p:                 # an unquantized module of a quantized checkpoint
            return p["weight"].float()
        return _dense_of(method, p, shapes[module], q).float()

    get = lambda name: ck.store.get(name).float()  # noqa: E731
    layers = []
    for i in range(cfg.num_layers):
        m = _layer_modules(cfg, i)
        pre = f"model.layers.{i}"
        layers.append(DenseLayer(
            get(f"{pre}.input_layernorm.weight"), get(f"{pre}.post_attention_layernorm.weight"),
            lin(m["q"]), lin(m["k"]), lin(m["v"]), lin(m["o"]), lin(m["gate"]), lin(m["up"]), lin(m["down"]),
            get(f"{pre}.self_attn.q_norm.weight") if cfg.qk_norm else None,
            get(f"{pre}.self_attn.k_norm.weight") if cfg.qk_norm else None))
    embed = ck.plain_tensor("model.embed_tokens.weight").float()
    head = embed if cfg.tie_embeddings else ck.plain_tensor("lm_head.weight").float()
    return DenseWeights(embed, layers, get("model.norm.weight"), head)


def cubic_roundtrip(w: torch.Tensor, bits: int = 4, group: int = 128) -> torch.Tensor:
    scheme = cubic.CubicScheme(bits=bits, group_in=group)
    return cubic.decode(cubic.quantize(w, scheme), scheme, tuple(w.shape))


def quantize_dense_weights(w: DenseWeights, bits: int = 4, group: int = 128) -> DenseWeights:
    """Every linear projection replaced by its CubicQuant decode (embedding / norms / lm_head kept)."""
    q = lambda t: cubic_roundtrip(t, bits, group)  # noqa: E731
    layers = [DenseLayer(l.ln1, l.ln2, q(l.wq), q(l.wk), q(l.wv), q(l.wo), q(l.w_gate), q(l.w_up), q(l.w_down),
                         l.q_norm, l.k_norm) for l in w.layers]
    return DenseWeights(w.embed, layers, w.final_norm, w.lm_head)


class EagerDecoder:
    """Batched greedy decoding with a dense (optionally quantize-simulated) KV cache."""

    def __init__(self, cfg: ModelConfig, weights: DenseWeights, kv_bits: tuple[int, int] | None = None) -> None:
        self.cfg, self.w, self.kv_bits = cfg, weights, kv_bits
        self.inv_freq = eager.rope_inv_freq(cfg.rotary_dim or cfg.head_dim, cfg.rope_theta, scaling=cfg.rope_scaling)

    def _kvq(self, x: torch.Tensor, bits: int | None) -> torch.Tensor:
        if bits is None or bits >= 16:
            return x
        d = x.shape[-1]
        if d % eager.KV_GROUP:
            # heads narrower than / not a multiple of the group: one scale per head
            qmax = float((1 << (bits - 1)) - 1)
            amax = x.abs().amax(-1, keepdim=True)
            s = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
            return torch.round(x / s).clamp(-qmax, qmax) * s
        codes, scale = eager.kv_quantize(x, bits)
        return eager.kv_dequantize(codes, scale)

    def forward(self, tokens: torch.Tensor, start: int, cache: list | None):
        """``tokens``: ``[B, S]`` new tokens at positions ``start..start+S-1`` (same for every row).

        ``cache``: list per layer of ``(k, v)`` tensors ``[B, past, Hkv, D]`` or ``None``.
        Returns fp32 logits ``[B, S, V]`` and the updated cache.
        """
        cfg, w = self.cfg, self.w
        B, S = tokens.shape
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        pos = torch.arange(start, start + S)
        h = w.embed[tokens].float()
        new_cache = []
        for li, l in enumerate(w.layers):
            x = eager.rmsnorm(h, l.ln1, cfg.rms_eps, cfg.zero_centered_norm)
            q = (x @ l.wq.t()).view(B, S, Hq, D)
            k = (x @ l.wk.t()).view(B, S, Hkv, D)
            v = (x @ l.wv.t()).view(B, S, Hkv, D)
            if l.q_norm is not None:
                q = eager.rmsnorm(q, l.q_norm, cfg.rms_eps)
                k = eager.rmsnorm(k, l.k_norm, cfg.rms_eps)
            q = torch.stack([eager.rope(q[b], pos, self.inv_freq) for b in range(B)])
            k = torch.stack([eager.rope(k[b], pos, self.inv_freq) for b in range(B)])
            if self.kv_bits is not None:
                k, v = self._kvq(k, self.kv_bits[0]), self._kvq(v, self.kv_bits[1])
            if cache is not None and cache[li] is not None:
                k = torch.cat([cache[li][0], k], 1)
                v = torch.cat([cache[li][1], v], 1)
            new_cache.append((k, v))
            vis = torch.arange(start + 1, start + S + 1)
            attn = torch.stack([eager.attention_rows(q[b], k[b], v[b], vis, cfg.attention_scale) for b in range(B)])
            h = h + attn.reshape(B, S, Hq * D) @ l.wo.t()
            x = eager.rmsnorm(h, l.ln2, cfg.rms_eps, cfg.zero_centered_norm)
            h = h + (torch.nn.functional.silu(x @ l.w_gate.t()) * (x @ l.w_up.t())) @ l.w_down.t()
        logits = eager.rmsnorm(h, w.final_norm, cfg.rms_eps, cfg.zero_centered_norm) @ w.lm_head.t()
        return logits, new_cache

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, steps: int):
        """Greedy decode ``steps`` tokens for ``[B, P]`` prompts; returns tokens ``[B, steps]`` and per-step logits."""
        logits, cache = self.forward(prompts, 0, None)
        out, all_logits = [], []
        nxt = logits[:, -1].argmax(-1)
        for i in range(steps):
            out.append(nxt)
            all_logits.append(logits[:, -1])
            if i + 1 == steps:
                break
            logits, cache = self.forward(nxt[:, None], prompts.shape[1] + i, cache)
            nxt = logits[:, -1].argmax(-1)
        return torch.stack(out, 1), torch.stack(all_logits, 1)
