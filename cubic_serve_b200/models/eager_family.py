"""One eager model for every decoder family of ``ModelConfig``: dense, mixture-of-experts (with or without a shared
expert), hybrid Gated DeltaNet / gated attention, and their combination; any head width; projection biases; partial
and three-axis rotary positions.

This is the execution mode that serves what the native runner has no kernels for (shared experts, q / k / v biases,
attention heads wider than 128, feature rows of a vision tower) and the oracle the native runner's families are
compared with.  Weights are the checkpoint's logical tensors decoded to fp32 by their quantization extension and
addressed by checkpoint name; nothing is re-laid out, so the row conventions of the checkpoint are stated once, here:

* ``linear_attn.in_proj_qkvz`` rows are grouped by key head ``[q | k | v x r | z x r]`` (``r`` value heads per key
  head), ``in_proj_ba`` likewise ``[b x r | a x r]``; the convolution's channels are ``q | k | v`` of all heads;
* a gated attention layer's ``q_proj`` rows are ``[q_h | gate_h]`` per head; the attention output is multiplied by
  ``sigmoid(gate)``;
* norms of the hybrid families are zero-centred (weight ``1 + w``), including the per-head q / k norms; the Gated
  DeltaNet output norm is not.

``EagerFamilyModel.forward`` appends ONE request's tokens to its explicit state (K / V per attention layer,
convolution and recurrent state per Gated DeltaNet layer), so chunked prefill, decoding and one pass agree.
``EagerFamilyExecutor`` puts it behind the engine's ``execute(segments)``.

Reference counterpart: ``models/qwen3_5/model.py:1399-1510`` (reference math of the hybrid family),
``models/qwen3_5_moe`` (shared expert), ``runtime/reference_engine.py`` (the eager serving mode).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

import numpy as np
import torch
import torch.nn.functional as F

from ..executor.stateful_executor import StatefulEagerExecutor
from ..ops import eager
from .config import ModelConfig


# ------------------------------------------------------------------ weights
def family_tensor_shapes(cfg: ModelConfig) -> dict[str, tuple[int, ...]]:
    """Logical tensors by checkpoint name: ``<module>.weight`` for every linear, the plain tensors as they are."""
    from .checkpoint import logical_inventory
    linears, plain = logical_inventory(cfg)
    H, D = cfg.hidden_size, cfg.head_dim
    out = {f"{m}.weight": shape for m, shape in linears.items()}
    for name in plain:
        if name.endswith("conv1d.weight"):
            out[name] = ((2 * cfg.gdn_k_heads + cfg.gdn_v_heads) * 128, 1, 4)
        elif name.endswith(("A_log", "dt_bias")):
            out[name] = (cfg.gdn_v_heads,)
        elif name.endswith("linear_attn.norm.weight"):
            out[name] = (128,)
        elif name.endswith(("q_norm.weight", "k_norm.weight")):
            out[name] = (D,)
        elif name.endswith("norm.weight") or "pre_fc_norm" in name:
            out[name] = (H,)
        elif name.endswith("mlp.gate.weight"):
            out[name] = (cfg.num_experts, H)
        elif name.endswith("shared_expert_gate.weight"):
            out[name] = (1, H)
        elif name.endswith("q_proj.bias"):
            out[name] = (cfg.q_size,)
        elif name.endswith(("k_proj.bias", "v_proj.bias")):
            out[name] = (cfg.kv_size,)
        else:                                                   # embeddings, lm_head
            out[name] = (cfg.vocab_size, H)
    return out


def random_family_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in family_tensor_shapes(cfg).items():
        if name.endswith("A_log"):
            w[name] = torch.rand(shape, generator=g) * 1.5
        elif name.endswith("dt_bias"):
            w[name] = torch.randn(shape, generator=g) * 0.5
        elif name.endswith("linear_attn.norm.weight"):
            w[name] = 1 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("norm.weight") or "pre_fc_norm" in name:
            centre = 0.0 if cfg.zero_centered_norm else 1.0
            w[name] = centre + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("conv1d.weight"):
            w[name] = 0.3 * torch.randn(shape, generator=g)
        else:
            w[name] = std * torch.randn(shape, generator=g)
    return w


def family_weights_from_checkpoint(ck) -> dict[str, torch.Tensor]:
    """fp32 logical tensors of an admitted checkpoint: every linear decoded by its quantization extension."""
    from .checkpoint import _dense_of, logical_inventory
    cfg = ck.cfg
    linears, plain = logical_inventory(cfg)
    w = {}
    for module, shape in linears.items():
        p = ck.payload(module)
        w[f"{module}.weight"] = p["weight"].float() if len(p) == 1 and "weight" in p else \
            _dense_of(cfg.quant.method, p, shape, cfg.quant).float()
    for name in plain:
        w[name] = ck.plain_tensor(name).float()
    return w


# ------------------------------------------------------------------ state
@dataclass
class FamilyLayerState:
    key: torch.Tensor | None = None           # [S, Hkv, D]
    value: torch.Tensor | None = None
    conv: torch.Tensor | None = None          # [3, C] bf16
    recurrent: torch.Tensor | None = None     # [Hv, 128, 128] fp32


@dataclass
class FamilyState:
    length: int = 0
    layers: list = field(default_factory=list)


class EagerFamilyModel:
    def __init__(self, cfg: ModelConfig, weights: Mapping[str, torch.Tensor], kv_bits: tuple[int, int] | None = None,
                 exact: bool = False) -> None:
        """``exact``: the Gated DeltaNet layers run without the storage roundings of the native kernels (bf16 between
        their steps); the default reproduces those roundings, which is what the kernels are compared with."""
        self.exact = exact
        want = family_tensor_shapes(cfg)
        missing = sorted(set(want) - set(weights))
        if missing:
            raise ValueError(f"tensors missing: {missing[:3]}")
        for n, shape in want.items():
            if tuple(weights[n].shape) != shape:
                raise ValueError(f"{n}: shape {tuple(weights[n].shape)}, expected {shape}")
        self.cfg, self.kv_bits = cfg, kv_bits
        self.w = {n: weights[n].float() for n in want}
        self.inv_freq = eager.rope_inv_freq(cfg.rotary_dim or cfg.head_dim, cfg.rope_theta, scaling=cfg.rope_scaling)

    def _lin(self, x: torch.Tensor, module: str) -> torch.Tensor:
        y = x @ self.w[module + ".weight"].t()
        b = self.w.get(module + ".bias")
        return y if b is None else y + b

    def _norm(self, x: torch.Tensor, name: str, centred: bool | None = None) -> torch.Tensor:
        c = self.cfg.zero_centered_norm if centred is None else centred
        return eager.rmsnorm(x, self.w[name], self.cfg.rms_eps, c)

    def _kvq(self, x: torch.Tensor, bits: int) -> torch.Tensor:
        if bits >= 16 or x.shape[-1] % eager.KV_GROUP:
            return x
        return eager.kv_dequantize(*eager.kv_quantize(x, bits))

    def _attention(self, x: torch.Tensor, st: FamilyLayerState, p: str, start: int, pos3) -> torch.Tensor:
        c = self.cfg
        T, Hq, Hkv, D = x.shape[0], c.num_q_heads, c.num_kv_heads, c.head_dim
        q = self._lin(x, p + ".q_proj")
        gate = None
        if c.attn_output_gate:
            q = q.view(T, Hq, 2 * D)
            q, gate = q[..., :D], q[..., D:]
        q = q.reshape(T, Hq, D)
        k = self._lin(x, p + ".k_proj").view(T, Hkv, D)
        v = self._lin(x, p + ".v_proj").view(T, Hkv, D)
        if c.qk_norm:
            q, k = self._norm(q, p + ".q_norm.weight"), self._norm(k, p + ".k_norm.weight")
        if pos3 is not None and c.mrope_section is not None:
            q, k = (eager.rope3(t, pos3, self.inv_freq, c.mrope_section) for t in (q, k))
        else:
            pos = torch.arange(start, start + T) if pos3 is None else pos3[0]
            q, k = eager.rope(q, pos, self.inv_freq), eager.rope(k, pos, self.inv_freq)
        if self.kv_bits is not None:
            k, v = self._kvq(k, self.kv_bits[0]), self._kvq(v, self.kv_bits[1])
        st.key = k if st.key is None else torch.cat([st.key, k], 0)
        st.value = v if st.value is None else torch.cat([st.value, v], 0)
        out = eager.attention_rows(q, st.key, st.value, torch.arange(start + 1, start + T + 1), c.attention_scale)
        if gate is not None:
            out = out * torch.sigmoid(gate)
        return out.reshape(T, Hq * D) @ self.w[p + ".o_proj.weight"].t()

    def _gdn(self, x: torch.Tensor, st: FamilyLayerState, p: str) -> torch.Tensor:
        c = self.cfg
        T, gk, gv = x.shape[0], c.gdn_k_heads, c.gdn_v_heads
        r = gv // gk
        qkvz = self._lin(x, p + ".in_proj_qkvz").view(T, gk, (2 + 2 * r) * 128)
        q, k = qkvz[..., :128], qkvz[..., 128:256]
        v, z = qkvz[..., 256:256 + r * 128], qkvz[..., 256 + r * 128:]
        mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], -1)
        mixed = mixed if self.exact else mixed.to(torch.bfloat16)
        ba = self._lin(x, p + ".in_proj_ba").view(T, gk, 2, r)
        ba = torch.cat([ba[:, :, 0].reshape(T, gv), ba[:, :, 1].reshape(T, gv)], -1)
        conv_w = self.w[p + ".conv1d.weight"].reshape(-1, 4)
        mixed, st.conv = eager.gdn_conv(mixed, conv_w, st.conv, exact=self.exact)
        out, st.recurrent = eager.gdn_delta(mixed, z.reshape(T, gv * 128), ba, self.w[p + ".A_log"], self.w[p + ".dt_bias"],
                                            self.w[p + ".norm.weight"], st.recurrent, gk, gv, eps_norm=c.rms_eps,
                                            exact=self.exact)
        return out.float() @ self.w[p + ".out_proj.weight"].t()

    def _ffn(self, x: torch.Tensor, p: str) -> torch.Tensor:
        c = self.cfg
        if not c.is_moe:
            return (F.silu(self._lin(x, p + ".gate_proj")) * self._lin(x, p + ".up_proj")) @ self.w[p + ".down_proj.weight"].t()
        logits = x @ self.w[p + ".gate.weight"].t()
        order = torch.argsort(-logits, dim=-1, stable=True)[:, :c.experts_per_token]        # ties: the lower expert id
        sel = torch.gather(logits, 1, order)
        wt = torch.softmax(sel, -1) if c.norm_topk_prob else torch.softmax(logits, -1).gather(1, order)
        out = torch.zeros_like(x)
        for e in order.unique().tolist():
            rows, slot = (order == e).nonzero(as_tuple=True)
            xe, ep = x[rows], f"{p}.experts.{e}"
            ye = (F.silu(self._lin(xe, ep + ".gate_proj")) * self._lin(xe, ep + ".up_proj")) @ self.w[ep + ".down_proj.weight"].t()
            out.index_add_(0, rows, ye * wt[rows, slot][:, None])
        if c.shared_intermediate_size:
            s = p + ".shared_expert"
            shared = (F.silu(self._lin(x, s + ".gate_proj")) * self._lin(x, s + ".up_proj")) @ self.w[s + ".down_proj.weight"].t()
            out = out + shared * torch.sigmoid(x @ self.w[p + ".shared_expert_gate.weight"].t())
        return out

    @torch.no_grad()
    def forward(self, tokens, state: FamilyState | None = None, positions3=None, embeds=None, last_only: bool = False,
                deep=None):
        """Logits ``[T, vocab]`` (``[1, vocab]`` with ``last_only``) of ``tokens`` appended to ``state`` (updated in
        place and returned)."""
        c = self.cfg
        tokens = [int(t) for t in tokens]
        if not tokens or min(tokens) < 0 or max(tokens) >= c.vocab_size:
            raise ValueError("a non-empty list of token ids inside the vocabulary")
        state = state or FamilyState()
        if not state.layers:
            state.layers = [FamilyLayerState() for _ in range(c.num_layers)]
        T, start = len(tokens), state.length
        pos3 = None if positions3 is None else torch.as_tensor(np.asarray(positions3), dtype=torch.long)
        if pos3 is not None and pos3.shape != (3, T):
            raise ValueError("positions are [3, tokens]")
        h = self.w["model.embed_tokens.weight"][torch.tensor(tokens)]
        for off, rows in (embeds or ()):
            h[off:off + rows.shape[0]] = rows.float()
        for i in range(c.num_layers):
            p, st = f"model.layers.{i}", state.layers[i]
            x = self._norm(h, p + ".input_layernorm.weight")
            h = h + (self._gdn(x, st, p + ".linear_attn") if c.layer_is_gdn(i) else
                     self._attention(x, st, p + ".self_attn", start, pos3))
            h = h + self._ffn(self._norm(h, p + ".post_attention_layernorm.weight"), p + ".mlp")
            for off, rows in (deep or ()):                    # the tower's intermediate outputs join after early layers
                if i < rows.shape[1]:
                    h[off:off + rows.shape[0]] += rows[:, i].float()
        state.length = start + T
        self.last_feedback = h                                    # the hidden rows before the final norm feed a draft head
        last = self._norm(h[-1:] if last_only else h, "model.norm.weight")
        head = self.w["model.embed_tokens.weight"] if c.tie_embeddings else self.w["lm_head.weight"]
        return last @ head.t(), state

    @property
    def has_draft_head(self) -> bool:
        return "mtp.fc.weight" in self.w

    @torch.no_grad()
    def draft_forward(self, tokens, feedback: torch.Tensor, state: FamilyState | None = None):
        """The multi-token-prediction head on ``tokens`` (token ``i + 1``) paired with ``feedback`` (the target's hidden
        row of position ``i``): ``fc([norm(embedding) ; norm(hidden)])`` enters one full-attention layer of the model's
        kind, whose output (before ``mtp.norm``) is the feedback of the next proposal; logits through the shared head."""
        c = self.cfg
        if not self.has_draft_head:
            raise ValueError("the checkpoint carries no draft head")
        tokens = [int(t) for t in tokens]
        T = len(tokens)
        if feedback.shape != (T, c.hidden_size):
            raise ValueError("one hidden row per token")
        state = state or FamilyState()
        if not state.layers:
            state.layers = [FamilyLayerState()]
        start = state.length
        e = self._norm(self.w["model.embed_tokens.weight"][torch.tensor(tokens)], "mtp.pre_fc_norm_embedding.weight")
        hh = self._norm(feedback.float(), "mtp.pre_fc_norm_hidden.weight")
        h = torch.cat([e, hh], -1) @ self.w["mtp.fc.weight"].t()
        p, st = "mtp.layers.0", state.layers[0]
        h = h + self._attention(self._norm(h, p + ".input_layernorm.weight"), st, p + ".self_attn", start, None)
        h = h + self._ffn(self._norm(h, p + ".post_attention_layernorm.weight"), p + ".mlp")
        state.length = start + T
        head = self.w["model.embed_tokens.weight"] if c.tie_embeddings else self.w["lm_head.weight"]
        return self._norm(h, "mtp.norm.weight") @ head.t(), h, state


def copy_family_state(state: FamilyState) -> FamilyState:
    """A state that can be advanced without touching ``state`` (the model never writes its tensors in place)."""
    from dataclasses import replace
    return FamilyState(state.length, [replace(l) for l in state.layers])


class EagerFamilyExecutor(StatefulEagerExecutor):
    """``execute(segments)`` on ``EagerFamilyModel`` with one explicit state per request slot (no pages, no prefix
    sharing: ``keeps_request_state`` tells the engine so); with ``speculative_depth`` > 0 and a checkpoint that carries
    the multi-token-prediction head, greedy requests decode in lossless draft / review rounds."""

    accepts_deepstack = True

    def __init__(self, cfg: ModelConfig, weights: Mapping[str, torch.Tensor], kv_bits: tuple[int, int] | None = None,
                 speculative_depth: int = 0) -> None:
        self.cfg = cfg
        super().__init__(EagerFamilyModel(cfg, weights, kv_bits), speculative_depth)

    def _new_state(self) -> FamilyState:
        return FamilyState()

    def _copy(self, state: FamilyState) -> FamilyState:
        return copy_family_state(state)
