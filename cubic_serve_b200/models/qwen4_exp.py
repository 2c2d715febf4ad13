"""The ``qwen4_exp`` family: configuration, tensor inventory and the eager model.

What distinguishes the family from the hybrid decoders of ``models/decoder.py``:

* the residual carries ``S`` parallel streams of the hidden width.  Every block reads a gated mean over the streams
  (group norm per stream, low-rank sigmoid gate) and writes its output back into every stream through per-stream gates
  in (0, 2); there are no separate input layer norms, and the final mixer feeds ``lm_head`` directly
  (``ops/eager_sparse.py``: ``stream_mix`` / ``stream_injection`` / ``stream_combine``);
* the full-attention layers select what they attend to: raw index keys are mean-pooled over ``compression`` tokens,
  a small multi-head indexer scores the pooled keys, and each query attends to the tokens of the best
  ``budget / compression`` blocks plus the incomplete tail block (``select_blocks`` / ``attend_selected``).  Below the
  budget this is plain causal attention;
* layers listed in ``ple_layer_ids`` add a lexical signal before their blocks: hashed n-gram ids of the last tokens look
  up rows of a large sharded table; a per-stream signed-root gate of (projected embedding . normalised residual)
  scales a value projection, and a dilated depthwise convolution over the gated rows (dilation = n-gram size) adds
  context;
* Gated DeltaNet layers with separate ``in_proj_qkv / z / a / b`` projections and a sigmoid output gate;
* mixture-of-experts feed-forward with packed expert tensors and a sigmoid-gated shared expert.

``Qwen4ExpModel.forward`` runs ONE request's new tokens against its explicit state (per layer: convolution and
recurrent matrices, K / V, raw and pooled index keys, n-gram history and convolution history), so prefill in chunks,
token-by-token decoding and one pass over the whole sequence give the same logits.  fp32 arithmetic on the weights as
stored.  ``Qwen4ExpEagerExecutor`` serves the family through the engine (``--execution-mode eager``); the native runner
does not.

Reference counterpart: ``models/qwen4_exp/model.py:588-1060`` (configuration), ``:1102-1549`` (reference model),
``models/qwen4_exp/weights.py:166-497`` (tensor inventory), ``ops/eager/ngram.py`` (hashing, dilated convolution).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, replace
from typing import Mapping

import numpy as np
import torch
import torch.nn.functional as F

from ..executor.stateful_executor import StatefulEagerExecutor
from ..ops import eager
from ..ops import eager_sparse as sp

LM = "model.language_model"


class Qwen4ExpConfigError(ValueError):
    pass


@dataclass(frozen=True)
class Qwen4ExpConfig:
    vocab_size: int
    hidden_size: int
    num_layers: int
    layer_types: tuple[str, ...]                  # "linear_attention" | "full_attention" per layer
    max_position: int
    rms_eps: float
    # full attention
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    rotary_dim: int
    rope_theta: float
    mrope_section: tuple[int, int, int]
    # Gated DeltaNet
    gdn_k_heads: int
    gdn_v_heads: int
    gdn_k_dim: int
    gdn_v_dim: int
    gdn_conv_kernel: int
    gdn_output_gate: str
    # experts
    num_experts: int
    experts_per_token: int
    moe_intermediate_size: int
    shared_intermediate_size: int
    norm_topk_prob: bool
    # residual streams
    streams: int
    stream_low_rank: int
    # sparse attention indexer
    index_heads: int
    index_dim: int
    index_budget: int
    index_compression: int
    # lexical n-gram embedding
    ple_layer_ids: tuple[int, ...]                # 1-based layer numbers
    ple_embed_dim: int
    ple_conv_kernel: int
    ngram_size: int
    heads_per_ngram: int
    ngram_vocab_base: int
    ngram_vocab_multiple: int
    ngram_split_parts: int
    ngram_shard_rows: int = 2_500_012
    eos_token_id: int | None = None
    mtp_layers: int = 0
    name: str = "qwen4_exp"
    family: str = "qwen4_exp"
    vision: object | None = None                  # ``models.vision.VisionConfig`` of multimodal checkpoints

    is_hybrid = True                              # recurrent state: the engine keeps the prefix cache off
    is_moe = True

    @property
    def stream_width(self) -> int:
        return self.hidden_size * self.streams

    @property
    def ngram_heads(self) -> int:
        return (self.ngram_size - 1) * self.heads_per_ngram

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_k_heads * self.gdn_k_dim + self.gdn_v_heads * self.gdn_v_dim

    def layer_is_gdn(self, i: int) -> bool:
        return self.layer_types[i] == "linear_attention"

    def uses_ple(self, i: int) -> bool:
        return i + 1 in self.ple_layer_ids

    def validate(self) -> None:
        c = self
        if len(c.layer_types) != c.num_layers or any(t not in ("linear_attention", "full_attention") for t in c.layer_types):
            raise Qwen4ExpConfigError("layer_types lists linear_attention / full_attention once per layer")
        if min(c.vocab_size, c.hidden_size, c.num_layers, c.num_q_heads, c.num_kv_heads, c.head_dim, c.streams,
               c.stream_low_rank, c.num_experts, c.experts_per_token, c.moe_intermediate_size, c.index_heads,
               c.index_dim, c.index_budget, c.index_compression) <= 0:
            raise Qwen4ExpConfigError("sizes are positive")
        if c.num_q_heads % c.num_kv_heads or c.experts_per_token > c.num_experts:
            raise Qwen4ExpConfigError("query heads divide into key/value groups; top-k is at most the expert count")
        if c.rotary_dim <= 0 or c.rotary_dim % 2 or c.rotary_dim > min(c.head_dim, c.index_dim):
            raise Qwen4ExpConfigError("the rotary width is even and fits the attention and indexer heads")
        eager.mrope_axes(c.mrope_section, c.rotary_dim // 2)
        if c.index_budget % c.index_compression:
            raise Qwen4ExpConfigError("the token budget is a whole number of compressed blocks")
        if c.gdn_k_dim != c.gdn_v_dim or c.gdn_v_heads % c.gdn_k_heads or c.gdn_conv_kernel != 4:
            raise Qwen4ExpConfigError("Gated DeltaNet heads share one width, value heads group over key heads, kernel 4")
        if c.gdn_output_gate not in ("sigmoid", "silu"):
            raise Qwen4ExpConfigError(f"unknown output gate {c.gdn_output_gate!r}")
        if c.ple_layer_ids:
            if any(not 1 <= i <= c.num_layers for i in c.ple_layer_ids) or len(set(c.ple_layer_ids)) != len(c.ple_layer_ids):
                raise Qwen4ExpConfigError("ple_layer_ids are distinct 1-based layer numbers")
            if c.ngram_size < 2 or c.heads_per_ngram <= 0 or c.ple_embed_dim % c.ngram_heads or c.ple_embed_dim != c.hidden_size:
                raise Qwen4ExpConfigError("the n-gram embedding divides over its heads and has the hidden width")
            if c.eos_token_id is None:
                raise Qwen4ExpConfigError("n-gram hashing needs the checkpoint's eos_token_id")
            if c.ngram_split_parts <= 0 or c.ngram_shard_rows <= 0 or c.ple_conv_kernel <= 0:
                raise Qwen4ExpConfigError("the n-gram table has a positive number of shards and rows")


_TEXT_KEYS = {
    "attention_bias", "attention_dropout", "dtype", "full_attention_interval", "hc_count", "hc_lowrank", "head_dim",
    "heads_per_ngram", "hidden_act", "hidden_size", "indexer_budget", "indexer_compress_ratio", "indexer_head_dim",
    "indexer_kv_heads", "indexer_n_heads", "layer_types", "linear_conv_kernel_dim", "linear_key_head_dim",
    "linear_num_key_heads", "linear_num_value_heads", "linear_value_head_dim", "make_ngram_vocab_size_divisible_by",
    "mamba_ssm_dtype", "max_position_embeddings", "model_type", "moe_intermediate_size", "mtp", "mtp_num_hidden_layers",
    "mtp_use_dedicated_embeddings", "ngram_size", "ngram_vocab_size_base", "num_attention_heads", "num_experts",
    "num_experts_per_tok", "num_hidden_layers", "num_key_value_heads", "output_gate_type", "partial_rotary_factor",
    "ple_conv_kernel_size", "ple_embed_dim", "ple_layer_ids", "rms_norm_eps", "rope_parameters",
    "shared_expert_intermediate_size", "split_ngram_parts", "use_cache", "vocab_size", "eos_token_id", "norm_topk_prob",
    "ngram_shard_rows", "ple_embedding_dtype", "torch_dtype", "initializer_range", "bos_token_id", "pad_token_id",
    "tie_word_embeddings"}


def parse_qwen4_exp_config(raw: Mapping[str, object]) -> Qwen4ExpConfig:
    """``config.json`` of a ``qwen4_exp`` checkpoint.  Unknown text keys, attention biases, tied embeddings and
    activations other than SiLU are refused rather than ignored."""
    if raw.get("model_type") != "qwen4_exp":
        raise Qwen4ExpConfigError("model_type must be 'qwen4_exp'")
    text = raw.get("text_config")
    if not isinstance(text, dict):
        raise Qwen4ExpConfigError("config.text_config is an object")
    extra = sorted(set(text) - _TEXT_KEYS)
    if extra:
        raise Qwen4ExpConfigError(f"text_config has unknown keys {extra}")
    if text.get("attention_bias") or raw.get("tie_word_embeddings") or text.get("tie_word_embeddings"):
        raise Qwen4ExpConfigError("attention biases and tied embeddings are not part of this family")
    if text.get("hidden_act", "silu") != "silu":
        raise Qwen4ExpConfigError("the feed-forward activation is SiLU")
    if int(text.get("indexer_kv_heads", 1)) != 1:
        raise Qwen4ExpConfigError("the indexer has one key head")
    rope = text.get("rope_parameters") or {}
    try:
        hd = int(text["head_dim"])
        factor = float(rope.get("partial_rotary_factor", text.get("partial_rotary_factor", 1.0)))
        vision = None
        if isinstance(raw.get("vision_config"), dict) and not raw.get("language_model_only", False):
            from .vision import VisionConfig
            vision = VisionConfig.from_hf({k: v for k, v in raw["vision_config"].items()})
        cfg = Qwen4ExpConfig(
            vocab_size=int(text["vocab_size"]), hidden_size=int(text["hidden_size"]),
            num_layers=int(text["num_hidden_layers"]), layer_types=tuple(str(t) for t in text["layer_types"]),
            max_position=int(text.get("max_position_embeddings", 262144)), rms_eps=float(text.get("rms_norm_eps", 1e-6)),
            num_q_heads=int(text["num_attention_heads"]), num_kv_heads=int(text["num_key_value_heads"]), head_dim=hd,
            rotary_dim=int(hd * factor), rope_theta=float(rope.get("rope_theta", 1e7)),
            mrope_section=tuple(int(v) for v in rope["mrope_section"]),
            gdn_k_heads=int(text["linear_num_key_heads"]), gdn_v_heads=int(text["linear_num_value_heads"]),
            gdn_k_dim=int(text["linear_key_head_dim"]), gdn_v_dim=int(text["linear_value_head_dim"]),
            gdn_conv_kernel=int(text.get("linear_conv_kernel_dim", 4)),
            gdn_output_gate=str(text.get("output_gate_type", "sigmoid")),
            num_experts=int(text["num_experts"]), experts_per_token=int(text["num_experts_per_tok"]),
            moe_intermediate_size=int(text["moe_intermediate_size"]),
            shared_intermediate_size=int(text.get("shared_expert_intermediate_size", 0)),
            norm_topk_prob=bool(text.get("norm_topk_prob", True)),
            streams=int(text["hc_count"]), stream_low_rank=int(text["hc_lowrank"]),
            index_heads=int(text["indexer_n_heads"]), index_dim=int(text["indexer_head_dim"]),
            index_budget=int(text["indexer_budget"]), index_compression=int(text["indexer_compress_ratio"]),
            ple_layer_ids=tuple(int(i) for i in text.get("ple_layer_ids", ())),
            ple_embed_dim=int(text.get("ple_embed_dim", text["hidden_size"])),
            ple_conv_kernel=int(text.get("ple_conv_kernel_size", 4)), ngram_size=int(text.get("ngram_size", 3)),
            heads_per_ngram=int(text.get("heads_per_ngram", 8)),
            ngram_vocab_base=int(text.get("ngram_vocab_size_base", 0)),
            ngram_vocab_multiple=int(text.get("make_ngram_vocab_size_divisible_by", 1)),
            ngram_split_parts=int(text.get("split_ngram_parts", 1)),
            ngram_shard_rows=int(text.get("ngram_shard_rows", 2_500_012)),
            eos_token_id=text.get("eos_token_id") if isinstance(text.get("eos_token_id"), int) else
            (raw.get("eos_token_id") if isinstance(raw.get("eos_token_id"), int) else None),
            mtp_layers=int(text.get("mtp_num_hidden_layers") or 0),
            name=str(raw.get("_name_or_path") or "qwen4_exp"), vision=vision)
    except KeyError as e:
        raise Qwen4ExpConfigError(f"text_config lacks {e.args[0]!r}") from None
    except (TypeError, ValueError) as e:
        if isinstance(e, Qwen4ExpConfigError):
            raise
        raise Qwen4ExpConfigError(f"malformed value: {e}") from None
    if vision is not None and vision.out_hidden_size != cfg.hidden_size:
        raise Qwen4ExpConfigError("the vision tower's output width equals the hidden size")
    cfg.validate()
    return cfg


def parse_qwen4_exp_config_json(document: str | bytes) -> Qwen4ExpConfig:
    def unique(pairs):
        out = {}
        for k, v in pairs:
            if k in out:
                raise Qwen4ExpConfigError(f"duplicate key {k!r}")
            out[k] = v
        return out

    def no_constant(name):
        raise Qwen4ExpConfigError(f"non-finite constant {name}")
    try:
        raw = json.loads(document, object_pairs_hook=unique, parse_constant=no_constant)
    except json.JSONDecodeError as e:
        raise Qwen4ExpConfigError(f"config.json is not JSON: {e}") from None
    if not isinstance(raw, dict):
        raise Qwen4ExpConfigError("config.json holds an object")
    return parse_qwen4_exp_config(raw)


# ------------------------------------------------------------------ tensor inventory
def _stream_mixer(p: str, cfg: Qwen4ExpConfig, inject: bool) -> dict[str, tuple[int, ...]]:
    sw = cfg.stream_width
    out = {f"{p}.hc_norm.weight": (sw,), f"{p}.input_mix_weight_down.weight": (cfg.stream_low_rank, sw),
           f"{p}.input_mix_weight_up.weight": (sw, cfg.stream_low_rank)}
    if inject:
        out[f"{p}.block_inject_weight.weight"] = (cfg.streams, sw)
    return out


def qwen4_exp_tensor_shapes(cfg: Qwen4ExpConfig) -> dict[str, tuple[int, ...]]:
    """Every text tensor of a checkpoint by name (int64 tensors: the three ``ple_embedding`` metadata vectors)."""
    H, sw = cfg.hidden_size, cfg.stream_width
    s: dict[str, tuple[int, ...]] = {f"{LM}.embed_tokens.weight": (cfg.vocab_size, H), "lm_head.weight": (cfg.vocab_size, H)}
    s.update(_stream_mixer(f"{LM}.hyper_connection_mixer", cfg, inject=False))
    for i in range(cfg.num_layers):
        p = f"{LM}.layers.{i}"
        s.update(_stream_mixer(f"{p}.attn_hyper_connection", cfg, True))
        s.update(_stream_mixer(f"{p}.mlp_hyper_connection", cfg, True))
        if cfg.layer_is_gdn(i):
            a, vd = f"{p}.linear_attn", cfg.gdn_v_heads * cfg.gdn_v_dim
            s.update({f"{a}.A_log": (cfg.gdn_v_heads,), f"{a}.dt_bias": (cfg.gdn_v_heads,),
                      f"{a}.conv1d.weight": (cfg.gdn_conv_dim, 1, cfg.gdn_conv_kernel),
                      f"{a}.in_proj_a.weight": (cfg.gdn_v_heads, H), f"{a}.in_proj_b.weight": (cfg.gdn_v_heads, H),
                      f"{a}.in_proj_qkv.weight": (cfg.gdn_conv_dim, H), f"{a}.in_proj_z.weight": (vd, H),
                      f"{a}.norm.weight": (cfg.gdn_v_dim,), f"{a}.out_proj.weight": (H, vd)})
        else:
            a, qd, kd = f"{p}.self_attn", cfg.num_q_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
            s.update({f"{a}.q_proj.weight": (2 * qd, H), f"{a}.k_proj.weight": (kd, H), f"{a}.v_proj.weight": (kd, H),
                      f"{a}.o_proj.weight": (H, qd), f"{a}.q_norm.weight": (cfg.head_dim,), f"{a}.k_norm.weight": (cfg.head_dim,),
                      f"{a}.indexer.index_qk_proj.weight": ((cfg.index_heads + 1) * cfg.index_dim, H),
                      f"{a}.indexer.q_layernorm.weight": (cfg.index_dim,), f"{a}.indexer.k_layernorm.weight": (cfg.index_dim,)})
        m, I = f"{p}.mlp", cfg.moe_intermediate_size
        s.update({f"{m}.experts.gate_up_proj": (cfg.num_experts, 2 * I, H), f"{m}.experts.down_proj": (cfg.num_experts, H, I),
                  f"{m}.gate.weight": (cfg.num_experts, H)})
        if cfg.shared_intermediate_size:
            si = cfg.shared_intermediate_size
            s.update({f"{m}.shared_expert.gate_proj.weight": (si, H), f"{m}.shared_expert.up_proj.weight": (si, H),
                      f"{m}.shared_expert.down_proj.weight": (H, si), f"{m}.shared_expert_gate.weight": (1, H)})
        if cfg.uses_ple(i):
            e = f"{p}.ple"
            s.update({f"{e}.conv1d.weight": (sw, 1, cfg.ple_conv_kernel), f"{e}.key_proj.weight": (sw, H),
                      f"{e}.value_proj.weight": (H, H), f"{e}.norm_conv.weight": (sw,), f"{e}.norm_key.weight": (sw,),
                      f"{e}.norm_query.weight": (sw,), f"{e}.ple_embedding.layer_multipliers": (cfg.ngram_size,),
                      f"{e}.ple_embedding.ngram_heads_offsets": (cfg.ngram_heads,),
                      f"{e}.ple_embedding.ngram_heads_vocab_sizes": (cfg.ngram_heads,)})
            for part in range(cfg.ngram_split_parts):
                s[f"{e}.ple_embedding.ngram_embedding.shard_{part}.weight"] = (cfg.ngram_shard_rows,
                                                                                cfg.ple_embed_dim // cfg.ngram_heads)
    return s


def qwen4_exp_mtp_tensor_shapes(cfg: Qwen4ExpConfig) -> dict[str, tuple[int, ...]]:
    """Tensors of the draft head (``mtp.*``): projections of the next token's embedding and of the target's multi-stream
    residual, one block-selective attention layer with experts, and its own final mixer; embeddings and ``lm_head`` are
    the target's."""
    H, sw = cfg.hidden_size, cfg.stream_width
    s: dict[str, tuple[int, ...]] = {"mtp.pre_fc_norm_embedding.weight": (H,), "mtp.fc_embedding.weight": (H, H),
                                     "mtp.pre_fc_norm_hidden.weight": (sw,), "mtp.fc_hidden.weight": (H, H)}
    s.update(_stream_mixer("mtp.hyper_connection_mixer", cfg, inject=False))
    one = replace(cfg, num_layers=1, layer_types=("full_attention",), ple_layer_ids=())
    for name, shape in qwen4_exp_tensor_shapes(one).items():
        if name.startswith(f"{LM}.layers.0."):
            s["mtp.layers.0." + name[len(f"{LM}.layers.0."):]] = shape
    return s


def ngram_head_vocab_sizes(cfg: Qwen4ExpConfig) -> list[int]:
    """Moduli of the hash heads: distinct multiples of ``ngram_vocab_multiple`` upward from the base size, so the heads
    of one order collide on different ids; their sum fits the table."""
    rows = cfg.ngram_split_parts * cfg.ngram_shard_rows
    per = rows // cfg.ngram_heads
    base = min(cfg.ngram_vocab_base or per, per)
    m = max(1, cfg.ngram_vocab_multiple)
    top = max(m, base // m * m)
    sizes = [max(m, top - j * m) for j in range(cfg.ngram_heads)]
    if sum(sizes) > rows:
        raise Qwen4ExpConfigError("the n-gram table is smaller than its heads' vocabularies")
    return sizes


def random_qwen4_exp_weights(cfg: Qwen4ExpConfig, seed: int = 0, std: float = 0.05, draft_head: bool = False) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}
    sizes = ngram_head_vocab_sizes(cfg) if cfg.ple_layer_ids else []
    shapes = dict(qwen4_exp_tensor_shapes(cfg))
    if draft_head:
        shapes.update(qwen4_exp_mtp_tensor_shapes(cfg))
    for name, shape in shapes.items():
        if name.endswith("layer_multipliers"):
            w[name] = torch.randint(1, 1 << 40, shape, generator=g, dtype=torch.int64) * 2 + 1
        elif name.endswith("ngram_heads_vocab_sizes"):
            w[name] = torch.tensor(sizes, dtype=torch.int64)
        elif name.endswith("ngram_heads_offsets"):
            w[name] = torch.tensor([sum(sizes[:j]) for j in range(len(sizes))], dtype=torch.int64)
        elif name.endswith("A_log"):
            w[name] = torch.rand(shape, generator=g) * 1.5
        elif name.endswith("dt_bias"):
            w[name] = torch.randn(shape, generator=g) * 0.5
        elif name.endswith(".norm.weight") and "linear_attn" in name:
            w[name] = 1 + 0.1 * torch.randn(shape, generator=g)
        elif "norm" in name.split(".")[-2] or name.endswith("layernorm.weight"):
            w[name] = 0.1 * torch.randn(shape, generator=g)            # zero-centred norms: weight = 1 + w
        elif name.endswith("conv1d.weight"):
            w[name] = 0.3 * torch.randn(shape, generator=g)
        else:
            w[name] = std * torch.randn(shape, generator=g)
    return w


def check_qwen4_exp_weights(cfg: Qwen4ExpConfig, weights: Mapping[str, torch.Tensor]) -> None:
    want = dict(qwen4_exp_tensor_shapes(cfg))
    if any(n.startswith("mtp.") for n in weights):
        want.update(qwen4_exp_mtp_tensor_shapes(cfg))                  # the draft head comes whole or not at all
    missing, extra = sorted(set(want) - set(weights)), sorted(set(weights) - set(want))
    if missing or extra:
        raise Qwen4ExpConfigError(f"tensors missing {missing[:3]} unexpected {extra[:3]}")
    for n, shape in want.items():
        if tuple(weights[n].shape) != shape:
            raise Qwen4ExpConfigError(f"{n}: shape {tuple(weights[n].shape)}, expected {shape}")


# ------------------------------------------------------------------ lexical hashing and the dilated convolution
_MASK = (1 << 64) - 1


def _wrap(v: int) -> int:
    """Two's-complement int64 of an unbounded integer."""
    v &= _MASK
    return v - (1 << 64) if v >> 63 else v


def ngram_hash_ids(tokens: list[int], history: list[int], multipliers: list[int], vocab_sizes: list[int],
                   offsets: list[int], eos: int) -> tuple[list[list[int]], list[int]]:
    """Table rows of every token's n-grams and the new history (the last ``order - 1`` tokens).

    With ``x_0`` the token and ``x_l`` the token ``l`` places back (everything at and before an EOS that precedes the
    token reads as EOS), the order-``l + 1`` hash is ``xor_{j <= l} x_j * m_j`` in wrapping 64-bit arithmetic; head
    ``h`` of that order reads row ``hash mod size_h + offset_h`` (non-negative remainder)."""
    order = len(multipliers)
    heads = len(vocab_sizes) // (order - 1)
    if order < 2 or len(history) != order - 1 or len(vocab_sizes) != heads * (order - 1) or len(offsets) != len(vocab_sizes):
        raise ValueError("the history holds order - 1 tokens and every order has the same number of heads")
    ctx = list(history)
    rows = []
    for tok in tokens:
        window = ctx + [tok]
        hashed = _wrap(tok * multipliers[0])
        reset = False
        ids = []
        for lag in range(1, order):
            prev = window[-1 - lag]
            reset = reset or prev == eos
            hashed ^= _wrap((eos if reset else prev) * multipliers[lag])
            for h in range((lag - 1) * heads, lag * heads):
                ids.append(hashed % vocab_sizes[h] + offsets[h])          # Python's % is the non-negative remainder
        rows.append(ids)
        ctx = window[1:]
    return rows, ctx


def dilated_causal_conv(x: torch.Tensor, history: torch.Tensor, weight: torch.Tensor, dilation: int):
    """Depthwise causal convolution over rows ``x [T, C]`` with taps ``dilation`` rows apart, then SiLU.
    ``history [(K - 1) dilation, C]`` holds the rows before ``x``; tap ``K - 1`` reads the current row.  Returns
    ``(y [T, C], new history)``."""
    K = weight.shape[-1]
    span = (K - 1) * dilation
    if history.shape != (span, x.shape[1]) or weight.shape[0] != x.shape[1]:
        raise ValueError("history is [(K - 1) dilation, C] and the kernel has one row per channel")
    seq = torch.cat([history, x], 0)
    T = x.shape[0]
    acc = torch.zeros_like(x, dtype=torch.float32)
    for k in range(K):
        acc = acc + seq[k * dilation:k * dilation + T].float() * weight[:, 0, k].float()
    return F.silu(acc), seq[T:T + span] if span else seq[:0]


# ------------------------------------------------------------------ state
@dataclass
class LayerState:
    conv: torch.Tensor | None = None               # GDN: last K - 1 inputs of the convolution [K - 1, C]
    recurrent: torch.Tensor | None = None          # GDN: [Hv, D, D] fp32
    key: torch.Tensor | None = None                # attention: [S, Hkv, D]
    value: torch.Tensor | None = None
    index_raw: torch.Tensor | None = None          # raw index keys [S, Di]
    index_pooled: torch.Tensor | None = None       # pooled, normalised, rotated [S // compression, Di]
    ngram_history: list | None = None
    ple_conv: torch.Tensor | None = None
    positions: torch.Tensor | None = None          # [3, S] (kept for the pooled keys' rotation)


@dataclass
class RequestState:
    length: int = 0
    layers: list = field(default_factory=list)


class Qwen4ExpModel:
    def __init__(self, cfg: Qwen4ExpConfig, weights: Mapping[str, torch.Tensor], expert_range: tuple[int, int] | None = None,
                 reduce_experts=None) -> None:
        cfg.validate()
        check_qwen4_exp_weights(cfg, weights)
        self.cfg = cfg
        self.w = {n: (t if t.dtype == torch.int64 else t.float()) for n, t in weights.items()}
        self.inv_freq = eager.rope_inv_freq(cfg.rotary_dim, cfg.rope_theta)
        self.expert_range = expert_range or (0, cfg.num_experts)
        if self.expert_range != (0, cfg.num_experts) and reduce_experts is None:
            raise ValueError("a share of the experts needs the reduction that completes the routed sum")
        self.reduce_experts = reduce_experts
        self._tables: dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ pieces
    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return x @ self.w[name + ".weight"].t()

    def _mix(self, h: torch.Tensor, p: str):
        w, c = self.w, self.cfg
        return sp.stream_mix(h, w[p + ".hc_norm.weight"], w[p + ".input_mix_weight_down.weight"],
                             w[p + ".input_mix_weight_up.weight"], c.streams, c.rms_eps)

    def _inject(self, h: torch.Tensor, block: torch.Tensor, n: torch.Tensor, p: str) -> torch.Tensor:
        gates = sp.stream_injection(n, self.w[p + ".block_inject_weight.weight"], self.cfg.streams)
        return sp.stream_combine(h, block, gates)

    def _rot(self, x: torch.Tensor, pos3: torch.Tensor) -> torch.Tensor:
        return eager.rope3(x, pos3, self.inv_freq, self.cfg.mrope_section)

    def _table(self, base: str) -> torch.Tensor:
        t = self._tables.get(base)
        if t is None:
            t = torch.cat([self.w[f"{base}.shard_{i}.weight"] for i in range(self.cfg.ngram_split_parts)], 0)
            self._tables[base] = t
        return t

    def _ple(self, h: torch.Tensor, tokens: list[int], st: LayerState, p: str) -> torch.Tensor:
        c, w = self.cfg, self.w
        e = p + ".ple_embedding"
        hist = st.ngram_history if st.ngram_history is not None else [c.eos_token_id] * (c.ngram_size - 1)
        ids, st.ngram_history = ngram_hash_ids(tokens, hist, w[e + ".layer_multipliers"].tolist(),
                                               w[e + ".ngram_heads_vocab_sizes"].tolist(),
                                               w[e + ".ngram_heads_offsets"].tolist(), c.eos_token_id)
        emb = self._table(e + ".ngram_embedding")[torch.tensor(ids, dtype=torch.long)].flatten(-2)     # [T, embed]
        T = h.shape[0]
        key = sp.grouped_rms_norm(self._lin(emb, p + ".key_proj"), w[p + ".norm_key.weight"], c.hidden_size, c.rms_eps)
        query = sp.grouped_rms_norm(h, w[p + ".norm_query.weight"], c.hidden_size, c.rms_eps)
        gated = sp.signed_root_gate(key.view(T, c.streams, -1), query.view(T, c.streams, -1), self._lin(emb, p + ".value_proj"))
        conv_in = sp.grouped_rms_norm(gated, w[p + ".norm_conv.weight"], c.hidden_size, c.rms_eps)
        prev = st.ple_conv if st.ple_conv is not None else torch.zeros((c.ple_conv_kernel - 1) * c.ngram_size, c.stream_width)
        conv, st.ple_conv = dilated_causal_conv(conv_in, prev, w[p + ".conv1d.weight"], c.ngram_size)
        return h + (gated + conv)

    def _gdn(self, x: torch.Tensor, st: LayerState, p: str) -> torch.Tensor:
        c, w = self.cfg, self.w
        bf = torch.bfloat16
        qkv, st.conv = eager.gdn_conv(self._lin(x, p + ".in_proj_qkv").to(bf), w[p + ".conv1d.weight"].squeeze(1), st.conv)
        ba = torch.cat([self._lin(x, p + ".in_proj_b"), self._lin(x, p + ".in_proj_a")], -1)
        out, st.recurrent = eager.gdn_delta(qkv, self._lin(x, p + ".in_proj_z"), ba, w[p + ".A_log"], w[p + ".dt_bias"],
                                            w[p + ".norm.weight"], st.recurrent, c.gdn_k_heads, c.gdn_v_heads,
                                            eps_norm=c.rms_eps, d=c.gdn_k_dim, gate=c.gdn_output_gate)
        return self._lin(out.float(), p + ".out_proj")

    def _attention(self, x: torch.Tensor, st: LayerState, p: str, start: int, pos3: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        T, Hq, Hkv, D = x.shape[0], c.num_q_heads, c.num_kv_heads, c.head_dim
        qg = self._lin(x, p + ".q_proj").view(T, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:]
        q = self._rot(eager.rmsnorm(q, w[p + ".q_norm.weight"], c.rms_eps, True), pos3)
        k = self._rot(eager.rmsnorm(self._lin(x, p + ".k_proj").view(T, Hkv, D), w[p + ".k_norm.weight"], c.rms_eps, True), pos3)
        v = self._lin(x, p + ".v_proj").view(T, Hkv, D)
        st.key = k if st.key is None else torch.cat([st.key, k], 0)
        st.value = v if st.value is None else torch.cat([st.value, v], 0)
        st.positions = pos3 if st.positions is None else torch.cat([st.positions, pos3], 1)
        # indexer: per-head queries, ONE raw key per token; whole groups of raw keys are pooled once and kept
        iqk = self._lin(x, p + ".indexer.index_qk_proj")
        iq = iqk[:, :c.index_heads * c.index_dim].view(T, c.index_heads, c.index_dim)
        iq = self._rot(eager.rmsnorm(iq, w[p + ".indexer.q_layernorm.weight"], c.rms_eps, True), pos3)
        raw = iqk[:, c.index_heads * c.index_dim:]
        st.index_raw = raw if st.index_raw is None else torch.cat([st.index_raw, raw], 0)
        r = c.index_compression
        have = 0 if st.index_pooled is None else st.index_pooled.shape[0]
        full = st.index_raw.shape[0] // r
        if full > have:
            groups = st.index_raw[have * r:full * r].view(full - have, r, c.index_dim).mean(1)
            groups = eager.rmsnorm(groups, w[p + ".indexer.k_layernorm.weight"], c.rms_eps, True)
            first = torch.arange(have, full) * r                                   # a block sits at its first token
            groups = self._rot(groups[:, None, :], st.positions[:, first])[:, 0, :]
            st.index_pooled = groups if st.index_pooled is None else torch.cat([st.index_pooled, groups], 0)
        pooled = st.index_pooled if st.index_pooled is not None else torch.zeros(0, c.index_dim)
        visible = torch.arange(start + 1, start + T + 1)[None]
        chosen = sp.select_blocks(iq[None], pooled[None], visible, r, c.index_budget)
        out = sp.attend_selected(q.transpose(0, 1)[None], st.key.transpose(0, 1)[None], st.value.transpose(0, 1)[None], chosen)
        out = out[0].transpose(0, 1) * torch.sigmoid(gate)
        return self._lin(out.reshape(T, Hq * D), p + ".o_proj")

    def _mlp(self, x: torch.Tensor, p: str) -> torch.Tensor:
        c, w = self.cfg, self.w
        logits = self._lin(x, p + ".gate")
        order = torch.argsort(-logits, dim=-1, stable=True)[:, :c.experts_per_token]       # ties: the lower expert id
        sel = torch.gather(logits, 1, order)
        wt = torch.softmax(sel, -1) if c.norm_topk_prob else torch.softmax(logits, -1).gather(1, order)
        lo, hi = self.expert_range
        gu, dn, I = w[p + ".experts.gate_up_proj"], w[p + ".experts.down_proj"], c.moe_intermediate_size
        out = torch.zeros_like(x)
        for t in range(x.shape[0]):
            for j in range(c.experts_per_token):
                e = int(order[t, j])
                if lo <= e < hi:
                    a = gu[e] @ x[t]
                    out[t] += wt[t, j] * (dn[e] @ (F.silu(a[:I]) * a[I:]))
        if self.reduce_experts is not None:
            out = self.reduce_experts(out)
        if c.shared_intermediate_size:
            s = p + ".shared_expert"
            shared = self._lin(F.silu(self._lin(x, s + ".gate_proj")) * self._lin(x, s + ".up_proj"), s + ".down_proj")
            out = out + shared * torch.sigmoid(self._lin(x, p + ".shared_expert_gate"))
        return out

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, tokens: list[int], state: RequestState | None = None, positions3=None, embeds=None,
                last_only: bool = False) -> tuple[torch.Tensor, RequestState]:
        """Logits ``[T, vocab]`` (``[1, vocab]`` with ``last_only``) of ``tokens`` appended to ``state``.  ``embeds``:
        ``[(offset, rows)]`` feature rows that replace token embeddings; ``positions3``: int ``[3, T]`` (default: the
        sequence index on all axes).  The state object is updated in place and returned."""
        c = self.cfg
        tokens = [int(t) for t in tokens]
        if not tokens or min(tokens) < 0 or max(tokens) >= c.vocab_size:
            raise ValueError("a non-empty list of token ids inside the vocabulary")
        if state is None:
            state = RequestState()
        if not state.layers:
            state.layers = [LayerState() for _ in range(c.num_layers)]
        T, start = len(tokens), state.length
        if start + T > c.max_position:
            raise ValueError("the sequence leaves the model's context")
        pos3 = torch.arange(start, start + T)[None].expand(3, -1) if positions3 is None else \
            torch.as_tensor(np.asarray(positions3), dtype=torch.long)
        if pos3.shape != (3, T):
            raise ValueError("positions are [3, tokens]")
        x = self.w[f"{LM}.embed_tokens.weight"][torch.tensor(tokens)]
        for off, rows in (embeds or ()):                                              # encoder features replace embeddings
            x[off:off + rows.shape[0]] = rows.float()
        h = x.repeat(1, c.streams)                                                    # every stream starts as the embedding
        for i in range(c.num_layers):
            p, st = f"{LM}.layers.{i}", state.layers[i]
            if c.uses_ple(i):
                h = self._ple(h, tokens, st, p + ".ple")
            mixed, n = self._mix(h, p + ".attn_hyper_connection")
            block = self._gdn(mixed, st, p + ".linear_attn") if c.layer_is_gdn(i) else \
                self._attention(mixed, st, p + ".self_attn", start, pos3)
            h = self._inject(h, block, n, p + ".attn_hyper_connection")
            mixed, n = self._mix(h, p + ".mlp_hyper_connection")
            h = self._inject(h, self._mlp(mixed, p + ".mlp"), n, p + ".mlp_hyper_connection")
        state.length = start + T
        self.last_feedback = h                                        # the multi-stream residual before the final mixer
        mixed, _ = self._mix(h[-1:] if last_only else h, f"{LM}.hyper_connection_mixer")
        return self._lin(mixed, "lm_head"), state

    # ------------------------------------------------------------------ draft head
    @property
    def has_draft_head(self) -> bool:
        return "mtp.fc_hidden.weight" in self.w

    @torch.no_grad()
    def draft_forward(self, tokens: list[int], feedback: torch.Tensor, state: RequestState | None = None):
        """The draft head on ``tokens`` (token ``i + 1`` of the sequence) paired with ``feedback`` (the target's
        multi-stream residual at position ``i``, ``[T, S H]``): logits for token ``i + 2``, the head's own residual
        (the feedback of the next proposal) and its state (one attention layer).  The embedding is normalised and
        projected, every stream of the feedback is normalised over the whole multi-stream width and projected by the
        same matrix, and the sum enters one decoder layer; the head has no lexical embedding."""
        c, w = self.cfg, self.w
        if not self.has_draft_head:
            raise ValueError("the checkpoint carries no draft head")
        T = len(tokens)
        if feedback.shape != (T, c.stream_width):
            raise ValueError("one multi-stream residual row per token")
        state = state or RequestState()
        if not state.layers:
            state.layers = [LayerState()]
        start = state.length
        emb = w[f"{LM}.embed_tokens.weight"][torch.tensor([int(t) for t in tokens])]
        pe = self._lin(eager.rmsnorm(emb, w["mtp.pre_fc_norm_embedding.weight"], c.rms_eps, True), "mtp.fc_embedding")
        nf = eager.rmsnorm(feedback.float(), w["mtp.pre_fc_norm_hidden.weight"], c.rms_eps, True)
        ph = self._lin(nf.view(T, c.streams, c.hidden_size), "mtp.fc_hidden")
        h = (ph + pe[:, None, :]).flatten(-2)
        pos3 = torch.arange(start, start + T)[None].expand(3, -1)
        p, st = "mtp.layers.0", state.layers[0]
        mixed, n = self._mix(h, p + ".attn_hyper_connection")
        h = self._inject(h, self._attention(mixed, st, p + ".self_attn", start, pos3), n, p + ".attn_hyper_connection")
        mixed, n = self._mix(h, p + ".mlp_hyper_connection")
        h = self._inject(h, self._mlp(mixed, p + ".mlp"), n, p + ".mlp_hyper_connection")
        state.length = start + T
        mixed, _ = self._mix(h, "mtp.hyper_connection_mixer")
        return self._lin(mixed, "lm_head"), h, state


# ------------------------------------------------------------------ serving
def copy_state(state: RequestState) -> RequestState:
    """A state that can be advanced without touching ``state``: tensors are never written in place by the model, so the
    copy shares them; the n-gram history is a list and is copied."""
    return RequestState(state.length, [replace(l, ngram_history=None if l.ngram_history is None else list(l.ngram_history))
                                       for l in state.layers])


class Qwen4ExpEagerExecutor(StatefulEagerExecutor):
    """``execute(segments)`` of the engine on the eager model: one explicit state per request slot (a segment that
    starts at position 0 starts a fresh state; the state holds K / V, so pages are not used and there is no prefix
    sharing).  With ``speculative_depth`` > 0 and a checkpoint that carries the draft head, decode steps of greedy,
    unconstrained requests run as lossless draft / review rounds (``executor/stateful_executor.py``)."""

    def __init__(self, cfg: Qwen4ExpConfig, weights: Mapping[str, torch.Tensor], speculative_depth: int = 0) -> None:
        self.cfg = cfg
        super().__init__(Qwen4ExpModel(cfg, weights), speculative_depth)

    def _new_state(self) -> RequestState:
        return RequestState()

    def _copy(self, state: RequestState) -> RequestState:
        return copy_state(state)


def admit_qwen4_exp_checkpoint(path):
    """``(cfg, weights, store)`` of a checkpoint directory under the closed inventory: every text tensor of
    ``qwen4_exp_tensor_shapes`` present with its shape, the vision tower's tensors when the configuration has one, the
    draft head (``mtp.*``) whole when the checkpoint carries it, and nothing else."""
    from pathlib import Path

    from .checkpoint import CheckpointError, SafetensorsDirectory
    from .vision import vision_tensor_shapes
    path = Path(path)
    cfg = parse_qwen4_exp_config_json((path / "config.json").read_bytes())
    store = SafetensorsDirectory(path)
    nested = "model."                                   # the store reads ``model.language_model.X`` as ``model.X``
    want = {(nested + n[len(LM) + 1:] if n.startswith(LM + ".") else n): shape for n, shape in qwen4_exp_tensor_shapes(cfg).items()}
    claimed = set()
    for alias, shape in want.items():
        if alias not in store:
            raise CheckpointError(f"missing tensor {alias}")
        if tuple(store.tensors[alias].shape) != shape:
            raise CheckpointError(f"{alias}: shape {tuple(store.tensors[alias].shape)}, expected {shape}")
        claimed.add(alias)
    if cfg.vision is not None:
        for n, shape in vision_tensor_shapes(cfg.vision).items():
            full = "model.visual." + n
            if full not in store or tuple(store.tensors[full].shape) != shape:
                raise CheckpointError(f"missing or misshaped tensor {full}")
            claimed.add(full)
    head = {}
    if any(n.startswith("mtp.") for n in store.tensors):                # the draft head comes whole, with its shapes
        head = qwen4_exp_mtp_tensor_shapes(cfg)
        for n, shape in head.items():
            if n not in store or tuple(store.tensors[n].shape) != shape:
                raise CheckpointError(f"missing or misshaped tensor {n}")
            claimed.add(n)
    unowned = sorted(set(store.tensors) - claimed)
    if unowned:
        raise CheckpointError(f"checkpoint has {len(unowned)} tensors no logical weight owns, e.g. {unowned[:3]}")
    weights = {}
    for n in qwen4_exp_tensor_shapes(cfg):
        alias = nested + n[len(LM) + 1:] if n.startswith(LM + ".") else n
        weights[n] = store.get(alias)
    for n in head:
        weights[n] = store.get(n)
    return cfg, weights, store


def tiny_config(**kw) -> Qwen4ExpConfig:
    """A small instance of the family for tests and ``random:qwen4-exp-tiny``."""
    base = dict(
        vocab_size=320, hidden_size=32, num_layers=4,
        layer_types=("linear_attention", "full_attention", "linear_attention", "full_attention"), max_position=4096,
        rms_eps=1e-6, num_q_heads=4, num_kv_heads=2, head_dim=16, rotary_dim=8, rope_theta=10000.0, mrope_section=(2, 1, 1),
        gdn_k_heads=2, gdn_v_heads=4, gdn_k_dim=8, gdn_v_dim=8, gdn_conv_kernel=4, gdn_output_gate="sigmoid",
        num_experts=8, experts_per_token=2, moe_intermediate_size=16, shared_intermediate_size=16, norm_topk_prob=True,
        streams=4, stream_low_rank=8, index_heads=2, index_dim=16, index_budget=16, index_compression=4,
        ple_layer_ids=(2,), ple_embed_dim=32, ple_conv_kernel=4, ngram_size=3, heads_per_ngram=2, ngram_vocab_base=500,
        ngram_vocab_multiple=4, ngram_split_parts=4, ngram_shard_rows=512, eos_token_id=1, name="qwen4-exp-tiny")
    base.update(kw)
    cfg = Qwen4ExpConfig(**base)
    cfg.validate()
    return cfg
