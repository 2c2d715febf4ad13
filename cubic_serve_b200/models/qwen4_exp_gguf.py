"""GGUF files of the ``qwen4exp`` architecture <-> the logical tensors of ``models/qwen4_exp.py``.

The exporter of that architecture changes names, merges and splits tensors and stores some values in another
convention; a loader has to undo exactly that, nothing else.  The conventions, stated once:

* names: ``token_embd``, ``output``, ``output_hc_{down,up,norm}``, ``blk.<i>.`` + the table below, the two stream
  mixers of a layer as ``hc_attn_*`` / ``hc_ffn_*``;
* experts are stacked per projection (``ffn_{gate,up,down}_exps``: ``[E, rows, cols]``); the logical gate / up pair is
  one ``[E, 2 I, H]`` tensor;
* the indexer's query and key projections are two tensors (logical: one, queries first);
* zero-centred norm weights are stored as ``1 + w`` (all norms except the Gated DeltaNet output norm and the three
  group norms of the lexical block);
* the Gated DeltaNet decay is stored as ``-exp(A_log)``;
* Gated DeltaNet value heads are stored ``[value head within its key head, key head]``-major, the logical order is
  ``[key head, value head within it]``: rows of ``in_proj_qkv`` (value part), ``conv1d`` (value part), ``in_proj_z``,
  ``in_proj_a / b``, ``A_log``, ``dt_bias`` and the columns of ``out_proj`` are regrouped;
* the lexical table is ONE tensor (``per_layer_token_embd``), its hash metadata are key / value arrays of the file.

``export_qwen4_exp_gguf`` writes that layout (tests, conversions), ``load_qwen4_exp_gguf`` reads it back into
``(config, logical tensors)`` for the eager model.  The vision tower and the draft head live in files of their own in
that format and are not read here.

Reference counterpart: ``models/qwen4_exp/gguf.py`` there (declarations that undo the exporter at weight loading).
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from ..quantization import gguf as gq
from .qwen4_exp import LM, Qwen4ExpConfig, Qwen4ExpConfigError, qwen4_exp_tensor_shapes

ARCH = "qwen4exp"

LAYER_NAMES = {
    "linear_attn.A_log": "ssm_a", "linear_attn.conv1d.weight": "ssm_conv1d.weight", "linear_attn.dt_bias": "ssm_dt.bias",
    "linear_attn.in_proj_a.weight": "ssm_alpha.weight", "linear_attn.in_proj_b.weight": "ssm_beta.weight",
    "linear_attn.in_proj_qkv.weight": "attn_qkv.weight", "linear_attn.in_proj_z.weight": "attn_gate.weight",
    "linear_attn.norm.weight": "ssm_norm.weight", "linear_attn.out_proj.weight": "ssm_out.weight",
    "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
    "self_attn.indexer.q_layernorm.weight": "indexer.q_norm.weight",
    "self_attn.indexer.k_layernorm.weight": "indexer.k_norm.weight",
    "mlp.gate.weight": "ffn_gate_inp.weight", "mlp.shared_expert_gate.weight": "ffn_gate_inp_shexp.weight",
    "mlp.shared_expert.gate_proj.weight": "ffn_gate_shexp.weight", "mlp.shared_expert.up_proj.weight": "ffn_up_shexp.weight",
    "mlp.shared_expert.down_proj.weight": "ffn_down_shexp.weight",
    "ple.conv1d.weight": "ple_conv1d.weight", "ple.key_proj.weight": "ple_key.weight", "ple.value_proj.weight": "ple_value.weight",
    "ple.norm_conv.weight": "ple_norm_conv.weight", "ple.norm_key.weight": "ple_norm_key.weight",
    "ple.norm_query.weight": "ple_norm_query.weight",
}
MIXER_NAMES = {"input_mix_weight_down.weight": "down.weight", "input_mix_weight_up.weight": "up.weight",
               "hc_norm.weight": "norm.weight", "block_inject_weight.weight": "inject.weight"}


def _stored_plus_one(member: str) -> bool:
    return member.endswith("norm.weight") and member != "linear_attn.norm.weight"


def value_head_order(key_heads: int, value_heads: int, width: int) -> np.ndarray:
    """Indices that gather the stored order ``[value within key, key, width]`` into the logical ``[key, value within
    key, width]``."""
    per = value_heads // key_heads
    k, v, d = np.meshgrid(np.arange(key_heads), np.arange(per), np.arange(width), indexing="ij")
    return ((v * key_heads + k) * width + d).reshape(-1)


def _orders(cfg: Qwen4ExpConfig):
    heads = value_head_order(cfg.gdn_k_heads, cfg.gdn_v_heads, 1)
    values = value_head_order(cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_v_dim)
    qk = 2 * cfg.gdn_k_heads * cfg.gdn_k_dim
    return heads, values, np.concatenate([np.arange(qk), qk + values])


def _physical(member: str) -> tuple[str | None, str | None]:
    """``(stored name, special)`` of a layer member; ``special`` names what needs more than a rename."""
    for kind, tag in (("attn_hyper_connection.", "hc_attn_"), ("mlp_hyper_connection.", "hc_ffn_")):
        if member.startswith(kind):
            return tag + MIXER_NAMES[member[len(kind):]], None
    if member in ("mlp.experts.gate_up_proj", "mlp.experts.down_proj", "self_attn.indexer.index_qk_proj.weight") \
            or member.startswith("ple.ple_embedding."):
        return None, member
    return LAYER_NAMES.get(member), None


# ------------------------------------------------------------------ export
def export_qwen4_exp_gguf(path: str | Path, cfg: Qwen4ExpConfig, weights: dict[str, torch.Tensor]) -> Path:
    """Write ``weights`` (the logical tensors, without a draft head) in the exporter's layout, all tensors F32."""
    import gguf
    if len(cfg.ple_layer_ids) > 1:
        raise Qwen4ExpConfigError("the file format holds one lexical table")
    w = gguf.GGUFWriter(str(path), ARCH)
    A = f"{ARCH}."
    w.add_uint32(A + "block_count", cfg.num_layers)
    w.add_uint32(A + "context_length", cfg.max_position)
    w.add_uint32(A + "embedding_length", cfg.hidden_size)
    w.add_uint32(A + "attention.head_count", cfg.num_q_heads)
    w.add_uint32(A + "attention.head_count_kv", cfg.num_kv_heads)
    w.add_uint32(A + "attention.key_length", cfg.head_dim)
    w.add_uint32(A + "attention.value_length", cfg.head_dim)
    w.add_float32(A + "attention.layer_norm_rms_epsilon", cfg.rms_eps)
    w.add_array(A + "rope.dimension_sections", [*cfg.mrope_section, 0])
    w.add_float32(A + "rope.freq_base", cfg.rope_theta)
    w.add_uint32(A + "rope.dimension_count", cfg.rotary_dim)
    w.add_uint32(A + "expert_count", cfg.num_experts)
    w.add_uint32(A + "expert_used_count", cfg.experts_per_token)
    w.add_uint32(A + "expert_feed_forward_length", cfg.moe_intermediate_size)
    w.add_uint32(A + "expert_shared_feed_forward_length", cfg.shared_intermediate_size)
    w.add_uint32(A + "ssm.conv_kernel", cfg.gdn_conv_kernel)
    w.add_uint32(A + "ssm.state_size", cfg.gdn_k_dim)
    w.add_uint32(A + "ssm.group_count", cfg.gdn_k_heads)
    w.add_uint32(A + "ssm.time_step_rank", cfg.gdn_v_heads)
    w.add_uint32(A + "ssm.inner_size", cfg.gdn_v_heads * cfg.gdn_v_dim)
    w.add_uint32(A + "hyper_connection.count", cfg.streams)
    w.add_uint32(A + "hyper_connection.low_rank", cfg.stream_low_rank)
    w.add_uint32(A + "attention.indexer.head_count", cfg.index_heads)
    w.add_uint32(A + "attention.indexer.key_length", cfg.index_dim)
    w.add_uint32(A + "attention.indexer.top_k", cfg.index_budget)
    w.add_array(A + "attention.compress_ratios", [0 if cfg.layer_is_gdn(i) else cfg.index_compression
                                                  for i in range(cfg.num_layers)])
    if cfg.ple_layer_ids:
        w.add_array(A + "ple.layers", [i - 1 for i in cfg.ple_layer_ids])
        w.add_uint32(A + "ple.ngram_size", cfg.ngram_size)
        w.add_uint32(A + "ple.heads_per_ngram", cfg.heads_per_ngram)
        w.add_uint32(A + "ple.conv_kernel", cfg.ple_conv_kernel)
        w.add_uint32(A + "ple.eos_token_id", cfg.eos_token_id)
        w.add_uint32(A + "embedding_length_per_layer_input", cfg.ple_embed_dim // cfg.ngram_heads)
    heads, values, qkv = _orders(cfg)
    inv = lambda order: np.argsort(order)                                       # noqa: E731  logical -> stored

    def put(name: str, t: torch.Tensor) -> None:
        w.add_tensor(name, np.ascontiguousarray(t.detach().float().numpy()))
    put("token_embd.weight", weights[f"{LM}.embed_tokens.weight"])
    put("output.weight", weights["lm_head.weight"])
    for member, short in MIXER_NAMES.items():
        if member.startswith("block_inject"):
            continue
        t = weights[f"{LM}.hyper_connection_mixer.{member}"]
        put("output_hc_" + short, t + 1 if member == "hc_norm.weight" else t)
    for name, t in weights.items():
        if not name.startswith(f"{LM}.layers."):
            continue
        i, member = name[len(f"{LM}.layers."):].split(".", 1)
        stored, special = _physical(member)
        pre = f"blk.{i}."
        if special == "mlp.experts.gate_up_proj":
            I = cfg.moe_intermediate_size
            put(pre + "ffn_gate_exps.weight", t[:, :I])
            put(pre + "ffn_up_exps.weight", t[:, I:])
        elif special == "mlp.experts.down_proj":
            put(pre + "ffn_down_exps.weight", t)
        elif special == "self_attn.indexer.index_qk_proj.weight":
            n = cfg.index_heads * cfg.index_dim
            put(pre + "indexer.q_proj.weight", t[:n])
            put(pre + "indexer.k_proj.weight", t[n:])
        elif special is not None:                                                # the lexical embedding's members
            leaf = member.split(".ple_embedding.", 1)[1]
            if leaf.startswith("ngram_embedding.shard_"):
                if leaf == "ngram_embedding.shard_0.weight":
                    table = torch.cat([weights[f"{LM}.layers.{i}.ple.ple_embedding.ngram_embedding.shard_{p}.weight"]
                                       for p in range(cfg.ngram_split_parts)])
                    put("per_layer_token_embd.weight", table)
            else:
                key = {"layer_multipliers": "layer_multipliers", "ngram_heads_offsets": "head_offsets",
                       "ngram_heads_vocab_sizes": "head_vocab_sizes"}[leaf]
                w.add_key_value(A + "ple." + key, [int(v) for v in t.tolist()], gguf.GGUFValueType.ARRAY,
                                sub_type=gguf.GGUFValueType.INT64)        # the hash multipliers need 64 bits
        elif stored is None:
            raise Qwen4ExpConfigError(f"no stored name for {name}")
        else:
            if member == "linear_attn.A_log":
                t = -torch.exp(t.float())
            if _stored_plus_one(member):
                t = t + 1
            if member in ("linear_attn.in_proj_qkv.weight", "linear_attn.conv1d.weight"):
                t = t[inv(qkv)]
            elif member == "linear_attn.in_proj_z.weight":
                t = t[inv(values)]
            elif member == "linear_attn.out_proj.weight":
                t = t[:, inv(values)]
            elif member in ("linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.in_proj_a.weight",
                            "linear_attn.in_proj_b.weight"):
                t = t[inv(heads)]
            put(pre + stored, t)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return Path(path)


# ------------------------------------------------------------------ import
def _meta(reader, key: str):
    f = reader.fields.get(f"{ARCH}.{key}")
    if f is None:
        raise Qwen4ExpConfigError(f"the file lacks {ARCH}.{key}")
    vals = [f.parts[i] for i in f.data]
    out = [v.tolist() for v in vals]
    flat = [x for v in out for x in (v if isinstance(v, list) else [v])]
    return flat if len(f.data) > 1 or (f.types and f.types[0].name == "ARRAY") else flat[0]


def config_from_qwen4_exp_gguf(reader, vocab_size: int, table_rows: int) -> Qwen4ExpConfig:
    arch = reader.fields.get("general.architecture")
    if arch is None or bytes(arch.parts[arch.data[0]]).decode() != ARCH:
        raise Qwen4ExpConfigError(f"the file's architecture is not {ARCH}")
    ratios = [int(v) for v in _meta(reader, "attention.compress_ratios")]
    sections = [int(v) for v in _meta(reader, "rope.dimension_sections")][:3]
    has_ple = f"{ARCH}.ple.layers" in reader.fields
    hidden, heads_ng = int(_meta(reader, "embedding_length")), 0
    ple = {}
    if has_ple:
        layers = _meta(reader, "ple.layers")
        layers = layers if isinstance(layers, list) else [layers]
        ngram, per = int(_meta(reader, "ple.ngram_size")), int(_meta(reader, "ple.heads_per_ngram"))
        heads_ng = (ngram - 1) * per
        ple = dict(ple_layer_ids=tuple(int(i) + 1 for i in layers), ngram_size=ngram, heads_per_ngram=per,
                   ple_conv_kernel=int(_meta(reader, "ple.conv_kernel")), eos_token_id=int(_meta(reader, "ple.eos_token_id")),
                   ple_embed_dim=int(_meta(reader, "embedding_length_per_layer_input")) * heads_ng,
                   ngram_split_parts=1, ngram_shard_rows=table_rows)
    cfg = Qwen4ExpConfig(
        vocab_size=vocab_size, hidden_size=hidden, num_layers=int(_meta(reader, "block_count")),
        layer_types=tuple("full_attention" if r else "linear_attention" for r in ratios),
        max_position=int(_meta(reader, "context_length")), rms_eps=float(_meta(reader, "attention.layer_norm_rms_epsilon")),
        num_q_heads=int(_meta(reader, "attention.head_count")), num_kv_heads=int(_meta(reader, "attention.head_count_kv")),
        head_dim=int(_meta(reader, "attention.key_length")), rotary_dim=int(_meta(reader, "rope.dimension_count")),
        rope_theta=float(_meta(reader, "rope.freq_base")), mrope_section=tuple(sections),
        gdn_k_heads=int(_meta(reader, "ssm.group_count")), gdn_v_heads=int(_meta(reader, "ssm.time_step_rank")),
        gdn_k_dim=int(_meta(reader, "ssm.state_size")),
        gdn_v_dim=int(_meta(reader, "ssm.inner_size")) // int(_meta(reader, "ssm.time_step_rank")),
        gdn_conv_kernel=int(_meta(reader, "ssm.conv_kernel")), gdn_output_gate="sigmoid",
        num_experts=int(_meta(reader, "expert_count")), experts_per_token=int(_meta(reader, "expert_used_count")),
        moe_intermediate_size=int(_meta(reader, "expert_feed_forward_length")),
        shared_intermediate_size=int(_meta(reader, "expert_shared_feed_forward_length")), norm_topk_prob=True,
        streams=int(_meta(reader, "hyper_connection.count")), stream_low_rank=int(_meta(reader, "hyper_connection.low_rank")),
        index_heads=int(_meta(reader, "attention.indexer.head_count")), index_dim=int(_meta(reader, "attention.indexer.key_length")),
        index_budget=int(_meta(reader, "attention.indexer.top_k")), index_compression=max(ratios),
        ngram_vocab_base=0, ngram_vocab_multiple=1,
        **(ple or dict(ple_layer_ids=(), ple_embed_dim=hidden, ple_conv_kernel=4, ngram_size=3, heads_per_ngram=1,
                       ngram_split_parts=1)), name=ARCH)
    cfg.validate()
    return cfg


def load_qwen4_exp_gguf(path: str | Path) -> tuple[Qwen4ExpConfig, dict[str, torch.Tensor]]:
    """``(config, logical tensors)`` of a main-model file; every tensor is decoded to fp32 and the exporter's
    conventions are undone.  Unknown tensors and missing ones are refused."""
    import gguf
    reader = gguf.GGUFReader(str(path))
    stored = {}
    for t in reader.tensors:
        tname = t.tensor_type.name
        if tname not in gq.ADMITTED:
            raise gq.GGUFFormatError(f"{t.name}: GGML type {tname} is not admitted")
        shape = tuple(int(x) for x in reversed(t.shape))
        rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        stored[t.name] = torch.from_numpy(gq.dense(tname, np.asarray(t.data), (rows, shape[-1]))).reshape(shape)
    if "token_embd.weight" not in stored:
        raise Qwen4ExpConfigError("the file has no token embedding")
    table = stored.get("per_layer_token_embd.weight")
    cfg = config_from_qwen4_exp_gguf(reader, stored["token_embd.weight"].shape[0], 0 if table is None else table.shape[0])
    heads, values, qkv = _orders(cfg)
    used: set[str] = set()

    def take(name: str) -> torch.Tensor:
        if name not in stored:
            raise Qwen4ExpConfigError(f"missing tensor {name}")
        used.add(name)
        return stored[name]
    out: dict[str, torch.Tensor] = {}
    for name, shape in qwen4_exp_tensor_shapes(cfg).items():
        if name == f"{LM}.embed_tokens.weight":
            t = take("token_embd.weight")
        elif name == "lm_head.weight":
            t = take("output.weight")
        elif name.startswith(f"{LM}.hyper_connection_mixer."):
            member = name[len(f"{LM}.hyper_connection_mixer."):]
            t = take("output_hc_" + MIXER_NAMES[member])
            t = t - 1 if member == "hc_norm.weight" else t
        else:
            i, member = name[len(f"{LM}.layers."):].split(".", 1)
            pre = f"blk.{i}."
            phys, special = _physical(member)
            if special == "mlp.experts.gate_up_proj":
                t = torch.cat([take(pre + "ffn_gate_exps.weight"), take(pre + "ffn_up_exps.weight")], 1)
            elif special == "mlp.experts.down_proj":
                t = take(pre + "ffn_down_exps.weight")
            elif special == "self_attn.indexer.index_qk_proj.weight":
                t = torch.cat([take(pre + "indexer.q_proj.weight"), take(pre + "indexer.k_proj.weight")])
            elif special is not None:
                leaf = member.split(".ple_embedding.", 1)[1]
                if leaf.startswith("ngram_embedding."):
                    t = take("per_layer_token_embd.weight")
                else:
                    key = {"layer_multipliers": "layer_multipliers", "ngram_heads_offsets": "head_offsets",
                           "ngram_heads_vocab_sizes": "head_vocab_sizes"}[leaf]
                    v = _meta(reader, "ple." + key)
                    t = torch.tensor(v if isinstance(v, list) else [v], dtype=torch.int64)
            elif phys is None:
                raise Qwen4ExpConfigError(f"no stored name for {name}")
            else:
                t = take(pre + phys)
                if member in ("linear_attn.in_proj_qkv.weight", "linear_attn.conv1d.weight"):
                    t = t.reshape(len(qkv), -1)[qkv]
                elif member == "linear_attn.in_proj_z.weight":
                    t = t[values]
                elif member == "linear_attn.out_proj.weight":
                    t = t[:, values]
                elif member in ("linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.in_proj_a.weight",
                                "linear_attn.in_proj_b.weight"):
                    t = t[heads]
                if member == "linear_attn.A_log":
                    if not bool((t < 0).all()):
                        raise Qwen4ExpConfigError("the stored decay must be negative")
                    t = torch.log(-t)
                if _stored_plus_one(member):
                    t = t - 1
        if tuple(t.shape) != shape:
            t = t.reshape(shape)                                     # 1-D and 3-D tensors come back in their stored rank
        out[name] = t.contiguous()
    unknown = sorted(set(stored) - used)
    if unknown:
        raise Qwen4ExpConfigError(f"the file has {len(unknown)} tensors no logical weight owns, e.g. {unknown[:3]}")
    return cfg, out
