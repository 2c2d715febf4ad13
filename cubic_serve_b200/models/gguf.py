"""GGUF file inventory and logical weight views (reference: ``models/gguf.py:172``, ``models/gguf_weights.py:433``)."""
from __future__ import annotations

import math

from pathlib import Path

import numpy as np

from ..quantization import gguf as gq

# llama.cpp tensor names -> HuggingFace-style module names used by the runner
NAME_MAP = {"attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
            "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj",
            "ffn_down": "mlp.down_proj", "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm",
            "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm"}


def hf_name(gguf_name: str) -> str:
    if gguf_name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if gguf_name == "output_norm.weight":
        return "model.norm.weight"
    if gguf_name == "output.weight":
        return "lm_head.weight"
    if gguf_name == "rope_freqs.weight":
        return gguf_name                   # precomputed rotary scaling factors of some exporters: carried, not used
    parts = gguf_name.split(".")
    if parts[0] == "blk" and len(parts) == 4 and parts[2] in NAME_MAP:
        return f"model.layers.{parts[1]}.{NAME_MAP[parts[2]]}.{parts[3]}"
    raise gq.GGUFFormatError(f"unrecognised GGUF tensor {gguf_name}")


def inspect_gguf(path: str | Path) -> dict:
    import gguf
    reader = gguf.GGUFReader(str(path))
    types: dict[str, int] = {}
    rejected = []
    for t in reader.tensors:
        name = t.tensor_type.name
        types[name] = types.get(name, 0) + 1
        if name not in gq.ADMITTED:
            rejected.append(t.name)
    arch = None
    f = reader.fields.get("general.architecture")
    if f is not None:
        arch = bytes(f.parts[-1]).decode("utf-8", errors="replace")
    info = {"file": str(path), "architecture": arch, "tensors": len(reader.tensors), "types": types,
            "admitted": not rejected, "rejected": rejected[:8]}
    try:
        cfg = config_from_gguf(reader)
        info.update(model=cfg.name, layers=cfg.num_layers, hidden=cfg.hidden_size, vocab=cfg.vocab_size,
                    heads=f"{cfg.num_q_heads}q/{cfg.num_kv_heads}kv x {cfg.head_dim}", intermediate=cfg.intermediate_size,
                    rope_theta=cfg.rope_theta, qk_norm=cfg.qk_norm, tied_embeddings=cfg.tie_embeddings,
                    qk_rows_unpermuted=arch in PERMUTED_QK_ARCHITECTURES, served=not rejected)
    except gq.GGUFFormatError as exc:
        info.update(served=False, reason=str(exc))
    return info


def load_gguf_tensors(path: str | Path):
    """Yield ``(hf name, GGML type name, logical shape, raw ndarray)`` for every tensor (closed inventory)."""
    import gguf
    reader = gguf.GGUFReader(str(path))
    for t in reader.tensors:
        tname = t.tensor_type.name
        if tname not in gq.ADMITTED:
            raise gq.GGUFFormatError(f"{t.name}: GGML type {tname} is not admitted")
        shape = tuple(int(x) for x in reversed(t.shape))            # GGUF stores dims innermost-first
        yield hf_name(t.name), tname, shape, np.asarray(t.data)


# ------------------------------------------------------------------ metadata -> architecture
def _field(reader, key: str, default=None):
    f = reader.fields.get(key)
    if f is None:
        return default
    v = f.contents() if hasattr(f, "contents") else None
    if v is None:
        part = f.parts[f.data[0]] if len(f.data) else f.parts[-1]
        v = bytes(part).decode("utf-8", errors="replace") if part.dtype == np.uint8 and len(part) > 1 else part.tolist()
        if isinstance(v, list) and len(v) == 1:
            v = v[0]
    return v


# exporters of these architectures store the query / key projection rows in the interleaved-pair rotary order
# (``permute`` of llama.cpp's converter); the kernels use the half-rotated order of the original checkpoints
PERMUTED_QK_ARCHITECTURES = ("llama", "mistral")


def config_from_gguf(reader):
    """``ModelConfig`` of a GGUF file's decoder (llama-family architectures: llama, mistral, qwen2, qwen3)."""
    from .config import ModelConfig, QuantSpec
    arch = _field(reader, "general.architecture")
    if arch not in ("llama", "mistral", "qwen2", "qwen3"):
        raise gq.GGUFFormatError(f"GGUF architecture {arch!r} is not served")
    names = {t.name for t in reader.tensors}
    shapes = {t.name: tuple(int(x) for x in reversed(t.shape)) for t in reader.tensors}

    def need(key):
        v = _field(reader, f"{arch}.{key}")
        if v is None:
            raise gq.GGUFFormatError(f"GGUF metadata lacks {arch}.{key}")
        return v

    layers, hidden, hq = int(need("block_count")), int(need("embedding_length")), int(need("attention.head_count"))
    hkv = int(_field(reader, f"{arch}.attention.head_count_kv", hq))
    head_dim = int(_field(reader, f"{arch}.attention.key_length", hidden // hq))
    vocab = shapes["token_embd.weight"][0]
    types = {t.tensor_type.name for t in reader.tensors if t.name.endswith(("attn_q.weight", "ffn_down.weight"))}
    # rotary scaling: a per-slot divisor table (the exporter's form of the llama3 rule) or the linear / yarn metadata
    scaling = None
    kind = str(_field(reader, f"{arch}.rope.scaling.type", "none") or "none")
    factor = float(_field(reader, f"{arch}.rope.scaling.factor", 1.0) or 1.0)
    table = next((t for t in reader.tensors if t.name == "rope_freqs.weight"), None)
    if table is not None:
        if kind not in ("none", "linear") or (kind == "linear" and factor != 1.0):
            raise gq.GGUFFormatError("a GGUF file with both a rotary divisor table and rotary scaling metadata is not served")
        scaling = ("factors", tuple(float(v) for v in np.asarray(table.data, dtype=np.float32).reshape(-1)))
        if len(scaling[1]) != head_dim // 2:
            raise gq.GGUFFormatError("rope_freqs.weight does not hold one divisor per rotary slot")
    elif kind == "linear" and factor != 1.0:
        scaling = ("linear", factor)
    elif kind == "yarn":
        original = int(need("rope.scaling.original_context_length"))
        scaling = ("yarn", factor, original, 32.0, 1.0, 1.0 if factor <= 1 else 0.1 * math.log(factor) + 1.0)
    elif kind not in ("none", "linear"):
        raise gq.GGUFFormatError(f"rotary scaling of type {kind!r} is not served")
    return ModelConfig(rope_scaling=scaling, 
        name=str(_field(reader, "general.name", Path(str(getattr(reader, "path", "gguf"))).stem)), family="gqa_decoder",
        num_layers=layers, hidden_size=hidden, num_q_heads=hq, num_kv_heads=hkv, head_dim=head_dim,
        intermediate_size=int(need("feed_forward_length")), vocab_size=vocab,
        rope_theta=float(_field(reader, f"{arch}.rope.freq_base", 10000.0)),
        rms_eps=float(_field(reader, f"{arch}.attention.layer_norm_rms_epsilon", 1e-6)),
        max_position=int(_field(reader, f"{arch}.context_length", 8192)),
        qk_norm="blk.0.attn_q_norm.weight" in names, tie_embeddings="output.weight" not in names,
        quant=QuantSpec("gguf", 4 if types == {"Q4_K"} else 16, 32))


def qk_unpermute_order(rows: int, heads: int) -> np.ndarray:
    """Row order that undoes the converter's ``permute``: stored row ``order[i]`` is logical row ``i``.

    The converter reshapes a head's rows ``[2, d/2]`` -> ``[d/2, 2]`` (the two rotary halves interleaved); logical row
    ``h d + j`` (half ``j // (d/2)``, index ``j % (d/2)``) therefore sits at stored row ``h d + 2 (j % (d/2)) + j // (d/2)``."""
    d = rows // heads
    j = np.arange(d)
    within = 2 * (j % (d // 2)) + j // (d // 2)
    return (np.arange(heads)[:, None] * d + within[None, :]).reshape(-1)


class _View:
    """One logical weight of the file: rows may be re-ordered (exporter permutation undone) and sliced."""

    def __init__(self, type_name: str, shape, raw) -> None:
        self.type, self.shape = type_name, tuple(shape)
        n = self.shape[0]
        self.raw = np.ascontiguousarray(raw).reshape(n, -1) if len(self.shape) == 2 else np.asarray(raw)

    def rows(self, index) -> "_View":
        """Row selection works on the stored blocks: every GGML block type quantizes within a row."""
        raw = self.raw[index]
        return _View(self.type, (raw.shape[0], self.shape[1]), raw)

    def dense(self) -> np.ndarray:
        if len(self.shape) == 1:                          # norm weights and other vectors: one row
            return gq.dense(self.type, np.asarray(self.raw).reshape(1, -1), (1, self.shape[0])).reshape(-1)
        return gq.dense(self.type, self.raw, self.shape)

    def triple(self):
        return gq.q4k_decode(self.raw)


def _fuse(views: list[_View], cols: slice | None = None):
    """Several weights with the same K stacked along N as one GEMM operand: natively as affine 4-bit when all parts are
    Q4_K (codes, scales and offsets are concatenated, nothing is re-quantized), else decoded to bf16.  ``cols``
    restricts K (a multiple of 256 on both ends keeps whole super-blocks)."""
    from ..ops import wq_pack
    import torch
    if all(v.type == "Q4_K" for v in views):
        parts = [v.triple() for v in views]
        codes, scale, offset = (np.concatenate([p[i] for p in parts]) for i in range(3))
        if cols is not None:
            codes, scale, offset = codes[:, cols], scale[:, cols.start // 32:cols.stop // 32], offset[:, cols.start // 32:cols.stop // 32]
        return wq_pack.pack_affine4(torch.from_numpy(np.ascontiguousarray(codes)), torch.from_numpy(np.ascontiguousarray(scale)),
                                    torch.from_numpy(np.ascontiguousarray(offset)), 32)
    dense = np.concatenate([v.dense() for v in views])
    if cols is not None:
        dense = dense[:, cols]
    return wq_pack.pack_bf16(torch.from_numpy(np.ascontiguousarray(dense)))


def load_gguf_decoder_weights(path: str | Path, device="cpu", tp_rank: int = 0, tp_size: int = 1,
                              layer_range: tuple[int, int] | None = None):
    """``(ModelConfig, DecoderWeights)`` of a GGUF file, rank-local for tensor parallelism.

    Q4_K projections stay 4-bit (affine codes with the file's own scales and minima, group 32); other admitted block
    types are decoded to bf16.  Query / key rows of architectures whose exporter interleaves the rotary halves are put
    back into the half-rotated order.  The inventory is closed: an unknown tensor name or block type is an error."""
    import gguf
    import torch
    from .decoder import DecoderWeights, LayerWeights
    from .parallel_weights import AxisSpan
    reader = gguf.GGUFReader(str(path))
    cfg = config_from_gguf(reader)
    arch = _field(reader, "general.architecture")
    views: dict[str, _View] = {}
    for name, tname, shape, raw in load_gguf_tensors(path):
        views[name] = _View(tname, shape, raw)
    bf = torch.bfloat16
    D = cfg.head_dim
    qh = AxisSpan.shard(cfg.num_q_heads, tp_rank, tp_size, what="query heads").scaled(D)
    kvh = AxisSpan.shard(cfg.num_kv_heads, tp_rank, tp_size, what="key/value heads").scaled(D)
    inter = AxisSpan.shard(cfg.intermediate_size, tp_rank, tp_size, 256, "intermediate size")
    q_order = k_order = None
    if arch in PERMUTED_QK_ARCHITECTURES:
        q_order, k_order = qk_unpermute_order(cfg.q_size, cfg.num_q_heads), qk_unpermute_order(cfg.kv_size, cfg.num_kv_heads)

    def vec(name: str) -> "torch.Tensor":
        return torch.from_numpy(views[name].dense().reshape(-1).copy()).to(device, bf)

    def rows(name: str, span: AxisSpan, order=None) -> _View:
        index = np.arange(span.start, span.stop) if order is None else order[span.start:span.stop]
        return views[name].rows(index)

    used = {"model.embed_tokens.weight", "model.norm.weight"}
    layers = []
    for i in range(*(layer_range or (0, cfg.num_layers))):
        p = f"model.layers.{i}"
        names = {k: f"{p}.{v}.weight" for k, v in NAME_MAP.items()}
        qkv = _fuse([rows(names["attn_q"], qh, q_order), rows(names["attn_k"], kvh, k_order), rows(names["attn_v"], kvh)])
        o = _fuse([views[names["attn_output"]]], slice(qh.start, qh.stop))
        gate_up = _fuse([rows(names["ffn_gate"], inter), rows(names["ffn_up"], inter)])
        down = _fuse([views[names["ffn_down"]]], slice(inter.start, inter.stop))
        lw = LayerWeights(ln1=vec(names["attn_norm"]), ln2=vec(names["ffn_norm"]), qkv=qkv.to(device), o=o.to(device),
                          gate_up=gate_up.to(device), down=down.to(device))
        used |= {names[k] for k in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down",
                                     "attn_norm", "ffn_norm")}
        if cfg.qk_norm:
            lw.q_norm, lw.k_norm = vec(names["attn_q_norm"]), vec(names["attn_k_norm"])
            used |= {names["attn_q_norm"], names["attn_k_norm"]}
        layers.append(lw)
    if layer_range is None:
        ignorable = {n for n in views if n.endswith("rope_freqs.weight")}
        extra = set(views) - used - {"lm_head.weight"} - ignorable
        if extra:
            raise gq.GGUFFormatError(f"GGUF file has tensors no logical weight owns: {sorted(extra)[:4]}")
    embed_full = torch.from_numpy(views["model.embed_tokens.weight"].dense()).to(device, bf)
    vocab = AxisSpan.shard(cfg.vocab_size, tp_rank, tp_size, what="vocabulary")
    head = embed_full if cfg.tie_embeddings else torch.from_numpy(views["lm_head.weight"].dense()).to(device, bf)
    from ..ops import wq_pack
    weights = DecoderWeights(embed=embed_full[vocab.slice()], layers=layers, final_norm=vec("model.norm.weight"),
                             lm_head=wq_pack.pack_bf16(head[vocab.slice()].contiguous()), vocab_start=vocab.start,
                             extras={"embed_full": embed_full})
    return cfg, weights
