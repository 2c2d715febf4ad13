"""Checkpoint admission: HF-style safetensors directories (all weight formats) and GGUF files.

Counterpart of the reference's ``inspect_checkpoint`` (``models/checkpoint.py:1010``),
``CheckpointWeights.admit`` (``models/quantized_checkpoint.py:207``) and the GGUF readers
(``models/gguf.py:172``, ``models/gguf_weights.py:433``).  The inventory is *closed*: every tensor in the
shards must be claimed by exactly one logical weight, otherwise admission fails.  A logical linear weight
``<module>.weight`` of a quantized checkpoint is stored as payload tensors named ``<module>.<suffix>``.

``load_decoder_weights`` turns an admitted checkpoint into rank-local ``DecoderWeights`` (tensor-parallel
slices taken on whole heads / whole scale groups) ready for the native runner; ``write_random_checkpoint``
produces a random-init checkpoint in any format with exactly that on-disk layout (used by tests and benchmarks,
there being no network to fetch real ones).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from pathlib import Path

import torch

from ..ops import wq_pack
from ..quantization import cubic, formats, registry
from .config import ModelConfig, QuantSpec

class CheckpointError(ValueError):
    pass


@dataclass
class TensorRef:
    name: str
    file: str
    dtype: str
    shape: tuple[int, ...]


class SafetensorsDirectory:
    """Lazy reader over one or many ``*.safetensors`` shards."""

    def __init__(self, path: str | Path) -> None:
        from safetensors import safe_open
        self.path = Path(path)
        index = self.path / "model.safetensors.index.json"
        self.tensors: dict[str, TensorRef] = {}
        self._open = safe_open
        files = sorted(p.name for p in self.path.glob("*.safetensors"))
        if index.exists():
            wm = json.loads(index.read_text())["weight_map"]
            files = sorted(set(wm.values()))
        if not files:
            raise CheckpointError(f"no safetensors shards in {self.path}")
        for f in files:
            with safe_open(str(self.path / f), framework="pt") as sf:
                for name in sf.keys():
                    if name in self.tensors:
                        raise CheckpointError(f"tensor {name} appears in two shards")
                    sl = sf.get_slice(name)
                    self.tensors[name] = TensorRef(name, f, str(sl.get_dtype()), tuple(sl.get_shape()))
        # multimodal checkpoints keep the decoder under ``model.language_model.``: it is read under the text-only names
        # (``TensorRef.name`` stays the name in the file)
        nested = "model.language_model."
        if any(n.startswith(nested) for n in self.tensors):
            renamed = {}
            for n, ref in self.tensors.items():
                alias = "model." + n[len(nested):] if n.startswith(nested) else n
                if alias in renamed or (alias != n and alias in self.tensors):
                    raise CheckpointError(f"tensor {alias} exists both nested and at the top level")
                renamed[alias] = ref
            self.tensors = renamed
        # Mixtral names its expert block ``block_sparse_moe`` with projections w1 / w3 / w2 (gate / up / down): read under
        # the names every other expert family uses
        if any(".block_sparse_moe." in n for n in self.tensors):
            swap = {".w1.": ".gate_proj.", ".w3.": ".up_proj.", ".w2.": ".down_proj."}
            renamed = {}
            for n, ref in self.tensors.items():
                alias = n.replace(".block_sparse_moe.", ".mlp.")
                if ".experts." in alias:
                    for a, b in swap.items():
                        alias = alias.replace(a, b)
                if alias in renamed:
                    raise CheckpointError(f"tensor {alias} appears under two names")
                renamed[alias] = ref
            self.tensors = renamed
        self._handles: dict[str, object] = {}

    def get(self, name: str) -> torch.Tensor:
        ref = self.tensors[name]
        h = self._handles.get(ref.file)
        if h is None:
            h = self._handles[ref.file] = self._open(str(self.path / ref.file), framework="pt")
        return h.get_tensor(ref.name)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors


def _layer_modules(cfg: ModelConfig, i: int) -> dict[str, str]:
    p = f"model.layers.{i}"
    if cfg.layer_is_gdn(i):
        # Gated DeltaNet layer of the hybrid family (reference weight schema: models/qwen3_5/model.py:498)
        mods = {"qkvz": f"{p}.linear_attn.in_proj_qkvz", "ba": f"{p}.linear_attn.in_proj_ba",
                "gdn_out": f"{p}.linear_attn.out_proj"}
    else:
        mods = {"q": f"{p}.self_attn.q_proj", "k": f"{p}.self_attn.k_proj", "v": f"{p}.self_attn.v_proj",
                "o": f"{p}.self_attn.o_proj"}
    if not cfg.is_moe:
        mods.update(gate=f"{p}.mlp.gate_proj", up=f"{p}.mlp.up_proj", down=f"{p}.mlp.down_proj")
    return mods


def logical_inventory(cfg: ModelConfig) -> tuple[dict[str, tuple[int, int]], list[str]]:
    """Logical linear weights ``module -> (N, K)`` and the plain (unquantized) tensor names of a GQA decoder."""
    H, D = cfg.hidden_size, cfg.head_dim
    linears: dict[str, tuple[int, int]] = {}
    plain = ["model.embed_tokens.weight", "model.norm.weight"]
    if not cfg.tie_embeddings:
        plain.append("lm_head.weight")
    for i in range(cfg.num_layers):
        m = _layer_modules(cfg, i)
        if cfg.layer_is_gdn(i):
            gk, gv = cfg.gdn_k_heads, cfg.gdn_v_heads
            linears[m["qkvz"]] = (2 * gk * 128 + 2 * gv * 128, H)
            linears[m["ba"]] = (2 * gv, H)
            linears[m["gdn_out"]] = (H, gv * 128)
            lp = f"model.layers.{i}.linear_attn"
            plain += [f"{lp}.conv1d.weight", f"{lp}.dt_bias", f"{lp}.A_log", f"{lp}.norm.weight"]
        else:
            # with an output gate the query projection carries [q_h | gate_h] per head
            linears[m["q"]] = (cfg.q_size * (2 if cfg.attn_output_gate else 1), H)
            linears[m["k"]] = (cfg.kv_size, H)
            linears[m["v"]] = (cfg.kv_size, H)
            linears[m["o"]] = (H, cfg.q_size)
            if cfg.qkv_bias:
                plain += [f"{m[k]}.bias" for k in ("q", "k", "v")]
        if cfg.is_moe:
            plain.append(f"model.layers.{i}.mlp.gate.weight")
            if cfg.shared_intermediate_size:
                sp = f"model.layers.{i}.mlp.shared_expert"
                linears[f"{sp}.gate_proj"] = (cfg.shared_intermediate_size, H)
                linears[f"{sp}.up_proj"] = (cfg.shared_intermediate_size, H)
                linears[f"{sp}.down_proj"] = (H, cfg.shared_intermediate_size)
                plain.append(f"model.layers.{i}.mlp.shared_expert_gate.weight")
            for e in range(cfg.num_experts):
                ep = f"model.layers.{i}.mlp.experts.{e}"
                linears[f"{ep}.gate_proj"] = (cfg.moe_intermediate_size, H)
                linears[f"{ep}.up_proj"] = (cfg.moe_intermediate_size, H)
                linears[f"{ep}.down_proj"] = (H, cfg.moe_intermediate_size)
        else:
            linears[m["gate"]] = (cfg.intermediate_size, H)
            linears[m["up"]] = (cfg.intermediate_size, H)
            linears[m["down"]] = (H, cfg.intermediate_size)
        plain += [f"model.layers.{i}.input_layernorm.weight", f"model.layers.{i}.post_attention_layernorm.weight"]
        if cfg.qk_norm and not cfg.layer_is_gdn(i):
            plain += [f"model.layers.{i}.self_attn.q_norm.weight", f"model.layers.{i}.self_attn.k_norm.weight"]
    if cfg.mtp_layers:
        # multi-token-prediction head: fc over [normed embedding ; normed hidden] and one full-attention decoder layer
        # with a dense feed-forward (reference schema: models/qwen3_5/model.py:1512-1644)
        if cfg.mtp_layers != 1:
            raise CheckpointError(f"checkpoints with {cfg.mtp_layers} MTP layers are not served (one layer is)")
        mp = "mtp.layers.0"
        linears["mtp.fc"] = (H, 2 * H)
        # the head's layer is a full-attention layer of the model's own kind: gated query projection where the model
        # has one, routed (and shared) experts where the model has them
        linears[f"{mp}.self_attn.q_proj"] = (cfg.q_size * (2 if cfg.attn_output_gate else 1), H)
        linears[f"{mp}.self_attn.k_proj"] = (cfg.kv_size, H)
        linears[f"{mp}.self_attn.v_proj"] = (cfg.kv_size, H)
        linears[f"{mp}.self_attn.o_proj"] = (H, cfg.q_size)
        if cfg.is_moe:
            plain.append(f"{mp}.mlp.gate.weight")
            for e in range(cfg.num_experts):
                linears[f"{mp}.mlp.experts.{e}.gate_proj"] = (cfg.moe_intermediate_size, H)
                linears[f"{mp}.mlp.experts.{e}.up_proj"] = (cfg.moe_intermediate_size, H)
                linears[f"{mp}.mlp.experts.{e}.down_proj"] = (H, cfg.moe_intermediate_size)
            if cfg.shared_intermediate_size:
                linears[f"{mp}.mlp.shared_expert.gate_proj"] = (cfg.shared_intermediate_size, H)
                linears[f"{mp}.mlp.shared_expert.up_proj"] = (cfg.shared_intermediate_size, H)
                linears[f"{mp}.mlp.shared_expert.down_proj"] = (H, cfg.shared_intermediate_size)
                plain.append(f"{mp}.mlp.shared_expert_gate.weight")
        else:
            linears[f"{mp}.mlp.gate_proj"] = (cfg.intermediate_size, H)
            linears[f"{mp}.mlp.up_proj"] = (cfg.intermediate_size, H)
            linears[f"{mp}.mlp.down_proj"] = (H, cfg.intermediate_size)
        plain += ["mtp.pre_fc_norm_embedding.weight", "mtp.pre_fc_norm_hidden.weight", "mtp.norm.weight",
                  f"{mp}.input_layernorm.weight", f"{mp}.post_attention_layernorm.weight"]
        if cfg.qk_norm:
            plain += [f"{mp}.self_attn.q_norm.weight", f"{mp}.self_attn.k_norm.weight"]
    return linears, plain


@dataclass
class AdmittedCheckpoint:
    cfg: ModelConfig
    store: SafetensorsDirectory
    payloads: dict[str, dict[str, str]]      # module -> suffix -> tensor name
    plain: dict[str, str]
    # multimodal checkpoints: the tower's configuration, the name prefix of its tensors and the raw config.json
    vision: object | None = None
    vision_prefix: str = ""
    raw_config: dict | None = None

    def payload(self, module: str) -> dict[str, torch.Tensor]:
        return {suffix: self.store.get(name) for suffix, name in self.payloads[module].items()}

    def plain_tensor(self, name: str) -> torch.Tensor:
        """A tensor of the plain inventory.  The embedding table and ``lm_head`` of some checkpoints are quantized like
        the projections; they are decoded here, once, at load (the kernels read them as bf16 rows)."""
        module = name[:-len(".weight")] if name.endswith(".weight") else None
        if module not in self.payloads:
            return self.store.get(name)
        rows = self.cfg.vocab_size
        return _dense_of(self.cfg.quant.method, self.payload(module), (rows, self.cfg.hidden_size), self.cfg.quant)


def admit_checkpoint(path: str | Path) -> AdmittedCheckpoint:
    path = Path(path)
    cfg = ModelConfig.from_hf_config(path / "config.json")
    store = SafetensorsDirectory(path)
    linears, plain = logical_inventory(cfg)
    method = cfg.quant.method
    try:
        suffixes = registry.get(method).payload_suffixes
    except registry.QuantizationRegistryError as exc:
        raise CheckpointError(f"no loader for weight format {method!r}") from exc
    claimed: set[str] = set()
    payloads: dict[str, dict[str, str]] = {}
    for module in linears:
        found = {s: f"{module}.{s}" for s in suffixes if f"{module}.{s}" in store}
        if not found and f"{module}.weight" in store:
            found = {"weight": f"{module}.weight"}     # ignored (unquantized) module of a quantized checkpoint
        if not found:
            raise CheckpointError(f"no payload tensors for {module}")
        payloads[module] = found
        claimed.update(found.values())
        if "weight_g_idx" in found:
            # activation-order checkpoints permute the columns' scale groups; the loaders assume group = column // G
            g_idx = store.get(found["weight_g_idx"]).to(torch.int64).flatten()
            g = cfg.quant.group_size if cfg.quant.group_size > 0 else max(1, g_idx.numel())
            if not torch.equal(g_idx, torch.arange(g_idx.numel()) // g):
                raise CheckpointError(f"{module}: act-order (non-trivial weight_g_idx) checkpoints are not supported")
    plain_map = {}
    for name in plain:
        if name in ("model.embed_tokens.weight", "lm_head.weight"):
            module = name[:-len(".weight")]
            found = {s: f"{module}.{s}" for s in suffixes if f"{module}.{s}" in store}
            if set(found) - {"weight"}:                    # a quantized table: decoded at load (``plain_tensor``)
                payloads[module] = found
                claimed.update(found.values())
                plain_map[name] = module
                continue
        if name not in store:
            raise CheckpointError(f"missing tensor {name}")
        plain_map[name] = name
        claimed.add(name)
    raw = json.loads((path / "config.json").read_text())
    vision, vprefix = None, ""
    if isinstance(raw.get("vision_config"), dict):
        from .vision import VisionConfig, VisionConfigError, vision_tensor_shapes
        try:
            vision = VisionConfig.from_hf(raw["vision_config"])
        except VisionConfigError as exc:
            raise CheckpointError(str(exc)) from exc
        if vision.out_hidden_size != cfg.hidden_size:
            raise CheckpointError("the vision tower's output width differs from the decoder's hidden size")
        vprefix = next((p for p in ("model.visual.", "visual.") if f"{p}pos_embed.weight" in store), "model.visual.")
        for name, shape in vision_tensor_shapes(vision).items():
            full = vprefix + name
            if full not in store:
                raise CheckpointError(f"missing tensor {full}")
            if tuple(store.tensors[full].shape) != shape:
                raise CheckpointError(f"{full}: shape {tuple(store.tensors[full].shape)}, expected {shape}")
            claimed.add(full)
    unowned = sorted(set(store.tensors) - claimed)
    if unowned:
        raise CheckpointError(f"checkpoint has {len(unowned)} tensors no logical weight owns, e.g. {unowned[:3]}")
    return AdmittedCheckpoint(cfg, store, payloads, plain_map, vision, vprefix, raw)


def load_vision_weights(ck: AdmittedCheckpoint, device="cpu", dtype=torch.bfloat16, tp_rank: int = 0, tp_size: int = 1) -> dict:
    """The tower's tensors of an admitted multimodal checkpoint (this rank's shard under tensor parallelism)."""
    from .vision import shard_vision_weights, vision_tensor_shapes
    if ck.vision is None:
        raise CheckpointError("the checkpoint has no vision tower")
    w = {n: ck.store.get(ck.vision_prefix + n).to(dtype) for n in vision_tensor_shapes(ck.vision)}
    w = shard_vision_weights(ck.vision, w, tp_rank, tp_size)
    return {n: t.to(device) for n, t in w.items()}


def inspect_checkpoint(path: str | Path) -> dict:
    path = Path(path)
    if path.suffix == ".gguf":
        from .gguf import inspect_gguf
        return inspect_gguf(path)
    from ..contracts.model import WeightManifest
    cfg_file = path / "config.json"
    if cfg_file.is_file() and json.loads(cfg_file.read_text()).get("model_type") == "qwen4_exp":
        from .qwen4_exp import admit_qwen4_exp_checkpoint
        qcfg, _w, store = admit_qwen4_exp_checkpoint(path)
        return {"model": qcfg.name, "family": qcfg.family, "layers": qcfg.num_layers, "hidden": qcfg.hidden_size,
                "heads": f"{qcfg.num_q_heads}q/{qcfg.num_kv_heads}kv x {qcfg.head_dim}", "vocab": qcfg.vocab_size,
                "residual_streams": qcfg.streams, "experts": f"{qcfg.num_experts} top-{qcfg.experts_per_token}",
                "gated_deltanet_layers": sum(qcfg.layer_is_gdn(i) for i in range(qcfg.num_layers)),
                "ngram_layers": list(qcfg.ple_layer_ids), "vision_tower": qcfg.vision is not None,
                "tensors": len(store.tensors), "elements": sum(math.prod(t.shape) for t in store.tensors.values()),
                "manifest_digest": WeightManifest.from_store(store).digest, "execution_mode": "eager"}
    ck = admit_checkpoint(path)
    total = sum(math.prod(t.shape) for t in ck.store.tensors.values())
    by_dtype: dict[str, int] = {}
    for t in ck.store.tensors.values():
        by_dtype[t.dtype] = by_dtype.get(t.dtype, 0) + 1
    return {"model": ck.cfg.name, "family": ck.cfg.family, "layers": ck.cfg.num_layers, "hidden": ck.cfg.hidden_size,
            "heads": f"{ck.cfg.num_q_heads}q/{ck.cfg.num_kv_heads}kv x {ck.cfg.head_dim}", "vocab": ck.cfg.vocab_size,
            "quantization": f"{ck.cfg.quant.method} {ck.cfg.quant.bits}-bit group {ck.cfg.quant.group_size}",
            "tensors": len(ck.store.tensors), "elements": total, "dtypes": by_dtype,
            "manifest_digest": WeightManifest.from_store(ck.store).digest,
            "logical_linears": len(ck.payloads)}


# ------------------------------------------------------------ rank-local load
def _slice_rows(payload: dict, method: str, lo: int, hi: int, n: int, bits: int = 4) -> dict:
    """Output-dimension slice of a payload (all formats keep N as the leading axis except AWQ)."""
    out = {}
    for k, t in payload.items():
        if method == "awq":
            out[k] = t[:, lo // 8:hi // 8] if k in ("qweight", "qzeros") else t[:, lo:hi]
        elif k == "weight_zero_point":
            # zero points are packed ALONG N (``[words(N), groups]``): unpack all N, keep rows [lo, hi), pack again,
            # so that the decoder of the slice finds row lo's zero point first
            zp = formats.int_unpack(t.t().contiguous(), bits, n)[:, lo:hi]
            out[k] = formats.int_pack(zp, bits).t().contiguous()
        elif k in ("weight_shape", "weight_g_idx"):
            out[k] = t
        elif t.dim() >= 1 and t.shape[0] == n:
            out[k] = t[lo:hi]
        elif k == "weight_scale_inv":
            out[k] = t[lo // 128:-(-hi // 128)]
        else:
            out[k] = t
    return out


def _dense_of(method: str, payload: dict, shape, q: QuantSpec) -> torch.Tensor:
    """Dense fp32 matrix of a payload, decoded by the format's quantization extension."""
    try:
        return registry.get(method).dense(payload, shape, q)
    except registry.QuantizationRegistryError as exc:
        raise CheckpointError(method) from exc


def pack_logical(method: str, parts: list[tuple[dict, tuple[int, int]]], q: QuantSpec, k_slice: tuple[int, int] | None = None
                 ) -> wq_pack.PackedWeight:
    """Concatenate logical matrices along N (e.g. q, k, v) and pack them for the GEMM.

    4-bit Cubic / INT / AWQ / NVFP4 payloads stay 4-bit and FP8 payloads (one scale per row, or per 128 x 128 block)
    stay e4m3 bytes (the fp8 tensor-core GEMM consumes them as stored); everything else is decoded to bf16 at load.
    ``k_slice`` selects a column range (row-parallel shards), aligned to the scale groups.
    """
    lo, hi = k_slice if k_slice else (0, parts[0][1][1])
    native4 = method == "cubic" and q.bits == 4 or method in ("awq",) or (method == "int" and q.bits == 4) or method == "nvfp4"
    plain = any(len(p) == 1 and "weight" in p and p["weight"].dtype in (torch.bfloat16, torch.float16, torch.float32)
                for p, _ in parts)
    fp8_rows = (method == "fp8" and not plain and (hi - lo) % 64 == 0 and all(
        "weight" in p and "weight_scale" in p and p["weight"].dtype == torch.float8_e4m3fn
        and p["weight_scale"].numel() == s[0] for p, s in parts))
    if fp8_rows:
        # e4m3 weights with one scale per output row: W8A8 on the fp8 tensor path, no expansion
        w8 = torch.cat([p["weight"].view(torch.uint8)[:, lo:hi] for p, _ in parts], 0)
        return wq_pack.pack_fp8(w8, torch.cat([p["weight_scale"].float().reshape(-1) for p, _ in parts]))
    def block_scales(p):
        return p["weight_scale_inv"] if "weight_scale_inv" in p else p.get("weight_scale")

    fp8_blocks = (method in ("fp8", "fp8_block") and not plain and lo % 128 == 0 and (hi - lo) % 64 == 0 and all(
        "weight" in p and p["weight"].dtype == torch.float8_e4m3fn and block_scales(p) is not None
        and block_scales(p).dim() == 2 and tuple(block_scales(p).shape) == (-(-s[0] // 128), -(-s[1] // 128))
        and (s[0] % 128 == 0 or len(parts) == 1) for p, s in parts)) and not fp8_rows
    if fp8_blocks:
        # e4m3 weights with one scale per 128 x 128 block: the block-scaled form of the fp8 tensor-core GEMM
        w8 = torch.cat([p["weight"].view(torch.uint8)[:, lo:hi] for p, _ in parts], 0)
        bs = torch.cat([block_scales(p).float()[:, lo // 128:-(-hi // 128)] for p, _ in parts], 0)
        return wq_pack.pack_fp8_block(w8, bs)
    if not native4 or plain:
        dense = torch.cat([_dense_of(method, p, s, q) for p, s in parts], 0)
        return wq_pack.pack_bf16(dense[:, lo:hi])
    if method == "cubic":
        g = q.group_size
        if lo % g or (hi % g and hi != parts[0][1][1]):
            raise CheckpointError("column shard cuts a Cubic scale group")
        codes, sc, aa, bb = [], [], [], []
        for p, s in parts:
            codes.append(cubic.unpack_codes(p["weight_packed"], 4, s[1])[:, lo:hi])
            t = cubic.metadata_triple(p, cubic.CubicScheme(4, g, metadata=_cubic_variant(p)), s)
            sc.append(t[0][:, lo // g:-(-hi // g)]); aa.append(t[1][:, lo // g:-(-hi // g)]); bb.append(t[2][:, lo // g:-(-hi // g)])
        return wq_pack.pack_cubic4(torch.cat(codes), torch.cat(sc), torch.cat(aa), torch.cat(bb), g)
    if method in ("int", "awq"):
        g = q.group_size if q.group_size > 0 else parts[0][1][1]
        qs, ss, zs = [], [], []
        for p, s in parts:
            cq, cs, cz = formats.int_decode(p, 4, q.group_size, s) if method == "int" else formats.awq_decode(p, g)
            qs.append(cq[:, lo:hi]); ss.append(cs[:, lo // g:-(-hi // g)]); zs.append(cz[:, lo // g:-(-hi // g)])
        qq, sc, zz = torch.cat(qs), torch.cat(ss), torch.cat(zs)
        return wq_pack.pack_affine4(qq.to(torch.uint8), sc, -zz * sc, min(g, hi - lo))
    # nvfp4: every part carries its own global scale; fold the ratio into the block scales
    mults = [formats.nvfp4_global_multiplier(p) for p, _ in parts]
    ref = max(mults)
    packed = torch.cat([(p["weight_packed"] if "weight_packed" in p else p["weight"])[:, lo // 2:hi // 2] for p, _ in parts])
    scales = torch.cat([p["weight_scale"].float()[:, lo // 16:hi // 16] * (m / ref) for (p, _), m in zip(parts, mults)])
    return wq_pack.pack_nvfp4(packed, scales, ref)


def _cubic_variant(p: dict) -> str:
    if "weight_ab" in p:
        return cubic.METADATA_B
    if "weight_metadata" in p:
        return cubic.METADATA_C
    return cubic.METADATA_A


def load_decoder_weights(ck: AdmittedCheckpoint, device, tp_rank: int = 0, tp_size: int = 1,
                         layer_range: tuple[int, int] | None = None):
    """Admitted checkpoint -> rank-local ``DecoderWeights`` (dense FFN decoders).

    ``layer_range`` = ``[lo, hi)`` loads only the decoder layers of one pipeline stage.
    """
    from .decoder import DecoderWeights, GdnWeights, LayerWeights
    cfg, q = ck.cfg, ck.cfg.quant
    method = q.method
    if tp_size > 1:
        from .parallel_weights import PartitionError, plan_partition
        try:                              # name what does not divide before any tensor is read
            plan_partition(cfg, tp_size, 1, tp_size if cfg.is_moe else 1)
        except PartitionError as exc:
            raise CheckpointError(f"{cfg.name} does not split over {tp_size} ranks: {exc}") from exc
    D = cfg.head_dim
    from .config import kv_heads_of_rank
    kv_first, hkv = kv_heads_of_rank(cfg.num_kv_heads, tp_rank, tp_size)     # a copy of a shared head when ranks outnumber them
    hq = cfg.num_q_heads // tp_size
    inter = cfg.intermediate_size // tp_size
    bf = torch.bfloat16

    cache: dict[str, dict] = {}

    def payload(module: str) -> dict:
        if module not in cache:
            cache.clear()                     # one module at a time: a layer's row ranges come from the same tensors
            cache[module] = ck.payload(module)
        return cache[module]

    def rows(module: str, lo: int, hi: int, n: int):
        return _slice_rows(payload(module), method, lo, hi, n, q.bits), (hi - lo, ck_shapes[module][1])

    ck_shapes, _ = logical_inventory(cfg)
    if cfg.head_dim > 128:
        raise CheckpointError(f"attention heads of width {cfg.head_dim} are served by the eager execution mode "
                              "(--execution-mode eager); the native attention kernels are built for 128")
    layers = []
    for i in range(*(layer_range or (0, cfg.num_layers))):
        m = _layer_modules(cfg, i)
        p = f"model.layers.{i}"
        gdn = attn_gate = qkv = o = None
        if cfg.layer_is_gdn(i):
            # The checkpoint groups the projection rows by key head: [q | k | v x r | z x r] (and [b x r | a x r]) for
            # each of the Hk key heads, r = Hv / Hk value heads per key head.  The kernels take q | k | v | z of all
            # (rank-local) heads in turn, so the rows are gathered section by section; a rank owns whole key heads.
            gk_all, gv_all = cfg.gdn_k_heads, cfg.gdn_v_heads
            r = gv_all // gk_all
            gk, gv = gk_all // tp_size, gv_all // tp_size
            group = (2 + 2 * r) * 128
            heads = range(tp_rank * gk, (tp_rank + 1) * gk)
            n_all = ck_shapes[m["qkvz"]][0]
            parts = []
            for lo, width in ((0, 128), (128, 128), (256, r * 128), (256 + r * 128, r * 128)):
                parts += [rows(m["qkvz"], h * group + lo, h * group + lo + width, n_all) for h in heads]
            in_proj = pack_logical(method, parts, q)
            ba = _dense_of(method, ck.payload(m["ba"]), ck_shapes[m["ba"]], q).view(gk_all, 2, r, cfg.hidden_size)
            ba = ba[tp_rank * gk:(tp_rank + 1) * gk]
            in_ba = wq_pack.pack_bf16(torch.cat([ba[:, 0].reshape(gv, -1), ba[:, 1].reshape(gv, -1)]))
            out = pack_logical(method, [(ck.payload(m["gdn_out"]), ck_shapes[m["gdn_out"]])], q,
                               (tp_rank * gv * 128, (tp_rank + 1) * gv * 128))
            lp = f"{p}.linear_attn"
            # conv channels: q of all key heads | k | v (rank-local slices of each section)
            cw = ck.store.get(f"{lp}.conv1d.weight").float().reshape(-1, 4)
            qk, vv = gk_all * 128, gv_all * 128
            sel = torch.cat([torch.arange(tp_rank * gk * 128, (tp_rank + 1) * gk * 128),
                             qk + torch.arange(tp_rank * gk * 128, (tp_rank + 1) * gk * 128),
                             2 * qk + torch.arange(tp_rank * gv * 128, (tp_rank + 1) * gv * 128)])
            assert cw.shape[0] == 2 * qk + vv
            f32 = dict(device=device, dtype=torch.float32)
            gdn = GdnWeights(in_proj=in_proj.to(device), in_ba=in_ba.to(device), conv_w=cw[sel].contiguous().to(**f32),
                             a_log=ck.store.get(f"{lp}.A_log")[tp_rank * gv:(tp_rank + 1) * gv].to(**f32),
                             dt_bias=ck.store.get(f"{lp}.dt_bias")[tp_rank * gv:(tp_rank + 1) * gv].to(**f32),
                             norm_w=ck.store.get(f"{lp}.norm.weight").to(**f32), out=out.to(device), hk=gk, hv=gv)
        else:
            if cfg.attn_output_gate:
                # query projection rows per head: [q_h | gate_h]
                heads = range(tp_rank * hq, (tp_rank + 1) * hq)
                qn = 2 * cfg.q_size
                q_parts = [rows(m["q"], h * 2 * D, h * 2 * D + D, qn) for h in heads]
                attn_gate = pack_logical(method, [rows(m["q"], h * 2 * D + D, (h + 1) * 2 * D, qn) for h in heads], q)
            else:
                q_parts = [rows(m["q"], tp_rank * hq * D, (tp_rank + 1) * hq * D, cfg.q_size)]
            qkv = pack_logical(method, q_parts + [rows(m["k"], kv_first * D, (kv_first + hkv) * D, cfg.kv_size),
                                                  rows(m["v"], kv_first * D, (kv_first + hkv) * D, cfg.kv_size)], q)
            o = pack_logical(method, [(ck.payload(m["o"]), ck_shapes[m["o"]])], q,
                             (tp_rank * hq * D, (tp_rank + 1) * hq * D))
        moe = gu = down = None
        if cfg.is_moe:
            from .moe import load_moe_layer
            moe = load_moe_layer(ck, i, device, tp_rank, tp_size)
        else:
            gu = pack_logical(method, [rows(m["gate"], tp_rank * inter, (tp_rank + 1) * inter, cfg.intermediate_size),
                                       rows(m["up"], tp_rank * inter, (tp_rank + 1) * inter, cfg.intermediate_size)], q)
            down = pack_logical(method, [(ck.payload(m["down"]), ck_shapes[m["down"]])], q,
                                (tp_rank * inter, (tp_rank + 1) * inter))
        lw = LayerWeights(ln1=ck.store.get(f"{p}.input_layernorm.weight").to(device, bf),
                          ln2=ck.store.get(f"{p}.post_attention_layernorm.weight").to(device, bf),
                          qkv=None if qkv is None else qkv.to(device), o=None if o is None else o.to(device), gdn=gdn,
                          attn_gate=None if attn_gate is None else attn_gate.to(device),
                          gate_up=None if gu is None else gu.to(device), down=None if down is None else down.to(device),
                          moe=moe)
        if cfg.qkv_bias and gdn is None:
            if cfg.attn_output_gate:
                raise CheckpointError("projection biases together with a gated query projection are not served")
            # this rank's heads of the q / k / v biases, in the order of the fused projection's rows
            bq, bk, bv = (ck.store.get(f"{m[k]}.bias").float() for k in ("q", "k", "v"))
            lw.qkv_bias = torch.cat([bq[tp_rank * hq * D:(tp_rank + 1) * hq * D], bk[kv_first * D:(kv_first + hkv) * D],
                                     bv[kv_first * D:(kv_first + hkv) * D]]).to(device, bf).contiguous()
        if cfg.qk_norm and gdn is None:
            # the kernels multiply by the vector they are given: checkpoints with zero-centred norms store w of (1 + w)
            one = 1.0 if cfg.zero_centered_norm else 0.0
            lw.q_norm = (ck.store.get(f"{p}.self_attn.q_norm.weight").float() + one).to(device, bf)
            lw.k_norm = (ck.store.get(f"{p}.self_attn.k_norm.weight").float() + one).to(device, bf)
        layers.append(lw)
    embed_full = ck.plain_tensor("model.embed_tokens.weight").to(device, bf)
    v_local = cfg.vocab_size // tp_size
    head = embed_full if cfg.tie_embeddings else ck.plain_tensor("lm_head.weight").to(device, bf)
    head = head[tp_rank * v_local:(tp_rank + 1) * v_local].contiguous()
    return DecoderWeights(embed=embed_full[tp_rank * v_local:(tp_rank + 1) * v_local], layers=layers,
                          final_norm=ck.store.get("model.norm.weight").to(device, bf), lm_head=wq_pack.pack_bf16(head),
                          vocab_start=tp_rank * v_local, extras={"embed_full": embed_full})


def load_mtp_weights(ck: AdmittedCheckpoint, device):
    """The checkpoint's multi-token-prediction head as ``models.mtp.MtpWeights`` (single rank: speculative rounds run
    in the single-process executor)."""
    from .decoder import LayerWeights
    from .mtp import MtpWeights
    cfg, q = ck.cfg, ck.cfg.quant
    if not cfg.mtp_layers:
        raise CheckpointError("this checkpoint carries no MTP head (no mtp_num_hidden_layers in its config)")
    if cfg.is_moe or cfg.is_hybrid:
        raise CheckpointError("MTP heads are served for dense full-attention decoders")
    shapes, _ = logical_inventory(cfg)
    bf = torch.bfloat16
    mp = "mtp.layers.0"

    def fused(*modules: str):
        return pack_logical(q.method, [(ck.payload(m), shapes[m]) for m in modules], q).to(device)

    def vec(name: str):
        return ck.store.get(name).to(device, bf)

    layer = LayerWeights(ln1=vec(f"{mp}.input_layernorm.weight"), ln2=vec(f"{mp}.post_attention_layernorm.weight"),
                         qkv=fused(f"{mp}.self_attn.q_proj", f"{mp}.self_attn.k_proj", f"{mp}.self_attn.v_proj"),
                         o=fused(f"{mp}.self_attn.o_proj"), gate_up=fused(f"{mp}.mlp.gate_proj", f"{mp}.mlp.up_proj"),
                         down=fused(f"{mp}.mlp.down_proj"))
    if cfg.qk_norm:
        layer.q_norm, layer.k_norm = vec(f"{mp}.self_attn.q_norm.weight"), vec(f"{mp}.self_attn.k_norm.weight")
    return MtpWeights(vec("mtp.pre_fc_norm_embedding.weight"), vec("mtp.pre_fc_norm_hidden.weight"), fused("mtp.fc"), layer,
                      vec("mtp.norm.weight"))


# ------------------------------------------------------- random checkpoints
def _quant_config_json(q: QuantSpec) -> dict | None:
    return registry.get(q.method).config_json(q)


def quantize_payload(w: torch.Tensor, q: QuantSpec) -> dict[str, torch.Tensor]:
    return registry.get(q.method).quantize(w, q)


def write_random_checkpoint(path: str | Path, cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> Path:
    """Random-init decoder written as a HuggingFace-style directory in ``cfg.quant``'s on-disk format."""
    from safetensors.torch import save_file
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    linears, plain = logical_inventory(cfg)
    tensors: dict[str, torch.Tensor] = {}
    for module, (n, k) in linears.items():
        w = torch.randn(n, k, generator=g) * std
        if module.endswith("in_proj_ba"):
            tensors[f"{module}.weight"] = w.to(torch.bfloat16)      # a 2 Hv-row module: left unquantized
            continue
        for suffix, t in quantize_payload(w, cfg.quant).items():
            tensors[f"{module}.{suffix}"] = t.contiguous()
    for name in plain:
        if ".linear_attn." in name:
            gk, gv = cfg.gdn_k_heads, cfg.gdn_v_heads
            if name.endswith("conv1d.weight"):
                tensors[name] = (torch.randn((2 * gk + gv) * 128, 1, 4, generator=g) * 0.3).to(torch.bfloat16)
            elif name.endswith("norm.weight"):
                tensors[name] = torch.ones(128, dtype=torch.bfloat16)
            else:                              # A_log, dt_bias
                tensors[name] = torch.randn(gv, generator=g) * 0.5
        elif "pre_fc_norm" in name:
            tensors[name] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
        elif name.endswith("norm.weight"):
            tensors[name] = torch.ones(cfg.head_dim if "_norm" in name.split(".")[-2] and "self_attn" in name else cfg.hidden_size,
                                       dtype=torch.bfloat16)
        elif name.endswith("mlp.gate.weight"):
            tensors[name] = (torch.randn(cfg.num_experts, cfg.hidden_size, generator=g) * std).to(torch.bfloat16)
        elif name.endswith("shared_expert_gate.weight"):
            tensors[name] = (torch.randn(1, cfg.hidden_size, generator=g) * std).to(torch.bfloat16)
        elif name.endswith("_proj.bias"):
            rows = cfg.q_size if name.endswith("q_proj.bias") else cfg.kv_size
            tensors[name] = (torch.randn(rows, generator=g) * std).to(torch.bfloat16)
        else:
            tensors[name] = (torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * std).to(torch.bfloat16)
    save_file(tensors, str(path / "model.safetensors"))
    arch = ("Qwen3MoeForCausalLM" if cfg.qk_norm else "Qwen2MoeForCausalLM") if cfg.is_moe else \
        ("Qwen3ForCausalLM" if cfg.qk_norm else "LlamaForCausalLM")
    hf = {"architectures": ["Qwen3NextForCausalLM" if cfg.is_hybrid else arch],
          "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_q_heads,
          "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size,
          "vocab_size": cfg.vocab_size, "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps,
          "tie_word_embeddings": cfg.tie_embeddings, "max_position_embeddings": cfg.max_position, "_name_or_path": cfg.name}
    if cfg.is_hybrid:
        hf.update(linear_num_key_heads=cfg.gdn_k_heads, linear_num_value_heads=cfg.gdn_v_heads, linear_key_head_dim=128,
                  linear_value_head_dim=128, full_attention_interval=cfg.gdn_interval, attn_output_gate=cfg.attn_output_gate,
                  partial_rotary_factor=(cfg.rotary_dim or cfg.head_dim) / cfg.head_dim)
    if cfg.mtp_layers:
        hf["mtp_num_hidden_layers"] = cfg.mtp_layers
    if cfg.is_moe:
        hf.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.experts_per_token,
                  moe_intermediate_size=cfg.moe_intermediate_size, norm_topk_prob=cfg.norm_topk_prob)
        if cfg.shared_intermediate_size:
            hf["shared_expert_intermediate_size"] = cfg.shared_intermediate_size
    hf["qkv_bias"] = cfg.qkv_bias
    if cfg.mrope_section is not None:
        hf["rope_parameters"] = {"mrope_section": list(cfg.mrope_section), "rope_theta": cfg.rope_theta}
    qc = _quant_config_json(cfg.quant)
    if qc:
        hf["quantization_config"] = qc
    (path / "config.json").write_text(json.dumps(hf, indent=1))
    return path
