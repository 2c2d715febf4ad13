"""Model architecture description shared by the loader, the runners and the benchmarks.

Plays the role of the reference's ``ModelSpec`` / per-family config parsers
(``contracts/model.py:66-273``, ``models/qwen3_5/model.py:498``) for the decoder
families this engine serves: plain GQA decoders (Llama/Qwen3 style, dense or
MoE) and hybrid linear-attention decoders.
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass(frozen=True)
class QuantSpec:
    """How the linear weights are stored."""
    method: str = "cubic"          # cubic | int | awq | fp8 | fp8_block | nvfp4 | gguf | none
    bits: int = 4
    group_size: int = 128
    lm_head_quantized: bool = False


def _served_positions(text: dict, arch: str) -> int:
    """Context the checkpoint is served at.  A model trained with sliding-window attention equals full attention only
    inside one window: the kernels attend to the whole context, so such a checkpoint is served up to its window."""
    limit = int(text.get("max_position_embeddings", 40960))
    window = text.get("sliding_window")
    applies = text.get("use_sliding_window", arch.startswith(("Mistral", "Mixtral")))
    if isinstance(window, int) and window > 0 and applies:
        limit = min(limit, window)
    return limit


def _rope_scaling(text: dict):
    """``rope_scaling`` / ``rope_parameters`` of a checkpoint as ``ModelConfig.rope_scaling``.  Forms that change the
    rotation with the sequence length or need per-dimension logit factors (dynamic, longrope) are refused: served with
    the plain table they would silently lose quality at long context."""
    for key in ("rope_scaling", "rope_parameters"):
        rs = text.get(key)
        if not isinstance(rs, dict):
            continue
        kind = rs.get("rope_type", rs.get("type", "default"))
        if kind in ("default", None) or "mrope_section" in rs and kind == "default":
            continue
        if kind == "linear":
            return ("linear", float(rs["factor"]))
        if kind == "llama3":
            return ("llama3", float(rs["factor"]), float(rs["low_freq_factor"]), float(rs["high_freq_factor"]),
                    int(rs["original_max_position_embeddings"]))
        if kind == "yarn":
            if rs.get("mscale") or rs.get("mscale_all_dim") or rs.get("truncate", True) is not True:
                raise ValueError("yarn rotary scaling with mscale / mscale_all_dim / truncate=false is not served")
            if float(text.get("partial_rotary_factor", rs.get("partial_rotary_factor", 1.0)) or 1.0) != 1.0:
                raise ValueError("yarn rotary scaling of partly rotated heads is not served")
            factor = float(rs["factor"])
            original = int(rs.get("original_max_position_embeddings") or text.get("max_position_embeddings", 40960))
            af = rs.get("attention_factor")
            af = float(af) if af is not None else (1.0 if factor <= 1 else 0.1 * math.log(factor) + 1.0)
            return ("yarn", factor, original, float(rs.get("beta_fast") or 32), float(rs.get("beta_slow") or 1), af)
        raise ValueError(f"rotary scaling of type {kind!r} is not served")
    return None


def _mrope_section(text: dict):
    """``mrope_section`` of ``rope_parameters`` / ``rope_scaling`` when the checkpoint declares three-axis positions."""
    for key in ("rope_parameters", "rope_scaling"):
        sec = (text.get(key) or {}).get("mrope_section") if isinstance(text.get(key), dict) else None
        if sec is not None:
            if len(sec) != 3:
                raise ValueError("mrope_section lists three counts")
            return tuple(int(v) for v in sec)
    return None


@dataclass(frozen=True)
class ModelConfig:
    name: str = "toy"
    family: str = "gqa_decoder"    # gqa_decoder | gqa_moe | qwen3_5 | qwen3_5_moe | qwen4_exp
    num_layers: int = 2
    hidden_size: int = 256
    num_q_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 512
    vocab_size: int = 1024
    rope_theta: float = 10000.0
    rotary_dim: int | None = None
    rms_eps: float = 1e-6
    qk_norm: bool = False
    zero_centered_norm: bool = False
    tie_embeddings: bool = False
    max_position: int = 40960
    # MoE
    num_experts: int = 0
    mtp_layers: int = 0              # multi-token-prediction draft layers carried by the checkpoint (``mtp.*`` tensors)
    experts_per_token: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # hybrid family (qwen3_5 style): every ``gdn_interval``-th layer is full attention, the others are Gated
    # DeltaNet linear-attention layers with ``gdn_k_heads`` key / ``gdn_v_heads`` value heads of width 128
    # (reference: ``models/qwen3_5/model.py:1399``); 0 = no such layers
    gdn_interval: int = 0
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    attn_output_gate: bool = False      # full-attention output multiplied by sigmoid(gate projection)
    # MTP head (1 extra decoder layer sharing embeddings and lm_head)
    mtp_layers: int = 0
    quant: QuantSpec = field(default_factory=QuantSpec)
    eos_token_id: int | None = None
    # sigmoid-gated shared expert beside the routed experts (width of its SwiGLU; 0 = none) and biases on the q / k / v
    # projections (Qwen2 family): both are served by the eager execution mode only
    shared_intermediate_size: int = 0
    qkv_bias: bool = False
    # static rescaling of the rotary frequencies: ("linear", factor), ("llama3", factor, low_freq_factor,
    # high_freq_factor, original_max_position_embeddings) or ("yarn", factor, original_max_position_embeddings, beta_fast,
    # beta_slow, attention_factor); None = the plain table
    rope_scaling: tuple | None = None
    # three-axis rotary positions of the multimodal checkpoints: how many frequency slots follow the (temporal, row,
    # column) axis; None = one axis
    mrope_section: tuple[int, int, int] | None = None

    @property
    def attention_scale(self) -> float | None:
        """Softmax scale of the attention logits when it is not ``1 / sqrt(head_dim)``: yarn scaling multiplies the
        rotated queries AND keys by its attention factor, i.e. the logits of fully rotated heads by its square."""
        rs = self.rope_scaling
        if rs is None or rs[0] != "yarn" or rs[5] == 1.0:
            return None
        return rs[5] * rs[5] / math.sqrt(self.head_dim)

    @property
    def q_size(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_hybrid(self) -> bool:
        return self.gdn_interval > 0

    def layer_is_gdn(self, layer: int) -> bool:
        """Layer ``layer`` (global index) is a Gated DeltaNet layer (every ``gdn_interval``-th one is full attention)."""
        return self.gdn_interval > 0 and (layer + 1) % self.gdn_interval != 0

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @staticmethod
    def from_dict(d: dict) -> "ModelConfig":
        d = dict(d)
        q = d.pop("quant", None)
        if isinstance(q, dict):
            d["quant"] = QuantSpec(**q)
        return ModelConfig(**d)

    @staticmethod
    def from_hf_config(path: str | Path) -> "ModelConfig":
        """Parse a HuggingFace ``config.json`` (Llama / Qwen2 / Qwen3 / Qwen3-MoE style)."""
        cfg = json.loads(Path(path).read_text())
        text = cfg.get("text_config", cfg)
        qc = cfg.get("quantization_config") or text.get("quantization_config") or {}
        arch = (cfg.get("architectures") or ["?"])[0]
        heads = text["num_attention_heads"]
        hd = text.get("head_dim") or text["hidden_size"] // heads
        n_exp = text.get("num_experts") or text.get("num_local_experts") or 0
        rope = text.get("rope_parameters") if isinstance(text.get("rope_parameters"), dict) else {}
        if text.get("attention_bias"):
            raise ValueError("checkpoints with biases on all attention projections (attention_bias) are not served")
        if text.get("mlp_bias"):
            raise ValueError("checkpoints with biases on the feed-forward projections (mlp_bias) are not served")
        if n_exp and (text.get("mlp_only_layers") or int(text.get("decoder_sparse_step", 1) or 1) != 1):
            raise ValueError("checkpoints that mix dense and expert feed-forward layers are not served")
        hybrid = {}
        if text.get("linear_num_value_heads"):
            if int(text.get("linear_key_head_dim", 128)) != 128 or int(text.get("linear_value_head_dim", 128)) != 128:
                raise ValueError("Gated DeltaNet layers are built for key / value head width 128")
            hybrid = dict(gdn_interval=int(text.get("full_attention_interval", 4)),
                          gdn_k_heads=int(text["linear_num_key_heads"]), gdn_v_heads=int(text["linear_num_value_heads"]),
                          attn_output_gate=bool(text.get("attn_output_gate", True)), zero_centered_norm=True,
                          rotary_dim=int(hd * float(rope.get("partial_rotary_factor", text.get("partial_rotary_factor", 0.25)))))
        return ModelConfig(
            **hybrid,
            name=cfg.get("_name_or_path") or arch,
            family=("qwen3_5_moe" if n_exp else "qwen3_5") if hybrid else ("gqa_moe" if n_exp else "gqa_decoder"),
            num_layers=text["num_hidden_layers"],
            hidden_size=text["hidden_size"],
            num_q_heads=heads,
            num_kv_heads=text.get("num_key_value_heads", heads),
            head_dim=hd,
            intermediate_size=text.get("intermediate_size", 0),
            vocab_size=text["vocab_size"],
            rope_theta=float(text.get("rope_theta", rope.get("rope_theta", 10000.0))),
            rms_eps=float(text.get("rms_norm_eps", 1e-6)),
            qk_norm="Qwen3" in arch,
            shared_intermediate_size=int(text.get("shared_expert_intermediate_size") or 0) if n_exp else 0,
            qkv_bias=bool(text.get("qkv_bias", arch.startswith("Qwen2"))),
            tie_embeddings=bool(text.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))),
            max_position=_served_positions(text, arch),
            num_experts=n_exp,
            experts_per_token=text.get("num_experts_per_tok", 0) if n_exp else 0,
            # Mixtral gives its experts the width named ``intermediate_size``
            moe_intermediate_size=(text.get("moe_intermediate_size") or text.get("intermediate_size", 0)) if n_exp else 0,
            norm_topk_prob=bool(text.get("norm_topk_prob", True)),
            mtp_layers=int(text.get("mtp_num_hidden_layers") or text.get("num_nextn_predict_layers") or 0),
            quant=quant_spec_from_hf(qc),
            eos_token_id=(text.get("eos_token_id") if isinstance(text.get("eos_token_id"), int) else None),
            mrope_section=_mrope_section(text),
            rope_scaling=_rope_scaling(text),
        )


def quant_spec_from_hf(qc: dict) -> QuantSpec:
    """Map a ``quantization_config`` block to a QuantSpec: the registered quantization extensions are asked in turn
    (``quantization/registry.py``; reference: ``models/quantization.py:79-124``)."""
    from ..quantization import registry
    return registry.detect(qc or {})


# ----------------------------------------------------------------- named configs
def toy_config() -> ModelConfig:
    """CPU toy decoder: 2 layers, hidden 256, 4q/2kv heads of 64, FFN 512, vocab 1024."""
    return ModelConfig(name="toy", num_layers=2, hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=64,
                       intermediate_size=512, vocab_size=1024, rope_theta=10000.0, rms_eps=1e-6)


def dense_8b_config() -> ModelConfig:
    return ModelConfig(name="dense-8b", num_layers=36, hidden_size=4096, num_q_heads=32, num_kv_heads=8,
                       head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_eps=1e-6,
                       quant=QuantSpec("cubic", 4, 128))


def moe_30b_config() -> ModelConfig:
    return ModelConfig(name="moe-30b-a3b", family="gqa_moe", num_layers=48, hidden_size=2048, num_q_heads=32,
                       num_kv_heads=4, head_dim=128, intermediate_size=0, vocab_size=151936, rope_theta=1e6,
                       num_experts=128, experts_per_token=8, moe_intermediate_size=768,
                       quant=QuantSpec("nvfp4", 4, 16))


def hybrid_8b_config() -> ModelConfig:
    """8B-class hybrid decoder: three Gated DeltaNet layers for every full-attention layer (qwen3_5 layout)."""
    return ModelConfig(name="hybrid-8b", family="qwen3_5", num_layers=36, hidden_size=4096, num_q_heads=32, num_kv_heads=8,
                       head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e7, rotary_dim=64,
                       qk_norm=True, zero_centered_norm=True, gdn_interval=4, gdn_k_heads=16, gdn_v_heads=32,
                       attn_output_gate=True, quant=QuantSpec("cubic", 4, 128))


def moe_235b_config() -> ModelConfig:
    return ModelConfig(name="moe-235b-a22b", family="gqa_moe", num_layers=94, hidden_size=4096, num_q_heads=64,
                       num_kv_heads=4, head_dim=128, intermediate_size=0, vocab_size=151936, rope_theta=1e6,
                       num_experts=128, experts_per_token=8, moe_intermediate_size=1536,
                       quant=QuantSpec("fp8_block", 8, 128))


def kv_heads_of_rank(num_kv_heads: int, tp_rank: int, tp_size: int) -> tuple[int, int]:
    """Key/value heads ``[first, first + count)`` that tensor-parallel rank ``tp_rank`` holds.  With at least as many
    heads as ranks every rank owns ``num_kv_heads / tp_size`` of them; with fewer, ``tp_size / num_kv_heads``
    neighbouring ranks hold a copy of the same head (their query heads share it), as the reference replicates key/value
    heads of grouped-query models across a wide tensor-parallel group."""
    if num_kv_heads >= tp_size:
        if num_kv_heads % tp_size:
            raise ValueError(f"{num_kv_heads} key/value heads do not split over {tp_size} ranks")
        n = num_kv_heads // tp_size
        return tp_rank * n, n
    if tp_size % num_kv_heads:
        raise ValueError(f"{tp_size} ranks do not share {num_kv_heads} key/value heads evenly")
    return tp_rank // (tp_size // num_kv_heads), 1


NAMED_CONFIGS = {
    "toy": toy_config,
    "dense-8b": dense_8b_config,
    "moe-30b-a3b": moe_30b_config,
    "hybrid-8b": hybrid_8b_config,
    "moe-235b-a22b": moe_235b_config,
}


def _qwen4_exp_tiny():
    from .qwen4_exp import tiny_config
    return tiny_config()


NAMED_CONFIGS["qwen4-exp-tiny"] = _qwen4_exp_tiny          # served by the eager executor of ``models/qwen4_exp.py``
