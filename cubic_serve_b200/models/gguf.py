"""GGUF file inventory and logical weight views (reference: ``models/gguf.py:172``, ``models/gguf_weights.py:433``)."""
from __future__ import annotations

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
    return {"file": str(path), "architecture": arch, "tensors": len(reader.tensors), "types": types,
            "admitted": not rejected, "rejected": rejected[:8]}


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
