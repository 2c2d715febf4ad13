"""The built-in quantization extensions: none (bf16), cubic, int, awq, fp8 (per channel), fp8_block, nvfp4, gguf.

Each bundles the format's recognition rule, payload tensor names, dense decoder, quantizer and the
``quantization_config`` it writes (reference: ``quantization/extensions/*/`` and ``models/quantization.py:79-124``).
"""
from __future__ import annotations

import torch

from ..ops import wq_pack
from . import cubic, formats
from .registry import QuantizationExtension


def _spec(method: str, bits: int, group: int):
    from ..models.config import QuantSpec
    return QuantSpec(method, bits, group)


def _first_group_weights(qc: dict) -> dict:
    groups = qc.get("config_groups") or {}
    for g in groups.values():
        if isinstance(g, dict) and isinstance(g.get("weights"), dict):
            return g["weights"]
    return qc


def _plain_or(decode):
    """A module a quantized checkpoint leaves unquantized is stored as a single ``weight`` tensor."""
    def dense(payload: dict, shape, q):
        if "weight" in payload and len(payload) == 1 and payload["weight"].dtype in (torch.bfloat16, torch.float16, torch.float32):
            return payload["weight"].float()
        return decode(payload, shape, q)
    return dense


# ------------------------------------------------------------------ none
def _none_detect(qc: dict):
    return None if qc else _spec("none", 16, 0)


# ------------------------------------------------------------------ cubic
def _cubic_detect(qc: dict):
    if qc.get("quant_method") == "cubic" or qc.get("format") == "cubic-pack-quantized":
        w = _first_group_weights(qc)
        gs = w.get("group_size", 128)
        return _spec("cubic", int(w.get("num_bits", 4)), int(gs[1] if isinstance(gs, list) else gs))
    return None


def _cubic_config(q) -> dict:
    return {"quant_method": "cubic", "format": "cubic-pack-quantized", "ignore": ["lm_head"], "config_groups": {
        "group_0": {"targets": ["Linear"], "input_activations": None, "weights": {
            "num_bits": q.bits, "group_size": q.group_size, "dynamic": False, "symmetric": True,
            "packing": "little-endian-bitstream", "reserved_code": "zero",
            "metadata_format": cubic.METADATA_A, "scale_dtype": "float32", "param_dtype": "float16"}}}}


# ------------------------------------------------------------------ int (compressed-tensors pack-quantized)
def _int_detect(qc: dict):
    if qc.get("format") == "pack-quantized":
        w = _first_group_weights(qc)
        return _spec("int", int(w.get("num_bits", 4)), int(w.get("group_size") or 0))
    return None


def _int_config(q) -> dict:
    return {"quant_method": "compressed-tensors", "format": "pack-quantized", "ignore": ["lm_head"], "config_groups": {
        "group_0": {"targets": ["Linear"], "weights": {"num_bits": q.bits, "group_size": q.group_size,
                                                       "symmetric": True, "type": "int", "strategy": "group"}}}}


# ------------------------------------------------------------------ awq
def _awq_detect(qc: dict):
    if qc.get("quant_method") == "awq":
        return _spec("awq", int(qc.get("bits", 4)), int(qc.get("group_size", 128)))
    return None


def _awq_quantize(w: torch.Tensor, q) -> dict:
    n, k = w.shape
    g = q.group_size
    wg = w.float().reshape(n, k // g, g)
    lo, hi = wg.amin(-1), wg.amax(-1)
    s = ((hi - lo) / 15).clamp_min(1e-8)
    z = torch.round(-lo / s).clamp(0, 15)
    qv = torch.round(wg / s[..., None] + z[..., None]).clamp(0, 15).reshape(n, k)
    return {"qweight": formats.awq_pack(qv.t().contiguous()), "qzeros": formats.awq_pack(z.t().contiguous()),
            "scales": s.t().contiguous().half()}


# ------------------------------------------------------------------ fp8 (per channel) and fp8_block (128 x 128)
def _fp8_detect(qc: dict):
    if qc.get("format") == "float-quantized":
        w = _first_group_weights(qc)
        block = w.get("block_structure") or qc.get("weight_block_size")
        return _spec("fp8_block" if block else "fp8", 8, 128 if block else 0)
    if qc.get("quant_method") == "fp8":
        return _spec("fp8_block" if qc.get("weight_block_size") else "fp8", 8, 128)
    return None


# ------------------------------------------------------------------ nvfp4
def _nvfp4_detect(qc: dict):
    if qc.get("format") == "nvfp4-pack-quantized" or qc.get("quant_algo") == "NVFP4" or qc.get("quant_method") == "modelopt":
        return _spec("nvfp4", 4, 16)
    return None


# ------------------------------------------------------------------ gguf
def _gguf_detect(qc: dict):
    return _spec("gguf", 4, 256) if qc.get("quant_method") == "gguf" else None


def _unsupported(what: str):
    def fn(*_a, **_k):
        raise NotImplementedError(what)
    return fn


def extensions() -> list[QuantizationExtension]:
    return [
        QuantizationExtension(
            "none", ("weight",), ("bf16",), wq_pack.FMT_BF16, _none_detect,
            lambda p, shape, q: p["weight"].float(), lambda w, q: {"weight": w.to(torch.bfloat16)}, lambda q: None,
            "unquantized bf16 weights"),
        QuantizationExtension(
            "cubic", ("weight_packed", "weight_scale", "weight_a", "weight_b", "weight_ab", "weight_scale_global",
                      "weight_a_global", "weight_b_global", "weight_metadata", "weight_curve_a", "weight_curve_b"),
            ("w4a16",), wq_pack.FMT_CUBIC4, _cubic_detect,
            _plain_or(lambda p, shape, q: cubic.decode(p, cubic.CubicScheme(q.bits, q.group_size), shape)),
            lambda w, q: cubic.quantize(w, cubic.CubicScheme(q.bits, q.group_size)), _cubic_config,
            "CubicQuant: signed codes on a per-group cubic level curve (three metadata variants)"),
        QuantizationExtension(
            "int", ("weight_packed", "weight_scale", "weight_zero_point", "weight_shape", "weight_g_idx"),
            ("w4a16",), wq_pack.FMT_AFFINE4, _int_detect,
            _plain_or(lambda p, shape, q: formats.int_dense(p, q.bits, q.group_size, shape)),
            lambda w, q: formats.int_quantize(w, q.bits, q.group_size, True), _int_config,
            "compressed-tensors pack-quantized integers (2-8 bit, symmetric or with zero points)"),
        QuantizationExtension(
            "awq", ("qweight", "qzeros", "scales"), ("w4a16",), wq_pack.FMT_AFFINE4, _awq_detect,
            _plain_or(lambda p, shape, q: formats.awq_dense(p, q.group_size)), _awq_quantize,
            lambda q: {"quant_method": "awq", "bits": 4, "group_size": q.group_size, "version": "gemm", "zero_point": True},
            "AutoAWQ GEMM layout"),
        QuantizationExtension(
            "fp8", ("weight", "weight_scale", "input_scale"), ("w8a16",), None, _fp8_detect,
            _plain_or(lambda p, shape, q: formats.fp8_dense(p)), lambda w, q: formats.fp8_quantize(w, block=False),
            lambda q: {"quant_method": "compressed-tensors", "format": "float-quantized", "config_groups": {
                "group_0": {"targets": ["Linear"], "weights": {"num_bits": 8, "type": "float", "strategy": "channel"}}}},
            "e4m3 weights with one scale per output channel"),
        QuantizationExtension(
            "fp8_block", ("weight", "weight_scale_inv", "weight_scale"), ("w8a16",), None, lambda qc: None,
            _plain_or(lambda p, shape, q: formats.fp8_dense(p)), lambda w, q: formats.fp8_quantize(w, block=True),
            lambda q: {"quant_method": "fp8", "weight_block_size": [128, 128]},
            "e4m3 weights with one scale per 128 x 128 block (recognised by the fp8 extension's rule)"),
        QuantizationExtension(
            "nvfp4", ("weight_packed", "weight", "weight_scale", "weight_global_scale", "input_global_scale",
                      "weight_scale_2", "input_scale"),
            ("w4a16",), wq_pack.FMT_NVFP4, _nvfp4_detect,
            _plain_or(lambda p, shape, q: formats.nvfp4_dense(p)), lambda w, q: formats.nvfp4_quantize(w),
            lambda q: {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized", "config_groups": {
                "group_0": {"targets": ["Linear"], "weights": {"num_bits": 4, "type": "float", "group_size": 16}}}},
            "e2m1 codes with e4m3 scales per 16 columns (compressed-tensors and ModelOpt spellings)"),
        QuantizationExtension(
            "gguf", (), ("w4a16",), wq_pack.FMT_AFFINE4, _gguf_detect,
            _unsupported("GGUF tensors are decoded by quantization.gguf from the .gguf file, not from safetensors payloads"),
            _unsupported("GGUF files are written by quantization.gguf.q4k_quantize"),
            lambda q: {"quant_method": "gguf"},
            "GGUF files: Q4_K natively, the other block types through the reference dequantizers"),
    ]
