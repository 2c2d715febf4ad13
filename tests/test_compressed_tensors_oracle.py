"""Payloads written by the ``compressed-tensors`` library (the format of the INT / FP8 checkpoints on the hub) decoded by
this build's loaders against the library's own decompression.  Skipped when the library is not importable."""
import pytest
import torch

from cubic_serve_b200.models import checkpoint as C
from cubic_serve_b200.models.config import QuantSpec


def _compress(name, args, seed=0):
    ct = pytest.importorskip("compressed_tensors")
    from compressed_tensors.compressors import BaseCompressor
    from compressed_tensors.quantization import QuantizationScheme
    from compressed_tensors.quantization.utils import calculate_qparams
    c = BaseCompressor.load_from_registry(name)
    scheme = QuantizationScheme(targets=["Linear"], weights=args)
    w = torch.randn(256, 512, generator=torch.Generator().manual_seed(seed)) * 0.05
    if args.strategy == "group":
        g = w.view(256, -1, args.group_size)
        mn, mx = g.amin(-1), g.amax(-1)
    else:
        mn, mx = w.amin(-1, keepdim=True), w.amax(-1, keepdim=True)
    scale, zp = calculate_qparams(mn, mx, args)
    out = c.compress({"weight": w, "weight_scale": scale, "weight_zero_point": zp}, scheme)
    payload = {k: v for k, v in out.items() if v is not None}
    want = c.decompress(dict(out), scheme)["weight"].float()
    return w, payload, want


@pytest.mark.parametrize("bits,symmetric", [(4, True), (4, False), (8, True), (8, False)])
def test_pack_quantized_payloads(bits, symmetric):
    pytest.importorskip("compressed_tensors")
    from compressed_tensors.quantization import QuantizationArgs
    args = QuantizationArgs(num_bits=bits, type="int", symmetric=symmetric, strategy="group", group_size=128)
    w, payload, want = _compress("pack-quantized", args)
    assert set(payload) == {"weight_packed", "weight_scale", "weight_shape"} | ({"weight_zero_point"} if not symmetric else set())
    got = C._dense_of("int", payload, (256, 512), QuantSpec("int", bits, 128)).float()
    assert torch.allclose(got, want, atol=1e-6), float((got - want).abs().max())
    # a row slice, as a tensor-parallel rank or a per-head gather takes it
    part = C._slice_rows(payload, "int", 64, 192, 256, bits)
    got_part = C._dense_of("int", part, (128, 512), QuantSpec("int", bits, 128)).float()
    assert torch.allclose(got_part, want[64:192], atol=1e-6)


def test_float_quantized_payloads():
    pytest.importorskip("compressed_tensors")
    from compressed_tensors.quantization import QuantizationArgs
    args = QuantizationArgs(num_bits=8, type="float", symmetric=True, strategy="channel")
    w, payload, want = _compress("float-quantized", args, seed=1)
    assert payload["weight"].dtype == torch.float8_e4m3fn
    got = C._dense_of("fp8", payload, (256, 512), QuantSpec("fp8", 8, 0)).float()
    assert torch.allclose(got, want, atol=1e-6), float((got - want).abs().max())


def test_nvfp4_pack_quantized_payloads(monkeypatch):
    """NVFP4 (e2m1 codes, e4m3 scales per 16 weights, one fp32 global scale): the library's payload decoded here equals the
    library's decompression, and this build's own quantizer writes a payload the library decodes to the same weights."""
    pytest.importorskip("compressed_tensors")
    import torch._dynamo
    from compressed_tensors.compressors import BaseCompressor
    from compressed_tensors.quantization import QuantizationArgs, QuantizationScheme
    from compressed_tensors.quantization.utils import calculate_qparams, generate_gparam

    from cubic_serve_b200.quantization import formats
    monkeypatch.setattr(torch._dynamo.config, "disable", True)            # the library's packers are compiled lazily
    c = BaseCompressor.load_from_registry("nvfp4-pack-quantized")
    args = QuantizationArgs(num_bits=4, type="float", symmetric=True, strategy="tensor_group", group_size=16,
                            scale_dtype=torch.float8_e4m3fn)
    scheme = QuantizationScheme(targets=["Linear"], weights=args)
    w = torch.randn(128, 256, generator=torch.Generator().manual_seed(2)) * 0.05
    gs = generate_gparam(w.min().reshape(1), w.max().reshape(1))
    g = w.view(128, -1, 16)
    scale, zp = calculate_qparams(g.amin(-1), g.amax(-1), args, global_scale=gs)
    out = c.compress({"weight": w, "weight_scale": scale, "weight_zero_point": zp, "weight_global_scale": gs}, scheme)
    payload = {k: v for k, v in out.items() if v is not None}
    dec = c.decompress(dict(out), scheme)["weight"]
    want = dec.float()
    got = formats.nvfp4_dense(payload).float()
    # the library multiplies code, block scale and 1 / global scale in its compute dtype; here the product is fp32
    tol = 1e-6 if dec.dtype == torch.float32 else 2 ** -7
    assert float(((got - want).abs() / want.abs().clamp_min(1e-6)).max()) <= tol, (dec.dtype, float((got - want).abs().max()))
    mine = formats.nvfp4_quantize(w)
    assert mine["weight_packed"].shape == payload["weight_packed"].shape and mine["weight_scale"].dtype == torch.float8_e4m3fn
    theirs = c.decompress({k: mine[k] for k in ("weight_packed", "weight_scale", "weight_global_scale")}, scheme)["weight"].float()
    ours = formats.nvfp4_dense(mine).float()
    assert float(((theirs - ours).abs() / ours.abs().clamp_min(1e-6)).max()) <= tol
    assert float((theirs - w).norm() / w.norm()) < 0.12
