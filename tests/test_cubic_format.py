import math

import pytest
import torch

from cubic_serve_b200.ops import wq_pack
from cubic_serve_b200.quantization import cubic


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_bitstream_roundtrip(bits):
    g = torch.Generator().manual_seed(bits)
    k = 37
    if bits == 1:
        codes = torch.randint(0, 2, (5, k), generator=g) * 2 - 1
    else:
        lim = (1 << (bits - 1)) - 1
        codes = torch.randint(-lim, lim + 1, (5, k), generator=g)
    packed = cubic.pack_codes(codes.to(torch.int8), bits)
    assert packed.shape == (5, math.ceil(k * bits / 8))
    assert torch.equal(cubic.unpack_codes(packed, bits, k).long(), codes)


def test_reserved_code_decodes_to_zero_and_bit_order():
    # 4-bit: byte 0x8F -> low nibble 0xF = -1, high nibble 0x8 = reserved -> 0
    packed = torch.tensor([[0x8F, 0x17]], dtype=torch.uint8)
    assert cubic.unpack_codes(packed, 4, 4).tolist() == [[-1, 0, 7, 1]]
    # 3-bit little-endian bitstream: codes 1, -2(110), 3 -> bits 100 011 110 -> 0b10110001 (+1 bit)
    codes = torch.tensor([[1, -2, 3]], dtype=torch.int8)
    p = cubic.pack_codes(codes, 3)
    assert p.tolist() == [[0b11110001, 0b0]]
    assert cubic.unpack_codes(p, 3, 3).tolist() == [[1, -2, 3]]


def test_decode_formula_variant_a():
    scheme = cubic.CubicScheme(bits=4, group_in=4)
    codes = torch.tensor([[7, -7, 3, 0, 1, -1, 2, -8]], dtype=torch.int8)
    payload = {
        "weight_packed": cubic.pack_codes(codes, 4),
        "weight_scale": torch.tensor([[2.0, 0.5]]),
        "weight_a": torch.tensor([[0.75, 1.0]], dtype=torch.float16),
        "weight_b": torch.tensor([[0.5, 0.0]], dtype=torch.float16),
    }
    w = cubic.decode(payload, scheme, (1, 8))
    t = 3 / 7
    f = t * (0.75 + t * (0.5 + t * (1 - 0.75 - 0.5)))
    assert torch.allclose(w[0, :4], torch.tensor([2.0, -2.0, 2.0 * f, 0.0]), atol=1e-6)
    assert torch.allclose(w[0, 4:], torch.tensor([0.5 / 7, -0.5 / 7, 1.0 / 7, 0.0]), atol=1e-6)


def test_variant_b_and_c_metadata():
    n, k = 4, 8
    codes = torch.randint(-7, 8, (n, k), generator=torch.Generator().manual_seed(0)).to(torch.int8)
    sb = cubic.CubicScheme(bits=4, group_in=4, metadata=cubic.METADATA_B)
    payload = {
        "weight_packed": cubic.pack_codes(codes, 4),
        "weight_scale": torch.tensor([[10, 20]] * n, dtype=torch.int8),
        "weight_ab": torch.tensor([[0x1F, 0x20]] * n, dtype=torch.uint8),  # a4=-1,b4=1 ; a4=0,b4=2
        "weight_scale_global": torch.tensor([0.01, 0.02]),
        "weight_a_global": torch.tensor([0.1, 0.1]),
        "weight_b_global": torch.tensor([0.05, 0.05]),
    }
    s, a, b = cubic.metadata_triple(payload, sb, (n, k), (2, 2))
    assert torch.allclose(s[0], torch.tensor([0.1, 0.2])) and torch.allclose(s[3], torch.tensor([0.2, 0.4]))
    assert torch.allclose(a[0].float(), torch.tensor([0.9, 1.0]), atol=1e-3)
    assert torch.allclose(b[0].float(), torch.tensor([0.05, 0.1]), atol=1e-3)
    assert cubic.decode(payload, sb, (n, k), (2, 2)).shape == (n, k)
    sc = cubic.CubicScheme(bits=4, group_in=4, metadata=cubic.METADATA_C)
    half_bits = torch.tensor([1.5], dtype=torch.float16).view(torch.int16).item()
    word = ((half_bits >> 1) & 0x3FFF) | (2 << 14)
    payload_c = {
        "weight_packed": cubic.pack_codes(codes, 4),
        "weight_metadata": torch.full((n, 2), word, dtype=torch.int32).to(torch.uint16),
        "weight_curve_a": torch.tensor([[1.0, 0.9, 0.8, 0.7]], dtype=torch.float16),
        "weight_curve_b": torch.tensor([[0.0, 0.1, 0.2, 0.3]], dtype=torch.float16),
    }
    s, a, b = cubic.metadata_triple(payload_c, sc, (n, k))
    assert torch.allclose(s, torch.full((n, 2), 1.5)) and float(a[0, 0]) == pytest.approx(0.8, abs=1e-3)
    assert float(b[0, 0]) == pytest.approx(0.2, abs=1e-3)


def test_quantizer_error_and_pack_roundtrip():
    w = torch.randn(200, 512, generator=torch.Generator().manual_seed(0)) * 0.02
    scheme = cubic.CubicScheme(bits=4, group_in=128)
    p = cubic.quantize(w, scheme)
    assert p["weight_packed"].shape == (200, 256) and p["weight_scale"].shape == (200, 4)
    d = cubic.decode(p, scheme, (200, 512))
    assert ((d - w).norm() / w.norm()).item() < 0.12
    codes = cubic.unpack_codes(p["weight_packed"], 4, 512)
    pw = wq_pack.pack_cubic4(codes, p["weight_scale"], p["weight_a"], p["weight_b"], 128)
    assert pw.codes.shape == (2, 8, 2, 128, 16)
    # the packed metadata holds the curve coefficients rounded to bf16
    assert ((wq_pack.unpack_to_dense(pw) - d).norm() / d.norm()).item() < 4e-3


def test_bad_payload_rejected():
    scheme = cubic.CubicScheme()
    with pytest.raises(cubic.CubicFormatError):
        cubic.unpack_codes(torch.zeros(2, 3, dtype=torch.uint8), 4, 128)
    with pytest.raises(cubic.CubicFormatError):
        cubic.metadata_triple({"weight_scale": torch.zeros(2, 1)}, scheme, (2, 128))
