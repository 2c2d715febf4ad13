import numpy as np
import pytest
import torch

from cubic_serve_b200.models.gguf import hf_name
from cubic_serve_b200.ops import wq_pack
from cubic_serve_b200.quantization import gguf as gq


def test_q4k_matches_the_gguf_library_decoder():
    import gguf
    rng = np.random.default_rng(0)
    raw = rng.integers(0, 256, size=(6, 2 * gq.Q4K_BLOCK_BYTES), dtype=np.uint8)
    # keep d / dmin finite fp16 values
    raw = raw.reshape(6, 2, gq.Q4K_BLOCK_BYTES)
    raw[..., 0:4] = np.array([0.01, 0.02], dtype=np.float16).view(np.uint8)
    raw = raw.reshape(6, -1)
    ref = gguf.quants.dequantize(raw, gguf.GGMLQuantizationType.Q4_K)
    mine = gq.q4k_dense(raw)
    assert mine.shape == (6, 512) and np.allclose(mine, ref, atol=1e-6)


def test_q4k_quantize_roundtrip_and_gemm_operand():
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((128, 512)) * 0.02).astype(np.float32)
    raw = gq.q4k_quantize(w)
    assert raw.shape == (128, 2 * gq.Q4K_BLOCK_BYTES)
    d = gq.q4k_dense(raw)
    assert np.linalg.norm(d - w) / np.linalg.norm(w) < 0.12
    pw = gq.to_packed_weight("Q4_K", raw, (128, 512))
    assert pw.fmt == wq_pack.FMT_AFFINE4 and pw.group_k == 32
    got = wq_pack.unpack_to_dense(pw).numpy()
    assert np.linalg.norm(got - d) / np.linalg.norm(d) < 6e-3


def test_library_backed_types_and_rejection():
    import gguf
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((4, 64)) * 0.1).astype(np.float32)
    q8 = gguf.quants.quantize(w, gguf.GGMLQuantizationType.Q8_0)
    d = gq.dense("Q8_0", q8, (4, 64))
    assert np.abs(d - w).max() < 2e-3
    assert gq.to_packed_weight("Q8_0", q8, (4, 64)).fmt == wq_pack.FMT_BF16
    bf = torch.from_numpy(w).to(torch.bfloat16)
    assert np.allclose(gq.dense("BF16", bf.view(torch.int16).numpy(), (4, 64)), bf.float().numpy())
    with pytest.raises(gq.GGUFFormatError):
        gq.to_packed_weight("Q2_K", q8, (4, 64))


def test_name_mapping():
    assert hf_name("blk.3.attn_q.weight") == "model.layers.3.self_attn.q_proj.weight"
    assert hf_name("blk.0.ffn_down.weight") == "model.layers.0.mlp.down_proj.weight"
    assert hf_name("token_embd.weight") == "model.embed_tokens.weight"
    with pytest.raises(gq.GGUFFormatError):
        hf_name("blk.0.mystery.weight")
