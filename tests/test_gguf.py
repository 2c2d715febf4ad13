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


def _write_toy_gguf(path, arch, rng, mixed=False, dims=(256, 4, 2, 64, 512, 320, 2)):
    """A two-layer llama-family GGUF as the converter writes it: metadata, Q4_K projections (optionally one of another
    block type), F32 norms, F16 embeddings; for ``llama`` the q / k rows go through the converter's ``permute``."""
    import gguf
    H, hq, hkv, D, I, V, L = dims
    w = gguf.GGUFWriter(str(path), arch)
    w.add_name("toy")
    w.add_block_count(L)
    w.add_embedding_length(H)
    w.add_head_count(hq)
    w.add_head_count_kv(hkv)
    w.add_feed_forward_length(I)
    w.add_rope_freq_base(50000.0)
    w.add_layer_norm_rms_eps(1e-5)
    w.add_context_length(4096)
    w.add_key_length(D)
    dense = {}

    def permute(x, heads):          # llama.cpp convert_hf_to_gguf.py LlamaModel.permute
        return x.reshape(heads, 2, x.shape[0] // heads // 2, *x.shape[1:]).swapaxes(1, 2).reshape(x.shape)

    def q4k(name, hf, n, k, heads=None, other=None):
        x = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
        stored = permute(x, heads) if (heads and arch == "llama") else x
        if other:
            raw = gguf.quants.quantize(stored, getattr(gguf.GGMLQuantizationType, other))
            deq = gguf.quants.dequantize(raw, getattr(gguf.GGMLQuantizationType, other))
            w.add_tensor(name, raw, raw_dtype=getattr(gguf.GGMLQuantizationType, other))
        else:
            raw = gq.q4k_quantize(stored)
            deq = gq.q4k_dense(raw)
            w.add_tensor(name, raw, raw_dtype=gguf.GGMLQuantizationType.Q4_K)
        # what the file represents, in logical (un-permuted) row order
        if heads and arch == "llama":
            inv = np.empty(n, dtype=np.int64)
            inv[permute(np.arange(n), heads)] = np.arange(n)
            deq = deq[inv]
        dense[hf] = deq.astype(np.float32)

    emb = (rng.standard_normal((V, H)) * 0.05).astype(np.float16)
    w.add_tensor("token_embd.weight", emb)
    dense["embed"] = emb.astype(np.float32)
    w.add_tensor("output_norm.weight", np.ones(H, dtype=np.float32))
    for i in range(L):
        q4k(f"blk.{i}.attn_q.weight", f"{i}.q", hq * D, H, heads=hq)
        q4k(f"blk.{i}.attn_k.weight", f"{i}.k", hkv * D, H, heads=hkv)
        q4k(f"blk.{i}.attn_v.weight", f"{i}.v", hkv * D, H, other="Q8_0" if mixed else None)
        q4k(f"blk.{i}.attn_output.weight", f"{i}.o", H, hq * D)
        q4k(f"blk.{i}.ffn_gate.weight", f"{i}.gate", I, H)
        q4k(f"blk.{i}.ffn_up.weight", f"{i}.up", I, H)
        q4k(f"blk.{i}.ffn_down.weight", f"{i}.down", H, I)
        dense[f"{i}.ln1"] = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        w.add_tensor(f"blk.{i}.attn_norm.weight", dense[f"{i}.ln1"])
        w.add_tensor(f"blk.{i}.ffn_norm.weight", np.ones(H, dtype=np.float32))
        if arch == "qwen3":
            w.add_tensor(f"blk.{i}.attn_q_norm.weight", np.ones(D, dtype=np.float32))
            w.add_tensor(f"blk.{i}.attn_k_norm.weight", np.ones(D, dtype=np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return dense


def _rel(a, b):
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.mark.parametrize("arch", ["llama", "qwen3"])
def test_gguf_file_to_decoder_weights(tmp_path, arch):
    from cubic_serve_b200.models.gguf import load_gguf_decoder_weights, qk_unpermute_order
    rng = np.random.default_rng(7)
    path = tmp_path / "toy.gguf"
    dense = _write_toy_gguf(path, arch, rng)
    cfg, w = load_gguf_decoder_weights(path)
    assert (cfg.num_layers, cfg.hidden_size, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim) == (2, 256, 4, 2, 64)
    assert cfg.intermediate_size == 512 and cfg.vocab_size == 320 and cfg.rope_theta == 50000.0 and cfg.tie_embeddings
    assert abs(cfg.rms_eps - 1e-5) < 1e-12 and cfg.qk_norm == (arch == "qwen3") and cfg.quant.method == "gguf" and cfg.quant.bits == 4
    l0 = w.layers[0]
    assert l0.qkv.fmt == wq_pack.FMT_AFFINE4 and l0.qkv.group_k == 32 and (l0.qkv.n, l0.qkv.k) == (512, 256)
    want = np.concatenate([dense["0.q"], dense["0.k"], dense["0.v"]])
    assert _rel(wq_pack.unpack_to_dense(l0.qkv)[:512].numpy(), want) < 6e-3        # bf16 rounding of scales only
    assert _rel(wq_pack.unpack_to_dense(w.layers[1].gate_up)[:1024].numpy(), np.concatenate([dense["1.gate"], dense["1.up"]])) < 6e-3
    assert _rel(wq_pack.unpack_to_dense(l0.down)[:256].numpy(), dense["0.down"]) < 6e-3
    assert (l0.q_norm is not None) == (arch == "qwen3")
    assert torch.allclose(w.embed.float(), torch.from_numpy(dense["embed"]), atol=1e-3) and w.lm_head.n == 320
    # tensor parallel: rank 1 of 2 owns the second half of the heads / features and the matching columns
    cfg2, w2 = load_gguf_decoder_weights(path, tp_rank=1, tp_size=2)
    q, k, v = dense["0.q"][128:], dense["0.k"][64:], dense["0.v"][64:]
    assert _rel(wq_pack.unpack_to_dense(w2.layers[0].qkv)[:256].numpy(), np.concatenate([q, k, v])) < 6e-3
    assert _rel(wq_pack.unpack_to_dense(w2.layers[0].o)[:256].numpy(), dense["0.o"][:, 128:]) < 6e-3
    assert _rel(wq_pack.unpack_to_dense(w2.layers[0].down)[:256].numpy(), dense["0.down"][:, 256:]) < 6e-3
    assert w2.vocab_start == 160 and w2.embed.shape[0] == 160
    order = qk_unpermute_order(8, 2)
    assert order.tolist() == [0, 2, 1, 3, 4, 6, 5, 7]


def test_gguf_mixed_block_types_and_closed_inventory(tmp_path):
    import gguf
    from cubic_serve_b200.models.gguf import load_gguf_decoder_weights
    rng = np.random.default_rng(8)
    path = tmp_path / "mixed.gguf"
    dense = _write_toy_gguf(path, "qwen2", rng, mixed=True)
    cfg, w = load_gguf_decoder_weights(path)
    assert cfg.quant.bits == 4                                    # the projections that decide it are Q4_K
    assert w.layers[0].qkv.fmt == wq_pack.FMT_BF16                # one part is Q8_0: the fused operand is decoded
    want = np.concatenate([dense["0.q"], dense["0.k"], dense["0.v"]])
    assert _rel(wq_pack.unpack_to_dense(w.layers[0].qkv).numpy(), want) < 4e-3
    assert w.layers[0].gate_up.fmt == wq_pack.FMT_AFFINE4
    from cubic_serve_b200.models.gguf import inspect_gguf
    info = inspect_gguf(path)
    assert info["served"] and info["architecture"] == "qwen2" and info["layers"] == 2 and info["heads"] == "4q/2kv x 64"
    assert info["types"]["Q4_K"] == 12 and info["types"]["Q8_0"] == 2 and not info["qk_rows_unpermuted"]
    bad = tmp_path / "bad.gguf"
    wtr = gguf.GGUFWriter(str(bad), "gpt2")
    wtr.add_block_count(1)
    wtr.add_tensor("token_embd.weight", np.zeros((4, 4), dtype=np.float32))
    wtr.write_header_to_file()
    wtr.write_kv_data_to_file()
    wtr.write_tensors_to_file()
    wtr.close()
    with pytest.raises(gq.GGUFFormatError, match="not served"):
        load_gguf_decoder_weights(bad)
    assert inspect_gguf(bad)["served"] is False and "not served" in inspect_gguf(bad)["reason"]


@pytest.mark.gpu
def test_gguf_model_decodes_like_the_eager_reference(tmp_path):
    """A GGUF file served by the native runner (Q4_K projections stay 4-bit) against the fp32 eager decoder run on
    the values the file represents."""
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner
    from cubic_serve_b200.models.gguf import load_gguf_decoder_weights
    from cubic_serve_b200.models.reference import DenseLayer, DenseWeights, EagerDecoder
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    rng = np.random.default_rng(11)
    path = tmp_path / "toy128.gguf"
    H, hq, hkv, D, I, V, L = dims = (512, 4, 2, 128, 1024, 512, 2)
    dense = _write_toy_gguf(path, "llama", rng, dims=dims)
    dev = torch.device("cuda")
    cfg, w = load_gguf_decoder_weights(path, dev)
    runner = DecoderRunner(cfg, w, num_pages=64, max_tokens=256)
    ex = GpuExecutor(runner, max_rows=4, max_prefill_tokens=256, max_model_len=128, use_graphs=False)
    eng = LLMEngine(ex, 64, SchedulerConfig(max_running_requests=4, max_model_len=128, max_batched_tokens=256,
                                            enable_prefix_cache=False))
    prompts = [rng.integers(0, V, n).tolist() for n in (12, 12)]
    got = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    runner.ws.check_status()
    t = lambda k: torch.from_numpy(dense[k])  # noqa: E731
    layers = [DenseLayer(t(f"{i}.ln1"), torch.ones(H), t(f"{i}.q"), t(f"{i}.k"), t(f"{i}.v"), t(f"{i}.o"), t(f"{i}.gate"),
                         t(f"{i}.up"), t(f"{i}.down")) for i in range(L)]
    ref = EagerDecoder(cfg, DenseWeights(t("embed"), layers, torch.ones(H), t("embed")), kv_bits=(8, 8))
    want, _ = ref.generate(torch.tensor(prompts), 8)
    agree = np.mean([a == b for ga, wa in zip(got, want.tolist()) for a, b in zip(ga, wa)])
    assert agree >= 0.75, (agree, got, want.tolist())


def _metadata_only_file(path, arch="llama", scaling=None, table=None):
    """A file with the metadata and the two tensors the configuration reader needs."""
    import gguf
    w = gguf.GGUFWriter(str(path), arch)
    w.add_block_count(1)
    w.add_embedding_length(64)
    w.add_head_count(4)
    w.add_head_count_kv(2)
    w.add_feed_forward_length(128)
    w.add_rope_freq_base(500000.0)
    w.add_key_length(16)
    w.add_context_length(4096)
    if scaling:
        kind, factor, original = scaling
        w.add_rope_scaling_type(getattr(gguf.RopeScalingType, kind))
        w.add_rope_scaling_factor(factor)
        if original:
            w.add_rope_scaling_orig_ctx_len(original)
    w.add_tensor("token_embd.weight", np.zeros((32, 64), dtype=np.float16))
    if table is not None:
        w.add_tensor("rope_freqs.weight", np.asarray(table, dtype=np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    import gguf as g2
    return g2.GGUFReader(str(path))


def test_rotary_scaling_of_a_gguf_file_is_served_not_dropped(tmp_path):
    """The exporter's divisor table (its form of the llama3 rule) and the linear / yarn metadata reach the frequency
    table; a file that announces a form this build does not serve is refused."""
    import math

    from cubic_serve_b200.models.gguf import config_from_gguf
    from cubic_serve_b200.ops import eager
    plain = eager.rope_inv_freq(16, 500000.0)
    want = eager.rope_inv_freq(16, 500000.0, scaling=("llama3", 8.0, 1.0, 4.0, 64))
    table = (plain / want).tolist()                               # what the converter stores: base frequency / scaled one
    cfg = config_from_gguf(_metadata_only_file(tmp_path / "a.gguf", table=table))
    assert cfg.rope_scaling[0] == "factors"
    assert torch.allclose(eager.rope_inv_freq(16, 500000.0, scaling=cfg.rope_scaling), want, rtol=1e-6)
    assert config_from_gguf(_metadata_only_file(tmp_path / "b.gguf")).rope_scaling is None
    assert config_from_gguf(_metadata_only_file(tmp_path / "c.gguf", scaling=("LINEAR", 4.0, None))).rope_scaling == ("linear", 4.0)
    y = config_from_gguf(_metadata_only_file(tmp_path / "d.gguf", arch="qwen3", scaling=("YARN", 4.0, 1024)))
    assert y.rope_scaling[:5] == ("yarn", 4.0, 1024, 32.0, 1.0) and abs(y.rope_scaling[5] - (0.1 * math.log(4) + 1)) < 1e-12
    assert y.attention_scale is not None
    with pytest.raises(gq.GGUFFormatError, match="one divisor per rotary slot"):
        config_from_gguf(_metadata_only_file(tmp_path / "e.gguf", table=[1.0] * 5))
    with pytest.raises(gq.GGUFFormatError, match="both"):
        config_from_gguf(_metadata_only_file(tmp_path / "f.gguf", scaling=("YARN", 4.0, 1024), table=table))
    if hasattr(__import__("gguf").RopeScalingType, "LONGROPE"):
        with pytest.raises(gq.GGUFFormatError, match="longrope"):
            config_from_gguf(_metadata_only_file(tmp_path / "g.gguf", scaling=("LONGROPE", 4.0, 1024)))
