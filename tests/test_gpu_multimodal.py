"""Three-axis rotary positions and encoder feature rows on the native runner (one GPU)."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec
from cubic_serve_b200.ops import eager

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rotary,section", [(128, (24, 20, 20)), (64, (11, 11, 10))])
def test_cache_write_kernel_rotates_by_axis(rotary, section):
    """Queries out of the cache-write kernel against the fp32 three-axis rotation of the same inputs; equal axes give the
    one-axis kernel's bits."""
    from cubic_serve_b200.ops import kernels as K
    dev = torch.device("cuda")
    T, hq, hkv, D = 37, 4, 2, 128
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(T, (hq + 2 * hkv) * D, generator=g).to(torch.bfloat16).to(dev)
    pos = torch.randint(0, 4000, (3, T), generator=g, dtype=torch.int32)
    inv = eager.rope_inv_freq(rotary, 1e6)
    cache = torch.zeros(4, hkv, K.kv_blob_bytes(D, 8, 8), dtype=torch.uint8, device=dev)
    slots = torch.full((T,), -1, dtype=torch.int32, device=dev)            # queries only: nothing is written
    q = torch.empty(T, hq * D, dtype=torch.bfloat16, device=dev)
    p = pos.to(dev)
    K.rope_kv_write(qkv, q, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary,
                    positions_hw=(p[1].contiguous(), p[2].contiguous()), mrope_section=section)
    want = eager.rope3(qkv[:, :hq * D].float().cpu().view(T, hq, D), pos.long(), inv, section).reshape(T, hq * D)
    got = q.float().cpu()
    assert ((got - want).norm() / want.norm()).item() < 4e-3
    one = torch.empty_like(q)
    K.rope_kv_write(qkv, one, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary)
    same = torch.empty_like(q)
    K.rope_kv_write(qkv, same, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary,
                    positions_hw=(p[0].contiguous(), p[0].contiguous()), mrope_section=section)
    assert torch.equal(same, one) and not torch.equal(q, one)
    with pytest.raises(ValueError):
        K.rope_kv_write(qkv, q, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary,
                        positions_hw=(p[1].contiguous(), p[2].contiguous()), mrope_section=(1, 1, 1))


def _engine(chunk=512):
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="mm", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, mrope_section=(24, 20, 20),
                      quant=QuantSpec("cubic", 4, 128))
    w = random_decoder_weights(cfg, dev, seed=0, std=0.05)
    runner = DecoderRunner(cfg, w, num_pages=256, max_tokens=512)
    ex = GpuExecutor(runner, max_rows=8, max_prefill_tokens=512, max_model_len=256)
    ex.capture_decode_graphs()
    eng = LLMEngine(ex, 256, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                             prefill_chunk_tokens=chunk))
    return eng, ex, w


def _run(eng, prompt, mm, n=8):
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rid = eng.add_request(prompt, SamplingParams(max_tokens=n, ignore_eos=True), multimodal=mm)
    out = []
    while eng.has_unfinished:
        out += [o.token_id for o in eng.step() if o.request_id == rid and o.token_id is not None]
    return out


def test_native_runner_takes_feature_rows_and_axes():
    from cubic_serve_b200.models.vision import mrope_positions
    from cubic_serve_b200.runtime.multimodal import MultimodalInput
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 2048, 70).tolist()
    eng, ex, w = _engine()
    assert ex.accepts_features
    plain = _run(eng, prompt, None)
    embed = w.extras["embed_full"] if "embed_full" in w.extras else w.embed
    own = embed[torch.tensor(prompt[5:29], device=embed.device)].float().cpu()         # the rows' own embeddings
    line = np.stack([np.arange(70)] * 3)

    def mm(rows, positions, delta, digest):
        return MultimodalInput([(5, rows, digest)], positions, delta)
    # feature rows equal to the embeddings they replace, positions equal on all axes: nothing changes
    assert _run(_engine()[0], prompt, mm(own, line, 0, b"own")) == plain
    # other rows, or a grid on the row / column axes, change the continuation
    feats = torch.randn(24, 512, generator=torch.Generator().manual_seed(1)) * own.std()
    a = _run(_engine()[0], prompt, mm(feats, line, 0, b"f"))
    assert a != plain
    pos, delta = mrope_positions(prompt, [(5, 24, (1, 8, 12))], 2)
    b = _run(_engine()[0], prompt, mm(feats, np.asarray(pos), delta, b"f"))
    assert b != a and delta < 0
    # chunked prefill cuts the media span: the same tokens; and the cached pages of equal media are reused
    assert _run(_engine(chunk=16)[0], prompt, mm(feats, np.asarray(pos), delta, b"f")) == b
    eng2 = _engine()[0]
    first = _run(eng2, prompt, mm(feats, np.asarray(pos), delta, b"f"))
    hits = eng2.prefix.hit_tokens
    again = _run(eng2, prompt, mm(feats, np.asarray(pos), delta, b"f"))
    assert first == b and again == b and eng2.prefix.hit_tokens > hits
    other = _run(eng2, prompt, mm(own, np.asarray(pos), delta, b"g"))             # other media: its span is not shared
    assert other != b


def test_multimodal_checkpoint_served_by_the_native_runner(tmp_path):
    """Checkpoint with a vision tower -> native weights + tower on the GPU -> chat request with an image through the
    media processor -> tokens; the same image again comes from the feature store, another image changes the answer."""
    import base64
    import io
    import json
    from argparse import Namespace

    from PIL import Image
    from safetensors.torch import load_file, save_file

    from cubic_serve_b200.contracts.request import CanonicalChatRequest, ContentPart, Message, Role
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models.decoder import DecoderRunner
    from cubic_serve_b200.models.vision import VisionConfig, random_vision_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    from cubic_serve_b200.runtime.serving import build_media_processor
    dev = torch.device("cuda")
    base = ModelConfig(name="Qwen3ForCausalLM", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                       intermediate_size=1024, vocab_size=1024, rope_theta=1e6, qk_norm=True, quant=QuantSpec("cubic", 4, 128))
    path = C.write_random_checkpoint(tmp_path / "mm", base, seed=2, std=0.05)
    t = load_file(str(path / "model.safetensors"))
    nested = {("model.language_model." + n[len("model."):] if n.startswith("model.") else n): v for n, v in t.items()}
    raw_v = dict(depth=2, hidden_size=64, hidden_act="gelu_pytorch_tanh", intermediate_size=128, num_heads=4, in_channels=3,
                 patch_size=4, spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=512, num_position_embeddings=64,
                 deepstack_visual_indexes=[])
    vcfg = VisionConfig.from_hf(raw_v)
    nested.update({"model.visual." + n: v.to(torch.bfloat16) for n, v in random_vision_weights(vcfg, 9, std=0.2).items()})
    save_file(nested, str(path / "model.safetensors"))
    raw = json.loads((path / "config.json").read_text())
    text = {k: v for k, v in raw.items() if k != "architectures"}
    text["rope_parameters"] = {"mrope_section": [24, 20, 20], "rope_theta": 1e6}
    doc = {"architectures": raw["architectures"], "text_config": text, "image_token_id": 261, "video_token_id": 262,
           "vision_start_token_id": 259, "vision_end_token_id": 260, "vision_config": {**raw_v, "model_type": "x"}}
    if "quantization_config" in raw:
        doc["quantization_config"] = raw["quantization_config"]
    (path / "config.json").write_text(json.dumps(doc))
    ck = C.admit_checkpoint(path)
    assert ck.vision is not None and ck.cfg.mrope_section == (24, 20, 20)
    runner = DecoderRunner(ck.cfg, C.load_decoder_weights(ck, dev), num_pages=128, max_tokens=512)
    ex = GpuExecutor(runner, max_rows=4, max_prefill_tokens=512, max_model_len=256)
    ex.capture_decode_graphs()
    assert ex.accepts_features

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    proc = build_media_processor(Namespace(thinking=None, encoder_memory_gib=0.25, feature_store_mib=4), ck, tok, ex, 256)
    assert proc is not None and str(proc.vision.encoder.device).startswith("cuda")
    proc.geometry = replace(proc.geometry, min_pixels=8 * 8, max_pixels=32 * 32)

    def url(seed):
        arr = np.random.default_rng(seed).integers(0, 256, (24, 40, 3), dtype=np.uint8)
        buf = io.BytesIO()
        Image.fromarray(arr).save(buf, "PNG")
        return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

    def ask(seed):
        msg = Message(Role.USER, (ContentPart("text", "see "), ContentPart("image", media_url=url(seed)), ContentPart("text", "?")))
        out = proc.build(CanonicalChatRequest("openai", "m", (msg,), request_id=f"r{seed}"))
        eng = LLMEngine(ex, 128, SchedulerConfig(max_running_requests=4, max_model_len=256, max_batched_tokens=512))
        return _run(eng, out.token_ids, out.multimodal, n=8), out
    a, plan_a = ask(1)
    again, _ = ask(1)
    b, _ = ask(2)
    assert len(a) == 8 and again == a and proc.vision.store.hits >= 1
    assert b != a
    first, rows, _ = plan_a.multimodal.spans[0]
    assert rows.shape == (15, 512) and plan_a.token_ids[first - 1] == 259
    runner.ws.check_status()
