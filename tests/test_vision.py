"""Vision tower, patch preprocessing, feature store / encoder service and the multimodal path through the engine
(CPU).  The tower and the patch cutter are checked against the HuggingFace implementations of the same public
architecture when those are importable."""
import base64
import io
import threading

import numpy as np
import pytest
import torch

from cubic_serve_b200.executor.vision import (EncodedFeatureStore, EncoderCapacityError, EncoderMemoryPlan, VisionService,
                                              media_digest)
from cubic_serve_b200.inputs.vision_patches import (PatchGeometry, VisionInputError, decode_image, patchify_frames,
                                                    patchify_image, patchify_video, smart_resize)
from cubic_serve_b200.models.vision import (VisionConfig, VisionConfigError, VisionEncoder, check_vision_weights,
                                            mrope_positions, random_vision_weights, shard_vision_weights)
from cubic_serve_b200.ops import eager

RAW = dict(depth=2, hidden_size=64, hidden_act="gelu_pytorch_tanh", intermediate_size=128, num_heads=4, in_channels=3,
           patch_size=4, spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=32, num_position_embeddings=64,
           deepstack_visual_indexes=[])


def _cfg(**kw) -> VisionConfig:
    return VisionConfig.from_hf({**RAW, **kw})


# ------------------------------------------------------------------ tower
@pytest.mark.parametrize("deep", [[], [0]])
def test_tower_matches_the_public_implementation(deep):
    hf_cfg = pytest.importorskip("transformers.models.qwen3_vl.configuration_qwen3_vl")
    hf_mod = pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
    c = hf_cfg.Qwen3VLVisionConfig(**{**RAW, "deepstack_visual_indexes": deep})
    c._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = hf_mod.Qwen3VLVisionModel(c).eval()
    for p in ref.parameters():
        p.data.normal_(0, 0.1)
    cfg = _cfg(deepstack_visual_indexes=deep)
    w = {n: p.detach().clone() for n, p in ref.named_parameters()}
    check_vision_weights(cfg, w)
    grid = torch.tensor([[1, 4, 6], [2, 2, 2], [1, 10, 4]])
    px = torch.randn(int(grid.prod(-1).sum()), cfg.patch_width)
    with torch.no_grad():
        out = ref(px, grid_thw=grid)
    mine, deepstack = VisionEncoder(cfg, w).encode(px, grid)
    assert mine.shape == out.pooler_output.shape == (18, 32)
    assert (mine - out.pooler_output).abs().max() < 1e-5
    if deep:
        assert (deepstack[0] - out.deepstack_features[0]).abs().max() < 1e-5


def test_frames_are_independent_and_rows_follow_the_grid():
    cfg = _cfg()
    enc = VisionEncoder(cfg, random_vision_weights(cfg, 1))
    g = torch.Generator().manual_seed(2)
    a, b = torch.randn(24, cfg.patch_width, generator=g), torch.randn(16, cfg.patch_width, generator=g)
    both, _ = enc.encode(torch.cat([a, b]), torch.tensor([[1, 4, 6], [1, 4, 4]]))
    ra, _ = enc.encode(a, torch.tensor([[1, 4, 6]]))
    rb, _ = enc.encode(b, torch.tensor([[1, 4, 4]]))
    assert both.shape == (10, 32)
    assert torch.allclose(both, torch.cat([ra, rb]), atol=1e-6)
    with pytest.raises(ValueError):
        enc.encode(a, torch.tensor([[1, 4, 5]]))                # width not a whole number of merge blocks
    with pytest.raises(ValueError):
        enc.encode(a[:, :-1], torch.tensor([[1, 4, 6]]))


def test_sharded_tower_sums_to_the_whole():
    cfg = _cfg()
    w = random_vision_weights(cfg, 3)
    px = torch.randn(24, cfg.patch_width, generator=torch.Generator().manual_seed(4))
    grid = torch.tensor([[1, 4, 6]])
    want, _ = VisionEncoder(cfg, w).encode(px, grid)
    size = 2
    barrier = threading.Barrier(size)
    slots: list = [None] * size
    out: list = [None] * size

    def rank(r: int) -> None:
        def reduce(t: torch.Tensor) -> torch.Tensor:
            slots[r] = t
            barrier.wait()
            total = sum(slots[i] for i in range(size))          # ascending rank order on every rank
            barrier.wait()
            return total
        enc = VisionEncoder(cfg, shard_vision_weights(cfg, w, r, size), r, size, reduce)
        out[r] = enc.encode(px, grid)[0]
    ts = [threading.Thread(target=rank, args=(r,)) for r in range(size)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert torch.equal(out[0], out[1])
    assert (out[0] - want).abs().max() < 1e-5
    with pytest.raises(VisionConfigError):
        shard_vision_weights(cfg, w, 0, 3)
    with pytest.raises(ValueError):
        VisionEncoder(cfg, w, 0, 2)


def test_config_is_strict():
    with pytest.raises(VisionConfigError):
        _cfg(surprise=1)
    with pytest.raises(VisionConfigError):
        _cfg(num_position_embeddings=60)
    with pytest.raises(VisionConfigError):
        _cfg(deepstack_visual_indexes=[5])
    with pytest.raises(VisionConfigError):
        check_vision_weights(_cfg(), {})


# ------------------------------------------------------------------ patches
@pytest.mark.parametrize("hw", [(70, 123), (224, 224), (31, 500)])
def test_patches_match_the_public_image_processor(hw):
    mod = pytest.importorskip("transformers.models.qwen2_vl.image_processing_qwen2_vl")
    from PIL import Image
    arr = np.random.default_rng(0).integers(0, 256, (*hw, 3), dtype=np.uint8)
    img = Image.fromarray(arr)
    geo = PatchGeometry(16, 2, 2, min_pixels=64 * 64, max_pixels=256 * 256)
    proc = mod.Qwen2VLImageProcessor(patch_size=16, merge_size=2, temporal_patch_size=2, min_pixels=64 * 64,
                                     max_pixels=256 * 256, image_mean=[0.5] * 3, image_std=[0.5] * 3)
    want = proc(images=[img], return_tensors="pt")
    mine = patchify_image(img, geo)
    assert list(mine.grid) == want["image_grid_thw"][0].tolist()
    assert np.abs(want["pixel_values"].numpy() - mine.pixels).max() < 1e-6


def test_resize_and_patch_order():
    assert smart_resize(100, 100, 32, 32 * 32, 1 << 20) == (96, 96)
    h, w = smart_resize(4000, 3000, 32, 32 * 32, 256 * 256)
    assert h % 32 == 0 and w % 32 == 0 and h * w <= 256 * 256
    h, w = smart_resize(10, 20, 32, 64 * 64, 1 << 20)
    assert h * w >= 64 * 64
    with pytest.raises(VisionInputError):
        smart_resize(1, 500, 32, 1, 1 << 20)
    # merge-block order: rows 0..3 of the output are the 2 x 2 block at the top left
    geo = PatchGeometry(2, 2, 1, mean=(0.0,), std=(1.0,))
    frame = np.zeros((1, 8, 8, 1), dtype=np.uint8)
    for r in range(4):
        for c in range(4):
            frame[0, 2 * r:2 * r + 2, 2 * c:2 * c + 2, 0] = r * 4 + c
    p = patchify_frames(frame, geo)
    assert p.grid == (1, 4, 4) and p.pixels.shape == (16, 4)
    ids = np.rint(p.pixels[:, 0] * 255).astype(int).tolist()
    assert ids == [0, 1, 4, 5, 2, 3, 6, 7, 8, 9, 12, 13, 10, 11, 14, 15]
    # an odd number of frames is padded with the last one
    geo2 = PatchGeometry(2, 2, 2, mean=(0.0,), std=(1.0,))
    three = np.stack([np.full((4, 4, 1), v, dtype=np.uint8) for v in (10, 20, 30)])
    v = patchify_frames(three, geo2)
    assert v.grid == (2, 2, 2) and v.rows(2) == 2
    assert np.allclose(v.pixels[4:, :] * 255, 30)


def _png(h: int, w: int, seed: int = 0, mode: str = "RGB") -> bytes:
    from PIL import Image
    ch = {"RGB": 3, "RGBA": 4}[mode]
    arr = np.random.default_rng(seed).integers(0, 256, (h, w, ch), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr, mode).save(buf, "PNG")
    return buf.getvalue()


def test_decode_image_bounds_and_alpha():
    img = decode_image(_png(20, 30, mode="RGBA"))
    assert img.mode == "RGB" and img.size == (30, 20)
    with pytest.raises(VisionInputError):
        decode_image(b"\x89PNG\r\n\x1a\nnot a png")
    with pytest.raises(VisionInputError):
        decode_image(_png(20, 30), max_side=16)
    from PIL import Image
    frames = [Image.fromarray(np.full((40, 40, 3), v, dtype=np.uint8)) for v in (0, 100, 200)]
    clip = patchify_video(frames, PatchGeometry(4, 2, 2, min_pixels=16 * 16, max_pixels=64 * 64))
    assert clip.grid[0] == 2
    with pytest.raises(VisionInputError):
        patchify_video([], PatchGeometry())


# ------------------------------------------------------------------ positions
def test_three_axis_positions():
    # 3 text tokens, an image of 4 x 6 patches (2 x 3 rows after the merge), 2 text tokens
    pos, delta = mrope_positions(list(range(11)), [(3, 6, (1, 4, 6))], 2)
    assert pos[0] == [0, 1, 2, 3, 3, 3, 3, 3, 3, 6, 7]
    assert pos[1] == [0, 1, 2, 3, 3, 3, 4, 4, 4, 6, 7]
    assert pos[2] == [0, 1, 2, 3, 4, 5, 3, 4, 5, 6, 7]
    assert delta == 8 - 11
    # a clip advances the temporal axis per frame group
    pos, delta = mrope_positions([0] * 9, [(1, 8, (2, 4, 4))], 2)
    assert pos[0][1:9] == [1, 1, 1, 1, 2, 2, 2, 2]
    with pytest.raises(ValueError):
        mrope_positions([0] * 4, [(0, 6, (1, 4, 6))], 2)
    # equal axes reduce to the one-axis rotation
    x = torch.randn(5, 2, 16)
    inv = eager.rope_inv_freq(8, 10000.0)
    p = torch.arange(3, 8)
    assert torch.allclose(eager.rope3(x, p[None].expand(3, -1), inv, (2, 1, 1)), eager.rope(x, p, inv))
    assert eager.mrope_axes((11, 11, 10), 32).count(1) == 11
    assert eager.mrope_axes((2, 1, 1), 4) == [0, 1, 2, 0]
    with pytest.raises(ValueError):
        eager.mrope_axes((1, 2, 1), 4)
    y = eager.rope3(x, torch.stack([p, p + 1, p + 2]), inv, (2, 1, 1))
    assert not torch.allclose(y, eager.rope(x, p, inv))


# ------------------------------------------------------------------ store, plan, service
def test_feature_store_is_bounded_lru():
    st = EncodedFeatureStore(max_bytes=3 * 40)
    rows = [torch.full((10,), float(i)) for i in range(4)]          # 40 bytes each
    for i in range(3):
        st.put(bytes([i]), rows[i])
    assert st.get(bytes([0])) is not None                           # 0 is now the most recent
    st.put(bytes([3]), rows[3])
    assert st.get(bytes([1])) is None and st.get(bytes([0])) is not None and len(st) == 3
    assert st.bytes == 120 and st.evictions == 1
    st.put(b"big", torch.zeros(100))                                # larger than the store: not kept
    assert st.get(b"big") is None
    assert media_digest(np.zeros((4, 8), np.float32), (1, 2, 2)) != media_digest(np.zeros((4, 8), np.float32), (1, 2, 2), b"x")


def test_service_cuts_clips_and_reuses_features():
    cfg = _cfg()
    enc = VisionEncoder(cfg, random_vision_weights(cfg, 5))
    px = np.random.default_rng(6).standard_normal((6 * 16, cfg.patch_width)).astype(np.float32)
    whole = VisionService(enc, memory_bytes=1 << 30)
    rows, digest = whole.encode([(px, (6, 4, 4))])[0]
    assert rows.shape == (6 * 4, 32) and whole.encode_calls == 1
    # a budget that holds two frames per call
    per = enc.activation_bytes(1)
    small = VisionService(enc, memory_bytes=int(2.6 * 16 * per) + 4 * 32 * 32 * 4 * 2)
    assert small.plan.max_patches_per_call < 6 * 16
    rows2, digest2 = small.encode([(px, (6, 4, 4))])[0]
    assert small.encode_calls > 1 and digest2 == digest
    assert torch.allclose(rows2, rows, atol=1e-6)
    small.encode([(px, (6, 4, 4))])
    assert small.store.hits == 1
    with pytest.raises(EncoderCapacityError):
        small.encode([(np.zeros((400, cfg.patch_width), np.float32), (1, 20, 20))])
    with pytest.raises(EncoderCapacityError):
        EncoderMemoryPlan.build(enc, 16, 100)
    tiny = VisionService(enc, max_prompt_tokens=8)
    with pytest.raises(EncoderCapacityError):
        tiny.encode([(px, (6, 4, 4))])
    # the owned thread serves futures and survives a failing request
    fut_bad = small.submit([(px[:5], (1, 4, 4))])
    fut_ok = small.submit([(px, (6, 4, 4))])
    with pytest.raises(ValueError):
        fut_bad.result(60)
    assert torch.allclose(fut_ok.result(60)[0][0], rows, atol=1e-6)
    small.close()


# ------------------------------------------------------------------ through the engine
def _engine(max_tokens_per_step=None, pages=64):
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.models.config import ModelConfig
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    from dataclasses import replace
    cfg = replace(ModelConfig(), mrope_section=(16, 8, 8), vocab_size=1024)
    ex = EagerPagedExecutor(cfg, random_dense_weights(cfg, 0, std=0.2), pages)
    sc = SchedulerConfig() if max_tokens_per_step is None else SchedulerConfig(prefill_chunk_tokens=max_tokens_per_step)
    return LLMEngine(ex, pages, sc), cfg


def _mm(prompt_len, first, feats, digest, grid):
    from cubic_serve_b200.runtime.multimodal import MultimodalInput
    pos, delta = mrope_positions([0] * prompt_len, [(first, feats.shape[0], grid)], 2)
    return MultimodalInput([(first, feats, digest)], np.asarray(pos), delta)


def _run(eng, prompt, mm, n=6):
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rid = eng.add_request(prompt, SamplingParams(max_tokens=n), multimodal=mm)
    toks = []
    while eng.has_unfinished:
        toks += [o.token_id for o in eng.step() if o.request_id == rid and o.token_id is not None]
    return toks


def test_engine_serves_feature_rows():
    prompt = [5, 6, 7] + [900] * 24 + list(range(20, 43))          # 50 tokens, 24 placeholder rows at 3
    g = torch.Generator().manual_seed(1)
    fa, fb = torch.randn(24, 256, generator=g), torch.randn(24, 256, generator=g)
    grid = (1, 8, 12)
    eng, _ = _engine()
    a1 = _run(eng, prompt, _mm(50, 3, fa, b"A", grid))
    hits0 = eng.prefix.hit_tokens
    a2 = _run(eng, prompt, _mm(50, 3, fa, b"A", grid))             # same media: resumed from cached pages
    assert eng.prefix.hit_tokens > hits0 and a2 == a1
    hits1 = eng.prefix.hit_tokens
    b1 = _run(eng, prompt, _mm(50, 3, fb, b"B", grid))             # other media: nothing of the span is shared
    assert eng.prefix.hit_tokens == hits1
    cold, _ = _engine()
    assert _run(cold, prompt, _mm(50, 3, fb, b"B", grid)) == b1
    assert b1 != a1
    # chunked prefill cuts the media span; the tokens do not change
    chunked, _ = _engine(max_tokens_per_step=16)
    assert _run(chunked, prompt, _mm(50, 3, fa, b"A", grid)) == a1
    # the positions matter: the same rows under another grid give another continuation
    other = _run(_engine()[0], prompt, _mm(50, 3, fa, b"A", (1, 4, 24)))
    assert other != a1


def test_text_only_executor_refuses_media():
    from cubic_serve_b200.runtime.scheduler import AdmissionError
    eng, _ = _engine()
    eng.executor.accepts_features = False
    with pytest.raises(AdmissionError):
        eng.add_request([1, 2, 3], multimodal=_mm(3, 0, torch.zeros(1, 256), b"x", (1, 2, 2)))
    eng2, _ = _engine()
    with pytest.raises(AdmissionError):
        eng2.add_request([1, 2], multimodal=_mm(3, 0, torch.zeros(1, 256), b"x", (1, 2, 2)))


def test_chat_processor_expands_media_parts():
    from cubic_serve_b200.contracts.request import CanonicalChatRequest, ContentPart, Message, RequestError, Role
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.inputs.multimodal import MultimodalChatProcessor, VisionTokens

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    ids = tok.special_ids
    vt = VisionTokens(ids["<|image_pad|>"], ids["<|video_pad|>"], ids["<|vision_start|>"], ids["<|vision_end|>"])
    cfg = _cfg()
    svc = VisionService(VisionEncoder(cfg, random_vision_weights(cfg, 7)))
    proc = MultimodalChatProcessor(tok, svc, vt, PatchGeometry(4, 2, 2, min_pixels=8 * 8, max_pixels=32 * 32))
    url = "data:image/png;base64," + base64.b64encode(_png(24, 40)).decode()
    msg = Message(Role.USER, (ContentPart("text", "look: "), ContentPart("image", media_url=url), ContentPart("text", " what?")))
    kw = {"protocol": "openai", "model": "m", "messages": (msg,), "request_id": "r1"}
    req = CanonicalChatRequest(**kw)
    out = proc.build(req)
    mm = out.multimodal
    assert mm is not None and len(mm.spans) == 1
    first, rows, digest = mm.spans[0]
    assert rows.shape[1] == 32 and out.token_ids[first - 1] == vt.start and out.token_ids[first + rows.shape[0]] == vt.end
    assert all(t == vt.image for t in out.token_ids[first:first + rows.shape[0]])
    assert mm.positions.shape == (3, len(out.token_ids))
    assert mm.delta < 0 or rows.shape[0] == 1
    keys = mm.key_tokens(out.token_ids)
    assert all(k < 0 for k in keys[first:first + rows.shape[0]]) and keys[:first] == out.token_ids[:first]
    again = proc.build(req)
    assert svc.store.hits == 1 and again.multimodal.spans[0][2] == digest
    # text-only requests go through unchanged
    plain = proc.build(CanonicalChatRequest(**{**kw, "messages": (Message(Role.USER, (ContentPart("text", "hi"),)),)}))
    assert plain.multimodal is None
    bad = Message(Role.USER, (ContentPart("image", media_url="data:image/png;base64,AAAA"),))
    with pytest.raises(RequestError):
        proc.build(CanonicalChatRequest(**{**kw, "messages": (bad,)}))
    vid = Message(Role.USER, (ContentPart("video", media_url="data:video/mp4;base64,AAAAGGZ0eXBtcDQy"),))
    with pytest.raises(RequestError):
        proc.build(CanonicalChatRequest(**{**kw, "messages": (vid,)}))


def test_multimodal_checkpoint_is_admitted_and_served(tmp_path):
    """A checkpoint with the decoder nested under ``model.language_model.`` and a vision tower: the closed inventory
    owns the tower's tensors, and the serving builder yields a processor whose output the eager engine serves."""
    import json
    from argparse import Namespace
    from dataclasses import replace

    from safetensors.torch import load_file, save_file

    from cubic_serve_b200.contracts.request import CanonicalChatRequest, ContentPart, Message, Role
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models.config import ModelConfig, QuantSpec
    from cubic_serve_b200.models.reference import dense_weights_from_checkpoint
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.serving import build_media_processor
    base = replace(ModelConfig(), qk_norm=True, name="Qwen3ForCausalLM", quant=QuantSpec("none", 16, 0))
    path = C.write_random_checkpoint(tmp_path / "mm", base, seed=2, std=0.1)
    t = load_file(str(path / "model.safetensors"))
    nested = {("model.language_model." + n[len("model."):] if n.startswith("model.") else n): v for n, v in t.items()}
    vcfg = _cfg(out_hidden_size=base.hidden_size)
    nested.update({"model.visual." + n: v.to(torch.bfloat16) for n, v in random_vision_weights(vcfg, 9).items()})
    save_file(nested, str(path / "model.safetensors"))
    raw = json.loads((path / "config.json").read_text())
    text = {k: v for k, v in raw.items() if k not in ("architectures",)}
    text["rope_parameters"] = {"mrope_section": [16, 8, 8], "rope_theta": raw.get("rope_theta", 10000.0)}
    doc = {"architectures": raw["architectures"], "text_config": text, "image_token_id": 261, "video_token_id": 262,
           "vision_start_token_id": 259, "vision_end_token_id": 260,
           "vision_config": {**RAW, "out_hidden_size": base.hidden_size, "model_type": "x"}}
    if "quantization_config" in raw:
        doc["quantization_config"] = raw["quantization_config"]
    (path / "config.json").write_text(json.dumps(doc))
    ck = C.admit_checkpoint(path)
    assert ck.vision is not None and ck.vision_prefix == "model.visual." and ck.cfg.mrope_section == (16, 8, 8)
    vw = C.load_vision_weights(ck, dtype=torch.float32)
    assert vw["pos_embed.weight"].shape == (64, 64)
    # a missing tower tensor is refused like any other
    broken = dict(nested)
    del broken["model.visual.merger.norm.bias"]
    save_file(broken, str(path / "model.safetensors"))
    with pytest.raises(C.CheckpointError, match="missing tensor"):
        C.admit_checkpoint(path)
    save_file(nested, str(path / "model.safetensors"))

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    assert (tok.special_ids["<|image_pad|>"], tok.special_ids["<|vision_start|>"]) == (261, 259)
    ex = EagerPagedExecutor(ck.cfg, dense_weights_from_checkpoint(ck), 64)
    args = Namespace(thinking=None, encoder_memory_gib=0.25, feature_store_mib=4)
    proc = build_media_processor(args, ck, tok, ex, 512)
    proc.geometry = replace(proc.geometry, min_pixels=8 * 8, max_pixels=32 * 32)
    url = "data:image/png;base64," + base64.b64encode(_png(24, 40)).decode()
    msg = Message(Role.USER, (ContentPart("text", "see "), ContentPart("image", media_url=url)))
    out = proc.build(CanonicalChatRequest("openai", "m", (msg,), request_id="r"))
    eng = LLMEngine(ex, 64)
    toks = _run(eng, out.token_ids, out.multimodal, n=4)
    assert len(toks) == 4
    ex.accepts_features = False
    assert build_media_processor(args, ck, tok, ex, 512) is None


def test_http_request_with_an_image_goes_through_the_encoder_thread():
    """OpenAI ``image_url`` part -> plan on the request's thread, encoding on the vision service's thread, admission when
    the rows exist; a broken image is a 400 before anything is queued; the same image again is served from the store."""
    import asyncio
    import json
    from dataclasses import replace

    from test_api import _call

    from cubic_serve_b200.api.server import CubicASGIApp
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.inputs.multimodal import MultimodalChatProcessor, VisionTokens
    from cubic_serve_b200.models.config import ModelConfig
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.async_engine import TokenChatBackend
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    ids = tok.special_ids
    cfg = replace(ModelConfig(num_layers=1, hidden_size=64, num_q_heads=2, num_kv_heads=1, head_dim=32, intermediate_size=128,
                              vocab_size=tok.vocab_size), mrope_section=(8, 4, 4))
    eng = LLMEngine(EagerPagedExecutor(cfg, random_dense_weights(cfg, 0), 64), 64,
                    SchedulerConfig(max_running_requests=4, max_model_len=512, max_batched_tokens=256))
    vcfg = _cfg(out_hidden_size=64)
    svc = VisionService(VisionEncoder(vcfg, random_vision_weights(vcfg, 3)))
    threads = []
    encode = svc.encode
    svc.encode = lambda items: (threads.append(threading.current_thread().name), encode(items))[1]
    proc = MultimodalChatProcessor(tok, svc, VisionTokens(ids["<|image_pad|>"], ids["<|video_pad|>"], ids["<|vision_start|>"],
                                                          ids["<|vision_end|>"]),
                                   PatchGeometry(4, 2, 2, min_pixels=8 * 8, max_pixels=32 * 32), max_model_len=512)
    url = "data:image/png;base64," + base64.b64encode(_png(24, 40)).decode()

    async def go():
        backend = TokenChatBackend(eng, tok, default_max_tokens=8, processor=proc)
        app = CubicASGIApp(backend, "toy")
        body = {"model": "toy", "max_tokens": 5, "temperature": 0, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "what is this? "}, {"type": "image_url", "image_url": {"url": url}}]}]}
        first = await _call(app, "POST", "/v1/chat/completions", body)
        second = await _call(app, "POST", "/v1/chat/completions", body)
        text = await _call(app, "POST", "/v1/chat/completions", {**body, "messages": [{"role": "user", "content": "hi"}]})
        bad = {**body, "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {
            "url": "data:image/png;base64,iVBORw0KGgoAAAANSUhEUg=="}}]}]}
        broken = await _call(app, "POST", "/v1/chat/completions", bad)
        metrics = await _call(app, "GET", "/metrics")
        backend.close()
        return first, second, text, broken, metrics
    (s1, b1), (s2, b2), (s3, _), (s4, b4), (sm, bm) = asyncio.run(go())
    m = {l.split(" ")[0].split("{")[0]: float(l.split(" ")[1]) for l in bm.decode().splitlines() if l and not l.startswith("#")}
    assert sm == 200 and m["cubic_media_encode_calls_total"] == 1 and m["cubic_media_feature_store_hits_total"] >= 1
    assert m["cubic_media_feature_store_bytes"] > 0 and m["cubic_media_feature_store_misses_total"] == 1
    assert s1 == s2 == s3 == 200 and s4 == 400
    j1, j2 = json.loads(b1), json.loads(b2)
    assert j1["usage"]["completion_tokens"] == 5 and j1["usage"]["prompt_tokens"] > 15
    assert j1["choices"][0]["message"]["content"] == j2["choices"][0]["message"]["content"]
    assert threads and all(t == "vision-encoder" for t in threads)
    assert svc.store.hits >= 1 and "messages" in json.dumps(json.loads(b4))
    svc.close()


def _tower_rank(rank, world, port, q):
    import datetime
    import os

    import torch.distributed as dist

    from cubic_serve_b200.models.vision import group_reduce
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    torch.set_num_threads(1)
    cfg = _cfg()
    w = random_vision_weights(cfg, 3)
    px = torch.randn(40, cfg.patch_width, generator=torch.Generator().manual_seed(4))
    enc = VisionEncoder(cfg, shard_vision_weights(cfg, w, rank, world), rank, world, group_reduce())
    q.put((rank, enc.encode(px, torch.tensor([[1, 4, 6], [1, 4, 4]]))[0]))
    dist.barrier()
    dist.destroy_process_group()


def test_tower_sharded_over_a_process_group():
    import socket

    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tower_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    cfg = _cfg()
    px = torch.randn(40, cfg.patch_width, generator=torch.Generator().manual_seed(4))
    want, _ = VisionEncoder(cfg, random_vision_weights(cfg, 3)).encode(px, torch.tensor([[1, 4, 6], [1, 4, 4]]))
    assert torch.equal(got[0], got[1]) and (got[0] - want).abs().max() < 1e-5


def test_fixed_shape_buckets_equal_the_exact_encode():
    """The bucket form (padded to a capacity, frames separated by a mask) gives the rows of the exact call; the service
    sends calls that fit to the smallest bucket and the rest to the eager path."""
    from cubic_serve_b200.executor.vision import VisionGraphBucket
    cfg = _cfg()
    enc = VisionEncoder(cfg, random_vision_weights(cfg, 11))
    g = torch.Generator().manual_seed(12)
    for grid in ([[1, 4, 6]], [[3, 4, 4]], [[1, 2, 2]]):
        n = sum(t * h * w for t, h, w in grid)
        px = torch.randn(n, cfg.patch_width, generator=g)
        want, _ = enc.encode(px, torch.tensor(grid))
        got = VisionGraphBucket(enc, 64).encode(px, torch.tensor(grid))
        assert got.shape == want.shape and (got - want).abs().max() < 1e-5
    bucket = VisionGraphBucket(enc, 32)
    a = bucket.encode(torch.randn(24, cfg.patch_width, generator=g), torch.tensor([[1, 4, 6]]))
    px = torch.randn(16, cfg.patch_width, generator=g)
    b = bucket.encode(px, torch.tensor([[1, 4, 4]]))                       # a reused bucket forgets the previous item
    assert (b - enc.encode(px, torch.tensor([[1, 4, 4]]))[0]).abs().max() < 1e-5 and bucket.replays == 2 and a.shape[0] == 6
    with pytest.raises(ValueError):
        bucket.encode(torch.randn(48, cfg.patch_width), torch.tensor([[1, 8, 6]]))
    with pytest.raises(ValueError):
        VisionGraphBucket(enc, 30)
    svc = VisionService(enc, graph_buckets=(16, 64))
    small = np.random.default_rng(0).standard_normal((16, cfg.patch_width)).astype(np.float32)
    big = np.random.default_rng(1).standard_normal((96, cfg.patch_width)).astype(np.float32)
    rows_small = svc.encode([(small, (1, 4, 4))])[0][0]
    rows_big = svc.encode([(big, (1, 8, 12))])[0][0]
    assert [b.replays for b in svc.buckets] == [1, 0]
    assert (rows_small - enc.encode(torch.from_numpy(small), torch.tensor([[1, 4, 4]]))[0]).abs().max() < 1e-5
    assert rows_big.shape == (24, 32)


def test_clip_of_decoded_frames_through_the_processor():
    from PIL import Image

    from cubic_serve_b200.contracts.request import CanonicalChatRequest, ContentPart, Message, RequestError, Role
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.inputs.multimodal import MultimodalChatProcessor, VisionTokens

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    ids = tok.special_ids
    vt = VisionTokens(ids["<|image_pad|>"], ids["<|video_pad|>"], ids["<|vision_start|>"], ids["<|vision_end|>"])
    cfg = _cfg()
    svc = VisionService(VisionEncoder(cfg, random_vision_weights(cfg, 7)))
    proc = MultimodalChatProcessor(tok, svc, vt, PatchGeometry(4, 2, 2, min_pixels=8 * 8, max_pixels=16 * 16), video_max_frames=6)
    frames = [Image.fromarray(np.full((16, 16, 3), v, dtype=np.uint8)) for v in (0, 60, 120, 180)]
    msg = Message(Role.USER, (ContentPart("video", data=frames), ContentPart("text", "what happens?")))
    plan = proc.plan(CanonicalChatRequest("openai", "m", (msg,), request_id="v"))
    (p,) = plan.placements
    assert p.kind == "video" and p.grid == (2, 4, 4) and p.rows == 8                  # 4 frames = 2 temporal patches
    assert all(t == vt.video for t in plan.token_ids[p.first_token:p.first_token + 8])
    t_axis = plan.positions[0, p.first_token:p.first_token + 8].tolist()
    assert t_axis == [t_axis[0]] * 4 + [t_axis[0] + 1] * 4                            # the temporal axis advances per patch
    out = proc.build(CanonicalChatRequest("openai", "m", (msg,), request_id="v"))
    assert out.multimodal.spans[0][1].shape == (8, 32)
    too_long = Message(Role.USER, (ContentPart("video", data=frames * 2),))
    with pytest.raises(RequestError):
        proc.plan(CanonicalChatRequest("openai", "m", (too_long,), request_id="w"))


def test_segment_inputs_cover_every_cut_of_a_prompt():
    """However a prompt with two media spans is cut into segments, the pieces put together are the whole: feature rows
    land on their tokens exactly once, positions follow the prompt and then the sequence index plus the offset."""
    from cubic_serve_b200.runtime.multimodal import MultimodalInput
    n = 40
    a, b = torch.arange(6 * 4).float().view(6, 4), 100 + torch.arange(4 * 4).float().view(4, 4)
    pos, delta = mrope_positions([0] * n, [(3, 6, (1, 4, 6)), (20, 4, (1, 4, 4))], 2)
    mm = MultimodalInput([(3, a, b"a"), (20, b, b"b")], np.asarray(pos), delta)
    rng = np.random.default_rng(0)
    for _ in range(50):
        cuts = sorted(set(rng.integers(1, n + 8, size=rng.integers(0, 6)).tolist()) | {0, n + 8})
        rows = torch.full((n + 8, 4), -1.0)
        got_pos = np.full((3, n + 8), -1, dtype=np.int64)
        for lo, hi in zip(cuts, cuts[1:]):
            embeds, p3 = mm.segment_inputs(lo, hi - lo)
            assert p3.shape == (3, hi - lo)
            got_pos[:, lo:hi] = p3
            for off, r in embeds:
                assert (rows[lo + off:lo + off + r.shape[0]] == -1).all()          # written once
                rows[lo + off:lo + off + r.shape[0]] = r
        assert torch.equal(rows[3:9], a) and torch.equal(rows[20:24], b) and float(rows[9:20].max()) == -1
        assert (got_pos[:, :n] == np.asarray(pos)).all()
        assert (got_pos[:, n:] == np.arange(n, n + 8)[None, :] + delta).all()
    keys = mm.key_tokens(list(range(n)))
    assert keys[:3] == [0, 1, 2] and all(k < 0 for k in keys[3:9] + keys[20:24]) and keys[9:20] == list(range(9, 20))
    assert len(set(keys[3:9])) == 6
    other = MultimodalInput([(3, a, b"x"), (20, b, b"b")], np.asarray(pos), delta).key_tokens(list(range(n)))
    assert other[3:9] != keys[3:9] and other[20:24] == keys[20:24]
    with pytest.raises(ValueError):
        MultimodalInput([(3, a, b"a"), (5, b, b"b")], np.asarray(pos), delta)


def test_several_images_are_prepared_concurrently_and_keep_their_order():
    from cubic_serve_b200.contracts.request import CanonicalChatRequest, ContentPart, Message, RequestError, Role
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.inputs.multimodal import MultimodalChatProcessor, VisionTokens

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    ids = tok.special_ids
    vt = VisionTokens(ids["<|image_pad|>"], ids["<|video_pad|>"], ids["<|vision_start|>"], ids["<|vision_end|>"])
    cfg = _cfg()
    svc = VisionService(VisionEncoder(cfg, random_vision_weights(cfg, 7)))
    geo = PatchGeometry(4, 2, 2, min_pixels=8 * 8, max_pixels=32 * 32)
    sizes = [(8, 8), (16, 24), (24, 8), (8, 32)]
    urls = ["data:image/png;base64," + base64.b64encode(_png(h, w, seed=i)).decode() for i, (h, w) in enumerate(sizes)]
    parts = []
    for u in urls:
        parts += [ContentPart("text", "and "), ContentPart("image", media_url=u)]
    req = CanonicalChatRequest("openai", "m", (Message(Role.USER, tuple(parts)),), request_id="many")
    threads = []
    many = MultimodalChatProcessor(tok, svc, vt, geo, preprocess_workers=3)
    inner = many._patches
    many._patches = lambda p: (threads.append(threading.current_thread().name), inner(p))[1]
    plan = many.plan(req)
    one = MultimodalChatProcessor(tok, svc, vt, geo, preprocess_workers=1).plan(req)
    assert [p.grid for p in plan.placements] == [(1, h // 4, w // 4) for h, w in sizes]
    assert [p.digest for p in plan.placements] == [p.digest for p in one.placements] and plan.token_ids == one.token_ids
    assert any(t.startswith("media-prep") for t in threads)
    with pytest.raises(RequestError):
        MultimodalChatProcessor(tok, svc, vt, geo, max_items=3).plan(req)


def test_preempted_request_with_media_recomputes_to_the_same_tokens():
    """A pool too small for two requests preempts one; when it is recomputed (prompt and the tokens it had generated in
    one prefill) its feature rows and positions are applied again, and the outputs equal those of a roomy pool."""
    g = torch.Generator().manual_seed(5)
    prompt_a = [5, 6, 7] + [900] * 24 + list(range(20, 41))             # 48 tokens
    prompt_b = [8, 9] + [900] * 24 + list(range(50, 72))
    fa, fb = torch.randn(24, 256, generator=g), torch.randn(24, 256, generator=g)
    grid = (1, 8, 12)

    def run(pages):
        from cubic_serve_b200.runtime.scheduler import SamplingParams
        eng, _ = _engine(pages=pages)
        ra = eng.add_request(prompt_a, SamplingParams(max_tokens=40), multimodal=_mm(48, 3, fa, b"A", grid))
        rb = eng.add_request(prompt_b, SamplingParams(max_tokens=40), multimodal=_mm(48, 2, fb, b"B", grid))
        out = {ra: [], rb: []}
        preempted = 0
        while eng.has_unfinished:
            for o in eng.step():
                if o.token_id is not None:
                    out[o.request_id].append(o.token_id)
            preempted = max(preempted, sum(r.preemptions for r in eng.requests.values()))
        return out[ra], out[rb], preempted
    a0, b0, p0 = run(64)
    a1, b1, p1 = run(10)                                                # 9 usable pages: not enough for 2 x 88 tokens
    assert p0 == 0 and p1 > 0
    assert (a1, b1) == (a0, b0) and len(a0) == 40


def test_a_failing_encoder_ends_the_request_with_a_server_error():
    """The tower failing for one request (not a capacity refusal) is that request's 500; the backend keeps serving."""
    import asyncio
    import json
    from dataclasses import replace

    from test_api import _call

    from cubic_serve_b200.api.server import CubicASGIApp
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.inputs.multimodal import MultimodalChatProcessor, VisionTokens
    from cubic_serve_b200.models.config import ModelConfig
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.async_engine import TokenChatBackend
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig

    class Tok(ByteTokenizer):
        SPECIALS = ByteTokenizer.SPECIALS + ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>")
    tok = Tok()
    ids = tok.special_ids
    cfg = replace(ModelConfig(num_layers=1, hidden_size=64, num_q_heads=2, num_kv_heads=1, head_dim=32, intermediate_size=128,
                              vocab_size=tok.vocab_size), mrope_section=(8, 4, 4))
    eng = LLMEngine(EagerPagedExecutor(cfg, random_dense_weights(cfg, 0), 64), 64,
                    SchedulerConfig(max_running_requests=4, max_model_len=512, max_batched_tokens=256))
    vcfg = _cfg(out_hidden_size=64)
    svc = VisionService(VisionEncoder(vcfg, random_vision_weights(vcfg, 3)))
    calls = {"n": 0}
    real = svc.encoder.encode

    def flaky(px, grid):
        calls["n"] += 1
        if calls["n"] == 1:
            raise RuntimeError("out of memory")
        return real(px, grid)
    svc.encoder.encode = flaky
    proc = MultimodalChatProcessor(tok, svc, VisionTokens(ids["<|image_pad|>"], ids["<|video_pad|>"], ids["<|vision_start|>"],
                                                          ids["<|vision_end|>"]),
                                   PatchGeometry(4, 2, 2, min_pixels=8 * 8, max_pixels=32 * 32), max_model_len=512)
    url = "data:image/png;base64," + base64.b64encode(_png(16, 16)).decode()
    body = {"model": "toy", "max_tokens": 3, "temperature": 0, "messages": [{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": url}}]}]}

    async def go():
        backend = TokenChatBackend(eng, tok, default_max_tokens=8, processor=proc)
        app = CubicASGIApp(backend, "toy")
        first = await _call(app, "POST", "/v1/chat/completions", body)
        second = await _call(app, "POST", "/v1/chat/completions", body)
        backend.close()
        return first, second
    (s1, b1), (s2, b2) = asyncio.run(go())
    assert s1 == 500 and json.loads(b1)["error"]["type"] == "api_error" and "out of memory" not in b1.decode()
    assert s2 == 200 and json.loads(b2)["usage"]["completion_tokens"] == 3
    svc.close()
