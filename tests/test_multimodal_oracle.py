"""The whole multimodal eager stack against the public Qwen3-VL implementation (when importable): vision tower with
intermediate outputs, placeholder positions on three axes, feature rows in place of embeddings, additions after the
first decoder layers, prefill and a decode step."""
import numpy as np
import pytest
import torch

from cubic_serve_b200.models import eager_family as EF
from cubic_serve_b200.models.config import ModelConfig
from cubic_serve_b200.models.vision import VisionConfig, VisionEncoder, mrope_positions
from cubic_serve_b200.runtime.multimodal import MultimodalInput

VIS = dict(depth=2, hidden_size=64, hidden_act="gelu_pytorch_tanh", intermediate_size=128, num_heads=4, in_channels=3,
           patch_size=4, spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=64,
           deepstack_visual_indexes=[0, 1])
TEXT = dict(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
            intermediate_size=128, vocab_size=300, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512,
            rope_scaling={"rope_type": "default", "mrope_section": [4, 2, 2], "mrope_interleaved": True},
            tie_word_embeddings=False, attention_bias=False)


def _public_model():
    c = pytest.importorskip("transformers.models.qwen3_vl.configuration_qwen3_vl")
    m = pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
    cfg = c.Qwen3VLConfig(text_config=TEXT, vision_config=VIS, image_token_id=290, video_token_id=291,
                          vision_start_token_id=292, vision_end_token_id=293)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    model = m.Qwen3VLForConditionalGeneration(cfg).eval()
    for p in model.parameters():
        p.data.normal_(0, 0.08)
    for n, p in model.named_parameters():
        if n.endswith("norm.weight") or "layernorm.weight" in n or ".norm1.weight" in n or ".norm2.weight" in n:
            p.data.copy_(1 + 0.1 * torch.randn_like(p))
    return model


@pytest.mark.parametrize("grids", [[(1, 4, 6)], [(1, 4, 6), (1, 2, 4)]])
def test_eager_stack_equals_the_public_model(grids):
    ref = _public_model()
    sd = {n: p.detach() for n, p in ref.named_parameters()}
    cfg = ModelConfig(name="Qwen3VL", num_layers=3, hidden_size=64, num_q_heads=4, num_kv_heads=2, head_dim=16,
                      intermediate_size=128, vocab_size=300, rope_theta=10000.0, qk_norm=True, mrope_section=(4, 2, 2))
    w = {("model." + n[len("model.language_model."):] if n.startswith("model.language_model.") else n): t
         for n, t in sd.items() if not n.startswith("model.visual.")}
    model = EF.EagerFamilyModel(cfg, w)
    tower = VisionEncoder(VisionConfig.from_hf(VIS), {n[len("model.visual."):]: t for n, t in sd.items()
                                                      if n.startswith("model.visual.")})
    g = torch.Generator().manual_seed(1)
    ids, spans = [5, 6], []
    for t, h, wd in grids:
        rows = t * h * wd // 4
        ids += [292]
        spans.append((len(ids), rows, (t, h, wd)))
        ids += [290] * rows + [293, 7]
    ids += [8, 9, 10]
    px = torch.randn(sum(t * h * wd for t, h, wd in grids), 3 * 2 * 4 * 4, generator=g)
    grid = torch.tensor(grids)
    tid = torch.tensor([ids])
    with torch.no_grad():
        out = ref(input_ids=tid, pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(tid == 290).long(), use_cache=True)
    # this build's path: tower -> rows with their intermediate outputs in extra columns -> request input -> eager model
    feats, deep = tower.encode(px, grid)
    rows_all = torch.cat([feats] + deep, 1)
    pos, delta = mrope_positions(ids, spans, 2)
    assert delta == int(ref.model.rope_deltas[0, 0])
    at, media = 0, []
    for first, n, _ in spans:
        media.append((first, rows_all[at:at + n], bytes([first])))
        at += n
    mm = MultimodalInput(media, np.asarray(pos), delta, hidden=64)
    assert mm.deep_layers == 2
    embeds, p3 = mm.segment_inputs(0, len(ids))
    logits, state = model.forward(ids, positions3=p3, embeds=embeds, deep=mm.segment_deep(0, len(ids)))
    assert (logits - out.logits[0]).abs().max() < 2e-4
    # in two chunks that cut the first image, then one decode step at sequence index + offset
    cut = spans[0][0] + 2
    e1, q1 = mm.segment_inputs(0, cut)
    l1, st = model.forward(ids[:cut], positions3=q1, embeds=e1, deep=mm.segment_deep(0, cut))
    e2, q2 = mm.segment_inputs(cut, len(ids) - cut)
    l2, st = model.forward(ids[cut:], st, positions3=q2, embeds=e2, deep=mm.segment_deep(cut, len(ids) - cut))
    assert (torch.cat([l1, l2]) - out.logits[0]).abs().max() < 2e-4
    nxt = int(out.logits[0, -1].argmax())
    with torch.no_grad():
        step = ref(input_ids=torch.tensor([[nxt]]), past_key_values=out.past_key_values, use_cache=True)
    _, q3 = mm.segment_inputs(len(ids), 1)
    l3, _ = model.forward([nxt], st, positions3=q3)
    assert (l3[0] - step.logits[0, 0]).abs().max() < 2e-4


def test_engine_carries_the_intermediate_outputs():
    """Through the engine (chunked prefill that cuts the image, then decoding) the eager executors emit the greedy tokens
    of the model run directly; an executor that does not consume intermediate outputs refuses such a request."""
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.models.reference import DenseLayer, DenseWeights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import AdmissionError, SamplingParams, SchedulerConfig
    cfg = ModelConfig(name="mm", num_layers=3, hidden_size=64, num_q_heads=4, num_kv_heads=2, head_dim=16,
                      intermediate_size=128, vocab_size=300, rope_theta=10000.0, qk_norm=True, mrope_section=(4, 2, 2))
    w = EF.random_family_weights(cfg, 2, std=0.15)
    model = EF.EagerFamilyModel(cfg, w)
    g = torch.Generator().manual_seed(3)
    rows_all = torch.randn(6, 3 * 64, generator=g) * 0.3                    # rows + two layers of additions
    ids = [5, 6, 292] + [290] * 6 + [293, 7, 8, 9]
    pos, delta = mrope_positions(ids, [(3, 6, (1, 4, 6))], 2)

    def mm():
        return MultimodalInput([(3, rows_all, b"img")], np.asarray(pos), delta, hidden=64)
    m0 = mm()
    embeds, p3 = m0.segment_inputs(0, len(ids))
    lg, st = model.forward(ids, positions3=p3, embeds=embeds, deep=m0.segment_deep(0, len(ids)), last_only=True)
    want = []
    for _ in range(5):
        want.append(int(lg[0].argmax()))
        lg, st = model.forward([want[-1]], st, positions3=m0.segment_inputs(st.length, 1)[1], last_only=True)

    def run(ex):
        eng = LLMEngine(ex, 64, SchedulerConfig(prefill_chunk_tokens=5, max_model_len=128))
        rid = eng.add_request(ids, SamplingParams(max_tokens=5), multimodal=mm())
        out = []
        while eng.has_unfinished:
            out += [o.token_id for o in eng.step() if o.request_id == rid and o.token_id is not None]
        return out
    assert run(EF.EagerFamilyExecutor(cfg, w)) == want
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}"
        t = lambda n: w[f"{p}.{n}"]                                            # noqa: E731
        layers.append(DenseLayer(t("input_layernorm.weight"), t("post_attention_layernorm.weight"), t("self_attn.q_proj.weight"),
                                 t("self_attn.k_proj.weight"), t("self_attn.v_proj.weight"), t("self_attn.o_proj.weight"),
                                 t("mlp.gate_proj.weight"), t("mlp.up_proj.weight"), t("mlp.down_proj.weight"),
                                 t("self_attn.q_norm.weight"), t("self_attn.k_norm.weight")))
    dense = DenseWeights(w["model.embed_tokens.weight"], layers, w["model.norm.weight"], w["lm_head.weight"])
    assert run(EagerPagedExecutor(cfg, dense, 64)) == want
    refusing = EagerPagedExecutor(cfg, dense, 64)
    refusing.accepts_deepstack = False
    with pytest.raises(AdmissionError):
        LLMEngine(refusing, 64).add_request(ids, multimodal=mm())


def test_checkpoint_of_the_public_multimodal_model_is_admitted(tmp_path):
    """``save_pretrained`` of the public model: nested decoder names, tower tensors and the two-level ``config.json`` are
    admitted by the closed inventory; tower and decoder loaded from it give the public model's logits."""
    from cubic_serve_b200.inputs.multimodal import VisionTokens
    from cubic_serve_b200.models import checkpoint as C
    ref = _public_model()
    ref.save_pretrained(tmp_path, safe_serialization=True)
    ck = C.admit_checkpoint(tmp_path)
    assert ck.vision is not None and ck.vision.deepstack_visual_indexes == (0, 1) and ck.cfg.mrope_section == (4, 2, 2)
    assert ck.cfg.qk_norm and ck.cfg.num_layers == 3 and ck.vision_prefix == "model.visual."
    tokens = VisionTokens.from_hf(ck.raw_config)
    assert (tokens.image, tokens.start, tokens.end) == (290, 292, 293)
    tower = VisionEncoder(ck.vision, C.load_vision_weights(ck, dtype=torch.float32))
    model = EF.EagerFamilyModel(ck.cfg, EF.family_weights_from_checkpoint(ck))
    ids = [5, 6, 292] + [290] * 6 + [293, 7, 8, 9]
    px = torch.randn(24, 96, generator=torch.Generator().manual_seed(4))
    grid = torch.tensor([[1, 4, 6]])
    tid = torch.tensor([ids])
    with torch.no_grad():
        want = ref(input_ids=tid, pixel_values=px, image_grid_thw=grid, mm_token_type_ids=(tid == 290).long()).logits[0]
    feats, deep = tower.encode(px, grid)
    pos, delta = mrope_positions(ids, [(3, 6, (1, 4, 6))], 2)
    mm = MultimodalInput([(3, torch.cat([feats] + deep, 1), b"i")], np.asarray(pos), delta, hidden=64)
    embeds, p3 = mm.segment_inputs(0, len(ids))
    got, _ = model.forward(ids, positions3=p3, embeds=embeds, deep=mm.segment_deep(0, len(ids)))
    assert (got - want).abs().max() < 2e-4
