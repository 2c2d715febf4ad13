"""The qwen4_exp family on CPU: configuration, lexical hashing, dilated convolution, state consistency of the eager
model (whole sequence = chunks = token by token), the sparse attention below and above its budget, the engine."""
import json
from dataclasses import replace

import numpy as np
import pytest
import torch

from cubic_serve_b200.models import qwen4_exp as Q
from cubic_serve_b200.ops import eager


def _raw_config():
    layers = ["full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(48)]
    return {
        "architectures": ["Qwen4ExpForConditionalGeneration"], "image_token_id": 248056, "language_model_only": False,
        "model_type": "qwen4_exp",
        "text_config": {
            "attention_bias": False, "attention_dropout": 0.0, "dtype": "bfloat16", "full_attention_interval": 4,
            "hc_count": 4, "hc_lowrank": 320, "head_dim": 256, "heads_per_ngram": 8, "hidden_act": "silu",
            "hidden_size": 2560, "indexer_budget": 2048, "indexer_compress_ratio": 4, "indexer_head_dim": 128,
            "indexer_kv_heads": 1, "indexer_n_heads": 4, "layer_types": layers, "linear_conv_kernel_dim": 4,
            "linear_key_head_dim": 128, "linear_num_key_heads": 16, "linear_num_value_heads": 48,
            "linear_value_head_dim": 128, "make_ngram_vocab_size_divisible_by": 128, "mamba_ssm_dtype": "float32",
            "max_position_embeddings": 262144, "model_type": "qwen4_exp_text", "moe_intermediate_size": 640,
            "mtp": {"hybrid": True, "layer_types": ["full_attention"], "mtp_use_hidden_state_from_layer": None,
                    "num_hidden_layers": 1, "rope_theta": 10_000_000},
            "mtp_num_hidden_layers": 1, "mtp_use_dedicated_embeddings": False, "ngram_size": 3,
            "ngram_vocab_size_base": 20_000_000, "num_attention_heads": 24, "num_experts": 512,
            "num_experts_per_tok": 10, "num_hidden_layers": 48, "num_key_value_heads": 2, "output_gate_type": "sigmoid",
            "partial_rotary_factor": 0.25, "ple_conv_kernel_size": 4, "ple_embed_dim": 2560, "ple_layer_ids": [2],
            "rms_norm_eps": 1e-6,
            "rope_parameters": {"mrope_interleaved": True, "mrope_section": [11, 11, 10], "partial_rotary_factor": 0.25,
                                "rope_theta": 10_000_000, "rope_type": "default"},
            "shared_expert_intermediate_size": 640, "split_ngram_parts": 128, "use_cache": True, "vocab_size": 248320,
            "eos_token_id": 248044},
        "tie_word_embeddings": False, "video_token_id": 248057,
        "vision_config": {"deepstack_visual_indexes": [], "depth": 27, "hidden_act": "gelu_pytorch_tanh",
                          "hidden_size": 1152, "in_channels": 3, "intermediate_size": 4304, "model_type": "qwen4_exp",
                          "num_heads": 16, "num_position_embeddings": 2304, "out_hidden_size": 2560, "patch_size": 16,
                          "spatial_merge_size": 2, "temporal_patch_size": 2},
        "vision_end_token_id": 248054, "vision_start_token_id": 248053}


def test_release_configuration_parses():
    cfg = Q.parse_qwen4_exp_config(_raw_config())
    assert cfg.num_layers == 48 and sum(cfg.layer_is_gdn(i) for i in range(48)) == 36
    assert cfg.uses_ple(1) and not cfg.uses_ple(0)
    assert (cfg.streams, cfg.stream_low_rank, cfg.num_experts, cfg.experts_per_token) == (4, 320, 512, 10)
    assert cfg.rotary_dim == 64 and cfg.mrope_section == (11, 11, 10) and cfg.ngram_heads == 16
    assert cfg.vision is not None and cfg.vision.depth == 27 and cfg.is_hybrid
    shapes = Q.qwen4_exp_tensor_shapes(cfg)
    p = "model.language_model.layers.1"
    assert shapes[p + ".ple.ple_embedding.ngram_embedding.shard_127.weight"] == (2_500_012, 160)
    assert shapes[p + ".attn_hyper_connection.block_inject_weight.weight"] == (4, 10240)
    assert shapes["model.language_model.layers.3.self_attn.indexer.index_qk_proj.weight"] == (5 * 128, 2560)
    assert shapes["model.language_model.layers.3.self_attn.q_proj.weight"] == (2 * 24 * 256, 2560)
    assert shapes[p + ".mlp.experts.gate_up_proj"] == (512, 1280, 2560)
    assert shapes["model.language_model.layers.0.linear_attn.in_proj_qkv.weight"] == (2 * 16 * 128 + 48 * 128, 2560)
    assert "model.language_model.hyper_connection_mixer.block_inject_weight.weight" not in shapes
    assert Q.parse_qwen4_exp_config_json(json.dumps(_raw_config())).num_experts == 512


@pytest.mark.parametrize("edit,match", [
    (lambda r: r["text_config"].update(surprise=1), "unknown keys"),
    (lambda r: r["text_config"].update(attention_bias=True), "biases"),
    (lambda r: r["text_config"].pop("hc_count"), "lacks"),
    (lambda r: r["text_config"].update(layer_types=["full_attention"]), "once per layer"),
    (lambda r: r["text_config"].update(indexer_budget=2046), "whole number"),
    (lambda r: r["text_config"]["rope_parameters"].update(mrope_section=[30, 1, 2]), "sum to half"),
    (lambda r: r.update(model_type="qwen3_5"), "model_type"),
    (lambda r: r["vision_config"].update(out_hidden_size=1024), "output width"),
    (lambda r: r["text_config"].update(ple_layer_ids=[49]), "1-based"),
])
def test_configuration_is_strict(edit, match):
    raw = _raw_config()
    edit(raw)
    with pytest.raises(ValueError, match=match):
        Q.parse_qwen4_exp_config(raw)


def test_configuration_json_rejects_duplicates_and_constants():
    with pytest.raises(Q.Qwen4ExpConfigError, match="duplicate"):
        Q.parse_qwen4_exp_config_json('{"model_type": "qwen4_exp", "model_type": "qwen4_exp"}')
    with pytest.raises(Q.Qwen4ExpConfigError, match="non-finite"):
        Q.parse_qwen4_exp_config_json('{"model_type": "qwen4_exp", "x": NaN}')
    with pytest.raises(Q.Qwen4ExpConfigError):
        Q.parse_qwen4_exp_config_json("[1]")


# ------------------------------------------------------------------ lexical hashing, dilated convolution
def test_ngram_hash_matches_int64_tensor_arithmetic():
    g = torch.Generator().manual_seed(0)
    mult = (torch.randint(1, 1 << 62, (3,), generator=g, dtype=torch.int64) * 2 + 1)
    sizes = [997, 1009, 1013, 1019]
    offs = [0, 997, 2006, 3019]
    eos = 7
    tokens = [5, 9, 7, 11, 12, 13, 7, 7, 3]
    hist = [eos, eos]
    rows, ctx = Q.ngram_hash_ids(tokens, hist, mult.tolist(), sizes, offs, eos)
    assert ctx == tokens[-2:]
    # the same in wrapping int64 tensor arithmetic, written out per token
    seq = hist + tokens
    for t, tok in enumerate(tokens):
        prev1, prev2 = seq[t + 1], seq[t]
        if prev1 == eos:
            prev2 = eos                                          # everything behind an EOS reads as EOS
        h1 = (torch.tensor(tok) * mult[0]) ^ (torch.tensor(prev1) * mult[1])
        h2 = h1 ^ (torch.tensor(prev2) * mult[2])
        want = [int(h1.remainder(sizes[0])) + offs[0], int(h1.remainder(sizes[1])) + offs[1],
                int(h2.remainder(sizes[2])) + offs[2], int(h2.remainder(sizes[3])) + offs[3]]
        assert rows[t] == want
    # chunking does not change the ids
    a, mid = Q.ngram_hash_ids(tokens[:4], hist, mult.tolist(), sizes, offs, eos)
    b, _ = Q.ngram_hash_ids(tokens[4:], mid, mult.tolist(), sizes, offs, eos)
    assert a + b == rows
    with pytest.raises(ValueError):
        Q.ngram_hash_ids(tokens, [eos], mult.tolist(), sizes, offs, eos)


def test_dilated_convolution_against_a_direct_loop():
    g = torch.Generator().manual_seed(1)
    T, C, K, dil = 9, 5, 4, 3
    x, w = torch.randn(T, C, generator=g), torch.randn(C, 1, K, generator=g)
    hist = torch.randn((K - 1) * dil, C, generator=g)
    y, new = Q.dilated_causal_conv(x, hist, w, dil)
    seq = torch.cat([hist, x])
    for t in range(T):
        acc = sum(seq[t + k * dil] * w[:, 0, k] for k in range(K))
        assert torch.allclose(y[t], torch.nn.functional.silu(acc), atol=1e-6)
    assert torch.equal(new, seq[-(K - 1) * dil:])
    y1, mid = Q.dilated_causal_conv(x[:2], hist, w, dil)               # a chunk shorter than the history
    y2, end = Q.dilated_causal_conv(x[2:], mid, w, dil)
    assert torch.allclose(torch.cat([y1, y2]), y, atol=1e-6) and torch.equal(end, new)


# ------------------------------------------------------------------ the model
@pytest.fixture(scope="module")
def tiny():
    cfg = Q.tiny_config()
    return cfg, Q.random_qwen4_exp_weights(cfg, 3, std=0.15)


def test_chunked_and_stepwise_runs_equal_one_pass(tiny):
    cfg, w = tiny
    model = Q.Qwen4ExpModel(cfg, w)
    toks = torch.randint(2, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(4)).tolist()
    toks[10] = cfg.eos_token_id                                        # the n-gram context resets behind it
    whole, st = model.forward(toks)
    assert whole.shape == (37, cfg.vocab_size) and st.length == 37 and bool(torch.isfinite(whole).all())
    st2 = None
    parts = []
    for a, b in ((0, 5), (5, 6), (6, 23), (23, 37)):
        lg, st2 = model.forward(toks[a:b], st2)
        parts.append(lg)
    assert (torch.cat(parts) - whole).abs().max() < 2e-3
    st3 = None
    rows = []
    for t in toks[:12]:
        lg, st3 = model.forward([t], st3, last_only=True)
        rows.append(lg)
    assert (torch.cat(rows) - whole[:12]).abs().max() < 2e-3
    # the pooled index keys were built once per complete group
    att = st.layers[1]
    assert att.index_pooled.shape[0] == 37 // cfg.index_compression and att.key.shape[0] == 37
    assert st.layers[0].recurrent.shape == (cfg.gdn_v_heads, cfg.gdn_v_dim, cfg.gdn_k_dim)
    assert st.layers[1].ngram_history == toks[-2:]


def test_sparse_attention_is_dense_below_the_budget_and_selective_above(tiny):
    cfg, w = tiny
    toks = torch.randint(2, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(5)).tolist()
    sparse, _ = Q.Qwen4ExpModel(cfg, w).forward(toks)
    dense_cfg = replace(cfg, index_budget=4096)
    dense, _ = Q.Qwen4ExpModel(dense_cfg, w).forward(toks)
    # while a query sees at most budget + tail tokens every block is selected: the two agree
    agree = cfg.index_budget + cfg.index_compression - 1
    assert (sparse[:agree] - dense[:agree]).abs().max() < 1e-4
    assert (sparse[agree + 4:] - dense[agree + 4:]).abs().max() > 1e-4


def test_features_positions_and_expert_shares(tiny):
    cfg, w = tiny
    model = Q.Qwen4ExpModel(cfg, w)
    toks = list(range(2, 14))
    base, _ = model.forward(toks)
    feats = torch.randn(4, cfg.hidden_size, generator=torch.Generator().manual_seed(6))
    with_feats, _ = model.forward(toks, embeds=[(3, feats)])
    assert torch.allclose(with_feats[:3], base[:3], atol=1e-5) and not torch.allclose(with_feats[3:], base[3:], atol=1e-3)
    pos = np.stack([np.arange(12), np.arange(12) * 2, np.arange(12) // 3])     # a constant shift would cancel: rotary is relative
    moved, _ = model.forward(toks, positions3=pos)
    assert not torch.allclose(moved, base, atol=1e-4)
    same, _ = model.forward(toks, positions3=np.stack([np.arange(12)] * 3))
    assert torch.allclose(same, base, atol=1e-6)
    # two ranks that own half of the experts each sum to the whole routed output
    x = torch.randn(5, cfg.hidden_size, generator=torch.Generator().manual_seed(7))
    p = "model.language_model.layers.0.mlp"
    full = model._mlp(x, p)
    nosh = replace(cfg, shared_intermediate_size=0)
    w2 = {n: t for n, t in w.items() if "shared_expert" not in n}
    routed = Q.Qwen4ExpModel(nosh, w2)._mlp(x, p)
    parts = [Q.Qwen4ExpModel(nosh, w2, (r * 4, r * 4 + 4), lambda t: t)._mlp(x, p) for r in range(2)]
    assert torch.allclose(parts[0] + parts[1], routed, atol=1e-5)
    assert not torch.allclose(routed, full, atol=1e-4)                  # the shared expert contributes
    with pytest.raises(ValueError):
        Q.Qwen4ExpModel(cfg, w, (0, 4))
    with pytest.raises(Q.Qwen4ExpConfigError):
        Q.Qwen4ExpModel(cfg, {k: v for k, v in w.items() if not k.endswith("A_log")})
    with pytest.raises(ValueError):
        model.forward([cfg.vocab_size])


def test_engine_serves_the_family(tiny):
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg, w = tiny
    model = Q.Qwen4ExpModel(cfg, w)
    prompts = [list(range(2, 25)), [9, 8, 7, 6, 5, 4, 3]]
    want = []
    for p in prompts:                                                   # greedy decoding on the model itself
        lg, st = model.forward(p, last_only=True)
        out = []
        for _ in range(5):
            out.append(int(lg[0].argmax()))
            lg, st = model.forward([out[-1]], st, last_only=True)
        want.append(out)
    ex = Q.Qwen4ExpEagerExecutor(cfg, w)
    eng = LLMEngine(ex, 64, SchedulerConfig(prefill_chunk_tokens=16, max_model_len=256))
    assert not eng.prefix.enabled                                       # recurrent state: no prefix sharing
    ids = [eng.add_request(p, SamplingParams(max_tokens=5)) for p in prompts]
    got = {i: [] for i in ids}
    while eng.has_unfinished:
        for o in eng.step():
            if o.token_id is not None:
                got[o.request_id].append(o.token_id)
    assert [got[i] for i in ids] == want
    # the slot is reused by a later request: a fresh state, the same answer
    again = eng.add_request(prompts[1], SamplingParams(max_tokens=5))
    out = []
    while eng.has_unfinished:
        out += [o.token_id for o in eng.step() if o.request_id == again and o.token_id is not None]
    assert out == want[1]


def test_registry_lists_the_family():
    from cubic_serve_b200.models import registry
    d = registry.for_architecture("Qwen4ExpForConditionalGeneration")
    assert d.family == "qwen4_exp" and "qwen4_exp" in registry.families()
    cfg = Q.tiny_config()
    ex = d.build_runner(cfg, d.random_weights(cfg, "cpu", 1))
    assert isinstance(ex, Q.Qwen4ExpEagerExecutor)


def test_checkpoint_admission_and_serving_backend(tmp_path):
    from argparse import Namespace

    from safetensors.torch import save_file

    from cubic_serve_b200.models.checkpoint import CheckpointError
    from cubic_serve_b200.runtime.serving import build_backend
    cfg = Q.tiny_config()
    w = Q.random_qwen4_exp_weights(cfg, 2)
    raw = {"model_type": "qwen4_exp", "architectures": ["Qwen4ExpForConditionalGeneration"], "language_model_only": True,
           "text_config": {
               "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
               "layer_types": list(cfg.layer_types), "max_position_embeddings": cfg.max_position, "rms_norm_eps": cfg.rms_eps,
               "num_attention_heads": cfg.num_q_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
               "rope_parameters": {"mrope_section": list(cfg.mrope_section), "rope_theta": cfg.rope_theta,
                                   "partial_rotary_factor": cfg.rotary_dim / cfg.head_dim},
               "linear_num_key_heads": cfg.gdn_k_heads, "linear_num_value_heads": cfg.gdn_v_heads,
               "linear_key_head_dim": cfg.gdn_k_dim, "linear_value_head_dim": cfg.gdn_v_dim, "linear_conv_kernel_dim": 4,
               "output_gate_type": "sigmoid", "num_experts": cfg.num_experts, "num_experts_per_tok": cfg.experts_per_token,
               "moe_intermediate_size": cfg.moe_intermediate_size,
               "shared_expert_intermediate_size": cfg.shared_intermediate_size, "hc_count": cfg.streams,
               "hc_lowrank": cfg.stream_low_rank, "indexer_n_heads": cfg.index_heads, "indexer_head_dim": cfg.index_dim,
               "indexer_budget": cfg.index_budget, "indexer_compress_ratio": cfg.index_compression, "indexer_kv_heads": 1,
               "ple_layer_ids": list(cfg.ple_layer_ids), "ple_embed_dim": cfg.ple_embed_dim, "ple_conv_kernel_size": 4,
               "ngram_size": cfg.ngram_size, "heads_per_ngram": cfg.heads_per_ngram,
               "ngram_vocab_size_base": cfg.ngram_vocab_base, "make_ngram_vocab_size_divisible_by": cfg.ngram_vocab_multiple,
               "split_ngram_parts": cfg.ngram_split_parts, "ngram_shard_rows": cfg.ngram_shard_rows,
               "eos_token_id": cfg.eos_token_id}}
    d = tmp_path / "q4"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(raw))
    save_file({n: t.contiguous() for n, t in w.items()}, str(d / "model.safetensors"))
    got_cfg, got_w, _ = Q.admit_qwen4_exp_checkpoint(d)
    assert replace(got_cfg, name=cfg.name) == cfg
    assert all(torch.equal(got_w[n], w[n]) for n in w)
    toks = list(range(3, 20))
    assert torch.equal(Q.Qwen4ExpModel(got_cfg, got_w).forward(toks)[0], Q.Qwen4ExpModel(cfg, w).forward(toks)[0])
    stray = dict(w)
    stray["model.language_model.layers.0.stray"] = torch.zeros(1)
    save_file({n: t.contiguous() for n, t in stray.items()}, str(d / "model.safetensors"))
    with pytest.raises(CheckpointError, match="no logical weight owns"):
        Q.admit_qwen4_exp_checkpoint(d)
    save_file({n: t.contiguous() for n, t in w.items() if not n.endswith("dt_bias")}, str(d / "model.safetensors"))
    with pytest.raises(CheckpointError, match="missing tensor"):
        Q.admit_qwen4_exp_checkpoint(d)
    args = Namespace(model="random:qwen4-exp-tiny", execution_mode="eager", pp_size=1, seed=0, max_model_len=256,
                     max_running_requests=4, token_budget=64, prefill_chunk_tokens=32, prefix_cache=True, thinking=None,
                     served_model_name=None)
    backend, name = build_backend(args, [0], 1, None, 8, 8)
    assert name == "qwen4-exp-tiny" and not backend.engine.prefix.enabled


def test_inspect_reports_the_family(tmp_path):
    from safetensors.torch import save_file

    from cubic_serve_b200.models.checkpoint import inspect_checkpoint
    cfg = Q.tiny_config()
    d = tmp_path / "q"
    d.mkdir()
    raw = {"model_type": "qwen4_exp", "language_model_only": True, "text_config": {
        "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
        "layer_types": list(cfg.layer_types), "num_attention_heads": cfg.num_q_heads, "num_key_value_heads": cfg.num_kv_heads,
        "head_dim": cfg.head_dim, "rope_parameters": {"mrope_section": [2, 1, 1], "rope_theta": 1e4, "partial_rotary_factor": 0.5},
        "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 8, "linear_value_head_dim": 8,
        "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 16, "shared_expert_intermediate_size": 16,
        "hc_count": 4, "hc_lowrank": 8, "indexer_n_heads": 2, "indexer_head_dim": 16, "indexer_budget": 16,
        "indexer_compress_ratio": 4, "ple_layer_ids": [2], "ple_embed_dim": 32, "ngram_size": 3, "heads_per_ngram": 2,
        "ngram_vocab_size_base": 500, "make_ngram_vocab_size_divisible_by": 4, "split_ngram_parts": 4,
        "ngram_shard_rows": 512, "eos_token_id": 1, "max_position_embeddings": 4096}}
    (d / "config.json").write_text(json.dumps(raw))
    save_file({n: t.contiguous() for n, t in Q.random_qwen4_exp_weights(cfg, 1).items()}, str(d / "model.safetensors"))
    info = inspect_checkpoint(d)
    assert info["family"] == "qwen4_exp" and info["residual_streams"] == 4 and info["gated_deltanet_layers"] == 2
    assert info["ngram_layers"] == [2] and info["execution_mode"] == "eager" and not info["vision_tower"]


def test_draft_head_rounds_are_lossless_and_accept_agreeing_drafts():
    """The draft head's rounds through the engine emit exactly the tokens of plain greedy decoding; with a head that
    agrees with the target (its logits replaced by the target's own next-token choice) whole rounds are accepted and the
    committed state stays that of the accepted tokens."""
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = Q.tiny_config()
    w = Q.random_qwen4_exp_weights(cfg, 3, std=0.15, draft_head=True)
    assert set(Q.qwen4_exp_mtp_tensor_shapes(cfg)) <= set(w) and "mtp.layers.0.self_attn.indexer.index_qk_proj.weight" in w
    assert "mtp.layers.0.ple.conv1d.weight" not in w
    prompts = [list(range(2, 25)), [9, 8, 7, 6, 5, 4, 3], [11]]

    def run(depth, patch=None, n=12):
        ex = Q.Qwen4ExpEagerExecutor(cfg, w, speculative_depth=depth)
        if patch:
            patch(ex)
        eng = LLMEngine(ex, 64, SchedulerConfig(prefill_chunk_tokens=16, max_model_len=256))
        ids = [eng.add_request(p, SamplingParams(max_tokens=n)) for p in prompts]
        got = {i: [] for i in ids}
        while eng.has_unfinished:
            for o in eng.step():
                if o.token_id is not None:
                    got[o.request_id].append(o.token_id)
        return [got[i] for i in ids], ex, eng
    plain, _, _ = run(0)
    spec, ex, eng = run(3)
    assert spec == plain and all(len(o) == 12 for o in spec)
    assert getattr(eng, "spec_rounds", 0) > 0 and ex.last_round["proposed"]

    with pytest.raises(ValueError):
        Q.Qwen4ExpEagerExecutor(cfg, Q.random_qwen4_exp_weights(cfg, 3), speculative_depth=2)
    with pytest.raises(Q.Qwen4ExpConfigError):
        Q.Qwen4ExpModel(cfg, {k: v for k, v in w.items() if k != "mtp.fc_hidden.weight"})


def test_round_bookkeeping_with_a_scripted_model():
    """Acceptance, emitted tokens and what the committed states hold, on a model whose answers are scripted: the target
    continues every token t with t + 1; the head agrees for its first two proposals of a round and errs on the third."""
    from cubic_serve_b200.executor.gpu_executor import Segment

    class Scripted:
        has_draft_head = True
        cfg = Q.tiny_config()

        def __init__(self):
            self.target_calls, self.head_calls = [], []

        def forward(self, tokens, state=None, positions3=None, embeds=None, last_only=False):
            state = state or Q.RequestState()
            self.target_calls.append((state.length, list(tokens)))
            state.length += len(tokens)
            logits = torch.zeros(len(tokens), 320)
            for i, t in enumerate(tokens):
                logits[i, (t + 1) % 320] = 1
            self.last_feedback = torch.tensor([[float(t)] for t in tokens]).repeat(1, 128)
            return (logits[-1:] if last_only else logits), state

        def draft_forward(self, tokens, feedback, state=None):
            state = state or Q.RequestState()
            self.head_calls.append((state.length, list(tokens), feedback[:, 0].tolist()))
            n_before = getattr(state, "steps_in_round", 0)
            state.length += len(tokens)
            logits = torch.zeros(len(tokens), 320)
            for i, t in enumerate(tokens):
                wrong = getattr(state, "drafting", False) and n_before + i >= 2
                logits[i, (t + (5 if wrong else 1)) % 320] = 1
            if getattr(state, "drafting", False):
                state.steps_in_round = n_before + len(tokens)
            return logits, feedback.clone(), state
    ex = Q.Qwen4ExpEagerExecutor.__new__(Q.Qwen4ExpEagerExecutor)
    ex.cfg, ex.model, ex.speculative_depth, ex._slots, ex.last_round = Scripted.cfg, Scripted(), 3, {}, None
    real_copy = Q.copy_state

    def marking_copy(st):                       # the copies made for drafting are marked, so the script can err there
        c = real_copy(st)
        c.drafting = True
        return c
    Q.copy_state = marking_copy
    try:
        first = ex.execute([Segment(0, [10, 11, 12], 0, [], uid=1)])          # prefill: the target answers 13
        assert first.tolist() == [13]
        out = ex.execute_speculative([Segment(0, [13], 3, [], uid=1)])
    finally:
        Q.copy_state = real_copy
    # drafts 14, 15 agree, the third (20) does not: two accepted, the target's 14, 15, 16 are emitted
    assert out == [[14, 15, 16]] and ex.last_round["accepted"] == [2] and ex.last_round["proposed"] == [3]
    slot = ex._slots[0]
    assert slot.state.length == 6                                             # 10 11 12 | 13 14 15 committed
    calls = ex.model.target_calls
    assert calls[0] == (0, [10, 11, 12]) and calls[1] == (3, [13, 14, 15, 20]) and calls[2] == (3, [13, 14, 15])
    # the head followed the committed tokens with the TARGET's residuals: (11, f10) (12, f11) | (13, f12) (14, f13) (15, f14)
    committed = [c for c in ex.model.head_calls if c[1] in ([11, 12], [13, 14, 15])]
    assert committed[0][2] == [10.0, 11.0] and committed[1][2] == [12.0, 13.0, 14.0]
    assert slot.draft.length == 5 and float(slot.carried[0, 0]) == 15.0
    # the next root is 16 at position 6
    out2 = ex.execute_speculative([Segment(0, [16], 6, [], uid=1)], depths=[0])
    assert out2 == [[17]] and ex.last_round["proposed"] == [0] and slot.state.length == 7


def test_serving_backend_with_the_draft_head(tmp_path):
    from argparse import Namespace

    from safetensors.torch import save_file

    from cubic_serve_b200.cli import SpeculativeConfig
    from cubic_serve_b200.models.checkpoint import CheckpointError
    from cubic_serve_b200.runtime.serving import build_backend
    args = Namespace(model="random:qwen4-exp-tiny", execution_mode="eager", pp_size=1, seed=0, max_model_len=256,
                     max_running_requests=4, token_budget=64, prefill_chunk_tokens=32, prefix_cache=True, thinking=None,
                     served_model_name=None)
    backend, _ = build_backend(args, [0], 1, SpeculativeConfig("mtp", 2), 8, 8)
    assert backend.engine.executor.speculative_depth == 2 and backend.engine.scheduler.decode_lookahead == 2
    backend.close()
    # a checkpoint with half a draft head is refused
    cfg = Q.tiny_config()
    w = Q.random_qwen4_exp_weights(cfg, 1, draft_head=True)
    d = tmp_path / "q"
    d.mkdir()
    src = json.loads(json.dumps({"model_type": "qwen4_exp", "language_model_only": True}))
    src["text_config"] = {
        "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
        "layer_types": list(cfg.layer_types), "num_attention_heads": cfg.num_q_heads, "num_key_value_heads": cfg.num_kv_heads,
        "head_dim": cfg.head_dim, "rope_parameters": {"mrope_section": [2, 1, 1], "rope_theta": 1e4, "partial_rotary_factor": 0.5},
        "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 8, "linear_value_head_dim": 8,
        "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 16, "shared_expert_intermediate_size": 16,
        "hc_count": 4, "hc_lowrank": 8, "indexer_n_heads": 2, "indexer_head_dim": 16, "indexer_budget": 16,
        "indexer_compress_ratio": 4, "ple_layer_ids": [2], "ple_embed_dim": 32, "ngram_size": 3, "heads_per_ngram": 2,
        "ngram_vocab_size_base": 500, "make_ngram_vocab_size_divisible_by": 4, "split_ngram_parts": 4,
        "ngram_shard_rows": 512, "eos_token_id": 1, "max_position_embeddings": 4096, "mtp_num_hidden_layers": 1}
    (d / "config.json").write_text(json.dumps(src))
    save_file({n: t.contiguous() for n, t in w.items()}, str(d / "model.safetensors"))
    got_cfg, got_w, _ = Q.admit_qwen4_exp_checkpoint(d)
    assert got_cfg.mtp_layers == 1 and "mtp.fc_embedding.weight" in got_w and len(got_w) == len(w)
    save_file({n: t.contiguous() for n, t in w.items() if n != "mtp.fc_hidden.weight"}, str(d / "model.safetensors"))
    with pytest.raises(CheckpointError, match="mtp.fc_hidden"):
        Q.admit_qwen4_exp_checkpoint(d)
