"""Checkpoints written by the public ``transformers`` implementations of the served architectures: admitted by the closed
inventory from their own ``config.json`` and tensor names, and run by the eager family model to the public model's logits.
Skipped where an architecture is not importable."""
import pytest
import torch

from cubic_serve_b200.models import checkpoint as C
from cubic_serve_b200.models import eager_family as EF

BASE = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False)
MOE = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[])
CASES = {
    "llama": ({}, "gqa_decoder"),
    "llama:llama3-scaling": (dict(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                "high_freq_factor": 4.0, "original_max_position_embeddings": 16}), "gqa_decoder"),
    "llama:linear-scaling": (dict(rope_scaling={"rope_type": "linear", "factor": 4.0}), "gqa_decoder"),
    "llama:yarn-scaling": (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 16,
                                              "beta_fast": 8.0, "beta_slow": 1.0}), "gqa_decoder"),
    "qwen3:yarn-scaling": (dict(head_dim=16, rope_scaling={"rope_type": "yarn", "factor": 8.0, "attention_factor": 1.3,
                                                           "original_max_position_embeddings": 64}), "gqa_decoder"),
    "mistral": (dict(head_dim=16, sliding_window=None), "gqa_decoder"),
    "mixtral": (dict(intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, sliding_window=None), "gqa_moe"),
    "mistral:window": (dict(head_dim=16, sliding_window=64), "gqa_decoder"),
    "qwen2": ({}, "gqa_decoder"),
    "qwen3": (dict(head_dim=16), "gqa_decoder"),
    "qwen3_moe": (dict(head_dim=16, norm_topk_prob=True, **MOE), "gqa_moe"),
    "qwen2_moe": (dict(shared_expert_intermediate_size=48, norm_topk_prob=False, **MOE), "gqa_moe"),
    "qwen3_next": (dict(num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1, head_dim=32, partial_rotary_factor=0.5,
                        linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_value_head_dim=128, linear_num_key_heads=1,
                        linear_num_value_heads=2, shared_expert_intermediate_size=48, norm_topk_prob=True,
                        full_attention_interval=4, **MOE), "qwen3_5_moe"),
}


@pytest.mark.parametrize("model_type", sorted(CASES))
def test_checkpoints_of_the_public_implementations(model_type, tmp_path):
    transformers = pytest.importorskip("transformers")
    extra, family = CASES[model_type]
    try:
        cfg = transformers.AutoConfig.for_model(model_type.split(":")[0], **{**BASE, **extra})
    except (ValueError, KeyError):
        pytest.skip(f"{model_type} is not known to this transformers")
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = transformers.AutoModelForCausalLM.from_config(cfg).eval().float()
    g = torch.Generator().manual_seed(1)
    for n, p in ref.named_parameters():
        if n.endswith("A_log"):
            p.data.copy_(torch.rand(p.shape, generator=g) * 1.5)
        elif n.endswith("linear_attn.norm.weight"):
            p.data.copy_(1 + 0.1 * torch.randn(p.shape, generator=g))
        elif n.endswith("norm.weight"):
            centre = 0.0 if model_type == "qwen3_next" else 1.0               # that family stores w of (1 + w)
            p.data.copy_(centre + 0.1 * torch.randn(p.shape, generator=g))
        elif n.endswith(("conv1d.weight", "dt_bias")):
            p.data.copy_(0.3 * torch.randn(p.shape, generator=g))
        else:
            p.data.copy_(0.08 * torch.randn(p.shape, generator=g))
    ref.save_pretrained(tmp_path, safe_serialization=True)
    ck = C.admit_checkpoint(tmp_path)
    assert ck.cfg.family == family and ck.cfg.num_layers == cfg.num_hidden_layers
    assert ck.cfg.qkv_bias == (model_type in ("qwen2", "qwen2_moe")) and ck.cfg.qk_norm == model_type.startswith("qwen3")
    assert (ck.cfg.rope_scaling is not None) == ("scaling" in model_type)
    assert ck.cfg.max_position == (64 if model_type == "mistral:window" else 512)
    model = EF.EagerFamilyModel(ck.cfg, EF.family_weights_from_checkpoint(ck), exact=True)
    ids = torch.randint(0, 320, (1, 20), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = ref(input_ids=ids).logits[0]
    got, state = model.forward(ids[0].tolist())
    assert float((got - want).norm() / want.norm()) < 1e-4, model_type
    # and one decode step on the public model's own cache
    with torch.no_grad():
        first = ref(input_ids=ids, use_cache=True)
        nxt = int(first.logits[0, -1].argmax())
        step = ref(input_ids=torch.tensor([[nxt]]), past_key_values=first.past_key_values, use_cache=True).logits[0, 0]
    mine, _ = model.forward([nxt], state)
    assert float((mine[0] - step).norm() / step.norm()) < 1e-4, model_type


@pytest.mark.parametrize("model_type", ["llama", "qwen2", "qwen3_moe", "qwen2_moe"])
def test_native_loader_reads_the_same_tensors(model_type, tmp_path):
    """The native runner's loader on a checkpoint of the public implementation: its fused projections, biases, expert
    stacks and shared expert hold the tensors the eager model runs on (bf16 here: the checkpoint is unquantized)."""
    from cubic_serve_b200.ops import wq_pack
    transformers = pytest.importorskip("transformers")
    extra, _ = CASES[model_type]
    if "moe_intermediate_size" in extra:                         # the GEMM operands are tiled along K in blocks of 64
        extra = {**extra, "moe_intermediate_size": 64}
    if "shared_expert_intermediate_size" in extra:
        extra = {**extra, "shared_expert_intermediate_size": 128}
    cfg = transformers.AutoConfig.for_model(model_type, **{**BASE, **extra})
    torch.manual_seed(3)
    ref = transformers.AutoModelForCausalLM.from_config(cfg).eval().float()
    for p in ref.parameters():
        p.data.normal_(0, 0.08)
    ref.save_pretrained(tmp_path, safe_serialization=True)
    ck = C.admit_checkpoint(tmp_path)
    fam = EF.family_weights_from_checkpoint(ck)
    w = C.load_decoder_weights(ck, "cpu")
    bf = lambda t: t.to(torch.bfloat16).float()                                 # noqa: E731
    p = "model.layers.1"
    lw = w.layers[1]
    want = torch.cat([fam[f"{p}.self_attn.{n}_proj.weight"] for n in "qkv"])
    assert torch.equal(wq_pack.unpack_to_dense(lw.qkv)[:want.shape[0]].float(), bf(want))
    assert torch.equal(wq_pack.unpack_to_dense(lw.o)[:64].float(), bf(fam[f"{p}.self_attn.o_proj.weight"]))
    if ck.cfg.qkv_bias:
        assert torch.equal(lw.qkv_bias.float(), bf(torch.cat([fam[f"{p}.self_attn.{n}_proj.bias"] for n in "qkv"])))
    else:
        assert lw.qkv_bias is None
    if ck.cfg.is_moe:
        gu = wq_pack.unpack_to_dense(lw.moe.gate_up).float()
        gu = gu.view(4, -1, gu.shape[-1])
        for e in (0, 3):
            pair = torch.cat([fam[f"{p}.mlp.experts.{e}.gate_proj.weight"], fam[f"{p}.mlp.experts.{e}.up_proj.weight"]])
            assert torch.equal(gu[e][:pair.shape[0]], bf(pair))
        assert torch.equal(wq_pack.unpack_to_dense(lw.moe.router)[:4].float(), bf(fam[f"{p}.mlp.gate.weight"]))
        if ck.cfg.shared_intermediate_size:
            sg = wq_pack.unpack_to_dense(lw.moe.shared_gate)[:1].float()
            assert torch.equal(sg, bf(fam[f"{p}.mlp.shared_expert_gate.weight"]))
            sd = wq_pack.unpack_to_dense(lw.moe.shared_down)[:64].float()
            assert torch.equal(sd, bf(fam[f"{p}.mlp.shared_expert.down_proj.weight"]))
    else:
        gu = wq_pack.unpack_to_dense(lw.gate_up)[:256].float()
        assert torch.equal(gu, bf(torch.cat([fam[f"{p}.mlp.gate_proj.weight"], fam[f"{p}.mlp.up_proj.weight"]])))
    assert torch.equal(wq_pack.unpack_to_dense(w.lm_head)[:320].float(), bf(fam["lm_head.weight"]))
