"""The eager model of the hybrid expert family against the public Qwen3-Next implementation (when importable): Gated
DeltaNet layers with their per-key-head row grouping, gated attention with partial rotary and zero-centred norms, routed
experts with a sigmoid-gated shared expert."""
import pytest
import torch

from cubic_serve_b200.models import eager_family as EF
from cubic_serve_b200.models.config import ModelConfig


def _public_model():
    c = pytest.importorskip("transformers.models.qwen3_next.configuration_qwen3_next")
    m = pytest.importorskip("transformers.models.qwen3_next.modeling_qwen3_next")
    hf = c.Qwen3NextConfig(
        vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=1,
        head_dim=32, partial_rotary_factor=0.5, linear_conv_kernel_dim=4, linear_key_head_dim=128, linear_value_head_dim=128,
        linear_num_key_heads=1, linear_num_value_heads=2, decoder_sparse_step=1, moe_intermediate_size=32,
        shared_expert_intermediate_size=48, num_experts_per_tok=2, num_experts=4, norm_topk_prob=True, mlp_only_layers=[],
        full_attention_interval=4, rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False, rms_norm_eps=1e-6)
    hf._attn_implementation = "eager"
    torch.manual_seed(0)
    model = m.Qwen3NextForCausalLM(hf).eval()
    g = torch.Generator().manual_seed(1)
    for n, p in model.named_parameters():
        if n.endswith("A_log"):
            p.data.copy_(torch.rand(p.shape, generator=g) * 1.5)
        elif n.endswith("dt_bias"):
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.5)
        elif n.endswith("linear_attn.norm.weight"):
            p.data.copy_(1 + 0.1 * torch.randn(p.shape, generator=g))
        elif n.endswith("norm.weight"):
            p.data.copy_(0.1 * torch.randn(p.shape, generator=g))          # zero-centred: the weight is 1 + w
        elif n.endswith("conv1d.weight"):
            p.data.copy_(0.3 * torch.randn(p.shape, generator=g))
        else:
            p.data.copy_(0.08 * torch.randn(p.shape, generator=g))
    return model


def test_hybrid_expert_model_equals_the_public_implementation():
    ref = _public_model()
    cfg = ModelConfig(name="next", family="qwen3_5_moe", num_layers=4, hidden_size=64, num_q_heads=2, num_kv_heads=1,
                      head_dim=32, intermediate_size=0, vocab_size=320, rope_theta=10000.0, rotary_dim=16, qk_norm=True,
                      zero_centered_norm=True, gdn_interval=4, gdn_k_heads=1, gdn_v_heads=2, attn_output_gate=True,
                      num_experts=4, experts_per_token=2, moe_intermediate_size=32, shared_intermediate_size=48)
    w = {}
    for n, p in ref.named_parameters():
        t = p.detach()
        if n.endswith("mlp.experts.gate_up_proj"):                       # stacked [E, gate rows ; up rows, H]
            for e in range(4):
                w[f"{n[:-len('gate_up_proj')]}{e}.gate_proj.weight"] = t[e, :32]
                w[f"{n[:-len('gate_up_proj')]}{e}.up_proj.weight"] = t[e, 32:]
        elif n.endswith("mlp.experts.down_proj"):
            for e in range(4):
                w[f"{n[:-len('down_proj')]}{e}.down_proj.weight"] = t[e]
        else:
            w[n] = t
    assert set(w) == set(EF.family_tensor_shapes(cfg))
    ids = torch.randint(0, 320, (1, 24), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = ref(input_ids=ids).logits[0]
    # fp32 throughout: the same function
    exact, _ = EF.EagerFamilyModel(cfg, w, exact=True).forward(ids[0].tolist())
    assert float((exact - want).norm() / want.norm()) < 1e-4 and bool((exact.argmax(-1) == want.argmax(-1)).all())
    # with the storage roundings of the native kernels (bf16 between the steps of a Gated DeltaNet layer): close
    model = EF.EagerFamilyModel(cfg, w)
    rounded, _ = model.forward(ids[0].tolist())
    assert float((rounded - want).norm() / want.norm()) < 0.05
    a, st = EF.EagerFamilyModel(cfg, w, exact=True).forward(ids[0, :10].tolist())
    b, st = EF.EagerFamilyModel(cfg, w, exact=True).forward(ids[0, 10:].tolist(), st)
    assert float((torch.cat([a, b]) - want).norm() / want.norm()) < 1e-4      # chunked prefill: the same function too
