"""The eager model of the decoder families (CPU): it equals the dense reference decoder on dense models, its expert block
equals the mixture-of-experts oracle, its Gated DeltaNet row conventions equal the native loader's, and it serves
checkpoints that the native runner refuses (shared experts, projection biases, 256-wide heads) through the engine."""
from dataclasses import replace

import pytest
import torch

from cubic_serve_b200.models import checkpoint as C
from cubic_serve_b200.models import eager_family as EF
from cubic_serve_b200.models.config import ModelConfig, QuantSpec
from cubic_serve_b200.ops import eager, wq_pack


@pytest.mark.parametrize("scaling", [None, ("yarn", 4.0, 16, 32.0, 1.0, 1.2)])
def test_dense_model_equals_the_reference_decoder(scaling):
    from cubic_serve_b200.models.reference import DenseLayer, DenseWeights, EagerDecoder
    cfg = replace(ModelConfig(), qk_norm=True, rotary_dim=32 if scaling is None else 0, rope_scaling=scaling)
    w = EF.random_family_weights(cfg, 1, std=0.15)
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}"
        g = lambda n: w[f"{p}.{n}"]                                     # noqa: E731
        layers.append(DenseLayer(g("input_layernorm.weight"), g("post_attention_layernorm.weight"),
                                 g("self_attn.q_proj.weight"), g("self_attn.k_proj.weight"), g("self_attn.v_proj.weight"),
                                 g("self_attn.o_proj.weight"), g("mlp.gate_proj.weight"), g("mlp.up_proj.weight"),
                                 g("mlp.down_proj.weight"), g("self_attn.q_norm.weight"), g("self_attn.k_norm.weight")))
    dense = DenseWeights(w["model.embed_tokens.weight"], layers, w["model.norm.weight"], w["lm_head.weight"])
    toks = torch.randint(0, cfg.vocab_size, (1, 21), generator=torch.Generator().manual_seed(2))
    want, _ = EagerDecoder(cfg, dense).forward(toks, 0, None)
    model = EF.EagerFamilyModel(cfg, w)
    got, st = model.forward(toks[0].tolist())
    assert (got - want[0]).abs().max() < 1e-4
    a, st2 = model.forward(toks[0, :9].tolist())
    b, st2 = model.forward(toks[0, 9:].tolist(), st2)
    assert (torch.cat([a, b]) - got).abs().max() < 1e-4 and st2.length == 21
    with pytest.raises(ValueError):
        EF.EagerFamilyModel(cfg, {k: v for k, v in w.items() if not k.endswith("lm_head.weight")})


def test_expert_block_with_a_shared_expert():
    from cubic_serve_b200.models.moe import moe_reference
    cfg = replace(ModelConfig(), family="gqa_moe", num_experts=6, experts_per_token=2, moe_intermediate_size=32,
                  intermediate_size=0, shared_intermediate_size=48)
    w = EF.random_family_weights(cfg, 3, std=0.2)
    model = EF.EagerFamilyModel(cfg, w)
    x = torch.randn(7, cfg.hidden_size, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).float()
    p = "model.layers.0.mlp"
    got = model._ffn(x, p)
    gu = [torch.cat([w[f"{p}.experts.{e}.gate_proj.weight"], w[f"{p}.experts.{e}.up_proj.weight"]]) for e in range(6)]
    dn = [w[f"{p}.experts.{e}.down_proj.weight"] for e in range(6)]
    routed = moe_reference(x, w[f"{p}.gate.weight"], gu, dn, 2)
    s = p + ".shared_expert"
    shared = (torch.nn.functional.silu(x @ w[s + ".gate_proj.weight"].t()) * (x @ w[s + ".up_proj.weight"].t())) \
        @ w[s + ".down_proj.weight"].t()
    want = routed + shared * torch.sigmoid(x @ w[p + ".shared_expert_gate.weight"].t())
    assert float((got - want).norm() / want.norm()) < 2e-2               # the oracle rounds to bf16 between its steps
    assert float(shared.norm()) > 0.05 * float(routed.norm())


def test_gated_deltanet_rows_agree_with_the_native_loader(tmp_path):
    cfg = ModelConfig(name="hyb", family="qwen3_5", num_layers=4, hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=512, vocab_size=512, rotary_dim=64, qk_norm=True, zero_centered_norm=True,
                      gdn_interval=4, gdn_k_heads=2, gdn_v_heads=4, attn_output_gate=True, quant=QuantSpec("none", 16, 0))
    ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "h", cfg, seed=2, std=0.05))
    model = EF.EagerFamilyModel(ck.cfg, EF.family_weights_from_checkpoint(ck))
    native = C.load_decoder_weights(ck, "cpu")
    x = (torch.randn(6, 256, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16).float()
    # the native layout: sections q | k | v | z of all heads, b | a; the same oracle kernels on both sides
    gd = native.layers[0].gdn
    proj = x @ wq_pack.unpack_to_dense(gd.in_proj)[:gd.in_proj.n].float().t()
    C_ = (2 * gd.hk + gd.hv) * 128
    ba = x @ wq_pack.unpack_to_dense(gd.in_ba)[:2 * gd.hv].float().t()
    mixed, _ = eager.gdn_conv(proj[:, :C_].to(torch.bfloat16), gd.conv_w, None)
    out, _ = eager.gdn_delta(mixed, proj[:, C_:], ba, gd.a_log, gd.dt_bias, gd.norm_w, None, gd.hk, gd.hv, eps_norm=cfg.rms_eps)
    want = out.float() @ wq_pack.unpack_to_dense(gd.out)[:256].float().t()
    got = model._gdn(x, EF.FamilyLayerState(), "model.layers.0.linear_attn")
    assert float((got - want).norm() / want.norm()) < 1e-2
    # the gated attention layer: per-head [q | gate] rows, zero-centred q / k norms (the loader hands the kernels 1 + w)
    lw = native.layers[3]
    qn = ck.store.get("model.layers.3.self_attn.q_norm.weight").float()
    assert torch.allclose(lw.q_norm.float(), qn + 1)
    whole, st = model.forward(list(range(40, 70)))
    a, s2 = model.forward(list(range(40, 52)))
    b, s2 = model.forward(list(range(52, 70)), s2)
    # the Gated DeltaNet oracle rounds its operands to bf16 as the kernels do: a chunk boundary can flip such a rounding
    assert (torch.cat([a, b]) - whole).abs().max() < 5e-3 * whole.abs().max() and bool(torch.isfinite(whole).all())
    assert st.layers[3].key.shape == (30, 2, 128) and st.layers[0].recurrent.shape == (4, 128, 128)


def test_engine_serves_what_the_native_runner_refuses(tmp_path):
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = ModelConfig(name="wide", family="gqa_moe", num_layers=2, hidden_size=128, num_q_heads=2, num_kv_heads=1,
                      head_dim=256, intermediate_size=0, vocab_size=512, rotary_dim=64, qk_norm=True, num_experts=4,
                      experts_per_token=2, moe_intermediate_size=128, shared_intermediate_size=128, qkv_bias=True,
                      mrope_section=(16, 8, 8), quant=QuantSpec("cubic", 4, 128))
    ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "w", cfg, seed=6, std=0.08))
    assert ck.cfg.head_dim == 256 and ck.cfg.shared_intermediate_size == 128 and ck.cfg.qkv_bias
    assert ck.cfg.mrope_section == (16, 8, 8)
    with pytest.raises(C.CheckpointError, match="eager execution mode"):
        C.load_decoder_weights(ck, "cpu")
    w = EF.family_weights_from_checkpoint(ck)
    assert w["model.layers.0.self_attn.q_proj.bias"].shape == (512,)
    model = EF.EagerFamilyModel(ck.cfg, w)
    prompt = list(range(100, 131))
    lg, st = model.forward(prompt, last_only=True)
    want = []
    for _ in range(5):
        want.append(int(lg[0].argmax()))
        lg, st = model.forward([want[-1]], st, last_only=True)
    ex = EF.EagerFamilyExecutor(ck.cfg, w)
    eng = LLMEngine(ex, 64, SchedulerConfig(prefill_chunk_tokens=16, max_model_len=128))
    assert not eng.prefix.enabled
    rid = eng.add_request(prompt, SamplingParams(max_tokens=5))
    got = []
    while eng.has_unfinished:
        got += [o.token_id for o in eng.step() if o.request_id == rid and o.token_id is not None]
    assert got == want
    # the bias matters, and the stray-tensor rule still holds for such checkpoints
    w2 = dict(w)
    w2["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(512)
    assert not torch.allclose(EF.EagerFamilyModel(ck.cfg, w2).forward(prompt, last_only=True)[0],
                              model.forward(prompt, last_only=True)[0], atol=1e-4)


def test_draft_head_of_a_hybrid_expert_checkpoint_runs_lossless_rounds(tmp_path):
    """A hybrid + experts checkpoint with its multi-token-prediction head (gated attention layer with routed and shared
    experts): admitted by the closed inventory, and its draft / review rounds through the engine emit the tokens of
    plain greedy decoding."""
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = ModelConfig(name="hm", family="qwen3_5_moe", num_layers=4, hidden_size=128, num_q_heads=2, num_kv_heads=1,
                      head_dim=64, intermediate_size=0, vocab_size=384, rotary_dim=32, qk_norm=True, zero_centered_norm=True,
                      gdn_interval=4, gdn_k_heads=1, gdn_v_heads=2, attn_output_gate=True, num_experts=4, experts_per_token=2,
                      moe_intermediate_size=128, shared_intermediate_size=128, mtp_layers=1, quant=QuantSpec("none", 16, 0))
    ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "hm", cfg, seed=8, std=0.08))
    assert ck.cfg.mtp_layers == 1 and ck.cfg.is_hybrid and ck.cfg.is_moe
    assert "mtp.layers.0.mlp.experts.3.down_proj" in ck.payloads and "mtp.layers.0.mlp.shared_expert_gate.weight" in ck.plain
    w = EF.family_weights_from_checkpoint(ck)
    assert w["mtp.layers.0.self_attn.q_proj.weight"].shape == (2 * 2 * 64, 128) and w["mtp.fc.weight"].shape == (128, 256)
    model = EF.EagerFamilyModel(ck.cfg, w)
    assert model.has_draft_head
    toks = list(range(30, 52))
    _, st = model.forward(toks)
    fb = model.last_feedback
    d_all, h_all, _ = model.draft_forward(toks[1:], fb[:-1])
    d1, _, s1 = model.draft_forward(toks[1:9], fb[:8])
    d2, _, s1 = model.draft_forward(toks[9:], fb[8:-1], s1)
    assert (torch.cat([d1, d2]) - d_all).abs().max() < 1e-4 and h_all.shape == (21, 128)
    prompts = [toks, [7, 8, 9, 10, 11]]

    def run(depth):
        ex = EF.EagerFamilyExecutor(ck.cfg, w, speculative_depth=depth)
        eng = LLMEngine(ex, 64, SchedulerConfig(prefill_chunk_tokens=16, max_model_len=128))
        ids = [eng.add_request(p, SamplingParams(max_tokens=8)) for p in prompts]
        got = {i: [] for i in ids}
        while eng.has_unfinished:
            for o in eng.step():
                if o.token_id is not None:
                    got[o.request_id].append(o.token_id)
        return [got[i] for i in ids], eng, ex
    plain, _, _ = run(0)
    spec, eng, ex = run(2)
    assert spec == plain and getattr(eng, "spec_rounds", 0) > 0 and ex.last_round["proposed"]
    no_head = {k: v for k, v in w.items() if not k.startswith("mtp.")}
    with pytest.raises(ValueError):
        EF.EagerFamilyExecutor(replace(ck.cfg, mtp_layers=0), no_head, speculative_depth=2)
