"""Projection biases (Qwen2 family) on the native runner: logits against the eager model of the same checkpoint."""
import numpy as np
import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec

pytestmark = pytest.mark.gpu


def test_biased_projections_match_the_eager_model(tmp_path):
    from safetensors.torch import load_file, save_file

    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models import eager_family as EF
    from cubic_serve_b200.parallel.tp_check import _rel_rows, _step_logits
    dev = torch.device("cuda")
    cfg = ModelConfig(name="Qwen2ForCausalLM", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, qkv_bias=True, quant=QuantSpec("cubic", 4, 128))
    path = C.write_random_checkpoint(tmp_path / "q2", cfg, seed=4, std=0.05)
    t = load_file(str(path / "model.safetensors"))
    g = torch.Generator().manual_seed(1)
    for n in list(t):
        if n.endswith("_proj.bias"):                                   # biases large enough to matter
            t[n] = torch.randn(t[n].shape, generator=g).to(torch.bfloat16)
    save_file(t, str(path / "model.safetensors"))
    ck = C.admit_checkpoint(path)
    assert ck.cfg.qkv_bias
    rng = np.random.default_rng(0)
    prompts = rng.integers(0, cfg.vocab_size, size=(6, 40)).tolist()
    w = C.load_decoder_weights(ck, dev)
    (l0, l1), (ids0, _) = _step_logits(ck.cfg, w, dev, None, prompts, 8, 8)
    model = EF.EagerFamilyModel(ck.cfg, EF.family_weights_from_checkpoint(ck), kv_bits=(8, 8))
    want0, want1 = [], []
    for p, first in zip(prompts, ids0):
        lg, st = model.forward(p, last_only=True)
        want0.append(lg[0])
        want1.append(model.forward([first], st, last_only=True)[0][0])      # the decode step on the native run's token
    e0 = _rel_rows(l0.cpu(), torch.stack(want0))
    e1 = _rel_rows(l1.cpu(), torch.stack(want1))
    assert float(e0.max()) < 0.06 and float(e1.max()) < 0.06, (e0, e1)
    # without the biases the same weights give clearly different logits: the comparison above has power
    for lw in w.layers:
        lw.qkv_bias = None
    (n0, _), _ = _step_logits(ck.cfg, w, dev, None, prompts, 8, 8)
    assert float(_rel_rows(n0.cpu(), torch.stack(want0)).min()) > 0.2


def test_shared_expert_matches_the_eager_model_and_replays_in_graphs(tmp_path):
    """Qwen2-MoE style checkpoint (routed experts + sigmoid-gated shared expert + projection biases) on the native runner."""
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models import eager_family as EF
    from cubic_serve_b200.models.decoder import DecoderRunner
    from cubic_serve_b200.parallel.tp_check import _rel_rows, _step_logits
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="Qwen2MoeForCausalLM", family="gqa_moe", num_layers=2, hidden_size=512, num_q_heads=8,
                      num_kv_heads=2, head_dim=128, intermediate_size=0, vocab_size=2048, rope_theta=1e6, qkv_bias=True,
                      num_experts=8, experts_per_token=2, moe_intermediate_size=256, shared_intermediate_size=512,
                      quant=QuantSpec("cubic", 4, 128))
    ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "q2m", cfg, seed=5, std=0.05))
    assert ck.cfg.shared_intermediate_size == 512 and ck.cfg.qkv_bias and ck.cfg.is_moe
    rng = np.random.default_rng(1)
    prompts = rng.integers(0, cfg.vocab_size, size=(8, 40)).tolist()
    w = C.load_decoder_weights(ck, dev)
    assert w.layers[0].moe.shared_gate_up is not None
    (l0, _), _ = _step_logits(ck.cfg, w, dev, None, prompts, 8, 8)
    model = EF.EagerFamilyModel(ck.cfg, EF.family_weights_from_checkpoint(ck), kv_bits=(8, 8))
    want = torch.stack([model.forward(p, last_only=True)[0][0] for p in prompts])
    err = _rel_rows(l0.cpu(), want)
    # a row whose near-tied router choice rounds the other way moves by more than rounding: the median and most rows bound
    assert float(err.median()) < 0.06 and int((err < 0.08).sum()) >= 6, err
    # engine level: eager launches and CUDA-graph replays of the decode step give the same tokens
    outs = []
    for graphs in (False, True):
        runner = DecoderRunner(ck.cfg, w, num_pages=128, max_tokens=512)
        ex = GpuExecutor(runner, max_rows=8, max_prefill_tokens=512, max_model_len=128, use_graphs=graphs)
        if graphs:
            ex.capture_decode_graphs()
        eng = LLMEngine(ex, 128, SchedulerConfig(max_running_requests=8, max_model_len=128, max_batched_tokens=512))
        outs.append(eng.generate(prompts[:4], SamplingParams(max_tokens=10, ignore_eos=True)))
        runner.ws.check_status()
    assert outs[0] == outs[1] and all(len(o) == 10 for o in outs[0])
    # without the shared expert the logits move clearly
    for lw in w.layers:
        lw.moe.shared_gate_up = None
    (n0, _), _ = _step_logits(ck.cfg, w, dev, None, prompts, 8, 8)
    assert float(_rel_rows(n0.cpu(), want).median()) > 0.15
