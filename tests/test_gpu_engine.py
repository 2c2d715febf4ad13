"""Engine-level behaviour on the GPU: overlapped decode launches give the same tokens as step-by-step execution."""
import numpy as np
import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec

pytestmark = pytest.mark.gpu


def _engine(overlap, eos=None):
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="eng", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    runner = DecoderRunner(cfg, random_decoder_weights(cfg, dev, seed=0, std=0.05), num_pages=256, max_tokens=512)
    ex = GpuExecutor(runner, max_rows=16, max_prefill_tokens=512, max_model_len=256)
    ex.capture_decode_graphs()
    eng = LLMEngine(ex, 256, SchedulerConfig(max_running_requests=16, max_model_len=256, max_batched_tokens=512,
                                             enable_prefix_cache=False), eos_token_id=eos)
    eng.overlap_decode = overlap
    return eng, ex, runner


def test_overlapped_decode_matches_stepwise_on_device():
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (17, 40, 33, 64, 5, 9, 21)]
    sp = SamplingParams(max_tokens=24, ignore_eos=False)
    eng0, _, r0 = _engine(False)
    plain = eng0.generate(prompts, sp)
    # a token that really occurs in the middle of an output becomes the stop token of both runs
    eos = plain[3][9]
    eng_a, _, ra = _engine(False, eos)
    a = eng_a.generate(prompts, sp)
    eng_b, ex_b, rb = _engine(True, eos)
    launches = []
    orig = ex_b.launch
    ex_b.launch = lambda segs, feedback_rows=0: (launches.append(feedback_rows), orig(segs, feedback_rows))[1]
    b = eng_b.generate(prompts, sp)
    ra.ws.check_status()
    rb.ws.check_status()
    assert b == a and any(len(o) < 24 for o in a)
    assert sum(1 for f in launches if f) >= 10          # the steady state really ran ahead
    assert eng_b.pool.num_used == 0
    # sampling with temperature: the draw counters of look-ahead rows count the pending commit
    sp2 = SamplingParams(max_tokens=16, temperature=0.8, top_k=20, seed=7, ignore_eos=True)
    assert _engine(True)[0].generate(prompts[:4], sp2) == _engine(False)[0].generate(prompts[:4], sp2)
