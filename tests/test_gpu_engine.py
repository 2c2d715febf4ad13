"""Engine-level behaviour on the GPU: overlapped decode launches give the same tokens as step-by-step execution."""
import numpy as np
import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec

pytestmark = pytest.mark.gpu


def _engine(overlap, eos=None, pool_pages=256):
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
    eng = LLMEngine(ex, pool_pages, SchedulerConfig(max_running_requests=16, max_model_len=256, max_batched_tokens=512,
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


def test_programmatic_dependent_launch_changes_no_token():
    """Kernels may start while their predecessor is still running (csrc/launch.cuh); each waits for it before it
    touches dependent memory.  Eager steps and graph replays with the overlap on give the tokens of a run with it off."""
    from cubic_serve_b200.ops import native
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    lib = native.lib()
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (17, 40, 33, 64, 5, 9, 21, 50, 31, 12)]
    sp = SamplingParams(max_tokens=32, ignore_eos=True)
    try:
        lib.cb_set_pdl(0)
        want = _engine(True)[0].generate(prompts, sp)
        lib.cb_set_pdl(1)
        assert lib.cb_pdl_enabled() == 1
        for _ in range(3):
            eng, _, runner = _engine(True)
            assert eng.generate(prompts, sp) == want
            runner.ws.check_status()
    finally:
        lib.cb_set_pdl(1)


def test_preempted_requests_read_their_own_pages_after_readmission():
    """A pool too small for all requests: some are preempted, re-admitted (often into their old slot, with other
    pages) and must produce the tokens of an unpreempted run.  A stale page-table row would make attention read
    pages that now belong to other requests."""
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (40, 37, 45, 33, 50, 41)]
    sp = SamplingParams(max_tokens=40, ignore_eos=True)
    want = _engine(False)[0].generate(prompts, sp)
    for overlap in (False, True):
        eng, _, runner = _engine(overlap, pool_pages=20)          # 19 usable pages; six requests end at 5-6 pages each
        ids = [eng.add_request(p, SamplingParams(**vars(sp))) for p in prompts]
        reqs = [eng.requests[i] for i in ids]
        while eng.has_unfinished:
            eng.step()
        runner.ws.check_status()
        assert sum(r.preemptions for r in reqs) > 0
        assert [r.output for r in reqs] == want


def test_thinking_budget_state_machine_and_engine():
    """Device-side thinking budgets: the kernel against a Python model of the state machine, then end to end: after
    the budget the forced end sequence appears in the request's output, other requests are untouched."""
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    dev = torch.device("cuda")
    end, seq = 7, [3, 7, 9]
    rb = K.ReasoningBudget(8, end, seq, dev)
    rng = np.random.default_rng(0)
    left, fpos = [-1] * 8, [0] * 8
    for step in range(40):
        rows = 6
        slots = rng.permutation(8)[:rows].astype(np.int32)            # a request has one sampled row per step
        if step % 5 == 0:
            slots[rng.integers(0, rows)] = -1                           # a padding row now and then
        init = rng.choice([-2, -2, -2, -1, 0, 2, 5], rows).astype(np.int32)
        ids = rng.integers(0, 12, rows).astype(np.int32)
        want = ids.copy()
        for r in range(rows):
            s = int(slots[r])
            if s < 0:
                continue
            if init[r] >= -1:
                left[s], fpos[s] = int(init[r]), 0
            if left[s] >= 0:
                if fpos[s] > 0 or left[s] == 0:
                    want[r] = seq[fpos[s]]
                    fpos[s] += 1
                    if fpos[s] >= len(seq):
                        left[s], fpos[s] = -1, 0
                elif want[r] == end:
                    left[s] = -1
                else:
                    left[s] -= 1
        d_ids = torch.tensor(ids, device=dev)
        rb.apply(d_ids, torch.tensor(slots, device=dev), torch.tensor(init, device=dev), rows)
        assert d_ids.cpu().tolist() == want.tolist()
        assert rb.left.cpu().tolist() == left and rb.fpos.cpu().tolist() == fpos

    # end to end (decode graphs + overlapped launches): request 1 has a budget of 5 tokens
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    cfg = ModelConfig(name="eng", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    outs = {}
    for budgets in (False, True):
        runner = DecoderRunner(cfg, random_decoder_weights(cfg, dev, seed=0, std=0.05), num_pages=256, max_tokens=512,
                               max_requests=16)
        runner.enable_reasoning_budget(2047, [2046, 2047])
        ex = GpuExecutor(runner, max_rows=16, max_prefill_tokens=512, max_model_len=256)
        ex.capture_decode_graphs()
        eng = LLMEngine(ex, 256, SchedulerConfig(max_running_requests=16, max_model_len=256, max_batched_tokens=512,
                                                 enable_prefix_cache=False))
        prompts = [np.random.default_rng(i).integers(0, 2000, 20 + i).tolist() for i in range(3)]
        ids = [eng.add_request(p, SamplingParams(max_tokens=14, ignore_eos=True,
                                                 thinking_budget=5 if (budgets and i == 1) else None))
               for i, p in enumerate(prompts)]
        reqs = [eng.requests[i] for i in ids]
        while eng.has_unfinished:
            eng.step()
        outs[budgets] = [r.output for r in reqs]
        runner.ws.check_status()
    plain, forced = outs[False], outs[True]
    assert forced[0] == plain[0] and forced[2] == plain[2]
    assert forced[1][:5] == plain[1][:5] and forced[1][5:7] == [2046, 2047] and len(forced[1]) == 14


def test_qualification_run_passes():
    from cubic_serve_b200.guardrail.qualify import run_qualification
    rep = run_qualification(0, quick=True)
    assert rep["ok"], [r for r in rep["results"] if r["class"] == "mismatch"]
    names = " ".join(r["kernel"] for r in rep["results"])
    for part in ("CTA pairs", "SwiGLU", "gdn_delta", "hadamard", "graph replay", "cross-M wq_gemm", "cross-M rmsnorm"):
        assert part in names
    cross = {r["kernel"]: r["class"] for r in rep["results"] if r["kernel"].startswith("cross-M")}
    assert cross["cross-M rmsnorm rows 3 of 256"] == "exact"            # row-wise kernels are batch invariant bit for bit
    print("cross-M classes:", cross)


def test_constrained_requests_decode_in_graphs():
    """Structured-output masks are an input of the captured sampler: a constrained request decodes by graph replay
    (no eager step), next to an unconstrained one whose tokens do not change."""
    from cubic_serve_b200.generation.constraints import ChoiceMatcher
    from cubic_serve_b200.runtime.scheduler import SamplingParams

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [ord(c) for c in text]

    eos = 3
    options = ["yes", "no", "maybe"]
    free_prompt = np.random.default_rng(5).integers(0, 2000, 30).tolist()
    eng0, _, _ = _engine(False)
    baseline = eng0.generate([free_prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0]
    eng, ex, runner = _engine(True)
    eager_steps = []
    body = ex._body
    ex._body = lambda b: (eager_steps.append(b.num_tokens), body(b))[1]
    m = ChoiceMatcher(options, Tok(), eos)
    rid = eng.add_request([5, 6, 7, 8], SamplingParams(temperature=1.0, top_k=20, seed=1, max_tokens=12,
                                                       stop_token_ids=(eos,), matcher=m))
    other = eng.add_request(free_prompt, SamplingParams(max_tokens=10, ignore_eos=True))
    reqs = {rid: eng.requests[rid], other: eng.requests[other]}
    while eng.has_unfinished:
        eng.step()
    runner.ws.check_status()
    toks = reqs[rid].output
    assert toks[-1] == eos and "".join(chr(t) for t in toks[:-1]) in options
    assert reqs[other].output == baseline
    assert eager_steps and all(n > 1 for n in eager_steps)          # only the prefill step ran eagerly


def test_prefix_resume_equals_cold_start_on_device():
    """Cold vs prefix-resumed identity on the native executor: a request that finds its prompt's pages in the prefix
    cache (shared pages, copy-on-write of the partly filled last page) continues exactly as the cold request did;
    a request that shares only the first part of a cached prompt reuses those pages and prefills the rest."""
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="pfx", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    weights = random_decoder_weights(cfg, dev, seed=0, std=0.05)

    def engine(prefix):
        runner = DecoderRunner(cfg, weights, num_pages=256, max_tokens=512)
        ex = GpuExecutor(runner, max_rows=16, max_prefill_tokens=512, max_model_len=256)
        ex.capture_decode_graphs([4, 16])
        return LLMEngine(ex, 256, SchedulerConfig(max_running_requests=16, max_model_len=256, max_batched_tokens=512,
                                                  enable_prefix_cache=prefix)), runner

    rng = np.random.default_rng(4)
    base = rng.integers(0, 2048, 70).tolist()                   # four full pages and a part of the fifth
    fork = base[:48] + rng.integers(0, 2048, 20).tolist()       # shares three pages with it
    sp = SamplingParams(max_tokens=12, ignore_eos=True)
    cold_eng, r0 = engine(False)
    cold = [cold_eng.generate([p], sp)[0] for p in (base, fork)]
    eng, r1 = engine(True)
    first = eng.generate([base], sp)[0]
    assert first == cold[0] and eng.prefix.hit_tokens == 0
    again = eng.generate([base], sp)[0]                         # every full page of the prompt comes from the cache
    assert eng.prefix.hit_tokens >= 64 and again == cold[0]
    hits = eng.prefix.hit_tokens
    forked = eng.generate([fork], sp)[0]
    assert eng.prefix.hit_tokens - hits >= 48 and forked == cold[1]
    both = eng.generate([base, fork], sp)                       # two requests sharing cached pages in one batch
    assert both == cold
    r0.ws.check_status()
    r1.ws.check_status()
    assert eng.pool.num_used == len(eng.prefix)                 # only cache entries keep pages


def test_captured_decode_graphs_pass_the_graph_level_audits():
    """Whole-graph audits (``guardrail/graph_audit.py``): two bucket sizes agree, poisoned padding rows change no bit
    of the real rows, and a request's logits do not depend on the row it occupies."""
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.guardrail.graph_audit import audit_decode_graphs
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    dev = torch.device("cuda")
    cfg = ModelConfig(name="audit", num_layers=3, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    w = random_decoder_weights(cfg, dev, seed=0, std=0.05)

    def build():
        runner = DecoderRunner(cfg, w, num_pages=64, max_tokens=256)
        return GpuExecutor(runner, max_rows=32, max_prefill_tokens=256, max_model_len=128)

    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (19, 33, 40, 27, 16)]
    rep = audit_decode_graphs(build, prompts, capacities=(8, 32), steps=3)
    assert rep.cross_m_ids_equal and rep.cross_m_max_rel < 2e-2, rep
    assert rep.poisoned_padding_bit_identical and rep.poisoned_padding_finite, rep
    assert rep.permutation_bit_identical, rep
    assert rep.ok
