"""Speculative decoding with the MTP head: greedy rounds reproduce plain greedy decoding."""
import numpy as np
import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec

pytestmark = pytest.mark.gpu


def _build(spec_depth, force=None):
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.executor.spec_executor import SpeculativeGpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.models.mtp import MtpRunner, random_mtp_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="spec", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    w = random_decoder_weights(cfg, dev, seed=0, std=0.05)
    runner = DecoderRunner(cfg, w, num_pages=128, max_tokens=512)
    kw = dict(max_rows=8, max_prefill_tokens=512, max_model_len=256)
    if spec_depth:
        ex = SpeculativeGpuExecutor(runner, MtpRunner(runner, random_mtp_weights(cfg, dev, std=0.05)), spec_depth,
                                    force_acceptance=force, **kw)
    else:
        ex = GpuExecutor(runner, use_graphs=False, **kw)
    eng = LLMEngine(ex, 128, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                             enable_prefix_cache=False))
    return eng, ex, runner


def test_speculative_rounds_match_plain_greedy():
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (17, 40, 33, 64)]
    eng, ex, runner = _build(0)
    plain = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    eng2, ex2, runner2 = _build(3)
    spec = eng2.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    runner2.ws.check_status()
    assert all(len(o) == 12 for o in spec)
    agree = np.mean([a == b for pa, pb in zip(plain, spec) for a, b in zip(pa, pb)])
    assert agree >= 0.9, (agree, plain[0], spec[0])
    assert ex2.stats["rounds"] > 0 and ex2.stats["proposed"] == ex2.stats["rounds"] * 0 + ex2.stats["proposed"]
    assert eng2.pool.num_used == 0


def test_forced_acceptance_rate_and_tokens_per_round():
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 2048, 24).tolist() for _ in range(6)]
    eng, ex, runner = _build(4, force=0.7)
    out = eng.generate(prompts, SamplingParams(max_tokens=60, ignore_eos=True))
    runner.ws.check_status()
    assert all(len(o) == 60 for o in out)
    rate = ex.stats["accepted"] / ex.stats["proposed"]
    per_round = ex.stats["emitted"] / (ex.stats["proposed"] / 4)      # tokens per request and verify step
    # first-failure model with p = 0.7 and depth 4: E[accepted] = p + p^2 + p^3 + p^4 = 1.77 (about 140 samples here)
    assert 0.3 < rate < 0.6 and 2.0 < per_round < 3.4, (rate, per_round)


def test_dynamic_draft_length_stays_lossless_and_adapts():
    """With the planner on, random weights (drafts almost never match) drive every request's draft length down
    one level per decision boundary until drafting stops; the emitted tokens stay those of plain greedy decoding."""
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    from cubic_serve_b200.runtime.speculative import DraftPolicyConfig
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (21, 35, 50)]
    eng, ex, runner = _build(0)
    plain = eng.generate(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    eng2, ex2, runner2 = _build(3)
    ex2.timing = True
    eng2.enable_dynamic_draft(DraftPolicyConfig(decision_tokens=2, decision_min_rounds=2))
    spec = eng2.generate(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    runner2.ws.check_status()
    agree = np.mean([a == b for pa, pb in zip(plain, spec) for a, b in zip(pa, pb)])
    assert all(len(o) == 40 for o in spec) and agree >= 0.9
    # fewer proposals than the fixed depth would have made: the planner shortened / stopped the drafts
    assert ex2.stats["proposed"] < ex2.stats["rounds"] * 3 * len(prompts)
    assert eng2.pool.num_used == 0


def test_ngram_rounds_match_plain_greedy_and_accept_repetitions():
    """Prompt-lookup drafts verified by the target: the same tokens as plain greedy decoding; a model made to repeat
    itself gets most of its tokens from accepted drafts; steps without a draft replay the decode graphs."""
    from cubic_serve_b200.executor.spec_executor import NgramSpeculativeGpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    rng = np.random.default_rng(3)
    base = [rng.integers(0, 2048, n).tolist() for n in (9, 14, 11)]
    prompts = [p * 4 for p in base]                          # repeated context: the drafts have something to find
    eng, ex, runner = _build(0)
    plain = eng.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    dev = torch.device("cuda")
    cfg = runner.cfg
    runner2 = DecoderRunner(cfg, random_decoder_weights(cfg, dev, seed=0, std=0.05), num_pages=128, max_tokens=512)
    ex2 = NgramSpeculativeGpuExecutor(runner2, 3, max_rows=8, max_prefill_tokens=512, max_model_len=256)
    assert ex2.capture_decode_graphs([4, 8]) == [4, 8]
    eng2 = LLMEngine(ex2, 128, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                               enable_prefix_cache=False))
    spec = eng2.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    runner2.ws.check_status()
    assert all(len(o) == 24 for o in spec)
    agree = np.mean([a == b for pa, pb in zip(plain, spec) for a, b in zip(pa, pb)])
    assert agree >= 0.9, (agree, plain[0], spec[0])
    assert ex2.stats["rounds"] > 0 and ex2.stats["proposed"] > 0
    assert ex2.stats["accepted"] <= ex2.stats["proposed"]
    assert eng2.pool.num_used == 0
    # a sequence the proposer cannot have seen twice (a short random prompt) takes plain graph-replayed decode steps
    eng3 = LLMEngine(ex2, 128, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                               enable_prefix_cache=False))
    before = dict(ex2.graph_rt.stats()["slots"][4])
    eng3.generate([rng.integers(0, 2048, 6).tolist()], SamplingParams(max_tokens=3, ignore_eos=True))
    assert ex2.graph_rt.stats()["slots"][4]["replays"] > before["replays"]


def test_mtp_head_loaded_from_a_checkpoint_drafts_losslessly(tmp_path):
    import dataclasses
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.executor.spec_executor import SpeculativeGpuExecutor
    from cubic_serve_b200.models.checkpoint import admit_checkpoint, load_decoder_weights, load_mtp_weights, \
        write_random_checkpoint
    from cubic_serve_b200.models.decoder import DecoderRunner
    from cubic_serve_b200.models.mtp import MtpRunner
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="spec-ck", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, qk_norm=True, mtp_layers=1,
                      quant=QuantSpec("cubic", 4, 128))
    ck = admit_checkpoint(write_random_checkpoint(tmp_path / "ck", cfg, seed=1, std=0.05))
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (21, 34)]
    sched = SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512, enable_prefix_cache=False)
    kw = dict(max_rows=8, max_prefill_tokens=512, max_model_len=256)
    r1 = DecoderRunner(ck.cfg, load_decoder_weights(ck, dev), num_pages=128, max_tokens=512)
    plain = LLMEngine(GpuExecutor(r1, use_graphs=False, **kw), 128, sched).generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    r2 = DecoderRunner(ck.cfg, load_decoder_weights(ck, dev), num_pages=128, max_tokens=512)
    ex = SpeculativeGpuExecutor(r2, MtpRunner(r2, load_mtp_weights(ck, dev)), 2, **kw)
    spec = LLMEngine(ex, 128, sched).generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    r2.ws.check_status()
    agree = np.mean([a == b for pa, pb in zip(plain, spec) for a, b in zip(pa, pb)])
    assert agree >= 0.9 and ex.stats["rounds"] > 0, (agree, plain, spec)


def _shaped(val, temp, top_p, top_k):
    """fp64 oracle of the sampler's shaping over one candidate row (value desc)."""
    k = len(val) if top_k <= 0 else min(top_k, len(val))
    w = np.exp((val[:k] - val[0]) / temp)
    pr = w / w.sum()
    keep = k
    if top_p < 1.0:
        keep = int(np.searchsorted(np.cumsum(pr), top_p) + 1)
    out = np.zeros(len(val))
    out[:keep] = w[:keep] / w[:keep].sum()
    return out


def test_rejection_sampling_emits_the_targets_distribution():
    """p / q verification (``verify_sampled_kernel``): with drafts drawn from q, the first emitted token is distributed
    as the target's shaped distribution p whatever q is; greedy rows reduce to the prefix match; a replay is equal."""
    from cubic_serve_b200.ops import kernels as K
    dev = torch.device("cuda")
    C, R, D = K.SAMPLE_CANDIDATES, 40000, 2
    rng = np.random.default_rng(0)
    ids = np.arange(100, 100 + C)
    p_val = np.sort(rng.normal(0, 1.5, C))[::-1].copy()
    q_order = rng.permutation(C)                       # the head ranks the same tokens differently
    q_val = np.sort(rng.normal(0, 1.5, C))[::-1].copy()
    q_ids = ids[q_order]
    temp, top_p, top_k = 0.8, 0.9, 12
    P, Q = _shaped(p_val, temp, top_p, top_k), _shaped(q_val, temp, top_p, top_k)
    drafts = q_ids[rng.choice(C, size=(R, D), p=Q)]

    def t(a, dt):
        return torch.tensor(np.ascontiguousarray(a), dtype=dt, device=dev)

    qv = t(np.broadcast_to(q_val, (R, D, C)), torch.float32)
    qi = t(np.broadcast_to(q_ids, (R, D, C)), torch.int32)
    pv = t(np.broadcast_to(p_val, (R, D + 1, C)), torch.float32)
    pi = t(np.broadcast_to(ids, (R, D + 1, C)), torch.int32)
    args = dict(draft_ids=t(drafts, torch.int32), depth=torch.full((R,), D, dtype=torch.int32, device=dev), max_depth=D,
                temperature=torch.full((R,), temp, device=dev), top_p=torch.full((R,), top_p, device=dev),
                top_k=torch.full((R,), top_k, dtype=torch.int32, device=dev),
                seeds=torch.arange(R, dtype=torch.int64, device=dev) * 7919 + 13,
                counters=torch.full((R,), 5, dtype=torch.int64, device=dev))
    acc, bonus = torch.zeros(R, dtype=torch.int32, device=dev), torch.zeros(R, dtype=torch.int32, device=dev)
    out = torch.zeros(R, D + 1, dtype=torch.int32, device=dev)
    K.verify_sampled(qv, qi, pv, pi, accepted=acc, bonus=bonus, emitted=out, **args)
    torch.cuda.synchronize()
    first = out[:, 0].cpu().numpy()
    emp = np.array([(first == i).mean() for i in ids])
    assert np.abs(emp - P).max() < 0.012, (emp, P)                      # ~4 sigma at 40 k samples
    assert set(np.unique(first)) <= set(ids[P > 0])                      # nothing outside the shaped support
    a = acc.cpu().numpy()
    # acceptance rate of one draft = sum_x min(p, q)
    Qp = np.zeros(C); Qp[q_order] = Q                                    # q's probability of token ids[j]
    assert abs((a >= 1).mean() - np.minimum(P, Qp).sum()) < 0.012
    # the token after the accepted prefix is the bonus, the prefix itself is the drafts
    o = out.cpu().numpy()
    assert all((o[r, :a[r]] == drafts[r, :a[r]]).all() and o[r, a[r]] == bonus[r].item() for r in range(0, R, 997))
    out2 = torch.zeros_like(out)
    K.verify_sampled(qv, qi, pv, pi, accepted=acc, bonus=bonus, emitted=out2, **args)
    assert torch.equal(out, out2)
    # greedy requests: one-hot distributions, longest matching prefix
    args["temperature"] = torch.zeros(R, device=dev)
    g_drafts = np.full((R, D), ids[0]); g_drafts[::2, 1] = ids[3]
    args["draft_ids"] = t(g_drafts, torch.int32)
    # (a greedy draft is the head's own first candidate: q is one-hot there, so q ranks the tokens like p here)
    qi_g = t(np.broadcast_to(ids, (R, D, C)), torch.int32)
    K.verify_sampled(qv, qi_g, pv, pi, accepted=acc, bonus=bonus, emitted=out, **args)
    a = acc.cpu().numpy()
    assert (a[1::2] == 2).all() and (a[::2] == 1).all() and (bonus.cpu().numpy() == ids[0]).all()


def test_sampled_requests_take_speculative_rounds():
    """Requests with temperature > 0 run through the rounds (drafts drawn from the head, p / q verification): same
    seeds give the same tokens, and every token lies in the target's top-k."""
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (20, 35, 48)]
    sp = SamplingParams(max_tokens=16, ignore_eos=True, temperature=0.9, top_k=8, top_p=0.95, seed=1234)
    eng, ex, runner = _build(3)
    a = eng.generate(prompts, sp)
    runner.ws.check_status()
    assert ex.stats["rounds"] > 0 and all(len(o) == 16 for o in a)
    eng2, ex2, runner2 = _build(3)
    b = eng2.generate(prompts, sp)
    assert a == b
    # a different seed gives other tokens
    eng3, ex3, _ = _build(3)
    c = eng3.generate(prompts, SamplingParams(max_tokens=16, ignore_eos=True, temperature=0.9, top_k=8, top_p=0.95, seed=99))
    assert a != c


def test_constrained_requests_take_speculative_rounds_under_their_grammar():
    """A ``choice`` constraint during MTP rounds: every review row is sampled under the grammar's mask for its position,
    so the emitted tokens spell one of the options and equal what plain constrained decoding emits."""
    from cubic_serve_b200.generation.constraints import ChoiceMatcher
    from cubic_serve_b200.runtime.scheduler import SamplingParams

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [100 + ord(c) for c in text]

    eos = 3
    options = ["alpha beta", "alphabet soup", "gamma"]
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (18, 31)]

    def run(depth):
        eng, ex, runner = _build(depth)
        outs = []
        for p in prompts:
            sp = SamplingParams(max_tokens=24, stop_token_ids=(eos,), matcher=ChoiceMatcher(options, Tok(), eos))
            rid = eng.add_request(p, sp)
            req = eng.requests[rid]
            free = eng.add_request(p[::-1], SamplingParams(max_tokens=9, ignore_eos=True))   # shares the rounds
            free_req = eng.requests[free]
            while eng.has_unfinished:
                eng.step()
            assert len(free_req.output) == 9
            outs.append(list(req.output))
        runner.ws.check_status()
        return outs, ex

    plain, _ = run(0)
    spec, ex = run(3)
    assert ex.stats["rounds"] > 0
    for toks in spec:
        assert toks[-1] == eos and "".join(chr(t - 100) for t in toks[:-1]) in options
    assert spec == plain


def test_captured_rounds_equal_eager_rounds():
    """Greedy rounds replay captured graphs (a proposal graph per capacity, a review + verification graph per
    capacity and depth); they must emit exactly what the eager rounds emit, also when the number of requests changes
    between rounds (other capacity, padded rows) and with forced acceptance (accepted prefixes of every length)."""
    from cubic_serve_b200.executor.spec_executor import SpeculativeGpuExecutor
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, 2048, n).tolist() for n in (17, 40, 33, 64, 21)]
    lens = [12, 5, 9, 12, 7]                           # requests leave at different times: capacities 8 -> 4 -> 2 -> 1

    def run(graphs, force):
        eng, ex, runner = _build(3, force=force)
        ex.round_graphs = graphs
        ex._rng = np.random.default_rng(0)
        rids = [eng.add_request(p, SamplingParams(max_tokens=n, ignore_eos=True)) for p, n in zip(prompts, lens)]
        reqs = [eng.requests[r] for r in rids]
        while eng.has_unfinished:
            eng.step()
        runner.ws.check_status()
        return [list(r.output) for r in reqs], ex.stats

    for force in (None, 0.6):
        eager, st_e = run(False, force)
        graphed, st_g = run(True, force)
        assert st_e["graphed_rounds"] == 0 and st_g["graphed_rounds"] == st_g["rounds"] > 0
        assert [len(o) for o in graphed] == lens
        assert graphed == eager, (force, graphed[0], eager[0])
        if force is not None:
            assert st_g["accepted"] == st_e["accepted"] > 0
