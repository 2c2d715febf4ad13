import pytest

from cubic_serve_b200.runtime.speculative import (CostCurve, DraftAction, DraftPlanner, DraftPolicyConfig,
                                                  RequestDraftState)


def test_config_validation():
    DraftPolicyConfig.from_dict({"decision_tokens": 10})
    for bad in ({"cost_sample_window": 2}, {"history_decay": 1.0}, {"prior_success": 0}, {"bogus": 1}, {"terminal_stop_margin": -1}):
        with pytest.raises(ValueError):
            DraftPolicyConfig.from_dict(bad)


def test_survival_curve_prior_and_updates():
    s = RequestDraftState(3, 4)
    assert s.survival() == pytest.approx((0.8, 0.64, 0.512, 0.4096))        # Beta(4, 1) prior mean 0.8 per depth
    for _ in range(50):
        s.observe(accepted=1, proposed=3)                                     # depth 1 always accepted, depth 2 never
    sv = s.survival()
    assert sv[0] > 0.95 and sv[1] < 0.2 and sv[2] < sv[1] and sv == tuple(sorted(sv, reverse=True))
    assert s.expected_tokens(0) == 1.0 and s.expected_tokens(2) == pytest.approx(1 + sv[0] + sv[1])
    with pytest.raises(ValueError):
        s.observe(accepted=4, proposed=3)
    with pytest.raises(ValueError):
        s.observe(accepted=0, proposed=4)


def test_decisions_need_boundary_and_move_one_level():
    s = RequestDraftState(2, 4)
    assert s.move_toward(4).action is DraftAction.HOLD                       # not ready yet
    for _ in range(8):
        s.observe(accepted=2, proposed=2)                                     # 8 rounds x 3 tokens = 24
    assert s.ready
    d = s.move_toward(4)
    assert (d.action, d.previous_tokens, d.next_tokens) == (DraftAction.PROMOTE, 2, 3) and not s.ready
    for _ in range(8):
        s.observe(accepted=0, proposed=3)
    assert not s.ready                                                         # 8 rounds but only 8 tokens
    for _ in range(16):
        s.observe(accepted=0, proposed=3)
    assert s.move_toward(0).next_tokens == 2
    s2 = RequestDraftState(1, 2)
    for _ in range(24):
        s2.observe(accepted=0, proposed=1)
    d = s2.move_toward(0)
    assert d.next_tokens == 0 and s2.stopped
    with pytest.raises(RuntimeError):
        s2.observe(accepted=0, proposed=1)
    assert RequestDraftState(3, 3).stop_for_capacity().next_tokens == 0


def test_cost_curve_median_ema_and_interpolation():
    c = CostCurve(alpha=0.5, window=3)
    assert c.estimate(8) is None
    c.observe(8, 10.0)
    c.observe(8, 100.0); c.observe(8, 12.0)
    assert c.estimate(8) == 10.0                                             # window not full yet
    c.observe(8, 14.0)                                                       # median(100, 12, 14) = 14
    assert c.estimate(8) == pytest.approx(12.0)
    c.observe(32, 30.0)
    assert c.estimate(20) == pytest.approx(12 + (20 - 8) / 24 * 18)
    assert c.estimate(4) == pytest.approx(12.0)                              # no downward extrapolation
    assert c.estimate(64) == pytest.approx(60.0)


def test_planner_prefers_drafting_when_cheap_and_stops_when_useless():
    p = DraftPlanner((8, 16, 32, 64, 128))
    for cap, ms in ((8, 5.0), (16, 5.2), (32, 5.6), (64, 6.5), (128, 8.0)):
        p.target_cost.observe(cap, ms)
        p.proposal_cost.observe(cap, 0.3)
    good = [RequestDraftState(2, 4) for _ in range(8)]
    for s in good:
        for _ in range(12):
            s.observe(accepted=2, proposed=2)
    assert p.best_uniform_k(good, 4) >= 3                                     # high acceptance: longer drafts
    plans = p.plan({f"r{i}": s for i, s in enumerate(good)})
    assert all(pl.draft_tokens == 3 and pl.decision.action is DraftAction.PROMOTE for pl in plans)
    bad = [RequestDraftState(1, 4) for _ in range(8)]
    for s in bad:
        for _ in range(150):
            s.observe(accepted=0, proposed=1)
    assert p.best_uniform_k(bad, 4) == 0
    # marginal benefit below the 3 % stop margin keeps drafting alive
    p2 = DraftPlanner((8,), DraftPolicyConfig(terminal_stop_margin=0.5))
    p2.target_cost.observe(8, 5.0)
    p2.proposal_cost.observe(8, 0.01)
    assert p2.best_uniform_k(bad, 1) == 1
    assert DraftPlanner((8,)).best_uniform_k(good, 4) == 4                    # no cost data yet: keep the maximum


def test_engine_round_loop_uses_planned_depths():
    """LLMEngine asks the planner for every request's draft length, passes them to the executor, and feeds the
    acceptance back; with drafts that never match the lengths shrink to zero and decoding continues."""
    import numpy as np
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig

    class FakeSpec:
        speculative_depth = 3
        vocab_size = 64

        def __init__(self):
            self.seen = []
            self.last_round = None

        def copy_pages(self, pairs):
            pass

        def execute(self, segs):
            return np.asarray([7 for s in segs if s.sample], dtype=np.int32)

        def execute_speculative(self, segs, depths=None):
            depths = depths or [self.speculative_depth] * len(segs)
            self.seen.append(list(depths))
            self.last_round = {"depth": max(depths), "accepted": [0] * len(segs), "proposed": list(depths),
                               "proposal_ms": 1.0 * max(depths), "target_ms": 5.0}
            return [[9] for _ in segs]                     # nothing accepted: only the bonus token

    ex = FakeSpec()
    eng = LLMEngine(ex, num_pages=64, scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=256,
                                                                       enable_prefix_cache=False))
    eng.enable_dynamic_draft(DraftPolicyConfig(decision_tokens=2, decision_min_rounds=2))
    out = eng.generate([[1, 2, 3], [4, 5, 6, 7]], SamplingParams(max_tokens=30, ignore_eos=True))
    assert all(len(o) == 30 for o in out)
    assert ex.seen[0] == [3, 3]
    assert max(ex.seen[-1]) < 3                             # shortened
    flat = [d for round_ in ex.seen for d in round_]
    assert all(a >= b for a, b in zip([r[0] for r in ex.seen], [r[0] for r in ex.seen][1:]))   # monotone, one level a time
    assert set(flat) <= {0, 1, 2, 3}


def test_ngram_index_proposes_what_followed_the_latest_match():
    from cubic_serve_b200.runtime.ngram import NgramIndex, NgramProposer
    i = NgramIndex(max_n=4, min_n=2)
    i.extend([1, 2, 3, 4, 5, 1, 2, 3])
    assert i.propose(3) == [4, 5, 1] and i.propose(5) == [4, 5, 1, 2, 3] and i.propose(0) == []
    i.extend([9, 1, 2, 3])                                   # the latest occurrence wins: after "1 2 3" came 9
    assert i.propose(2) == [9, 1]
    loop = NgramIndex(3, 2)
    loop.extend([7, 8, 7, 8])
    assert loop.propose(5) == [7, 8, 7, 8, 7]                # a repetition continues into itself
    fresh = NgramIndex()
    fresh.extend([1, 2, 3, 4])
    assert fresh.propose(3) == []
    fresh.truncate(2)
    assert fresh.tokens == [1, 2]
    import pytest
    with pytest.raises(ValueError):
        NgramIndex(max_n=1, min_n=2)
    p = NgramProposer()
    assert p.propose("a", [5, 6, 7, 5, 6], 2) == [7, 5]
    assert p.propose("a", [5, 6, 7, 5, 6, 7], 2) == [5, 6]   # incremental: only the new token is indexed
    assert p.propose("a", [1, 2], 2) == []                   # another sequence under the same id: rebuilt
    p.forget("a")
    assert p.stats == {"lookups": 3, "hits": 2, "proposed": 4}


def test_engine_ngram_rounds_are_lossless_on_a_deterministic_model():
    """A fake target whose next token is a function of the previous one: rounds verified against it must emit exactly
    the plain greedy sequence, in fewer steps once the sequence starts repeating."""
    import numpy as np
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig

    def nxt(t):
        return (t * 5 + 3) % 11                              # a short cycle: the n-gram index soon predicts it

    class FakeNgram:
        speculative_depth = 4
        draft_source = "ngram"
        vocab_size = 64

        def __init__(self):
            self.rounds, self.accepted, self.plain = 0, 0, 0

        def copy_pages(self, pairs):
            pass

        def execute(self, segs):
            self.plain += 1
            return np.asarray([nxt(int(s.token_ids[-1])) for s in segs if s.sample], dtype=np.int32)

        def execute_speculative(self, segs, depths=None, drafts=None):
            self.rounds += 1
            out = []
            for s, d in zip(segs, drafts):
                assert len(d) <= self.speculative_depth
                cur, emitted = int(s.token_ids[0]), []
                for tok in d:
                    want = nxt(cur)
                    if tok != want:
                        break
                    emitted.append(want)
                    cur = want
                self.accepted += len(emitted)
                emitted.append(nxt(cur))                      # bonus token
                out.append(emitted)
            return out

    def run(executor):
        eng = LLMEngine(executor, num_pages=64, scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=256,
                                                                                  enable_prefix_cache=False))
        out = eng.generate([[1, 2, 3], [4, 9]], SamplingParams(max_tokens=40, ignore_eos=True))
        return out, eng

    class Plain(FakeNgram):
        speculative_depth = 0

    want, plain_eng = run(Plain())
    ex = FakeNgram()
    got, eng = run(ex)
    assert got == want and all(len(o) == 40 for o in got)
    assert ex.accepted > 40 and eng.steps < plain_eng.steps // 2      # most tokens came from accepted drafts
    assert eng.ngram.stats["hits"] > 0 and not eng.ngram._index       # indices are dropped with their requests
    # a sampled (temperature > 0) request takes the plain path
    ex2 = FakeNgram()
    eng2 = LLMEngine(ex2, num_pages=64, scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=256,
                                                                         enable_prefix_cache=False))
    eng2.generate([[1, 2, 3]], SamplingParams(max_tokens=8, ignore_eos=True, temperature=0.8, seed=1))
    assert ex2.rounds == 0 and ex2.plain > 0
