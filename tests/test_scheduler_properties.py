"""Property tests of the scheduler / page pool / prefix cache under random arrivals, aborts and tight memory."""
import numpy as np
from hypothesis import HealthCheck, given, settings, strategies as st

from cubic_serve_b200.runtime.engine import LLMEngine
from cubic_serve_b200.runtime.scheduler import AdmissionError, SamplingParams, SchedulerConfig


class CountingExecutor:
    """Deterministic fake: the next token is a function of the request's last input token and position."""
    vocab_size = 97

    def __init__(self):
        self.steps = 0

    def copy_pages(self, pairs):
        for src, dst in pairs:
            assert src != dst

    def execute(self, segs):
        self.steps += 1
        return np.asarray([(int(s.token_ids[-1]) * 31 + s.start + len(s.token_ids)) % 97 for s in segs if s.sample], dtype=np.int32)


events = st.lists(st.one_of(
    st.tuples(st.just("add"), st.integers(1, 70), st.integers(1, 12), st.integers(0, 3)),     # prompt len, max_tokens, family
    st.tuples(st.just("step"), st.integers(1, 4)),
    st.tuples(st.just("abort"), st.integers(0, 30))), min_size=1, max_size=40)


@settings(max_examples=150, deadline=None, derandomize=True, database=None, suppress_health_check=[HealthCheck.too_slow])
@given(events=events, pages=st.integers(12, 48), prefix=st.booleans(), rows=st.integers(1, 6))
def test_pages_are_never_leaked_and_outputs_do_not_depend_on_scheduling(events, pages, prefix, rows):
    ex = CountingExecutor()
    eng = LLMEngine(ex, num_pages=pages, scheduler_config=SchedulerConfig(
        max_running_requests=rows, max_model_len=96, max_batched_tokens=64, prefill_chunk_tokens=32,
        enable_prefix_cache=prefix))
    added, aborted, outputs = {}, set(), {}
    n = 0
    for ev in events:
        if ev[0] == "add":
            _, plen, max_tokens, fam = ev
            # families share long prefixes, so the prefix cache and copy-on-write get exercised
            prompt = [(fam * 7 + i) % 97 for i in range(min(plen, 40))] + [(n * 13 + i) % 97 for i in range(max(0, plen - 40))]
            if plen + max_tokens > 96:
                continue
            try:
                rid = eng.add_request(prompt, SamplingParams(max_tokens=max_tokens, ignore_eos=True), f"r{n}")
            except AdmissionError:                       # the waiting queue is bounded: a refused request leaves no trace
                n += 1
                continue
            added[rid] = (prompt, max_tokens)
            n += 1
        elif ev[0] == "abort":
            rid = f"r{ev[1]}"
            if rid in added and rid not in aborted and rid in eng.requests:
                eng.abort(rid)
                aborted.add(rid)
        else:
            for _ in range(ev[1]):
                if eng.has_unfinished:
                    for o in eng.step():
                        outputs.setdefault(o.request_id, []).append(o.token_id)
        assert 0 <= eng.pool.num_used <= pages
    for _ in range(2000):
        if not eng.has_unfinished:
            break
        for o in eng.step():
            outputs.setdefault(o.request_id, []).append(o.token_id)
    assert not eng.has_unfinished and not eng.poisoned
    # only prefix-cache entries keep pages once every request has ended
    assert eng.pool.num_used == (len(eng.prefix) if prefix else 0)
    # every request that was not aborted produced exactly its tokens, the ones the same request produces alone
    for rid, (prompt, max_tokens) in added.items():
        if rid in aborted:
            continue
        want, last, pos = [], prompt[-1], len(prompt)
        for _ in range(max_tokens):
            last = (last * 31 + pos) % 97
            want.append(last)
            pos += 1
        assert outputs.get(rid) == want, (rid, outputs.get(rid), want)


def test_preemption_under_tight_memory_recomputes_the_same_tokens():
    """Six requests that cannot all hold their pages at once: the newest are preempted and resumed; everybody still
    gets the tokens it would get alone, and the preemptions really happened."""
    ex = CountingExecutor()
    eng = LLMEngine(ex, num_pages=14, scheduler_config=SchedulerConfig(
        max_running_requests=6, max_model_len=96, max_batched_tokens=96, prefill_chunk_tokens=48, enable_prefix_cache=False))
    prompts = [[(7 * r + i) % 97 for i in range(30 + r)] for r in range(6)]
    reqs = []
    for i, p in enumerate(prompts):
        rid = eng.add_request(p, SamplingParams(max_tokens=30, ignore_eos=True), f"p{i}")
        reqs.append(eng.requests[rid])
    out = {}
    for _ in range(3000):
        if not eng.has_unfinished:
            break
        for o in eng.step():
            out.setdefault(o.request_id, []).append(o.token_id)
    assert not eng.has_unfinished and eng.pool.num_used == 0
    assert sum(r.preemptions for r in reqs) > 0
    for i, p in enumerate(prompts):
        want, last, pos = [], p[-1], len(p)
        for _ in range(30):
            last = (last * 31 + pos) % 97
            want.append(last)
            pos += 1
        assert out[f"p{i}"] == want


def test_a_lone_request_that_outgrows_the_pool_ends_with_length_instead_of_waiting_forever():
    """A 4-page pool, a 20-token prompt, 200 requested tokens: the request can never hold its last position.  It is
    cut to what the pool can hold and ends with finish reason LENGTH; the engine does not spin."""
    from cubic_serve_b200.runtime.scheduler import FinishReason
    eng = LLMEngine(CountingExecutor(), num_pages=4, scheduler_config=SchedulerConfig(
        max_running_requests=2, max_model_len=4096, max_batched_tokens=64, enable_prefix_cache=False))
    rid = eng.add_request(list(range(20)), SamplingParams(max_tokens=200, ignore_eos=True), "lone")
    req = eng.requests[rid]
    outs = []
    for _ in range(400):
        if not eng.has_unfinished:
            break
        outs += eng.step()
    assert not eng.has_unfinished and eng.pool.num_used == 0
    assert outs[-1].finished and outs[-1].finish_reason is FinishReason.LENGTH
    assert 0 < len(req.output) <= (4 - eng.pool.reserved) * 16 - 20


def test_scheduler_ends_a_running_request_that_cannot_grow_even_alone():
    """The safety net behind the admission cap: pages taken away from under a lone request (here: by shrinking the
    free list by hand) must end it with LENGTH and a token-less finish event, not leave it RUNNING forever."""
    from cubic_serve_b200.runtime.scheduler import FinishReason
    eng = LLMEngine(CountingExecutor(), num_pages=8, scheduler_config=SchedulerConfig(
        max_running_requests=2, max_model_len=4096, max_batched_tokens=64, enable_prefix_cache=False))
    eng.add_request(list(range(20)), SamplingParams(max_tokens=60, ignore_eos=True), "r")
    eng.step()
    stolen = eng.pool.alloc(eng.pool.num_free)          # somebody else holds every free page from now on
    outs = []
    for _ in range(100):
        if not eng.has_unfinished:
            break
        outs += eng.step()
    assert not eng.has_unfinished
    assert outs[-1].finished and outs[-1].token_id is None and outs[-1].finish_reason is FinishReason.LENGTH
    eng.pool.release(stolen)
    assert eng.pool.num_used == 0


def test_requests_that_do_not_fit_together_do_not_preempt_each_other_in_turn():
    """Three requests whose contexts cannot be resident together: the older ones are never preempted by a newer one,
    and nobody is preempted more than a couple of times (each preemption is a full recompute)."""
    ex = CountingExecutor()
    eng = LLMEngine(ex, num_pages=9, scheduler_config=SchedulerConfig(
        max_running_requests=3, max_model_len=128, max_batched_tokens=128, prefill_chunk_tokens=64, enable_prefix_cache=False))
    reqs = []
    for i in range(3):
        rid = eng.add_request([(5 * i + j) % 97 for j in range(40)], SamplingParams(max_tokens=40, ignore_eos=True), f"q{i}")
        reqs.append(eng.requests[rid])
    out = {}
    for _ in range(3000):
        if not eng.has_unfinished:
            break
        for o in eng.step():
            out.setdefault(o.request_id, []).append(o.token_id)
    assert not eng.has_unfinished and eng.pool.num_used == 0
    assert reqs[0].preemptions == 0
    assert all(r.preemptions <= 2 for r in reqs), [r.preemptions for r in reqs]
    assert all(len(out[f"q{i}"]) == 40 for i in range(3))
