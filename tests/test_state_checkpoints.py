"""Prefix caching for models with recurrent layers: a cached prefix is resumed from a snapshot of the recurrent state
taken at its last page boundary (the reference keeps such state snapshots beside its cached pages,
``runtime/performance.py:11018-11152`` there).  The executor double carries a rolling per-row state, so a missing or
wrong restore changes the tokens."""
import numpy as np

from cubic_serve_b200.runtime.cache.pool import PagePool
from cubic_serve_b200.runtime.cache.prefix import PrefixCache
from cubic_serve_b200.runtime.engine import LLMEngine
from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig


class RecurrentExecutor:
    """state[row] folds every token the row has consumed since position 0; the sampled id depends on it."""

    def __init__(self, rows=4, snapshots=4):
        self.state = np.zeros(rows + snapshots, dtype=np.int64)
        self.state_checkpoint_rows = tuple(range(rows, rows + snapshots))
        self.state_copies = []
        self.computed = 0

    def copy_state(self, pairs):
        for s, d in pairs:
            self.state[d] = self.state[s]
        self.state_copies.extend(pairs)

    def copy_pages(self, pairs):
        pass

    def execute(self, segs):
        out = []
        for s in segs:
            st = 0 if s.start == 0 else int(self.state[s.request_slot])
            for t in s.token_ids:
                st = (st * 31 + int(t) + 1) % 1_000_003
            self.state[s.request_slot] = st
            self.computed += len(s.token_ids)
            if s.sample:
                out.append(st % 89)
        return np.asarray(out, dtype=np.int32)


def _engine(ex, pages=64, **kw):
    cfg = SchedulerConfig(max_running_requests=4, max_batched_tokens=64, prefill_chunk_tokens=32, max_model_len=256, **kw)
    return LLMEngine(ex, num_pages=pages, scheduler_config=cfg)


def _tokens(eng, prompt, n):
    return [int(t) for t in eng.generate([prompt], SamplingParams(max_tokens=n))[0]]


def test_a_cached_prefix_of_a_recurrent_model_resumes_from_its_snapshot():
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, 1000, size=70)]
    cold = _tokens(_engine(RecurrentExecutor(), enable_prefix_cache=False), prompt, 6)

    ex = RecurrentExecutor()
    eng = _engine(ex)
    assert eng.prefix.enabled and eng.prefix.needs_checkpoint          # kept on because the executor has snapshot rows
    first = _tokens(eng, prompt, 6)
    assert first == cold
    saved = [d for _, d in ex.state_copies]
    assert saved and all(d in ex.state_checkpoint_rows for d in saved)
    before = ex.computed
    again = _tokens(eng, prompt, 6)
    assert again == cold
    # the second run computed only the tail after the last checkpointed boundary: 70 -> 64 cached
    assert ex.computed - before == (70 - 64) + 5
    restores = [p for p in ex.state_copies if p[0] in ex.state_checkpoint_rows]
    assert len(restores) == 1
    # a different continuation of the same 64-token prefix resumes there too
    other = prompt[:64] + [5, 6, 7]
    ref = _tokens(_engine(RecurrentExecutor(), enable_prefix_cache=False), other, 3)
    assert _tokens(eng, other, 3) == ref


def test_without_snapshot_rows_the_prefix_cache_of_a_recurrent_model_is_off():
    class NoRows(RecurrentExecutor):
        state_checkpoint_rows = ()

    class Hybrid:
        is_hybrid = True
    ex = NoRows()
    ex.state_checkpoint_rows = ()
    ex.cfg = Hybrid()
    eng = _engine(ex)
    assert not eng.prefix.needs_checkpoint


def test_match_stops_at_the_last_boundary_with_a_snapshot_and_slots_are_recycled():
    pool = PagePool(32)
    pc = PrefixCache(pool, checkpoint_slots=(100, 101))
    toks = list(range(64))
    pages = pool.alloc(4)
    pc.publish(toks, pages)
    assert pc.match(toks + [1]) == []                       # pages cached, no snapshot anywhere: nothing resumable
    s2 = pc.publish_checkpoint(toks[:32])
    assert s2 in (100, 101) and pc.publish_checkpoint(toks[:32]) is None
    got = pc.match(toks + [1])
    assert got == pages[:2] and pc.last_checkpoint == s2
    pool.release(got)
    s4 = pc.publish_checkpoint(toks)
    assert s4 is not None and s4 != s2
    got = pc.match(toks + [1])
    assert got == pages and pc.last_checkpoint == s4
    pool.release(got)
    # both slots taken: a third boundary evicts the least recently used snapshot nobody else holds
    pool.release(pages)                                     # the requests that wrote the pages are gone
    other = list(range(500, 532))
    op = pool.alloc(2)
    pc.publish(other, op)
    s = pc.publish_checkpoint(other)
    assert s in (s2, s4)
    # evicting pages frees their snapshot slots
    pool.release(op)
    pc.evict(100)
    assert len(pc) == 0 and sorted(pc._free_ckpt) == [100, 101]
    assert pool.num_used == 0


def test_a_preempted_request_of_a_recurrent_model_recomputes_the_same_tokens():
    rng = np.random.default_rng(3)
    prompts = [[int(t) for t in rng.integers(0, 1000, size=40)] for _ in range(3)]
    ref = [_tokens(_engine(RecurrentExecutor(), enable_prefix_cache=False), p, 40) for p in prompts]
    ex = RecurrentExecutor()
    eng = _engine(ex, pages=13)                              # 3 x (80 tokens = 5 pages) do not fit together
    outs = eng.generate(prompts, SamplingParams(max_tokens=40))
    assert [[int(t) for t in o] for o in outs] == ref
