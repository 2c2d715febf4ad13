"""Page pool, prefix cache, scheduler and engine on CPU (eager executor / fake executor)."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
from cubic_serve_b200.models.config import toy_config
from cubic_serve_b200.models.reference import EagerDecoder, random_dense_weights
from cubic_serve_b200.runtime.cache.pool import OutOfPages, PagePool, PoolPoisoned
from cubic_serve_b200.runtime.cache.prefix import PrefixCache, block_digests
from cubic_serve_b200.runtime.engine import LLMEngine
from cubic_serve_b200.runtime.scheduler import (AdmissionError, ContinuousScheduler, FinishReason, Request,
                                                SamplingParams, SchedulerConfig)


def test_pool_refcount_and_cow():
    pool = PagePool(8)
    a = pool.alloc(3)
    assert a == [1, 2, 3] and pool.num_free == 4
    pool.retain(a[:1])
    assert not pool.writable(a[0]) and pool.writable(a[1])
    new, copy = pool.cow(a[0])
    assert copy and new == 4 and pool.refcount(a[0]) == 1
    same, copy2 = pool.cow(a[1])
    assert same == a[1] and not copy2
    pool.release([a[0], a[1], a[2], new])
    assert pool.num_free == 7
    with pytest.raises(OutOfPages):
        pool.alloc(8)
    with pytest.raises(PoolPoisoned):
        pool.release([5])
    with pytest.raises(PoolPoisoned):
        pool.alloc(1)


def test_prefix_digest_chain_and_lru():
    toks = list(range(40))
    d = block_digests(toks)
    assert len(d) == 2 and d[0] != d[1]
    assert block_digests(toks[:32]) == d
    assert block_digests([1] + toks[1:])[1] != d[1]          # chained: a change in block 0 changes block 1
    pool = PagePool(6)
    cache = PrefixCache(pool)
    pages = pool.alloc(2)
    assert cache.publish(toks[:32], pages) == 2
    pool.release(pages)                                       # cache is now the only owner
    got = cache.match(toks, max_tokens=39)
    assert got == pages and pool.refcount(pages[0]) == 2
    pool.release(got)
    assert cache.match(toks[:20] + [99] * 20) == pages[:1]
    pool.release(pages[:1])
    assert cache.evict(5) == 2 and pool.num_free == 5 and len(cache) == 0


class FakeExecutor:
    """Next token = (last token + 1) % 100; records every segment it saw."""
    def __init__(self):
        self.calls = []
        self.copies = []
    def copy_pages(self, pairs):
        self.copies.extend(pairs)
    def execute(self, segs):
        self.calls.append([(s.request_slot, s.start, len(s.token_ids), s.sample) for s in segs])
        return np.asarray([(int(s.token_ids[-1]) + 1) % 100 for s in segs if s.sample], dtype=np.int32)


def test_engine_continuous_batching_chunked_prefill():
    ex = FakeExecutor()
    eng = LLMEngine(ex, num_pages=64, scheduler_config=SchedulerConfig(max_running_requests=4, max_batched_tokens=48,
                                                                       prefill_chunk_tokens=32, max_model_len=256))
    a = eng.add_request(list(range(50)), SamplingParams(max_tokens=3))
    b = eng.add_request([7] * 5, SamplingParams(max_tokens=2))
    outs = []
    while eng.has_unfinished:
        outs.extend(eng.step())
    toks = {rid: [o.token_id for o in outs if o.request_id == rid] for rid in (a, b)}
    assert toks[a] == [50, 51, 52] and toks[b] == [8, 9]
    assert [o.finish_reason for o in outs if o.finished] == [FinishReason.LENGTH] * 2
    # first step: a gets a page-aligned chunk, b fits entirely; nothing sampled for a yet
    first = ex.calls[0]
    assert any(cnt == 16 and not smp for (_, st, cnt, smp) in first)   # fair share 24, cut to a page boundary
    assert any(cnt == 5 and smp for (_, st, cnt, smp) in first)
    assert eng.pool.num_used == len(eng.prefix)          # only prefix-cache entries keep pages
    assert sum(c for call in ex.calls for (_, _, c, _) in call) == 50 + 5 + 2 + 1


def test_prefix_reuse_and_cow_between_requests():
    ex = FakeExecutor()
    eng = LLMEngine(ex, num_pages=32, scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=128))
    shared = list(range(40))
    eng.generate([shared + [1, 2]], SamplingParams(max_tokens=1))
    assert len(eng.prefix) == 2
    ex.calls.clear()
    eng.generate([shared + [3]], SamplingParams(max_tokens=2))
    # the second request starts computing at token 32 (two cached blocks)
    assert ex.calls[0][0][1] == 32 and ex.calls[0][0][2] == 9
    assert eng.prefix.hit_tokens == 32


def test_stop_token_and_abort_and_admission():
    ex = FakeExecutor()
    eng = LLMEngine(ex, num_pages=16, scheduler_config=SchedulerConfig(max_running_requests=2, max_model_len=64),
                    eos_token_id=12)
    out = eng.generate([[10]], SamplingParams(max_tokens=10))
    assert out == [[11, 12]]
    rid = eng.add_request([1, 2, 3], SamplingParams(max_tokens=50))
    eng.step()
    assert eng.abort(rid) and not eng.has_unfinished and eng.pool.num_used == 0
    with pytest.raises(AdmissionError):
        eng.add_request(list(range(100)))
    with pytest.raises(ValueError):
        eng.add_request([1], SamplingParams(top_k=21))


def test_preemption_when_pool_runs_dry():
    ex = FakeExecutor()
    cfg = SchedulerConfig(max_running_requests=4, max_model_len=200, enable_prefix_cache=False)
    eng = LLMEngine(ex, num_pages=9, scheduler_config=cfg)          # 8 usable pages = 128 tokens
    ids = [eng.add_request([i] * 40, SamplingParams(max_tokens=40)) for i in range(3)]
    reqs = [eng.requests[i] for i in ids]
    while eng.has_unfinished:
        eng.step()
    assert all(len(r.output) == 40 for r in reqs)
    assert sum(r.preemptions for r in reqs) >= 1
    assert eng.pool.num_used == 0


@pytest.mark.parametrize("scaling", [None, ("yarn", 4.0, 16, 32.0, 1.0, 1.25), ("llama3", 8.0, 1.0, 4.0, 16)])
def test_engine_eager_executor_matches_reference_decoder(scaling):
    cfg = replace(toy_config(), rope_scaling=scaling)
    w = random_dense_weights(cfg, seed=0)
    prompts = torch.randint(0, cfg.vocab_size, (3, 21), generator=torch.Generator().manual_seed(1))
    ref, _ = EagerDecoder(cfg, w).generate(prompts, 6)
    eng = LLMEngine(EagerPagedExecutor(cfg, w, num_pages=32), num_pages=32,
                    scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=64,
                                                     prefill_chunk_tokens=16, max_batched_tokens=40))
    out = eng.generate([p.tolist() for p in prompts], SamplingParams(max_tokens=6))
    assert out == ref.tolist()
    # cold vs prefix-resumed: same continuation
    out2 = eng.generate([prompts[0].tolist()], SamplingParams(max_tokens=6))
    assert out2[0] == ref[0].tolist() and eng.prefix.hit_tokens >= 16


def test_choice_constraint_masks_sampling_end_to_end():
    """A ``choice`` matcher forces the engine's output to be exactly one of the options, then EOS."""
    from cubic_serve_b200.generation.constraints import ChoiceMatcher

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [ord(c) for c in text]

    cfg = toy_config()
    w = random_dense_weights(cfg, seed=0)
    eng = LLMEngine(EagerPagedExecutor(cfg, w, num_pages=32), num_pages=32,
                    scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=64))
    eos = 3
    options = ["yes", "no", "maybe"]
    outs = []
    for seed in range(3):
        m = ChoiceMatcher(options, Tok(), eos)
        sp = SamplingParams(temperature=1.0, top_k=20, seed=seed, max_tokens=12, stop_token_ids=(eos,), matcher=m)
        free = SamplingParams(max_tokens=5)
        rid = eng.add_request([5, 6, 7, 8 + seed], sp)
        other = eng.add_request([9, 10, 11], free)               # an unconstrained request shares the steps
        reqs = {rid: eng.requests[rid], other: eng.requests[other]}
        while eng.has_unfinished:
            eng.step()
        toks = reqs[rid].output
        assert toks[-1] == eos
        text = "".join(chr(t) for t in toks[:-1])
        assert text in options
        assert len(reqs[other].output) == 5
        outs.append(text)
    assert eng._mask_words == cfg.vocab_size // 32


class _FeedbackExecutor:
    """Executor double with the launch / collect interface: the sampled id is a function of the row's input token
    and position, and a look-ahead launch reads its input tokens from the previous launch's ids ("device" memory)."""

    def __init__(self, vocab=97, eos=None):
        self.vocab, self.eos = vocab, eos
        self.dev_ids = np.zeros(0, dtype=np.int64)
        self.launches = self.feedback_launches = 0
        self.outstanding = 0

    def launch(self, segs, feedback_rows=0):
        assert self.outstanding < 2
        self.outstanding += 1
        self.launches += 1
        self.feedback_launches += bool(feedback_rows)
        out = []
        for i, s in enumerate(segs):
            tok = int(self.dev_ids[i]) if i < feedback_rows else int(s.token_ids[-1])
            if s.sample:
                out.append((tok * 7 + (s.start + len(s.token_ids) - 1) * 3 + 1) % self.vocab)
        self.dev_ids = np.asarray(out, dtype=np.int64)
        return {"ids": self.dev_ids.copy()}

    def collect(self, handle):
        self.outstanding -= 1
        return handle["ids"]

    def execute(self, segs):
        return self.collect(self.launch(segs))

    def copy_pages(self, pairs):
        pass


def _run_engine(overlap, eos, arrivals):
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    ex = _FeedbackExecutor(eos=eos)
    eng = LLMEngine(ex, num_pages=256, scheduler_config=SchedulerConfig(max_running_requests=8, max_batched_tokens=64,
                                                                         prefill_chunk_tokens=64, max_model_len=128,
                                                                         enable_prefix_cache=False), eos_token_id=eos)
    eng.overlap_decode = overlap
    rng = np.random.default_rng(3)
    reqs, step = {}, 0
    pending = sorted(arrivals)
    while pending or eng.has_unfinished or eng._ahead is not None:
        while pending and pending[0][0] <= step:
            _, n_prompt, max_tokens = pending.pop(0)
            rid = eng.add_request(rng.integers(1, 90, n_prompt).tolist(), SamplingParams(max_tokens=max_tokens))
            reqs[rid] = eng.requests[rid]
        eng.step()
        step += 1
        assert step < 500
    assert eng.pool.num_used == 0
    return [r.output for r in reqs.values()], ex


def test_overlapped_decode_steps_give_the_same_tokens():
    """Look-ahead launches (next decode step enqueued before this step's ids are read, input tokens fed back on the
    "device") must not change any request's tokens: stop tokens ending a request while its look-ahead row is in
    flight, length limits, and requests arriving in the middle of a decode phase."""
    arrivals = [(0, 5, 30), (0, 9, 17), (0, 3, 40), (12, 7, 25), (13, 4, 6), (40, 11, 33)]
    base, _ = _run_engine(False, None, arrivals)
    # stop tokens that do occur in the middle of some request's output
    for eos in (None, base[2][10], base[0][4], base[5][20]):
        plain, ex0 = _run_engine(False, eos, arrivals)
        fast, ex1 = _run_engine(True, eos, arrivals)
        assert fast == plain
        assert ex0.feedback_launches == 0 and ex1.feedback_launches > 10
        if eos is not None:
            assert any(o and o[-1] == eos and len(o) < m for o, (_, _, m) in zip(plain, arrivals))   # a request was stopped


def test_grammar_engine_constraints_end_to_end():
    """xgrammar-backed constraints (regex, JSON schema) through the adapter: masks reach the sampler, the output
    matches, the matcher can roll back (speculative rounds); the byte tokenizer is described as a raw vocabulary."""
    pytest = __import__("pytest")
    pytest.importorskip("xgrammar")
    import json
    import re
    from cubic_serve_b200.contracts.request import StructuredKind, StructuredOutput
    from cubic_serve_b200.generation.constraints import GrammarTransaction, compile_matcher
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    tok = ByteTokenizer()
    cfg = toy_config()
    w = random_dense_weights(cfg, seed=0)
    eng = LLMEngine(EagerPagedExecutor(cfg, w, num_pages=64), num_pages=64,
                    scheduler_config=SchedulerConfig(max_running_requests=4, max_model_len=128))
    eos = tok.eos_token_id
    pattern = r"(yes|no)-[0-9]{3}"
    for seed in range(2):
        m = compile_matcher(StructuredOutput(StructuredKind.REGEX, pattern), tok, eos, cfg.vocab_size)
        rid = eng.add_request([5, 6, 7, 8 + seed], SamplingParams(temperature=1.0, top_k=20, seed=seed, max_tokens=16,
                                                                  stop_token_ids=(eos,), matcher=m))
        req = eng.requests[rid]
        while eng.has_unfinished:
            eng.step()
        assert req.output[-1] == eos and re.fullmatch(pattern, tok.decode(req.output[:-1]))
        assert m.finished
    # JSON schema by a random walk inside the masks, with a rejected speculative tail rolled back on the way
    schema = {"type": "object", "properties": {"n": {"type": "integer"}, "ok": {"type": "boolean"}}, "required": ["n", "ok"],
              "additionalProperties": False}
    m = compile_matcher(StructuredOutput(StructuredKind.JSON_SCHEMA, schema), tok, eos, cfg.vocab_size)
    rng = np.random.default_rng(0)
    out: list[int] = []
    for step in range(400):
        bm = np.zeros(cfg.vocab_size // 32, dtype=np.uint32)
        m.fill_bitmask(bm)
        allowed = [i for i in range(cfg.vocab_size) if bm[i // 32] >> (i % 32) & 1 and chr(i % 256) not in " \n\t\r"]
        t = int(rng.choice(allowed))
        if step == 5:
            tr = GrammarTransaction(m)
            assert tr.try_accept(t)
            tr.commit(0)                    # the draft token is rejected after all: the matcher is back where it was
            bm2 = np.zeros_like(bm)
            m.fill_bitmask(bm2)
            assert np.array_equal(bm, bm2)
        assert m.accept(t)
        if t == eos:
            break
        out.append(t)
    doc = json.loads(tok.decode(out))
    assert isinstance(doc["n"], int) and isinstance(doc["ok"], bool) and set(doc) == {"n", "ok"}


def test_structural_tags_constrain_only_the_tagged_regions():
    pytest = __import__("pytest")
    pytest.importorskip("xgrammar")
    from cubic_serve_b200.contracts.request import StructuredKind, StructuredOutput
    from cubic_serve_b200.generation.constraints import compile_matcher
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    tok = ByteTokenizer()
    eos, vocab = tok.eos_token_id, 512

    def allowed(m):
        bm = np.zeros(vocab // 32, dtype=np.uint32)
        m.fill_bitmask(bm)
        return {i for i in range(vocab) if bm[i // 32] >> (i % 32) & 1}

    schema = {"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"], "additionalProperties": False}
    legacy = {"structures": [{"begin": "<tool=add>", "schema": schema, "end": "</tool>"}], "triggers": ["<tool="]}
    m = compile_matcher(StructuredOutput(StructuredKind.STRUCTURAL_TAG, legacy), tok, eos, vocab)
    assert {ord("x"), ord("<"), eos} <= allowed(m)                     # free text: anything goes, the answer may end
    for ch in b'ok <tool=add>{"a"':
        assert m.accept(ch)
    inside = allowed(m)
    assert ord(":") in inside and ord("x") not in inside and eos not in inside     # the schema rules inside the tag
    for ch in b': 12}</tool> done':
        assert ch in allowed(m) and m.accept(ch)
    assert eos in allowed(m)
    # a tag whose name no structure defines cannot be opened
    m2 = compile_matcher(StructuredOutput(StructuredKind.STRUCTURAL_TAG, legacy), tok, eos, vocab)
    for ch in b"<tool=":
        assert m2.accept(ch)
    assert allowed(m2) == {ord("a")}
    current = {"type": "structural_tag", "format": {"type": "triggered_tags", "triggers": ["<f>"], "tags": [
        {"begin": "<f>", "content": {"type": "json_schema", "json_schema": {"type": "integer"}}, "end": "</f>"}]}}
    m3 = compile_matcher(StructuredOutput(StructuredKind.STRUCTURAL_TAG, current), tok, eos, vocab)
    for ch in b"x<f>42</f>":
        assert m3.accept(ch)
    with pytest.raises(ValueError):
        compile_matcher(StructuredOutput(StructuredKind.STRUCTURAL_TAG, {"structures": [{"begin": "<a>", "end": "</a>"}],
                                                                         "triggers": ["<b"]}), tok, eos, vocab)


def test_delayed_constraint_starts_after_the_reasoning_block():
    from cubic_serve_b200.generation.constraints import ChoiceMatcher, DelayedMatcher, GrammarTransaction
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    tok = ByteTokenizer()
    eos = tok.eos_token_id
    end = list(b"</t>")
    m = DelayedMatcher(ChoiceMatcher(["yes", "no"], tok, eos), end)

    def allowed(m):
        bm = np.zeros(16, dtype=np.uint32)
        m.fill_bitmask(bm)
        return {i for i in range(512) if bm[i // 32] >> (i % 32) & 1}

    assert len(allowed(m)) == 512 and not m.finished
    for ch in b"hmm </t":
        assert m.accept(ch)
    assert len(allowed(m)) == 512                       # the closing sequence is not complete yet
    assert m.accept(ord(">")) and m.active
    assert allowed(m) == {ord("y"), ord("n")}
    # a speculative round that crosses the boundary and is rejected puts the matcher back into the thinking phase
    m.rollback(2)
    assert not m.active and len(allowed(m)) == 512
    tr = GrammarTransaction(m)
    for ch in b"t>ye":
        assert tr.try_accept(ch)
    tr.commit(3)                                        # keep "t>y", drop "e"
    assert m.active and allowed(m) == {ord("e")}
    assert not m.accept(ord("x"))
    for ch in b"es":
        assert m.accept(ch)
    assert allowed(m) == {eos} and m.accept(eos) and m.finished
    __import__("pytest").raises(ValueError, DelayedMatcher, None, [])


def test_prefix_cache_evicts_a_chain_from_its_leaf():
    """After a match or a publish the blocks of a chain are ordered leaf (oldest) to root (newest): eviction drops
    the leaf first and never strands later blocks behind a missing first block."""
    from cubic_serve_b200.runtime.cache.pool import PagePool
    from cubic_serve_b200.runtime.cache.prefix import PrefixCache
    pool = PagePool(16)
    cache = PrefixCache(pool)
    toks = list(range(64))
    pages = pool.alloc(4)
    cache.publish(toks, pages)
    pool.release(pages)                                  # only the cache holds them now
    assert cache.evictable() == 4
    assert cache.evict(1) == 1
    got = cache.match(toks)
    assert got == pages[:3]                              # the first three blocks are still reachable
    pool.release(got)
    assert cache.evict(2) == 2
    got = cache.match(toks)
    assert got == pages[:1]
    pool.release(got)
