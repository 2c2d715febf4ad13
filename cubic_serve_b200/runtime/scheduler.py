"""Continuous-batching scheduler over the shared page pool.

Same policy family as the reference controller (``runtime/performance.py:11154``
``_next_batch_locked``; plan-only version ``runtime/scheduler.py:216`` there):
decode-ready requests first, then prefill chunks inside a token budget with a
fair share per prefilling request, request order rotated for fairness, pages
reserved before a request enters a batch, prefix pages restored at admission and
published as pages fill, capacity exhaustion handled by evicting prefix entries
(LRU) and then preempting the newest request.
"""
from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass, field

from .cache.pool import OutOfPages, PagePool
from .cache.prefix import BLOCK, PrefixCache


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    ERROR = "error"


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int | None = None
    max_tokens: int = 256
    stop_token_ids: tuple[int, ...] = ()
    ignore_eos: bool = False
    # structured output: an object with ``fill_bitmask(uint32 words)`` and ``accept(token) -> bool``
    # (``generation/constraints.py``); the engine masks the sampler with it and advances it on every commit
    matcher: object | None = None
    # thinking-token budget of a request that starts inside a reasoning block: after this many tokens the executor
    # forces the end of the block (enforced on the device, see ``csrc/sampling.cu``); None = unlimited
    thinking_budget: int | None = None

    def validate(self) -> None:
        if not 0.0 <= self.temperature <= 2.0:
            raise ValueError("temperature must be in [0, 2]")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0 <= self.top_k <= 20:
            raise ValueError("top_k must be in [0, 20]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.thinking_budget is not None and self.thinking_budget < 0:
            raise ValueError("thinking_budget must be >= 0")


@dataclass
class Request:
    request_id: str
    prompt: list[int]
    sampling: SamplingParams
    arrival: int = 0
    status: RequestStatus = RequestStatus.WAITING
    output: list[int] = field(default_factory=list)
    pages: list[int] = field(default_factory=list)
    num_computed: int = 0          # tokens whose KV is in the cache
    num_published: int = 0         # leading pages already offered to the prefix cache
    num_cached_prefix: int = 0     # tokens restored from the prefix cache at admission
    finish_reason: FinishReason | None = None
    slot: int = -1                 # row of the executor's page table
    draws: int = 0                 # sampler draw counter
    preemptions: int = 0
    last_committed: int = 0        # tokens kept by the most recent commit (a stop can cut a speculative burst)
    tokens: list[int] = field(default_factory=list)   # prompt + output, maintained incrementally
    # multimodal prompt (``runtime/multimodal.py::MultimodalInput``): encoder feature rows that replace the embedding
    # of placeholder tokens, three-axis positions, and per-row content keys for the prefix cache
    multimodal: object | None = None

    def __post_init__(self) -> None:
        if not self.tokens:
            self.tokens = list(self.prompt) + list(self.output)

    def append_output(self, tok: int) -> None:
        self.output.append(tok)
        self.tokens.append(tok)

    @property
    def num_tokens(self) -> int:
        return len(self.tokens)

    @property
    def is_prefill(self) -> bool:
        return self.num_computed < self.num_tokens - 1 or not self.output and self.num_computed < len(self.prompt)

    @property
    def remaining(self) -> int:
        return self.num_tokens - self.num_computed


def _keys(req: Request, tokens: list[int]) -> list[int]:
    """What the prefix cache hashes for ``tokens`` (a prefix of the request's tokens): placeholder tokens of a media
    item are replaced by numbers derived from the item's content and the row, so two prompts share cached pages over
    a media span only when the media are the same."""
    return tokens if req.multimodal is None else req.multimodal.key_tokens(tokens)


@dataclass
class PlannedSegment:
    request: Request
    start: int
    count: int
    sample: bool


@dataclass
class BatchPlan:
    segments: list[PlannedSegment]
    copies: list[tuple[int, int]] = field(default_factory=list)   # (src page, dst page) copy-on-write
    preempted: list[Request] = field(default_factory=list)
    # requests the scheduler itself ended while planning: the pool cannot hold their next position even when
    # they run alone (finish reason LENGTH); the engine reports them without a token
    finished: list[Request] = field(default_factory=list)
    # recurrent-state row copies (src row, dst row) to run BEFORE the step (a resumed request gets the snapshot of its
    # cached prefix) -- models with recurrent layers only
    state_restores: list[tuple[int, int]] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.count for s in self.segments)

    @property
    def is_decode_only(self) -> bool:
        return all(s.count == 1 for s in self.segments)


@dataclass
class SchedulerConfig:
    max_running_requests: int = 256
    max_batched_tokens: int = 8192
    prefill_chunk_tokens: int = 4096
    max_model_len: int = 4096
    enable_prefix_cache: bool = True
    # rows of the executor's recurrent-state arrays reserved for prefix snapshots (models with recurrent layers: a
    # cached prefix is resumable only with the state at its end); () = the model has no recurrent state
    state_checkpoint_slots: tuple[int, ...] = ()


class AdmissionError(RuntimeError):
    """Request can never run (too long) or the server is at capacity (maps to 400 / 429)."""

    def __init__(self, message: str, status: int = 400) -> None:
        super().__init__(message)
        self.status = status


class ContinuousScheduler:
    def __init__(self, cfg: SchedulerConfig, pool: PagePool, prefix: PrefixCache | None = None) -> None:
        self.cfg = cfg
        self.pool = pool
        self.prefix = prefix if prefix is not None else PrefixCache(
            pool, enabled=cfg.enable_prefix_cache, checkpoint_slots=cfg.state_checkpoint_slots or None)
        self._pending_restores: list[tuple[int, int]] = []
        self.state_saves: list[tuple[int, int]] = []      # (request row, snapshot row) copies to run AFTER the last step
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self._clock = itertools.count()
        self._free_slots = list(range(cfg.max_running_requests - 1, -1, -1))
        self._rotate = 0
        self.decode_lookahead = 0      # extra positions reserved per decode row (speculative drafts)

    # ---------------------------------------------------------------- admission
    def add(self, req: Request) -> None:
        req.sampling.validate()
        if not req.prompt:
            raise AdmissionError("empty prompt")
        if len(req.prompt) + 1 > self.cfg.max_model_len:
            raise AdmissionError(f"prompt of {len(req.prompt)} tokens exceeds max_model_len {self.cfg.max_model_len}")
        need = -(-(len(req.prompt) + 1) // BLOCK)
        if need > self.pool.num_pages - self.pool.reserved:
            raise AdmissionError("prompt can never fit in the KV cache")
        req.arrival = next(self._clock)
        # a request alone in the pool must be able to reach its last position: cap the output length by what the
        # pool can ever hold (otherwise it would wait for pages that no eviction or preemption can free)
        pool_tokens = (self.pool.num_pages - self.pool.reserved) * BLOCK - self.decode_lookahead
        req.sampling.max_tokens = max(1, min(req.sampling.max_tokens, self.cfg.max_model_len - len(req.prompt),
                                             pool_tokens - len(req.prompt)))
        self.waiting.append(req)

    def abort(self, request_id: str) -> Request | None:
        for q in (self.waiting, self.running):
            for r in q:
                if r.request_id == request_id:
                    q.remove(r)
                    self._finish(r, FinishReason.ABORT, RequestStatus.ABORTED)
                    return r
        return None

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ pages
    def _reserve(self, n: int) -> list[int]:
        if n > self.pool.num_free:
            self.prefix.evict(n - self.pool.num_free)
        return self.pool.alloc(n)

    def _ensure_pages(self, req: Request, upto_tokens: int, copies: list) -> None:
        """Make pages cover ``upto_tokens`` and make the page being appended to privately owned."""
        first_new_page = req.num_computed // BLOCK
        if first_new_page < len(req.pages) and req.num_computed % BLOCK:
            page = req.pages[first_new_page]
            if not self.pool.writable(page):
                if self.pool.num_free == 0:
                    self.prefix.evict(1)
                new, copy = self.pool.cow(page)
                if copy:
                    copies.append((page, new))
                req.pages[first_new_page] = new
        need = -(-upto_tokens // BLOCK) - len(req.pages)
        if need > 0:
            req.pages.extend(self._reserve(need))

    def _admit(self, req: Request) -> bool:
        if not self._free_slots:
            return False
        # restore the longest cached prefix, always leaving >= 1 prompt token to compute
        pages = self.prefix.match(_keys(req, req.prompt), max_tokens=len(req.prompt) - 1) if not req.pages else []
        if pages:
            req.pages = list(pages)
            req.num_computed = len(pages) * BLOCK
            req.num_cached_prefix = req.num_computed
            req.num_published = len(pages)
        if self.running:
            # beside running requests, admit only what can hold its whole current context: a request that was
            # preempted for lack of pages would otherwise come straight back, prefill and be preempted again
            need = -(-(req.num_tokens + 1) // BLOCK) - len(req.pages)
            if need > self.pool.num_free + self.prefix.evictable():
                if pages:
                    self.pool.release(pages)
                    req.pages = []
                    req.num_computed = req.num_cached_prefix = req.num_published = 0
                return False
        req.slot = self._free_slots.pop()
        req.status = RequestStatus.RUNNING
        self.running.append(req)
        if pages and self.prefix.needs_checkpoint:
            self._pending_restores.append((self.prefix.last_checkpoint, req.slot))
        return True

    def _preempt_newest(self, keep: Request | None) -> Request | None:
        """Preempt the newest running request that arrived AFTER ``keep`` (any request if ``keep`` is None).  A
        request never takes pages from an older one: two requests that do not fit together would otherwise preempt
        each other in turn, each time recomputing a whole context for one token of progress."""
        victims = [r for r in self.running if r is not keep and (keep is None or r.arrival > keep.arrival)]
        if not victims:
            return None
        return self._preempt(max(victims, key=lambda r: r.arrival))

    def _preempt(self, v: Request) -> Request:
        self.running.remove(v)
        self.pool.release(v.pages)
        v.pages = []
        v.num_computed = v.num_published = v.num_cached_prefix = 0
        self._free_slots.append(v.slot)
        v.slot = -1
        v.status = RequestStatus.WAITING
        v.preemptions += 1
        self.waiting.insert(0, v)
        return v

    # ------------------------------------------------------------------- plan
    def next_plan(self) -> BatchPlan | None:
        cfg = self.cfg
        while self.waiting and len(self.running) < cfg.max_running_requests:
            if not self._admit(self.waiting[0]):
                break
            self.waiting.pop(0)
        if not self.running:
            return None
        plan = BatchPlan([])
        plan.state_restores, self._pending_restores = self._pending_restores, []
        budget = cfg.max_batched_tokens
        order = self.running[self._rotate % len(self.running):] + self.running[:self._rotate % len(self.running)]
        self._rotate += 1
        decodes = [r for r in order if r.remaining == 1]
        prefills = [r for r in order if r.remaining > 1]
        scheduled: set[str] = set()
        for r in decodes:
            if budget <= 0:
                break
            if not self._try_segment(r, 1, plan, scheduled):
                continue
            budget -= 1
        if prefills and budget > 0:
            share = max(BLOCK, budget // len(prefills))
            for r in prefills:
                if budget <= 0:
                    break
                if r.status is not RequestStatus.RUNNING:
                    continue
                n = min(r.remaining, share, cfg.prefill_chunk_tokens, budget)
                if self.prefix.needs_checkpoint and self.prefix.enabled and not r.output:
                    # a chunk ends exactly at the last page boundary of the prompt: the recurrent state after it is the
                    # snapshot that makes the prompt's pages resumable
                    ck = (len(r.prompt) - 1) // BLOCK * BLOCK
                    if r.num_computed < ck < r.num_computed + n:
                        n = ck - r.num_computed
                if n < r.remaining:
                    n = max(BLOCK, n - (r.num_computed + n) % BLOCK) if n >= BLOCK else n  # end chunks on page boundaries
                    n = min(n, r.remaining, budget)
                if n <= 0:
                    continue
                if self._try_segment(r, n, plan, scheduled):
                    budget -= n
        plan.segments = [s for s in plan.segments if s.request.status is RequestStatus.RUNNING and s.request.slot >= 0]
        return plan if plan.segments or plan.preempted or plan.finished else None

    def _try_segment(self, r: Request, n: int, plan: BatchPlan, scheduled: set) -> bool:
        if r.status is not RequestStatus.RUNNING:
            return False
        reserve = n + (self.decode_lookahead if n == 1 and r.remaining == 1 else 0)
        while True:
            try:
                self._ensure_pages(r, min(r.num_computed + reserve, self.cfg.max_model_len + self.decode_lookahead),
                                   plan.copies)
                break
            except OutOfPages:
                victim = self._preempt_newest(keep=r)
                if victim is None:
                    if len(self.running) > 1:
                        # r is the newest: it gives way itself and waits until older requests have finished
                        plan.preempted.append(self._preempt(r))
                    else:
                        # alone and still out of pages: nothing can ever free any, so the request ends here
                        self._retire(r, FinishReason.LENGTH)
                        plan.finished.append(r)
                    return False
                plan.preempted.append(victim)
                plan.segments = [s for s in plan.segments if s.request is not victim]
                scheduled.discard(victim.request_id)
        sample = r.num_computed + n == r.num_tokens
        plan.segments.append(PlannedSegment(r, r.num_computed, n, sample))
        scheduled.add(r.request_id)
        return True

    def lookahead_plan(self, prev: BatchPlan) -> BatchPlan | None:
        """The decode step that follows ``prev`` if ``prev`` finishes nobody, planned BEFORE ``prev`` is committed.

        Only for the steady state: ``prev`` is one sampled decode row for every running request, nothing waits, no
        request can reach its length limit in ``prev``, none is constrained by a matcher, and the pages of the next
        position can be had without evicting or preempting anybody.  The rows keep ``prev``'s order, so row ``i`` of
        the new step continues row ``i`` of ``prev`` (its input token is still on the device).  A request that
        ``prev`` ends after all (stop token) simply leaves its row's result unused: ``commit`` skips rows whose
        request is no longer running.  Returns None whenever a condition fails; nothing is rolled back then (pages
        reserved so far are the ones the next regular plan would reserve).
        """
        if self.waiting or len(prev.segments) != len(self.running) or prev.copies or prev.preempted:
            return None
        segs = []
        for s in prev.segments:
            r = s.request
            sp = r.sampling
            if s.count != 1 or not s.sample or r.status is not RequestStatus.RUNNING or sp.matcher is not None:
                return None
            if len(r.output) + 2 > sp.max_tokens or r.num_tokens + 2 > self.cfg.max_model_len:
                return None                       # ``prev`` may end it by length: plan the next step the regular way
            start = s.start + 1
            need = -(-(start + 1) // BLOCK) - len(r.pages)
            if need > 0:
                if need > self.pool.num_free:
                    return None
                r.pages.extend(self.pool.alloc(need))
            segs.append(PlannedSegment(r, start, 1, True))
        return BatchPlan(segs)

    # ----------------------------------------------------------------- commit
    def commit(self, plan: BatchPlan, sampled: dict[str, int], eos_token_id: int | None = None) -> list[Request]:
        """Apply a finished step: advance computed counts, append sampled tokens, retire finished requests."""
        finished = []
        for seg in plan.segments:
            r = seg.request
            if r.status is not RequestStatus.RUNNING:
                continue
            r.num_computed += seg.count
            full = r.num_computed // BLOCK
            if full > r.num_published and self.prefix.enabled:
                self.prefix.publish(_keys(r, r.tokens[:full * BLOCK]), r.pages[:full])
                r.num_published = full
                if self.prefix.needs_checkpoint and r.num_computed == full * BLOCK and not seg.sample:
                    # the step ended on a page boundary inside the prompt: its recurrent state is a valid snapshot
                    slot = self.prefix.publish_checkpoint(_keys(r, r.tokens[:full * BLOCK]))
                    if slot is not None:
                        self.state_saves.append((r.slot, slot))
            if seg.sample:
                toks = sampled[r.request_id]
                # a speculative round hands back several tokens (accepted drafts + the bonus token); each extra
                # token also means one more position whose KV is already in the cache
                toks = [toks] if isinstance(toks, int) else list(toks)
                sp = r.sampling
                r.last_committed = 0
                for j, tok in enumerate(toks):
                    r.append_output(tok)
                    r.last_committed += 1
                    r.draws += 1
                    if j:
                        r.num_computed += 1
                    stop = tok in sp.stop_token_ids or (eos_token_id is not None and tok == eos_token_id and not sp.ignore_eos)
                    if stop:
                        self._retire(r, FinishReason.STOP)
                        finished.append(r)
                        break
                    if len(r.output) >= sp.max_tokens or r.num_tokens >= self.cfg.max_model_len:
                        self._retire(r, FinishReason.LENGTH)
                        finished.append(r)
                        break
        return finished

    def _retire(self, r: Request, reason: FinishReason) -> None:
        if r in self.running:
            self.running.remove(r)
        self._finish(r, reason, RequestStatus.FINISHED)

    def _finish(self, r: Request, reason: FinishReason, status: RequestStatus) -> None:
        if r.pages:
            self.pool.release(r.pages)
            r.pages = []
        if r.slot >= 0:
            self._free_slots.append(r.slot)
            r.slot = -1
        r.status = status
        r.finish_reason = reason

    def stats(self) -> dict:
        total = self.pool.num_pages - self.pool.reserved
        return {
            "running": len(self.running), "waiting": len(self.waiting),
            "kv_used_frac": self.pool.num_used / total if total else 0.0,
            "prefix_entries": len(self.prefix), "prefix_hit_rate": self.prefix.hit_rate,
        }
