"""The synchronous serving engine: scheduler + page pool + an executor.

``LLMEngine.step()`` is one iteration of the reference's dispatch loop
(``runtime/performance.py:10519`` ``_dispatch`` -> ``_next_batch_locked`` ->
worker replay -> ``_receive_batch`` commit), without the process boundary: the
async front end (``runtime/async_engine.py``) drives it from a dispatcher thread.
The executor is anything with ``execute(segments) -> token ids`` and
``copy_pages(pairs)``: the native GPU executor, the tensor-parallel group
executor, or the eager CPU executor.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass

import numpy as np

from ..executor.gpu_executor import Segment
from .cache.pool import PagePool
from .cache.prefix import PrefixCache
from .scheduler import (AdmissionError, BatchPlan, ContinuousScheduler, FinishReason, Request, RequestStatus,
                        SamplingParams, SchedulerConfig)


@dataclass
class StepOutput:
    request_id: str
    token_id: int | None
    finished: bool
    finish_reason: FinishReason | None = None


class EnginePoisoned(RuntimeError):
    """A step failed; the engine fails closed (reference: ``performance.py:10991-11016``)."""


class LLMEngine:
    def __init__(self, executor, num_pages: int, scheduler_config: SchedulerConfig | None = None,
                 eos_token_id: int | None = None) -> None:
        self.executor = executor
        self.cfg = scheduler_config or SchedulerConfig()
        rows = tuple(getattr(executor, "state_checkpoint_rows", ()) or ())
        if (getattr(getattr(executor, "cfg", None), "is_hybrid", False) or rows
                or getattr(executor, "keeps_request_state", False)) and self.cfg.enable_prefix_cache:
            # recurrent (Gated DeltaNet) state: a cached prefix is resumable only with a snapshot of the state at its
            # end; executors that set rows aside for snapshots (``state_checkpoint_rows``) keep the prefix cache on
            from dataclasses import replace
            if rows and hasattr(executor, "copy_state"):
                self.cfg = replace(self.cfg, state_checkpoint_slots=rows)
            else:
                self.cfg = replace(self.cfg, enable_prefix_cache=False)
        self.pool = PagePool(num_pages)
        self.prefix = PrefixCache(self.pool, enabled=self.cfg.enable_prefix_cache,
                                  checkpoint_slots=self.cfg.state_checkpoint_slots or None)
        self.scheduler = ContinuousScheduler(self.cfg, self.pool, self.prefix)
        self.scheduler.decode_lookahead = getattr(executor, "speculative_depth", 0)
        self.eos_token_id = eos_token_id
        # dynamic draft length (reference: runtime/speculative.py DynamicDraftPlanner.plan): per-request acceptance
        # history + measured round costs choose each request's draft length; off = the executor's fixed depth
        self.draft_planner = None
        # launch the next decode step before this one's results are read (steady decode state only)
        self.overlap_decode = True
        self._ahead = None
        self.ngram = None                # n-gram draft proposer (created by the first round of an n-gram executor)
        self._ahead_stale = False
        self._budget_sig: dict[str, tuple[int, int]] = {}
        self._draft_states: dict = {}
        vocab = getattr(getattr(executor, "cfg", None), "vocab_size", None) or getattr(executor, "vocab_size", 0)
        self._mask_words = -(-int(vocab) // 32) if vocab else 0
        self._ids = itertools.count()
        self.requests: dict[str, Request] = {}
        self.poisoned = False
        self.steps = 0
        self.generated_tokens = 0
        self.prefill_tokens = 0
        self.last_step_seconds = 0.0

    # ------------------------------------------------------------------ API
    def add_request(self, prompt_token_ids: list[int], sampling: SamplingParams | None = None,
                    request_id: str | None = None, multimodal=None) -> str:
        """``multimodal``: a ``runtime.multimodal.MultimodalInput`` for prompts whose media were expanded into
        placeholder tokens; only executors that take feature rows (``accepts_features``) admit such requests."""
        if self.poisoned:
            raise EnginePoisoned("engine is poisoned")
        if multimodal is not None:
            if not getattr(self.executor, "accepts_features", False):
                raise AdmissionError("this executor serves text only; requests with media are not accepted", status=400)
            if getattr(multimodal, "deep_layers", 0) and not getattr(self.executor, "accepts_deepstack", False):
                raise AdmissionError("this executor does not consume the vision tower's intermediate outputs", status=400)
            if multimodal.prompt_length != len(prompt_token_ids):
                raise AdmissionError("the media positions do not cover the prompt", status=400)
        rid = request_id or f"req-{next(self._ids)}"
        if rid in self.requests:
            raise AdmissionError(f"duplicate request id {rid}")
        if len(self.scheduler.waiting) + len(self.scheduler.running) >= 4 * self.cfg.max_running_requests:
            raise AdmissionError("too many queued requests", status=429)
        req = Request(rid, list(prompt_token_ids), sampling or SamplingParams(), multimodal=multimodal)
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def abort(self, request_id: str) -> bool:
        r = self.scheduler.abort(request_id)
        self.requests.pop(request_id, None)
        return r is not None

    @property
    def has_unfinished(self) -> bool:
        return self.scheduler.has_work

    def step(self) -> list[StepOutput]:
        """One engine step.  In the steady decode state the NEXT step is launched before this step's results are
        read (``overlap_decode``): the device then never waits for the host's scheduling and output handling.
        The look-ahead step takes its input tokens from the device and is planned by
        ``ContinuousScheduler.lookahead_plan``; whenever its conditions fail the step runs the regular way."""
        if self.poisoned:
            raise EnginePoisoned("engine is poisoned")
        t0 = time.perf_counter()
        try:
            ahead, self._ahead = self._ahead, None
            if ahead is not None:
                plan, handle = ahead
            else:
                plan = self.scheduler.next_plan()
                if plan is None:
                    return []
                handle = None
                if plan.finished and not plan.segments:
                    return self._ended_by_scheduler(plan)
            if handle is None and not self._can_overlap(plan):
                outputs = self._run(plan)
            else:
                if handle is None:
                    handle = self.executor.launch(self._segments(plan))
                nxt = self.scheduler.lookahead_plan(plan) if self._can_overlap(plan) else None
                if nxt is not None:
                    rows = len(nxt.segments)
                    self._ahead = (nxt, self.executor.launch(self._segments(nxt, ahead=True), feedback_rows=rows))
                outputs = self._complete(plan, self.executor.collect(handle))
                if self._ahead is not None and len(self.scheduler.running) != len(self._ahead[0].segments):
                    # a request ended in this step: its look-ahead row is dropped at commit, and no further step is
                    # launched from the shortened one until a regular plan has been made
                    self._ahead_stale = True
        except Exception:
            self.poisoned = True
            self.pool.poison()
            raise
        self.last_step_seconds = time.perf_counter() - t0
        self.steps += 1
        return outputs

    def _ended_by_scheduler(self, plan: BatchPlan) -> list[StepOutput]:
        """Outputs of requests that the scheduler ended while planning (out of cache pages for good): no token, only
        the finish event, so that the client's stream closes."""
        outs = []
        for r in plan.finished:
            if self.requests.pop(r.request_id, None) is None:
                continue
            self._draft_states.pop(r.request_id, None)
            self._budget_sig.pop(r.request_id, None)
            if self.ngram is not None:
                self.ngram.forget(r.request_id)
            outs.append(StepOutput(r.request_id, None, True, r.finish_reason))
        plan.finished = []
        return outs

    def _can_overlap(self, plan: BatchPlan) -> bool:
        if not self.overlap_decode or not hasattr(self.executor, "launch") or getattr(self.executor, "speculative_depth", 0):
            return False
        if getattr(self, "_ahead_stale", False):
            self._ahead_stale = False
            return False
        return bool(plan.segments) and not plan.copies and not plan.finished and not plan.state_restores and all(
            s.count == 1 and s.sample and s.request.sampling.matcher is None for s in plan.segments)

    def _segments(self, plan: BatchPlan, ahead: bool = False) -> list:
        """Executor segments of a plan.  ``ahead``: the plan is a look-ahead step whose input tokens are not known on
        the host yet (the previous step's commit will append them); draws count that commit in."""
        segs = []
        end_id = getattr(self.executor, "reasoning_end_id", None)
        for s in plan.segments:
            r = s.request
            toks = [0] if ahead else r.tokens[s.start:s.start + s.count]
            sp = r.sampling
            mask = mask_fn = None
            if s.sample and sp.matcher is not None:
                mask = np.zeros(self._mask_words, dtype=np.uint32)
                sp.matcher.fill_bitmask(mask)
                mask_fn = self._review_masks_of(sp.matcher)
            segs.append(Segment(r.slot, toks, s.start, r.pages, s.sample, sp.temperature, sp.top_p, sp.top_k,
                                sp.seed if sp.seed is not None else hash(r.request_id) & 0x7FFFFFFF,
                                r.draws + (1 if ahead else 0), (r.arrival << 16) | (r.preemptions & 0xFFFF), mask,
                                self._budget_init(r) if s.sample and end_id is not None else -2, mask_fn))
            if r.multimodal is not None:
                segs[-1].embeds, segs[-1].positions3 = r.multimodal.segment_inputs(s.start, s.count)
                if getattr(r.multimodal, "deep_layers", 0):
                    segs[-1].deep_embeds = r.multimodal.segment_deep(s.start, s.count)
        return segs

    def _review_masks_of(self, matcher):
        """The mask rows of a speculative round for one constrained request: row j allows what the grammar allows after
        it has accepted the first j drafts.  The drafts are fed to the matcher tentatively and rolled back, so the
        matcher is where it was afterwards; rows behind a draft the grammar refuses are never reached by the
        verification (the refused draft cannot equal the masked choice) and are left open."""
        words = self._mask_words

        def masks(drafts: list[int]) -> np.ndarray:
            out = np.full((len(drafts) + 1, words), 0xFFFFFFFF, dtype=np.uint32)
            row = np.zeros(words, dtype=np.uint32)
            matcher.fill_bitmask(row)
            out[0] = row
            fed = 0
            for j, t in enumerate(drafts):
                if getattr(matcher, "finished", False) or not matcher.accept(int(t)):
                    break
                fed += 1
                row = np.zeros(words, dtype=np.uint32)
                matcher.fill_bitmask(row)
                out[j + 1] = row
            if fed:
                matcher.rollback(fed)
            return out
        return masks

    def _budget_init(self, r: Request) -> int:
        """Thinking-budget command of a sampled row: the device counter of the request's slot is (re)armed on the
        first sampled step after the request got its slot (admission, or re-admission after a preemption)."""
        sig = (r.slot, r.preemptions)
        if self._budget_sig.get(r.request_id) == sig:
            return -2
        self._budget_sig[r.request_id] = sig
        b = r.sampling.thinking_budget
        if b is None or self.executor.reasoning_end_id in r.output:
            return -1
        return max(0, b - len(r.output))

    def _run(self, plan: BatchPlan) -> list[StepOutput]:
        if plan.state_restores:
            self.executor.copy_state(plan.state_restores)
        if plan.copies:
            self.executor.copy_pages(plan.copies)
            if hasattr(self.executor, "invalidate_page_rows"):
                self.executor.invalidate_page_rows([s.request.slot for s in plan.segments])
        segs = self._segments(plan)
        spec = getattr(self.executor, "speculative_depth", 0)
        constrained = any(s.mask is not None for s in segs)
        # rounds serve greedy requests (drafts verified against the target's greedy choice) and, on executors that
        # verify by p / q rejection sampling (``speculative_sampling``), sampling requests too; a step with a
        # constrained request runs the plain way
        samples = bool(getattr(self.executor, "speculative_sampling", False))
        if constrained and getattr(self.executor, "speculative_grammar", False):
            constrained = False          # the review rows are sampled under the grammars' masks (Segment.mask_fn)
        if spec and segs and not constrained and all(len(s.token_ids) == 1 and s.sample and (samples or s.temperature == 0)
                                                     for s in segs):
            # speculative round: every request gets its accepted drafts plus one bonus token
            ids = self._speculative_round(plan, segs, spec)
            self.spec_rounds = getattr(self, "spec_rounds", 0) + 1
        else:
            ids = self.executor.execute(segs) if segs else []
        return self._complete(plan, ids) + self._ended_by_scheduler(plan)

    def _complete(self, plan: BatchPlan, ids) -> list[StepOutput]:
        """Second half of a step: match ids to requests, commit, build the outputs.  Rows of a look-ahead step whose
        request ended in the step before are skipped."""
        sampled = {}
        it = iter(ids)
        for s in plan.segments:
            if s.sample:
                v = next(it)
                if s.request.status is not RequestStatus.RUNNING:
                    continue
                sampled[s.request.request_id] = [int(t) for t in v] if isinstance(v, (list, tuple)) else int(v)
                m = s.request.sampling.matcher
                if m is not None:
                    # a speculative round hands back several tokens: accepted drafts and the next token, all sampled
                    # under the grammar's masks; tokens after the one that completes the grammar are cut by the stop rule
                    for t in (v if isinstance(v, (list, tuple)) else [v]):
                        if getattr(m, "finished", False):
                            break
                        if not m.accept(int(t)):
                            raise RuntimeError(f"request {s.request.request_id}: sampled token {int(t)} violates its constraint")
            else:
                self.prefill_tokens += s.count
        finished = {r.request_id: r for r in self.scheduler.commit(plan, sampled, self.eos_token_id)}
        if self.scheduler.state_saves:
            # snapshots of the recurrent state at freshly published page boundaries (stream-ordered after the step)
            saves, self.scheduler.state_saves = self.scheduler.state_saves, []
            self.executor.copy_state(saves)
        outs = []
        for s in plan.segments:
            if not s.sample or s.request.request_id not in sampled:
                continue
            rid = s.request.request_id
            toks = sampled[rid] if isinstance(sampled[rid], list) else [sampled[rid]]
            fin = finished.get(rid)
            toks = toks[:s.request.last_committed]      # a stop / length limit may cut a speculative burst short
            self.generated_tokens += len(toks)
            for j, tok in enumerate(toks):
                last = j == len(toks) - 1
                outs.append(StepOutput(rid, tok, fin is not None and last, fin.finish_reason if (fin and last) else None))
            if fin is not None:
                self.requests.pop(rid, None)
                self._draft_states.pop(rid, None)
                if self.ngram is not None:
                    self.ngram.forget(rid)
                self._budget_sig.pop(rid, None)
        return outs

    def enable_dynamic_draft(self, config=None, graph_capacities: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512,
                                                                                    1024, 2048, 4096)) -> None:
        """Let the planner choose every request's draft length (up to the executor's depth) round by round."""
        from .speculative import DraftPlanner, DraftPolicyConfig
        self._draft_cfg = config or DraftPolicyConfig()
        self.draft_planner = DraftPlanner(graph_capacities, self._draft_cfg)

    def _speculative_round(self, plan: BatchPlan, segs: list, max_depth: int):
        if getattr(self.executor, "draft_source", "model") == "ngram":
            return self._ngram_round(plan, segs, max_depth)
        if self.draft_planner is None:
            return self.executor.execute_speculative(segs)
        from .speculative import RequestDraftState
        rids = [s.request.request_id for s in plan.segments]
        for rid in rids:
            if rid not in self._draft_states:
                self._draft_states[rid] = RequestDraftState(max_depth, max_depth, self._draft_cfg)
        planned = {p.request_id: p.draft_tokens for p in self.draft_planner.plan({rid: self._draft_states[rid] for rid in rids})}
        depths = [planned.get(rid, max_depth) for rid in rids]
        ids = self.executor.execute_speculative(segs, depths)
        info = getattr(self.executor, "last_round", None)
        if info:
            for rid, acc, prop in zip(rids, info["accepted"], info["proposed"]):
                st = self._draft_states[rid]
                if prop > 0 and not st.stopped:
                    st.observe(min(acc, prop), prop)
            if info["target_ms"]:
                self.draft_planner.observe_round(sum(p + 1 for p in info["proposed"]), info["target_ms"], len(rids),
                                                 info["proposal_ms"], info["depth"])
        return ids

    def _ngram_round(self, plan: BatchPlan, segs: list, max_depth: int):
        """Drafts from the requests' own token histories (``runtime/ngram.py``); a request proposes at most what its
        token limit still allows."""
        if self.ngram is None:
            from .ngram import NgramProposer
            self.ngram = NgramProposer()
        drafts = []
        for s in plan.segments:
            r = s.request
            room = max(0, r.sampling.max_tokens - len(r.output) - 1)
            drafts.append(self.ngram.propose(r.request_id, r.tokens, min(max_depth, room)))
        return self.executor.execute_speculative(segs, drafts=drafts)

    def generate(self, prompts: list[list[int]], sampling: SamplingParams | None = None) -> list[list[int]]:
        """Blocking helper: run all prompts to completion, return the generated ids per prompt."""
        ids = [self.add_request(p, SamplingParams(**vars(sampling)) if sampling else None) for p in prompts]
        reqs = [self.requests[i] for i in ids]
        while self.has_unfinished:
            self.step()
        return [r.output for r in reqs]

    def stats(self) -> dict:
        s = self.scheduler.stats()
        s.update(steps=self.steps, generated_tokens=self.generated_tokens, prefill_tokens=self.prefill_tokens)
        return s
