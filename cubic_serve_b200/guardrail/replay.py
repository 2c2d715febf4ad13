"""Canonical execution traces and their deterministic replay.

A trace is a JSON-lines file: one ``request`` record per admitted request (arrival step, prompt token ids, sampling
parameters) and one ``step`` record per engine step (the ids every request emitted in that step, its finish reason
when it ended).  ``replay_trace`` re-admits the requests at the same steps into a fresh engine, steps it, and compares
what it emits with the trace, token by token; the first difference is reported with its step and request.

Every step record also carries the cache's lifecycle at the end of the step (``lifecycle``): pages in use, blocks the
prefix cache holds, tokens served from it so far, preemptions so far, and for every request admitted in that step how
many of its prompt tokens came from cached pages.  ``replay_trace(..., check_lifecycle=True)`` compares these too: two
executions that emit the same tokens but share, evict or preempt differently are told apart (the comparison needs the
same scheduler settings and pool size on both sides, so it is opt-in).

Used to check that two executions agree: CUDA-graph replay against eager launches, one tensor-parallel size against
another, overlapped decode launches against step-by-step execution, a new build against a recorded run.  Emission order
inside a step is not compared (schedulers may order rows differently); the tokens of every request are.

Reference counterpart: ``guardrail/replay.py`` and ``guardrail/engine_replay.py`` (canonical traces, deterministic
replay with prefix-lifecycle evidence).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path

from ..runtime.scheduler import SamplingParams

_SAMPLING_FIELDS = ("temperature", "top_p", "top_k", "seed", "max_tokens", "stop_token_ids", "ignore_eos", "thinking_budget")


@dataclass
class ReplayReport:
    ok: bool
    steps: int
    tokens: int
    first_difference: dict | None = None
    notes: list[str] = field(default_factory=list)

    def to_json(self) -> str:
        return json.dumps(asdict(self))


class TraceRecorder:
    """Records what an ``LLMEngine`` is given and what it emits.  Use ``add_request`` / ``step`` of the recorder in
    place of the engine's."""

    def __init__(self, engine) -> None:
        self.engine = engine
        self.records: list[dict] = []
        self._step = 0
        self._seen: set[str] = set()

    def add_request(self, prompt_token_ids: list[int], sampling: SamplingParams | None = None,
                    request_id: str | None = None) -> str:
        sp = sampling or SamplingParams()
        if sp.matcher is not None:
            raise ValueError("requests with a structured-output matcher are not replayable from a token trace")
        rid = self.engine.add_request(prompt_token_ids, sp, request_id)
        rec = {"kind": "request", "at_step": self._step, "request_id": rid, "prompt": list(prompt_token_ids),
               "sampling": {k: getattr(sp, k) for k in _SAMPLING_FIELDS}}
        rec["sampling"]["stop_token_ids"] = list(rec["sampling"]["stop_token_ids"])
        self.records.append(rec)
        return rid

    def step(self):
        outs = self.engine.step()
        emitted: dict[str, list[int]] = {}
        finished: dict[str, str] = {}
        for o in outs:
            if o.token_id is not None:
                emitted.setdefault(o.request_id, []).append(int(o.token_id))
            if o.finished:
                finished[o.request_id] = getattr(o.finish_reason, "value", str(o.finish_reason))
        self.records.append({"kind": "step", "index": self._step, "emitted": emitted, "finished": finished,
                             "lifecycle": lifecycle_of(self.engine, self._seen)})
        self._step += 1
        return outs

    def run(self) -> None:
        """Step until the engine has nothing left to do (including a step it launched ahead)."""
        while self.engine.has_unfinished or getattr(self.engine, "_ahead", None) is not None:
            self.step()

    def save(self, path: str | Path) -> Path:
        path = Path(path)
        with path.open("w") as f:
            for r in self.records:
                f.write(json.dumps(r) + "\n")
        return path


def lifecycle_of(engine, seen: set) -> dict:
    """The cache's state after a step: what is resident, what was shared, who was admitted with how long a cached
    prefix.  ``seen`` collects the requests already reported as admitted."""
    pool, prefix = getattr(engine, "pool", None), getattr(engine, "prefix", None)
    admitted = {}
    preemptions = 0
    for rid, r in getattr(engine, "requests", {}).items():
        preemptions += getattr(r, "preemptions", 0)
        if rid not in seen and (getattr(r, "pages", None) or getattr(r, "num_computed", 0)):
            seen.add(rid)
            admitted[rid] = int(getattr(r, "num_cached_prefix", 0))
    return {"pages_used": getattr(pool, "num_used", 0), "prefix_blocks": len(prefix) if prefix is not None else 0,
            "prefix_hit_tokens": getattr(prefix, "hit_tokens", 0), "preemptions_running": preemptions, "admitted": admitted}


def load_trace(path: str | Path) -> list[dict]:
    return [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]


def replay_trace(trace: list[dict] | str | Path, engine, max_extra_steps: int = 64,
                 check_lifecycle: bool = False) -> ReplayReport:
    """Feed the trace's requests to ``engine`` at their recorded steps and compare every request's tokens.

    Step boundaries may differ between executions (a look-ahead step, another chunking of a prefill), so the
    comparison is per request over the whole run, and per step only as far as the step records line up: the report
    names the first request whose token sequence differs and the position of the difference.
    """
    records = load_trace(trace) if not isinstance(trace, list) else trace
    by_step: dict[int, list[dict]] = {}
    for r in records:
        if r["kind"] == "request":
            by_step.setdefault(r["at_step"], []).append(r)
    want: dict[str, list[int]] = {}
    want_finish: dict[str, str] = {}
    n_steps = 0
    for r in records:
        if r["kind"] == "step":
            n_steps += 1
            for rid, toks in r["emitted"].items():
                want.setdefault(rid, []).extend(toks)
            want_finish.update(r["finished"])
    got: dict[str, list[int]] = {}
    got_finish: dict[str, str] = {}
    want_life = [r.get("lifecycle") for r in records if r["kind"] == "step"]
    got_life: list[dict] = []
    seen: set[str] = set()
    step = 0
    last_arrival = max(by_step) if by_step else -1
    while step <= last_arrival or engine.has_unfinished or getattr(engine, "_ahead", None) is not None:
        for r in by_step.get(step, []):
            sp = dict(r["sampling"])
            sp["stop_token_ids"] = tuple(sp.get("stop_token_ids", ()))
            engine.add_request(r["prompt"], SamplingParams(**sp), r["request_id"])
        for o in engine.step():
            if o.token_id is not None:
                got.setdefault(o.request_id, []).append(int(o.token_id))
            if o.finished:
                got_finish[o.request_id] = getattr(o.finish_reason, "value", str(o.finish_reason))
        got_life.append(lifecycle_of(engine, seen))
        step += 1
        if step > n_steps + max_extra_steps:
            return ReplayReport(False, step, sum(map(len, got.values())),
                                {"reason": "the replay did not finish within the recorded number of steps"})
    tokens = sum(map(len, got.values()))
    for rid, toks in want.items():
        mine = got.get(rid, [])
        if mine != toks:
            pos = next((i for i, (a, b) in enumerate(zip(mine, toks)) if a != b), min(len(mine), len(toks)))
            return ReplayReport(False, step, tokens, {"request_id": rid, "position": pos,
                                                      "recorded": toks[pos:pos + 4], "replayed": mine[pos:pos + 4]})
    for rid, why in want_finish.items():
        if got_finish.get(rid) != why:
            return ReplayReport(False, step, tokens, {"request_id": rid, "recorded_finish": why,
                                                      "replayed_finish": got_finish.get(rid)})
    extra = sorted(set(got) - set(want))
    if extra:
        return ReplayReport(False, step, tokens, {"reason": "requests emitted tokens that the trace does not have", "ids": extra[:4]})
    notes = [] if step == n_steps else [f"the replay took {step} steps, the recording {n_steps}"]
    if check_lifecycle:
        if step != n_steps:
            return ReplayReport(False, step, tokens, {"reason": "the cache lifecycle is compared step by step, and the "
                                                                "replay took another number of steps"}, notes)
        for i, (a, b) in enumerate(zip(want_life, got_life)):
            if a is None:
                return ReplayReport(False, step, tokens, {"reason": "the trace carries no lifecycle records"}, notes)
            if a != b:
                keys = [k for k in a if a[k] != b.get(k)]
                return ReplayReport(False, step, tokens, {"step": i, "lifecycle": keys,
                                                          "recorded": {k: a[k] for k in keys},
                                                          "replayed": {k: b.get(k) for k in keys}}, notes)
    return ReplayReport(True, step, tokens, None, notes)
