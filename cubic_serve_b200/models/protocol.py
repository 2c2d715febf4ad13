"""What the engine asks of an executor, and what a model family has to supply to get one.

The engine (``runtime/engine.py``) drives every executor through the same small surface; everything else is an optional
capability that the engine discovers by attribute and uses when present.  The protocols below state that surface in one
place, so that a new executor (or an adapter's, ``models/registry.py``) can be checked against it before it serves:
``check_executor`` reports what is missing and which capabilities were found.

Required:

* ``execute(segments) -> int32 array``: run one step; one sampled token per segment with ``sample`` set, in order;
* ``copy_pages(pairs)``: copy-on-write of KV pages ``(source, destination)`` before the step that writes them.

Optional capabilities (attribute -> meaning):

* ``launch(segments, feedback_rows) / collect(handle)``: the step split in two, so the engine can queue the next decode
  step before it reads this one's tokens;
* ``execute_speculative(segments, depths)`` + ``speculative_depth``: draft / review rounds that return several tokens;
* ``copy_state(pairs)`` + ``state_checkpoint_rows``: snapshot rows of recurrent state, which keep the prefix cache on for
  models with recurrent layers;
* ``invalidate_page_rows(slots)``: a cached device page table exists and must forget these request slots;
* ``accepts_features``: segments may carry encoder feature rows and three-axis positions;
* ``keeps_request_state``: the executor holds a request's context itself (no pages): the engine keeps prefix sharing off;
* ``reasoning_end_id``: thinking budgets are enforced by the executor.

Reference counterpart: ``models/protocol.py:28-251`` there (``ModelSegment``, ``ModelStepResult``, the semantic-op
executor protocol that adapters implement).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol, Sequence, runtime_checkable

import numpy as np

from ..executor.gpu_executor import Segment as ModelSegment          # one request's slice of a step


@runtime_checkable
class StepExecutor(Protocol):
    def execute(self, segs: Sequence[ModelSegment]) -> np.ndarray: ...

    def copy_pages(self, pairs) -> None: ...


@runtime_checkable
class OverlappedExecutor(StepExecutor, Protocol):
    def launch(self, segs: Sequence[ModelSegment], feedback_rows: int = 0): ...

    def collect(self, handle) -> np.ndarray: ...


@runtime_checkable
class SpeculativeExecutor(StepExecutor, Protocol):
    speculative_depth: int

    def execute_speculative(self, segs: Sequence[ModelSegment], depths=None): ...


@runtime_checkable
class StatefulExecutor(StepExecutor, Protocol):
    state_checkpoint_rows: tuple

    def copy_state(self, pairs) -> None: ...


@dataclass(frozen=True)
class ExecutorCapabilities:
    overlapped: bool
    speculative: bool
    state_snapshots: bool
    page_table_cache: bool
    features: bool
    request_state: bool
    reasoning_budget: bool


def check_executor(executor) -> ExecutorCapabilities:
    """Raise ``TypeError`` when ``executor`` lacks the required surface; otherwise report its optional capabilities."""
    missing = [n for n in ("execute", "copy_pages") if not callable(getattr(executor, n, None))]
    if missing:
        raise TypeError(f"{type(executor).__name__} is not an executor: it lacks {missing}")
    half = [n for n in ("launch", "collect") if callable(getattr(executor, n, None))]
    if len(half) == 1:
        raise TypeError(f"{type(executor).__name__} has {half[0]} without its counterpart")
    if callable(getattr(executor, "execute_speculative", None)) and not hasattr(executor, "speculative_depth"):
        raise TypeError(f"{type(executor).__name__} runs speculative rounds but states no speculative_depth")
    rows = tuple(getattr(executor, "state_checkpoint_rows", ()) or ())
    if rows and not callable(getattr(executor, "copy_state", None)):
        raise TypeError(f"{type(executor).__name__} sets snapshot rows aside but cannot copy state into them")
    return ExecutorCapabilities(
        overlapped=len(half) == 2, speculative=callable(getattr(executor, "execute_speculative", None)),
        state_snapshots=bool(rows), page_table_cache=callable(getattr(executor, "invalidate_page_rows", None)),
        features=bool(getattr(executor, "accepts_features", False)),
        request_state=bool(getattr(executor, "keeps_request_state", False)),
        reasoning_budget=getattr(executor, "reasoning_end_id", None) is not None)
