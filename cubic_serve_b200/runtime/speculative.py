"""Dynamic MTP draft-length policy: per-request acceptance tracking and a load-aware planner.

Behavioural twin of the reference's ``runtime/speculative.py`` (``DraftPolicyConfig`` ``:18``,
``DynamicDraftPolicy`` ``:68``, ``_EmaCurve`` ``:212``, ``DynamicDraftPlanner.plan`` ``:802``), written from
its documented rules (``runtime/README.md:207-309`` there):

* each request keeps, per draft depth ``d``, decayed counts of "depth d was tried" / "depth d was accepted
  given depth d-1 was" with a Beta(4, 1) prior; the product of the conditional means is the survival curve
  ``P(accepted >= d)``;
* a request may change its draft length K only at a decision boundary (>= 24 emitted tokens AND >= 8 rounds
  since the last decision), and only by ONE level per decision;
* the planner prices a round as target-review cost at the padded row count + K proposal passes + fixed
  overhead, all taken from EMA curves over graph capacities fed with median-of-3 samples, and picks for every
  request the K with the best expected tokens per millisecond given the load;
* K = 0 (no drafting) is terminal for a request, and is chosen only if it beats the best K >= 1 by more than a
  3 % margin; capacity pressure may force it earlier (``stop_for_capacity``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field, fields
from math import isfinite


class DraftAction(str, enum.Enum):
    PROMOTE = "promote"
    HOLD = "hold"
    DEMOTE = "demote"


@dataclass(frozen=True)
class DraftPolicyConfig:
    decision_tokens: int = 24
    decision_min_rounds: int = 8
    prior_success: float = 4.0
    prior_failure: float = 1.0
    history_decay: float = 0.99
    cost_ema_alpha: float = 0.2
    cost_sample_window: int = 3
    terminal_stop_margin: float = 0.03

    def __post_init__(self) -> None:
        for v in (self.prior_success, self.prior_failure, self.history_decay, self.cost_ema_alpha, self.terminal_stop_margin):
            if not isinstance(v, (int, float)) or isinstance(v, bool) or not isfinite(v):
                raise ValueError("draft policy parameters must be finite numbers")
        if self.cost_sample_window not in (1, 3, 5, 7):
            raise ValueError("cost sample window must be 1, 3, 5 or 7")
        if self.terminal_stop_margin < 0 or not 0 < self.cost_ema_alpha <= 1:
            raise ValueError("margin must be >= 0 and EMA alpha in (0, 1]")
        if self.decision_tokens < 1 or self.decision_min_rounds < 1:
            raise ValueError("decision interval must be positive")
        if self.prior_success <= 0 or self.prior_failure <= 0 or not 0 < self.history_decay < 1:
            raise ValueError("prior must be positive and the decay in (0, 1)")

    @classmethod
    def from_dict(cls, d: object) -> "DraftPolicyConfig":
        if not isinstance(d, dict) or set(d) - {f.name for f in fields(cls)}:
            raise ValueError("unknown dynamic draft policy fields")
        return cls(**d)


@dataclass(frozen=True)
class DraftDecision:
    action: DraftAction
    previous_tokens: int
    next_tokens: int


class RequestDraftState:
    """One request's acceptance history and current draft length."""

    def __init__(self, initial_tokens: int, max_tokens: int, config: DraftPolicyConfig | None = None) -> None:
        if not 1 <= initial_tokens <= max_tokens:
            raise ValueError("need 1 <= initial <= max draft tokens")
        self.cfg = config or DraftPolicyConfig()
        self.max_tokens = max_tokens
        self.current_tokens = initial_tokens
        self.stopped = False
        self._hit = [0.0] * max_tokens
        self._tried = [0.0] * max_tokens
        self._rounds = 0
        self._window_tokens = 0

    @property
    def ready(self) -> bool:
        return self._rounds >= self.cfg.decision_min_rounds and self._window_tokens >= self.cfg.decision_tokens

    def observe(self, accepted: int, proposed: int) -> None:
        if self.stopped:
            raise RuntimeError("a request that stopped drafting takes no more observations")
        if not 1 <= proposed <= self.current_tokens or not 0 <= accepted <= proposed:
            raise ValueError("observation does not match the active draft length")
        g = self.cfg.history_decay
        self._hit = [h * g for h in self._hit]
        self._tried = [t * g for t in self._tried]
        for depth in range(1, proposed + 1):
            if accepted < depth - 1:
                break                       # depth d is only "tried" if depth d-1 survived
            self._tried[depth - 1] += 1.0
            self._hit[depth - 1] += 1.0 if accepted >= depth else 0.0
        self._rounds += 1
        self._window_tokens += accepted + 1

    def survival(self) -> tuple[float, ...]:
        """Monotone ``P(accepted >= d)`` for d = 1..max; untried depths inherit the last conditional mean."""
        a, b = self.cfg.prior_success, self.cfg.prior_failure
        cond = a / (a + b)
        s, out = 1.0, []
        for hit, tried in zip(self._hit, self._tried):
            if tried:
                cond = (a + hit) / (a + b + tried)
            s *= cond
            out.append(s)
        return tuple(out)

    def expected_tokens(self, k: int) -> float:
        """Tokens emitted per round with draft length k: the bonus token plus the surviving drafts."""
        return 1.0 + sum(self.survival()[:k])

    def stop_for_capacity(self) -> DraftDecision:
        prev = self.current_tokens
        self.current_tokens, self.stopped = 0, True
        return DraftDecision(DraftAction.HOLD if prev == 0 else DraftAction.DEMOTE, prev, 0)

    def move_toward(self, target: int) -> DraftDecision:
        if self.stopped:
            raise RuntimeError("a request that stopped drafting makes no more decisions")
        if not 0 <= target <= self.max_tokens:
            raise ValueError("target outside the request's bounds")
        prev = self.current_tokens
        if not self.ready:
            return DraftDecision(DraftAction.HOLD, prev, prev)
        self._rounds = self._window_tokens = 0
        if target == prev:
            return DraftDecision(DraftAction.HOLD, prev, prev)
        nxt = prev + (1 if target > prev else -1)
        self.current_tokens = nxt
        if nxt == 0:
            self.stopped = True
        return DraftDecision(DraftAction.PROMOTE if nxt > prev else DraftAction.DEMOTE, prev, nxt)


class CostCurve:
    """Milliseconds as a function of graph capacity: EMA over the median of ``window`` samples, interpolated."""

    def __init__(self, alpha: float = 0.2, window: int = 3) -> None:
        self.alpha, self.window = alpha, window
        self.values: dict[int, float] = {}
        self._pending: dict[int, list[float]] = {}

    def observe(self, capacity: int, ms: float) -> None:
        if capacity <= 0 or not isfinite(ms) or ms <= 0:
            return
        if capacity not in self.values:
            self.values[capacity] = ms
            return
        buf = self._pending.setdefault(capacity, [])
        buf.append(ms)
        if len(buf) >= self.window:
            med = sorted(buf)[len(buf) // 2]
            self.values[capacity] += self.alpha * (med - self.values[capacity])
            buf.clear()

    def estimate(self, capacity: int) -> float | None:
        if not self.values:
            return None
        if capacity in self.values:
            return self.values[capacity]
        pts = sorted(self.values.items())
        lo = max((p for p in pts if p[0] < capacity), default=None)
        hi = min((p for p in pts if p[0] > capacity), default=None)
        if lo and hi:
            f = (capacity - lo[0]) / (hi[0] - lo[0])
            return lo[1] + f * (hi[1] - lo[1])
        if hi:
            return hi[1]           # small batches are bandwidth-bound: do not extrapolate savings downwards
        return lo[1] * capacity / lo[0]


@dataclass
class PlannedDraft:
    request_id: str
    draft_tokens: int
    decision: DraftDecision | None = None


class DraftPlanner:
    """Chooses each request's draft length for the next round from acceptance history and measured step costs."""

    def __init__(self, graph_capacities: tuple[int, ...], config: DraftPolicyConfig | None = None) -> None:
        self.caps = tuple(sorted(graph_capacities))
        self.cfg = config or DraftPolicyConfig()
        a, w = self.cfg.cost_ema_alpha, self.cfg.cost_sample_window
        self.target_cost = CostCurve(a, w)       # review pass, indexed by padded review rows
        self.proposal_cost = CostCurve(a, w)     # one MTP proposal pass, indexed by padded request rows
        self.overhead_ms = 0.0

    def bucket(self, rows: int) -> int:
        return next((c for c in self.caps if c >= rows), self.caps[-1])

    def observe_round(self, review_rows: int, target_ms: float, request_rows: int, proposal_ms: float, depth: int) -> None:
        self.target_cost.observe(self.bucket(review_rows), target_ms)
        if depth > 0:
            self.proposal_cost.observe(self.bucket(request_rows), proposal_ms / depth)

    def round_cost(self, rows_by_k: dict[int, int]) -> float | None:
        """Cost of one round in which ``rows_by_k[k]`` requests draft k tokens."""
        n = sum(rows_by_k.values())
        review = sum(cnt * (k + 1) for k, cnt in rows_by_k.items())
        t = self.target_cost.estimate(self.bucket(review))
        if t is None:
            return None
        depth = max((k for k, c in rows_by_k.items() if c), default=0)
        p = self.proposal_cost.estimate(self.bucket(n)) or 0.0
        return t + depth * p + self.overhead_ms

    def best_uniform_k(self, states: list[RequestDraftState], max_k: int) -> int:
        """The single K that maximises expected tokens per millisecond for this cohort (cold start: keep max)."""
        best_k, best_rate = None, -1.0
        for k in range(0, max_k + 1):
            cost = self.round_cost({k: len(states)})
            if cost is None:
                return max_k
            rate = sum(s.expected_tokens(k) for s in states) / cost
            # K0 is terminal: it must beat the best drafting choice by the stop margin
            if k == 0:
                rate /= 1.0 + self.cfg.terminal_stop_margin
            if rate > best_rate:
                best_k, best_rate = k, rate
        return best_k if best_k is not None else max_k

    def plan(self, requests: dict[str, RequestDraftState]) -> list[PlannedDraft]:
        """One-level moves toward the cohort optimum for the requests that reached a decision boundary."""
        active = {rid: s for rid, s in requests.items() if not s.stopped}
        out = [PlannedDraft(rid, 0) for rid, s in requests.items() if s.stopped]
        if not active:
            return out
        max_k = max(s.max_tokens for s in active.values())
        target = self.best_uniform_k(list(active.values()), max_k)
        for rid, s in active.items():
            dec = s.move_toward(min(target, s.max_tokens)) if s.ready else None
            out.append(PlannedDraft(rid, s.current_tokens, dec))
        return out
