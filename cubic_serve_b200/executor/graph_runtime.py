"""Qualified CUDA-graph runtime: capture -> qualify -> seal -> replay, with replay leases and poisoning.

A captured graph replays fixed kernels on fixed addresses, so three things can go wrong that an eager launch cannot
show: the capture differs from the eager execution it was recorded from (a kernel that reads host state at launch
time), two replays overlap on the same fixed-address result buffer, or a graph keeps being replayed after one of its
replays reported a device-side error.  The runtime makes each of them a checked state:

* a slot is ``CAPTURED`` until ``qualify`` compared one replay with the eager run of the same inputs (the caller
  supplies the comparison); a slot that fails is ``POISONED`` and never dispatched;
* ``seal`` closes the set: afterwards nothing is captured (serving never captures), and only ``SEALED`` slots replay;
* every replay needs a ``ReplayLease`` on the resource it writes (a result buffer); a resource has one holder at a
  time, a second ``acquire`` is an error instead of a silent overwrite;
* ``poison`` takes a slot (or all) out of service for good; dispatch falls back to the next larger sealed capacity
  and finally to eager execution (``None``).

``readiness`` is the seal a rank reports before serving: which capacities are sealed, which are poisoned; all ranks of
a deployment must report the same (``runtime.preparation.consensus``).  Nothing here touches CUDA: a graph is any
object with ``replay()``, which is what the CPU tests use.

Reference counterpart: ``executor/cuda_graph.py:332`` (``CudaGraphRuntime``), ``:771`` (decode dispatcher),
``executor/replay_lease.py:33`` (``ReplayLeasePool``), ``executor/readiness.py:15`` (``execution_ready``).
"""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass, field
from typing import Callable, Hashable


class GraphRuntimeError(RuntimeError):
    pass


class LeaseError(GraphRuntimeError):
    pass


class GraphState(enum.Enum):
    CAPTURED = "captured"
    QUALIFIED = "qualified"
    SEALED = "sealed"
    POISONED = "poisoned"


@dataclass
class GraphSlot:
    capacity: int
    graph: object
    launches: int = 0                 # kernels inside one replay (accounting)
    state: GraphState = GraphState.CAPTURED
    replays: int = 0
    reason: str | None = None         # why it was poisoned


@dataclass
class ReplayLease:
    resource: Hashable
    holder: str
    serial: int
    released: bool = False


class ReplayLeasePool:
    """Exclusive leases on named resources (result buffers, staging areas).  Thread-safe."""

    def __init__(self, resources) -> None:
        self._lock = threading.Lock()
        self._held: dict[Hashable, ReplayLease | None] = {r: None for r in resources}
        self._serial = 0

    def acquire(self, resource: Hashable, holder: str = "") -> ReplayLease:
        with self._lock:
            if resource not in self._held:
                raise LeaseError(f"unknown resource {resource!r}")
            cur = self._held[resource]
            if cur is not None:
                raise LeaseError(f"resource {resource!r} is still leased to {cur.holder!r} (lease {cur.serial}); "
                                 f"its result has not been collected")
            self._serial += 1
            lease = ReplayLease(resource, holder, self._serial)
            self._held[resource] = lease
            return lease

    def release(self, lease: ReplayLease) -> None:
        with self._lock:
            if lease.released or self._held.get(lease.resource) is not lease:
                raise LeaseError(f"lease {lease.serial} on {lease.resource!r} is not current")
            lease.released = True
            self._held[lease.resource] = None

    def outstanding(self) -> list[ReplayLease]:
        with self._lock:
            return [l for l in self._held.values() if l is not None]

    def release_all(self) -> None:
        """After a failure: nothing in flight will be collected any more."""
        with self._lock:
            for r, l in self._held.items():
                if l is not None:
                    l.released = True
                    self._held[r] = None


@dataclass
class Readiness:
    sealed: tuple[int, ...]
    poisoned: tuple[int, ...]
    ready: bool

    def as_dict(self) -> dict:
        return {"graph_capacities": list(self.sealed), "poisoned_capacities": list(self.poisoned), "ready": self.ready}


class CudaGraphRuntime:
    def __init__(self, resources=(0, 1), require_qualification: bool = True) -> None:
        self.slots: dict[int, GraphSlot] = {}
        self.leases = ReplayLeasePool(resources)
        self.require_qualification = require_qualification
        self.sealed = False
        self.poison_log: list[tuple[int, str]] = []

    # ------------------------------------------------------------------ start-up
    def add(self, capacity: int, graph, launches: int = 0) -> GraphSlot:
        if self.sealed:
            raise GraphRuntimeError("the graph set is sealed: nothing is captured while serving")
        if capacity in self.slots:
            raise GraphRuntimeError(f"a graph for capacity {capacity} exists already")
        slot = self.slots[capacity] = GraphSlot(capacity, graph, launches)
        return slot

    def qualify(self, capacity: int, check: Callable[[GraphSlot], bool | str]) -> bool:
        """Run the caller's comparison for a captured slot.  ``check`` replays the graph on known inputs and returns
        True when the result equals the eager run's, else False or a description of the difference."""
        slot = self.slots[capacity]
        if slot.state is not GraphState.CAPTURED:
            raise GraphRuntimeError(f"capacity {capacity} is {slot.state.value}, not captured")
        try:
            verdict = check(slot)
        except Exception as exc:  # noqa: BLE001 - a check that cannot run does not qualify the slot
            verdict = f"{type(exc).__name__}: {exc}"
        if verdict is True:
            slot.state = GraphState.QUALIFIED
            return True
        self.poison(capacity, "qualification failed" if verdict is False else f"qualification failed: {verdict}")
        return False

    def seal(self) -> Readiness:
        for slot in self.slots.values():
            if slot.state is GraphState.QUALIFIED or (slot.state is GraphState.CAPTURED and not self.require_qualification):
                slot.state = GraphState.SEALED
            elif slot.state is GraphState.CAPTURED:
                self.poison(slot.capacity, "never qualified")
        self.sealed = True
        return self.readiness()

    def readiness(self) -> Readiness:
        sealed = tuple(sorted(c for c, s in self.slots.items() if s.state is GraphState.SEALED))
        poisoned = tuple(sorted(c for c, s in self.slots.items() if s.state is GraphState.POISONED))
        return Readiness(sealed, poisoned, self.sealed and not self.leases.outstanding())

    # ------------------------------------------------------------------ serving
    def dispatch(self, rows: int) -> int | None:
        """Smallest sealed capacity that holds ``rows``; None = run eagerly."""
        best = None
        for c, s in self.slots.items():
            if c >= rows and s.state is GraphState.SEALED and (best is None or c < best):
                best = c
        return best

    def replay(self, capacity: int, lease: ReplayLease) -> GraphSlot:
        slot = self.slots[capacity]
        if slot.state is not GraphState.SEALED:
            raise GraphRuntimeError(f"capacity {capacity} is {slot.state.value}: only sealed graphs replay")
        if lease.released:
            raise LeaseError(f"lease {lease.serial} was released already")
        slot.graph.replay()
        slot.replays += 1
        return slot

    def poison(self, capacity: int | None, reason: str) -> None:
        """Take one slot (or, with None, every slot) out of service for good."""
        for c in ([capacity] if capacity is not None else list(self.slots)):
            slot = self.slots[c]
            if slot.state is not GraphState.POISONED:
                slot.state, slot.reason = GraphState.POISONED, reason
                self.poison_log.append((c, reason))

    def stats(self) -> dict:
        return {"sealed": self.sealed, "slots": {c: {"state": s.state.value, "replays": s.replays, "launches": s.launches,
                                                     **({"reason": s.reason} if s.reason else {})}
                                                 for c, s in sorted(self.slots.items())}}


def execution_ready(local: Readiness, group=None) -> dict:
    """The readiness seal of a deployment: every rank reports its sealed and poisoned capacities; they must be equal
    (a rank that poisoned a capacity the others replay would desynchronise the collectives inside the graphs)."""
    from ..runtime.preparation import consensus
    if not local.ready:
        raise GraphRuntimeError("this rank is not ready: the graph set is not sealed or a replay is outstanding")
    return consensus(local.as_dict(), group=group)
