"""Qualified graph runtime: slot states, dispatch, replay leases, poisoning, readiness (no CUDA: graphs are fakes)."""
import pytest

from cubic_serve_b200.executor.graph_runtime import (CudaGraphRuntime, GraphRuntimeError, GraphState, LeaseError,
                                                     ReplayLeasePool, execution_ready)


class FakeGraph:
    def __init__(self):
        self.replays = 0

    def replay(self):
        self.replays += 1


def _runtime(caps=(1, 16, 64, 256), bad=()):
    rt = CudaGraphRuntime(resources=(0, 1))
    for c in caps:
        rt.add(c, FakeGraph(), launches=100 + c)
        rt.qualify(c, lambda slot: slot.capacity not in bad)
    return rt


def test_capture_qualify_seal_dispatch():
    rt = _runtime(bad=(64,))
    assert rt.slots[64].state is GraphState.POISONED and rt.slots[16].state is GraphState.QUALIFIED
    with pytest.raises(GraphRuntimeError):
        rt.replay(16, rt.leases.acquire(0))                 # not sealed yet
    rt.leases.release_all()
    ready = rt.seal()
    assert ready.sealed == (1, 16, 256) and ready.poisoned == (64,) and ready.ready
    assert rt.dispatch(1) == 1 and rt.dispatch(2) == 16 and rt.dispatch(17) == 256      # 64 is out of service
    assert rt.dispatch(257) is None                                                    # eager
    with pytest.raises(GraphRuntimeError):
        rt.add(512, FakeGraph())                            # nothing is captured after the seal
    lease = rt.leases.acquire(0, "step 0")
    assert rt.replay(16, lease).launches == 116 and rt.slots[16].graph.replays == 1
    assert not rt.readiness().ready                         # a replay is outstanding
    rt.leases.release(lease)
    with pytest.raises(LeaseError):
        rt.replay(16, lease)                                # a released lease does not replay
    assert rt.stats()["slots"][64]["reason"] == "qualification failed"


def test_unqualified_slots_are_poisoned_at_seal_unless_qualification_is_off():
    rt = CudaGraphRuntime()
    rt.add(8, FakeGraph())
    rt.add(16, FakeGraph())
    rt.qualify(16, lambda s: True)
    assert rt.seal().sealed == (16,) and rt.slots[8].reason == "never qualified"
    loose = CudaGraphRuntime(require_qualification=False)
    loose.add(8, FakeGraph())
    assert loose.seal().sealed == (8,)


def test_qualification_verdicts():
    rt = CudaGraphRuntime()
    for c in (1, 2, 4):
        rt.add(c, FakeGraph())
    assert rt.qualify(1, lambda s: True)
    assert not rt.qualify(2, lambda s: "logits differ (relative L2 0.3)")
    assert not rt.qualify(4, lambda s: 1 / 0)
    assert rt.slots[2].reason == "qualification failed: logits differ (relative L2 0.3)"
    assert "ZeroDivisionError" in rt.slots[4].reason
    with pytest.raises(GraphRuntimeError):
        rt.qualify(1, lambda s: True)                       # already qualified


def test_leases_are_exclusive():
    pool = ReplayLeasePool((0, 1))
    a, b = pool.acquire(0, "launch 0"), pool.acquire(1, "launch 1")
    with pytest.raises(LeaseError, match="launch 0"):
        pool.acquire(0, "launch 2")                         # a third outstanding launch would overwrite a result buffer
    pool.release(a)
    c = pool.acquire(0, "launch 2")
    with pytest.raises(LeaseError):
        pool.release(a)                                     # stale lease
    assert {l.serial for l in pool.outstanding()} == {b.serial, c.serial}
    with pytest.raises(LeaseError):
        pool.acquire(7)
    pool.release_all()
    assert not pool.outstanding() and b.released


def test_poison_falls_back_and_is_permanent():
    rt = _runtime()
    rt.seal()
    rt.poison(16, "device status word set after a replay")
    assert rt.dispatch(8) == 64 and rt.readiness().poisoned == (16,)
    rt.poison(None, "engine poisoned")
    assert rt.dispatch(1) is None and len(rt.poison_log) == 4
    with pytest.raises(GraphRuntimeError):
        rt.replay(64, rt.leases.acquire(1))


def test_execution_ready_needs_a_sealed_idle_runtime():
    rt = _runtime((4,))
    with pytest.raises(GraphRuntimeError):
        execution_ready(rt.readiness())
    rt.seal()
    assert execution_ready(rt.readiness()) == {"graph_capacities": [4], "poisoned_capacities": [], "ready": True}
