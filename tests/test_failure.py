"""Failure detection and fail-closed behaviour, exercised on the host (no GPU fault is ever provoked)."""
import asyncio
import json
import multiprocessing as mp
import os
import time

import numpy as np
import pytest
import torch

from cubic_serve_b200.runtime.engine import EnginePoisoned, LLMEngine
from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig


class FlakyExecutor:
    def __init__(self, fail_at):
        self.calls, self.fail_at = 0, fail_at

    def copy_pages(self, pairs):
        pass

    def execute(self, segs):
        self.calls += 1
        if self.calls == self.fail_at:
            raise RuntimeError("injected executor failure")
        return np.asarray([1 for s in segs if s.sample], dtype=np.int32)


def test_engine_poisons_itself_and_pool_on_step_failure():
    eng = LLMEngine(FlakyExecutor(fail_at=3), 32, SchedulerConfig(max_running_requests=4, max_model_len=64))
    eng.add_request([1, 2, 3], SamplingParams(max_tokens=10))
    eng.step(); eng.step()
    with pytest.raises(RuntimeError, match="injected"):
        eng.step()
    assert eng.poisoned
    with pytest.raises(EnginePoisoned):
        eng.step()
    with pytest.raises(EnginePoisoned):
        eng.add_request([1])


def test_backend_fails_closed_streams_get_5xx_and_health_turns_503():
    from cubic_serve_b200.api.server import CubicASGIApp
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.runtime.async_engine import TokenChatBackend
    from tests.test_api import _call
    eng = LLMEngine(FlakyExecutor(fail_at=2), 64, SchedulerConfig(max_running_requests=4, max_model_len=256))

    async def go():
        backend = TokenChatBackend(eng, ByteTokenizer())
        app = CubicASGIApp(backend, "m")
        body = {"model": "m", "messages": [{"role": "user", "content": "x"}], "max_tokens": 20, "stream": True}
        st, payload = await _call(app, "POST", "/v1/chat/completions", body)
        health = await _call(app, "GET", "/health")
        late = await _call(app, "POST", "/v1/chat/completions", {**body, "stream": False})
        return st, payload, health, late

    st, payload, health, late = asyncio.run(go())
    assert st == 200 and b"generation failed" in payload and b"injected" not in payload   # public message only
    assert health[0] == 503 and late[0] == 503


def _rank(rank, world, port, die_at, q):
    """A CPU rank of a 2-rank gloo job; rank 1 leaves between steps, rank 0 must notice on the host."""
    import datetime

    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    store = dist.distributed_c10d._get_default_store()
    try:
        for step in range(6):
            if rank == 1 and step == die_at:
                store.set("left:1", str(step))          # announces its exit between steps, nothing in flight
                q.put((rank, "left", step))
                return
            # heartbeat check on the host BEFORE the next collective is launched
            if rank == 0 and store.check(["left:1"]):
                q.put((rank, "peer_left_detected", step))
                return
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            time.sleep(0.05)
        q.put((rank, "finished", 6))
    except Exception as exc:  # a collective that outlives its peer ends with the group timeout
        q.put((rank, "collective_error", type(exc).__name__))


def test_rank_departure_is_detected_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_rank, args=(r, 2, port, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
    events = {}
    while not q.empty():
        r, what, step = q.get()
        events[r] = (what, step)
    assert events[1] == ("left", 2)
    assert events[0][0] in ("peer_left_detected", "collective_error")
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.gpu
def test_bounded_device_wait_reports_status_and_context_survives():
    """A wait on a flag that nothing raises runs out after its budget; the host reads the status word."""
    from cubic_serve_b200.ops import kernels as K, native
    dev = torch.device("cuda")
    ws = K.workspace(dev)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    t0 = time.time()
    native.check(native.lib().cb_tp_wait(flags.data_ptr(), state.data_ptr(), 1, 2, ws.status.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream), "cb_tp_wait")
    torch.cuda.synchronize()
    assert time.time() - t0 < 10
    with pytest.raises(native.NativeLibraryError, match="status 2"):
        ws.check_status()
    # the context is still usable and the status word was cleared
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
    ws.check_status()
