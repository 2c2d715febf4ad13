"""Controller <-> rank worker protocol with CPU stand-in workers (no GPU): readiness, results, liveness."""
import os
import signal
import time

import numpy as np
import pytest

from cubic_serve_b200.executor.gpu_executor import Segment
from cubic_serve_b200.executor.multiproc import MultiprocExecutor, WorkerFailure, WorkerSpec, describe_exit

SPEC = WorkerSpec("random:toy", [0, 1], 2, 8, 8, 8, 256, 128, 64)


def _fake_worker(rank, spec, port, conn):
    conn.send(("progress", rank, "up"))
    conn.send(("ready", rank, {"pages": 64, "capacities": [8], "vocab": 1024, "name": "toy"}))
    while True:
        cmd = conn.recv()
        if cmd[0] == "execute":
            if rank == 0:
                conn.send(("result", np.asarray([int(s.token_ids[-1]) + 1 for s in cmd[1] if s.sample], dtype=np.int32), 7))
        elif cmd[0] == "close":
            return


def _dying_worker(rank, spec, port, conn):
    conn.send(("ready", rank, {"pages": 64, "capacities": [8], "vocab": 1024, "name": "toy"}))
    cmd = conn.recv()
    if rank == 1:
        os.kill(os.getpid(), signal.SIGKILL)        # a rank vanishes between steps
    time.sleep(30)


def _failing_startup(rank, spec, port, conn):
    if rank == 1:
        conn.send(("error", rank, "ValueError: shard does not fit"))
        return
    conn.send(("ready", rank, {"pages": 64, "capacities": [8], "vocab": 1024, "name": "toy"}))
    time.sleep(5)


def test_protocol_roundtrip():
    ex = MultiprocExecutor(SPEC, worker_target=_fake_worker)
    assert ex.info["pages"] == 64
    out = ex.execute([Segment(0, [5], 3, [1]), Segment(1, [9], 3, [2], sample=False), Segment(2, [1], 0, [3])])
    assert out.tolist() == [6, 2] and ex.kernel_launches_last == 7
    ex.copy_pages([(1, 2)])
    ex.close()


def test_dead_rank_poisons_with_decoded_signal():
    ex = MultiprocExecutor(SPEC, worker_target=_dying_worker, result_timeout=20)
    with pytest.raises(WorkerFailure, match="rank 1 terminated by SIGKILL"):
        ex.execute([Segment(0, [5], 3, [1])])
    assert ex.poisoned
    with pytest.raises(WorkerFailure, match="poisoned"):
        ex.execute([Segment(0, [5], 3, [1])])
    ex.close()


def test_startup_error_is_reported():
    with pytest.raises(WorkerFailure, match="rank 1 failed during start-up: ValueError"):
        MultiprocExecutor(SPEC, worker_target=_failing_startup)


def test_exit_code_messages():
    assert "SIGSEGV" in describe_exit(-11) and "memory fault" in describe_exit(-11)
    assert "out-of-memory" in describe_exit(-9)
    assert describe_exit(3) == "exited with status 3" and describe_exit(0) == "exited normally"


def _hybrid_worker(rank, spec, port, conn):
    """A worker of a model with recurrent layers: announces snapshot rows and keeps a rolling state per row."""
    state = np.zeros(16, dtype=np.int64)
    conn.send(("ready", rank, {"pages": 64, "capacities": [8], "vocab": 1024, "name": "toy-hybrid", "hybrid": True,
                               "state_rows": [8, 9, 10, 11]}))
    while True:
        cmd = conn.recv()
        if cmd[0] == "execute":
            out = []
            for s in cmd[1]:
                st = 0 if s.start == 0 else int(state[s.request_slot])
                for t in s.token_ids:
                    st = (st * 31 + int(t) + 1) % 1_000_003
                state[s.request_slot] = st
                if s.sample:
                    out.append(st % 89)
            if rank == 0:
                conn.send(("result", np.asarray(out, dtype=np.int32), 3))
        elif cmd[0] == "copy_state":
            for a, b in cmd[1]:
                state[b] = state[a]
        elif cmd[0] == "close":
            return


def test_hybrid_workers_keep_prefix_caching_through_state_snapshots():
    """The controller keeps the prefix cache on for a model with recurrent layers when the workers announce snapshot
    rows, and drives snapshot / restore copies on every rank; a constrained request's segments cross the pipe."""
    from cubic_serve_b200.generation.constraints import ChoiceMatcher
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    ex = MultiprocExecutor(SPEC, worker_target=_hybrid_worker)
    assert ex.cfg.is_hybrid and ex.state_checkpoint_rows == (8, 9, 10, 11)
    eng = LLMEngine(ex, num_pages=64, scheduler_config=SchedulerConfig(max_running_requests=4, max_batched_tokens=64,
                                                                       prefill_chunk_tokens=32, max_model_len=256))
    assert eng.prefix.enabled and eng.prefix.needs_checkpoint
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, 1000, size=70)]
    first = [int(t) for t in eng.generate([prompt], SamplingParams(max_tokens=5))[0]]
    again = [int(t) for t in eng.generate([prompt], SamplingParams(max_tokens=5))[0]]
    assert again == first and eng.prefix.hit_tokens == 64

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [ord(c) % 80 for c in text]
    m = ChoiceMatcher(["ab", "cd"], Tok(), 3)
    rid = eng.add_request([5, 6, 7], SamplingParams(max_tokens=4, stop_token_ids=(3,), matcher=m))
    req = eng.requests[rid]
    for _ in range(3):                      # the segments carry a mask callback on the controller: it must not be pickled
        try:
            eng.step()
        except RuntimeError as exc:         # the stand-in worker samples without the mask: a violation is fine here
            assert "violates its constraint" in str(exc)
            break
    ex.close()
