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
