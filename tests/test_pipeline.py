"""Pipeline-parallel plumbing: lane split, stage neighbours, gloo transport, and (on >= 2 GPUs) PP2 == PP1 tokens."""
import datetime
import json
import multiprocessing as mp
import os
import socket
import subprocess
import sys

import pytest
import torch

from cubic_serve_b200.contracts.execution import ParallelTopology
from cubic_serve_b200.parallel.pp import PipelineStage, split_lanes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_split_lanes_covers_rows_once_and_aligns():
    for t in (32, 48, 64, 100, 256, 512):
        lanes = split_lanes(t, t)
        assert lanes[0][0] == 0 and lanes[-1][1] == t
        for a, b in zip(lanes, lanes[1:]):
            assert a[1] == b[0] and a[3] == b[2]
            assert a[1] % 16 == 0
        assert all(l[0] == l[2] and l[1] == l[3] for l in lanes)
        assert len(lanes) == 2


def test_split_lanes_single_lane_cases():
    assert split_lanes(8, 8) == [(0, 8, 0, 8)]                # too few rows to be worth a second lane
    assert split_lanes(4096, 16) == [(0, 4096, 0, 16)]        # prefill: row blocks are not single rows
    assert split_lanes(256, 256, lanes=1) == [(0, 256, 0, 256)]


def test_stage_neighbours_tp2_pp2():
    topo = ParallelTopology.single_node(range(4), tp=2, pp=2)
    s = [PipelineStage.from_topology(topo, r) for r in range(4)]
    assert [x.stage for x in s] == [0, 0, 1, 1]
    assert [x.next_rank for x in s] == [2, 3, None, None]
    assert [x.prev_rank for x in s] == [None, None, 0, 1]
    assert all(x.sampler_rank == 2 for x in s)
    assert s[0].is_first and not s[0].is_last and s[3].is_last
    assert topo.layer_range(0, 36) == (0, 18) and topo.layer_range(1, 36) == (18, 36)
    assert topo.layer_range(1, 5) == (3, 5)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_stage(rank, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=30))
    topo = ParallelTopology.single_node(range(2), tp=1, pp=2)
    st = PipelineStage.from_topology(topo, rank, dist.group.WORLD)
    h = torch.zeros(64, 8)
    ids = torch.zeros(64, dtype=torch.int32)
    for t0, t1, _, _ in split_lanes(64, 64):
        if not st.is_first:
            st.recv(h[t0:t1])
        h[t0:t1] += (rank + 1) * torch.arange(t0, t1, dtype=torch.float32)[:, None]   # this stage's "layers"
        if not st.is_last:
            st.send(h[t0:t1])
    if st.is_last:
        ids.copy_(h[:, 0].to(torch.int32))
    st.share_token_ids(ids)
    q.put((rank, ids.tolist()))
    dist.destroy_process_group()


def test_two_stage_wavefront_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_stage, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    want = [3 * i for i in range(64)]                         # stage 0 adds i, stage 1 adds 2i
    assert got[0] == want and got[1] == want


@pytest.mark.gpu
def test_pp2_tokens_match_single_gpu():
    """Two pipeline stages on two GPUs must emit exactly the tokens of the one-GPU run (same kernels, same order)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    one = subprocess.run([sys.executable, "-m", "cubic_serve_b200.parallel.pp_check"], env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert one.returncode == 0, one.stderr[-2000:]
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m",
                          "cubic_serve_b200.parallel.pp_check", "--pp", "2"],
                         env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert two.returncode == 0, two.stderr[-2000:]
    a = json.loads(one.stdout.strip().splitlines()[-1])
    b = json.loads(two.stdout.strip().splitlines()[-1])
    assert a["tokens"] == b["tokens"]
