"""Declared collective schedules: group agreement, pipeline matching and progress; the eager partitioned decoder issues
exactly the declared calls (gloo)."""
import datetime
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from cubic_serve_b200.contracts.execution import ParallelTopology
from cubic_serve_b200.guardrail.collective_schedule import CollectiveStep, check_schedules, decoder_step_schedule
from cubic_serve_b200.models.config import ModelConfig, QuantSpec


def _cfg():
    return ModelConfig(name="dist-toy", num_layers=4, hidden_size=64, num_q_heads=4, num_kv_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=128, rope_theta=1e4, qk_norm=True, quant=QuantSpec("none", 16, 0))


@pytest.mark.parametrize("tp,pp", [(1, 1), (2, 1), (4, 1), (1, 2), (2, 2), (4, 2)])
def test_declared_schedules_prove_progress(tp, pp):
    cfg = _cfg()
    topo = ParallelTopology.single_node(range(tp * pp), tp=tp, pp=pp)
    sch = {r: decoder_step_schedule(cfg, topo, r, rows=10) for r in range(tp * pp)}
    assert check_schedules(topo, sch) == []
    n_reduce = sum(s.kind == "all_reduce" for s in sch[0])
    assert n_reduce == (0 if tp == 1 else 2 * cfg.num_layers // pp)
    if pp == 2:
        assert sch[0][-2].kind == "send" and sch[tp][0].kind == "recv" and sch[0][-1].kind == "broadcast"


def test_wrong_schedules_are_named():
    cfg = _cfg()
    topo = ParallelTopology.single_node(range(4), tp=2, pp=2)
    good = {r: decoder_step_schedule(cfg, topo, r, rows=10) for r in range(4)}
    # a rank that skips one sum
    bad = dict(good)
    bad[1] = tuple(s for i, s in enumerate(good[1]) if i != 2)
    assert any("group tp:0" in p for p in check_schedules(topo, bad))
    # a rank that sums another number of rows
    bad = dict(good)
    bad[3] = tuple(CollectiveStep(s.kind, s.group, s.elements + 1, s.site) if s.kind == "all_reduce" else s for s in good[3])
    assert any("group tp:1" in p for p in check_schedules(topo, bad))
    # a stage that never hands over
    bad = dict(good)
    bad[0] = tuple(s for s in good[0] if s.kind != "send")
    assert any("one end only" in p for p in check_schedules(topo, bad))
    # the classic cycle: both stages receive before they send
    a = (CollectiveStep("recv", "p2p:1->0", 5, "x"), CollectiveStep("send", "p2p:0->1", 5, "x"))
    b = (CollectiveStep("recv", "p2p:0->1", 5, "x"), CollectiveStep("send", "p2p:1->0", 5, "x"))
    topo2 = ParallelTopology.single_node(range(2), tp=1, pp=2)
    assert any("cannot finish" in p for p in check_schedules(topo2, {0: a, 1: b}))
    assert check_schedules(topo2, {0: a}) == ["a schedule is needed for every rank of the topology"]


def _rank(rank, world, tp, pp, port, q):
    import torch.distributed as dist

    from cubic_serve_b200.guardrail.collective_schedule import record_collectives
    from cubic_serve_b200.models.distributed_reference import DistributedEagerDecoder
    from cubic_serve_b200.models.parallel_weights import plan_partition
    from cubic_serve_b200.models.reference import random_dense_weights
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    torch.set_num_threads(1)
    cfg = _cfg()
    groups = [dist.new_group(list(range(s * tp, (s + 1) * tp))) for s in range(pp)]
    dec = DistributedEagerDecoder(cfg, plan_partition(cfg, tp, pp), rank, random_dense_weights(cfg, seed=5, std=0.08),
                                  groups[rank // tp])
    log = []
    with record_collectives(log):
        dec.forward(torch.tensor([[3, 17, 99, 4, 56], [8, 8, 120, 33, 2]]), 0, None)
    q.put((rank, log))
    dist.barrier()
    dist.destroy_process_group()


def test_the_eager_partition_issues_the_declared_calls():
    tp, pp = 2, 2
    world = tp * pp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, tp, pp, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    logs = dict(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    cfg = _cfg()
    topo = ParallelTopology.single_node(range(world), tp=tp, pp=pp)
    for r in range(world):
        declared = decoder_step_schedule(cfg, topo, r, rows=10, feed_token_back=False)
        # the eager reference sums in rank order after an all-gather of the partial rows: a declared sum is recorded as
        # a gather of the same number of elements
        want = [("all_gather" if s.kind == "all_reduce" else s.kind, s.elements) for s in declared]
        assert logs[r] == want, r
