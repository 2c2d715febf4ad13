"""Declared collective schedules of a partitioned decoder step, and the checks that make them a proof of progress.

A rank of a tensor x pipeline partition issues a fixed sequence of communication calls per step; the sequence depends
only on the model's layer structure and the rank's place in the topology.  ``decoder_step_schedule`` states it; two
checks then hold for every correct partition and fail for the usual ways of getting one wrong:

* **group agreement**: all members of a process group issue the same collectives on that group, in the same order,
  with the same element counts.  Collectives on one communicator execute in issue order, so agreement on the order
  is what rules out a deadlock inside a group;
* **pipeline matching**: every ``send`` has a ``recv`` of the same size on the peer, and, walking all ranks' schedules
  together (a rank can only pass a blocking call when its partners have reached theirs), the step runs to the end.

``record_collectives`` wraps ``torch.distributed`` so that a real run (gloo on CPU, NCCL on GPUs) can be compared
with the declaration: the eager partitioned decoder is checked that way in the tests.

Reference counterpart: ``contracts/execution.py:358-412`` (``PartitionPlan`` with ordered ``CollectiveStep``s) and
``guardrail/quantized_graph/collective.py`` (collective-order audit) there.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass

from ..contracts.execution import GroupKind, ParallelTopology


@dataclass(frozen=True)
class CollectiveStep:
    kind: str            # all_reduce | all_gather | send | recv | broadcast
    group: str           # process-group id of the topology, or "p2p:<src>-><dst>" for pipeline transfers, or "world"
    elements: int        # elements this rank contributes (all_reduce, all_gather, broadcast) or transfers (send / recv)
    site: str            # where in the step: "layer 3 attention", "logits", "stage hand-over", "token"


def _group_of(topo: ParallelTopology, rank: int, kind: GroupKind) -> str:
    return next(g.name for g in topo.groups_of(rank) if g.kind is kind)


def decoder_step_schedule(cfg, topo: ParallelTopology, rank: int, rows: int, feed_token_back: bool = True) -> tuple:
    """The communication calls of one step of ``rows`` token rows on ``rank``, in issue order: a stage receives the
    residual stream from the stage before it, runs its layers (two sums over the tensor group per layer: after the
    attention output projection and after the feed-forward), hands the stream on or, on the last stage, gathers the
    vocabulary shards of the logits; with more than one stage the sampled token goes back to everybody."""
    p = topo.placement(rank)
    lo, hi = topo.layer_range(p.stage, cfg.num_layers)
    steps: list[CollectiveStep] = []
    H = cfg.hidden_size
    if p.stage > 0:
        steps.append(CollectiveStep("recv", f"p2p:{rank - topo.tp}->{rank}", rows * H, "stage hand-over"))
    if topo.tp > 1:
        tg = _group_of(topo, rank, GroupKind.TENSOR)
        for layer in range(lo, hi):
            steps.append(CollectiveStep("all_reduce", tg, rows * H, f"layer {layer} attention"))
            steps.append(CollectiveStep("all_reduce", tg, rows * H, f"layer {layer} feed-forward"))
    if p.stage < topo.pp - 1:
        steps.append(CollectiveStep("send", f"p2p:{rank}->{rank + topo.tp}", rows * H, "stage hand-over"))
    elif topo.tp > 1:
        steps.append(CollectiveStep("all_gather", _group_of(topo, rank, GroupKind.TENSOR), rows * cfg.vocab_size // topo.tp,
                                    "logits"))
    if topo.pp > 1 and feed_token_back:
        steps.append(CollectiveStep("broadcast", "world", 1, "token"))
    return tuple(steps)


def check_schedules(topo: ParallelTopology, schedules: dict[int, tuple]) -> list[str]:
    """Problems of a set of per-rank schedules (empty = the step is proven to run to its end)."""
    problems: list[str] = []
    if sorted(schedules) != list(range(topo.world_size)):
        return ["a schedule is needed for every rank of the topology"]
    members = {g.name: tuple(g.ranks) for g in topo.groups}
    members["world"] = tuple(range(topo.world_size))
    # group agreement
    for gid, ranks in members.items():
        views = {r: [(s.kind, s.elements) for s in schedules[r] if s.group == gid] for r in ranks}
        first = views[ranks[0]]
        for r in ranks[1:]:
            if views[r] != first:
                at = next((i for i, (a, b) in enumerate(zip(views[r], first)) if a != b), min(len(views[r]), len(first)))
                problems.append(f"group {gid}: rank {r} and rank {ranks[0]} differ at their call {at} on this group")
    # pipeline matching: every transfer has both ends and the same size
    sends = {(s.group, s.elements) for sch in schedules.values() for s in sch if s.kind == "send"}
    recvs = {(s.group, s.elements) for sch in schedules.values() for s in sch if s.kind == "recv"}
    for gid, n in sorted(sends ^ recvs):
        problems.append(f"transfer {gid} of {n} elements has one end only")
    if problems:
        return problems
    # progress: advance every rank as far as its partners allow; all schedules must be consumed
    at = {r: 0 for r in schedules}
    moved = True
    while moved:
        moved = False
        for r, sch in schedules.items():
            if at[r] >= len(sch):
                continue
            s = sch[at[r]]
            if s.kind in ("send", "recv"):
                src, dst = (int(v) for v in s.group[4:].split("->"))
                peer = dst if s.kind == "send" else src
                want = "recv" if s.kind == "send" else "send"
                ps = schedules[peer][at[peer]] if at[peer] < len(schedules[peer]) else None
                ready = ps is not None and ps.kind == want and ps.group == s.group
                partners = (r, peer) if ready else ()
            else:
                grp = members[s.group]
                ready = all(at[m] < len(schedules[m]) and schedules[m][at[m]].group == s.group
                            and schedules[m][at[m]].kind == s.kind for m in grp)
                partners = grp if ready else ()
            for m in partners:
                at[m] += 1
            moved = moved or bool(partners)
    stuck = {r: sch[at[r]].site for r, sch in schedules.items() if at[r] < len(sch)}
    if stuck:
        problems.append(f"the step cannot finish: ranks wait at {stuck}")
    return problems


@contextmanager
def record_collectives(log: list):
    """Record ``(kind, elements)`` of this process's ``torch.distributed`` calls into ``log`` while the block runs."""
    import torch.distributed as dist
    names = {"all_reduce": 0, "all_gather": 1, "send": 0, "recv": 0, "broadcast": 0}
    originals = {n: getattr(dist, n) for n in names}

    def wrap(name, tensor_arg):
        fn = originals[name]

        def inner(*a, **kw):
            log.append((name, int(a[tensor_arg].numel())))
            return fn(*a, **kw)
        return inner
    try:
        for n, idx in names.items():
            setattr(dist, n, wrap(n, idx))
        yield log
    finally:
        for n, fn in originals.items():
            setattr(dist, n, fn)
