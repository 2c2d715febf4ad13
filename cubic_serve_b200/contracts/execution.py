"""Execution contracts: parallel topology, process groups, graph buckets and launch plans.

Same role as the reference's ``contracts/execution.py``: ``ParallelTopology.single_node`` (``:265`` there;
rank = stage * TP + tensor_rank, groups ``tp:`` / ``pp:`` / ``ep:`` / ``etp:``), expert ownership
(owner = tensor_rank // ETP, shard lane = tensor_rank % ETP, ``:238-248``), and the graph-bucket padding rules
(``GraphBucket`` / ``LaunchPlan`` ``:784-942``): a launch pads the live rows up to a captured capacity with rows
that write nothing and read nothing.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field


class GroupKind(str, enum.Enum):
    TENSOR = "tp"
    PIPELINE = "pp"
    EXPERT = "ep"
    EXPERT_TENSOR = "etp"


@dataclass(frozen=True)
class ProcessGroupSpec:
    name: str                # e.g. "tp:0" (stage 0), "pp:3" (tensor rank 3), "ep:0:1" (stage 0, shard lane 1)
    kind: GroupKind
    ranks: tuple[int, ...]


@dataclass(frozen=True)
class RankPlacement:
    rank: int
    device: int
    stage: int
    tensor_rank: int
    expert_rank: int         # which expert-parallel shard this rank owns
    expert_tensor_rank: int  # lane inside the expert-tensor group


@dataclass(frozen=True)
class ParallelTopology:
    tp: int
    pp: int
    ep: int
    devices: tuple[int, ...]
    placements: tuple[RankPlacement, ...]
    groups: tuple[ProcessGroupSpec, ...]

    @property
    def world_size(self) -> int:
        return self.tp * self.pp

    @property
    def etp(self) -> int:
        return self.tp // self.ep

    @staticmethod
    def single_node(devices, tp: int, pp: int = 1, ep: int = 1) -> "ParallelTopology":
        devices = tuple(devices)
        if tp < 1 or pp < 1 or ep < 1:
            raise ValueError("parallel sizes must be positive")
        if pp not in (1, 2):
            raise ValueError("pipeline parallelism supports 1 or 2 stages")
        if tp % ep:
            raise ValueError("expert parallel size must divide tensor parallel size")
        if len(devices) != tp * pp or len(set(devices)) != len(devices):
            raise ValueError("need exactly tp * pp distinct devices")
        etp = tp // ep
        placements = []
        for stage in range(pp):
            for t in range(tp):
                r = stage * tp + t
                placements.append(RankPlacement(r, devices[r], stage, t, t // etp, t % etp))
        groups = []
        for stage in range(pp):
            base = stage * tp
            groups.append(ProcessGroupSpec(f"tp:{stage}", GroupKind.TENSOR, tuple(range(base, base + tp))))
            for lane in range(etp):
                groups.append(ProcessGroupSpec(f"ep:{stage}:{lane}", GroupKind.EXPERT,
                                               tuple(base + e * etp + lane for e in range(ep))))
            for e in range(ep):
                groups.append(ProcessGroupSpec(f"etp:{stage}:{e}", GroupKind.EXPERT_TENSOR,
                                               tuple(base + e * etp + lane for lane in range(etp))))
        for t in range(tp):
            groups.append(ProcessGroupSpec(f"pp:{t}", GroupKind.PIPELINE, tuple(s * tp + t for s in range(pp))))
        return ParallelTopology(tp, pp, ep, devices, tuple(placements), tuple(groups))

    def placement(self, rank: int) -> RankPlacement:
        return self.placements[rank]

    def groups_of(self, rank: int) -> tuple[ProcessGroupSpec, ...]:
        return tuple(g for g in self.groups if rank in g.ranks)

    @property
    def sampler_rank(self) -> int:
        """First rank of the last stage samples and reports tokens (reference: ``quantized_graph.py:1557``)."""
        return (self.pp - 1) * self.tp

    def expert_slice(self, rank: int, num_experts: int) -> tuple[int, int]:
        """Contiguous expert ids ``[lo, hi)`` owned by the rank's expert shard."""
        if num_experts % self.ep:
            raise ValueError("experts must divide evenly over the expert-parallel size")
        per = num_experts // self.ep
        e = self.placements[rank].expert_rank
        return e * per, (e + 1) * per

    def expert_feature_slice(self, rank: int, intermediate: int) -> tuple[int, int]:
        """Intermediate features ``[lo, hi)`` of every owned expert that the rank's lane holds (the lanes of one expert
        owner divide each expert's gate / up rows and down columns)."""
        if intermediate % self.etp:
            raise ValueError("expert features must divide evenly over the expert-tensor lanes")
        per = intermediate // self.etp
        lane = self.placements[rank].expert_tensor_rank
        return lane * per, (lane + 1) * per

    def layer_range(self, stage: int, num_layers: int) -> tuple[int, int]:
        per = -(-num_layers // self.pp)
        return stage * per, min(num_layers, (stage + 1) * per)


@dataclass(frozen=True)
class GraphBucket:
    """A captured CUDA graph that serves any launch of up to ``capacity`` rows of ``rows_per_request`` each."""
    capacity: int
    rows_per_request: int = 1

    def fits(self, live_rows: int) -> bool:
        return 0 < live_rows <= self.capacity


@dataclass(frozen=True)
class LaunchPlan:
    bucket: GraphBucket
    live_rows: int

    @property
    def padding_rows(self) -> int:
        return self.bucket.capacity - self.live_rows

    @staticmethod
    def choose(buckets, live_rows: int) -> "LaunchPlan":
        """Smallest bucket that fits (buckets are powers of two captured largest-first)."""
        fitting = [b for b in buckets if b.fits(live_rows)]
        if not fitting:
            raise ValueError(f"no graph bucket holds {live_rows} rows")
        return LaunchPlan(min(fitting, key=lambda b: b.capacity), live_rows)
