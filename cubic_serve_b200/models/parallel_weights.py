"""Ownership of weights under tensor / pipeline / expert parallelism, as data.

``plan_partition`` answers, before any process is spawned or any tensor is read: can this model be split this way
(heads, feature dimensions and experts divide, shards keep the alignment the kernels need), which rows or columns of
every logical weight does each rank own, and how many bytes of weights does it hold.  The loaders slice checkpoints
with the same spans (``AxisSpan.shard``); ``cubic inspect-model --tp N --pp M`` prints the per-rank totals and
``executor.multiproc`` refuses an impossible split with the planner's message instead of a shape error in a worker.

Reference counterpart: ``models/parallel_weights.py:72,196,266`` (``AxisSpan``, rank-local slicing, expert slices) and
the TP / PP / EP ownership planners of the model packages.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .config import ModelConfig


class PartitionError(ValueError):
    pass


@dataclass(frozen=True)
class AxisSpan:
    """Half-open range ``[start, stop)`` of an axis of length ``total``."""
    start: int
    stop: int
    total: int

    def __post_init__(self) -> None:
        if not 0 <= self.start <= self.stop <= self.total:
            raise PartitionError(f"span [{self.start}, {self.stop}) does not lie in an axis of {self.total}")

    @property
    def size(self) -> int:
        return self.stop - self.start

    @property
    def full(self) -> bool:
        return self.start == 0 and self.stop == self.total

    def slice(self) -> slice:
        return slice(self.start, self.stop)

    def scaled(self, factor: int) -> "AxisSpan":
        """The same share of an axis ``factor`` times as long (heads -> rows of ``head_dim`` each)."""
        return AxisSpan(self.start * factor, self.stop * factor, self.total * factor)

    @staticmethod
    def whole(total: int) -> "AxisSpan":
        return AxisSpan(0, total, total)

    @staticmethod
    def shard(total: int, rank: int, size: int, unit: int = 1, what: str = "axis") -> "AxisSpan":
        """Rank ``rank``'s equal share of ``total``; shares are whole multiples of ``unit``."""
        if size < 1 or not 0 <= rank < size:
            raise PartitionError(f"rank {rank} is not in a group of {size}")
        if total % size or (total // size) % unit:
            raise PartitionError(f"{what} of {total} does not split into {size} shares that are multiples of {unit}")
        share = total // size
        return AxisSpan(rank * share, (rank + 1) * share, total)


@dataclass(frozen=True)
class WeightShare:
    module: str
    rows: AxisSpan            # output features owned
    cols: AxisSpan            # input features owned
    bits: float               # storage bits per weight including group metadata

    @property
    def nbytes(self) -> int:
        return int(self.rows.size * self.cols.size * self.bits / 8)


@dataclass
class RankPartition:
    rank: int
    stage: int
    tensor_rank: int
    layers: tuple[int, int]
    experts: AxisSpan | None
    shares: list[WeightShare] = field(default_factory=list)
    plain_bytes: int = 0      # embeddings, head, norms (bf16)

    @property
    def weight_bytes(self) -> int:
        return sum(s.nbytes for s in self.shares) + self.plain_bytes


@dataclass
class PartitionPlan:
    tp: int
    pp: int
    ep: int
    ranks: list[RankPartition]

    def summary(self) -> list[dict]:
        return [{"rank": r.rank, "stage": r.stage, "tensor_rank": r.tensor_rank, "layers": list(r.layers),
                 "experts": None if r.experts is None else [r.experts.start, r.experts.stop],
                 "weights_gib": round(r.weight_bytes / 2 ** 30, 3)} for r in self.ranks]


def storage_bits(cfg: ModelConfig) -> float:
    """Bits per stored weight of the checkpoint's format, group metadata included."""
    q = cfg.quant
    if q.method == "none":
        return 16.0
    if q.method in ("fp8", "fp8_block"):
        return 8.0 + (16.0 / 128 if q.method == "fp8" else 32.0 / (128 * 128))
    if q.method == "nvfp4":
        return 4.0 + 8.0 / 16
    group = q.group_size or 128
    meta = {"cubic": 3 * 16, "awq": 16 + q.bits, "int": 16, "gguf": 6 + 6 + 32 / 8}.get(q.method, 16)
    return q.bits + meta / group


def plan_partition(cfg: ModelConfig, tp: int = 1, pp: int = 1, ep: int = 1) -> PartitionPlan:
    """Ownership of every logical weight for ``tp x pp`` ranks (rank = stage * tp + tensor rank); experts are split
    over ``ep`` ranks of a stage (``ep`` divides ``tp``: expert parallelism reuses the tensor-parallel ranks)."""
    from ..contracts.execution import ParallelTopology
    if tp < 1 or pp < 1 or ep < 1:
        raise PartitionError("parallel sizes are positive")
    if pp > cfg.num_layers:
        raise PartitionError(f"{pp} pipeline stages for {cfg.num_layers} layers")
    if ep > 1 and (not cfg.is_moe or tp % ep):
        raise PartitionError("expert parallelism needs a mixture-of-experts model and an ep size that divides tp")
    topo = ParallelTopology.single_node(list(range(tp * pp)), tp, pp)
    H, D = cfg.hidden_size, cfg.head_dim
    bits = storage_bits(cfg)
    ranks = []
    for rank in range(tp * pp):
        place = topo.placement(rank)
        t = place.tensor_rank
        lo, hi = topo.layer_range(place.stage, cfg.num_layers)
        experts = AxisSpan.shard(cfg.num_experts, t % ep, ep, what="experts") if cfg.is_moe and ep > 1 else (
            AxisSpan.whole(cfg.num_experts) if cfg.is_moe else None)
        part = RankPartition(rank, place.stage, t, (lo, hi), experts)
        qh = AxisSpan.shard(cfg.num_q_heads, t, tp, what="query heads")
        if cfg.num_kv_heads >= tp:
            kvh = AxisSpan.shard(cfg.num_kv_heads, t, tp, what="key/value heads")
        else:
            # fewer key/value heads than ranks: neighbouring ranks hold a copy of the same head
            from .config import kv_heads_of_rank
            try:
                first, count = kv_heads_of_rank(cfg.num_kv_heads, t, tp)
            except ValueError as exc:
                raise PartitionError(str(exc)) from exc
            kvh = AxisSpan(first, first + count, cfg.num_kv_heads)
        whole_h = AxisSpan.whole(H)
        for i in range(lo, hi):
            p = f"model.layers.{i}"
            if cfg.layer_is_gdn(i):
                gk = AxisSpan.shard(cfg.gdn_k_heads, t, tp, what="Gated DeltaNet key heads")
                gv = AxisSpan.shard(cfg.gdn_v_heads, t, tp, what="Gated DeltaNet value heads")
                r = cfg.gdn_v_heads // cfg.gdn_k_heads
                part.shares += [WeightShare(f"{p}.linear_attn.in_proj_qkvz", gk.scaled((2 + 2 * r) * 128), whole_h, bits),
                                WeightShare(f"{p}.linear_attn.in_proj_ba", gk.scaled(2 * r), whole_h, 16.0),
                                WeightShare(f"{p}.linear_attn.out_proj", whole_h, gv.scaled(128), bits)]
            else:
                gate = 2 if cfg.attn_output_gate else 1
                part.shares += [WeightShare(f"{p}.self_attn.q_proj", qh.scaled(D * gate), whole_h, bits),
                                WeightShare(f"{p}.self_attn.k_proj", kvh.scaled(D), whole_h, bits),
                                WeightShare(f"{p}.self_attn.v_proj", kvh.scaled(D), whole_h, bits),
                                WeightShare(f"{p}.self_attn.o_proj", whole_h, qh.scaled(D), bits)]
            if cfg.is_moe:
                inter_tp = tp // ep                    # ranks that share one expert split its intermediate features
                inter = AxisSpan.shard(cfg.moe_intermediate_size, t // ep if ep > 1 else t, inter_tp, 64,
                                       "expert intermediate size")
                for e in range(experts.start, experts.stop):
                    ep_ = f"{p}.mlp.experts.{e}"
                    part.shares += [WeightShare(f"{ep_}.gate_proj", inter, whole_h, bits),
                                    WeightShare(f"{ep_}.up_proj", inter, whole_h, bits),
                                    WeightShare(f"{ep_}.down_proj", whole_h, inter, bits)]
                part.plain_bytes += cfg.num_experts * H * 2
            else:
                inter = AxisSpan.shard(cfg.intermediate_size, t, tp, 64, "intermediate size")
                part.shares += [WeightShare(f"{p}.mlp.gate_proj", inter, whole_h, bits),
                                WeightShare(f"{p}.mlp.up_proj", inter, whole_h, bits),
                                WeightShare(f"{p}.mlp.down_proj", whole_h, inter, bits)]
            part.plain_bytes += 2 * H * 2
        vocab = AxisSpan.shard(cfg.vocab_size, t, tp, what="vocabulary")
        if place.stage == 0:
            part.plain_bytes += vocab.size * H * 2                                  # embedding rows
        if place.stage == pp - 1:
            part.plain_bytes += H * 2 + (0 if cfg.tie_embeddings and pp == 1 else vocab.size * H * 2)   # norm, head
        ranks.append(part)
    return PartitionPlan(tp, pp, ep, ranks)
