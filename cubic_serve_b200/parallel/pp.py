"""Pipeline-parallel stage link: NCCL point-to-point transfers of the residual stream between stages.

Reference behaviour (``executor/text_serving.py:484-503``, ``executor/model_runner.py:3189-3197``): one or two
stages; the ``[M, H]`` bf16 hidden rows go stage to stage with NCCL p2p calls that are captured inside the CUDA
graph, and a two-lane "wavefront" (``runtime/performance.py:199-211``) lets stage 0 work on the second half
of the rows while stage 1 works on the first half.  Sampler rank = first rank of the last stage
(``executor/quantized_graph.py:1557``); every rank needs the sampled ids for its own bookkeeping, so the
last stage broadcasts them.

This module is transport only.  The lane split and the per-stage layer loop live in
``models/decoder.py::DecoderRunner``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def split_lanes(num_tokens: int, num_row_blocks: int, lanes: int = 2, align: int = 16, min_rows: int = 32):
    """Row ranges ``(t0, t1, rb0, rb1)`` of the wavefront lanes for a pure-decode step.

    A step is split only when every row block is one row (decode: token i <-> row block i); anything else
    (prefill chunks, review rows of a speculative round) runs as a single lane.
    """
    if lanes < 2 or num_tokens != num_row_blocks or num_tokens < min_rows:
        return [(0, num_tokens, 0, num_row_blocks)]
    per = -(-num_tokens // lanes)
    per = -(-per // align) * align
    out = []
    t = 0
    while t < num_tokens:
        e = min(num_tokens, t + per)
        out.append((t, e, t, e))
        t = e
    return out


@dataclass
class PipelineStage:
    """This rank's place in the pipeline and its neighbours (global ranks of the same tensor lane)."""
    stage: int
    num_stages: int
    prev_rank: int | None
    next_rank: int | None
    sampler_rank: int
    group: object | None = None          # process group that spans every stage (the world group)
    lanes: int = 2

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.num_stages - 1

    @staticmethod
    def from_topology(topology, rank: int, group=None, lanes: int = 2) -> "PipelineStage":
        p = topology.placement(rank)
        tp = topology.tp
        if tp > 1:
            # Stages of tensor-parallel width > 1 run ONE lane per step.  With two lanes such stages stopped making
            # progress on 4 and on 8 GPUs at 256 rows per step (every rank's GPU work enqueued, none finishing: the
            # lanes interleave point-to-point transfers on the world communicator with all-reduces on the stage's
            # own communicator); one lane per step ran to completion.  Stages of width 1 keep the two-lane wavefront.
            lanes = 1
        prev_rank = rank - tp if p.stage > 0 else None
        next_rank = rank + tp if p.stage + 1 < topology.pp else None
        return PipelineStage(p.stage, topology.pp, prev_rank, next_rank, topology.sampler_rank, group, lanes)

    # transfers are enqueued on the current stream's NCCL side stream; the blocking forms make the current
    # stream wait for the transfer, which is what orders the lanes
    def recv(self, t: torch.Tensor) -> None:
        dist.recv(t, src=self.prev_rank, group=self.group)

    def send(self, t: torch.Tensor) -> None:
        dist.send(t, dst=self.next_rank, group=self.group)

    def share_token_ids(self, ids: torch.Tensor) -> None:
        """Sampled ids from the sampler rank to every rank (in place)."""
        dist.broadcast(ids, src=self.sampler_rank, group=self.group)
