"""Eager tensor x pipeline parallel reference decoder over ``torch.distributed`` (gloo on CPU, NCCL on GPUs).

The oracle for everything that shards a model: every rank holds exactly the rows / columns of every weight that
``parallel_weights.plan_partition`` assigns to it, computes with plain PyTorch in fp32, and meets the others only in
the reference collectives below.  Partial sums are gathered and added in rank order, so the result does not depend on
arrival order and equals the single-process ``EagerDecoder`` up to fp32 summation order.  It is slow on purpose: one
collective per operator, no fusion, no overlap -- the thing the fused kernels are compared with, never a serving path.

Reference counterpart: ``executor/distributed_reference.py`` (bit-exact eager TP x PP reference, operands gathered per
operator) and the reference collectives of ``executor/eager_nccl.py`` (``tp_all_reduce``, ``tp_all_gather``,
``pipeline_send`` / ``pipeline_recv``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import eager
from .config import ModelConfig
from .parallel_weights import PartitionPlan, RankPartition
from .reference import DenseLayer, DenseWeights


# ------------------------------------------------------------------ reference collectives
def tp_all_gather(x: torch.Tensor, group, dim: int = -1) -> torch.Tensor:
    """Concatenation of every rank's ``x`` along ``dim`` in rank order."""
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim)


def tp_all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    """Sum of every rank's ``x``, added in rank order (identical bits on all ranks)."""
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    total = parts[0].clone()
    for p in parts[1:]:
        total += p
    return total


def pipeline_send(x: torch.Tensor, dst: int) -> None:
    dist.send(x.contiguous(), dst)


def pipeline_recv(like: torch.Tensor, src: int) -> torch.Tensor:
    out = torch.empty_like(like)
    dist.recv(out, src)
    return out


# ------------------------------------------------------------------ sharding by the ownership plan
def shard_dense_weights(w: DenseWeights, cfg: ModelConfig, part: RankPartition) -> DenseWeights:
    """The rank's shard of dense reference weights, cut by the spans of its ``RankPartition`` (layers of its stage
    only; embedding and head are split over the vocabulary)."""
    spans = {s.module: s for s in part.shares}

    def cut(t: torch.Tensor, module: str) -> torch.Tensor:
        s = spans[module]
        assert tuple(t.shape) == (s.rows.total, s.cols.total), (module, tuple(t.shape), s)
        return t[s.rows.slice(), s.cols.slice()].contiguous()

    layers = []
    for i in range(*part.layers):
        l, p = w.layers[i], f"model.layers.{i}"
        layers.append(DenseLayer(
            l.ln1, l.ln2, cut(l.wq, f"{p}.self_attn.q_proj"), cut(l.wk, f"{p}.self_attn.k_proj"),
            cut(l.wv, f"{p}.self_attn.v_proj"), cut(l.wo, f"{p}.self_attn.o_proj"), cut(l.w_gate, f"{p}.mlp.gate_proj"),
            cut(l.w_up, f"{p}.mlp.up_proj"), cut(l.w_down, f"{p}.mlp.down_proj"), l.q_norm, l.k_norm))
    return DenseWeights(w.embed, layers, w.final_norm, w.lm_head)


def moe_expert_parallel_reference(x: torch.Tensor, router: torch.Tensor, gate_up: list[torch.Tensor],
                                  down: list[torch.Tensor], top_k: int, group, normalize: bool = True,
                                  ep_size: int | None = None) -> torch.Tensor:
    """Eager expert-parallel mixture-of-experts block: every rank of ``group`` routes ALL tokens with the replicated
    router, computes only the experts it owns (contiguous expert ids in owner order; ``gate_up`` / ``down`` hold this
    rank's experts) and the partial outputs are summed in rank order.  With ``ep_size`` smaller than the group, the
    group is ``ep_size`` owners times lanes: the lanes of an owner hold the same experts, ``gate_up`` / ``down`` then
    carry this lane's share of every expert's intermediate features (gate rows, up rows; down columns), and the same
    sum over all ranks completes both the experts and their features.  Equals the single-process ``moe_reference``
    over all experts up to summation order and the rounding of the per-expert output (each lane rounds its partial).
    Reference counterpart: ``models/qwen3_5_moe/distributed.py`` and ``contracts/execution.py:238-248`` there."""
    from .moe import expert_coordinates, moe_reference
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    owner, _lane, lanes = expert_coordinates(rank, size, ep_size)
    total, owners = router.shape[0], size // lanes
    if total % owners or len(gate_up) != total // owners or len(down) != len(gate_up):
        raise ValueError("every owner holds num_experts / owners experts")
    partial = moe_reference(x, router, gate_up, down, top_k, normalize, expert_lo=owner * (total // owners))
    return tp_all_reduce(partial, group)


def moe_dispatch_combine_reference(x_local: torch.Tensor, router: torch.Tensor, gate_up: list[torch.Tensor],
                                   down: list[torch.Tensor], top_k: int, group, normalize: bool = True):
    """Eager expert parallelism on a ROW-SHARDED stream, the schedule of ``parallel/ep.py``: every rank holds its own
    rows ``x_local`` and the experts ``[rank E / n, (rank + 1) E / n)``.

    1. dispatch: a rank routes its rows and sends each row ONCE to every rank that owns at least one of the row's
       experts, with the ids and weights of the experts that rank has to apply;
    2. the owner runs its experts on the rows it received and pre-sums a row's expert outputs with their weights:
       one row goes back per (row, owner);
    3. combine: the home rank adds the returned rows in ascending owner order.

    Returns ``(y_local, rows_sent)`` where ``rows_sent[d]`` counts the rows this rank sent to rank ``d`` (its own
    included).  ``y_local`` equals ``moe_reference`` over all experts on the same rows up to the order of the final
    sum.  Reference counterpart: ``models/qwen3_5_moe/distributed.py:191`` (``_DistributedMoe``) there."""
    from .moe import moe_reference
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    E = router.shape[0]
    if E % size or len(gate_up) != E // size or len(down) != len(gate_up):
        raise ValueError("every rank owns num_experts / group size experts")
    per = E // size
    xf = x_local.float()
    logits = (xf @ router.float().t()).to(torch.bfloat16).float()
    order = torch.argsort(-logits, dim=-1, stable=True)[:, :top_k]
    sel = torch.gather(logits, 1, order)
    w = torch.softmax(sel, -1) if normalize else torch.softmax(logits, -1).gather(1, order)
    outbox: list[list] = [[] for _ in range(size)]                  # per destination: (row, [(expert, weight)...], vector)
    for t in range(x_local.shape[0]):
        by_dest: dict[int, list] = {}
        for j in range(top_k):
            e = int(order[t, j])
            by_dest.setdefault(e // per, []).append((e, float(w[t, j])))
        for d, routes in sorted(by_dest.items()):
            outbox[d].append((t, routes, x_local[t]))
    inbox: list = [None] * size
    dist.all_gather_object(inbox, outbox, group=group)              # inbox[src][dst]
    returned: list[list] = [[] for _ in range(size)]                # per source rank: (row, pre-summed vector)
    for src in range(size):
        for t, routes, vec in inbox[src][rank]:
            acc = torch.zeros(x_local.shape[1])
            for e, weight in routes:
                le = e - rank * per
                gu = (vec.float() @ gate_up[le].float().t()).to(torch.bfloat16).float()
                half = gu.shape[0] // 2
                act = (torch.nn.functional.silu(gu[:half]) * gu[half:]).to(torch.bfloat16).float()
                acc += weight * (act @ down[le].float().t()).to(torch.bfloat16).float()
            returned[src].append((t, acc))
    back: list = [None] * size
    dist.all_gather_object(back, returned, group=group)             # back[owner][home]
    y = torch.zeros(x_local.shape[0], x_local.shape[1])
    for owner in range(size):                                       # ascending owner order: the same bits on any run
        for t, vec in back[owner][rank]:
            y[t] += vec
    return y, [len(o) for o in outbox]


class DistributedEagerDecoder:
    """One rank of the reference.  ``tp_group``: the ranks of this stage; ``prev`` / ``next``: global ranks of the
    same tensor rank in the neighbouring stages (None at the ends)."""

    def __init__(self, cfg: ModelConfig, plan: PartitionPlan, rank: int, full: DenseWeights, tp_group) -> None:
        self.cfg, self.plan, self.part = cfg, plan, plan.ranks[rank]
        self.w = shard_dense_weights(full, cfg, self.part)
        self.tp_group, self.tp = tp_group, plan.tp
        self.prev = rank - plan.tp if self.part.stage > 0 else None
        self.next = rank + plan.tp if self.part.stage < plan.pp - 1 else None
        self.inv_freq = eager.rope_inv_freq(cfg.rotary_dim or cfg.head_dim, cfg.rope_theta, scaling=cfg.rope_scaling)
        v = cfg.vocab_size // plan.tp
        self.vocab = slice(self.part.tensor_rank * v, (self.part.tensor_rank + 1) * v)

    def _sum(self, x: torch.Tensor) -> torch.Tensor:
        return tp_all_reduce(x, self.tp_group) if self.tp > 1 else x

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, start: int, cache: list | None):
        """As ``EagerDecoder.forward`` for this rank's heads and layers.  Returns the full-vocabulary logits on the
        ranks of the last stage (None elsewhere) and this rank's cache."""
        cfg, w = self.cfg, self.w
        B, S = tokens.shape
        D = cfg.head_dim
        Hq, Hkv = cfg.num_q_heads // self.tp, cfg.num_kv_heads // self.tp
        pos = torch.arange(start, start + S)
        if self.prev is None:
            h = w.embed[tokens].float()
        else:
            h = pipeline_recv(torch.empty(B, S, cfg.hidden_size), self.prev)
        new_cache = []
        for li, l in enumerate(w.layers):
            x = eager.rmsnorm(h, l.ln1, cfg.rms_eps, cfg.zero_centered_norm)
            q = (x @ l.wq.t()).view(B, S, Hq, D)
            k = (x @ l.wk.t()).view(B, S, Hkv, D)
            v = (x @ l.wv.t()).view(B, S, Hkv, D)
            if l.q_norm is not None:
                q = eager.rmsnorm(q, l.q_norm, cfg.rms_eps)
                k = eager.rmsnorm(k, l.k_norm, cfg.rms_eps)
            q = torch.stack([eager.rope(q[b], pos, self.inv_freq) for b in range(B)])
            k = torch.stack([eager.rope(k[b], pos, self.inv_freq) for b in range(B)])
            if cache is not None and cache[li] is not None:
                k = torch.cat([cache[li][0], k], 1)
                v = torch.cat([cache[li][1], v], 1)
            new_cache.append((k, v))
            vis = torch.arange(start + 1, start + S + 1)
            attn = torch.stack([eager.attention_rows(q[b], k[b], v[b], vis, cfg.attention_scale) for b in range(B)])
            h = h + self._sum(attn.reshape(B, S, Hq * D) @ l.wo.t())            # row-parallel: partial sums
            x = eager.rmsnorm(h, l.ln2, cfg.rms_eps, cfg.zero_centered_norm)
            h = h + self._sum((torch.nn.functional.silu(x @ l.w_gate.t()) * (x @ l.w_up.t())) @ l.w_down.t())
        if self.next is not None:
            pipeline_send(h, self.next)
            return None, new_cache
        local = eager.rmsnorm(h, w.final_norm, cfg.rms_eps, cfg.zero_centered_norm) @ w.lm_head[self.vocab].t()
        logits = tp_all_gather(local, self.tp_group) if self.tp > 1 else local
        return logits, new_cache

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, steps: int, world_group=None):
        """Greedy decode on all ranks; the last stage's choice is broadcast so that every rank feeds the same token.
        Returns ``(tokens [B, steps], logits of every step)`` -- logits are None except on the last stage."""
        last_stage_rank0 = (self.plan.pp - 1) * self.plan.tp
        out, all_logits = [], []
        cache = None
        tokens, start = prompts, 0
        for _ in range(steps):
            logits, cache = self.forward(tokens, start, cache)
            nxt = logits[:, -1].argmax(-1) if logits is not None else torch.zeros(prompts.shape[0], dtype=torch.long)
            if self.plan.pp > 1:
                dist.broadcast(nxt, last_stage_rank0, group=world_group)
            out.append(nxt)
            all_logits.append(None if logits is None else logits[:, -1])
            start += tokens.shape[1]
            tokens = nxt[:, None]
        return torch.stack(out, 1), all_logits
