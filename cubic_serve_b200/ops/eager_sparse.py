"""Eager oracles of the sparse-attention family's two special operators: compressed-block selection with attention over
the selected tokens, and gated multi-stream residual mixing ("hyperconnections").

Plain PyTorch in fp32, vectorised over batch and query rows; no cache layout, no kernels.  They state the math the
native kernels of that family have to reproduce and are tested against direct per-row loops.

Block selection: keys are pooled into one vector per ``compression`` tokens.  A query scores every *complete* visible
block by ``sum_h relu(q_h . k_block) / sqrt(D)``, keeps the ``budget / compression`` best (ties: lower block index) and
always keeps the tokens of the incomplete tail block.  The result lists token indices, selected blocks first in score
order, then the tail, ``-1`` where nothing is selected.

Residual mixing: the residual stream carries ``S`` parallel streams of width ``W``.  A block reads the mean over
streams of the group-normalised, gated residual; its output is written back into every stream through per-stream
injection gates in (0, 2).

Reference counterpart: ``ops/eager/sparse_indexer.py`` (``select_blocks``, ``attend_selected``) and
``ops/eager/hyperconnection.py`` (``mix``, ``injection``, ``combine``, ``signed_root_gate``).
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ compressed-block selection
def block_scores(queries: torch.Tensor, block_keys: torch.Tensor) -> torch.Tensor:
    """``[B, T, N]`` scores of ``[B, T, H, D]`` queries against ``[B, N, D]`` pooled keys."""
    dots = torch.einsum("bthd,bnd->bthn", queries.float(), block_keys.float())
    return dots.clamp_min(0).sum(2) / math.sqrt(queries.shape[-1])


def select_blocks(queries: torch.Tensor, block_keys: torch.Tensor, visible: torch.Tensor, compression: int,
                  token_budget: int) -> torch.Tensor:
    """Token indices ``[B, T, budget + compression - 1]`` (int32, ``-1`` = none) every query attends to."""
    if queries.dim() != 4 or block_keys.dim() != 3 or queries.shape[0] != block_keys.shape[0] \
            or queries.shape[-1] != block_keys.shape[-1]:
        raise ValueError("queries are [B, T, H, D] and pooled keys [B, N, D] with the same B and D")
    if visible.shape != queries.shape[:2]:
        raise ValueError("one visible length per query")
    if compression <= 0 or token_budget <= 0 or token_budget % compression:
        raise ValueError("the token budget is a positive number of whole blocks")
    B, T = visible.shape
    N = block_keys.shape[1]
    complete = visible.long() // compression                          # blocks that compete
    if bool((visible < 0).any()) or bool((complete > N).any()):
        raise ValueError("visible lengths exceed the pooled keys supplied")
    tail = visible.long() - complete * compression
    keep = token_budget // compression
    scores = block_scores(queries, block_keys)
    block_id = torch.arange(N, device=scores.device)
    scores = scores.masked_fill(block_id[None, None, :] >= complete[..., None], float("-inf"))
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices[..., :keep]      # ties: lower id first
    if order.shape[-1] < keep:                                        # fewer pooled keys than the budget has blocks
        order = torch.nn.functional.pad(order, (0, keep - order.shape[-1]), value=0)
    rank = torch.arange(keep, device=scores.device)
    chosen = rank[None, None, :] < complete.clamp_max(keep)[..., None]                        # [B, T, keep]
    within = torch.arange(compression, device=scores.device)
    block_tokens = (order[..., None] * compression + within).reshape(B, T, keep * compression)
    block_tokens = block_tokens.masked_fill(~chosen.repeat_interleave(compression, -1), -1)
    # output position p: a token of a selected block while p < selected tokens, then the tail tokens, then nothing
    width = token_budget + compression - 1
    p = torch.arange(width, device=scores.device)
    selected = (complete.clamp_max(keep) * compression)[..., None]
    padded = torch.nn.functional.pad(block_tokens, (0, width - keep * compression), value=-1)
    t = p - selected
    tail_tokens = (complete * compression)[..., None] + t
    out = torch.where(p < selected, padded, torch.where(t < tail[..., None], tail_tokens, torch.full_like(tail_tokens, -1)))
    return out.to(torch.int32)


def attend_selected(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention of ``[B, H, T, D]`` queries over the tokens listed per query in ``indices``
    ``[B, T, L]`` (``-1`` entries are skipped; the order of the listed tokens does not matter); K / V are
    ``[B, Hkv, S, D]``.  Returns fp32 ``[B, H, T, D]``."""
    B, H, T, D = query.shape
    Hkv = key.shape[1]
    if H % Hkv or key.shape != value.shape or indices.shape[:2] != (B, T):
        raise ValueError("head groups, K / V shapes or the index rows do not fit")
    present = indices >= 0
    if not bool(present.any(-1).all()) or bool((indices >= key.shape[2]).any()):
        raise ValueError("every query needs at least one valid token index")
    safe = indices.clamp_min(0).long()                                                        # [B, T, L]
    gather = safe[:, None, :, :, None].expand(B, Hkv, T, safe.shape[-1], D)
    k = torch.gather(key.float()[:, :, None].expand(B, Hkv, T, key.shape[2], D), 3, gather)   # [B, Hkv, T, L, D]
    v = torch.gather(value.float()[:, :, None].expand(B, Hkv, T, key.shape[2], D), 3, gather)
    g = H // Hkv
    q = query.float().reshape(B, Hkv, g, T, D)
    logits = torch.einsum("bkgtd,bktld->bkgtl", q, k) / math.sqrt(D)
    logits = logits.masked_fill(~present[:, None, None], float("-inf"))
    return torch.einsum("bkgtl,bktld->bkgtd", torch.softmax(logits, -1), v).reshape(B, H, T, D)


# ------------------------------------------------------------------ multi-stream residual mixing
def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, group: int, eps: float) -> torch.Tensor:
    """RMS normalisation over consecutive groups of ``group`` channels, zero-centred weight ``(1 + w)``."""
    if group <= 0 or x.shape[-1] % group or weight.shape != x.shape[-1:]:
        raise ValueError("whole groups and one weight per channel")
    g = x.float().unflatten(-1, (-1, group))
    g = g * torch.rsqrt(g.square().mean(-1, keepdim=True) + eps)
    return (g.flatten(-2) * (1 + weight.float())).to(x.dtype)


def stream_mix(x: torch.Tensor, norm_w: torch.Tensor, down: torch.Tensor, up: torch.Tensor, streams: int, eps: float):
    """Input of a block from a ``[..., S W]`` residual: group norm per stream, a low-rank gate
    ``sigmoid(up(silu(down(n) / S)))`` on it, mean over the streams.  Returns ``(block input [..., W], n)``."""
    if streams <= 0 or x.shape[-1] % streams:
        raise ValueError("the residual width is a whole number of streams")
    width = x.shape[-1] // streams
    n = grouped_rms_norm(x, norm_w, width, eps)
    low = torch.nn.functional.silu((n.float() @ down.float().t()).to(x.dtype).float() / streams).to(x.dtype)
    gate = torch.sigmoid((low.float() @ up.float().t()).to(x.dtype).float()).to(x.dtype)
    gated = (gate * n).float().unflatten(-1, (streams, width))
    return gated.mean(-2).to(x.dtype), n


def stream_injection(n: torch.Tensor, weight: torch.Tensor, streams: int) -> torch.Tensor:
    """Per-stream write gates in (0, 2): ``2 sigmoid(W n / S)`` with one row of ``W`` per stream."""
    if weight.shape[0] != streams:
        raise ValueError("one gate row per stream")
    return (torch.sigmoid((n.float() @ weight.float().t()).to(n.dtype).float() / streams) * 2).to(n.dtype)


def stream_combine(residual: torch.Tensor, output: torch.Tensor, gates: torch.Tensor) -> torch.Tensor:
    """Every stream receives the block output scaled by its gate: ``residual[..., s, :] += gates[..., s] * output``."""
    streams = gates.shape[-1]
    if residual.shape[-1] != streams * output.shape[-1] or gates.shape[:-1] != output.shape[:-1]:
        raise ValueError("residual, block output and gates do not fit")
    return residual + (gates.unsqueeze(-1) * output.unsqueeze(-2)).flatten(-2)


def signed_root_gate(key: torch.Tensor, query: torch.Tensor, value: torch.Tensor, floor: float = 1e-6) -> torch.Tensor:
    """``sigmoid(sign(s) sqrt(max(|s|, floor)))`` with ``s = k . q / sqrt(D)`` per (row, head), applied to the row's
    value vector: ``[..., H, D] x [..., H, D] x [..., D] -> [..., H D]``."""
    if key.shape != query.shape or key.shape[:-2] != value.shape[:-1] or key.shape[-1] != value.shape[-1]:
        raise ValueError("key / query are [..., H, D], value [..., D]")
    s = (key.float() * query.float()).sum(-1).to(key.dtype).float() / math.sqrt(key.shape[-1])
    t = s.abs().clamp_min(floor).sqrt() * s.sign()
    return (torch.sigmoid(t).to(key.dtype).unsqueeze(-1) * value.unsqueeze(-2)).flatten(-2)
