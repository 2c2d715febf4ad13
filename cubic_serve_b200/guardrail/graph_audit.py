"""Audits of whole captured decode graphs (not of single operators): what a request computes must not depend on
which bucket the step was padded to, on what the padding rows hold, or on the row it occupies.

Three runs of the same requests through freshly built executors (same weights, same pages per request):

* **cross-M**: decode graphs of two capacities; the real rows' logits are compared (bit-identical when both buckets
  launch the same attention split, else within rounding of the differently ordered split merge; the sampled ids must
  agree either way);
* **poisoned padding**: the larger bucket again with the padding rows' inputs randomised and the activations a step
  leaves unwritten for them set to NaN (``GpuExecutor.audit_poison_padding``): bit-identical to the clean run;
* **row permutation**: the requests in reverse order on other page-table rows: every request's logits bit-identical.

Reference counterparts: ``guardrail/quantized_graph/text_cross_m.py`` (cross-M identity of captured graphs) and
``guardrail/graph_padding.py`` (poisoned padding rows) there.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class GraphAuditReport:
    capacities: tuple[int, int]
    steps: int
    cross_m_max_rel: float = 0.0
    cross_m_bit_identical: bool = False
    cross_m_ids_equal: bool = False
    poisoned_padding_bit_identical: bool = False
    poisoned_padding_finite: bool = False
    permutation_bit_identical: bool = False
    notes: list[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return (self.cross_m_ids_equal and self.cross_m_max_rel < 2e-2 and self.poisoned_padding_bit_identical
                and self.poisoned_padding_finite and self.permutation_bit_identical)


def _run(build_executor, prompts, capacity: int, steps: int, order=None, poison: bool = False):
    """Prefill ``prompts`` eagerly (one step), then ``steps`` decode steps through the graph of ``capacity`` rows.
    Returns per step the logits ``[R, V]`` (bf16 bits as int16) and ids, both in REQUEST order."""
    import torch

    from ..executor.gpu_executor import Segment
    ex = build_executor()
    caps = ex.capture_decode_graphs([capacity])
    if caps != [capacity]:
        raise RuntimeError(f"decode graph of {capacity} rows was not sealed: {ex.graph_rt.poison_log}")
    R = len(prompts)
    order = list(range(R)) if order is None else list(order)
    pages_per = -(-(max(len(p) for p in prompts) + steps + 2) // 16)
    pages = [list(range(1 + i * pages_per, 1 + (i + 1) * pages_per)) for i in range(R)]
    slot_of = {req: row for row, req in enumerate(order)}          # the request's page-table row = its row in the step

    def segs(tokens_of, start_of):
        return [Segment(slot_of[req], tokens_of(req), start_of(req), pages[req], True, uid=100 + req) for req in order]

    def in_request_order(t):
        return torch.stack([t[slot_of[req]] for req in range(R)])

    ids = ex.execute(segs(lambda r: prompts[r], lambda r: 0))
    last = {req: int(ids[slot_of[req]]) for req in range(R)}
    ex.audit_poison_padding = poison
    out_logits, out_ids = [], []
    for step in range(steps):
        ids = ex.execute(segs(lambda r: [last[r]], lambda r: len(prompts[r]) + step))
        torch.cuda.synchronize(ex.device)
        out_logits.append(in_request_order(ex.logits[:R]).view(torch.int16).clone())
        out_ids.append([int(ids[slot_of[req]]) for req in range(R)])
        last = {req: out_ids[-1][req] for req in range(R)}
    ex.runner.ws.check_status()
    return out_logits, out_ids


def audit_decode_graphs(build_executor, prompts, capacities: tuple[int, int] = (8, 32), steps: int = 3) -> GraphAuditReport:
    """``build_executor()`` returns a fresh ``GpuExecutor`` over the same weights every time (graphs not yet captured);
    ``prompts``: token lists, fewer than ``min(capacities)``."""
    import torch
    small, large = sorted(capacities)
    if len(prompts) >= small:
        raise ValueError("the audit needs padding rows in both buckets")
    rep = GraphAuditReport((small, large), steps)
    a_logits, a_ids = _run(build_executor, prompts, small, steps)
    b_logits, b_ids = _run(build_executor, prompts, large, steps)
    rep.cross_m_ids_equal = a_ids == b_ids
    rep.cross_m_bit_identical = all(torch.equal(x, y) for x, y in zip(a_logits, b_logits))
    worst = 0.0
    for x, y in zip(a_logits, b_logits):
        xf, yf = x.view(torch.bfloat16).float(), y.view(torch.bfloat16).float()
        worst = max(worst, float(((xf - yf).norm(dim=1) / yf.norm(dim=1).clamp_min(1e-20)).max()))
    rep.cross_m_max_rel = worst
    if not rep.cross_m_bit_identical:
        rep.notes.append("the buckets split the attention context differently: logits agree to rounding, not bit for bit")
    c_logits, c_ids = _run(build_executor, prompts, large, steps, poison=True)
    rep.poisoned_padding_bit_identical = all(torch.equal(x, y) for x, y in zip(b_logits, c_logits)) and b_ids == c_ids
    rep.poisoned_padding_finite = all(bool(torch.isfinite(x.view(torch.bfloat16).float()).all()) for x in c_logits)
    d_logits, d_ids = _run(build_executor, prompts, large, steps, order=reversed(range(len(prompts))))
    rep.permutation_bit_identical = all(torch.equal(x, y) for x, y in zip(b_logits, d_logits)) and b_ids == d_ids
    return rep
