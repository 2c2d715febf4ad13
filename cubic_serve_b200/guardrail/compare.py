"""Witness-based numeric comparison (no single global tolerance).

Like the reference's ``guardrail/compare.py``: a candidate tensor is judged against an oracle computed by
independent code, with a bound derived from the operation (how many products were summed, in which dtype the
result is rounded) instead of one magic epsilon; the verdict records where the worst element is.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class DifferenceClass(str, enum.Enum):
    EXACT = "exact"            # bitwise equal
    ROUNDING = "rounding"      # within the bound implied by the output dtype and reduction length
    MISMATCH = "mismatch"


@dataclass(frozen=True)
class Verdict:
    klass: DifferenceClass
    max_abs: float
    rel_l2: float
    bound: float
    worst_index: tuple[int, ...]

    @property
    def ok(self) -> bool:
        return self.klass is not DifferenceClass.MISMATCH


_EPS = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -24}


def reduction_bound(reference: torch.Tensor, out_dtype: torch.dtype, reduction_length: int, operand_dtype=torch.bfloat16,
                    slack: float = 4.0) -> float:
    """Relative L2 bound for a length-``reduction_length`` dot product of ``operand_dtype`` values rounded to ``out_dtype``.

    Operand rounding errors are independent, so they grow with sqrt(K) in absolute and stay ~eps in relative terms;
    the output rounding adds one more eps of the output type.
    """
    eps_in, eps_out = _EPS.get(operand_dtype, 2.0 ** -24), _EPS.get(out_dtype, 2.0 ** -24)
    del reference, reduction_length
    return slack * (2 * eps_in + eps_out)


def compare_tensors(candidate: torch.Tensor, oracle: torch.Tensor, bound: float) -> Verdict:
    c, o = candidate.detach().float().cpu(), oracle.detach().float().cpu()
    if c.shape != o.shape:
        return Verdict(DifferenceClass.MISMATCH, float("inf"), float("inf"), bound, ())
    if not torch.isfinite(c).all():
        bad = (~torch.isfinite(c)).nonzero()[0].tolist()
        return Verdict(DifferenceClass.MISMATCH, float("inf"), float("inf"), bound, tuple(bad))
    diff = (c - o).abs()
    max_abs = float(diff.max()) if diff.numel() else 0.0
    worst = tuple(int(i) for i in torch.unravel_index(diff.argmax(), diff.shape)) if diff.numel() else ()
    rel = float((c - o).norm() / o.norm().clamp_min(1e-30))
    if max_abs == 0.0:
        return Verdict(DifferenceClass.EXACT, 0.0, 0.0, bound, worst)
    return Verdict(DifferenceClass.ROUNDING if rel <= bound else DifferenceClass.MISMATCH, max_abs, rel, bound, worst)


def poisoned_padding_preserved(active_before: torch.Tensor, active_after: torch.Tensor) -> bool:
    """Padding rows filled with NaN / garbage must not change any active row (graph-padding qualification)."""
    return torch.equal(active_before, active_after)
