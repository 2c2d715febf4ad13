"""Enclosures of the decoder's operators from their ACTUAL inputs: for one call of an operator, the interval that the
output of every implementation honouring the arithmetic contract must fall into, element by element.

The contract: operands are the stored values (bf16 activations, decoded weights, decoded cache codes); sums of
products are accumulated in fp32 in ANY order (tiles, split-K partial sums, tensor-core trees; an accumulator that
truncates instead of rounding is allowed, hence the unit ``2**-23``); transcendental functions are good to a few fp32
units; the result is rounded once to the output dtype.  Rounding to nearest is monotone, so an exact value inside
``[lo, hi]`` is stored inside ``[round(lo), round(hi)]``: that pair is the enclosure in the output dtype.

The error of a sum of products evaluated in floating point is bounded by ``gamma(n) * sum(|a_i| |b_i|)`` (the same
expression over the magnitudes), ``gamma(n) = n u / (1 - n u)``, ``n`` the length of the longest chain of roundings.
Every enclosure below is the double-precision value of the operator plus or minus that bound, with interval products
where an operand is itself only known as an interval (the softmax weights of attention).

An enclosure is a statement about ONE call ("cold state"): its inputs are what the implementation under test was
really given, so errors of earlier operators do not widen it and a single wrong operator is named, not smeared over a
tolerance of the whole model.  It is not a statement about a whole model or about a recurrent state after many steps.

A candidate outside its enclosure broke the contract (a lower-precision accumulator, a dropped term, a different
constant, a second storage rounding); ``Enclosure.check`` reports how many elements, the worst excess in units of the
output dtype's spacing and where.

Reference counterpart: ``guardrail/quantized_graph/bounds.py:1-318`` (products, route softmax, sigmoid enclosures),
``guardrail/quantized_graph/linear.py:1-273``, ``attention_bounds.py:1-163``, ``state_bounds.py:1-311``,
``nonlinear.py:1-491``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

U32 = 2.0 ** -23          # one fp32 spacing, relative: covers a truncating accumulator as well as a rounding one


def gamma(n: int, unit: float = U32) -> float:
    """Bound factor of ``n`` chained roundings of relative size ``unit``."""
    nu = n * unit
    if nu >= 1:
        raise ValueError("the chain is too long for this unit")
    return nu / (1 - nu)


def _d(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu", torch.float64)


@dataclass(frozen=True)
class EnclosureReport:
    ok: bool
    outside: int                 # elements outside the enclosure
    total: int
    worst_excess_ulps: float     # largest distance to the enclosure, in spacings of the output dtype at that element
    index: tuple | None          # where the worst one is

    def __bool__(self) -> bool:
        return self.ok


@dataclass(frozen=True)
class Enclosure:
    lo: torch.Tensor             # float64, already rounded to ``dtype``
    hi: torch.Tensor
    dtype: torch.dtype

    @staticmethod
    def of(lo: torch.Tensor, hi: torch.Tensor, dtype: torch.dtype) -> "Enclosure":
        if not (torch.isfinite(lo).all() and torch.isfinite(hi).all()):
            raise ValueError("an enclosure needs finite inputs")
        if (lo > hi).any():
            raise AssertionError("inverted enclosure")
        return Enclosure(lo.to(dtype).double(), hi.to(dtype).double(), dtype)

    def spacing(self) -> torch.Tensor:
        """Spacing of the output dtype at the larger end of each interval."""
        fi = torch.finfo(self.dtype)
        mag = torch.maximum(self.lo.abs(), self.hi.abs()).clamp_min(fi.tiny)
        return torch.exp2(torch.floor(torch.log2(mag))) * fi.eps

    def width_ulps(self) -> torch.Tensor:
        return (self.hi - self.lo) / self.spacing()

    def check(self, candidate: torch.Tensor) -> EnclosureReport:
        c = _d(candidate)
        if c.shape != self.lo.shape:
            raise ValueError(f"candidate {tuple(c.shape)} against enclosure {tuple(self.lo.shape)}")
        if not torch.isfinite(c).all():
            return EnclosureReport(False, int((~torch.isfinite(c)).sum()), c.numel(), float("inf"), None)
        excess = torch.maximum(self.lo - c, c - self.hi).clamp_min(0) / self.spacing()
        outside = int((excess > 0).sum())
        if not outside:
            return EnclosureReport(True, 0, c.numel(), 0.0, None)
        flat = int(excess.argmax())
        return EnclosureReport(False, outside, c.numel(), float(excess.flatten()[flat]),
                               tuple(int(v) for v in torch.unravel_index(torch.tensor(flat), excess.shape)))


def _interval_product(alo, ahi, blo, bhi):
    """All four corners of ``[alo, ahi] * [blo, bhi]``, element by element."""
    c = torch.stack([alo * blo, alo * bhi, ahi * blo, ahi * bhi])
    return c.amin(0), c.amax(0)


def _relative(value: torch.Tensor, rel: float, absolute: float = 0.0):
    e = value.abs() * rel + absolute
    return value - e, value + e


# ------------------------------------------------------------------------------------------------- linear layers
def linear_enclosure(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                     bias: torch.Tensor | None = None, partial_sums: int = 1, residual: torch.Tensor | None = None) -> Enclosure:
    """``x [m, k] @ w[n, k].T (+ bias) (+ residual)``.  ``w`` holds the DECODED weights (the values the format defines:
    decoding is exact by contract, a kernel that decodes differently is outside).  A bf16 x bf16 product is exact in
    fp32; the accumulation rounds ``k - 1`` times plus once per partial sum joined, bias and residual."""
    xd, wd = _d(x), _d(w)
    exact = xd @ wd.T
    mag = xd.abs() @ wd.abs().T
    steps = xd.shape[-1] - 1 + max(0, partial_sums - 1)
    for extra in (bias, residual):
        if extra is not None:
            e = _d(extra)
            exact, mag, steps = exact + e, mag + e.abs(), steps + 1
    err = gamma(max(1, steps)) * mag
    return Enclosure.of(exact - err, exact + err, out_dtype)


def rank_sum_enclosure(partials: list[torch.Tensor], out_dtype: torch.dtype = torch.bfloat16,
                       residual: torch.Tensor | None = None) -> Enclosure:
    """Sum over ranks of partial rows that were STORED (rounded) by their producers, plus a residual, in any order."""
    vals = [_d(p) for p in partials] + ([_d(residual)] if residual is not None else [])
    exact = sum(vals)
    mag = sum(v.abs() for v in vals)
    err = gamma(max(1, len(vals) - 1)) * mag
    return Enclosure.of(exact - err, exact + err, out_dtype)


# ------------------------------------------------------------------------------------------------- pointwise / norms
def rmsnorm_enclosure(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype = torch.bfloat16,
                      zero_centered: bool = False, round_before_weight: bool = False) -> Enclosure:
    """``x * rsqrt(mean(x^2) + eps) * w``.  The mean square is a sum of positive terms (relative error
    ``gamma(n + 1)``), the reciprocal root halves that and adds its own two units; two products follow.
    ``round_before_weight``: the normalised row is stored in the activation dtype before the weight multiplies it
    (the form of the public Llama implementation)."""
    xd, wd = _d(x), _d(w) + (1.0 if zero_centered else 0.0)
    n = xd.shape[-1]
    r = torch.rsqrt((xd * xd).mean(-1, keepdim=True) + eps)
    rel_r = 0.5 * gamma(n + 2) * 1.01 + 3 * U32
    t = xd * r
    lo, hi = _relative(t, rel_r + U32)
    if round_before_weight:
        lo, hi = lo.to(x.dtype).double(), hi.to(x.dtype).double()
    plo, phi = _interval_product(lo, hi, wd.expand_as(lo), wd.expand_as(hi))
    e = torch.maximum(plo.abs(), phi.abs()) * 2 * U32          # the product, and the weight's own ``1 + w``
    return Enclosure.of(plo - e, phi + e, out_dtype)


def _sigmoid_interval(g: torch.Tensor):
    """fp32 ``1 / (1 + exp(-g))``: the exponential is good to three units, the sum and the division add three."""
    s = torch.sigmoid(g)
    return _relative(s, 8 * U32, torch.finfo(torch.float32).tiny)


def silu_mul_enclosure(gate: torch.Tensor, up: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> Enclosure:
    """``gate * sigmoid(gate) * up`` on stored ``gate`` / ``up`` values."""
    g, u = _d(gate), _d(up)
    slo, shi = _sigmoid_interval(g)
    lo, hi = _interval_product(slo, shi, g * u, g * u)
    e = torch.maximum(lo.abs(), hi.abs()) * 3 * U32
    return Enclosure.of(lo - e, hi + e, out_dtype)


def sigmoid_enclosure(x: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> Enclosure:
    lo, hi = _sigmoid_interval(_d(x))
    return Enclosure.of(lo.clamp_min(0), hi.clamp_max(1), out_dtype)


def softmax_enclosure(logits: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> Enclosure:
    """Softmax over the last axis of stored logits (router weights of the selected experts, attention rows)."""
    lo, hi = _softmax_interval(_d(logits), _d(logits))
    return Enclosure.of(lo, hi, out_dtype)


def _softmax_interval(slo: torch.Tensor, shi: torch.Tensor, rescales: int = 0):
    """Softmax weights of scores known as intervals.  The shift by the row maximum cancels between numerator and
    denominator; each exponential is good to three units, each running-maximum rescale multiplies by one more
    exponential and rounds once more."""
    m = shi.amax(-1, keepdim=True)
    rel = (3 + 4 * rescales) * U32
    plo = torch.exp(slo - m) * (1 - rel)
    phi = torch.exp(shi - m) * (1 + rel)
    n = slo.shape[-1]
    g = gamma(max(1, n - 1 + rescales))
    dlo = plo.sum(-1, keepdim=True) * (1 - g)
    dhi = phi.sum(-1, keepdim=True) * (1 + g)
    return (plo / dhi) * (1 - 2 * U32), (phi / dlo) * (1 + 2 * U32)


# ------------------------------------------------------------------------------------------------- attention
def attention_enclosure(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                        out_dtype: torch.dtype = torch.bfloat16, p_dtype: torch.dtype | None = torch.bfloat16,
                        tiles: int = 1) -> Enclosure:
    """One query row per head against its visible keys: ``q [h, d]``, ``k`` / ``v`` ``[h, n, d]`` holding the DECODED
    cache entries (codes times scales: exact by contract).  ``p_dtype``: storage of the softmax weights before they
    multiply ``v`` (tensor-core kernels round them to bf16; None = kept in fp32).  ``tiles``: key tiles of a running
    maximum (each tile boundary may rescale what was accumulated)."""
    qd, kd, vd = _d(q), _d(k), _d(v)
    h, n, d = kd.shape
    s = torch.einsum("hd,hnd->hn", qd, kd)
    smag = torch.einsum("hd,hnd->hn", qd.abs(), kd.abs())
    serr = (gamma(d) * smag + U32 * s.abs()) * abs(scale)
    slo, shi = s * scale - serr, s * scale + serr
    # un-normalised weights and their sum are enclosed separately: the kernels divide once, after the value product
    m = shi.amax(-1, keepdim=True)
    rel = (3 + 4 * (tiles - 1)) * U32
    plo, phi = torch.exp(slo - m) * (1 - rel), torch.exp(shi - m) * (1 + rel)
    g = gamma(max(1, n - 1 + tiles))
    if p_dtype is not None:                       # the stored weights feed the value product; the sum may take either
        u = torch.finfo(p_dtype).eps / 2
        plo, phi = plo * (1 - u), phi * (1 + u)
    dlo, dhi = plo.sum(-1) * (1 - g), phi.sum(-1) * (1 + g)
    nlo, nhi = _interval_product(plo[..., None], phi[..., None], vd, vd)
    nerr = g * (phi[..., None] * vd.abs()).sum(1)
    nlo, nhi = nlo.sum(1) - nerr, nhi.sum(1) + nerr
    dlo, dhi = dlo[:, None], dhi[:, None]
    c = torch.stack([nlo / dlo, nlo / dhi, nhi / dlo, nhi / dhi])
    lo, hi = c.amin(0), c.amax(0)
    e = torch.maximum(lo.abs(), hi.abs()) * 2 * U32
    return Enclosure.of(lo - e, hi + e, out_dtype)


# ------------------------------------------------------------------------------------------------- recurrent state
def delta_rule_enclosure(state: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                         beta: torch.Tensor, state_dtype: torch.dtype = torch.float32,
                         out_dtype: torch.dtype = torch.bfloat16) -> tuple[Enclosure, Enclosure]:
    """One token of the gated delta rule on the state it was really applied to: ``state [h, dv, dk]``, normalised
    ``q`` / ``k`` ``[h, dk]``, ``v [h, dv]``, ``decay`` / ``beta`` ``[h]`` (all as the implementation held them).
    ``S <- decay S;  S <- S + beta (v - S k) k^T;  o = S q``.  Returns the enclosures of the new state and of ``o``."""
    S, qd, kd, vd, gd, bd = (_d(t) for t in (state, q, k, v, decay, beta))
    dk = S.shape[-1]
    S1, M1 = S * gd[:, None, None], (S * gd[:, None, None]).abs()
    mem = torch.einsum("hvk,hk->hv", S1, kd)
    mem_mag = torch.einsum("hvk,hk->hv", M1, kd.abs())
    delta = (vd - mem) * bd[:, None]
    delta_mag = (vd.abs() + mem_mag) * bd.abs()[:, None]
    S2 = S1 + delta[:, :, None] * kd[:, None, :]
    M2 = M1 + delta_mag[:, :, None] * kd.abs()[:, None, :]
    serr = gamma(dk + 5) * M2
    o = torch.einsum("hvk,hk->hv", S2, qd)
    oerr = gamma(2 * dk + 6) * torch.einsum("hvk,hk->hv", M2, qd.abs())
    return Enclosure.of(S2 - serr, S2 + serr, state_dtype), Enclosure.of(o - oerr, o + oerr, out_dtype)


# ------------------------------------------------------------------------------------------------- a layer, operator by operator
class EagerOperators:
    """The candidate set of the plain PyTorch operators, storing bf16 at every boundary a kernel stores at.  Another
    implementation (a kernel binding) supplies the same five methods and is audited by the same chain."""

    dtype = torch.bfloat16

    def rmsnorm(self, x, w, eps):
        from ..ops import eager
        return eager.rmsnorm(x, w, eps).to(self.dtype)

    def linear(self, x, w, residual=None):
        y = x.float() @ w.float().T
        return (y if residual is None else y + residual.float()).to(self.dtype)

    def attention(self, q, k, v, scale):
        p = torch.softmax(torch.einsum("hd,hnd->hn", q.float(), k.float()) * scale, -1)
        return torch.einsum("hn,hnd->hd", p, v.float()).to(self.dtype)

    def silu_mul(self, gate, up):
        from ..ops import eager
        return eager.swiglu(torch.cat([gate, up], -1)).to(self.dtype)


def audit_layer_operators(ops=None, hidden: int = 256, heads: int = 4, head_dim: int = 64, inter: int = 512, context: int = 96,
                          seed: int = 0, eps: float = 1e-6) -> list[tuple[str, EnclosureReport]]:
    """One decode token through the operators of a decoder layer.  Every operator is given what the candidate itself
    produced before it, and its output is checked against the enclosure built from exactly those inputs: a wrong
    operator is reported under its own name and the ones after it are still judged on their own arithmetic."""
    ops = ops if ops is not None else EagerOperators()
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(bf)
    x = rnd(1, hidden)
    w_norm1, w_norm2 = (1 + 0.1 * torch.randn(hidden, generator=g)).to(bf), (1 + 0.1 * torch.randn(hidden, generator=g)).to(bf)
    w_q, w_o = rnd(heads * head_dim, hidden, scale=hidden ** -0.5), rnd(hidden, heads * head_dim, scale=(heads * head_dim) ** -0.5)
    w_gate, w_up = rnd(inter, hidden, scale=hidden ** -0.5), rnd(inter, hidden, scale=hidden ** -0.5)
    w_down = rnd(hidden, inter, scale=inter ** -0.5)
    k_cache, v_cache = rnd(heads, context, head_dim), rnd(heads, context, head_dim)
    scale = head_dim ** -0.5
    out: list[tuple[str, EnclosureReport]] = []

    def judged(name, enc, y):
        out.append((name, enc.check(y)))
        return y
    h1 = judged("input_norm", rmsnorm_enclosure(x, w_norm1, eps), ops.rmsnorm(x, w_norm1, eps))
    q = judged("q_proj", linear_enclosure(h1, w_q), ops.linear(h1, w_q))
    qh = q.view(heads, head_dim)
    a = judged("attention", attention_enclosure(qh, k_cache, v_cache, scale, tiles=max(1, context // 64)),
               ops.attention(qh, k_cache, v_cache, scale))
    a = a.reshape(1, heads * head_dim)
    x2 = judged("o_proj+residual", linear_enclosure(a, w_o, residual=x), ops.linear(a, w_o, residual=x))
    h2 = judged("post_norm", rmsnorm_enclosure(x2, w_norm2, eps), ops.rmsnorm(x2, w_norm2, eps))
    gate = judged("gate_proj", linear_enclosure(h2, w_gate), ops.linear(h2, w_gate))
    up = judged("up_proj", linear_enclosure(h2, w_up), ops.linear(h2, w_up))
    act = judged("silu_mul", silu_mul_enclosure(gate, up), ops.silu_mul(gate, up))
    judged("down_proj+residual", linear_enclosure(act, w_down, residual=x2), ops.linear(act, w_down, residual=x2))
    return out


# ------------------------------------------------------------------------------------------------- expert routing
@dataclass(frozen=True)
class RouteEnclosure:
    """Which experts a row MUST select (their logit's lower end beats the upper end of every expert outside the best
    ``k``) and which it MAY select (their upper end reaches the ``k``-th largest lower end).  Between the two lies a
    near-tie: implementations that accumulate the router product in another order may legitimately pick either
    expert there, and token streams that part at such a row are both right."""
    lo: torch.Tensor             # [rows, experts] logit enclosure (float64)
    hi: torch.Tensor
    k: int
    normalise: bool              # selected weights divided by their sum

    @property
    def must(self) -> torch.Tensor:
        kth_hi_outside = self.hi.sort(-1, descending=True).values[:, self.k:self.k + 1]          # (k+1)-th largest upper end
        return self.lo > kth_hi_outside if self.hi.shape[-1] > self.k else torch.ones_like(self.lo, dtype=torch.bool)

    @property
    def may(self) -> torch.Tensor:
        kth_lo = self.lo.sort(-1, descending=True).values[:, self.k - 1:self.k]
        return self.hi >= kth_lo

    def ambiguous_rows(self) -> torch.Tensor:
        return (self.may.sum(-1) > self.k).nonzero().flatten()

    def check(self, ids: torch.Tensor, weights: torch.Tensor | None = None) -> dict:
        """``ids [rows, k]`` (any order), ``weights [rows, k]`` aligned with them.  Returns the rows with a selection no
        ordering of the sums can produce and, for valid rows, the weights outside their enclosure."""
        ids = ids.detach().cpu().long()
        rows = torch.arange(ids.shape[0])[:, None]
        chosen = torch.zeros_like(self.lo, dtype=torch.bool)
        chosen[rows, ids] = True
        bad = ((chosen & ~self.may).any(-1) | (self.must & ~chosen).any(-1) | (chosen.sum(-1) != self.k))
        out = {"invalid_rows": bad.nonzero().flatten().tolist(), "ambiguous_rows": self.ambiguous_rows().tolist()}
        if weights is not None:
            slo, shi = self.lo[rows, ids], self.hi[rows, ids]
            if self.normalise:                     # softmax over the selected logits = full softmax renormalised
                wlo, whi = _softmax_interval(slo, shi)
            else:
                m = self.hi.amax(-1, keepdim=True)
                rel, g = 3 * U32, gamma(self.lo.shape[-1])
                dlo = (torch.exp(self.lo - m) * (1 - rel)).sum(-1, keepdim=True) * (1 - g)
                dhi = (torch.exp(self.hi - m) * (1 + rel)).sum(-1, keepdim=True) * (1 + g)
                wlo = torch.exp(slo - m) * (1 - rel) / dhi * (1 - 2 * U32)
                whi = torch.exp(shi - m) * (1 + rel) / dlo * (1 + 2 * U32)
            rep = Enclosure.of(wlo[~bad], whi[~bad], weights.dtype).check(weights.detach().cpu()[~bad])
            out["weights"] = rep
        out["ok"] = not out["invalid_rows"] and (weights is None or out["weights"].ok)
        return out


def route_enclosure(x: torch.Tensor, w_router: torch.Tensor, k: int, normalise: bool = True) -> RouteEnclosure:
    """Router logits ``x [rows, hidden] @ w_router[experts, hidden].T`` accumulated in fp32 in any order and kept in
    fp32 (the selection reads them before any storage rounding)."""
    xd, wd = _d(x), _d(w_router)
    exact, mag = xd @ wd.T, xd.abs() @ wd.abs().T
    err = gamma(xd.shape[-1]) * mag
    return RouteEnclosure(exact - err, exact + err, int(k), bool(normalise))
