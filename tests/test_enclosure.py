"""Operator enclosures: the eager operators (and reorderings the contract allows) fall inside, implementations that
break the arithmetic contract fall outside, and the intervals are narrow enough to mean something."""
import math

import pytest
import torch

from cubic_serve_b200.guardrail import enclosure as E
from cubic_serve_b200.ops import eager

BF = torch.bfloat16


def _g(seed):
    return torch.Generator().manual_seed(seed)


def test_linear_any_order_inside_low_precision_outside():
    g = _g(1)
    x = torch.randn(8, 1024, generator=g).to(BF)
    w = (torch.randn(96, 1024, generator=g) * 0.05).to(BF)
    bias = torch.randn(96, generator=g).to(BF)
    enc = E.linear_enclosure(x, w, BF, bias=bias, partial_sums=4)
    plain = (x.float() @ w.float().T + bias.float()).to(BF)
    assert enc.check(plain)
    parts = [x[:, i:i + 256].float() @ w[:, i:i + 256].float().T for i in (768, 0, 512, 256)]     # split-K, odd order
    assert enc.check((parts[0] + parts[1] + parts[2] + parts[3] + bias.float()).to(BF))
    w_ulps = enc.width_ulps().flatten()                # wide only where the sum cancels (a small value of large terms)
    assert float(w_ulps.median()) <= 1.0 and float(w_ulps.quantile(0.9)) <= 8.0
    acc = torch.zeros(8, 96, dtype=BF)                                                            # a bf16 accumulator
    for i in range(0, 1024, 32):
        acc = (acc.float() + x[:, i:i + 32].float() @ w[:, i:i + 32].float().T).to(BF)
    bad = enc.check((acc.float() + bias.float()).to(BF))
    assert not bad and bad.outside > 100 and bad.index is not None
    dropped = x.clone()
    dropped[:, 1000:] = 0                                                                         # a lost k-tail
    rep = enc.check((dropped.float() @ w.float().T + bias.float()).to(BF))
    assert not rep and rep.worst_excess_ulps > 2
    with pytest.raises(ValueError):
        enc.check(plain[:4])
    nan = plain.clone()
    nan[0, 0] = float("nan")
    assert not enc.check(nan)


def test_rank_sum_order_free_and_a_missing_rank_is_seen():
    g = _g(2)
    parts = [torch.randn(16, 64, generator=g).to(BF) for _ in range(8)]
    res = torch.randn(16, 64, generator=g).to(BF)
    enc = E.rank_sum_enclosure(parts, BF, residual=res)
    fwd = sum(p.float() for p in parts) + res.float()
    rev = res.float() + sum(p.float() for p in reversed(parts))
    assert enc.check(fwd.to(BF)) and enc.check(rev.to(BF))
    assert not enc.check((fwd - parts[3].float()).to(BF))
    pairwise = fwd.clone()                       # a sum whose ranks were rounded to bf16 on the way (a bf16 ring)
    acc = res.clone()
    for p in parts:
        acc = (acc.float() + p.float()).to(BF)
    assert enc.check(acc).outside > 0


def test_rmsnorm_forms():
    g = _g(3)
    x = (torch.randn(6, 512, generator=g) * 3).to(BF)
    w = (1 + 0.2 * torch.randn(512, generator=g)).to(BF)
    enc = E.rmsnorm_enclosure(x, w, 1e-6, BF)
    assert enc.check(eager.rmsnorm(x, w, 1e-6).to(BF))
    assert float(enc.width_ulps().max()) <= 2.0
    assert not enc.check(eager.rmsnorm(x, w, 1e-2).to(BF))                                   # another epsilon
    wz = (w.float() - 1).to(BF)
    zc = E.rmsnorm_enclosure(x, wz, 1e-6, BF, zero_centered=True)
    assert zc.check(eager.rmsnorm(x, wz, 1e-6, zero_centered=True).to(BF))
    xf = x.float()
    two_step = w.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(BF).float()
    assert E.rmsnorm_enclosure(x, w, 1e-6, BF, round_before_weight=True).check(two_step.to(BF))
    assert enc.check(two_step.to(BF)).outside > 0                                            # the extra rounding shows


def test_activation_and_router_softmax():
    g = _g(4)
    gate, up = (torch.randn(4, 256, generator=g) * 4).to(BF), torch.randn(4, 256, generator=g).to(BF)
    enc = E.silu_mul_enclosure(gate, up, BF)
    assert enc.check(eager.swiglu(torch.cat([gate, up], -1)).to(BF))
    assert float(enc.width_ulps().max()) <= 1.0
    gelu = torch.nn.functional.gelu(gate.float()) * up.float()
    assert not enc.check(gelu.to(BF))
    assert E.sigmoid_enclosure(gate, BF).check(torch.sigmoid(gate.float()).to(BF))
    logits = torch.randn(32, 8, generator=g) * 3
    rs = E.softmax_enclosure(logits, torch.float32)
    assert rs.check(torch.softmax(logits, -1))
    assert rs.check(torch.softmax(logits.double(), -1).float())
    assert not rs.check(torch.softmax(logits.to(torch.float16), -1).float())                 # half-precision exponentials
    assert not rs.check(torch.softmax(logits, -1) * (1 + 1e-5))


def _online_attention(q, k, v, scale, tile):
    """Running-maximum form with bf16 weights into the value product (the shape of a tensor-core kernel)."""
    h, n, d = k.shape
    m = torch.full((h,), -float("inf"))
    l = torch.zeros(h)
    acc = torch.zeros(h, d)
    for t0 in range(0, n, tile):
        s = torch.einsum("hd,hnd->hn", q.float(), k[:, t0:t0 + tile].float()) * scale
        m_new = torch.maximum(m, s.amax(-1))
        a = torch.exp(m - m_new)
        p = torch.exp(s - m_new[:, None])
        l = l * a + p.sum(-1)
        acc = acc * a[:, None] + torch.einsum("hn,hnd->hd", p.to(BF).float(), v[:, t0:t0 + tile].float())
        m = m_new
    return acc / l[:, None]


def test_attention_on_decoded_cache_entries():
    g = _g(5)
    h, n, d = 4, 200, 64
    q = torch.randn(h, d, generator=g).to(BF)
    kc, ks = eager.kv_quantize(torch.randn(h, n, d, generator=g), 8)
    vc, vs = eager.kv_quantize(torch.randn(h, n, d, generator=g), 4)
    k, v = eager.kv_dequantize(kc.float(), ks.float()), eager.kv_dequantize(vc.float(), vs.float())
    scale = 1 / math.sqrt(d)
    enc = E.attention_enclosure(q, k, v, scale, BF, p_dtype=BF, tiles=4)
    direct = torch.einsum("hn,hnd->hd", torch.softmax(torch.einsum("hd,hnd->hn", q.float(), k) * scale, -1), v)
    assert enc.check(direct.to(BF))
    assert enc.check(_online_attention(q, k, v, scale, 64).to(BF))
    exact = E.attention_enclosure(q, k, v, scale, BF, p_dtype=None, tiles=1)
    assert exact.check(direct.to(BF)) and float(exact.width_ulps().flatten().quantile(0.9)) <= 2.0
    # weights stored in bf16 cost 2**-9 of sum(p |v|); the output of zero-mean values is ~ sqrt(n) smaller than that sum
    assert float(enc.width_ulps().median()) <= 32.0
    short = torch.einsum("hn,hnd->hd", torch.softmax(torch.einsum("hd,hnd->hn", q.float(), k[:, :-1]) * scale, -1), v[:, :-1])
    assert not enc.check(short.to(BF))                                                       # the newest key was not read
    other_scale = torch.einsum("hn,hnd->hd", torch.softmax(torch.einsum("hd,hnd->hn", q.float(), k) * scale * 1.02, -1), v)
    assert not exact.check(other_scale.to(BF))


def test_delta_rule_step_and_a_state_kept_in_bf16():
    g = _g(6)
    h, dv, dk = 2, 32, 32
    S = torch.randn(h, dv, dk, generator=g) * 0.3
    q = torch.nn.functional.normalize(torch.randn(h, dk, generator=g), dim=-1).to(BF).float() * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(h, dk, generator=g), dim=-1).to(BF).float()
    v = torch.randn(h, dv, generator=g).to(BF).float()
    decay, beta = torch.rand(h, generator=g) * 0.2 + 0.8, torch.rand(h, generator=g)
    s_enc, o_enc = E.delta_rule_enclosure(S, q, k, v, decay, beta)
    S1 = S * decay[:, None, None]
    S2 = S1 + ((v - (S1 * k[:, None, :]).sum(-1)) * beta[:, None])[:, :, None] * k[:, None, :]
    o = (S2 * q[:, None, :]).sum(-1)
    assert s_enc.check(S2) and o_enc.check(o.to(BF))
    assert float(s_enc.width_ulps().median()) <= 512                 # fp32 spacings: 9 of the 24 mantissa bits
    # another association of the same sums (decay applied to the memory read and to the state separately)
    mem = decay[:, None] * (S * k[:, None, :]).sum(-1)
    alt = decay[:, None, None] * S + ((v - mem) * beta[:, None])[:, :, None] * k[:, None, :]
    assert s_enc.check(alt)
    assert not s_enc.check(S2.to(BF).float())                        # a state stored in bf16 between tokens
    assert not s_enc.check(S1 + ((v - (S1 * k[:, None, :]).sum(-1)))[:, :, None] * k[:, None, :])   # beta forgotten


def test_guards():
    with pytest.raises(ValueError):
        E.linear_enclosure(torch.full((1, 4), float("inf")), torch.ones(2, 4))
    with pytest.raises(ValueError):
        E.gamma(1 << 24)
    assert E.gamma(1) > 0


def test_layer_audit_names_the_one_wrong_operator():
    clean = E.audit_layer_operators(seed=3)
    assert [n for n, _ in clean] == ["input_norm", "q_proj", "attention", "o_proj+residual", "post_norm", "gate_proj",
                                     "up_proj", "silu_mul", "down_proj+residual"]
    assert all(r.ok for _, r in clean), [(n, r) for n, r in clean if not r.ok]

    class Tanh(E.EagerOperators):
        def silu_mul(self, gate, up):                      # another activation
            return (torch.nn.functional.gelu(gate.float(), approximate="tanh") * up.float()).to(BF)

    class Bf16Norm(E.EagerOperators):
        def rmsnorm(self, x, w, eps):                      # the mean square accumulated in bf16
            ms = torch.zeros(x.shape[0], 1, dtype=BF)
            for i in range(x.shape[-1]):
                ms = (ms.float() + x[:, i:i + 1].float() ** 2).to(BF)
            return (x.float() * torch.rsqrt(ms.float() / x.shape[-1] + eps) * w.float()).to(BF)

    bad = dict(E.audit_layer_operators(Tanh(), seed=3))
    assert [n for n, r in bad.items() if not r.ok] == ["silu_mul"]        # what follows is judged on its own inputs
    bad = dict(E.audit_layer_operators(Bf16Norm(), seed=3))
    assert [n for n, r in bad.items() if not r.ok] == ["input_norm", "post_norm"]


def test_routing_must_may_sets_and_near_ties():
    g = _g(9)
    x = torch.randn(64, 256, generator=g).to(BF)
    w = (torch.randn(16, 256, generator=g) * 0.06).to(BF)
    w[5] = w[4]                                                # two experts with the same row: a tie wherever they rank
    x[7] = 0
    x[7, 0] = 1                                                # a row whose logits are single products: no slack at all
    enc = E.route_enclosure(x, w, k=4, normalise=True)
    logits = x.float() @ w.float().T
    top = logits.topk(4, -1)
    weights = torch.softmax(top.values, -1)
    rep = enc.check(top.indices, weights)
    assert rep["ok"] and not rep["invalid_rows"]
    # another order of the sums picks other experts only on rows the enclosure calls ambiguous
    rev = (x.float().flip(-1) @ w.float().flip(-1).T).topk(4, -1)
    differ = {r for r in range(64) if set(rev.indices[r].tolist()) != set(top.indices[r].tolist())}
    assert differ <= set(rep["ambiguous_rows"])
    assert enc.check(rev.indices, torch.softmax(rev.values, -1))["ok"]
    tied = [r for r in range(64) if (4 in top.indices[r]) != (5 in top.indices[r])]
    assert tied and set(tied) <= set(rep["ambiguous_rows"])     # the twin experts straddle the cut somewhere
    swapped = top.indices.clone()
    r = tied[0]
    swapped[r] = torch.where(swapped[r] == 4, 5, torch.where(swapped[r] == 5, 4, swapped[r]))
    assert enc.check(swapped)["ok"]                            # either twin is a right answer
    wrong = top.indices.clone()
    clear = next(r for r in range(64) if r not in rep["ambiguous_rows"])
    wrong[clear, 0] = logits[clear].argmin()
    assert enc.check(wrong)["invalid_rows"] == [clear]
    assert not enc.check(top.indices, weights * 1.001)["ok"]
    plain = E.route_enclosure(x, w, k=4, normalise=False)
    assert plain.check(top.indices, torch.softmax(logits, -1).gather(1, top.indices))["ok"]
    assert not plain.check(top.indices, weights)["ok"]         # renormalised weights where plain ones are declared
