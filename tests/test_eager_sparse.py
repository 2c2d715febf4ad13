"""Sparse-family oracles against direct per-row loops."""
import math

import pytest
import torch

from cubic_serve_b200.ops import eager_sparse as E


def _select_loop(q, bk, visible, c, budget):
    B, T = visible.shape
    out = torch.full((B, T, budget + c - 1), -1, dtype=torch.int32)
    for b in range(B):
        for t in range(T):
            complete, tail = divmod(int(visible[b, t]), c)
            toks = []
            if complete:
                sc = (q[b, t].float() @ bk[b, :complete].float().t()).clamp_min(0).sum(0) / math.sqrt(q.shape[-1])
                best = sorted(range(complete), key=lambda n: (-float(sc[n]), n))[:budget // c]
                toks = [n * c + j for n in best for j in range(c)]
            toks += list(range(complete * c, complete * c + tail))
            out[b, t, :len(toks)] = torch.tensor(toks, dtype=torch.int32)
    return out


def test_block_selection_matches_the_loop_and_keeps_the_tail():
    g = torch.Generator().manual_seed(0)
    B, T, H, D, N, c, budget = 2, 5, 3, 16, 9, 4, 12
    q, bk = torch.randn(B, T, H, D, generator=g), torch.randn(B, N, D, generator=g)
    bk[0, 3] = bk[0, 1]                                       # a tie: the lower block index wins
    visible = torch.tensor([[0, 3, 4, 17, 36], [1, 9, 12, 13, 30]])
    got = E.select_blocks(q, bk, visible, c, budget)
    assert got.dtype == torch.int32 and got.shape == (B, T, budget + c - 1)
    assert torch.equal(got, _select_loop(q, bk, visible, c, budget))
    assert got[0, 0].tolist() == [-1] * 15 and got[0, 1].tolist()[:4] == [0, 1, 2, -1]       # only a tail
    row = got[0, 3].tolist()                                  # 17 visible: 4 complete blocks, 3 kept, tail token 16
    assert row[12] == 16 and row[13] == -1 and len(set(row[:12])) == 12
    with pytest.raises(ValueError):
        E.select_blocks(q, bk, visible, c, 10)                # not whole blocks
    with pytest.raises(ValueError):
        E.select_blocks(q, bk, visible + 100, c, budget)      # more visible tokens than pooled keys


def test_attention_over_selected_tokens():
    g = torch.Generator().manual_seed(1)
    B, H, Hkv, T, S, D = 2, 4, 2, 3, 20, 8
    q, k, v = torch.randn(B, H, T, D, generator=g), torch.randn(B, Hkv, S, D, generator=g), torch.randn(B, Hkv, S, D, generator=g)
    idx = torch.tensor([[[3, 1, 7, -1], [0, -1, -1, -1], [19, 18, 17, 16]], [[5, 5, -1, 2], [1, 2, 3, 4], [9, -1, 0, -1]]])
    got = E.attend_selected(q, k, v, idx)
    for b in range(B):
        for t in range(T):
            sel = [int(i) for i in idx[b, t] if i >= 0]
            for h in range(H):
                kk, vv = k[b, h // 2, sel], v[b, h // 2, sel]
                p = torch.softmax(kk @ q[b, h, t] / math.sqrt(D), 0)
                assert torch.allclose(got[b, h, t], p @ vv, atol=1e-5)
    with pytest.raises(ValueError):
        E.attend_selected(q, k, v, torch.full((B, T, 2), -1))


def test_stream_mixing_round_trip():
    g = torch.Generator().manual_seed(2)
    S, W, R, rows = 4, 16, 8, 5
    x = torch.randn(rows, S * W, generator=g)
    norm_w, down, up = torch.randn(S * W, generator=g) * 0.1, torch.randn(R, S * W, generator=g) * 0.2, torch.randn(S * W, R, generator=g)
    inp, n = E.stream_mix(x, norm_w, down, up, S, 1e-6)
    assert inp.shape == (rows, W) and n.shape == x.shape
    for r in range(rows):                                     # per-stream RMS of the normalised residual (before the weight) is 1
        groups = (n[r] / (1 + norm_w)).view(S, W)
        assert torch.allclose(groups.square().mean(-1), torch.ones(S), atol=1e-4)
    low = torch.nn.functional.silu(n @ down.t() / S)
    want = (torch.sigmoid(low @ up.t()) * n).view(rows, S, W).mean(1)
    assert torch.allclose(inp, want, atol=1e-5)
    gates = E.stream_injection(n, torch.randn(S, S * W, generator=g), S)
    assert gates.shape == (rows, S) and bool(((gates > 0) & (gates < 2)).all())
    out = torch.randn(rows, W, generator=g)
    y = E.stream_combine(x, out, gates)
    assert torch.allclose(y.view(rows, S, W)[2, 3], x.view(rows, S, W)[2, 3] + gates[2, 3] * out[2], atol=1e-6)
    with pytest.raises(ValueError):
        E.stream_mix(x, norm_w, down, up, 5, 1e-6)
    key, query, value = torch.randn(rows, 3, W, generator=g), torch.randn(rows, 3, W, generator=g), torch.randn(rows, W, generator=g)
    gated = E.signed_root_gate(key, query, value)
    s = (key * query).sum(-1) / math.sqrt(W)
    want = torch.sigmoid(s.sign() * s.abs().clamp_min(1e-6).sqrt())[..., None] * value[:, None, :]
    assert gated.shape == (rows, 3 * W) and torch.allclose(gated, want.flatten(-2), atol=1e-6)
