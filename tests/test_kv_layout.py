"""The physical KV blob layout as the eager oracle reads it: every (token, channel) has its own bits."""
import pytest
import torch

from cubic_serve_b200.ops import eager


@pytest.mark.parametrize("kb,vb", [(8, 8), (6, 6), (4, 4), (6, 8), (4, 6)])
def test_blob_positions_are_a_bijection(kb, vb):
    d = 128
    lay = eager.blob_layout(d, kb, vb)
    assert lay["bytes"] == 16 * d * (kb + vb) // 8 + 2 * 16 * (d // 32) * 4
    g = torch.Generator().manual_seed(kb * 10 + vb)
    blob = torch.zeros(lay["bytes"], dtype=torch.int64)
    tok = torch.arange(16)[:, None].expand(16, d)
    ch = torch.arange(d)[None, :].expand(16, d)
    want = {}
    for name, bits, off in (("k", kb, 0), ("v", vb, lay["v_code"])):
        codes = torch.randint(-(2 ** (bits - 1)) + 1, 2 ** (bits - 1), (16, d), generator=g)
        want[name] = codes
        raw = codes + 2 ** (bits - 1)
        pos, shift = (eager._k_pos(bits, tok, ch) if name == "k" else eager._v_pos(bits, d, tok, ch))
        low = raw & 15 if bits == 6 else raw
        blob.index_put_((off + pos.reshape(-1),), (low << shift).reshape(-1), accumulate=True)   # disjoint bit fields
        if bits == 6:
            hpos, hshift = (eager._k_hi_pos(d, tok, ch) if name == "k" else eager._v_hi_pos(d, tok, ch))
            word = (raw >> 4) << hshift                       # a 16-bit little-endian word at hpos
            blob.index_put_((off + hpos.reshape(-1),), (word & 255).reshape(-1), accumulate=True)
            blob.index_put_((off + hpos.reshape(-1) + 1,), (word >> 8).reshape(-1), accumulate=True)
    assert int(blob.max()) <= 255                              # no two fields collided
    b8 = blob.to(torch.uint8)
    sc = torch.ones(16 * (d // 32), dtype=torch.float32).view(torch.uint8)
    b8[lay["k_scale"]:lay["v_code"]] = sc
    b8[lay["v_scale"]:lay["bytes"]] = sc
    k, v = eager.decode_cache_page(b8, d, kb, vb)
    assert torch.equal(k, want["k"].float()) and torch.equal(v, want["v"].float())
