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
            word = (raw >> 4) << hshift                       # a 32-bit little-endian word at hpos
            for byte in range(4):
                blob.index_put_((off + hpos.reshape(-1) + byte,), ((word >> (8 * byte)) & 255).reshape(-1), accumulate=True)
    assert int(blob.max()) <= 255                              # no two fields collided
    b8 = blob.to(torch.uint8)
    sc = torch.ones(16 * (d // 32), dtype=torch.float32).view(torch.uint8)
    b8[lay["k_scale"]:lay["v_code"]] = sc
    b8[lay["v_scale"]:lay["bytes"]] = sc
    k, v = eager.decode_cache_page(b8, d, kb, vb)
    assert torch.equal(k, want["k"].float()) and torch.equal(v, want["v"].float())


def test_six_bit_fragment_reconstruction_matches_layout():
    """The attention kernel rebuilds 6-bit code bytes as nibble | ((high-bit word >> s) & 0x30), one 32-bit word of
    high bits serving the two nibble words a lane loads together; the same arithmetic in Python must return the
    codes that the layout functions stored (this caught a carry bug in an earlier multiply-based spread)."""
    d = 128
    lay = eager.blob_layout(d, 6, 6)
    g = torch.Generator().manual_seed(0)
    tok = torch.arange(16)[:, None].expand(16, d)
    ch = torch.arange(d)[None, :].expand(16, d)
    blob = torch.zeros(lay["bytes"], dtype=torch.int64)
    want = {}
    for name, off in (("k", 0), ("v", lay["v_code"])):
        codes = torch.randint(-31, 32, (16, d), generator=g)
        want[name] = codes
        raw = codes + 32
        pos, shift = eager._k_pos(6, tok, ch) if name == "k" else eager._v_pos(6, d, tok, ch)
        blob.index_put_((off + pos.reshape(-1),), ((raw & 15) << shift).reshape(-1), accumulate=True)
        hpos, hshift = eager._k_hi_pos(d, tok, ch) if name == "k" else eager._v_hi_pos(d, tok, ch)
        word = (raw >> 4) << hshift
        for byte in range(4):
            blob.index_put_((off + hpos.reshape(-1) + byte,), ((word >> (8 * byte)) & 255).reshape(-1), accumulate=True)
    b = blob.tolist()
    u32 = lambda o: b[o] | b[o + 1] << 8 | b[o + 2] << 16 | b[o + 3] << 24          # noqa: E731
    m32, m = 0xFFFFFFFF, 0x30303030
    for cg in range(4):
        for gg in range(8):
            for t4 in range(4):
                hb = u32(1024 + cg * 128 + gg * 16 + t4 * 4)
                for nt in range(2):
                    w = u32(cg * 256 + (nt * 8 + gg) * 16 + t4 * 4)
                    h1, h2 = (hb, hb >> 2) if nt == 0 else ((hb << 4) & m32, (hb << 2) & m32)
                    lo, hi = (w & 0x0F0F0F0F) | (h1 & m), ((w >> 4) & 0x0F0F0F0F) | (h2 & m)
                    for e in range(4):
                        t = nt * 8 + gg
                        assert ((lo >> 8 * e) & 255) - 32 == int(want["k"][t, 32 * cg + 4 * t4 + e])
                        assert ((hi >> 8 * e) & 255) - 32 == int(want["k"][t, 32 * cg + 16 + 4 * t4 + e])
                chunk = (cg * 8 + gg) ^ ((t4 & 3) << 2)
                vo = lay["v_code"]
                lo, hi, hw = u32(vo + t4 * 128 + chunk * 4), u32(vo + (t4 + 4) * 128 + chunk * 4), u32(vo + 1024 + t4 * 128 + chunk * 4)
                parts = (((lo & 0x0F0F0F0F) | (hw & m), 2 * t4), (((lo >> 4) & 0x0F0F0F0F) | ((hw >> 2) & m), 2 * t4 + 1),
                         ((hi & 0x0F0F0F0F) | ((hw << 4) & m), 2 * t4 + 8), (((hi >> 4) & 0x0F0F0F0F) | ((hw << 2) & m), 2 * t4 + 9))
                for word, tk in parts:
                    for sub in range(4):
                        assert ((word >> 8 * sub) & 255) - 32 == int(want["v"][tk, (cg * 8 + gg) * 4 + sub])
