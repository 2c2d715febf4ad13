"""Numerics of every native kernel against fp32 PyTorch oracles (needs a B200)."""
import math

import pytest
import torch

from cubic_serve_b200.ops import eager, wq_pack
from cubic_serve_b200.quantization import cubic

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _k():
    from cubic_serve_b200.ops import kernels
    return kernels


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _cubic_weight(n, k, seed=0, group=128):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    scheme = cubic.CubicScheme(bits=4, group_in=group)
    payload = cubic.quantize(w, scheme)
    dense = cubic.decode(payload, scheme, (n, k))
    codes = cubic.unpack_codes(payload["weight_packed"], 4, k)
    pw = wq_pack.pack_cubic4(codes, payload["weight_scale"], payload["weight_a"], payload["weight_b"], group)
    return pw, dense


@pytest.mark.parametrize("m,n,k,splits", [(1, 128, 256, 1), (16, 256, 512, 1), (40, 384, 1024, 1),
                                          (256, 256, 4096, 1), (300, 128, 512, 1), (64, 200, 512, 1),
                                          (32, 256, 2048, 4), (256, 128, 4096, 3)])
def test_wq_gemm_cubic4(m, n, k, splits):
    K = _k()
    pw, dense = _cubic_weight(n, k, seed=m + n)
    # the packed levels are the fp32 decode rounded once to bf16 (the reference's contract), bit for bit
    assert torch.equal(wq_pack.unpack_to_dense(pw), dense.to(torch.bfloat16).float())
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16)
    ref = x.float() @ dense.t()
    y = K.wq_gemm(x.to(DEV), pw.to(DEV), splits=splits)
    torch.cuda.synchronize()
    K.workspace(y.device).check_status()
    assert y.shape == (m, n)
    assert _rel(y.cpu(), ref) < 1e-2
    # against the same bf16 weights the kernel decodes, only the fp32 accumulation order and the output rounding differ
    assert _rel(y.cpu(), x.float() @ wq_pack.unpack_to_dense(pw).t()) < 3e-3
    # repeat: split-K counters must have been restored
    y2 = K.wq_gemm(x.to(DEV), pw.to(DEV), splits=splits)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("m,n,k,min_units", [
    (1, 128, 256, 0), (16, 256, 512, 0), (40, 384, 1024, 0), (300, 128, 512, 0), (64, 200, 512, 0),
    (256, 256, 4096, 0),            # automatic schedule: tiles split into several runs
    (32, 256, 2048, 1),             # one k-block per run: 32 parts per tile
    (256, 384, 4096, 3),            # runs that straddle tile boundaries (64 k-blocks per tile, 3 per run)
    (48, 1280, 1024, 5),            # ten tiles, runs of five k-blocks, some CTAs own two partial runs
    (520, 640, 512, 2),             # three row tiles (256 + 256 + 8 rows)
    (16, 128 * 150, 256, 0),        # more tiles than SMs: whole tiles + a streamed remainder
    (272, 128 * 80, 256, 1),        # two row tiles x 80 column tiles = 160 tiles, streamed remainder of 12
])
def test_wq_gemm_stream_k(m, n, k, min_units):
    """The persistent stream-K kernel against the fp32 oracle, including forced many-part tiles."""
    K = _k()
    pw, dense = _cubic_weight(n, k, seed=m + n)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16)
    ref = x.float() @ dense.t()
    res = torch.randn(m, n, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    y = K.wq_gemm(x.to(DEV), pw.to(DEV), min_units=min_units)
    torch.cuda.synchronize()
    K.workspace(y.device).check_status()
    assert _rel(y.cpu(), ref) < 1e-2
    assert _rel(K.wq_gemm(x.to(DEV), pw.to(DEV)).cpu(), ref) < 1e-2     # whichever kernel the dispatcher picks
    # again with a residual: counters must have been restored, the fix-up adds the residual exactly once
    y2 = K.wq_gemm(x.to(DEV), pw.to(DEV), residual=res.to(DEV), min_units=min_units)
    torch.cuda.synchronize()
    K.workspace(y.device).check_status()
    assert _rel(y2.cpu(), ref + res.float()) < 1e-2
    assert torch.equal(K.wq_gemm(x.to(DEV), pw.to(DEV), min_units=min_units), y)      # deterministic


@pytest.mark.parametrize("m,inter,k,splits,min_units", [
    (1, 64, 256, 1, None), (40, 192, 1024, 1, None), (300, 128, 512, 1, None),     # per-tile kernel, staged epilogue
    (16, 80, 512, 1, None),                                                        # last tile only partly filled
    (64, 256, 2048, 4, None),                                                      # per-tile kernel, split-K fix-up
    (16, 256, 512, None, 0), (256, 192, 4096, None, 0),                            # persistent kernel, own schedule
    (32, 128, 2048, None, 1), (256, 192, 4096, None, 3), (48, 640, 1024, None, 5),  # many-part tiles, deferred fix-ups
    (520, 320, 512, None, 2), (16, 64 * 150, 256, None, 0),                        # row tiles; more tiles than SMs
])
def test_wq_gemm_fused_swiglu(m, inter, k, splits, min_units):
    """SwiGLU in the GEMM epilogue (interleaved gate / up rows) against the two-kernel path and the fp32 oracle."""
    K = _k()
    pw, dense = _cubic_weight(2 * inter, k, seed=m + inter)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16)
    ref = eager.swiglu((x.float() @ dense.t()).to(torch.bfloat16))
    pwi = wq_pack.swiglu_interleave(pw).to(DEV)
    assert pwi.act_interleaved and not pw.act_interleaved
    act = K.wq_gemm_act(x.to(DEV), pwi, splits=splits, min_units=min_units)
    torch.cuda.synchronize()
    K.workspace(act.device).check_status()
    assert act.shape == (m, inter)
    assert _rel(act.cpu(), ref) < 1.5e-2
    # the same kernel and schedule without the fusion (the interleaved matrix as a plain weight: a row keeps its
    # tile, hence its split points along K), columns put back in [gate | up] order, then the activation kernel:
    # identical values
    plain = wq_pack.PackedWeight(pwi.fmt, pwi.n, pwi.k, pwi.group_k, pwi.codes, pwi.meta, pwi.alpha)
    gu_i = K.wq_gemm(x.to(DEV), plain, splits=splits, min_units=min_units)
    gu = torch.empty_like(gu_i)
    gu[:, wq_pack.swiglu_row_order(inter).to(DEV)] = gu_i
    assert torch.equal(act, K.swiglu(gu))
    # into a wider buffer (row stride > inter), and whichever kernel the dispatcher picks
    wide = torch.zeros(m, inter + 64, dtype=torch.bfloat16, device=DEV)
    K.wq_gemm_act(x.to(DEV), pwi, out=wide[:, :inter], splits=splits, min_units=min_units)
    assert torch.equal(wide[:, :inter], act) and not wide[:, inter:].any()
    assert _rel(K.wq_gemm_act(x.to(DEV), pwi).cpu(), ref) < 1.5e-2


def test_wq_gemm_fused_swiglu_other_formats():
    K = _k()
    m, inter, k = 48, 128, 512
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    q = torch.randint(0, 16, (2 * inter, k), generator=g, dtype=torch.uint8)
    scale = torch.rand(2 * inter, k // 64, generator=g) * 0.01 + 0.001
    zero = torch.randint(0, 16, (2 * inter, k // 64), generator=g).float()
    packed = torch.randint(0, 256, (2 * inter, k // 2), generator=g, dtype=torch.uint8)
    bs = (torch.rand(2 * inter, k // 16, generator=g) * 2 + 0.25).to(torch.float8_e4m3fn)
    for pw in (wq_pack.pack_affine4(q, scale, -zero * scale, 64), wq_pack.pack_nvfp4(packed, bs.float(), 0.01),
               wq_pack.pack_bf16(torch.randn(2 * inter, k, generator=g) * 0.05)):
        pwi = wq_pack.swiglu_interleave(pw).to(DEV)
        plain = wq_pack.PackedWeight(pwi.fmt, pwi.n, pwi.k, pwi.group_k, pwi.codes, pwi.meta, pwi.alpha)
        order = wq_pack.swiglu_row_order(inter).to(DEV)
        for kw in ({"splits": 1}, {"min_units": 2}):
            gu_i = K.wq_gemm(x, plain, **kw)
            gu = torch.empty_like(gu_i)
            gu[:, order] = gu_i
            assert torch.equal(K.wq_gemm_act(x, pwi, **kw), K.swiglu(gu))
            assert _rel(gu, K.wq_gemm(x, pw.to(DEV), **kw)) < 2e-3


@pytest.mark.parametrize("m,n,k,min_units", [
    (256, 256, 4096, 0), (256, 512, 4096, 0),     # one pair-tile, two pair-tiles, automatic schedule
    (256, 1024, 1024, 3),                         # runs of three k-blocks that straddle pair-tile boundaries
    (300, 512, 512, 2),                           # two row tiles, the second with 44 rows (rank 1's half is all padding)
    (512, 128 * 40, 256, 0),                      # 40 pair-tiles on 74 pairs
    (272, 128 * 160, 256, 1),                     # more pair-tiles than pairs: whole pair-tiles + a streamed remainder
    (4096, 1024, 512, 0),                         # a prefill chunk: 16 row tiles
])
def test_wq_gemm_stream_k_cta_pairs(m, n, k, min_units):
    """Persistent kernel on CTA pairs (cta_group::2, M = 256 MMAs, half an activation tile per CTA) against the
    fp32 oracle and against the same launch with pairs switched off."""
    from cubic_serve_b200.ops import native
    K = _k()
    pw, dense = _cubic_weight(n, k, seed=m + n)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16)
    ref = x.float() @ dense.t()
    res = torch.randn(m, n, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    lib = native.lib()
    try:
        lib.cb_wq_gemm_pair_mode(2)
        y = K.wq_gemm(x.to(DEV), pw.to(DEV), min_units=min_units)
        torch.cuda.synchronize()
        K.workspace(y.device).check_status()
        assert _rel(y.cpu(), ref) < 1e-2
        y2 = K.wq_gemm(x.to(DEV), pw.to(DEV), residual=res.to(DEV), min_units=min_units)
        torch.cuda.synchronize()
        K.workspace(y.device).check_status()
        assert _rel(y2.cpu(), ref + res.float()) < 1e-2
        assert torch.equal(K.wq_gemm(x.to(DEV), pw.to(DEV), min_units=min_units), y)      # deterministic
        lib.cb_wq_gemm_pair_mode(0)
        single = K.wq_gemm(x.to(DEV), pw.to(DEV), min_units=min_units)
        assert _rel(y, single) < 2e-3
        # bf16 weights (TMA-loaded A tiles of both CTAs complete on rank 0's barrier) and the fused activation
        lib.cb_wq_gemm_pair_mode(2)
        wb = (torch.randn(n, k, generator=torch.Generator().manual_seed(3)) * 0.05).to(torch.bfloat16)
        yb = K.wq_gemm(x.to(DEV), wq_pack.pack_bf16(wb).to(DEV), min_units=min_units)
        assert _rel(yb.cpu(), x.float() @ wb.float().t()) < 1e-2
        pwi = wq_pack.swiglu_interleave(pw).to(DEV)
        act = K.wq_gemm_act(x.to(DEV), pwi, min_units=min_units)
        assert _rel(act.cpu(), eager.swiglu(ref.to(torch.bfloat16))) < 1.5e-2
        torch.cuda.synchronize()
        K.workspace(y.device).check_status()
    finally:
        lib.cb_wq_gemm_pair_mode(1)


def test_wq_gemm_stream_k_bf16_weights():
    K = _k()
    for m, n, k, mu in ((48, 256, 512, 0), (256, 1000, 1024, 2), (24, 128 * 150 + 40, 256, 0)):
        g = torch.Generator().manual_seed(n)
        w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16)
        x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16)
        y = K.wq_gemm(x.to(DEV), wq_pack.pack_bf16(w).to(DEV), min_units=mu)
        torch.cuda.synchronize()
        K.workspace(y.device).check_status()
        assert _rel(y.cpu(), x.float() @ w.float().t()) < 1e-2


def test_wq_gemm_residual_and_bf16():
    K = _k()
    m, n, k = 48, 256, 512
    w = (torch.randn(n, k) * 0.05).to(torch.bfloat16)
    x = (torch.randn(m, k) * 0.5).to(torch.bfloat16)
    res = torch.randn(m, n).to(torch.bfloat16)
    ref = x.float() @ w.float().t() + res.float()
    y = K.wq_gemm(x.to(DEV), wq_pack.pack_bf16(w).to(DEV), residual=res.to(DEV))
    assert _rel(y.cpu(), ref) < 1e-2


def test_wq_gemm_affine4_and_nvfp4():
    K = _k()
    m, n, k = 32, 256, 512
    g = torch.Generator().manual_seed(3)
    q = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
    scale = (torch.rand(n, k // 64, generator=g) * 0.01 + 0.001)
    zero = torch.randint(0, 16, (n, k // 64), generator=g).float()
    pw = wq_pack.pack_affine4(q, scale, -zero * scale, 64)
    dense = wq_pack.unpack_to_dense(pw)
    expect = (q.float() - zero.repeat_interleave(64, 1)) * scale.half().float().repeat_interleave(64, 1)
    assert _rel(dense, expect) < 4e-3
    x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16)
    y = K.wq_gemm(x.to(DEV), pw.to(DEV))
    assert _rel(y.cpu(), x.float() @ dense.to(torch.bfloat16).float().t()) < 1e-2

    packed = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    bs = (torch.rand(n, k // 16, generator=g) * 2 + 0.25).to(torch.float8_e4m3fn)
    pw4 = wq_pack.pack_nvfp4(packed, bs.float(), 0.01)
    dense4 = wq_pack.unpack_to_dense(pw4)
    y4 = K.wq_gemm(x.to(DEV), pw4.to(DEV))
    assert _rel(y4.cpu(), x.float() @ (dense4 / 0.01).to(torch.bfloat16).float().t() * 0.01) < 1e-2


def test_rmsnorm_swiglu_embedding():
    K = _k()
    x = torch.randn(37, 4096).to(torch.bfloat16).to(DEV)
    w = torch.randn(4096).to(torch.bfloat16).to(DEV)
    res = torch.randn(37, 4096).to(torch.bfloat16).to(DEV)
    assert _rel(K.rmsnorm(x, w, 1e-6), eager.rmsnorm(x, w, 1e-6)) < 5e-3
    summed = (x.float() + res.float()).to(torch.bfloat16)
    res2 = res.clone()
    out = K.rmsnorm(x, w, 1e-6, residual=res2, zero_centered=True)
    assert torch.equal(res2, summed)
    assert _rel(out, eager.rmsnorm(summed, w, 1e-6, zero_centered=True)) < 5e-3
    gu = torch.randn(19, 2 * 1536).to(torch.bfloat16).to(DEV)
    assert _rel(K.swiglu(gu), eager.swiglu(gu)) < 5e-3
    table = torch.randn(1000, 256).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([5, 999, 0, 1200, 17], dtype=torch.int32, device=DEV)
    e = K.embedding(ids, table)
    assert torch.equal(e[0], table[5]) and torch.equal(e[1], table[999]) and bool((e[3] == 0).all())


def _make_cache(pages, hkv, d, kb, vb):
    blob = eager.blob_layout(d, kb, vb)["bytes"]
    assert blob == _k().kv_blob_bytes(d, kb, vb)
    return torch.zeros(pages, hkv, blob, dtype=torch.uint8, device=DEV)


@pytest.mark.parametrize("kb,vb", [(8, 8), (4, 8), (4, 4), (8, 4), (6, 6), (6, 8), (4, 6)])
def test_rope_kv_write_roundtrip(kb, vb):
    K = _k()
    hq, hkv, d, t = 8, 2, 128, 37
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(t, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.arange(100, 100 + t, dtype=torch.int32, device=DEV)
    pages = torch.randperm(8, generator=g)[: (t + 15) // 16].to(torch.int32)
    slots = (pages[torch.arange(t) // 16] * 16 + torch.arange(t) % 16).to(torch.int32).to(DEV)
    slots[3] = -1  # padding row: nothing written
    cache = _make_cache(8, hkv, d, kb, vb)
    inv = eager.rope_inv_freq(d, 1e6, DEV)
    qn = (torch.rand(d, generator=g) + 0.5).to(torch.bfloat16).to(DEV)
    kn = (torch.rand(d, generator=g) + 0.5).to(torch.bfloat16).to(DEV)
    q_out = torch.empty(t, hq * d, dtype=torch.bfloat16, device=DEV)
    K.rope_kv_write(qkv, q_out, cache, pos, slots, inv, hq, hkv, d, kb, vb, q_norm=qn, k_norm=kn, eps=1e-6)
    x = qkv.view(t, hq + 2 * hkv, d)
    qr = eager.rope(eager.rmsnorm(x[:, :hq], qn, 1e-6).to(torch.bfloat16), pos, inv)
    kr = eager.rope(eager.rmsnorm(x[:, hq:hq + hkv], kn, 1e-6).to(torch.bfloat16), pos, inv).to(torch.bfloat16).float()
    vr = x[:, hq + hkv:].float()
    assert _rel(q_out.view(t, hq, d), qr) < 5e-3
    kq, ksc = eager.kv_quantize(kr, kb)
    vq, vsc = eager.kv_quantize(vr, vb)
    kd, vd = eager.kv_dequantize(kq, ksc), eager.kv_dequantize(vq, vsc)
    for tok in range(t):
        if tok == 3:
            continue
        page, off = int(slots[tok]) // 16, int(slots[tok]) % 16
        for h in range(hkv):
            kk, vv = eager.decode_cache_page(cache[page, h], d, kb, vb)
            # one code step of slack where rounding sits on a tie after bf16 effects
            assert (kk[off] - kd[tok, h]).abs().max() <= ksc[tok, h].max() * 1.01
            assert _rel(kk[off], kd[tok, h]) < {8: 0.02, 6: 0.06, 4: 0.2}[kb]
            assert (vv[off] - vd[tok, h]).abs().max() <= vsc[tok, h].max() * 1.01
            assert _rel(vv[off], vd[tok, h]) < {8: 0.01, 6: 0.03, 4: 0.1}[vb]


def _fill_cache_random(cache, t_total, hkv, d, kb, vb, page_ids, seed=0):
    """Write random K/V for tokens 0..t_total-1 of one request through the write kernel."""
    K = _k()
    g = torch.Generator().manual_seed(seed)
    hq = hkv
    qkv = torch.randn(t_total, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.arange(t_total, dtype=torch.int32, device=DEV)
    slots = (page_ids[torch.arange(t_total) // 16] * 16 + torch.arange(t_total) % 16).to(torch.int32).to(DEV)
    q_out = torch.empty(t_total, hq * d, dtype=torch.bfloat16, device=DEV)
    K.rope_kv_write(qkv, q_out, cache, pos, slots, eager.rope_inv_freq(d, 1e4, DEV), hq, hkv, d, kb, vb,
                    rotary_dim=0)


def _dense_kv(cache, page_ids, t_total, hkv, d, kb, vb):
    ks, vs = [], []
    for p in page_ids.tolist():
        kh, vh = zip(*[eager.decode_cache_page(cache[p, h], d, kb, vb) for h in range(hkv)])
        ks.append(torch.stack(kh, 1))
        vs.append(torch.stack(vh, 1))
    return torch.cat(ks)[:t_total], torch.cat(vs)[:t_total]


@pytest.mark.parametrize("kb,vb,hq,hkv,splits", [(8, 8, 8, 2, 1), (8, 8, 8, 2, 3), (4, 8, 16, 2, 1),
                                                 (4, 4, 8, 1, 2), (8, 4, 16, 1, 1), (6, 6, 8, 2, 1), (6, 8, 16, 2, 2),
                                                 (8, 6, 8, 1, 1), (4, 6, 8, 2, 1), (6, 4, 16, 1, 3)])
def test_paged_attention_decode(kb, vb, hq, hkv, splits):
    K = _k()
    d = 128
    lens = [1, 17, 100, 333]
    n_pages = 64
    cache = _make_cache(n_pages, hkv, d, kb, vb)
    cache.view(torch.float32)[:] = float("nan")  # stale slots must not leak into the result
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(7)).to(torch.int32)
    max_pages = 24
    table = torch.zeros(len(lens), max_pages, dtype=torch.int32)
    used = 0
    dense = []
    for r, ln in enumerate(lens):
        np_ = (ln + 15) // 16
        ids = perm[used:used + np_]
        used += np_
        table[r, :np_] = ids
        _fill_cache_random(cache, ln, hkv, d, kb, vb, ids, seed=r)
        dense.append(_dense_kv(cache, ids, ln, hkv, d, kb, vb))
    q = torch.randn(len(lens), hq, d, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(DEV)
    out = torch.zeros_like(q)
    ar = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    K.paged_attention(q, out, cache, table.to(DEV), ar, ar.clone(), torch.ones_like(ar),
                      torch.tensor(lens, dtype=torch.int32, device=DEV), hq, hkv, d, kb, vb, splits=splits)
    torch.cuda.synchronize()
    K.workspace(q.device).check_status()
    for r, ln in enumerate(lens):
        k, v = dense[r]
        ref = eager.attention_rows(q[r:r + 1], k, v, torch.tensor([ln], device=DEV))
        assert _rel(out[r:r + 1], ref) < 2e-2, (r, ln)


def test_paged_attention_prefill_rows():
    """Causal chunk: 4 positions x 4 heads per row block, context from earlier pages."""
    K = _k()
    kb = vb = 8
    hq, hkv, d = 8, 2, 128
    g_ = hq // hkv
    qb = 16 // g_
    total, chunk_start = 77, 30          # tokens 30..76 are the query chunk
    n_pages = 8
    cache = _make_cache(n_pages, hkv, d, kb, vb)
    ids = torch.tensor([5, 2, 7, 0, 3], dtype=torch.int32)
    _fill_cache_random(cache, total, hkv, d, kb, vb, ids, seed=11)
    k, v = _dense_kv(cache, ids, total, hkv, d, kb, vb)
    nq = total - chunk_start
    q = torch.randn(nq, hq, d, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    out = torch.zeros_like(q)
    table = torch.zeros(1, 8, dtype=torch.int32)
    table[0, :5] = ids
    nblk = (nq + qb - 1) // qb
    starts = torch.arange(nblk, dtype=torch.int32) * qb
    K.paged_attention(q, out, cache, table.to(DEV), torch.zeros(nblk, dtype=torch.int32, device=DEV),
                      starts.to(DEV), torch.clamp(nq - starts, max=qb).to(torch.int32).to(DEV),
                      (chunk_start + starts + 1).to(torch.int32).to(DEV), hq, hkv, d, kb, vb)
    vis = torch.arange(chunk_start + 1, total + 1, device=DEV)
    ref = eager.attention_rows(q, k, v, vis)
    assert _rel(out, ref) < 2e-2


def test_sampler():
    K = _k()
    rows, vocab = 6, 5000
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(rows, vocab, generator=g).to(torch.bfloat16)
    logits[0, 77] = logits[0, 4000] = 9.0   # tie: lowest id wins
    lg = logits.to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample(lg, out)
    expect = [int((logits[r].float() == logits[r].float().max()).nonzero()[0]) for r in range(rows)]
    assert out.tolist() == expect and out[0].item() == 77
    # grammar mask: only ids 10..19 allowed
    mask = torch.zeros(rows, (vocab + 31) // 32, dtype=torch.int32)
    mask[:, 0] = sum(1 << b for b in range(10, 20))
    K.sample(lg, out, mask=mask.to(DEV))
    assert out.tolist() == [10 + int(logits[r, 10:20].float().argmax()) for r in range(rows)]
    # stochastic: top_k = 3 draws stay inside the top-3 set and follow the seed
    temp = torch.full((rows,), 0.8, device=DEV)
    top_k = torch.full((rows,), 3, dtype=torch.int32, device=DEV)
    top_p = torch.full((rows,), 1.0, device=DEV)
    seeds = torch.arange(rows, dtype=torch.int64, device=DEV) + 123
    ctr = torch.zeros(rows, dtype=torch.int64, device=DEV)
    a = torch.empty(rows, dtype=torch.int32, device=DEV)
    b = torch.empty_like(a)
    K.sample(lg, a, temperature=temp, top_p=top_p, top_k=top_k, seeds=seeds, counters=ctr)
    K.sample(lg, b, temperature=temp, top_p=top_p, top_k=top_k, seeds=seeds, counters=ctr)
    assert torch.equal(a, b)
    top3 = logits.float().topk(3, -1).indices
    assert all(int(a[r]) in top3[r].tolist() for r in range(rows))
    seen = set()
    for c in range(40):
        K.sample(lg[:1], a[:1], temperature=temp[:1], top_p=top_p[:1], top_k=top_k[:1], seeds=seeds[:1],
                 counters=ctr[:1] + c)
        seen.add(int(a[0]))
    assert len(seen) >= 2


def test_hadamard_rotation_kernel_and_rotated_cache():
    """Walsh-Hadamard rotation: the stand-alone kernel against the matrix, its own inverse, and the fused
    q / k / v rotation of the cache write: attention over a rotated INT4 cache, rotated back, matches attention over
    the plain cache within the quantization error, and is the better of the two on outlier channels."""
    K = _k()
    g = torch.Generator().manual_seed(0)
    H = torch.ones(1, 1)
    for _ in range(7):
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    H = H / 128 ** 0.5
    x = torch.randn(5, 3 * 128, generator=g).to(torch.bfloat16)
    y = K.hadamard(x.to(DEV).clone())
    want = (x.float().view(5, 3, 128) @ H).view(5, 384)
    assert _rel(y.cpu(), want) < 5e-3
    assert _rel(K.hadamard(y.clone()).cpu(), x) < 1e-2

    hq, hkv, d, T = 8, 2, 128, 40
    qkv = torch.randn(T, (hq + 2 * hkv) * d, generator=g)
    qkv[:, hq * d + 5] *= 30.0                          # an outlier channel in K head 0 ...
    qkv[:, (hq + hkv) * d + 77] *= 30.0                 # ... and one in V head 0
    qkv = qkv.to(torch.bfloat16).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = (torch.arange(T, dtype=torch.int32, device=DEV) + 16)          # pages 1..3
    inv_freq = eager.rope_inv_freq(d, 1e6, DEV)
    table = torch.tensor([[1, 2, 3]], dtype=torch.int32, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    outs = {}
    for bits in (8, 4):
        for rot in (False, True):
            cache = torch.zeros(8, hkv, K.kv_blob_bytes(d, bits, bits), dtype=torch.uint8, device=DEV)
            q = torch.empty(T, hq * d, dtype=torch.bfloat16, device=DEV)
            K.rope_kv_write(qkv, q, cache, pos, slots, inv_freq, hq, hkv, d, bits, bits, rotate=rot)
            out = torch.zeros(T, hq, d, dtype=torch.bfloat16, device=DEV)
            # one row block: the last 4 query rows of the request attend to the whole context
            K.paged_attention(q.view(T, hq, d), out, cache, table, torch.zeros(1, **i32), torch.tensor([T - 4], **i32),
                              torch.tensor([4], **i32), torch.tensor([T - 3], **i32), hq, hkv, d, bits, bits)
            o = out[T - 4:].reshape(4, hq * d).clone()
            outs[bits, rot] = K.hadamard(o) if rot else o
    torch.cuda.synchronize()
    K.workspace(torch.device(DEV)).check_status()
    ref = outs[8, False].float()
    assert _rel(outs[8, True], ref) < 3e-2
    err_plain, err_rot = _rel(outs[4, False], ref), _rel(outs[4, True], ref)
    assert err_rot < err_plain and err_rot < 0.2, (err_plain, err_rot)


@pytest.mark.parametrize("m,n,k,splits", [(256, 512, 4096, 4), (40, 384, 1024, 2), (300, 256, 2048, 8), (17, 200, 1024, 3)])
def test_wq_gemm_split_k_through_cluster_shared_memory(m, n, k, splits):
    """The K splits of a tile as one thread-block cluster (partials summed through distributed shared memory) give
    bit-identical results to the workspace path (same summation order), with residual and fused activation."""
    from cubic_serve_b200.ops import native
    K = _k()
    pw, dense = _cubic_weight(n, k, seed=m + n)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16).to(DEV)
    res = torch.randn(m, n, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    lib = native.lib()
    outs = {}
    try:
        for mode in (1, 0):
            lib.cb_wq_gemm_cluster_splitk(mode)
            y = K.wq_gemm(x, pw.to(DEV), splits=splits)
            yr = K.wq_gemm(x, pw.to(DEV), residual=res, splits=splits)
            act = K.wq_gemm_act(x, wq_pack.swiglu_interleave(pw).to(DEV), splits=splits) if n % 32 == 0 else y
            torch.cuda.synchronize()
            K.workspace(y.device).check_status()
            outs[mode] = (y.clone(), yr.clone(), act.clone())
    finally:
        lib.cb_wq_gemm_cluster_splitk(1)
    assert _rel(outs[1][0].cpu(), x.float().cpu() @ dense.t()) < 1e-2
    for a, b in zip(outs[1], outs[0]):
        assert torch.equal(a, b)


def test_autotune_measures_and_installed_plans_are_used():
    from cubic_serve_b200.ops import autotune, kernels as K, wq_pack
    plan = autotune.tune([(wq_pack.FMT_CUBIC4, 512, 1024, False), (wq_pack.FMT_CUBIC4, 512, 1024, True)], [16], "cuda:0")
    assert set(plan) == {"0:16:512:1024:0", "0:16:512:1024:1"}
    for e in plan.values():
        assert e["us"] > 0 and e["rule_us"] > 0 and {"tile1", "tile2", "tile4", "stream_k"} <= set(e["all_us"])
    w = autotune._random_weight(wq_pack.FMT_CUBIC4, 512, 1024, False, "cuda:0")
    x = (torch.randn(16, 1024, device="cuda:0") * 0.5).to(torch.bfloat16)
    want = x.float() @ wq_pack.unpack_to_dense(w)[:512].to("cuda:0").t()
    by_rule = K.wq_gemm(x, w)
    try:
        for forced in ({"use": True, "kernel": "tile", "splits": 4}, {"use": True, "kernel": "stream_k", "splits": 0}):
            assert autotune.install({"0:16:512:1024:0": forced}) == 1
            got = K.wq_gemm(x, w)
            assert ((got.float() - want).norm() / want.norm()).item() < 1e-2
            assert ((got.float() - by_rule.float()).norm() / want.norm()).item() < 1e-2
    finally:
        autotune.install(None)
    K.workspace(torch.device("cuda:0")).check_status()
