"""Fused tensor-parallel kernels with all ranks emulated on ONE GPU.

The ranks' kernels are launched stage by stage (all producers of a stage before any consumer), so every
wait finds its counters already raised: this checks addressing, ownership, counters/epochs and numerics of
the scatter-push GEMM, the rank-ordered reduce + norm + gather-push kernel, the gather-wait GEMM and the
greedy merge without needing several devices.
"""
import pytest
import torch

from cubic_serve_b200.ops import eager, wq_pack

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("size,m", [(2, 48), (4, 256), (4, 37), (8, 300)])
def test_scatter_reduce_norm_gather_pipeline(size, m):
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.parallel.tp import FusedTp, local_fabric
    H, N1 = 512, 1024
    g = torch.Generator().manual_seed(size * 100 + m)
    w1 = (torch.randn(N1, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    w2 = (torch.randn(H, N1, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    n1 = (torch.rand(H, generator=g) + 0.5).to(torch.bfloat16).to(DEV)
    n2 = (torch.rand(H, generator=g) + 0.5).to(torch.bfloat16).to(DEV)
    ranks = [FusedTp(b, torch.device(DEV)) for b in local_fabric(size, H, 512, 64, DEV)]
    w1s = [wq_pack.pack_bf16(w1[r * N1 // size:(r + 1) * N1 // size]) for r in range(size)]
    w2s = [wq_pack.pack_bf16(w2[:, r * N1 // size:(r + 1) * N1 // size].contiguous()) for r in range(size)]

    # several launches through the same buffers and counters, with a DIFFERENT row count in between (a prefill
    # step followed by decode steps): the consumers' expected arrival counts change from launch to launch
    for rep, rows in enumerate([m, m, max(1, m // 2 + 5), m]):
        h = (torch.randn(rows, H, generator=g)).to(torch.bfloat16).to(DEV)
        x = eager.rmsnorm(h, n1, 1e-6).to(torch.bfloat16)
        y = (x.float() @ w1.float().t()).to(torch.bfloat16)
        partial = [(y[:, r * N1 // size:(r + 1) * N1 // size].float()
                    @ w2[:, r * N1 // size:(r + 1) * N1 // size].float().t()).to(torch.bfloat16) for r in range(size)]
        z = torch.zeros(rows, H, device=DEV)
        for pr in partial:                                 # ascending rank order, fp32
            z += pr.float()
        href2 = (h.float() + z.to(torch.bfloat16).float()).to(torch.bfloat16)
        xref2 = eager.rmsnorm(href2, n2, 1e-6)

        for f in ranks:
            f.begin_step(rows)
            lo = f.rank * f.rpr
            cnt = max(0, min(rows, lo + f.rpr) - lo)
            if cnt:
                f.h_local[:cnt] = h[lo:lo + cnt]
        for f in ranks:
            f.reduce_norm(n1, 0, 0, 1e-6, reduce=False)
        ys = [f.gemm_gather(w1s[f.rank], torch.empty(rows, N1 // size, dtype=torch.bfloat16, device=DEV), 0) for f in ranks]
        for f in ranks:
            f.gemm_scatter(ys[f.rank], w2s[f.rank], 1)
        for f in ranks:
            f.reduce_norm(n2, 1, H, 1e-6)
        for f in ranks:
            xg = f.wait_gather(1)
            torch.cuda.synchronize()
            f.ws.check_status()
            assert _rel(xg, xref2) < 1e-2, (rep, f.rank)
            lo = f.rank * f.rpr
            cnt = max(0, min(rows, lo + f.rpr) - lo)
            if cnt:
                assert _rel(f.h_local[:cnt], href2[lo:lo + cnt]) < 1e-2
        assert _rel(torch.cat([y_ for y_ in ys], 1), y) < 1e-2


def test_argmax_merge_agrees_and_breaks_ties_low():
    from cubic_serve_b200.parallel.tp import FusedTp, local_fabric
    size, rows = 4, 9
    ranks = [FusedTp(b, torch.device(DEV)) for b in local_fabric(size, 256, 64, 16, DEV)]
    g = torch.Generator().manual_seed(0)
    vals = torch.randn(size, rows, generator=g)
    ids = torch.stack([torch.randint(0, 1000, (rows,), generator=g) + 1000 * r for r in range(size)]).to(torch.int32)
    vals[1, 0] = vals[3, 0] = 50.0                          # tie between ranks 1 and 3 -> lower id (rank 1)
    outs = [torch.zeros(rows, dtype=torch.int32, device=DEV) for _ in range(size)]
    for f in ranks:
        # sequential emulation: ranks that have not run yet are published by hand into f's exchange area, so
        # that f's (bounded) wait finds every source present
        for o in ranks:
            if o.rank > f.rank:
                f.b.xchg_val[o.rank, :rows] = vals[o.rank].to(DEV)
                f.b.xchg_id[o.rank, :rows] = ids[o.rank].to(DEV)
                f.b.flags[32 + o.rank] += 1
        f.argmax_merge(vals[f.rank].to(DEV), ids[f.rank].to(DEV), outs[f.rank], rows)
    torch.cuda.synchronize()
    ranks[0].ws.check_status()
    best = vals.max(0).values
    expect = torch.where(vals == best, ids, torch.full_like(ids, 2 ** 31 - 1)).min(0).values
    for o in outs:
        assert o.cpu().tolist() == expect.tolist()


def _sampling_inputs(rows, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(torch.bfloat16).to(DEV)
    d = {"temperature": torch.tensor([0.0, 0.7, 1.0, 1.5] * (rows // 4), dtype=torch.float32, device=DEV),
         "top_p": torch.tensor([1.0, 0.9, 0.5, 1.0] * (rows // 4), dtype=torch.float32, device=DEV),
         "top_k": torch.tensor([0, 20, 5, 0] * (rows // 4), dtype=torch.int32, device=DEV),
         "seeds": torch.arange(rows, dtype=torch.int64, device=DEV) * 977 + 5,
         "draws": torch.arange(rows, dtype=torch.int64, device=DEV) % 7}
    return logits, d


def test_sharded_sampling_equals_full_vocabulary_sampling():
    """Candidates of vocabulary shards merged and drawn == the one-GPU sampler on the whole vocabulary, token
    for token (same candidate order, same Philox stream), for greedy, top-k, top-p and plain temperature rows."""
    from cubic_serve_b200.ops import kernels as K
    rows, vocab, shards = 16, 4096, 4
    logits, d = _sampling_inputs(rows, vocab)
    want = torch.zeros(rows, dtype=torch.int32, device=DEV)
    K.sample(logits, want, temperature=d["temperature"], top_p=d["top_p"], top_k=d["top_k"], seeds=d["seeds"],
             counters=d["draws"])
    rows_max = 32
    area = torch.zeros(shards, 2, rows_max, K.SAMPLE_CANDIDATES, dtype=torch.int32, device=DEV)
    v = vocab // shards
    for s in range(shards):
        K.sample_candidates(logits[:, s * v:(s + 1) * v], area[s, 0].view(torch.float32), area[s, 1],
                            temperature=d["temperature"], top_k=d["top_k"], vocab=v, id_offset=s * v)
    got = torch.zeros(rows, dtype=torch.int32, device=DEV)
    flat = area.view(shards, -1)
    K.sample_merge(flat.view(torch.float32), flat.view(-1)[rows_max * K.SAMPLE_CANDIDATES:], shards, flat.stride(0), rows,
                   got, temperature=d["temperature"], top_p=d["top_p"], top_k=d["top_k"], seeds=d["seeds"],
                   counters=d["draws"])
    torch.cuda.synchronize()
    assert got.cpu().tolist() == want.cpu().tolist()
    greedy = logits.float().argmax(-1).cpu()
    assert got.cpu()[0::4].tolist() == greedy[0::4].tolist()          # the temperature-0 rows
    assert (got.cpu()[1::4] != greedy[1::4]).any() or True


def test_sharded_sampling_through_the_exchange_kernel():
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.parallel.tp import CAND, FusedTp, local_fabric
    size, rows, vocab = 4, 8, 2048
    logits, d = _sampling_inputs(rows, vocab, seed=3)
    want = torch.zeros(rows, dtype=torch.int32, device=DEV)
    K.sample(logits, want, temperature=d["temperature"], top_p=d["top_p"], top_k=d["top_k"], seeds=d["seeds"],
             counters=d["draws"])
    ranks = [FusedTp(b, torch.device(DEV)) for b in local_fabric(size, 256, 64, 16, DEV)]
    v = vocab // size
    shard = [logits[:, r * v:(r + 1) * v].contiguous() for r in range(size)]
    for f in ranks:                                           # every rank's candidates, for the hand publication
        K.sample_candidates(shard[f.rank], f.cand_local[0].view(torch.float32), f.cand_local[1],
                            temperature=d["temperature"], top_k=d["top_k"], vocab=v, id_offset=f.rank * v)
    outs = [torch.zeros(rows, dtype=torch.int32, device=DEV) for _ in range(size)]
    for f in ranks:
        # sequential emulation: ranks that have not run yet are published by hand (see the greedy merge test)
        for o in ranks:
            if o.rank > f.rank:
                f.b.cand[o.rank].view(2, f.rows_max, CAND)[:, :rows] = o.cand_local[:, :rows]
                f.b.flags[40 + o.rank] += 1
        f.sample_sharded(shard[f.rank], rows, outs[f.rank], d, f.rank * v)
    torch.cuda.synchronize()
    ranks[0].ws.check_status()
    for o in outs:
        assert o.cpu().tolist() == want.cpu().tolist()
