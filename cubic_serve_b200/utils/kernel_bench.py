"""Micro-benchmarks of single native kernels (CUDA-event timed) -- also the small cases used for ncu captures.

Examples::

    python -m cubic_serve_b200.utils.kernel_bench gemm --m 256 --n 24576 --k 4096
    python -m cubic_serve_b200.utils.kernel_bench attn --rows 256 --ctx 1280
    python -m cubic_serve_b200.utils.kernel_bench sweep
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import eager, kernels as K, wq_pack

DEV = "cuda"


def timeit(fn, iters: int = 20, warmup: int = 5, flush: torch.Tensor | None = None) -> float:
    """Median milliseconds per call, CUDA events on the launching stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def timeit_graph(fn, flush: torch.Tensor, launches: int = 10, repeats: int = 3) -> float:
    """Device milliseconds per call measured INSIDE a CUDA graph, cold L2.

    An eager launch of a 15 us kernel is dominated by the host (tensor-map encoding, ctypes, the launch
    itself), which a serving step never pays because it replays a graph.  The graph holds ``launches`` times
    {write a buffer larger than L2, call}; the same graph without the calls is timed too and subtracted.
    """
    stream = torch.cuda.Stream()
    graphs = []
    with torch.cuda.stream(stream):
        fn()
        fn()
        stream.synchronize()
        for with_call in (True, False):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(launches):
                    flush.zero_()
                    if with_call:
                        fn()
            graphs.append(g)
        best = []
        for g in graphs:
            g.replay()
            stream.synchronize()
            t = []
            for _ in range(repeats):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                stream.synchronize()
                t.append(a.elapsed_time(b))
            best.append(min(t))
    return max(0.0, best[0] - best[1]) / launches


def random_cubic_weight(n: int, k: int, group: int = 128) -> wq_pack.PackedWeight:
    """Random codes with unit-ish curve metadata, packed without a quantizer pass."""
    codes = torch.randint(-7, 8, (n, k), dtype=torch.int8, device=DEV)
    g = k // group
    full = lambda v: torch.full((n, g), v, device=DEV)
    return wq_pack.pack_cubic4(codes, full(0.02), full(0.75), full(0.25), group)


def bench_gemm(m: int, n: int, k: int, splits: int | None, iters: int, fmt: str = "cubic4",
               kernel: str = "auto", act: bool = False) -> dict:
    """``kernel``: auto (the dispatcher's choice), tile (one CTA per tile and K split), streamk (persistent).
    ``act``: the weight is a [gate; up] projection and SwiGLU runs in the epilogue (output ``[m, n / 2]``)."""
    if fmt == "bf16":
        w = wq_pack.pack_bf16(torch.randn(n, k, device=DEV) * 0.02)
        wbytes = n * k * 2
    elif fmt in ("fp8", "fp8_block"):
        # e4m3 weights with row (or 128 x 128 block) scales; the timed call is the GEMM on activations quantized
        # beforehand (the fused norm / activation kernels produce them in a model step)
        from ..quantization import formats
        p = formats.fp8_quantize(torch.randn(n, k, device=DEV) * 0.02, block=fmt == "fp8_block")
        w = (wq_pack.pack_fp8_block(p["weight"], p["weight_scale_inv"]) if fmt == "fp8_block"
             else wq_pack.pack_fp8(p["weight"], p["weight_scale"]))
        wbytes = n * k + n * 4
    else:
        w = random_cubic_weight(n, k)
        wbytes = n * k // 2 + n * (k // 128) * 8
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    y = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    stream_k = fmt != "fp8_block" and (kernel == "streamk" or (kernel == "auto" and splits is None and K.use_stream_k(
        m, n, wq_pack.FMT_CUBIC4 if fmt == "fp8" else w.fmt, k=k // 2 if fmt == "fp8" else k)))
    sp = None if stream_k else (splits or K.choose_splits(m, n, k, fmt=w.fmt))
    if fmt.startswith("fp8"):
        x = K.fp8_quantize(x, out=K.Fp8Act(torch.empty(m, k, dtype=torch.uint8, device=DEV),
                                           torch.empty(m, dtype=torch.float32, device=DEV)))
    if act:
        w = wq_pack.swiglu_interleave(w)
        y = torch.empty(m, n // 2, device=DEV, dtype=torch.bfloat16)
        call = lambda: K.wq_gemm_act(x, w, out=y, splits=sp, min_units=0 if stream_k else None)   # noqa: E731
    elif stream_k:
        call = lambda: K.wq_gemm(x, w, out=y, min_units=0)                                   # noqa: E731
    else:
        call = lambda: K.wq_gemm(x, w, out=y, splits=sp)                                     # noqa: E731
    ms = timeit_graph(call, flush, launches=max(3, min(10, iters)))
    K.workspace(torch.device(DEV)).check_status()
    from ..ops import native
    return {"op": f"wq_gemm[{fmt}]" + ("+swiglu" if act else ""), "resident_pairs": native.lib().cb_wq_gemm_resident_pairs(w.fmt), "m": m, "n": n, "k": k, "kernel": "streamk" if stream_k else "tile",
            "splits": None if stream_k else sp, "us": round(ms * 1e3, 1), "timing": "in-graph, L2 flushed",
            "tflops": round(2 * m * n * k / ms / 1e9, 1), "weight_gbs": round(wbytes / ms / 1e6, 1)}


def bench_attn(rows: int, ctx: int, hq: int, hkv: int, kb: int, vb: int, splits: int, iters: int) -> dict:
    d = 128
    pages_per = -(-ctx // 16)
    blob = K.kv_blob_bytes(d, kb, vb)
    cache = torch.randint(0, 255, (rows * pages_per + 1, hkv, blob), dtype=torch.uint8, device=DEV)
    lay = eager.blob_layout(d, kb, vb)
    one = torch.full((64,), 0.01, device=DEV).view(torch.uint8)
    cache[:, :, lay["k_scale"]:lay["v_code"]] = one
    cache[:, :, lay["v_scale"]:] = one
    table = (torch.randperm(rows * pages_per, device=DEV).to(torch.int32) + 1).view(rows, pages_per)
    q = torch.randn(rows, hq, d, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    ar = torch.arange(rows, dtype=torch.int32, device=DEV)
    ones, ctxs = torch.ones_like(ar), torch.full_like(ar, ctx)
    ms = timeit(lambda: K.paged_attention(q, out, cache, table, ar, ar, ones, ctxs, hq, hkv, d, kb, vb, splits=splits),
                iters=iters, warmup=min(5, iters))
    K.workspace(torch.device(DEV)).check_status()
    kv_bytes = rows * pages_per * hkv * blob
    return {"op": f"paged_attn[k{kb}v{vb}]", "rows": rows, "ctx": ctx, "hq": hq, "hkv": hkv, "splits": splits,
            "us": round(ms * 1e3, 1), "kv_gbs": round(kv_bytes / ms / 1e6, 1)}


def bench_gdn(requests: int, tokens: int, hk: int, hv: int) -> dict:
    """Gated DeltaNet kernels of one layer: ``requests`` segments of ``tokens`` rows each (1 = a decode step)."""
    d, T = 128, requests * tokens
    C = (2 * hk + hv) * d
    i32 = dict(dtype=torch.int32, device=DEV)
    seg = K.GdnSegments(torch.arange(requests, **i32) * tokens, torch.full((requests,), tokens, **i32),
                        torch.arange(requests, **i32), torch.full((requests,), 5, **i32), requests)
    proj = torch.randn(T, C + hv * d + 2 * hv, device=DEV).to(torch.bfloat16)
    w = torch.randn(C, 4, device=DEV) * 0.3
    conv_state = torch.zeros(requests, 3, C, dtype=torch.bfloat16, device=DEV)
    state = torch.randn(requests, hv, d, d, device=DEV) * 0.01
    mix = torch.empty(T, C, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(T, hv * d, dtype=torch.bfloat16, device=DEV)
    a_log, dt_bias, norm_w = torch.zeros(hv, device=DEV), torch.zeros(hv, device=DEV), torch.ones(d, device=DEV)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    conv_ms = timeit_graph(lambda: K.gdn_conv(proj, w, conv_state, seg, mix), flush, launches=5)
    delta_ms = timeit_graph(lambda: K.gdn_delta(mix, proj[:, C:C + hv * d], proj[:, C + hv * d:], a_log, dt_bias, norm_w,
                                                state, seg, out, hk, hv), flush, launches=5)
    state_bytes = 2 * state.numel() * 4                       # read + written once per step
    return {"op": "gdn", "requests": requests, "tokens_per_request": tokens, "hk": hk, "hv": hv,
            "conv_us": round(conv_ms * 1e3, 1), "delta_us": round(delta_ms * 1e3, 1),
            "delta_state_gbs": round(state_bytes / delta_ms / 1e6, 1), "timing": "in-graph, L2 flushed"}


def bench_fused_tp(ranks: int, m: int, hidden: int, inter: int, iters: int) -> dict:
    """One o_proj -> norm -> gate/up boundary of the fused tensor-parallel path with all ranks on THIS device.

    The ranks' kernels run stage by stage (every producer of a stage is in the stream before any consumer), so
    the waits inside the kernels find their counters raised; "peer" buffers are other tensors of this process.
    It times the three kernels per rank (scatter-push GEMM, rank-ordered reduce + norm + gather push,
    gather-wait GEMM) without any NVLink hop, and gives ncu a one-GPU program that launches them.
    """
    from ..parallel.tp import FusedTp, local_fabric
    dev = torch.device(DEV)
    fab = [FusedTp(b, dev) for b in local_fabric(ranks, hidden, max(m, 64), 64, DEV)]
    o_w = [random_cubic_weight(hidden, hidden // ranks) for _ in range(ranks)]          # row-parallel shard
    gu_w = [random_cubic_weight(2 * inter // ranks, hidden) for _ in range(ranks)]       # column-parallel shard
    norm = torch.ones(hidden, dtype=torch.bfloat16, device=DEV)
    attn = [torch.randn(m, hidden // ranks, device=DEV, dtype=torch.bfloat16) for _ in range(ranks)]
    gu = [torch.empty(m, 2 * inter // ranks, device=DEV, dtype=torch.bfloat16) for _ in range(ranks)]
    for f in fab:
        f.begin_step(m)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    t = [[], [], []]
    for it in range(iters + 2):
        s = it & 1
        ev[0].record()
        for f in fab:
            f.gemm_scatter(attn[f.rank], o_w[f.rank], s)
        ev[1].record()
        for f in fab:
            f.reduce_norm(norm, s, hidden, 1e-6)
        ev[2].record()
        for f in fab:
            f.gemm_gather(gu_w[f.rank], gu[f.rank], s)
        ev[3].record()
        torch.cuda.synchronize()
        fab[0].ws.check_status()
        if it >= 2:
            for j in range(3):
                t[j].append(ev[j].elapsed_time(ev[j + 1]) / ranks)
    med = [sorted(x)[len(x) // 2] * 1e3 for x in t]
    return {"op": "fused_tp_site[emulated ranks on one device]", "ranks": ranks, "m": m, "hidden": hidden, "inter": inter,
            "gemm_scatter_us": round(med[0], 1), "reduce_norm_us": round(med[1], 1), "gemm_gather_us": round(med[2], 1),
            "timing": "eager launches, per rank (sum over ranks / ranks)"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "attn", "sweep", "fused-tp", "gdn"],
                    help="gdn: --rows requests x --ctx tokens per request (1 = decode) through one Gated DeltaNet layer")
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--n", type=int, default=24576)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--fmt", default="cubic4")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1280)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--kbits", type=int, default=8)
    ap.add_argument("--vbits", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--kernel", default="auto", choices=["auto", "tile", "streamk"])
    ap.add_argument("--pairs", type=int, default=1, choices=[0, 1, 2],
                    help="persistent kernel on CTA pairs (cta_group::2): never (0), above 256 rows (1), wherever eligible (2)")
    ap.add_argument("--act", action="store_true", help="gemm: [gate; up] projection with SwiGLU in the epilogue")
    a = ap.parse_args()
    from ..ops import native
    native.lib().cb_wq_gemm_pair_mode(a.pairs)
    if a.op == "gdn":
        print(json.dumps(bench_gdn(a.rows, a.ctx, 16, 32)))
    elif a.op == "gemm":
        print(json.dumps(bench_gemm(a.m, a.n, a.k, a.splits or None, a.iters, a.fmt, a.kernel, a.act)))
    elif a.op == "fused-tp":
        print(json.dumps(bench_fused_tp(a.ranks, a.m, a.hidden, a.inter, a.iters)))
    elif a.op == "attn":
        print(json.dumps(bench_attn(a.rows, a.ctx, a.hq, a.hkv, a.kbits, a.vbits, max(1, a.splits), a.iters)))
    else:
        for m in (16, 64, 256, 512):
            for n, k in ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)):
                print(json.dumps(bench_gemm(m, n, k, None, a.iters)), flush=True)
        print(json.dumps(bench_gemm(256, 151936, 4096, None, a.iters, "bf16")), flush=True)
        for m in (16, 256, 4096):
            for n, k in ((6144, 4096), (24576, 4096), (4096, 12288)):
                print(json.dumps(bench_gemm(m, n, k, None, a.iters, "fp8")), flush=True)
        for kb, vb in ((8, 8), (4, 8), (4, 4)):
            print(json.dumps(bench_attn(256, 1280, 32, 8, kb, vb, 1, a.iters)), flush=True)
        print(json.dumps(bench_attn(8, 4096, 32, 8, 8, 8, 8, a.iters)), flush=True)


if __name__ == "__main__":
    main()
