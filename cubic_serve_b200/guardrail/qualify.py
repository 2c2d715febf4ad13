"""Start-up / on-demand numerical qualification of the native kernels on the local GPU (``cubic qualify``).

A light version of the reference's start-up qualification (``runtime/quantized_qualification.py:75``,
``guardrail/harness.py:77`` there): each kernel runs a few small shapes against the independent eager oracle and
reports a verdict; the run also checks that padded graph rows cannot disturb live rows and that eager launches
and CUDA-graph replays produce identical tokens.  It takes seconds, not minutes.
"""
from __future__ import annotations

import time

import torch

from .compare import compare_tensors, reduction_bound


def _gemm_cases(quick: bool):
    return [(16, 256, 512), (48, 384, 1024)] if quick else [(1, 128, 256), (16, 256, 512), (48, 384, 1024), (256, 512, 4096)]


def run_qualification(device: int = 0, quick: bool = False) -> dict:
    from ..ops import eager, kernels as K, wq_pack
    from ..quantization import cubic
    dev = torch.device("cuda", device)
    torch.cuda.set_device(dev)
    results = []
    t0 = time.time()
    g = torch.Generator().manual_seed(0)
    for m, n, k in _gemm_cases(quick):
        w = torch.randn(n, k, generator=g) * 0.02
        scheme = cubic.CubicScheme(4, 128)
        p = cubic.quantize(w, scheme)
        pw = wq_pack.pack_cubic4(cubic.unpack_codes(p["weight_packed"], 4, k), p["weight_scale"], p["weight_a"],
                                 p["weight_b"], 128).to(dev)
        x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        y = K.wq_gemm(x, pw)
        ref = x.float() @ wq_pack.unpack_to_dense(pw).t()
        v = compare_tensors(y, ref, reduction_bound(ref, torch.bfloat16, k))
        results.append({"kernel": "wq_gemm[cubic4]", "shape": [m, n, k], "class": v.klass.value, "rel_l2": v.rel_l2})
    xs = torch.randn(33, 4096, generator=g).to(torch.bfloat16).to(dev)
    wn = torch.randn(4096, generator=g).to(torch.bfloat16).to(dev)
    v = compare_tensors(K.rmsnorm(xs, wn, 1e-6), eager.rmsnorm(xs, wn, 1e-6), 2.0 ** -6)
    results.append({"kernel": "rmsnorm", "shape": [33, 4096], "class": v.klass.value, "rel_l2": v.rel_l2})
    gu = torch.randn(17, 2048, generator=g).to(torch.bfloat16).to(dev)
    v = compare_tensors(K.swiglu(gu), eager.swiglu(gu), 2.0 ** -6)
    results.append({"kernel": "swiglu", "shape": [17, 1024], "class": v.klass.value, "rel_l2": v.rel_l2})
    # padding rows must not disturb live rows: same logical rows inside a larger, NaN-poisoned batch
    x_small = (torch.randn(16, 512, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    x_big = torch.full((64, 512), float("nan"), dtype=torch.bfloat16, device=dev)
    x_big[:16] = x_small
    w = torch.randn(256, 512, generator=g) * 0.02
    pw = wq_pack.pack_bf16(w).to(dev)
    same = torch.equal(K.wq_gemm(x_small, pw), K.wq_gemm(x_big, pw)[:16])
    results.append({"kernel": "wq_gemm padding isolation", "shape": [16, 64], "class": "exact" if same else "mismatch", "rel_l2": 0.0})
    results += _qualify_gemm_variants(dev, g, quick)
    results += _qualify_cross_m(dev, g, quick)
    results += _qualify_recurrent_and_rotation(dev, g)
    results.append(_qualify_graph_replay(dev))
    torch.cuda.synchronize(dev)
    K.workspace(dev).check_status()
    ok = all(r["class"] != "mismatch" for r in results)
    return {"ok": ok, "device": torch.cuda.get_device_name(dev), "seconds": round(time.time() - t0, 2), "results": results}


def tensor_digest(t: torch.Tensor) -> str:
    """Digest of a result's bits: two builds that print the same digest computed the same values."""
    import hashlib
    raw = t.detach().contiguous().cpu()
    return hashlib.sha256(raw.view(torch.uint8).numpy().tobytes()).hexdigest()[:16]


def _verdict(name: str, shape, got, ref, bound: float) -> dict:
    v = compare_tensors(got, ref, bound)
    return {"kernel": name, "shape": list(shape), "class": v.klass.value, "rel_l2": v.rel_l2, "digest": tensor_digest(got)}


def compare_reports(old: dict, new: dict) -> dict:
    """Operator artifacts of two qualification reports side by side: which checks kept their bits, which changed
    (and whether both sides still pass), which appeared or disappeared.  Reports come from ``run_qualification``
    (``cubic qualify --save``); only checks that carry a result digest can be called identical."""
    a = {r["kernel"] + " " + str(r["shape"]): r for r in old.get("results", [])}
    b = {r["kernel"] + " " + str(r["shape"]): r for r in new.get("results", [])}
    same, changed, regressed = [], [], []
    for key in sorted(set(a) & set(b)):
        ra, rb = a[key], b[key]
        if rb["class"] == "mismatch" and ra["class"] != "mismatch":
            regressed.append(key)
        elif ra.get("digest") and ra.get("digest") == rb.get("digest"):
            same.append(key)
        else:
            changed.append({"check": key, "old": {k: ra.get(k) for k in ("class", "rel_l2", "digest")},
                            "new": {k: rb.get(k) for k in ("class", "rel_l2", "digest")}})
    return {"identical": same, "changed": changed, "regressed": regressed, "added": sorted(set(b) - set(a)),
            "removed": sorted(set(a) - set(b)), "ok": not regressed and new.get("ok", False)}


def _qualify_gemm_variants(dev, g, quick: bool) -> list[dict]:
    """The persistent stream-K kernel (forced many-part tiles), its CTA-pair form (cta_group::2) and the fused
    SwiGLU epilogue against the fp32 oracle."""
    from ..ops import eager, kernels as K, native, wq_pack
    from ..quantization import cubic
    out = []
    m, n, k = (256, 512, 1024) if quick else (272, 1024, 2048)
    w = torch.randn(n, k, generator=g) * 0.02
    p = cubic.quantize(w, cubic.CubicScheme(4, 128))
    pw = wq_pack.pack_cubic4(cubic.unpack_codes(p["weight_packed"], 4, k), p["weight_scale"], p["weight_a"], p["weight_b"], 128)
    dense = wq_pack.unpack_to_dense(pw)[:n].to(dev)
    x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    ref = x.float() @ dense.t()
    bound = reduction_bound(ref, torch.bfloat16, k)
    lib = native.lib()
    try:
        for pairs, label in ((0, "stream-K"), (2, "stream-K, CTA pairs")):
            lib.cb_wq_gemm_pair_mode(pairs)
            out.append(_verdict(f"wq_gemm[cubic4] {label}", (m, n, k), K.wq_gemm(x, pw.to(dev), min_units=3), ref, bound))
        act = K.wq_gemm_act(x, wq_pack.swiglu_interleave(pw).to(dev), min_units=3)
        out.append(_verdict("wq_gemm[cubic4] + SwiGLU epilogue", (m, n // 2, k), act, eager.swiglu(ref.to(torch.bfloat16)),
                            2.0 ** -5))
    finally:
        lib.cb_wq_gemm_pair_mode(1)
    return out


def _qualify_cross_m(dev, g, quick: bool) -> list[dict]:
    """Cross-M audit: the result of a row must not depend on how many other rows share its batch beyond the order of
    fp32 partial sums (another launch form may split K elsewhere).  The first rows of a large batch are compared with
    the same rows run alone, for the kernels whose launch form changes with the row count: the weight GEMM (per-tile
    splits vs persistent kernel), the fused SwiGLU GEMM and row-wise RMSNorm.  ``exact`` = batch invariant bit for bit,
    ``rounding`` = equal to within the bf16 output rounding.  (Reference: ``guardrail/quantized_graph/cross_m.py``.)"""
    from ..ops import kernels as K, wq_pack
    from ..quantization import cubic
    out = []
    shapes = [(1024, 1024)] if quick else [(1024, 1024), (6144, 4096)]
    for n, k in shapes:
        w = torch.randn(n, k, generator=g) * 0.02
        p = cubic.quantize(w, cubic.CubicScheme(4, 128))
        pw = wq_pack.pack_cubic4(cubic.unpack_codes(p["weight_packed"], 4, k), p["weight_scale"], p["weight_a"], p["weight_b"],
                                 128)
        x = (torch.randn(256, k, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        big = K.wq_gemm(x, pw.to(dev))
        bound = 4 * 2.0 ** -8                       # a few bf16 output roundings of differently ordered fp32 sums
        for m in (1, 16, 64):
            out.append(_verdict(f"cross-M wq_gemm[cubic4] rows {m} of 256", (m, n, k), K.wq_gemm(x[:m].contiguous(), pw.to(dev)),
                                big[:m], bound))
        pa = wq_pack.swiglu_interleave(pw).to(dev)
        big_a = K.wq_gemm_act(x, pa)
        out.append(_verdict("cross-M wq_gemm + SwiGLU rows 16 of 256", (16, n // 2, k), K.wq_gemm_act(x[:16].contiguous(), pa),
                            big_a[:16], 8 * 2.0 ** -8))
    xs = torch.randn(256, 4096, generator=g).to(torch.bfloat16).to(dev)
    wn = torch.randn(4096, generator=g).to(torch.bfloat16).to(dev)
    out.append(_verdict("cross-M rmsnorm rows 3 of 256", (3, 4096), K.rmsnorm(xs[:3].contiguous(), wn, 1e-6),
                        K.rmsnorm(xs, wn, 1e-6)[:3], 2.0 ** -8))
    return out


def _qualify_recurrent_and_rotation(dev, g) -> list[dict]:
    """Gated DeltaNet kernels against their oracles (a fresh request and one that continues from stored state) and
    the Walsh-Hadamard rotation against the matrix."""
    from ..ops import eager, kernels as K
    out = []
    hk, hv, d = 2, 4, 128
    counts, slots, pos0 = [7, 1], [1, 0], [0, 4]
    T, C = sum(counts), (2 * hk + hv) * d
    i32 = dict(dtype=torch.int32, device=dev)
    seg = K.GdnSegments(torch.tensor([0, 7], **i32), torch.tensor(counts, **i32), torch.tensor(slots, **i32),
                        torch.tensor(pos0, **i32), 2)
    x = torch.randn(T, C, generator=g).to(torch.bfloat16)
    w = torch.randn(C, 4, generator=g) * 0.4
    cstate = torch.randn(2, 3, C, generator=g).to(torch.bfloat16)
    mix = torch.empty(T, C, dtype=torch.bfloat16, device=dev)
    K.gdn_conv(x.to(dev), w.to(dev), cstate.clone().to(dev), seg, mix)
    want = torch.cat([eager.gdn_conv(x[:7], w, None)[0], eager.gdn_conv(x[7:], w, cstate[0])[0]])
    out.append(_verdict("gdn_conv", (T, C), mix, want.to(dev), 2.0 ** -6))
    z = torch.randn(T, hv * d, generator=g).to(torch.bfloat16)
    ba = torch.randn(T, 2 * hv, generator=g).to(torch.bfloat16)
    a_log, dt_bias, nw = torch.randn(hv, generator=g) * 0.5, torch.randn(hv, generator=g) * 0.5, torch.ones(d)
    state = torch.randn(2, hv, d, d, generator=g) * 0.05
    got = torch.empty(T, hv * d, dtype=torch.bfloat16, device=dev)
    K.gdn_delta(mix, z.to(dev), ba.to(dev), a_log.to(dev), dt_bias.to(dev), nw.to(dev), state.clone().to(dev), seg, got, hk, hv)
    mc = mix.cpu()
    want = torch.cat([eager.gdn_delta(mc[:7], z[:7], ba[:7], a_log, dt_bias, nw, None, hk, hv)[0],
                      eager.gdn_delta(mc[7:], z[7:], ba[7:], a_log, dt_bias, nw, state[0], hk, hv)[0]])
    out.append(_verdict("gdn_delta", (T, hv * d), got, want.to(dev), 2.0 ** -5))
    h = torch.ones(1, 1)
    for _ in range(7):
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    v = torch.randn(9, 256, generator=g).to(torch.bfloat16)
    want = (v.float().view(9, 2, 128) @ (h / 128 ** 0.5)).view(9, 256)
    out.append(_verdict("hadamard", (9, 256), K.hadamard(v.to(dev).clone()), want.to(dev), 2.0 ** -6))
    return out


def _qualify_graph_replay(dev) -> dict:
    """A toy decoder generates the same tokens with eager launches and with captured decode graphs (padded rows)."""
    from ..executor.gpu_executor import GpuExecutor
    from ..models.config import ModelConfig, QuantSpec
    from ..models.decoder import DecoderRunner, random_decoder_weights
    from ..runtime.engine import LLMEngine
    from ..runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = ModelConfig(name="qualify", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    weights = random_decoder_weights(cfg, dev, seed=0, std=0.05)
    outs = []
    for graphs in (False, True):
        runner = DecoderRunner(cfg, weights, num_pages=64, max_tokens=256, max_requests=8)
        ex = GpuExecutor(runner, max_rows=8, max_prefill_tokens=256, max_model_len=128, use_graphs=graphs)
        if graphs:
            ex.capture_decode_graphs()
        eng = LLMEngine(ex, 64, SchedulerConfig(max_running_requests=8, max_model_len=128, max_batched_tokens=256,
                                                enable_prefix_cache=False))
        prompts = [[(7 * i + 3 * j) % 2000 for j in range(9 + 4 * i)] for i in range(3)]      # 3 rows in a 4-row graph
        outs.append(eng.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True)))
    same = outs[0] == outs[1]
    return {"kernel": "decode graph replay == eager launches", "shape": [3, 10], "class": "exact" if same else "mismatch",
            "rel_l2": 0.0}


def qualify_with_receipt(device: int = 0, quick: bool = False, evidence_dir=None, force: bool = False, run=None):
    """``run_qualification`` behind a start-up receipt: a passing report made by the same implementation (source
    closure + native sources + build flags) on the same GPU model is returned without running anything.  Returns
    ``(report, reused)``."""
    from ..contracts.implementation import PACKAGE_NAME, identity
    from ..runtime.preparation import EvidenceStore, StartupQualification, device_description
    ident = identity("qualification", (f"{PACKAGE_NAME}.guardrail.qualify",))
    sq = StartupQualification(EvidenceStore(evidence_dir), ident, device_description(device))
    return sq.ensure(run or (lambda: run_qualification(device, quick=quick)), operands={"quick": bool(quick)}, force=force)
