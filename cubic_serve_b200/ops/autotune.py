"""Measured launch plans for the weight GEMMs of a model.

``kernels.wq_gemm`` picks between its two kernels and a split-K factor by rules fitted to a handful of shapes
(``use_stream_k`` / ``choose_splits``).  This module replaces the rules by measurement for the shapes a model actually
has: every projection of the model, at every decode capacity the executor captures, is timed inside a CUDA graph with
a cold L2 under each candidate launch form, and the fastest is recorded.  The result is a JSON plan
(``"fmt:m:n:k:act" -> {"kernel": "tile" | "stream_k", "splits": s}``); ``install`` makes ``kernels`` consult it before
its rules.  Plans are start-up evidence: ``runtime.preparation.StartupPreparation`` keeps them keyed by the
implementation digest, the GPU model and the shape list, so a deployment measures once.

Reference counterpart: ``ops/cuda/launch_cost.py`` (start-up cost models and calibration cache) and the per-geometry
route choice of ``quantization/common/small_rows_cost.py``; here the choice is measured rather than modelled.

Run as a module on a GPU to print the table for a named configuration:
``python -m cubic_serve_b200.ops.autotune --model dense-8b --rows 16 64 256``.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import kernels as K
from . import wq_pack

SPLIT_CANDIDATES = (1, 2, 3, 4, 6, 8)


def plan_key(fmt: int, m: int, n: int, k: int, act: bool) -> str:
    return f"{fmt}:{m}:{n}:{k}:{int(act)}"


def model_shapes(cfg, tp: int = 1) -> list[tuple[int, int, int, bool]]:
    """``(fmt, n, k, act)`` of every distinct dense projection of ``cfg`` on one of ``tp`` ranks."""
    fmt = wq_pack.FMT_CUBIC4 if cfg.quant.method == "cubic" else (wq_pack.FMT_BF16 if cfg.quant.method == "none"
                                                                 else wq_pack.FMT_AFFINE4)
    if cfg.quant.method == "nvfp4":
        fmt = wq_pack.FMT_NVFP4
    h, d = cfg.hidden_size, cfg.head_dim
    shapes = [(fmt, (cfg.num_q_heads + 2 * cfg.num_kv_heads) * d // tp, h, False),
              (fmt, h, cfg.num_q_heads * d // tp, False)]
    if not getattr(cfg, "num_experts", 0):
        shapes += [(fmt, 2 * cfg.intermediate_size // tp, h, True), (fmt, h, cfg.intermediate_size // tp, False)]
    shapes.append((wq_pack.FMT_BF16, -(-cfg.vocab_size // tp), h, False))
    return sorted(set(shapes))


def _random_weight(fmt: int, n: int, k: int, act: bool, device) -> wq_pack.PackedWeight:
    """A weight of the right format and shape; its values do not matter for timing."""
    g = torch.Generator().manual_seed(n * 31 + k)
    if fmt == wq_pack.FMT_BF16:
        pw = wq_pack.pack_bf16(torch.randn(n, k, generator=g) * 0.02)
    elif fmt == wq_pack.FMT_CUBIC4:
        codes = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
        groups = k // 128
        pw = wq_pack.pack_cubic4(codes, torch.rand(n, groups, generator=g) * 0.02 + 0.01, torch.full((n, groups), 0.8),
                                 torch.full((n, groups), 0.1), 128)
    elif fmt == wq_pack.FMT_AFFINE4:
        codes = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
        groups = k // 128
        pw = wq_pack.pack_affine4(codes, torch.rand(n, groups, generator=g) * 0.01 + 0.005, torch.full((n, groups), -0.04), 128)
    elif fmt == wq_pack.FMT_NVFP4:
        packed = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
        pw = wq_pack.pack_nvfp4(packed, torch.rand(n, k // 16, generator=g) * 0.5 + 0.25, 0.02)
    else:
        raise NotImplementedError(f"no synthetic weight for format {fmt}")
    if act:
        pw = wq_pack.swiglu_interleave(pw)
    return pw.to(device)


def _time_graph(fn, flush: torch.Tensor, launches: int = 6, repeats: int = 3) -> float:
    """Device microseconds per call inside a CUDA graph, L2 flushed before every call (flush time subtracted)."""
    stream = torch.cuda.Stream()
    times = []
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        for with_call in (True, False):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(launches):
                    flush.zero_()
                    if with_call:
                        fn()
            g.replay()
            stream.synchronize()
            best = float("inf")
            for _ in range(repeats):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                g.replay()
                b.record(stream)
                stream.synchronize()
                best = min(best, a.elapsed_time(b))
            times.append(best)
    return max(times[0] - times[1], 0.0) * 1e3 / launches


def candidates(m: int, n: int, k: int) -> list[tuple[str, int]]:
    """Launch forms worth timing: the per-tile kernel with each split factor that leaves >= 4 k-blocks per CTA and does
    not exceed ~4 CTAs per SM, and the persistent kernel."""
    tiles = -(-n // 128) * -(-m // 256)
    out = [("tile", s) for s in SPLIT_CANDIDATES if (k // 64) // s >= 4 and (s == 1 or tiles * s <= 4 * 148)]
    out.append(("stream_k", 0))
    return out


def tune(shapes, rows, device, verbose: bool = False) -> dict:
    """Time every candidate for every (shape, row count); returns the plan with the measurements."""
    dev = torch.device(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ws = K.workspace(dev)
    plan: dict[str, dict] = {}
    for fmt, n, k, act in shapes:
        w = _random_weight(fmt, n, k, act, dev)
        for m in rows:
            x = (torch.randn(m, k, device=dev) * 0.5).to(torch.bfloat16)
            out = torch.empty(m, n // 2 if act else n, dtype=torch.bfloat16, device=dev)
            call = K.wq_gemm_act if act else K.wq_gemm
            timed: dict[str, float] = {}
            timed["rule"] = _time_graph(lambda: call(x, w, out=out, ws=ws), flush)
            for kernel, s in candidates(m, n, k):
                kw = {"splits": s} if kernel == "tile" else {"min_units": 0}
                timed[f"{kernel}{s or ''}"] = _time_graph(lambda: call(x, w, out=out, ws=ws, **kw), flush)
            best = min((v, name) for name, v in timed.items() if name != "rule")
            name = best[1]
            entry = {"kernel": "stream_k" if name.startswith("stream_k") else "tile",
                     "splits": int(name[4:] or 1) if name.startswith("tile") else 0,
                     "us": round(best[0], 2), "rule_us": round(timed["rule"], 2),
                     "all_us": {a: round(b, 2) for a, b in timed.items()}}
            # keep the rule's choice unless the measured winner is clearly (3 %) faster: noise must not flip plans
            entry["use"] = best[0] < 0.97 * timed["rule"]
            plan[plan_key(fmt, m, n, k, act)] = entry
            if verbose:
                print(json.dumps({"shape": [fmt, m, n, k, int(act)], **entry}), flush=True)
    ws.check_status()
    return plan


def install(plan: dict | None) -> int:
    """Make ``kernels.wq_gemm`` / ``wq_gemm_act`` use the plan's entries whose measured gain was kept.  Returns the
    number of installed entries; ``None`` clears the table."""
    K.TUNED_PLANS.clear()
    if not plan:
        return 0
    for key, e in plan.items():
        if e.get("use"):
            K.TUNED_PLANS[key] = (e["kernel"] == "stream_k", int(e["splits"]))
    return len(K.TUNED_PLANS)


def prepare(cfg, rows, device, preparation=None, tp: int = 1) -> dict:
    """The plan for ``cfg`` at the given row counts: from the plan cache when ``preparation`` holds one made by this
    implementation on this GPU model, else measured now (and stored)."""
    shapes = model_shapes(cfg, tp)
    operands = {"shapes": [list(s) for s in shapes], "rows": sorted(rows)}
    if preparation is None:
        return tune(shapes, sorted(rows), device)
    return preparation.plan("gemm_launch", operands, lambda: tune(shapes, sorted(rows), device))


def main(argv=None) -> int:
    from ..models.config import NAMED_CONFIGS
    ap = argparse.ArgumentParser(description="measure the launch plan of a model's weight GEMMs")
    ap.add_argument("--model", default="dense-8b", choices=sorted(NAMED_CONFIGS))
    ap.add_argument("--rows", type=int, nargs="+", default=[16, 64, 256])
    ap.add_argument("--tp", type=int, default=1)
    a = ap.parse_args(argv)
    plan = tune(model_shapes(NAMED_CONFIGS[a.model](), a.tp), a.rows, "cuda:0", verbose=True)
    gain = sum(e["rule_us"] - e["us"] for e in plan.values() if e["use"])
    print(json.dumps({"entries": len(plan), "kept": sum(e["use"] for e in plan.values()), "gain_us_per_call_sum": round(gain, 1)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
