"""Logit-level check of the tensor-parallel (and expert-parallel) paths on real GPUs.

Three executions of the SAME model are compared (``random_decoder_weights`` makes every partition a set of slices
of one rank-independent model):

* the fused NVLink path (``mode="fused"``: reduce-scatter / all-gather inside the GEMM kernels, expert-parallel
  dispatch / combine for MoE layers),
* the NCCL baseline (``mode="nccl"``: all-reduce after every row-parallel GEMM, replicated tokens for MoE),
* one GPU holding the whole model (rank 0 only; optional, on a model of few layers so that it fits and loads fast).

What is compared are the logits of the FIRST prefill step and of the decode step after it, before a near-tie of
random weights can send two greedy runs down different paths, as relative L2 error per row against a bound
derived from the reductions involved (``guardrail/compare.py::reduction_bound``), plus the greedy tokens.  The
reference checks its partitions the same way against a single-rank oracle computed in the same test
(``tests/executor/test_distributed_toy.py:339-437`` there).

Run under ``python -m torch.distributed.run --nproc-per-node N -m cubic_serve_b200.parallel.tp_check``; rank 0
prints one JSON line.  ``bench.py`` calls ``run_check`` in an untimed prologue.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import replace


def _step_logits(cfg, weights, dev, tp, prompts, k_bits, v_bits):
    """Prefill ``prompts`` in one eager step, then one decode step on the sampled tokens; returns the full-vocabulary
    fp32 logits of both steps (gathered over the tensor-parallel ranks) and the two token lists."""
    import torch
    import torch.distributed as dist

    from ..executor.gpu_executor import GpuExecutor, Segment
    from ..models.decoder import DecoderRunner
    R, P = len(prompts), len(prompts[0])
    pages_per = -(-(P + 2) // 16)
    T = max(R * P, 256)
    runner = DecoderRunner(cfg, weights, num_pages=R * pages_per + 8, max_tokens=T, k_bits=k_bits, v_bits=v_bits,
                           tp=tp, max_requests=max(R, 16))
    ex = GpuExecutor(runner, max_rows=max(R, 16), max_prefill_tokens=T, max_model_len=pages_per * 16, use_graphs=False)
    pages = [list(range(1 + i * pages_per, 1 + (i + 1) * pages_per)) for i in range(R)]

    def gathered():
        local = ex.logits[:R].float()
        if tp is None:
            return local.clone()
        parts = [torch.empty_like(local) for _ in range(tp.size)]
        dist.all_gather(parts, local.contiguous(), group=tp.group)
        return torch.cat(parts, 1)

    ids0 = [int(t) for t in ex.execute([Segment(i, prompts[i], 0, pages[i], True, uid=i) for i in range(R)])]
    torch.cuda.synchronize(dev)
    runner.ws.check_status()
    l0 = gathered()
    ids1 = [int(t) for t in ex.execute([Segment(i, [ids0[i]], P, pages[i], True, uid=i) for i in range(R)])]
    torch.cuda.synchronize(dev)
    runner.ws.check_status()
    l1 = gathered()
    del ex, runner
    return (l0, l1), (ids0, ids1)


def _rel_rows(a, b):
    """Per-row relative L2 error of ``a`` against ``b``."""
    return (a - b).norm(dim=1) / b.norm(dim=1).clamp_min(1e-20)


def _summary(errs, bound: float) -> dict:
    """Worst and median row, and the share of rows inside the bound.  A mixture-of-experts model routes by a discrete
    top-k: rounding noise can hand a row a different expert, which moves that row's logits by far more than the
    rounding itself, so for those models the median and the share of rows are what a correct execution bounds."""
    import torch
    e = torch.cat([x.flatten() for x in errs])
    return {"max_rel_logit_err": round(float(e.max()), 6), "p50_rel_logit_err": round(float(e.median()), 6),
            "rows_within_bound": round(float((e <= bound).float().mean()), 4)}


def run_check(cfg, dev, group, weights=None, requests: int = 16, prompt_len: int = 48, k_bits: int = 8, v_bits: int = 8,
              tp1_layers: int = 0, seed: int = 0, ep_size: int | None = None) -> dict:
    """Compare fused vs NCCL (on ``cfg`` with ``weights``, this rank's shard) and, when ``tp1_layers`` > 0, both against
    one GPU holding a ``tp1_layers``-layer version of the model.  Collective over ``group``; every rank returns the
    same dictionary.  ``ep_size`` below the group's size divides every expert's features over lanes (NCCL mode only)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from ..guardrail.compare import reduction_bound
    from ..models.decoder import random_decoder_weights
    from .tp import TensorParallel
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    rng = np.random.default_rng(seed + 7)
    prompts = rng.integers(0, cfg.vocab_size, size=(requests, prompt_len)).tolist()
    T = max(requests * prompt_len, 256)

    def both_modes(c, w):
        out = {}
        for mode in ("nccl", "fused"):
            if (c.is_hybrid or c.quant.method == "fp8" or (ep_size or size) != size or c.shared_intermediate_size) \
                    and mode == "fused":
                continue          # these run with the NCCL collectives (see DecoderRunner)
            tp = TensorParallel(group, dev, mode=mode, hidden=c.hidden_size, max_tokens=T, rows_max=max(requests, 16))
            out[mode] = _step_logits(c, w, dev, tp, prompts, k_bits, v_bits)
            del tp
            torch.cuda.synchronize(dev)
            dist.barrier(group)
        return out

    if weights is None:
        weights = random_decoder_weights(cfg, dev, seed=seed, tp_rank=rank, tp_size=size, ep_size=ep_size)
    res = both_modes(cfg, weights)
    report: dict = {"ranks": size, "model": cfg.name, "layers": cfg.num_layers, "rows": requests, "prompt_len": prompt_len,
                    "nvls": os.environ.get("CUBIC_SERVE_NVLS", "gather")}
    # a row of logits is the end of a chain of length-H .. length-I dot products of bf16 operands rounded to bf16 at every
    # layer boundary; one layer's bound times sqrt(2 x layers) independent roundings is what two correct executions with
    # different summation orders may differ by
    per_op = reduction_bound(None, torch.bfloat16, cfg.hidden_size)
    report["bound"] = round(per_op * (2 * max(1, cfg.num_layers)) ** 0.5, 5)
    if "fused" in res:
        (f0, f1), (fi0, fi1) = res["fused"]
        (n0, n1), (ni0, ni1) = res["nccl"]
        # the decode step consumes the token each execution sampled itself: its logits are compared for the rows where
        # both sampled the same one (a near-tie of random weights that rounding resolves differently is a different
        # input, not an error of the step)
        same = torch.tensor([a == b for a, b in zip(fi0, ni0)], device=dev)
        report.update(_summary([_rel_rows(f0, n0), _rel_rows(f1, n1)[same]], report["bound"]))
        report["first_tokens_equal"] = round(float(same.float().mean()), 4)
        report["fused_eq_nccl_tokens"] = round(float(np.mean([a == b for a, b in zip(fi0 + fi1, ni0 + ni1)])), 4)
        # every rank must hold the same tokens (the vocabulary-sharded samplers draw the same candidate everywhere)
        t = torch.tensor(fi0 + fi1 + ni0 + ni1, device=dev)
        parts = [torch.empty_like(t) for _ in range(size)]
        dist.all_gather(parts, t, group=group)
        report["ranks_agree"] = bool(all(torch.equal(p, parts[0]) for p in parts))
    if tp1_layers > 0:
        small = replace(cfg, num_layers=min(tp1_layers, cfg.num_layers))
        ws = random_decoder_weights(small, dev, seed=seed, tp_rank=rank, tp_size=size, ep_size=ep_size)
        part = both_modes(small, ws)
        del ws
        bound1 = per_op * (2 * small.num_layers) ** 0.5
        vals = torch.zeros(4, dtype=torch.float64, device=dev)
        if rank == 0:
            w1 = random_decoder_weights(small, dev, seed=seed)
            (o0, o1), (oi0, oi1) = _step_logits(small, w1, dev, None, prompts, k_bits, v_bits)
            del w1
            errs = []
            for mode, ((a0, a1), (ai0, _)) in part.items():
                same1 = torch.tensor([a == b for a, b in zip(ai0, oi0)], device=dev)
                errs += [_rel_rows(a0, o0), _rel_rows(a1, o1)[same1]]
            sm = _summary(errs, bound1)
            mode = "fused" if "fused" in part else "nccl"
            agree = float(np.mean([a == b for a, b in zip(part[mode][1][0] + part[mode][1][1], oi0 + oi1)]))
            vals = torch.tensor([sm["max_rel_logit_err"], agree, sm["p50_rel_logit_err"], sm["rows_within_bound"]],
                                dtype=torch.float64, device=dev)
        dist.broadcast(vals, src=dist.get_global_rank(group, 0), group=group)
        report["vs_one_gpu"] = {"layers": small.num_layers, "max_rel_logit_err": round(float(vals[0]), 6),
                                "p50_rel_logit_err": round(float(vals[2]), 6), "rows_within_bound": round(float(vals[3]), 4),
                                "token_agreement": round(float(vals[1]), 4), "bound": round(bound1, 5)}
    torch.cuda.synchronize(dev)
    dist.barrier(group)
    return report


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-8b")
    ap.add_argument("--layers", type=int, default=4, help="layers of the checked model (0 = the named config's own)")
    ap.add_argument("--experts", type=int, default=0, help="MoE: number of experts (0 = the config's own)")
    ap.add_argument("--kv-heads", type=int, default=0,
                    help="override the key/value head count (fewer heads than ranks: ranks share copies of a head)")
    ap.add_argument("--ep", type=int, default=0,
                    help="MoE: expert owners among the ranks (0 = every rank owns whole experts); the ranks of an owner "
                         "divide each expert's intermediate features")
    ap.add_argument("--shared-expert", type=int, default=0, help="MoE: width of a sigmoid-gated shared expert (0 = none)")
    ap.add_argument("--qkv-bias", action="store_true", help="biases on the q / k / v projections")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=48)
    ap.add_argument("--kv", default="8,8")
    args = ap.parse_args(argv)
    import torch
    import torch.distributed as dist

    from ..models.config import NAMED_CONFIGS
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = NAMED_CONFIGS[args.model]()
    if args.layers:
        cfg = replace(cfg, num_layers=args.layers)
    if args.experts and cfg.is_moe:
        cfg = replace(cfg, num_experts=args.experts)
    if args.kv_heads:
        cfg = replace(cfg, num_kv_heads=args.kv_heads)
    if args.shared_expert and cfg.is_moe:
        cfg = replace(cfg, shared_intermediate_size=args.shared_expert)
    if args.qkv_bias:
        cfg = replace(cfg, qkv_bias=True)
    kb, vb = (int(b) for b in args.kv.split(","))
    report = run_check(cfg, dev, dist.group.WORLD, requests=args.requests, prompt_len=args.prompt_len, k_bits=kb, v_bits=vb,
                       tp1_layers=cfg.num_layers, ep_size=args.ep or None)
    if rank == 0:
        print(json.dumps(report), flush=True)
    torch.cuda.synchronize(dev)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
