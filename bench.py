#!/usr/bin/env python
"""Headline serving benchmark: output tokens/s of the dense 8B-class decoder at 256 concurrent requests.

Config (BASELINE.json, second entry): 36 layers, hidden 4096, 32 q / 8 kv heads of 128, SwiGLU 12288, vocab
151936, RoPE theta 1e6; random-init N(0, 0.02) weights quantized offline to 4-bit CubicQuant (group 128);
INT8 K / INT8 V paged cache; 256 concurrent requests with 1024 random input tokens each; greedy decoding
under CUDA graphs; tensor parallel over ``--gpus`` ranks.

A *step* is one engine iteration in the steady decode phase: every one of the 256 running requests gets one
new token (context 1024 + i at step i).  The prompts are prefilled through the same engine before the timed
region (that phase is reported separately as ``prefill_tok_s``); nothing inside a timed step is skipped:
embedding, all layers, lm_head, sampling, and -- for the end-to-end number -- the per-step host -> device copy of
the step's inputs from pinned memory and the device -> host read of the sampled tokens.

Prints ONE JSON line on rank 0.  ``--impl reference`` runs the reference arm (see ``baseline/``).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

BASELINE_TOK_S = 2226.0   # reference's published dense total tok/s @ C=256 (4x SM120, different model/hardware)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="dense-8b")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"], help="TP collective path")
    ap.add_argument("--weights", default="", choices=["", "fp8", "fp8_block", "q4k"],
                    help="weight format instead of the config's own (fp8 / fp8_block: e4m3 weights with row or 128 x 128 "
                         "block scales, per-token e4m3 activations, fp8 tensor cores; q4k: 4-bit k-quant style affine "
                         "sub-blocks of 32; each is a different benchmark than the 4-bit Cubic headline)")
    ap.add_argument("--shared-prefix", type=int, default=0,
                    help="the first N tokens of every prompt are the same and the prefix cache is on: one request is "
                         "prefilled first, the others resume from its pages")
    ap.add_argument("--dynamic-draft", action="store_true", help="speculative rounds: per-request draft length 1..depth")
    ap.add_argument("--pp", type=int, default=1, choices=[1, 2], help="pipeline stages (tp = gpus / pp)")
    ap.add_argument("--kv", default="", help="K,V cache bits, e.g. 8,8 or 4,8 (default: 8,8 dense, 4,8 MoE)")
    ap.add_argument("--prefill-tokens", type=int, default=8192, help="token budget of a prefill step")
    ap.add_argument("--spec-depth", type=int, default=0, help="MTP draft tokens per round (0 = no speculation)")
    ap.add_argument("--context", default="mean", choices=["mean", "start"],
                    help="where in the 512-token decode the timed steps sit: around its mean context (input + 256) or "
                         "right after the prefill")
    ap.add_argument("--output-len", type=int, default=512, help="output tokens per request of the benchmark config")
    ap.add_argument("--no-check", action="store_true", help="skip the untimed multi-GPU logit check")
    ap.add_argument("--accept", type=float, default=0.7,
                    help="forced per-depth acceptance probability of speculative rounds (random weights never agree)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_reference(args) -> None:
    from baseline.reference_arm import run as ref_run
    print(json.dumps(ref_run(args)), flush=True)


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    import numpy as np
    import torch
    import torch.distributed as dist

    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.config import NAMED_CONFIGS
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = NAMED_CONFIGS[args.model]()
    if args.layers:
        from dataclasses import replace
        cfg = replace(cfg, num_layers=args.layers)
    if args.weights in ("fp8", "fp8_block"):
        from dataclasses import replace
        cfg = replace(cfg, quant=replace(cfg.quant, method=args.weights, bits=8, group_size=128 if args.weights == "fp8_block" else 0))
        if args.comm == "fused" and args.gpus > 1:
            args.comm = "nccl"          # the fp8 activation quantizer is a kernel of its own (see DecoderRunner)
    elif args.weights == "q4k":
        from dataclasses import replace
        cfg = replace(cfg, quant=replace(cfg.quant, method="gguf", bits=4, group_size=32))
    k_bits, v_bits = (int(b) for b in (args.kv or ("4,8" if cfg.is_moe else "8,8")).split(","))
    tp = pp = None
    tp_size, tp_rank, layer_range = world // args.pp, rank % (world // args.pp), None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from cubic_serve_b200.parallel.tp import TensorParallel
        tp_group = dist.group.WORLD
        if args.pp > 1:
            from cubic_serve_b200.contracts.execution import ParallelTopology
            from cubic_serve_b200.parallel.pp import PipelineStage
            topo = ParallelTopology.single_node(range(world), tp_size, args.pp)
            pp = PipelineStage.from_topology(topo, rank, dist.group.WORLD)
            layer_range = topo.layer_range(pp.stage, cfg.num_layers)
            for stage in range(args.pp):
                if tp_size > 1:
                    g = dist.new_group(list(range(stage * tp_size, (stage + 1) * tp_size)))
                    tp_group = g if stage == pp.stage else tp_group
        if tp_size > 1:
            mode = args.comm if pp is None else "nccl"
            tp = TensorParallel(tp_group, dev, mode=mode, hidden=cfg.hidden_size,
                                max_tokens=args.prefill_tokens, rows_max=max(args.concurrency, 512))
    C, L = args.concurrency, args.input_len
    # the config decodes `output_len` tokens per request: the timed steps sit around the MEAN context of that decode
    # (input + output / 2); the steps before them run untimed
    advance = 0
    if args.context == "mean" and not args.spec_depth:
        advance = max(0, args.output_len // 2 - args.steps // 2 - args.warmup)
    total_steps = args.warmup + args.steps + advance
    slack = 64 * (1 + args.spec_depth) if args.shared_prefix else 0   # the first request decodes while the others prefill
    max_len = L + total_steps * (1 + args.spec_depth) + 8 + args.spec_depth + slack
    pages_per_req = -(-max_len // 16)
    num_pages = C * pages_per_req + 8
    prefill_tokens = args.prefill_tokens

    weights = random_decoder_weights(cfg, dev, seed=0, tp_rank=tp_rank, tp_size=tp_size, layer_range=layer_range)
    # untimed prologue: the multi-GPU paths against each other and against one GPU, at the logit level
    check = {"n_gpus": world, "note": "one GPU: no partition to compare"}
    if tp is not None and pp is None and not args.no_check:
        from cubic_serve_b200.parallel.tp_check import run_check
        check = run_check(cfg, dev, tp_group, weights=weights, k_bits=k_bits, v_bits=v_bits, tp1_layers=4)
    runner = DecoderRunner(cfg, weights, num_pages=num_pages, max_tokens=prefill_tokens, k_bits=k_bits, v_bits=v_bits,
                           tp=tp, pp=pp, max_requests=max(C, 1))
    if args.spec_depth:
        from cubic_serve_b200.executor.spec_executor import SpeculativeGpuExecutor
        from cubic_serve_b200.models.mtp import MtpRunner, random_mtp_weights
        assert pp is None and (tp is None or tp.mode == "nccl"), "speculative rounds: --comm nccl, no pipeline stages"
        ex = SpeculativeGpuExecutor(runner, MtpRunner(runner, random_mtp_weights(cfg, dev, tp_rank=tp_rank, tp_size=tp_size)),
                                    args.spec_depth,
                                    force_acceptance=args.accept, max_rows=C, max_prefill_tokens=prefill_tokens,
                                    max_model_len=max_len)
    else:
        ex = GpuExecutor(runner, max_rows=C, max_prefill_tokens=prefill_tokens, max_model_len=max_len)
        ex.capture_decode_graphs([C])
    ex.timing = True
    eng = LLMEngine(ex, num_pages=num_pages,
                    scheduler_config=SchedulerConfig(max_running_requests=C, max_batched_tokens=prefill_tokens,
                                                     prefill_chunk_tokens=prefill_tokens, max_model_len=max_len,
                                                     enable_prefix_cache=args.shared_prefix > 0))
    if args.spec_depth and args.dynamic_draft:
        eng.enable_dynamic_draft()
    rng = np.random.default_rng(1)
    prompts = rng.integers(0, cfg.vocab_size, size=(C, L)).tolist()
    if args.shared_prefix:
        shared = rng.integers(0, cfg.vocab_size, size=min(args.shared_prefix, L - 1)).tolist()
        prompts = [shared + p[len(shared):] for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=total_steps * (1 + args.spec_depth) + 4 + slack, ignore_eos=True)
    if args.shared_prefix and C > 1:
        # the first request's prefill publishes the shared pages; the others are admitted after it and resume there
        eng.add_request(prompts[0], SamplingParams(**vars(sp)))
        while any(r.remaining > 1 for r in eng.scheduler.running + eng.scheduler.waiting):
            eng.step()
        prompts_rest = prompts[1:]
    else:
        prompts_rest = prompts
    for p in prompts_rest:
        eng.add_request(p, SamplingParams(**vars(sp)))

    def sync():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # everything the untimed prologue (weight generation, the multi-GPU check with its own buffers) left for the
    # garbage collector goes now: a collection of those objects inside the timed region frees device and
    # symmetric memory, which stalls the step it lands in (and, through the peer waits, the other ranks' step)
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    gc.freeze()
    # ---- prefill phase (untimed for the headline; reported on the side)
    sync()
    t0 = time.perf_counter()
    n_prefill_steps = 0
    first_token_at: dict[str, float] = {}          # request id -> seconds from submission to its first token
    while any(r.remaining > 1 for r in eng.scheduler.running + eng.scheduler.waiting) or eng.scheduler.waiting:
        for o in eng.step():
            first_token_at.setdefault(o.request_id, time.perf_counter() - t0)
        n_prefill_steps += 1
    sync()
    prefill_s = time.perf_counter() - t0
    assert len(eng.scheduler.running) == C, len(eng.scheduler.running)

    # ---- decode: the steps up to the mean context (untimed), W warm-up steps, K timed steps
    early_ms = None
    if advance:
        ex.device_ms = []
        for _ in range(advance):
            outs = eng.step()
        sync()
        early_ms = float(np.median(ex.device_ms[3:3 + args.steps])) if len(ex.device_ms) > 3 else None
    for _ in range(args.warmup):
        outs = eng.step()
        assert len(outs) >= C
    context_at_timed = int(L + advance + args.warmup)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ex.device_ms = []
    sync()
    t0 = time.perf_counter()
    launches = 0
    emitted = 0
    for _ in range(args.steps):
        outs = eng.step()
        emitted += len(outs)
        launches += ex.kernel_launches_last
    sync()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else {}
    assert len(outs) >= C
    runner.ws.check_status()
    dev_ms = float(sum(ex.device_ms))
    step_ms = sorted(float(v) for v in ex.device_ms)
    step_stats = {"p50": round(step_ms[len(step_ms) // 2], 4), "max": round(step_ms[-1], 4),
                  "slow_steps": [i for i, v in enumerate(ex.device_ms) if v > 1.25 * step_ms[len(step_ms) // 2]]}
    stats = torch.tensor([dev_ms, wall_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = stats.tolist()
    tokens = emitted
    value = tokens / (dev_ms / 1e3)
    e2e = tokens / (wall_ms / 1e3)
    if rank == 0:
        line = {
            "metric": f"output tok/s @{C} concurrent (decode steps, device-timed, max over ranks)",
            "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            # the reference publishes no B200 number: this ratio is against its best published figure on OTHER hardware
            # and another model (dense, 4 x SM120, C = 256), kept for context only
            "vs_baseline": round(value / BASELINE_TOK_S, 3), "vs_baseline_note": "published 4xSM120 figure, other model",
            "dtype": f"bf16 activations, {cfg.quant.method} {cfg.quant.bits}-bit weights, INT{k_bits}/INT{v_bits} KV",
            "data": "synthetic (random token ids; random-init N(0,0.02) weights quantized offline)",
            "impl": "ours",
            "config": {"model": cfg.name + ("" if not args.layers else f"-{args.layers}layers-INVALID"),
                       "global_batch": C, "seq_len": L, "parallelism": f"tp{tp_size}" + (f"pp{args.pp}" if args.pp > 1 else ""),
                       "comm": (tp.mode if tp is not None else "none"), "cuda_graphs": True, "kv_cache": f"int{k_bits}/int{v_bits}",
                       "l2": "inputs larger than L2 (weights + KV read per step >> 126 MB)",
                       "context_at_timed_steps": [context_at_timed, context_at_timed + args.steps],
                       "output_len": args.output_len, "timed_step_ms": step_stats,
                       **({"shared_prefix": args.shared_prefix, "prefix_hit_rate": round(eng.prefix.hit_rate, 4)}
                          if args.shared_prefix else {}),
                       **({"ms_per_step_at_start_of_decode": round(early_ms, 4),
                           "tok_s_at_start_of_decode": round(C / (early_ms / 1e3), 1)} if early_ms else {}),
                       "prefill_tok_s": round(C * L / prefill_s, 1), "prefill_steps": n_prefill_steps,
                       # all C requests are submitted at t = 0: TTFT includes queueing behind earlier prefill chunks
                       "ttft_p50_ms": round(1e3 * float(np.median(sorted(first_token_at.values()))), 1) if first_token_at else None,
                       "tpot_p50_ms": round(float(np.median(ex.device_ms)) / max(1.0, emitted / (C * args.steps)), 3),
                       "weights_gb": round(weights.nbytes() / 1e9, 2),
                       **({"speculative": {"depth": args.spec_depth, "forced_acceptance": args.accept,
                                           "tokens_per_verify_step": round(emitted / (C * args.steps), 3),
                                           "verify_step_ms": round(dev_ms / args.steps, 3)}} if args.spec_depth else {})},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": int(ex.h2d_bytes_last),
                    "d2h_bytes_per_step": int(ex.d2h_bytes_last), "api": "LLMEngine.step()"},
            "gpu_launches": int(launches),
            "check": check,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without tearing the communicator down: destroying a process group whose collectives are
        # referenced by live CUDA graphs can block forever, and there is nothing left to flush
        torch.cuda.synchronize(dev)
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
