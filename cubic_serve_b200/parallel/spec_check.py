"""Speculative decoding under tensor parallelism, on real GPUs: MTP rounds of a tensor-parallel model (NCCL
collectives, vocabulary-sharded sampling of drafts and review rows) must emit the tokens of plain greedy decoding of
the SAME partition, because greedy rounds are lossless (one GPU holding the whole model is decoded too, for the record:
its sums are ordered differently, and a token that rounding flips sends the rest of that request elsewhere).

Run under ``python -m torch.distributed.run --nproc-per-node N -m cubic_serve_b200.parallel.spec_check``; every rank
drives the same engine in lockstep (as ``bench.py`` does), rank 0 also decodes the same prompts on its own and prints
one JSON line.  (Reference: the tensor-parallel draft batches of ``runtime/performance.py:7189-7556`` there.)
"""
from __future__ import annotations

import argparse
import json
import os


def main(argv=None) -> dict | None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=16)
    args = ap.parse_args(argv)
    import numpy as np
    import torch
    import torch.distributed as dist

    from ..executor.gpu_executor import GpuExecutor
    from ..executor.spec_executor import SpeculativeGpuExecutor
    from ..models.config import ModelConfig, QuantSpec
    from ..models.decoder import DecoderRunner, random_decoder_weights
    from ..models.mtp import MtpRunner, random_mtp_weights
    from ..runtime.engine import LLMEngine
    from ..runtime.scheduler import SamplingParams, SchedulerConfig
    from .tp import TensorParallel
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = ModelConfig(name="spec-tp", num_layers=3, hidden_size=1024, num_q_heads=16, num_kv_heads=8, head_dim=128,
                      intermediate_size=2048, vocab_size=4096, rope_theta=1e6, quant=QuantSpec("cubic", 4, 128))
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (17, 40, 33, 64)]
    sp = SamplingParams(max_tokens=args.tokens, ignore_eos=True)
    sched = SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512, enable_prefix_cache=False)

    def generate(tp, tp_rank, tp_size, depth):
        w = random_decoder_weights(cfg, dev, seed=0, std=0.05, tp_rank=tp_rank, tp_size=tp_size)
        runner = DecoderRunner(cfg, w, num_pages=128, max_tokens=512, tp=tp)
        kw = dict(max_rows=8, max_prefill_tokens=512, max_model_len=256)
        if depth:
            mtp = MtpRunner(runner, random_mtp_weights(cfg, dev, std=0.05, tp_rank=tp_rank, tp_size=tp_size))
            ex = SpeculativeGpuExecutor(runner, mtp, depth, **kw)
        else:
            ex = GpuExecutor(runner, use_graphs=False, **kw)
        out = LLMEngine(ex, 128, sched).generate(prompts, sp)
        runner.ws.check_status()
        return out, (ex.stats if depth else None)

    tp = TensorParallel(dist.group.WORLD, dev, mode="nccl", hidden=cfg.hidden_size, max_tokens=512) if world > 1 else None
    spec, stats = generate(tp, rank if tp else 0, world if tp else 1, args.depth)
    same_partition, _ = generate(tp, rank if tp else 0, world if tp else 1, 0)
    report = None
    if rank == 0:
        plain, _ = generate(None, 0, 1, 0)

        def agreement(a, b):
            return round(float(np.mean([x == y for pa, pb in zip(a, b) for x, y in zip(pa, pb)])), 4)

        report = {"ranks": world, "depth": args.depth, "rounds": stats["rounds"], "proposed": stats["proposed"],
                  "accepted": stats["accepted"], "token_agreement_with_plain_greedy": agreement(same_partition, spec),
                  "token_agreement_with_one_gpu_greedy": agreement(plain, spec),
                  "first_tokens_equal_one_gpu": agreement([p[:1] for p in plain], [p[:1] for p in spec]),
                  "lengths_ok": all(len(o) == args.tokens for o in spec)}
        print(json.dumps(report), flush=True)
    if world > 1:
        torch.cuda.synchronize(dev)
        dist.barrier()
        os._exit(0)
    return report


if __name__ == "__main__":
    main()
