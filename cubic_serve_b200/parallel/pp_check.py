"""Self-check of the pipeline-parallel path: greedy tokens of a small random decoder, with or without stages.

Run alone (``python -m cubic_serve_b200.parallel.pp_check``) for the one-GPU tokens, or under
``python -m torch.distributed.run --nproc-per-node 2 -m cubic_serve_b200.parallel.pp_check --pp 2`` for two
stages; the token lists must be identical, because a stage boundary moves bf16 rows unchanged and every
kernel sees the same operands in the same order (the reference's TP x PP check compares logits the same way:
``executor/distributed_reference.py``).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import replace


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--requests", type=int, default=48)
    ap.add_argument("--steps", type=int, default=12)
    args = ap.parse_args(argv)
    import numpy as np
    import torch
    import torch.distributed as dist

    from ..contracts.execution import ParallelTopology
    from ..executor.gpu_executor import GpuExecutor
    from ..models.config import dense_8b_config
    from ..models.decoder import DecoderRunner, random_decoder_weights
    from ..runtime.engine import LLMEngine
    from ..runtime.scheduler import SamplingParams, SchedulerConfig
    from .pp import PipelineStage

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.pp:
        raise SystemExit(f"--pp {args.pp} needs exactly {args.pp} ranks (tensor parallel size 1), got {world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = replace(dense_8b_config(), name="pp-check", num_layers=4, hidden_size=1024, num_q_heads=8, num_kv_heads=2,
                  intermediate_size=3072, vocab_size=8192)
    pp = layer_range = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        topo = ParallelTopology.single_node(range(world), 1, args.pp)
        pp = PipelineStage.from_topology(topo, rank, dist.group.WORLD)
        layer_range = topo.layer_range(pp.stage, cfg.num_layers)
    C = args.requests
    weights = random_decoder_weights(cfg, dev, seed=3, layer_range=layer_range)
    runner = DecoderRunner(cfg, weights, num_pages=C * 8 + 8, max_tokens=2048, pp=pp)
    ex = GpuExecutor(runner, max_rows=64, max_prefill_tokens=2048, max_model_len=128)
    ex.capture_decode_graphs([64])
    eng = LLMEngine(ex, num_pages=C * 8 + 8,
                    scheduler_config=SchedulerConfig(max_running_requests=64, max_batched_tokens=2048,
                                                     prefill_chunk_tokens=2048, max_model_len=128,
                                                     enable_prefix_cache=False))
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg.vocab_size, size=int(n)).tolist() for n in rng.integers(20, 60, size=C)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=args.steps, ignore_eos=True))
    runner.ws.check_status()
    result = {"pp": args.pp, "tokens": outs}
    if world > 1:
        torch.cuda.synchronize(dev)
        dist.barrier()
        if rank == 0:
            print(json.dumps(result), flush=True)
        os._exit(0)                      # communicators referenced by live CUDA graphs are not torn down
    return result


if __name__ == "__main__":
    print(json.dumps(main()), flush=True)
