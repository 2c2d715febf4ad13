"""The tensor-parallel site of a decoder layer on REAL GPUs: row-parallel GEMM -> sum + residual + norm -> column-
parallel GEMM, in the fused NVLink form and in the NCCL form, timed on the device.

One layer has two such sites (after the attention output projection and after the down projection).  The script
runs the FFN half of a dense layer in a loop,

    scatter GEMM (down, [H, I / N])  ->  reduce + norm  ->  gather GEMM + SwiGLU (gate/up, [2 I / N, H])

which is exactly the kernel sequence of ``DecoderRunner.forward_hidden_fused`` between two attention blocks, and
reports per rank count N:

* the time of one site inside a CUDA graph of ``--sites`` sites (CUDA events around the replay, max over ranks),
  fused and NCCL (GEMM, ``all_reduce``, norm, GEMM);
* the time of each kernel of the fused site from CUDA events recorded between the launches (eager; the events keep
  a kernel's prologue from overlapping its predecessor, so the three do not add up to the graph figure);
* NVLink bytes per site: the algorithmic minimum of reduce-scatter + all-gather of ``M x H`` bf16 rows and what the
  GPU's NVLink counters saw (``nvidia-smi nvlink -gt d``: read before and after the graph replays).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29517 \
        -m cubic_serve_b200.parallel.tp_site_bench --rows 256

The reference's counterpart of the fused reduction is ``ops/cuda/collective/fixed_rank_sum.py:596-722`` there.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess


def _nvlink_kib(index: int) -> tuple[int, int] | None:
    """Sum of the data counters (tx, rx) over the GPU's links in KiB, or None when the tool does not report them."""
    try:
        out = subprocess.run(["nvidia-smi", "nvlink", "-gt", "d", "-i", str(index)], capture_output=True, text=True,
                             timeout=20).stdout
    except (OSError, subprocess.TimeoutExpired):
        return None
    tx = [int(v) for v in re.findall(r"Data Tx:\s*(\d+)\s*KiB", out)]
    rx = [int(v) for v in re.findall(r"Data Rx:\s*(\d+)\s*KiB", out)]
    return (sum(tx), sum(rx)) if tx and rx else None


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=256, help="batch rows of the step")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=12288)
    ap.add_argument("--sites", type=int, default=36, help="sites per captured graph")
    ap.add_argument("--replays", type=int, default=20)
    args = ap.parse_args(argv)
    import torch
    import torch.distributed as dist

    from ..ops import kernels as K
    from ..ops import wq_pack
    from .tp import TensorParallel
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    size = dist.get_world_size()
    M, H, I = args.rows, args.hidden, args.inter
    g = torch.Generator(device=dev).manual_seed(1 + rank)

    def cubic(n, k):
        codes = torch.randint(-7, 8, (n, k), dtype=torch.int8, device=dev, generator=g)
        full = lambda v: torch.full((n, k // 128), v, device=dev)          # noqa: E731
        return wq_pack.pack_cubic4(codes, full(0.02), full(0.75), full(0.25), 128)

    down = cubic(H, I // size)                                             # row-parallel shard
    gate_up = wq_pack.swiglu_interleave(cubic(2 * I // size, H))           # column-parallel shard
    norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    act = (torch.randn(M, I // size, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    gu = torch.empty(M, 2 * I // size, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(dev)
    report = {"ranks": size, "m": M, "hidden": H, "inter": I, "sites_per_graph": args.sites,
              "nvls": os.environ.get("CUBIC_SERVE_NVLS", "gather")}

    def max_over_ranks(ms: float) -> float:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def time_graph(site, begin=None) -> float:
        """Device time of one site: a graph of ``--sites`` sites, replayed; the graph of the same number of L2 flushes
        alone is subtracted."""
        times = []
        with torch.cuda.stream(stream):
            for with_site in (True, False):
                if begin is not None:
                    begin()
                if with_site:
                    for _ in range(3):
                        site()
                stream.synchronize()
                dist.barrier()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(args.sites):
                        flush.zero_()
                        if with_site:
                            site()
                for _ in range(3):
                    graph.replay()
                stream.synchronize()
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(args.replays):
                    graph.replay()
                b.record(stream)
                stream.synchronize()
                times.append(max_over_ranks(a.elapsed_time(b)) / (args.replays * args.sites))
                del graph
        return (times[0] - times[1]) * 1e3

    # ---------------------------------------------------------------- fused
    tp = TensorParallel(dist.group.WORLD, dev, mode="fused", hidden=H, max_tokens=max(M, 256), rows_max=max(M, 16))
    f = tp.fused
    f.begin_step(M)
    state = {"s": 0}

    def fused_site():
        s = state["s"] ^ 1
        f.gemm_scatter(act, down, s)
        f.reduce_norm(norm_w, s, H, 1e-6)
        f.gate_up_act(gate_up, gu, act, s)
        state["s"] = s

    before = _nvlink_kib(local)
    report["fused_site_us"] = round(time_graph(fused_site), 2)
    after = _nvlink_kib(local)
    f.ws.check_status()
    # reduce-scatter: this rank sends the partial rows it does not own; all-gather: it sends its own rows to N - 1
    # peers (through the switch's multicast: once)
    rs = M * H * 2 * (size - 1) / size
    ag = M * H * 2 / size * ((size - 1) if not f.nvls_gather else 1)
    report["nvlink_tx_bytes_per_site_algorithmic"] = int(rs + ag)
    if before is not None and after is not None:
        sites_run = (3 + 3 * args.sites + args.replays * args.sites)          # warm-up, graph warm-up, timed replays
        report["nvlink_tx_bytes_per_site_counted"] = int((after[0] - before[0]) * 1024 / sites_run)
        report["nvlink_rx_bytes_per_site_counted"] = int((after[1] - before[1]) * 1024 / sites_run)
    # per kernel, eager, events between the launches
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(20)]
    with torch.cuda.stream(stream):
        for it in range(20):
            flush.zero_()
            s = state["s"] ^ 1
            ev[it][0].record(stream)
            f.gemm_scatter(act, down, s)
            ev[it][1].record(stream)
            f.reduce_norm(norm_w, s, H, 1e-6)
            ev[it][2].record(stream)
            f.gate_up_act(gate_up, gu, act, s)
            ev[it][3].record(stream)
            state["s"] = s
        stream.synchronize()
    for i, name in enumerate(("scatter_gemm_us", "reduce_norm_us", "gather_gemm_us")):
        vals = sorted(e[i].elapsed_time(e[i + 1]) for e in ev[5:])
        report[name] = round(max_over_ranks(vals[len(vals) // 2]) * 1e3, 2)
    f.ws.check_status()

    # ---------------------------------------------------------------- NCCL baseline of the same kernels
    part = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    h = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
    x = torch.empty(M, H, dtype=torch.bfloat16, device=dev)

    def nccl_site():
        K.wq_gemm(act, down, out=part)
        dist.all_reduce(part)
        K.rmsnorm(part, norm_w, 1e-6, out=x, residual=h)
        K.wq_gemm_act(x, gate_up, out=act)

    report["nccl_site_us"] = round(time_graph(nccl_site), 2)
    # roofline of the site: the GEMMs' FLOPs at the sustained tensor figure against the bytes that must cross NVLink at
    # the measured 770 GB/s per direction
    flops = 2.0 * M * H * (I // size) * 3
    report["roofline_us"] = {"tensor_1335_tflops": round(flops / 1335e12 * 1e6, 2),
                             "weights_6556_gbs": round((down.nbytes + gate_up.nbytes) / 6556e9 * 1e6, 2),
                             "nvlink_770_gbs": round((rs + ag) / 770e9 * 1e6, 2)}
    if rank == 0:
        print(json.dumps(report), flush=True)
    torch.cuda.synchronize(dev)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
