"""Device time of the vision tower on one GPU: random weights of a release-sized tower, a few input geometries.

    python -m cubic_serve_b200.utils.vision_bench                 # 27 layers, 1152 wide, patch 16, bf16

For every geometry the script encodes the same input ``--iters`` times after ``--warmup`` calls, timed with CUDA events
on the launching stream, and reports milliseconds per call, patches per second and the tensor throughput of the
tower's GEMMs and attention (FLOPs counted from the shapes; library kernels: the tower is outside the decode loop).
Prints one JSON object.
"""
from __future__ import annotations

import argparse
import json


def tower_flops(cfg, grid: tuple[int, int, int]) -> float:
    t, h, w = grid
    n, hid, inter, frame = t * h * w, cfg.hidden_size, cfg.intermediate_size, h * w
    per_token_layer = 2 * (4 * hid * hid + 2 * hid * inter) + 4 * frame * hid          # projections, MLP, QK^T and PV
    merge = cfg.merge_width
    merger = (n // cfg.spatial_merge_size ** 2) * 2 * (merge * merge + merge * cfg.out_hidden_size)
    return n * (cfg.depth * per_token_layer + 2 * cfg.patch_width * hid) + merger


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--depth", type=int, default=27)
    ap.add_argument("--hidden", type=int, default=1152)
    ap.add_argument("--inter", type=int, default=4304)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--out", type=int, default=2560)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    import torch

    from ..models.vision import VisionConfig, VisionEncoder, random_vision_weights
    dev = torch.device("cuda", 0)
    cfg = VisionConfig(depth=args.depth, hidden_size=args.hidden, intermediate_size=args.inter, num_heads=args.heads,
                       out_hidden_size=args.out, patch_size=16, spatial_merge_size=2, temporal_patch_size=2,
                       num_position_embeddings=2304)
    enc = VisionEncoder(cfg, random_vision_weights(cfg, 0, torch.bfloat16, dev, std=0.02))
    report = {"tower": {"layers": cfg.depth, "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size,
                        "heads": cfg.num_heads, "dtype": "bf16"}, "cases": []}
    cases = [("image 448 x 448", (1, 28, 28)), ("image 1024 x 1024", (1, 64, 64)), ("image 2048 x 1024", (1, 128, 64)),
             ("clip 16 frames 448 x 448", (8, 28, 28))]
    stream = torch.cuda.current_stream(dev)
    for name, grid in cases:
        n = grid[0] * grid[1] * grid[2]
        px = torch.randn(n, cfg.patch_width, device=dev, dtype=torch.bfloat16)
        g = torch.tensor([list(grid)])
        for _ in range(args.warmup):
            enc.encode(px, g)
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(args.iters):
            rows, _ = enc.encode(px, g)
        b.record(stream)
        torch.cuda.synchronize(dev)
        ms = a.elapsed_time(b) / args.iters
        report["cases"].append({"input": name, "grid": list(grid), "patches": n, "feature_rows": int(rows.shape[0]),
                                "ms": round(ms, 3), "patches_per_s": round(n / ms * 1e3),
                                "tflops": round(tower_flops(cfg, grid) / ms / 1e9, 1)})
    print(json.dumps(report), flush=True)


if __name__ == "__main__":
    main()
