"""Same-box operator timings of the UNMODIFIED reference (``baseline/_ref``), for the benchmark's projection shapes.

The reference's serving engine cannot start on this image (it compiles its native kernels with a CUDA 13.0 ``nvcc``
and pins torch 2.13 / triton 3.7.1), but its operator layer is plain Python + Triton and imports under the installed
torch / triton.  This script drives that layer through the reference's own public operator API,
``PackedLinearOperators().bind_linear(x, weight, out).launch()`` (``ops/cuda/linear/quantized.py:559`` there; the call
its tests make, ``tests/ops/test_cuda_quantized.py:417``), on 4-bit CubicQuant matrices of the dense-8B shapes:

* first with the stock configuration (Cubic linears go to the reference's Marlin kernels, which need its native
  compiler: recorded as unavailable when that raises);
* then with the reference's own operator-config switch ``{"cubic_linear": {"marlin_enabled": false}}``, which selects
  its Triton weight-only GEMM (``quantization/common/kernels.py:68`` with the Cubic loader
  ``extensions/cubic/kernels.py:44``).

Nothing of this repository's package is imported.  Timing: each launch inside a CUDA graph, a buffer larger than L2
written before every launch, the same graph without the launches subtracted, CUDA events.  One JSON line per shape.

    python baseline/reference_ops.py            # on a GPU box
"""
from __future__ import annotations

import json
import os
import sys
import traceback

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def _timeit_graph(torch, fn, flush, launches: int = 5, repeats: int = 3) -> float:
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


def main() -> None:
    if not os.path.isdir(os.path.join(REF_DIR, "cubic_serve")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    sys.path.insert(0, REF_DIR)
    import torch
    import triton
    from cubic_serve.models.quantization import QuantizationScheme, WeightFormat
    from cubic_serve.models.quantized_checkpoint import QuantizedMatrix
    from cubic_serve.ops.cuda.linear.quantized import PackedLinearOperators
    from cubic_serve.ops.strategies import OperatorConfig

    dev = "cuda:0"
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
    triton_only = OperatorConfig.from_dict({"version": 1, "overrides": {"cubic_linear": {"marlin_enabled": False}}})
    info = {"impl": "reference", "torch": torch.__version__, "triton": triton.__version__,
            "gpu": torch.cuda.get_device_name(0), "note": "reference pins torch 2.13.0 / triton 3.7.1; run as installed"}
    print(json.dumps(info), flush=True)

    def cubic_matrix(n: int, k: int) -> QuantizedMatrix:
        g = k // 128
        payload = {
            "weight_packed": torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev),
            "weight_scale": torch.full((n, g), 0.02, dtype=torch.float32, device=dev),
            "weight_a": torch.full((n, g), 0.75, dtype=torch.float16, device=dev),
            "weight_b": torch.full((n, g), 0.25, dtype=torch.float16, device=dev),
        }
        return QuantizedMatrix(payload, QuantizationScheme(WeightFormat.CUBIC, 4, 128, metadata="float32-scale-float16-ab"),
                               (n, k))

    shapes = [(256, 6144, 4096), (256, 4096, 4096), (256, 24576, 4096), (256, 4096, 12288),
              (16, 24576, 4096), (64, 24576, 4096)]
    for m, n, k in shapes:
        w = cubic_matrix(n, k)
        x = torch.randn(m, k, dtype=torch.bfloat16, device=dev)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        for label, cfg in (("stock (Marlin)", None), ("marlin_enabled=false (Triton weight-only GEMM)", triton_only)):
            row = {"op": "reference cubic4 linear", "path": label, "m": m, "n": n, "k": k}
            try:
                ops = PackedLinearOperators(cfg) if cfg is not None else PackedLinearOperators()
                binding = ops.bind_linear(x, w, y)
                binding.launch()
                torch.cuda.synchronize()
                ms = _timeit_graph(torch, binding.launch, flush)
                row.update(us=round(ms * 1e3, 1), tflops=round(2 * m * n * k / ms / 1e9, 1), timing="in-graph, L2 flushed")
            except Exception as exc:  # noqa: BLE001 - the reason is the result
                row["unavailable"] = f"{type(exc).__name__}: {str(exc)[:200]}"
                if os.environ.get("REFERENCE_OPS_TRACE"):
                    traceback.print_exc()
            print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
