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
    torch.cuda.synchronize(dev)
    K.workspace(dev).check_status()
    ok = all(r["class"] != "mismatch" for r in results)
    return {"ok": ok, "device": torch.cuda.get_device_name(dev), "seconds": round(time.time() - t0, 2), "results": results}
