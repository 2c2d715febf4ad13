"""Canary regions (``guardrail/canary.py``): kernels given ragged shapes must not write outside their outputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_canaries_report_a_store_outside_the_tensor():
    from cubic_serve_b200.guardrail.canary import CanaryArena
    arena = CanaryArena("cuda")
    a = arena.tensor((10, 7), torch.bfloat16, "a")
    b = arena.tensor((33,), torch.float32, "b")
    a.fill_(1.0)
    b.fill_(2.0)
    assert arena.check() is None
    # one element past the end of b: inside the 256-byte slack, which belongs to the band after b
    raw = torch.empty(0, dtype=torch.float32, device="cuda").set_(b.untyped_storage(), b.storage_offset(), (40,))
    raw[35] = 5.0
    hit = arena.check()
    assert hit is not None and hit.name == "b" and hit.band == 3 and hit.damaged_words >= 1, hit


@pytest.mark.parametrize("fmt", ["cubic4", "fp8", "fp8_block"])
def test_gemm_epilogues_respect_ragged_edges(fmt):
    """200 rows (not a multiple of 16) and 1000 columns (not a multiple of 128): outputs, partial sums and the fused
    activation must stay inside their tensors in every kernel form."""
    from cubic_serve_b200.guardrail.canary import CanaryArena
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.quantization import formats
    from cubic_serve_b200.utils.kernel_bench import random_cubic_weight
    dev = torch.device("cuda")
    m, n, k = 200, 1000, 1152
    if fmt == "cubic4":
        w = random_cubic_weight(n, k)
    else:
        p = formats.fp8_quantize(torch.randn(n, k, device=dev) * 0.05, block=fmt == "fp8_block")
        w = (wq_pack.pack_fp8_block(p["weight"], p["weight_scale_inv"]) if fmt == "fp8_block"
             else wq_pack.pack_fp8(p["weight"], p["weight_scale"]))
    arena = CanaryArena(dev)
    x = arena.tensor((m, k), torch.bfloat16, "x")
    x.copy_(torch.randn(m, k, device=dev))
    res = arena.tensor((m, n), torch.bfloat16, "residual")
    res.zero_()
    outs = []
    for i, kw in enumerate((dict(splits=1), dict(splits=3), dict(splits=9)) + ((dict(min_units=2),) if fmt != "fp8_block" else ())):
        y = arena.tensor((m, n), torch.bfloat16, f"y{i}")
        K.wq_gemm(x, w, out=y, residual=res, **kw)
        outs.append(y)
    torch.cuda.synchronize()
    K.workspace(dev).check_status()
    hit = arena.check()
    assert hit is None, str(hit)
    ref = outs[0].float()
    for y in outs[1:]:
        assert float((y.float() - ref).norm() / ref.norm()) < 1e-2
