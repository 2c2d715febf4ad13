"""The fp8 tensor-core path (``tcgen05.mma.kind::f8f6f4``): e4m3 weights with one scale per output row times e4m3
activations quantized per token, against plain PyTorch fp32 arithmetic on the same codes (the reference checks its FP8
linear the same way, ``quantization/extensions/fp8/tests`` there)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-20))


def _fp8_weight(n, k, dev, seed=0):
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.quantization import formats
    g = torch.Generator(device=dev).manual_seed(seed)
    w = torch.randn(n, k, device=dev, generator=g) * 0.05
    w[:: 7] *= 4.0                                            # rows of different magnitude: the row scales matter
    p = formats.fp8_quantize(w, block=False)
    return wq_pack.pack_fp8(p["weight"], p["weight_scale"]), p


def _oracle(xq, xs, p):
    return (xq.float() @ p["weight"].float().t()) * xs.reshape(-1, 1) * p["weight_scale"].float().reshape(1, -1)


@pytest.mark.parametrize("m,k", [(5, 4096), (256, 1024), (300, 12288), (16, 192)])
def test_activation_quantizer_matches_the_rule(m, k):
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.quantization import formats
    dev = torch.device("cuda")
    x = (torch.randn(m, k, device=dev) * torch.rand(m, 1, device=dev) * 3).to(torch.bfloat16)
    x[0] = 0                                                  # an all-zero row takes the floor scale
    a = K.fp8_quantize(x)
    q_ref, s_ref = formats.fp8_activation_quantize(x)
    assert torch.equal(a.scale, s_ref.reshape(-1))
    got = a.q.view(torch.float8_e4m3fn).float()
    want = q_ref.float()
    # the kernel divides with round-to-nearest like the oracle; codes are equal
    assert torch.equal(got, want)


def test_fused_norm_and_swiglu_quantizers_equal_the_unfused_chain():
    from cubic_serve_b200.ops import kernels as K
    dev = torch.device("cuda")
    x = torch.randn(40, 4096, device=dev).to(torch.bfloat16)
    res = torch.randn(40, 4096, device=dev).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(4096, device=dev)).to(torch.bfloat16)
    r1, r2 = res.clone(), res.clone()
    plain = K.rmsnorm(x, w, 1e-6, residual=r1)
    a = K.fp8_quantize(plain)
    q1, s1 = a.q.clone(), a.scale.clone()
    b = K.rmsnorm_fp8(x, w, 1e-6, residual=r2)
    assert torch.equal(r1, r2) and torch.equal(q1, b.q) and torch.equal(s1, b.scale)
    gu = torch.randn(33, 2 * 1536, device=dev).to(torch.bfloat16)
    a = K.fp8_quantize(K.swiglu(gu))
    q1, s1 = a.q.clone(), a.scale.clone()
    b = K.swiglu_fp8(gu)
    assert torch.equal(q1, b.q) and torch.equal(s1, b.scale)


@pytest.mark.parametrize("m,n,k,splits", [(16, 256, 512, 1), (64, 4096, 4096, None), (256, 6144, 4096, None),
                                          (256, 4096, 12288, 4), (200, 1000, 1088, 1), (48, 512, 2048, 16),
                                          (700, 1024, 4096, 1),
                                          # the persistent kernel: stream-K (more tiles than SMs) and CTA pairs (> 256 rows)
                                          (256, 24576, 4096, None), (64, 24576, 2048, None), (1024, 6144, 4096, None),
                                          (2048, 24576, 1024, None),
                                          (2048, 512, 8192, None)])          # deep K at prefill size: CTA pairs by the dispatcher
def test_fp8_gemm_matches_fp32_on_the_same_codes(m, n, k, splits):
    from cubic_serve_b200.ops import kernels as K
    dev = torch.device("cuda")
    pw, p = _fp8_weight(n, k, dev)
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    a = K.fp8_quantize(x)
    want = _oracle(a.q.view(torch.float8_e4m3fn), a.scale, p)
    res = torch.randn(m, n, device=dev).to(torch.bfloat16)
    y = K.wq_gemm(x, pw, residual=res, splits=splits)
    torch.cuda.synchronize()
    K.workspace(dev).check_status()
    assert _rel(y.float() - res.float(), want) < 6e-3          # bf16 rounding of the output (plus the residual's)
    # against the unquantized product the error is the two quantizations'
    assert _rel(y.float() - res.float(), x.float() @ (p["weight"].float() * p["weight_scale"].float()).t()) < 5e-2


def test_fp8_gemm_with_swiglu_epilogue_and_grouped_experts():
    from cubic_serve_b200.models import moe
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.ops import wq_pack
    dev = torch.device("cuda")
    inter, h, m = 1536, 2048, 96
    pw, p = _fp8_weight(2 * inter, h, dev, seed=3)
    x = torch.randn(m, h, device=dev).to(torch.bfloat16)
    a = K.fp8_quantize(x)
    gu = _oracle(a.q.view(torch.float8_e4m3fn), a.scale, p).to(torch.bfloat16).float()
    want = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    act = K.wq_gemm_act(x, wq_pack.swiglu_interleave(pw))
    torch.cuda.synchronize()
    assert _rel(act, want) < 8e-3
    # grouped: 4 experts, top-2 routing through the MoE layer against the dense oracle
    E, top_k, I = 4, 2, 256
    gus, downs, gu_d, dn_d = [], [], [], []
    for e in range(E):
        a_pw, a_p = _fp8_weight(2 * I, h, dev, seed=10 + e)
        b_pw, b_p = _fp8_weight(h, I, dev, seed=20 + e)
        gus.append(a_pw); downs.append(b_pw)
        gu_d.append(wq_pack.unpack_to_dense(a_pw)); dn_d.append(wq_pack.unpack_to_dense(b_pw))
    gu_s, gcs, gms = moe.stack_experts(gus)
    dn_s, dcs, dms = moe.stack_experts(downs)
    router = (torch.randn(E, h, device=dev) * 0.05).to(torch.bfloat16)
    layer = moe.MoeLayer(wq_pack.pack_bf16(router), gu_s, dn_s, (gcs, gms, dcs, dms), E, top_k, 0, E)
    layer.fuse_activation()
    t = 50
    xt = torch.randn(t, h, device=dev).to(torch.bfloat16)
    y = layer.forward(xt)
    torch.cuda.synchronize()
    K.workspace(dev).check_status()
    want = moe.moe_reference(xt, router, gu_d, dn_d, top_k)
    assert _rel(y, want) < 6e-2                                # the oracle multiplies unquantized activations


def test_fp8_model_step_tracks_the_same_model_with_dequantized_weights():
    """A decoder whose projections are FP8 (W8A8 on the fp8 tensor path, quantizers fused behind the norms) against the
    same weights dequantized to bf16 (W16A16): the logits differ by the activation quantization only."""
    import dataclasses
    import numpy as np
    from cubic_serve_b200.models.config import toy_config
    from cubic_serve_b200.models.decoder import random_decoder_weights
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.parallel.tp_check import _rel_rows, _step_logits
    dev = torch.device("cuda")
    cfg = dataclasses.replace(toy_config(), num_layers=3, hidden_size=512, intermediate_size=1024, num_q_heads=4,
                              num_kv_heads=2, head_dim=128, vocab_size=1024)
    cfg = dataclasses.replace(cfg, quant=dataclasses.replace(cfg.quant, method="fp8", bits=8, group_size=0))
    w8 = random_decoder_weights(cfg, dev, seed=1, std=0.05)
    assert w8.layers[0].qkv.fmt == wq_pack.FMT_FP8 and w8.layers[0].down.fmt == wq_pack.FMT_FP8
    w16 = random_decoder_weights(cfg, dev, seed=1, std=0.05)
    for lw in w16.layers:
        for name in ("qkv", "o", "gate_up", "down"):
            setattr(lw, name, wq_pack.pack_bf16(wq_pack.unpack_to_dense(getattr(lw, name))))
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(6, 40)).tolist()
    (a0, a1), ids8 = _step_logits(cfg, w8, dev, None, prompts, 8, 8)
    (b0, b1), ids16 = _step_logits(cfg, w16, dev, None, prompts, 8, 8)
    # a dozen GEMMs with e4m3 activations (3 mantissa bits, ~2.5 % rms each) lie between the embedding and the logits;
    # the decode step is compared where both models sampled the same first token
    same = torch.tensor([a == b for a, b in zip(ids8[0], ids16[0])], device=dev)
    err = torch.cat([_rel_rows(a0, b0), _rel_rows(a1, b1)[same]])
    assert float(err.max()) < 0.25, err
    assert float(err.median()) < 0.16, err


@pytest.mark.parametrize("m,n,k,splits", [(16, 256, 512, 1), (64, 4096, 4096, None), (256, 1536, 4096, None),
                                          (256, 4096, 1536, 2), (200, 1000, 1088, 1), (700, 1024, 4096, 1),
                                          (48, 512, 2048, 16)])
def test_block_scaled_fp8_gemm_matches_fp32_on_the_same_codes(m, n, k, splits):
    """e4m3 weights with one scale per 128 x 128 block: every stage's product is promoted with its block's scale."""
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.quantization import formats
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(4)
    w = torch.randn(n, k, device=dev, generator=g) * 0.05
    # blocks of very different magnitude, so that a wrong or missing block scale cannot hide
    w *= (torch.rand(-(-n // 128), -(-k // 128), device=dev, generator=g) * 8 + 0.1).repeat_interleave(128, 0)[:n] \
        .repeat_interleave(128, 1)[:, :k]
    p = formats.fp8_quantize(w, block=True)
    pw = wq_pack.pack_fp8_block(p["weight"], p["weight_scale_inv"])
    dense = wq_pack.unpack_to_dense(pw)
    assert _rel(dense, w) < 0.04
    x = torch.randn(m, k, device=dev).to(torch.bfloat16)
    a = K.fp8_quantize(x)
    want = (a.q.view(torch.float8_e4m3fn).float() @ dense.t()) * a.scale.reshape(-1, 1)
    y = K.wq_gemm(x, pw, splits=splits)
    torch.cuda.synchronize()
    K.workspace(dev).check_status()
    assert _rel(y, want) < 5e-3


def test_block_scaled_fp8_experts_and_model_step():
    import dataclasses
    import numpy as np
    from cubic_serve_b200.models import moe
    from cubic_serve_b200.models.config import toy_config
    from cubic_serve_b200.models.decoder import random_decoder_weights
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.parallel.tp_check import _rel_rows, _step_logits
    from cubic_serve_b200.quantization import formats
    dev = torch.device("cuda")
    h, E, top_k, I = 1024, 4, 2, 256

    def blockw(n, k, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        p = formats.fp8_quantize(torch.randn(n, k, device=dev, generator=g) * 0.05, block=True)
        return wq_pack.pack_fp8_block(p["weight"], p["weight_scale_inv"])

    gus, downs = [blockw(2 * I, h, 10 + e) for e in range(E)], [blockw(h, I, 20 + e) for e in range(E)]
    gu_s, gcs, gms = moe.stack_experts(gus)
    dn_s, dcs, dms = moe.stack_experts(downs)
    router = (torch.randn(E, h, device=dev) * 0.05).to(torch.bfloat16)
    layer = moe.MoeLayer(wq_pack.pack_bf16(router), gu_s, dn_s, (gcs, gms, dcs, dms), E, top_k, 0, E)
    layer.fuse_activation()                       # a no-op for block-scaled experts: the activation stays a kernel
    assert not layer.gate_up.act_interleaved
    xt = torch.randn(50, h, device=dev).to(torch.bfloat16)
    y = layer.forward(xt)
    torch.cuda.synchronize()
    K.workspace(dev).check_status()
    want = moe.moe_reference(xt, router, [wq_pack.unpack_to_dense(w) for w in gus],
                             [wq_pack.unpack_to_dense(w) for w in downs], top_k)
    assert _rel(y, want) < 6e-2
    # a dense model whose projections are block-scaled, against the same weights dequantized
    cfg = dataclasses.replace(toy_config(), num_layers=3, hidden_size=512, intermediate_size=1024, num_q_heads=4,
                              num_kv_heads=2, head_dim=128, vocab_size=1024)
    cfg = dataclasses.replace(cfg, quant=dataclasses.replace(cfg.quant, method="fp8_block", bits=8, group_size=128))
    w8 = random_decoder_weights(cfg, dev, seed=1, std=0.05)
    assert w8.layers[0].gate_up.fmt == wq_pack.FMT_FP8_BLOCK
    w16 = random_decoder_weights(cfg, dev, seed=1, std=0.05)
    for lw in w16.layers:
        for name in ("qkv", "o", "gate_up", "down"):
            setattr(lw, name, wq_pack.pack_bf16(wq_pack.unpack_to_dense(getattr(lw, name))))
    prompts = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(6, 40)).tolist()
    (a0, a1), ids8 = _step_logits(cfg, w8, dev, None, prompts, 8, 8)
    (b0, b1), ids16 = _step_logits(cfg, w16, dev, None, prompts, 8, 8)
    assert float(_rel_rows(a0, b0).max()) < 0.25
