import pytest
import torch

from cubic_serve_b200.ops import wq_pack
from cubic_serve_b200.quantization import formats as F


def _rel(a, b):
    return ((a - b).norm() / b.norm()).item()


@pytest.mark.parametrize("bits,sym", [(4, True), (4, False), (8, True), (3, True)])
def test_int_roundtrip(bits, sym):
    w = torch.randn(64, 256, generator=torch.Generator().manual_seed(bits)) * 0.02
    p = F.int_quantize(w, bits, 128, sym)
    per = 32 // bits
    assert p["weight_packed"].shape == (64, -(-256 // per)) and p["weight_packed"].dtype == torch.int32
    d = F.int_dense(p, bits, 128, (64, 256))
    assert _rel(d, w) < {3: 0.35, 4: 0.15, 8: 0.01}[bits]
    q, s, z = F.int_decode(p, bits, 128, (64, 256))
    assert int(q.max()) < (1 << bits) and s.shape == (64, 2)
    if bits == 4:
        pw = F.to_packed_weight("int", p, (64, 256), 4, 128)
        assert pw.fmt == wq_pack.FMT_AFFINE4 and _rel(wq_pack.unpack_to_dense(pw), d) < 5e-3


def test_int_word_layout_is_lsb_first():
    codes = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 8, 9]])
    words = F.int_pack(codes, 4)
    assert words.tolist() == [[0x87654321 - 2 ** 32, 9]]
    assert F.int_unpack(words, 4, 9).tolist() == codes.tolist()


def test_awq_order_and_decode():
    vals = torch.arange(16).reshape(1, 16) % 16
    w = F.awq_pack(vals)
    # value i of a group of eight sits at nibble position AWQ_ORDER.index(i)
    assert (int(w[0, 0]) >> (4 * F.AWQ_ORDER.index(3))) & 15 == 3
    assert F.awq_unpack(w).tolist() == vals.tolist()
    g = torch.Generator().manual_seed(0)
    k, n, grp = 128, 64, 64
    q = torch.randint(0, 16, (k, n), generator=g)
    z = torch.randint(0, 16, (k // grp, n), generator=g)
    s = (torch.rand(k // grp, n, generator=g) * 0.01 + 0.001).half()
    payload = {"qweight": F.awq_pack(q), "qzeros": F.awq_pack(z), "scales": s}
    dense = F.awq_dense(payload, grp)
    expect = ((q.float() - z.repeat_interleave(grp, 0).float()) * s.float().repeat_interleave(grp, 0)).t()
    assert torch.allclose(dense, expect)
    pw = F.to_packed_weight("awq", payload, (n, k), 4, grp)
    assert _rel(wq_pack.unpack_to_dense(pw), dense) < 5e-3


def test_fp8_channel_and_block():
    w = torch.randn(200, 300, generator=torch.Generator().manual_seed(1)) * 0.05
    assert _rel(F.fp8_dense(F.fp8_quantize(w)), w) < 0.04
    pb = F.fp8_quantize(w, block=True)
    assert pb["weight_scale_inv"].shape == (2, 3)
    assert _rel(F.fp8_dense(pb), w) < 0.04
    q, s = F.fp8_activation_quantize(torch.zeros(2, 8))
    assert float(s.min()) == pytest.approx(1.0 / (448 * 512))


def test_nvfp4_levels_and_both_global_conventions():
    w = torch.randn(32, 128, generator=torch.Generator().manual_seed(2)) * 0.02
    p = F.nvfp4_quantize(w)
    assert p["weight_packed"].shape == (32, 64) and p["weight_scale"].dtype == torch.float8_e4m3fn
    d = F.nvfp4_dense(p)
    assert _rel(d, w) < 0.15
    modelopt = {"weight": p["weight_packed"], "weight_scale": p["weight_scale"],
                "weight_scale_2": 1.0 / p["weight_global_scale"]}
    assert torch.allclose(F.nvfp4_dense(modelopt), d, rtol=1e-5)
    # nibble semantics: 0x9 -> -0.5, 0x7 -> 6 ; low nibble first
    one = {"weight_packed": torch.tensor([[0x79] * 8], dtype=torch.uint8),
           "weight_scale": torch.ones(1, 1).to(torch.float8_e4m3fn), "weight_global_scale": torch.ones(1)}
    assert F.nvfp4_dense(one)[0, :2].tolist() == [-0.5, 6.0]
    pw = F.to_packed_weight("nvfp4", p, (32, 128))
    assert _rel(wq_pack.unpack_to_dense(pw), d) < 1e-5
    xq, xs = F.nvfp4_activation_quantize(torch.randn(4, 64), 100.0)
    assert xq.shape == (4, 64) and xs.shape == (4, 4)


def test_swiglu_row_order_and_packed_permutation():
    """Interleaved [gate; up] rows: 16 gate rows then the 16 up rows of the same features, for every packed format."""
    inter = 80
    order = wq_pack.swiglu_row_order(inter)
    assert sorted(order.tolist()) == list(range(2 * inter))
    for i in (0, 15, 16, 31, 32, 128, 159):
        feature = (i // 32) * 16 + i % 16
        assert int(order[i]) == feature + (inter if (i % 32) >= 16 else 0)
    with pytest.raises(ValueError):
        wq_pack.swiglu_row_order(40)
    g = torch.Generator().manual_seed(0)
    q = torch.randint(0, 16, (2 * inter, 256), generator=g, dtype=torch.uint8)
    scale = torch.rand(2 * inter, 4, generator=g) * 0.01 + 0.001
    pw = wq_pack.pack_affine4(q, scale, -8 * scale, 64)
    dense = wq_pack.unpack_to_dense(pw)
    pi = wq_pack.swiglu_interleave(pw)
    assert pi.act_interleaved and wq_pack.swiglu_interleave(pi) is pi
    assert torch.equal(wq_pack.unpack_to_dense(pi)[:2 * inter], dense[:2 * inter][order])
    stacked = wq_pack.PackedWeight(pw.fmt, pw.n, pw.k, pw.group_k, torch.stack([pw.codes, pi.codes]),
                                   torch.stack([pw.meta, pi.meta]))
    both = wq_pack.swiglu_interleave(stacked, stacked=True)
    assert torch.equal(both.codes[0], pi.codes) and torch.equal(both.meta[0], pi.meta)
    wb = wq_pack.pack_bf16(torch.randn(2 * inter, 64, generator=g))
    assert torch.equal(wq_pack.swiglu_interleave(wb).codes, wb.codes[order])


def test_quantization_registry_builtins_and_plugins():
    from cubic_serve_b200.models.config import QuantSpec
    from cubic_serve_b200.quantization import registry as R
    assert {"none", "cubic", "int", "awq", "fp8", "fp8_block", "nvfp4", "gguf"} <= set(R.names())
    assert R.get("cubic").native_format == wq_pack.FMT_CUBIC4 and R.get("fp8").native_format is None
    assert R.detect({}).method == "none"
    assert R.detect({"quant_method": "fp8", "weight_block_size": [128, 128]}).method == "fp8_block"
    assert R.detect({"format": "pack-quantized", "config_groups": {"g": {"weights": {"num_bits": 8, "group_size": 64}}}}) == \
        QuantSpec("int", 8, 64)
    assert R.resolve_compute_mode("nvfp4") == "w4a16" and R.resolve_compute_mode("cubic", "auto") == "w4a16"
    with pytest.raises(R.QuantizationRegistryError):
        R.resolve_compute_mode("cubic", "w4a4")
    with pytest.raises(R.QuantizationRegistryError):
        R.get("bitsandbytes")
    with pytest.raises(ValueError):
        R.detect({"quant_method": "bitsandbytes"})
    # an out-of-tree format: sign bits with one scale per row
    ext = R.QuantizationExtension(
        "sign1", ("weight_sign", "weight_scale"), ("w1a16",), None,
        lambda qc: QuantSpec("sign1", 1, 0) if qc.get("quant_method") == "sign1" else None,
        lambda p, shape, q: (p["weight_sign"].float() * 2 - 1) * p["weight_scale"].float()[:, None],
        lambda w, q: {"weight_sign": (w > 0).to(torch.uint8), "weight_scale": w.abs().mean(1)},
        lambda q: {"quant_method": "sign1"})
    R.register(ext)
    try:
        with pytest.raises(R.QuantizationRegistryError):
            R.register(ext)
        spec = R.detect({"quant_method": "sign1"})
        w = torch.randn(8, 16)
        back = R.get(spec.method).dense(R.get("sign1").quantize(w, spec), (8, 16), spec)
        assert back.shape == (8, 16) and torch.equal(back > 0, w > 0)
    finally:
        R._extensions.pop("sign1", None)


def test_out_of_tree_format_through_an_installed_entry_point(tmp_path, monkeypatch):
    """A synthetic external distribution publishes a weight format under the entry-point group; the registry finds
    it when a checkpoint names the format, and a checkpoint written in it is admitted, audited and loaded."""
    import importlib
    import sys
    import textwrap

    import torch

    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models.config import ModelConfig, QuantSpec
    from cubic_serve_b200.quantization import registry

    site = tmp_path / "site"
    (site / "halfscale_fmt").mkdir(parents=True)
    (site / "halfscale_fmt" / "__init__.py").write_text(textwrap.dedent('''
        import torch
        from cubic_serve_b200.quantization.registry import QuantizationExtension

        def _detect(qc):
            if qc.get("quant_method") == "halfscale":
                from cubic_serve_b200.models.config import QuantSpec
                return QuantSpec("halfscale", 8, 0)
            return None

        def extension():
            # int8 codes with one fp32 scale per row, stored as <module>.codes / <module>.row_scale
            return QuantizationExtension(
                "halfscale", ("codes", "row_scale"), ("w8a16",), None, _detect,
                lambda p, shape, q: p["codes"].float() * p["row_scale"].float()[:, None],
                lambda w, q: {"codes": torch.round(w / (w.abs().amax(1, keepdim=True) / 127)).to(torch.int8),
                              "row_scale": (w.abs().amax(1) / 127).float()},
                lambda q: {"quant_method": "halfscale"}, "test format")
    '''))
    info = site / "halfscale_fmt-0.1.dist-info"
    info.mkdir()
    (info / "METADATA").write_text("Metadata-Version: 2.1\nName: halfscale-fmt\nVersion: 0.1\n")
    (info / "entry_points.txt").write_text(f"[{registry.ENTRY_POINT_GROUP}]\nhalfscale = halfscale_fmt:extension\n")
    monkeypatch.syspath_prepend(str(site))
    importlib.invalidate_caches()
    monkeypatch.setattr(registry, "_entry_points_loaded", False)
    try:
        with pytest.raises(registry.QuantizationRegistryError):
            registry.resolve_compute_mode("halfscale", "w4a16")       # found by discovery, offers w8a16 only
        assert registry.get("halfscale").compute_modes == ("w8a16",)
        assert registry.detect({"quant_method": "halfscale"}).method == "halfscale"
        cfg = ModelConfig(name="ext", num_layers=1, hidden_size=128, num_q_heads=2, num_kv_heads=1, head_dim=64,
                          intermediate_size=256, vocab_size=256, quant=QuantSpec("halfscale", 8, 0))
        ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "ck", cfg, seed=0))
        assert ck.cfg.quant.method == "halfscale" and set(ck.payloads["model.layers.0.mlp.down_proj"]) == {"codes", "row_scale"}
        w = C.load_decoder_weights(ck, "cpu")
        from cubic_serve_b200.ops import wq_pack
        assert w.layers[0].down.fmt == wq_pack.FMT_BF16               # no native layout: decoded to bf16 at load
        from cubic_serve_b200.utils.audit_checkpoint import audit_checkpoint
        assert audit_checkpoint(ck.store.path, digests=False)["ok"]
    finally:
        registry._extensions.pop("halfscale", None)
        sys.modules.pop("halfscale_fmt", None)


def test_stacked_nvfp4_experts_keep_their_own_global_scales():
    """Every NVFP4 expert has its own global scale, the grouped GEMM applies one per stack: stacking folds each
    expert's ratio into its block scales, so every expert still decodes to its own values."""
    import torch
    from cubic_serve_b200.models.moe import stack_experts
    from cubic_serve_b200.ops import wq_pack
    from cubic_serve_b200.quantization import nvfp4
    torch.manual_seed(0)
    experts = []
    for e in range(3):
        q = nvfp4.quantize(torch.randn(128, 128) * 0.02 * (1 + e))
        experts.append(wq_pack.pack_nvfp4(q["weight_packed"], q["weight_scale"].float(), 1.0 / float(q["weight_global_scale"])))
    assert len({p.alpha for p in experts}) == 3
    st, _, _ = stack_experts(experts)
    for e, p in enumerate(experts):
        got = wq_pack.unpack_to_dense(wq_pack.PackedWeight(st.fmt, st.n, st.k, st.group_k, st.codes[e], st.meta[e], st.alpha))
        want = wq_pack.unpack_to_dense(p)
        assert float((got - want).norm() / want.norm()) < 4e-3
