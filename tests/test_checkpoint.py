"""Random checkpoints in every on-disk format: closed inventory, decode, TP slicing, GEMM packing."""
import json
from dataclasses import replace

import math

import pytest
import torch

from cubic_serve_b200.models import checkpoint as C
from cubic_serve_b200.models.config import ModelConfig, QuantSpec
from cubic_serve_b200.ops import wq_pack

BASE = ModelConfig(name="tiny", num_layers=2, hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=128,
                   intermediate_size=512, vocab_size=320, qk_norm=True)


@pytest.mark.parametrize("method,bits,group", [("cubic", 4, 128), ("int", 4, 128), ("int", 8, 128), ("awq", 4, 128),
                                               ("fp8", 8, 0), ("fp8_block", 8, 128), ("nvfp4", 4, 16), ("none", 16, 0)])
def test_write_admit_load(tmp_path, method, bits, group):
    cfg = replace(BASE, quant=QuantSpec(method, bits, group))
    path = C.write_random_checkpoint(tmp_path / method, cfg, seed=1)
    ck = C.admit_checkpoint(path)
    assert ck.cfg.quant.method == method and ck.cfg.num_layers == 2 and ck.cfg.qk_norm
    info = C.inspect_checkpoint(path)
    assert info["logical_linears"] == 2 * 7
    # dense decode of one module equals the packed GEMM operand built from it
    mod = "model.layers.1.mlp.down_proj"
    dense = C._dense_of(method, ck.payload(mod), (256, 512), cfg.quant)
    assert dense.shape == (256, 512) and float(dense.abs().mean()) > 1e-4
    w = C.load_decoder_weights(ck, "cpu")
    got = wq_pack.unpack_to_dense(w.layers[1].down)
    assert ((got - dense).norm() / dense.norm()).item() < 6e-3
    q = C._dense_of(method, ck.payload("model.layers.0.self_attn.q_proj"), (512, 256), cfg.quant)
    k = C._dense_of(method, ck.payload("model.layers.0.self_attn.k_proj"), (256, 256), cfg.quant)
    v = C._dense_of(method, ck.payload("model.layers.0.self_attn.v_proj"), (256, 256), cfg.quant)
    qkv = wq_pack.unpack_to_dense(w.layers[0].qkv)
    assert ((qkv - torch.cat([q, k, v])).norm() / qkv.norm()).item() < 6e-3
    # tensor-parallel rank 1 of 2: whole heads of q/k/v, column shard of o/down
    w1 = C.load_decoder_weights(ck, "cpu", tp_rank=1, tp_size=2)
    qkv1 = wq_pack.unpack_to_dense(w1.layers[0].qkv)
    assert ((qkv1 - torch.cat([q[256:], k[128:], v[128:]])).norm() / qkv1.norm()).item() < 6e-3
    d1 = wq_pack.unpack_to_dense(w1.layers[1].down)
    assert ((d1 - dense[:, 256:]).norm() / d1.norm()).item() < 6e-3
    assert w1.vocab_start == 160 and w1.lm_head.n == 160


def test_closed_inventory_rejects_stray_and_missing(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = replace(BASE, quant=QuantSpec("cubic", 4, 128))
    path = C.write_random_checkpoint(tmp_path / "c", cfg)
    t = load_file(str(path / "model.safetensors"))
    t["model.layers.0.stray"] = torch.zeros(1)
    save_file(t, str(path / "model.safetensors"))
    with pytest.raises(C.CheckpointError, match="no logical weight owns"):
        C.admit_checkpoint(path)
    del t["model.layers.0.stray"], t["model.norm.weight"]
    save_file(t, str(path / "model.safetensors"))
    with pytest.raises(C.CheckpointError, match="missing tensor"):
        C.admit_checkpoint(path)


def test_quantization_config_parsing_variants():
    from cubic_serve_b200.models.config import quant_spec_from_hf
    assert quant_spec_from_hf({}).method == "none"
    assert quant_spec_from_hf({"quant_method": "awq", "bits": 4, "group_size": 64}).group_size == 64
    assert quant_spec_from_hf({"quant_method": "modelopt", "quant_algo": "NVFP4"}).method == "nvfp4"
    assert quant_spec_from_hf({"quant_method": "fp8", "weight_block_size": [128, 128]}).method == "fp8_block"
    c = quant_spec_from_hf({"format": "cubic-pack-quantized", "config_groups": {"g": {"weights": {"num_bits": 4, "group_size": [1, 64]}}}})
    assert (c.method, c.bits, c.group_size) == ("cubic", 4, 64)
    with pytest.raises(ValueError):
        quant_spec_from_hf({"quant_method": "bitsandbytes"})


@pytest.mark.parametrize("method,bits,group", [("cubic", 4, 128), ("awq", 4, 128), ("fp8_block", 8, 128), ("none", 16, 0)])
def test_hybrid_checkpoint_row_mapping(tmp_path, method, bits, group):
    """Gated DeltaNet layers: the checkpoint's per-key-head grouping of in_proj_qkvz / in_proj_ba rows and the
    [q_h | gate_h] rows of the gated query projection map to the kernels' section layout, also per TP rank."""
    cfg = ModelConfig(name="hyb", family="qwen3_5", num_layers=4, hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=512, vocab_size=512, rotary_dim=64, qk_norm=True, zero_centered_norm=True,
                      gdn_interval=4, gdn_k_heads=2, gdn_v_heads=4, attn_output_gate=True, quant=QuantSpec(method, bits, group))
    path = C.write_random_checkpoint(tmp_path / method, cfg, seed=2)
    ck = C.admit_checkpoint(path)
    assert ck.cfg.is_hybrid and ck.cfg.gdn_k_heads == 2 and ck.cfg.attn_output_gate and ck.cfg.rotary_dim == 64
    H, r = 256, 2
    qkvz = C._dense_of(method, ck.payload("model.layers.0.linear_attn.in_proj_qkvz"), (2 * 2 * 128 + 2 * 4 * 128, H), cfg.quant)
    g = qkvz.view(2, (2 + 2 * r) * 128, H)                     # [key head, q | k | v x r | z x r, H]
    sect = lambda lo, n, heads: torch.cat([g[h, lo:lo + n] for h in heads])
    ba = ck.store.get("model.layers.0.linear_attn.in_proj_ba.weight").float().view(2, 2, r, H)
    conv = ck.store.get("model.layers.0.linear_attn.conv1d.weight").float().reshape(-1, 4)
    for tp, rank in ((1, 0), (2, 1)):
        w = C.load_decoder_weights(ck, "cpu", tp_rank=rank, tp_size=tp)
        heads = range(rank * 2 // tp, (rank + 1) * 2 // tp)
        gd = w.layers[0].gdn
        assert (gd.hk, gd.hv) == (2 // tp, 4 // tp) and w.layers[0].qkv is None and w.layers[3].gdn is None
        want = torch.cat([sect(0, 128, heads), sect(128, 128, heads), sect(256, r * 128, heads), sect(256 + r * 128, r * 128, heads)])
        got = wq_pack.unpack_to_dense(gd.in_proj)[:want.shape[0]]
        assert ((got - want).norm() / want.norm()).item() < 6e-3
        want_ba = torch.cat([torch.cat([ba[h, 0] for h in heads]), torch.cat([ba[h, 1] for h in heads])])
        assert torch.allclose(wq_pack.unpack_to_dense(gd.in_ba).float(), want_ba.to(torch.bfloat16).float())
        qk = 2 * 128
        idx = torch.cat([torch.arange(h * 128, (h + 1) * 128) for h in heads])
        vidx = torch.cat([torch.arange(h * r * 128, (h + 1) * r * 128) for h in heads])
        assert torch.equal(gd.conv_w, torch.cat([conv[idx], conv[qk + idx], conv[2 * qk + vidx]]))
        assert gd.a_log.shape == (4 // tp,) and gd.norm_w.shape == (128,)
        # the gated attention layer: q rows of every head, then k, v; the gate rows in their own matrix
        qp = C._dense_of(method, ck.payload("model.layers.3.self_attn.q_proj"), (2 * 4 * 128, H), cfg.quant).view(4, 2, 128, H)
        hq = range(rank * 4 // tp, (rank + 1) * 4 // tp)
        lw = w.layers[3]
        got_q = wq_pack.unpack_to_dense(lw.qkv)[:len(hq) * 128]
        assert ((got_q - torch.cat([qp[h, 0] for h in hq])).norm() / got_q.norm()).item() < 6e-3
        got_g = wq_pack.unpack_to_dense(lw.attn_gate)[:len(hq) * 128]
        assert ((got_g - torch.cat([qp[h, 1] for h in hq])).norm() / got_g.norm()).item() < 6e-3


@pytest.mark.parametrize("method,bits,group", [("cubic", 4, 128), ("int", 4, 128), ("none", 16, 0)])
def test_moe_checkpoint_experts_and_router(tmp_path, method, bits, group):
    """Experts of a written MoE checkpoint arrive whole on their owning rank, [gate; up] stacked, values equal to
    the format's own decode of the payload; the router is replicated."""
    import dataclasses
    from cubic_serve_b200.models.checkpoint import _dense_of, admit_checkpoint, load_decoder_weights, logical_inventory
    from cubic_serve_b200.ops import wq_pack
    cfg = dataclasses.replace(BASE, name="tiny-moe", family="gqa_moe", num_experts=4, experts_per_token=2,
                              moe_intermediate_size=128, quant=QuantSpec(method, bits, group))
    path = C.write_random_checkpoint(tmp_path / "moe", cfg, seed=2)
    ck = admit_checkpoint(path)
    assert ck.cfg.is_moe and ck.cfg.num_experts == 4
    shapes, _ = logical_inventory(ck.cfg)

    def dense(module):
        return _dense_of(method, ck.payload(module), shapes[module], ck.cfg.quant)

    def expert(stacked, j):
        return wq_pack.PackedWeight(stacked.fmt, stacked.n, stacked.k, stacked.group_k, stacked.codes[j],
                                    None if stacked.meta is None else stacked.meta[j], stacked.alpha)

    def rel(a, b):
        return ((a - b).norm() / b.norm()).item()

    full = load_decoder_weights(ck, "cpu")
    moe = full.layers[1].moe
    assert full.layers[1].gate_up is None and (moe.expert_lo, moe.expert_count, moe.num_experts, moe.top_k) == (0, 4, 4, 2)
    assert torch.equal(moe.router.codes.float(), ck.store.get("model.layers.1.mlp.gate.weight").float())
    r1 = load_decoder_weights(ck, "cpu", tp_rank=1, tp_size=2).layers[1].moe
    assert (r1.expert_lo, r1.expert_count) == (2, 2) and r1.gate_up.codes.shape[0] == 2
    for j, e in ((0, 2), (1, 3)):
        ep = f"model.layers.1.mlp.experts.{e}"
        want_gu = torch.cat([dense(f"{ep}.gate_proj"), dense(f"{ep}.up_proj")])
        assert rel(wq_pack.unpack_to_dense(expert(r1.gate_up, j))[:256], want_gu) < 6e-3
        assert rel(wq_pack.unpack_to_dense(expert(r1.down, j))[:256], dense(f"{ep}.down_proj")) < 6e-3
        assert rel(wq_pack.unpack_to_dense(expert(moe.gate_up, e))[:256], want_gu) < 6e-3
    gcs, gms, dcs, dms = r1.strides
    assert gcs == r1.gate_up.codes[0].numel() * r1.gate_up.codes.element_size()
    with pytest.raises(C.CheckpointError):
        load_decoder_weights(ck, "cpu", tp_rank=0, tp_size=3)


def test_mtp_head_from_checkpoint(tmp_path):
    import dataclasses
    from cubic_serve_b200.models.checkpoint import _dense_of, admit_checkpoint, load_mtp_weights, logical_inventory
    cfg = dataclasses.replace(BASE, name="tiny-mtp", mtp_layers=1, quant=QuantSpec("cubic", 4, 128))
    path = C.write_random_checkpoint(tmp_path / "mtp", cfg, seed=5)
    assert json.loads((path / "config.json").read_text())["mtp_num_hidden_layers"] == 1
    ck = admit_checkpoint(path)
    assert ck.cfg.mtp_layers == 1 and "mtp.fc" in ck.payloads and "mtp.norm.weight" in ck.plain
    shapes, _ = logical_inventory(ck.cfg)
    dense = lambda m: _dense_of("cubic", ck.payload(m), shapes[m], ck.cfg.quant)  # noqa: E731
    w = load_mtp_weights(ck, "cpu")
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()  # noqa: E731
    assert (w.fc.n, w.fc.k) == (256, 512) and rel(wq_pack.unpack_to_dense(w.fc)[:256], dense("mtp.fc")) < 6e-3
    mp = "mtp.layers.0"
    qkv = torch.cat([dense(f"{mp}.self_attn.q_proj"), dense(f"{mp}.self_attn.k_proj"), dense(f"{mp}.self_attn.v_proj")])
    assert rel(wq_pack.unpack_to_dense(w.layer.qkv)[:qkv.shape[0]], qkv) < 6e-3
    assert w.layer.q_norm.shape == (128,) and w.enorm.shape == (256,) and w.norm.dtype == torch.bfloat16
    # the same tensors under a config that does not announce the head are foreign tensors: closed inventory
    hf = json.loads((path / "config.json").read_text())
    del hf["mtp_num_hidden_layers"]
    (path / "config.json").write_text(json.dumps(hf))
    with pytest.raises(C.CheckpointError, match="no logical weight owns"):
        admit_checkpoint(path)
    plain = admit_checkpoint(C.write_random_checkpoint(tmp_path / "plain", BASE, seed=5))
    with pytest.raises(C.CheckpointError, match="no MTP head"):
        load_mtp_weights(plain, "cpu")


def test_asymmetric_int_checkpoint_slices_zero_points_with_the_rows(tmp_path):
    """Zero points are packed along N.  A tensor-parallel rank > 0 (or the per-head row gathering of the hybrid
    family) decodes a row slice [lo, hi) with lo > 0 and must find the zero points of THOSE rows."""
    from safetensors.torch import load_file, save_file
    from cubic_serve_b200.quantization import formats
    cfg = replace(BASE, quant=QuantSpec("int", 4, 128))
    path = C.write_random_checkpoint(tmp_path / "int_asym", cfg, seed=3)
    t = load_file(str(path / "model.safetensors"))
    g = torch.Generator().manual_seed(5)
    dense = {}
    for name in [n for n in t if n.endswith(".weight_packed")]:
        module = name[:-len(".weight_packed")]
        n, k = (int(v) for v in t[f"{module}.weight_shape"])
        w = torch.randn(n, k, generator=g) * 0.02 + 0.01 * torch.randn(n, 1, generator=g)     # rows with an offset
        for suffix, v in formats.int_quantize(w, 4, 128, symmetric=False).items():
            t[f"{module}.{suffix}"] = v.contiguous()
        dense[module] = formats.int_dense({s: t[f"{module}.{s}"] for s in ("weight_packed", "weight_scale", "weight_zero_point")},
                                          4, 128, (n, k))
    save_file(t, str(path / "model.safetensors"))
    ck = C.admit_checkpoint(path)
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    # _slice_rows of the upper half decodes to the upper half of the full decode
    mod = "model.layers.0.self_attn.q_proj"
    sl = C._slice_rows(ck.payload(mod), "int", 256, 512, 512, 4)
    assert torch.equal(formats.int_dense(sl, 4, 128, (256, 256)), dense[mod][256:])
    w1 = C.load_decoder_weights(ck, "cpu", tp_rank=1, tp_size=2)
    q, k, v = (dense[f"model.layers.0.self_attn.{p}_proj"] for p in "qkv")
    assert rel(wq_pack.unpack_to_dense(w1.layers[0].qkv), torch.cat([q[256:], k[128:], v[128:]])) < 6e-3
    gu = wq_pack.unpack_to_dense(w1.layers[1].gate_up)
    gate, up = dense["model.layers.1.mlp.gate_proj"][256:], dense["model.layers.1.mlp.up_proj"][256:]
    assert rel(gu.sort(0).values, torch.cat([gate, up]).sort(0).values) < 6e-3        # rows are interleaved at load
    assert rel(wq_pack.unpack_to_dense(w1.layers[1].down), dense["model.layers.1.mlp.down_proj"][:, 256:]) < 6e-3
    # an act-order checkpoint (non-trivial g_idx) is refused at admission, a trivial g_idx is admitted
    t[f"{mod}.weight_g_idx"] = (torch.arange(256) // 128).to(torch.int32)
    save_file(t, str(path / "model.safetensors"))
    C.admit_checkpoint(path)
    t[f"{mod}.weight_g_idx"] = (torch.arange(256).flip(0) // 128).to(torch.int32)
    save_file(t, str(path / "model.safetensors"))
    with pytest.raises(C.CheckpointError, match="act-order"):
        C.admit_checkpoint(path)


def test_random_weights_of_any_partition_are_slices_of_one_model():
    """``random_decoder_weights`` draws rank-independent full matrices: the shards of two ranks put together give the
    one-GPU model's matrices bit for bit (dense and MoE), so outputs of different partitions are comparable."""
    from cubic_serve_b200.models.decoder import random_decoder_weights
    cfg = replace(BASE, quant=QuantSpec("cubic", 4, 128))
    one = random_decoder_weights(cfg, "cpu", seed=3)
    two = [random_decoder_weights(cfg, "cpu", seed=3, tp_rank=r, tp_size=2) for r in range(2)]
    d = wq_pack.unpack_to_dense
    D = cfg.head_dim
    for li in range(cfg.num_layers):
        full, parts = one.layers[li], [t.layers[li] for t in two]
        qkv = d(full.qkv)
        hq, hkv = cfg.num_q_heads * D, cfg.num_kv_heads * D
        want = [torch.cat([qkv[r * hq // 2:(r + 1) * hq // 2], qkv[hq + r * hkv // 2:hq + (r + 1) * hkv // 2],
                           qkv[hq + hkv + r * hkv // 2:hq + hkv + (r + 1) * hkv // 2]]) for r in range(2)]
        for r in range(2):
            assert torch.equal(d(parts[r].qkv)[:want[r].shape[0]], want[r])
        assert torch.equal(torch.cat([d(p.o)[:cfg.hidden_size] for p in parts], 1), d(full.o)[:cfg.hidden_size])
        assert torch.equal(torch.cat([d(p.down)[:cfg.hidden_size] for p in parts], 1), d(full.down)[:cfg.hidden_size])
        gu, I = d(full.gate_up), cfg.intermediate_size
        for r in range(2):
            want_gu = torch.cat([gu[r * I // 2:(r + 1) * I // 2], gu[I + r * I // 2:I + (r + 1) * I // 2]])
            assert torch.equal(d(parts[r].gate_up)[:I], want_gu)
    assert torch.equal(torch.cat([d(t.lm_head)[:cfg.vocab_size // 2] for t in two]), d(one.lm_head)[:cfg.vocab_size])
    # NVFP4 has one scale per tensor: shards are quantized with the whole matrix's largest magnitude
    nv = replace(BASE, quant=QuantSpec("nvfp4", 4, 16))
    n1 = random_decoder_weights(nv, "cpu", seed=3)
    n2 = [random_decoder_weights(nv, "cpu", seed=3, tp_rank=r, tp_size=2) for r in range(2)]
    assert torch.equal(torch.cat([d(t.layers[0].down)[:nv.hidden_size] for t in n2], 1), d(n1.layers[0].down)[:nv.hidden_size])
    # fewer key/value heads than ranks: neighbouring ranks hold a copy of the same head, every rank its own query heads
    few = replace(BASE, num_kv_heads=2, quant=QuantSpec("cubic", 4, 128))
    k1 = random_decoder_weights(few, "cpu", seed=3)
    k4 = [random_decoder_weights(few, "cpu", seed=3, tp_rank=r, tp_size=4) for r in range(4)]
    fq, hq4 = d(k1.layers[0].qkv), few.num_q_heads // 4 * D
    kb, vb = few.num_q_heads * D, (few.num_q_heads + 2) * D
    for r in range(4):
        want = torch.cat([fq[r * hq4:(r + 1) * hq4], fq[kb + (r // 2) * D:kb + (r // 2 + 1) * D],
                          fq[vb + (r // 2) * D:vb + (r // 2 + 1) * D]])
        assert torch.equal(d(k4[r].layers[0].qkv)[:want.shape[0]], want)
    # FP8 has one scale per output row: column shards are quantized with the whole row's largest magnitude
    f8 = replace(BASE, quant=QuantSpec("fp8", 8, 0))
    f1 = random_decoder_weights(f8, "cpu", seed=3)
    f2 = [random_decoder_weights(f8, "cpu", seed=3, tp_rank=r, tp_size=2) for r in range(2)]
    assert f1.layers[0].down.fmt == wq_pack.FMT_FP8
    assert torch.equal(torch.cat([d(t.layers[0].down) for t in f2], 1), d(f1.layers[0].down))
    assert torch.equal(torch.cat([d(t.layers[1].o) for t in f2], 1), d(f1.layers[1].o))
    moe = replace(BASE, family="gqa_moe", num_experts=4, experts_per_token=2, moe_intermediate_size=128,
                  quant=QuantSpec("cubic", 4, 128))
    m1 = random_decoder_weights(moe, "cpu", seed=1)
    m2 = [random_decoder_weights(moe, "cpu", seed=1, tp_rank=r, tp_size=2) for r in range(2)]
    assert torch.equal(torch.cat([t.layers[1].moe.gate_up.codes for t in m2]), m1.layers[1].moe.gate_up.codes)
    assert torch.equal(m2[0].layers[0].moe.router.codes, m1.layers[0].moe.router.codes)
    assert not torch.equal(m1.layers[0].moe.router.codes, m1.layers[1].moe.router.codes)


@pytest.mark.parametrize("method,fmt", [("fp8", "FMT_FP8"), ("fp8_block", "FMT_FP8_BLOCK")])
def test_fp8_checkpoints_stay_e4m3_at_load(tmp_path, method, fmt):
    """FP8 checkpoints (one scale per row, or per 128 x 128 block) are not expanded: the loader hands the e4m3 bytes and
    their scales to the fp8 GEMM, whole and as tensor-parallel shards, and they decode to the checkpoint's values."""
    from safetensors.torch import load_file
    from cubic_serve_b200.quantization import formats
    cfg = replace(BASE, hidden_size=256, intermediate_size=512, num_q_heads=4, num_kv_heads=2, head_dim=128,
                  quant=QuantSpec(method, 8, 128 if method == "fp8_block" else 0))
    path = C.write_random_checkpoint(tmp_path / method, cfg, seed=5)
    t = load_file(str(path / "model.safetensors"))
    ck = C.admit_checkpoint(path)
    assert ck.cfg.quant.method == method
    want_fmt = getattr(wq_pack, fmt)

    def dense(module):
        keys = ("weight", "weight_scale", "weight_scale_inv")
        return formats.fp8_dense({k: t[f"{module}.{k}"] for k in keys if f"{module}.{k}" in t})

    w1 = C.load_decoder_weights(ck, "cpu")
    lw = w1.layers[0]
    assert lw.qkv.fmt == lw.o.fmt == lw.gate_up.fmt == lw.down.fmt == want_fmt
    assert lw.qkv.codes.dtype == torch.uint8 and lw.qkv.meta.dtype == torch.float32
    q, k, v = (dense(f"model.layers.0.self_attn.{p}_proj") for p in "qkv")
    assert torch.equal(wq_pack.unpack_to_dense(lw.qkv), torch.cat([q, k, v]))
    assert torch.equal(wq_pack.unpack_to_dense(lw.down), dense("model.layers.0.mlp.down_proj"))
    # two tensor-parallel ranks: row shards of q / k / v / gate / up, column shards of o / down
    two = [C.load_decoder_weights(ck, "cpu", tp_rank=r, tp_size=2) for r in range(2)]
    assert all(x.layers[0].down.fmt == want_fmt and x.layers[0].qkv.fmt == want_fmt for x in two)
    full_down = dense("model.layers.0.mlp.down_proj")
    assert torch.equal(torch.cat([wq_pack.unpack_to_dense(x.layers[0].down) for x in two], 1), full_down)
    full_o = dense("model.layers.0.self_attn.o_proj")
    assert torch.equal(torch.cat([wq_pack.unpack_to_dense(x.layers[0].o) for x in two], 1), full_o)
    hq, hkv = 2 * 128, 128
    for r, x in enumerate(two):
        want = torch.cat([q[r * hq:(r + 1) * hq], k[r * hkv:(r + 1) * hkv], v[r * hkv:(r + 1) * hkv]])
        assert torch.equal(wq_pack.unpack_to_dense(x.layers[0].qkv), want)


def test_fp8_block_experts_load_as_stacked_e4m3(tmp_path):
    """A mixture-of-experts checkpoint with 128 x 128 block-scaled FP8 experts: every expert keeps its e4m3 bytes and
    block scales in the stack the grouped GEMM reads."""
    from safetensors.torch import load_file
    from cubic_serve_b200.quantization import formats
    cfg = replace(BASE, family="gqa_moe", hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=128, num_experts=4,
                  experts_per_token=2, moe_intermediate_size=128, intermediate_size=0, quant=QuantSpec("fp8_block", 8, 128))
    path = C.write_random_checkpoint(tmp_path / "moe_fp8", cfg, seed=2)
    t = load_file(str(path / "model.safetensors"))
    w = C.load_decoder_weights(C.admit_checkpoint(path), "cpu")
    layer = w.layers[0].moe
    assert layer.gate_up.fmt == layer.down.fmt == wq_pack.FMT_FP8_BLOCK
    assert tuple(layer.gate_up.codes.shape) == (4, 256, 256) and tuple(layer.gate_up.meta.shape) == (4, 2, 2)
    for e in (0, 3):
        one = wq_pack.PackedWeight(layer.down.fmt, layer.down.n, layer.down.k, 128, layer.down.codes[e], layer.down.meta[e])
        mod = f"model.layers.0.mlp.experts.{e}.down_proj"
        want = formats.fp8_dense({k: t[f"{mod}.{k}"] for k in ("weight", "weight_scale_inv") if f"{mod}.{k}" in t})
        assert torch.equal(wq_pack.unpack_to_dense(one), want)


def test_projection_biases_follow_the_rank_heads(tmp_path):
    """Qwen2-style q / k / v biases: the loader hands every rank the biases of its own heads in the order of the fused
    projection's rows; random weights of a partition are slices of the one-GPU model's."""
    from cubic_serve_b200.models.decoder import random_decoder_weights
    cfg = replace(BASE, qk_norm=False, qkv_bias=True, name="Qwen2ForCausalLM", quant=QuantSpec("int", 4, 128))
    ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "b", cfg, seed=3))
    assert ck.cfg.qkv_bias and not ck.cfg.qk_norm
    bq, bk, bv = (ck.store.get(f"model.layers.1.self_attn.{n}_proj.bias").float() for n in "qkv")
    whole = C.load_decoder_weights(ck, "cpu").layers[1].qkv_bias
    assert torch.equal(whole.float(), torch.cat([bq, bk, bv]))
    r1 = C.load_decoder_weights(ck, "cpu", tp_rank=1, tp_size=2).layers[1].qkv_bias
    hq, hkv = cfg.q_size // 2, cfg.kv_size // 2
    assert torch.equal(r1.float(), torch.cat([bq[hq:], bk[hkv:], bv[hkv:]]))
    one = random_decoder_weights(cfg, "cpu", seed=5).layers[0].qkv_bias
    half = random_decoder_weights(cfg, "cpu", seed=5, tp_rank=1, tp_size=2).layers[0].qkv_bias
    assert torch.equal(half, torch.cat([one[hq:cfg.q_size], one[cfg.q_size + hkv:cfg.q_size + cfg.kv_size],
                                        one[cfg.q_size + cfg.kv_size + hkv:]]))
    assert random_decoder_weights(replace(cfg, qkv_bias=False), "cpu", seed=5).layers[0].qkv_bias is None


def test_shared_expert_is_loaded_per_rank(tmp_path):
    """A sigmoid-gated shared expert beside the routed ones: admitted by the closed inventory, loaded as this rank's share
    of its intermediate features; wide heads stay with the eager execution mode."""
    cfg = ModelConfig(name="shared", family="gqa_moe", num_layers=1, hidden_size=256, num_q_heads=2, num_kv_heads=1,
                      head_dim=128, intermediate_size=0, vocab_size=512, qk_norm=True, num_experts=4, experts_per_token=2,
                      moe_intermediate_size=128, shared_intermediate_size=256, quant=QuantSpec("cubic", 4, 128))
    ck = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "s", cfg, seed=3, std=0.05))
    sp = "model.layers.0.mlp.shared_expert"
    gate = C._dense_of("cubic", ck.payload(f"{sp}.gate_proj"), (256, 256), cfg.quant)
    up = C._dense_of("cubic", ck.payload(f"{sp}.up_proj"), (256, 256), cfg.quant)
    down = C._dense_of("cubic", ck.payload(f"{sp}.down_proj"), (256, 256), cfg.quant)
    for tp, rank in ((1, 0), (2, 1)):
        moe = C.load_decoder_weights(ck, "cpu", tp_rank=rank, tp_size=tp).layers[0].moe
        lo, hi = rank * 256 // tp, (rank + 1) * 256 // tp
        gu = wq_pack.unpack_to_dense(moe.shared_gate_up)[:2 * (hi - lo)]
        assert ((gu - torch.cat([gate[lo:hi], up[lo:hi]])).norm() / gu.norm()).item() < 6e-3
        dn = wq_pack.unpack_to_dense(moe.shared_down)[:256]
        assert ((dn - down[:, lo:hi]).norm() / dn.norm()).item() < 6e-3
        g = wq_pack.unpack_to_dense(moe.shared_gate)
        want = ck.store.get("model.layers.0.mlp.shared_expert_gate.weight").float()
        assert torch.equal(g[:1].float(), want.to(torch.bfloat16).float()) and float(g[1:].abs().max()) == 0
    wide = replace(cfg, head_dim=256, name="wide")
    ck2 = C.admit_checkpoint(C.write_random_checkpoint(tmp_path / "w", wide, seed=3))
    with pytest.raises(C.CheckpointError, match="eager execution mode"):
        C.load_decoder_weights(ck2, "cpu")


@pytest.mark.parametrize("method,bits,group", [("cubic", 4, 128), ("int", 8, 128), ("fp8", 8, 0)])
def test_quantized_head_and_embedding_are_decoded_at_load(tmp_path, method, bits, group):
    """Checkpoints that quantize ``lm_head`` / ``embed_tokens`` like their projections: the payload is owned by the
    inventory and decoded once at load."""
    from safetensors.torch import load_file, save_file

    from cubic_serve_b200.models.reference import dense_weights_from_checkpoint
    cfg = replace(BASE, quant=QuantSpec(method, bits, group))
    path = C.write_random_checkpoint(tmp_path / method, cfg, seed=6, std=0.05)
    t = {k: v.clone() for k, v in load_file(str(path / "model.safetensors")).items()}      # no view of the file: it is rewritten
    originals = {}
    for name in ("lm_head.weight", "model.embed_tokens.weight"):
        dense = t.pop(name).float()
        originals[name] = dense
        for suffix, v in C.quantize_payload(dense, cfg.quant).items():
            t[f"{name[:-len('.weight')]}.{suffix}"] = v.contiguous()
    save_file(t, str(path / "model.safetensors"))
    ck = C.admit_checkpoint(path)
    assert "lm_head" in ck.payloads and "model.embed_tokens" in ck.payloads
    for name, dense in originals.items():
        got = ck.plain_tensor(name).float()
        assert got.shape == dense.shape and ((got - dense).norm() / dense.norm()).item() < (0.12 if bits == 4 else 0.04)
    w = C.load_decoder_weights(ck, "cpu", tp_rank=1, tp_size=2)
    v = cfg.vocab_size // 2
    assert w.lm_head.n == v and w.embed.shape[0] == v
    head = wq_pack.unpack_to_dense(w.lm_head)[:v].float()
    assert ((head - ck.plain_tensor("lm_head.weight").float()[v:].to(torch.bfloat16).float()).abs().max()).item() < 1e-6
    dw = dense_weights_from_checkpoint(ck)
    assert dw.lm_head.shape == (cfg.vocab_size, cfg.hidden_size)
    # a checkpoint that has neither form is still refused
    for k in [k for k in t if k.startswith("lm_head.")]:
        del t[k]
    other = tmp_path / (method + "-nohead")
    other.mkdir()
    (other / "config.json").write_text((path / "config.json").read_text())
    save_file(t, str(other / "model.safetensors"))
    with pytest.raises(C.CheckpointError, match="missing tensor lm_head.weight"):
        C.admit_checkpoint(other)


def test_multimodal_config_keys_at_the_root(tmp_path):
    """``tie_word_embeddings`` of a multimodal ``config.json`` sits beside ``text_config``, rotary parameters inside it."""
    import json
    doc = {"architectures": ["Qwen3VLForConditionalGeneration"], "tie_word_embeddings": True,
           "text_config": {"hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
                           "head_dim": 64, "intermediate_size": 512, "vocab_size": 320,
                           "rope_parameters": {"rope_theta": 5e6, "mrope_section": [16, 8, 8]}}}
    p = tmp_path / "config.json"
    p.write_text(json.dumps(doc))
    cfg = ModelConfig.from_hf_config(p)
    assert cfg.tie_embeddings and cfg.rope_theta == 5e6 and cfg.mrope_section == (16, 8, 8) and cfg.qk_norm


def test_rotary_scaling_forms(tmp_path):
    import json

    from cubic_serve_b200.ops import eager
    base = {"architectures": ["LlamaForCausalLM"], "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
            "num_key_value_heads": 2, "intermediate_size": 512, "vocab_size": 320, "rope_theta": 500000.0}
    p = tmp_path / "config.json"
    p.write_text(json.dumps({**base, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}}))
    cfg = ModelConfig.from_hf_config(p)
    assert cfg.rope_scaling == ("llama3", 8.0, 1.0, 4.0, 8192)
    plain = eager.rope_inv_freq(64, 500000.0)
    scaled = eager.rope_inv_freq(64, 500000.0, scaling=cfg.rope_scaling)
    assert torch.equal(scaled[:8], plain[:8]) and torch.allclose(scaled[-1], plain[-1] / 8)      # short waves kept, long ones / 8
    assert bool((scaled <= plain).all()) and bool((scaled >= plain / 8 - 1e-12).all())
    assert torch.allclose(eager.rope_inv_freq(64, 1e4, scaling=("linear", 4.0)), eager.rope_inv_freq(64, 1e4) / 4)
    p.write_text(json.dumps({**base, "max_position_embeddings": 131072,
                             "rope_scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}}))
    cfg = ModelConfig.from_hf_config(p)
    assert cfg.rope_scaling[:5] == ("yarn", 4.0, 32768, 32.0, 1.0) and abs(cfg.rope_scaling[5] - (0.1 * math.log(4.0) + 1)) < 1e-12
    assert abs(cfg.attention_scale - cfg.rope_scaling[5] ** 2 / 8.0) < 1e-12                     # head width 64
    yarn = eager.rope_inv_freq(64, 500000.0, scaling=cfg.rope_scaling)
    assert torch.equal(yarn[:4], plain[:4]) and torch.allclose(yarn[-1], plain[-1] / 4)          # fast slots kept, slow ones / 4
    assert bool((yarn[1:] <= yarn[:-1]).all())
    for bad in ({"mscale": 1.0, "mscale_all_dim": 0.7}, {"truncate": False}):
        p.write_text(json.dumps({**base, "rope_scaling": {"rope_type": "yarn", "factor": 4.0, **bad}}))
        with pytest.raises(ValueError, match="yarn"):
            ModelConfig.from_hf_config(p)
    p.write_text(json.dumps({**base, "partial_rotary_factor": 0.5, "rope_scaling": {"rope_type": "yarn", "factor": 4.0}}))
    with pytest.raises(ValueError, match="partly rotated"):
        ModelConfig.from_hf_config(p)
    p.write_text(json.dumps({**base, "rope_scaling": {"rope_type": "longrope", "factor": 4.0}}))
    with pytest.raises(ValueError, match="longrope"):
        ModelConfig.from_hf_config(p)
    assert ModelConfig().attention_scale is None
    p.write_text(json.dumps({**base, "rope_scaling": None}))
    assert ModelConfig.from_hf_config(p).rope_scaling is None


def test_configurations_that_are_refused_by_name(tmp_path):
    import json
    base = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 256, "num_hidden_layers": 4, "num_attention_heads": 4,
            "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512, "vocab_size": 320, "num_experts": 8,
            "num_experts_per_tok": 2, "moe_intermediate_size": 128}
    p = tmp_path / "config.json"
    for extra, match in (({"mlp_only_layers": [0]}, "mix dense and expert"), ({"decoder_sparse_step": 2}, "mix dense and expert"),
                         ({"mlp_bias": True}, "mlp_bias"), ({"attention_bias": True}, "attention_bias")):
        p.write_text(json.dumps({**base, **extra}))
        with pytest.raises(ValueError, match=match):
            ModelConfig.from_hf_config(p)
    p.write_text(json.dumps({**base, "mlp_only_layers": [], "decoder_sparse_step": 1}))
    assert ModelConfig.from_hf_config(p).is_moe
    # sliding-window checkpoints are served inside one window; Qwen2's unused window does not limit them
    p.write_text(json.dumps({"architectures": ["MistralForCausalLM"], "hidden_size": 256, "num_hidden_layers": 2,
                             "num_attention_heads": 4, "vocab_size": 320, "intermediate_size": 512,
                             "max_position_embeddings": 32768, "sliding_window": 4096}))
    assert ModelConfig.from_hf_config(p).max_position == 4096
    p.write_text(json.dumps({"architectures": ["Qwen2ForCausalLM"], "hidden_size": 256, "num_hidden_layers": 2,
                             "num_attention_heads": 4, "vocab_size": 320, "intermediate_size": 512,
                             "max_position_embeddings": 32768, "sliding_window": 4096, "use_sliding_window": False}))
    assert ModelConfig.from_hf_config(p).max_position == 32768
