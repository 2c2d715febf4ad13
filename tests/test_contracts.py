import pytest

from cubic_serve_b200.contracts.execution import GraphBucket, GroupKind, LaunchPlan, ParallelTopology


def test_topology_tp4_pp2_ep2():
    t = ParallelTopology.single_node(range(8), tp=4, pp=2, ep=2)
    assert t.world_size == 8 and t.etp == 2 and t.sampler_rank == 4
    p = t.placement(6)
    assert (p.stage, p.tensor_rank, p.expert_rank, p.expert_tensor_rank, p.device) == (1, 2, 1, 0, 6)
    names = {g.name: g.ranks for g in t.groups}
    assert names["tp:1"] == (4, 5, 6, 7) and names["pp:3"] == (3, 7)
    assert names["ep:0:1"] == (1, 3) and names["etp:1:0"] == (4, 5)
    kinds = {g.kind for g in t.groups_of(6)}
    assert kinds == {GroupKind.TENSOR, GroupKind.PIPELINE, GroupKind.EXPERT, GroupKind.EXPERT_TENSOR}
    assert t.expert_slice(6, 128) == (64, 128) and t.expert_slice(1, 128) == (0, 64)
    assert t.layer_range(0, 94) == (0, 47) and t.layer_range(1, 94) == (47, 94)


@pytest.mark.parametrize("kw", [dict(tp=3, pp=1, ep=2), dict(tp=2, pp=3, ep=1), dict(tp=4, pp=1, ep=1)])
def test_topology_rejects(kw):
    with pytest.raises(ValueError):
        ParallelTopology.single_node(range(6 if kw["pp"] == 3 else 3), **kw)


def test_launch_plan_and_lease():
    buckets = [GraphBucket(c) for c in (256, 128, 64, 32)]
    plan = LaunchPlan.choose(buckets, 70)
    assert plan.bucket.capacity == 128 and plan.padding_rows == 58
    with pytest.raises(ValueError):
        LaunchPlan.choose(buckets, 300)


def test_hybrid_config_layer_types_and_hf_parse(tmp_path):
    import json
    from cubic_serve_b200.models.config import ModelConfig, hybrid_8b_config
    cfg = hybrid_8b_config()
    assert cfg.is_hybrid and [cfg.layer_is_gdn(i) for i in range(8)] == [True, True, True, False] * 2
    assert not ModelConfig().is_hybrid and not ModelConfig().layer_is_gdn(0)
    hf = {"architectures": ["Qwen3NextForCausalLM"], "num_hidden_layers": 8, "hidden_size": 512, "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 1024, "vocab_size": 1000, "rms_norm_eps": 1e-6,
          "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 128, "linear_value_head_dim": 128,
          "full_attention_interval": 4, "partial_rotary_factor": 0.25}
    (tmp_path / "config.json").write_text(json.dumps(hf))
    got = ModelConfig.from_hf_config(tmp_path / "config.json")
    assert got.family == "qwen3_5" and got.gdn_interval == 4 and (got.gdn_k_heads, got.gdn_v_heads) == (2, 4)
    assert got.rotary_dim == 32 and got.zero_centered_norm and got.attn_output_gate
    assert sum(got.layer_is_gdn(i) for i in range(8)) == 6


def test_model_registry_and_adapter_source_policy(tmp_path):
    from cubic_serve_b200.models import registry as R
    assert {"gqa_decoder", "gqa_moe", "qwen3_5"} <= set(R.families())
    assert R.for_architecture("Qwen3NextForCausalLM").family == "qwen3_5"
    assert R.for_architecture("LlamaForCausalLM") is R.get("gqa_decoder")
    import pytest
    with pytest.raises(R.ModelRegistryError):
        R.for_architecture("GPT2LMHeadModel")
    good = tmp_path / "toy_adapter.py"
    good.write_text(
        "from cubic_serve_b200.models.config import ModelConfig\n"
        "from cubic_serve_b200.models.registry import ModelDefinition, get\n"
        "base = get('gqa_decoder')\n"
        "def parse(path):\n"
        "    return ModelConfig(name='adapted', num_layers=3)\n"
        "MODEL_DEFINITION = ModelDefinition('toy_adapter', ('ToyForCausalLM',), parse, base.random_weights,\n"
        "                                   base.load_weights, base.build_runner, 'test adapter')\n")
    d = R.load_adapter(good)
    try:
        assert d.family == "toy_adapter" and R.for_architecture("ToyForCausalLM") is d
        assert d.parse_config(tmp_path).num_layers == 3
    finally:
        R._definitions.pop("toy_adapter", None)
    for body, needle in (("import os\n", "import of 'os'"), ("from subprocess import run\n", "subprocess"),
                         ("x = open('/etc/passwd')\n", "'open'"), ("y = ().__class__.__subclasses__()\n", "__subclasses__"),
                         ("import torch\ntorch.__builtins__\n", "__builtins__"), ("from . import sibling\n", "import from ."),
                         ("def f(:\n", "syntax error")):
        bad = tmp_path / "bad.py"
        bad.write_text(body + "MODEL_DEFINITION = None\n")
        v = R.audit_source(bad.read_text())
        assert v and any(needle in x.what for x in v), (body, v)
        with pytest.raises(R.ModelRegistryError):
            R.load_adapter(bad)


def test_axis_spans_and_partition_plans():
    import pytest
    from cubic_serve_b200.models.config import NAMED_CONFIGS
    from cubic_serve_b200.models.parallel_weights import AxisSpan, PartitionError, plan_partition, storage_bits
    s = AxisSpan.shard(32, 3, 8)
    assert (s.start, s.stop, s.size) == (12, 16, 4) and s.scaled(128).slice() == slice(1536, 2048) and not s.full
    assert AxisSpan.whole(7).full
    with pytest.raises(PartitionError):
        AxisSpan.shard(12288, 0, 5)
    with pytest.raises(PartitionError, match="multiples of 64"):
        AxisSpan.shard(768, 0, 8, 64)
    with pytest.raises(PartitionError):
        AxisSpan(3, 2, 10)
    dense = NAMED_CONFIGS["dense-8b"]()
    one = plan_partition(dense).ranks[0]
    assert 4.3 < storage_bits(dense) < 4.5
    assert 5.5e9 < one.weight_bytes < 7.5e9                   # ~6.4 GB of 4-bit weights + bf16 embedding and head
    plan = plan_partition(dense, tp=4, pp=2)
    assert [r["stage"] for r in plan.summary()] == [0, 0, 0, 0, 1, 1, 1, 1]
    r5 = plan.ranks[5]
    assert r5.tensor_rank == 1 and r5.layers == (18, 36) and r5.experts is None
    q = next(x for x in r5.shares if x.module == "model.layers.18.self_attn.q_proj")
    o = next(x for x in r5.shares if x.module == "model.layers.18.self_attn.o_proj")
    assert (q.rows.start, q.rows.stop, q.cols.full) == (1024, 2048, True) and (o.cols.start, o.cols.stop) == (1024, 2048)
    total = sum(r.weight_bytes for r in plan.ranks)
    assert abs(total - one.weight_bytes) / one.weight_bytes < 0.25         # a split moves bytes, it does not create many
    # more ranks than key/value heads: neighbouring ranks hold a copy of the same head (8 heads over 16 ranks)
    shared = plan_partition(dense, tp=16)
    k = [next(x for x in r.shares if x.module == "model.layers.0.self_attn.k_proj").rows for r in shared.ranks[:4]]
    assert [(s.start, s.stop) for s in k] == [(0, 128), (0, 128), (128, 256), (128, 256)]
    import dataclasses
    with pytest.raises(PartitionError, match="key/value heads"):
        plan_partition(dataclasses.replace(dense, num_kv_heads=3, num_q_heads=24), tp=2)
    moe = NAMED_CONFIGS["moe-30b-a3b"]()
    kv8 = plan_partition(moe, tp=8, ep=8)                      # 4 key/value heads on 8 ranks: two ranks per head
    assert next(x for x in kv8.ranks[5].shares if x.module.endswith("layers.0.self_attn.k_proj")).rows.start == 2 * 128
    wide = dataclasses.replace(moe, num_kv_heads=8)
    with pytest.raises(PartitionError, match="expert intermediate size"):
        plan_partition(wide, tp=8)                             # 768 / 8 = 96 columns: not a multiple of the K block
    ep = plan_partition(wide, tp=8, ep=8)                      # whole experts per rank instead
    assert ep.ranks[3].experts.size == moe.num_experts // 8 and ep.ranks[3].experts.start == 3 * (moe.num_experts // 8)
    assert plan_partition(moe, tp=4).ranks[0].experts.full
    hybrid = plan_partition(NAMED_CONFIGS["hybrid-8b"](), tp=2)
    assert any(x.module.endswith("linear_attn.in_proj_qkvz") for x in hybrid.ranks[1].shares)
    with pytest.raises(PartitionError):
        plan_partition(dense, pp=99)


def test_inspect_model_prints_partitions(capsys):
    import json
    from cubic_serve_b200.cli import main
    assert main(["inspect-model", "random:dense-8b", "--tp", "2", "--json"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert len(info["partition"]) == 2 and info["partition"][1]["tensor_rank"] == 1
    assert main(["inspect-model", "random:dense-8b", "--tp", "3", "--json"]) == 0
    assert "partition_error" in json.loads(capsys.readouterr().out)


def test_model_spec_cache_state_and_manifest(tmp_path):
    import dataclasses
    import pytest
    from cubic_serve_b200.contracts.model import CacheSpec, ModelSpec, StateSpec, WeightManifest
    from cubic_serve_b200.models.checkpoint import SafetensorsDirectory, inspect_checkpoint, write_random_checkpoint
    from cubic_serve_b200.models.config import NAMED_CONFIGS, ModelConfig, QuantSpec
    from cubic_serve_b200.ops.kernels import kv_blob_bytes
    c = CacheSpec(layers=36, kv_heads=8, head_dim=128, k_bits=8, v_bits=4)
    assert c.blob_bytes == kv_blob_bytes(128, 8, 4) == 16 * 128 + 16 * 64 + 2 * 16 * 4 * 4
    assert c.page_bytes == 36 * 8 * c.blob_bytes and c.bytes_per_token() == c.page_bytes / 16
    assert CacheSpec(1, 1, 128, 6, 6).blob_bytes == kv_blob_bytes(128, 6, 6)
    with pytest.raises(ValueError):
        CacheSpec(1, 1, 128, 5, 8)
    s = StateSpec(layers=27, k_heads=16, v_heads=32)
    assert s.delta_bytes == 32 * 128 * 128 * 4 and s.conv_bytes == 3 * 64 * 128 * 2
    dense = ModelSpec.from_config(NAMED_CONFIGS["dense-8b"](), 8, 8)
    assert dense.state is None and dense.cache.layers == 36
    # 20 GiB for pages: not capped by the request limit
    pages = dense.kv_pages(26 << 30, 6 << 30, 32768, 256)
    assert pages == (20 << 30) // dense.cache.page_bytes
    hybrid = ModelSpec.from_config(NAMED_CONFIGS["hybrid-8b"](), 8, 8, tp=2)
    assert hybrid.state.layers == 27 and hybrid.cache.layers == 9 and hybrid.cache.kv_heads == 4
    with_state = hybrid.kv_pages(26 << 30, 6 << 30, 32768, 256)
    assert with_state == ((20 << 30) - 256 * hybrid.state.bytes_per_request) // hybrid.cache.page_bytes
    stage = ModelSpec.from_config(NAMED_CONFIGS["dense-8b"](), 4, 8, tp=4, layers=(18, 36))
    assert stage.cache.layers == 18 and stage.cache.kv_heads == 2 and stage.digest != dense.digest
    with pytest.raises(ValueError):
        ModelSpec.from_config(NAMED_CONFIGS["dense-8b"](), tp=3)
    cfg = ModelConfig(name="toy", num_layers=1, hidden_size=128, num_q_heads=2, num_kv_heads=1, head_dim=64,
                      intermediate_size=256, vocab_size=256, rope_theta=1e4, quant=QuantSpec("cubic", 4, 128))
    a = write_random_checkpoint(tmp_path / "a", cfg, seed=0)
    b = write_random_checkpoint(tmp_path / "b", dataclasses.replace(cfg, intermediate_size=384), seed=0)
    ma, mb = WeightManifest.from_store(SafetensorsDirectory(a)), WeightManifest.from_store(SafetensorsDirectory(b))
    assert len(ma) == len(mb) and ma.digest != mb.digest and ma.files == ("model.safetensors",)
    assert ma.digest == WeightManifest.from_store(SafetensorsDirectory(a)).digest == inspect_checkpoint(a)["manifest_digest"]
    assert ModelSpec.from_config(cfg, manifest=ma).digest != ModelSpec.from_config(cfg, manifest=mb).digest
