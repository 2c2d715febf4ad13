import pytest

from cubic_serve_b200.contracts.execution import GraphBucket, GroupKind, LaunchPlan, ParallelTopology, ReplayLeasePool


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
    pool = ReplayLeasePool()
    a = pool.acquire()
    with pytest.raises(RuntimeError):
        pool.acquire()
    pool.release(a)
    b = pool.acquire()
    with pytest.raises(RuntimeError):
        pool.release(a)
    pool.release(b)


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
