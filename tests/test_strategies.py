import json

import pytest

from cubic_serve_b200.ops import strategies as S


def test_defaults_and_overrides(tmp_path):
    cfg = S.operator_config_from_dict({"gemm": {"stream_k_max_rows": 64, "stream_k_bf16": False}, "moe": {"rows_per_item_small": 48}})
    assert cfg.gemm.stream_k_max_rows == 64 and cfg.gemm.stream_k_bf16 is False and cfg.gemm.split_k_max == 8
    assert cfg.moe.rows_per_item_small == 48 and cfg.attention.target_ctas == 296
    p = tmp_path / "ops.json"
    p.write_text(json.dumps({"attention": {"max_splits": 4}}))
    assert S.load_operator_config(str(p)).attention.max_splits == 4


@pytest.mark.parametrize("bad", [{"gem": {}}, {"gemm": {"stream_k_max_row": 1}}, {"gemm": {"split_k_max": 0}},
                                 {"moe": {"rows_per_item_small": 40}}, {"gemm": {"stream_k_bf16": 1}},
                                 {"attention": {"max_splits": "4"}}, []])
def test_rejects_unknown_and_out_of_range(bad):
    with pytest.raises(ValueError):
        S.operator_config_from_dict(bad)


def test_policy_drives_kernel_choice():
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.ops.wq_pack import FMT_BF16, FMT_CUBIC4
    old = S.active()
    try:
        S.install(S.OperatorConfig())
        assert K.use_stream_k(64, 24576, FMT_CUBIC4) and K.use_stream_k(256, 24576, FMT_CUBIC4)
        # above 256 rows: CTA pairs when every pair gets enough k-blocks
        assert K.use_stream_k(512, 24576, FMT_CUBIC4) and K.use_stream_k(4096, 4096, FMT_CUBIC4, k=12288)
        assert not K.use_stream_k(512, 6144, FMT_CUBIC4) and not K.use_stream_k(1024, 4096, FMT_CUBIC4)
        assert not K.use_stream_k(4096, 24576 + 128, FMT_CUBIC4)          # odd number of weight tiles
        assert K.use_stream_k(256, 151936, FMT_BF16) and not K.use_stream_k(16, 6144, FMT_CUBIC4)
        assert K.choose_splits(256, 4096, 4096) == 4
        S.install(S.operator_config_from_dict({"gemm": {"stream_k_max_rows": 64, "split_k_max": 2}}))
        assert not K.use_stream_k(256, 24576, FMT_CUBIC4) and K.choose_splits(256, 4096, 4096) == 2
        S.install(S.operator_config_from_dict({"gemm": {"cta_pairs": False}}))
        assert not K.use_stream_k(512, 24576, FMT_CUBIC4) and K.use_stream_k(256, 24576, FMT_CUBIC4)
    finally:
        S.install(old)


def test_autotune_shapes_candidates_and_install():
    from cubic_serve_b200.models.config import NAMED_CONFIGS
    from cubic_serve_b200.ops import autotune, kernels as K, wq_pack
    shapes = autotune.model_shapes(NAMED_CONFIGS["dense-8b"]())
    assert (wq_pack.FMT_CUBIC4, 6144, 4096, False) in shapes and (wq_pack.FMT_CUBIC4, 24576, 4096, True) in shapes
    assert (wq_pack.FMT_BF16, 151936, 4096, False) in shapes
    tp2 = autotune.model_shapes(NAMED_CONFIGS["dense-8b"](), tp=2)
    assert (wq_pack.FMT_CUBIC4, 3072, 4096, False) in tp2 and (wq_pack.FMT_CUBIC4, 4096, 6144, False) in tp2
    # splits leave at least four k-blocks per CTA and at most ~4 CTAs per SM; the persistent kernel is always timed
    assert autotune.candidates(16, 151936, 4096) == [("tile", 1), ("stream_k", 0)]
    assert ("tile", 8) in autotune.candidates(16, 4096, 4096) and ("tile", 8) not in autotune.candidates(16, 4096, 1024)
    w = autotune._random_weight(wq_pack.FMT_CUBIC4, 256, 512, True, "cpu")
    assert w.act_interleaved and (w.n, w.k) == (256, 512)
    for fmt in (wq_pack.FMT_AFFINE4, wq_pack.FMT_NVFP4, wq_pack.FMT_BF16):
        assert autotune._random_weight(fmt, 128, 256, False, "cpu").fmt == fmt
    assert (wq_pack.FMT_NVFP4, 5120, 2048, False) in autotune.model_shapes(NAMED_CONFIGS["moe-30b-a3b"]())
    plan = {autotune.plan_key(0, 16, 6144, 4096, False): {"use": True, "kernel": "tile", "splits": 3},
            autotune.plan_key(0, 16, 4096, 4096, False): {"use": False, "kernel": "tile", "splits": 4},
            autotune.plan_key(3, 64, 151936, 4096, False): {"use": True, "kernel": "stream_k", "splits": 0}}
    try:
        assert autotune.install(plan) == 2
        assert K.TUNED_PLANS == {"0:16:6144:4096:0": (False, 3), "3:64:151936:4096:0": (True, 0)}
    finally:
        assert autotune.install(None) == 0 and not K.TUNED_PLANS


def test_operator_profiles_override_by_device_model_and_topology(tmp_path):
    import json
    import pytest
    from cubic_serve_b200.ops import strategies as S
    data = {"gemm": {"split_k_max": 4},
            "profiles": [{"name": "b200", "match": {"device": "nvidia b200*"}, "gemm": {"split_k_max": 8, "pair_min_blocks": 96}},
                         {"match": {"model": "moe-*", "tp": 4}, "moe": {"rows_per_item_small": 48}, "gemm": {"split_k_max": 6}},
                         {"match": {"sms": 132}, "attention": {"target_ctas": 264}}]}
    base = S.operator_config_from_dict(data)
    assert base.gemm.split_k_max == 4 and base.moe.rows_per_item_small == 32           # no context: nothing matches
    b200 = S.operator_config_from_dict(data, {"device": "NVIDIA B200", "sms": 148, "model": "dense-8b", "tp": 1})
    assert (b200.gemm.split_k_max, b200.gemm.pair_min_blocks, b200.attention.target_ctas) == (8, 96, 296)
    moe = S.operator_config_from_dict(data, {"device": "NVIDIA B200", "sms": 148, "model": "moe-30b-a3b", "tp": 4})
    assert moe.gemm.split_k_max == 6 and moe.gemm.pair_min_blocks == 96 and moe.moe.rows_per_item_small == 48   # later wins
    h100 = S.operator_config_from_dict(data, {"device": "NVIDIA H100", "sms": 132, "model": "moe-30b-a3b", "tp": 2})
    assert h100.gemm.split_k_max == 4 and h100.attention.target_ctas == 264
    for bad in ({"profiles": [{"match": {"gpu": "x"}}]}, {"profiles": [{"match": {}}]}, {"profiles": {}},
                {"profiles": [{"match": {"tp": 2}, "gemm": {"splitk": 1}}]}, {"profiles": [{"match": {"tp": 2}, "extra": 1}]}):
        with pytest.raises(ValueError):
            S.operator_config_from_dict(bad, {"tp": 1})
    f = tmp_path / "op.json"
    f.write_text(json.dumps(data))
    assert S.load_operator_config(str(f), {"sms": 132}).attention.target_ctas == 264
    ctx = S.launch_context("random:dense-8b", tp=2)
    assert ctx["model"] == "dense-8b" and ctx["tp"] == 2
    assert S.launch_context("/models/Qwen3-8B-cubic/", 1)["model"] == "Qwen3-8B-cubic"
