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
