"""The K-cache grouping study (CPU): without outliers the schemes agree; with outlier channels per-channel token groups
keep their error, per-token channel groups lose accuracy and the rotation option recovers part of it."""
import torch

from cubic_serve_b200.ops import eager
from cubic_serve_b200.utils.kv_layout_study import hadamard, study


def test_grouping_schemes_on_outlier_channels():
    flat = study(ratio=1.0)["errors"]["int4"]
    a, b = flat["channel_groups_of_a_token"]["logits"], flat["token_groups_of_a_channel"]["logits"]
    assert abs(a - b) < 0.02 and 0.05 < a < 0.15
    hot = study(ratio=20.0)["errors"]
    for bits in ("int8", "int6", "int4"):
        e = hot[bits]
        assert e["token_groups_of_a_channel"]["logits"] < e["channel_groups_after_rotation"]["logits"] \
            < e["channel_groups_of_a_token"]["logits"]
    assert hot["int4"]["token_groups_of_a_channel"]["logits"] < 0.12
    assert hot["int4"]["channel_groups_of_a_token"]["logits"] > 0.3


def test_token_group_oracle_keeps_the_tail_and_the_rotation_is_orthogonal():
    k = torch.randn(70, 2, 32, generator=torch.Generator().manual_seed(0))
    q = eager.kv_quantize_token_groups(k, 4)
    assert torch.equal(q[64:], k[64:]) and not torch.equal(q[:64], k[:64])        # 6 tokens wait in the tail
    assert (q[:64] - k[:64]).abs().max() <= k[:64].abs().amax() / 7 / 2 + 1e-6
    h = hadamard(128)
    assert torch.allclose(h @ h, torch.eye(128), atol=1e-5) and torch.equal(h, h.t())
