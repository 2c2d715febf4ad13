"""Captured encode calls of the vision tower on the GPU (sorts late: a failure here hides no other test)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bucket_replays_equal_the_eager_tower():
    from cubic_serve_b200.executor.vision import VisionGraphBucket
    from cubic_serve_b200.models.vision import VisionConfig, VisionEncoder, random_vision_weights
    dev = torch.device("cuda")
    cfg = VisionConfig(depth=3, hidden_size=128, intermediate_size=256, num_heads=4, out_hidden_size=64, patch_size=4,
                       spatial_merge_size=2, temporal_patch_size=2, num_position_embeddings=64)
    enc = VisionEncoder(cfg, random_vision_weights(cfg, 1, torch.bfloat16, dev, std=0.1))
    bucket = VisionGraphBucket(enc, 128)
    g = torch.Generator().manual_seed(2)
    for grid in ([[1, 8, 12]], [[2, 4, 4]], [[1, 2, 2]], [[1, 8, 12]]):
        n = sum(t * h * w for t, h, w in grid)
        px = torch.randn(n, cfg.patch_width, generator=g).to(dev, torch.bfloat16)
        want, _ = enc.encode(px, torch.tensor(grid))
        got = bucket.encode(px, torch.tensor(grid))
        torch.cuda.synchronize()
        rel = ((got.float() - want.float()).norm() / want.float().norm()).item()
        assert got.shape == want.shape and rel < 4e-2, (grid, rel)
    assert bucket.graph is not None and bucket.replays == 4
