"""Three-axis rotary positions and encoder feature rows on the native runner (one GPU)."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec
from cubic_serve_b200.ops import eager

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rotary,section", [(128, (24, 20, 20)), (64, (11, 11, 10))])
def test_cache_write_kernel_rotates_by_axis(rotary, section):
    """Queries out of the cache-write kernel against the fp32 three-axis rotation of the same inputs; equal axes give the
    one-axis kernel's bits."""
    from cubic_serve_b200.ops import kernels as K
    dev = torch.device("cuda")
    T, hq, hkv, D = 37, 4, 2, 128
    g = torch.Generator().manual_seed(0)
    qkv = torch.randn(T, (hq + 2 * hkv) * D, generator=g).to(torch.bfloat16).to(dev)
    pos = torch.randint(0, 4000, (3, T), generator=g, dtype=torch.int32)
    inv = eager.rope_inv_freq(rotary, 1e6)
    cache = torch.zeros(4, hkv, K.kv_blob_bytes(D, 8, 8), dtype=torch.uint8, device=dev)
    slots = torch.full((T,), -1, dtype=torch.int32, device=dev)            # queries only: nothing is written
    q = torch.empty(T, hq * D, dtype=torch.bfloat16, device=dev)
    p = pos.to(dev)
    K.rope_kv_write(qkv, q, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary,
                    positions_hw=(p[1].contiguous(), p[2].contiguous()), mrope_section=section)
    want = eager.rope3(qkv[:, :hq * D].float().cpu().view(T, hq, D), pos.long(), inv, section).reshape(T, hq * D)
    got = q.float().cpu()
    assert ((got - want).norm() / want.norm()).item() < 4e-3
    one = torch.empty_like(q)
    K.rope_kv_write(qkv, one, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary)
    same = torch.empty_like(q)
    K.rope_kv_write(qkv, same, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary,
                    positions_hw=(p[0].contiguous(), p[0].contiguous()), mrope_section=section)
    assert torch.equal(same, one) and not torch.equal(q, one)
    with pytest.raises(ValueError):
        K.rope_kv_write(qkv, q, cache, p[0].contiguous(), slots, inv.to(dev), hq, hkv, D, 8, 8, rotary_dim=rotary,
                        positions_hw=(p[1].contiguous(), p[2].contiguous()), mrope_section=(1, 1, 1))


def _engine(chunk=512):
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    dev = torch.device("cuda")
    cfg = ModelConfig(name="mm", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, rope_theta=1e6, mrope_section=(24, 20, 20),
                      quant=QuantSpec("cubic", 4, 128))
    w = random_decoder_weights(cfg, dev, seed=0, std=0.05)
    runner = DecoderRunner(cfg, w, num_pages=256, max_tokens=512)
    ex = GpuExecutor(runner, max_rows=8, max_prefill_tokens=512, max_model_len=256)
    ex.capture_decode_graphs()
    eng = LLMEngine(ex, 256, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                             prefill_chunk_tokens=chunk))
    return eng, ex, w


def _run(eng, prompt, mm, n=8):
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    rid = eng.add_request(prompt, SamplingParams(max_tokens=n, ignore_eos=True), multimodal=mm)
    out = []
    while eng.has_unfinished:
        out += [o.token_id for o in eng.step() if o.request_id == rid and o.token_id is not None]
    return out


def test_native_runner_takes_feature_rows_and_axes():
    from cubic_serve_b200.models.vision import mrope_positions
    from cubic_serve_b200.runtime.multimodal import MultimodalInput
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, 2048, 70).tolist()
    eng, ex, w = _engine()
    assert ex.accepts_features
    plain = _run(eng, prompt, None)
    embed = w.extras["embed_full"] if "embed_full" in w.extras else w.embed
    own = embed[torch.tensor(prompt[5:29], device=embed.device)].float().cpu()         # the rows' own embeddings
    line = np.stack([np.arange(70)] * 3)

    def mm(rows, positions, delta, digest):
        return MultimodalInput([(5, rows, digest)], positions, delta)
    # feature rows equal to the embeddings they replace, positions equal on all axes: nothing changes
    assert _run(_engine()[0], prompt, mm(own, line, 0, b"own")) == plain
    # other rows, or a grid on the row / column axes, change the continuation
    feats = torch.randn(24, 512, generator=torch.Generator().manual_seed(1)) * own.std()
    a = _run(_engine()[0], prompt, mm(feats, line, 0, b"f"))
    assert a != plain
    pos, delta = mrope_positions(prompt, [(5, 24, (1, 8, 12))], 2)
    b = _run(_engine()[0], prompt, mm(feats, np.asarray(pos), delta, b"f"))
    assert b != a and delta < 0
    # chunked prefill cuts the media span: the same tokens; and the cached pages of equal media are reused
    assert _run(_engine(chunk=16)[0], prompt, mm(feats, np.asarray(pos), delta, b"f")) == b
    eng2 = _engine()[0]
    first = _run(eng2, prompt, mm(feats, np.asarray(pos), delta, b"f"))
    hits = eng2.prefix.hit_tokens
    again = _run(eng2, prompt, mm(feats, np.asarray(pos), delta, b"f"))
    assert first == b and again == b and eng2.prefix.hit_tokens > hits
    other = _run(eng2, prompt, mm(own, np.asarray(pos), delta, b"g"))             # other media: its span is not shared
    assert other != b
