"""MoE routing, grouped expert GEMM and combine against a dense per-token oracle."""
from dataclasses import replace

import pytest
import torch

from cubic_serve_b200.models.config import ModelConfig, QuantSpec
from cubic_serve_b200.ops import wq_pack

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("persistent", [1, 0])
@pytest.mark.parametrize("method,tokens,ep", [("nvfp4", 37, 1), ("cubic", 200, 1), ("nvfp4", 64, 2), ("none", 5, 1),
                                              ("cubic", 700, 1)])
def test_moe_layer_matches_oracle(method, tokens, ep, persistent):
    """Both grouped-GEMM kernels: the persistent one (default) and one CTA per (work item, weight tile)."""
    from cubic_serve_b200.models.moe import moe_reference, random_moe_weights
    from cubic_serve_b200.ops import native
    native.lib().cb_wq_gemm_grouped_mode(persistent)
    cfg = ModelConfig(family="gqa_moe", hidden_size=256, num_experts=16, experts_per_token=4, moe_intermediate_size=128,
                      quant=QuantSpec(method, 4 if method != "none" else 16, {"nvfp4": 16, "cubic": 128, "none": 0}[method]))
    x = (torch.randn(tokens, 256, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16).to(DEV)
    total = torch.zeros(tokens, 256, device=DEV)
    ref_total = torch.zeros(tokens, 256, device=DEV)
    for rank in range(ep):
        gen = torch.Generator(device=DEV).manual_seed(7 + rank)
        layer = random_moe_weights(cfg, DEV, gen, tp_rank=rank, tp_size=ep, std=0.05)
        out = layer.forward(x)
        torch.cuda.synchronize()
        sc = layer.scratch
        counts = sc.counts.cpu()
        assert int(sc.total) == int(counts.sum())
        assert int(sc.total) == (tokens * 4 if ep == 1 else int(((sc.topk_ids // (16 // ep)) == rank).sum()))
        n_items = int(sc.tiles[0])
        assert n_items == int(((counts + sc.mb - 1) // sc.mb).sum())
        local = 16 // ep
        gu = [wq_pack.unpack_to_dense(wq_pack.PackedWeight(layer.gate_up.fmt, layer.gate_up.n, layer.gate_up.k,
                                                             layer.gate_up.group_k, layer.gate_up.codes[e],
                                                             None if layer.gate_up.meta is None else layer.gate_up.meta[e],
                                                             layer.gate_up.alpha)) for e in range(local)]
        dn = [wq_pack.unpack_to_dense(wq_pack.PackedWeight(layer.down.fmt, layer.down.n, layer.down.k, layer.down.group_k,
                                                             layer.down.codes[e],
                                                             None if layer.down.meta is None else layer.down.meta[e],
                                                             layer.down.alpha)) for e in range(local)]
        ref = moe_reference(x, layer.router.codes, gu, dn, 4, True, expert_lo=rank * local)
        total += out.float()
        ref_total += ref
        # SwiGLU in the epilogue of the grouped gate/up GEMM (rows of every expert interleaved): the grouped GEMM
        # gives a tile all of its k-blocks in order, so the output is identical
        plain = out.clone()
        layer.fuse_activation()
        assert layer.gate_up.act_interleaved
        assert torch.equal(layer.forward(x), plain)
    from cubic_serve_b200.ops import kernels as K
    native.lib().cb_wq_gemm_grouped_mode(1)
    K.workspace(torch.device(DEV)).check_status()
    assert _rel(total, ref_total) < 3e-2


def test_router_stable_ties_and_weights():
    from cubic_serve_b200.ops import kernels as K
    t, e, k = 9, 64, 8
    logits = torch.zeros(t, e)
    logits[:, 10:30] = 1.0                                   # a 20-way tie: lowest ids win
    logits[3, 50] = 5.0
    x = torch.randn(t, 128).to(torch.bfloat16).to(DEV)
    sc = K.MoeScratch(t, k, 128, 256, e, 32, DEV)
    K.moe_route(logits.to(torch.bfloat16).to(DEV), x, k, sc)
    ids = sc.topk_ids.cpu()
    assert ids[0].tolist() == list(range(10, 18))
    assert ids[3].tolist() == [50] + list(range(10, 17))
    w = sc.topk_w.cpu()
    assert torch.allclose(w.sum(-1), torch.ones(t), atol=1e-5)
    assert torch.allclose(w[0], torch.full((k,), 1 / k), atol=1e-6)
    # every route landed in its expert's range and carries its token's row
    off, cnt, pos = sc.offsets.cpu(), sc.counts.cpu(), sc.route_pos.cpu()
    for ti in range(t):
        for r in range(k):
            ex = int(ids[ti, r])
            assert off[ex] <= pos[ti, r] < off[ex] + cnt[ex]
            assert torch.equal(sc.xs[int(pos[ti, r])], x[ti])


@pytest.mark.parametrize("method,tokens,ranks", [("none", 50, 4), ("nvfp4", 200, 8), ("cubic", 7, 2)])
def test_expert_parallel_dispatch_combine_matches_single_rank(method, tokens, ranks):
    """Row-sharded tokens, experts spread over emulated ranks on one device: dispatch -> experts -> combine must
    reproduce residual + MoE(x) of the one-rank layer.  The ranks' kernels run phase by phase (a rank's wait is
    always for launches that are already in the stream)."""
    from cubic_serve_b200.models.decoder import quantize_linear
    from cubic_serve_b200.models.moe import MoeLayer, stack_experts
    from cubic_serve_b200.ops import kernels as K
    from cubic_serve_b200.parallel.ep import FusedEp, local_ep_fabric
    from cubic_serve_b200.parallel.tp import rows_per_rank
    E, k, H, I = 16, 4, 256, 128
    cfg = ModelConfig(family="gqa_moe", hidden_size=H, num_experts=E, experts_per_token=k, moe_intermediate_size=I,
                      quant=QuantSpec(method, 4 if method != "none" else 16, {"nvfp4": 16, "cubic": 128, "none": 0}[method]))
    g = torch.Generator(device=DEV).manual_seed(11)
    router = wq_pack.pack_bf16((torch.randn(E, H, device=DEV, generator=g) * 0.05).to(torch.bfloat16))
    gus = [quantize_linear(torch.randn(2 * I, H, device=DEV, generator=g) * 0.05, cfg) for _ in range(E)]
    dns = [quantize_linear(torch.randn(H, I, device=DEV, generator=g) * 0.05, cfg) for _ in range(E)]

    def layer_for(lo, n):
        gu, gcs, gms = stack_experts(gus[lo:lo + n])
        dn, dcs, dms = stack_experts(dns[lo:lo + n])
        return MoeLayer(router, gu, dn, (gcs, gms, dcs, dms), E, k, lo, n, True)

    x = (torch.randn(tokens, H, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    resid = (torch.randn(tokens, H, device=DEV, generator=g) * 0.5).to(torch.bfloat16)
    want = layer_for(0, E).forward(x, residual=resid, out=torch.empty_like(resid)).float()

    rpr = rows_per_rank(tokens, ranks)
    fabric = local_ep_fabric(ranks, H, k, max_tokens=max(tokens, 64), device=DEV)
    eps = [FusedEp(b, torch.device(DEV), E, 2 * I) for b in fabric]
    layers = [layer_for(r * (E // ranks), E // ranks) for r in range(ranks)]
    h_rows, x_rows, cnts = [], [], []
    for r in range(ranks):
        lo = r * rpr
        cnt = max(0, min(tokens, lo + rpr) - lo)
        cnts.append(cnt)
        xr = torch.zeros(rpr, H, dtype=torch.bfloat16, device=DEV)
        hr = torch.zeros(rpr, H, dtype=torch.bfloat16, device=DEV)
        xr[:cnt], hr[:cnt] = x[lo:lo + cnt], resid[lo:lo + cnt]
        x_rows.append(xr)
        h_rows.append(hr)
    for rounds in range(2):                                  # twice: counters are cumulative, buffers are reused
        for r in range(ranks):
            h_rows[r][:cnts[r]] = resid[r * rpr:r * rpr + cnts[r]]
        for r in range(ranks):
            eps[r].dispatch(layers[r], x_rows[r], cnts[r])
        for r in range(ranks):
            eps[r].experts(layers[r])
        for r in range(ranks):
            eps[r].finish(cnts[r], h_rows[r])
        torch.cuda.synchronize()
        K.workspace(torch.device(DEV)).check_status()
        got = torch.cat([h_rows[r][:cnts[r]] for r in range(ranks)]).float()
        assert got.shape == want.shape
        assert _rel(got, want) < 2e-2
    # every row went only to ranks that own one of its experts, once per rank
    sent = torch.stack([(eps[r].sent[:cnts[r]] >= 0).sum() for r in range(ranks)]).sum().item()
    assert tokens <= sent <= tokens * min(k, ranks)


def test_moe_checkpoint_serves_and_matches_the_oracle(tmp_path):
    """A written MoE checkpoint: the loaded expert layer equals the dense oracle built from the checkpoint's own
    decode, and the engine decodes with it (graphs captured, qualification passed)."""
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.checkpoint import _dense_of, admit_checkpoint, load_decoder_weights, logical_inventory, \
        write_random_checkpoint
    from cubic_serve_b200.models.decoder import DecoderRunner
    from cubic_serve_b200.models.moe import moe_reference
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = ModelConfig(name="moe-ck", family="gqa_moe", num_layers=2, hidden_size=256, num_q_heads=4, num_kv_heads=2,
                      head_dim=128, intermediate_size=512, vocab_size=512, qk_norm=True, num_experts=8, experts_per_token=2,
                      moe_intermediate_size=128, quant=QuantSpec("cubic", 4, 128))
    ck = admit_checkpoint(write_random_checkpoint(tmp_path / "moe", cfg, seed=4, std=0.05))
    w = load_decoder_weights(ck, torch.device(DEV))
    layer = w.layers[0].moe
    shapes, _ = logical_inventory(ck.cfg)
    dense = lambda m: _dense_of("cubic", ck.payload(m), shapes[m], ck.cfg.quant).to(DEV)  # noqa: E731
    gu = [torch.cat([dense(f"model.layers.0.mlp.experts.{e}.gate_proj"), dense(f"model.layers.0.mlp.experts.{e}.up_proj")])
          for e in range(8)]
    dn = [dense(f"model.layers.0.mlp.experts.{e}.down_proj") for e in range(8)]
    x = (torch.randn(40, 256, generator=torch.Generator().manual_seed(2)) * 0.5).to(torch.bfloat16).to(DEV)
    out = layer.forward(x)
    ref = moe_reference(x, layer.router.codes, gu, dn, 2, ck.cfg.norm_topk_prob)
    assert _rel(out, ref) < 2e-2
    runner = DecoderRunner(ck.cfg, w, num_pages=64, max_tokens=256)
    ex = GpuExecutor(runner, max_rows=4, max_prefill_tokens=256, max_model_len=128)
    assert ex.capture_decode_graphs([4]) == [4]
    eng = LLMEngine(ex, 64, SchedulerConfig(max_running_requests=4, max_model_len=128, max_batched_tokens=256,
                                            enable_prefix_cache=False))
    outs = eng.generate([[5, 9, 200, 31, 7], [3, 3, 100]], SamplingParams(max_tokens=6, ignore_eos=True))
    runner.ws.check_status()
    assert all(len(o) == 6 and all(0 <= t < 512 for t in o) for o in outs)
