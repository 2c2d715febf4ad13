"""Gated DeltaNet kernels (causal conv + gated delta rule + gated norm) against the fp32 oracles."""
import pytest
import torch

from cubic_serve_b200.ops import eager

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / b.float().cpu().norm().clamp_min(1e-12)).item()


def _segments(K, counts, slots, pos0):
    i32 = dict(dtype=torch.int32, device=DEV)
    row0 = [sum(counts[:i]) for i in range(len(counts))]
    return K.GdnSegments(torch.tensor(row0, **i32), torch.tensor(counts, **i32), torch.tensor(slots, **i32),
                         torch.tensor(pos0, **i32), len(counts))


def test_gdn_conv_segments_and_state():
    from cubic_serve_b200.ops import kernels as K
    g = torch.Generator().manual_seed(0)
    C, slots = 320, 6
    counts, slot_of, pos0 = [5, 1, 9, 0, 2], [2, 0, 5, 1, 3], [0, 7, 3, 4, 0]
    T = sum(counts)
    x = torch.randn(T, C + 64, generator=g).to(torch.bfloat16)               # wider rows: the conv reads the first C
    w = torch.randn(C, 4, generator=g) * 0.5
    bias = torch.randn(C, generator=g) * 0.1
    state = torch.randn(slots, 3, C, generator=g).to(torch.bfloat16)
    out = torch.zeros(T, C, dtype=torch.bfloat16, device=DEV)
    st_dev = state.clone().to(DEV)
    K.gdn_conv(x.to(DEV), w.to(DEV), st_dev, _segments(K, counts, slot_of, pos0), out, bias=bias.to(DEV))
    torch.cuda.synchronize()
    r = 0
    for n, sl, p0 in zip(counts, slot_of, pos0):
        if n == 0:
            assert torch.equal(st_dev[sl].cpu(), state[sl])                   # padding segment: untouched
            continue
        y, new = eager.gdn_conv(x[r:r + n, :C], w, state[sl] if p0 > 0 else None, bias)
        assert _rel(out[r:r + n], y) < 1e-2
        assert torch.equal(st_dev[sl].cpu(), new)
        r += n


@pytest.mark.parametrize("hk,hv", [(2, 4), (1, 1), (4, 8)])
def test_gdn_delta_matches_oracle_and_chunks_compose(hk, hv):
    from cubic_serve_b200.ops import kernels as K
    g = torch.Generator().manual_seed(hk * 10 + hv)
    d, slots = 128, 4
    counts, slot_of, pos0 = [6, 1, 11], [3, 1, 0], [0, 5, 2]
    T = sum(counts)
    qkv = (torch.randn(T, (2 * hk + hv) * d, generator=g) * 0.7).to(torch.bfloat16)
    z = torch.randn(T, hv * d, generator=g).to(torch.bfloat16)
    ba = torch.randn(T, 2 * hv, generator=g).to(torch.bfloat16)
    a_log = torch.randn(hv, generator=g) * 0.5
    dt_bias = torch.randn(hv, generator=g) * 0.5
    norm_w = 1 + 0.1 * torch.randn(d, generator=g)
    state = torch.randn(slots, hv, d, d, generator=g) * 0.05
    st_dev = state.clone().to(DEV)
    out = torch.zeros(T, hv * d, dtype=torch.bfloat16, device=DEV)
    K.gdn_delta(qkv.to(DEV), z.to(DEV), ba.to(DEV), a_log.to(DEV), dt_bias.to(DEV), norm_w.to(DEV), st_dev,
                _segments(K, counts, slot_of, pos0), out, hk, hv)
    torch.cuda.synchronize()
    r = 0
    for n, sl, p0 in zip(counts, slot_of, pos0):
        want, s_new = eager.gdn_delta(qkv[r:r + n], z[r:r + n], ba[r:r + n], a_log, dt_bias, norm_w,
                                      state[sl] if p0 > 0 else None, hk, hv)
        assert _rel(out[r:r + n], want) < 2e-2
        assert _rel(st_dev[sl], s_new) < 1e-3
        r += n
    # the same rows of request 0 fed as two steps (3 + 3 rows) give the same outputs and state as one step
    st2 = torch.zeros_like(st_dev)
    out2 = torch.zeros(6, hv * d, dtype=torch.bfloat16, device=DEV)
    for lo, hi in ((0, 3), (3, 6)):
        K.gdn_delta(qkv[lo:hi].to(DEV), z[lo:hi].to(DEV), ba[lo:hi].to(DEV), a_log.to(DEV), dt_bias.to(DEV),
                    norm_w.to(DEV), st2, _segments(K, [hi - lo], [3], [lo]), out2[lo:hi], hk, hv)
    assert torch.equal(out2, out[:6]) and torch.equal(st2[3], st_dev[3])


def test_sigmoid_gate():
    from cubic_serve_b200.ops import kernels as K
    x = torch.randn(37, 256).to(torch.bfloat16).to(DEV)
    gate = torch.randn(37, 512).to(torch.bfloat16).to(DEV)[:, 256:]
    want = (x.float() * torch.sigmoid(gate.float())).to(torch.bfloat16)
    assert _rel(K.sigmoid_gate(x.clone(), gate), want) < 5e-3


def _hybrid_cfg(layers=4, interval=4):
    from cubic_serve_b200.models.config import ModelConfig, QuantSpec
    return ModelConfig(name="hybrid-toy", family="qwen3_5", num_layers=layers, hidden_size=512, num_q_heads=8, num_kv_heads=2,
                       head_dim=128, intermediate_size=1024, vocab_size=2048, rope_theta=1e6, rotary_dim=64, qk_norm=True,
                       zero_centered_norm=True, gdn_interval=interval, gdn_k_heads=2, gdn_v_heads=4, attn_output_gate=True,
                       quant=QuantSpec("cubic", 4, 128))


def _engine(cfg, graphs, chunk, seed=0, snapshots=0):
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig
    dev = torch.device("cuda")
    w = random_decoder_weights(cfg, dev, seed=seed, std=0.05)
    runner = DecoderRunner(cfg, w, num_pages=128, max_tokens=512, max_requests=8, state_checkpoints=snapshots)
    ex = GpuExecutor(runner, max_rows=8, max_prefill_tokens=512, max_model_len=256, use_graphs=graphs)
    if graphs:
        ex.capture_decode_graphs()
    eng = LLMEngine(ex, 128, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                             prefill_chunk_tokens=chunk))
    # without snapshot rows a cached prefix of a recurrent model cannot be resumed: the cache is off
    assert eng.cfg.enable_prefix_cache == bool(snapshots)
    return eng, runner


def test_hybrid_layers_match_fp32_reference():
    """Two Gated DeltaNet layers + FFN through the runner against a PyTorch forward built from the oracles."""
    import numpy as np
    from cubic_serve_b200.executor.gpu_executor import Segment
    from cubic_serve_b200.ops import wq_pack
    cfg = _hybrid_cfg(layers=2, interval=100)
    eng, runner = _engine(cfg, graphs=False, chunk=512)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg.vocab_size, 21).tolist()
    b, _ = eng.executor._fill([Segment(request_slot=3, token_ids=toks, start=0, pages=[1, 2], uid=7)])
    eng.executor.stage.upload()
    h = runner.forward_hidden(b).float().cpu()
    torch.cuda.synchronize()
    runner.ws.check_status()

    def dense(pw):
        return wq_pack.unpack_to_dense(pw).float().cpu()[:pw.n]

    bf = torch.bfloat16
    w = runner.w
    x = w.embed.float().cpu()[toks]
    for lw in w.layers:
        g = lw.gdn
        xn = eager.rmsnorm(x.to(bf), lw.ln1.cpu(), cfg.rms_eps, zero_centered=True)
        proj = (xn.float() @ dense(g.in_proj).t()).to(bf)
        C = (2 * g.hk + g.hv) * 128
        mix, _ = eager.gdn_conv(proj[:, :C], g.conv_w, None)
        ba = (xn.float() @ dense(g.in_ba).t()).to(bf)
        out, _ = eager.gdn_delta(mix, proj[:, C:C + g.hv * 128], ba, g.a_log, g.dt_bias, g.norm_w,
                                 None, g.hk, g.hv, eps_norm=cfg.rms_eps)
        x = (x + out.float() @ dense(g.out).t()).to(bf).float()
        xn = eager.rmsnorm(x.to(bf), lw.ln2.cpu(), cfg.rms_eps, zero_centered=True)
        gate_up = dense(lw.gate_up)
        if lw.gate_up.act_interleaved:
            order = wq_pack.swiglu_row_order(lw.gate_up.n // 2)
            plain = torch.empty_like(gate_up)
            plain[order] = gate_up
            gate_up = plain
        act = eager.swiglu((xn.float() @ gate_up.t()).to(bf))
        x = (x + act.float() @ dense(lw.down).t()).to(bf).float()
    assert _rel(h, x) < 3e-2


def test_hybrid_engine_chunked_prefill_and_graph_decode_agree():
    """The mixed model (3 Gated DeltaNet layers + 1 gated full-attention layer): one-shot prefill with eager decode
    against 16-token prefill chunks with CUDA-graph decode; recurrent state must carry across steps and slots."""
    import numpy as np
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    cfg = _hybrid_cfg()
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (17, 40, 33, 64, 5)]
    eng_a, run_a = _engine(cfg, graphs=False, chunk=512)
    a = eng_a.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    eng_b, run_b = _engine(cfg, graphs=True, chunk=16)
    b = eng_b.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    run_a.ws.check_status()
    run_b.ws.check_status()
    assert all(len(o) == 12 for o in b)
    agree = np.mean([x == y for pa, pb in zip(a, b) for x, y in zip(pa, pb)])
    assert agree >= 0.9, (agree, a[0], b[0])
    # a second wave of requests reuses the state slots: same prompts, same tokens
    b2 = eng_b.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert b2 == b


def test_hybrid_prefix_cache_resumes_from_a_state_snapshot():
    """With snapshot rows the prefix cache serves a recurrent model: the second request with the same prompt restores
    the Gated DeltaNet state saved at the prompt's last page boundary and computes only the tail; same tokens."""
    import numpy as np
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    cfg = _hybrid_cfg()
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg.vocab_size, 70).tolist()
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    eng, runner = _engine(cfg, graphs=True, chunk=512, snapshots=4)
    first = eng.generate([prompt], sp)[0]
    assert eng.prefix.hit_tokens == 0
    before = eng.prefill_tokens
    again = eng.generate([prompt], sp)[0]
    runner.ws.check_status()
    assert eng.prefix.hit_tokens == 64 and eng.prefill_tokens - before == 0      # the 6-token tail is a sampling segment
    assert again == first
    # another continuation of the cached 64 tokens against an engine that computes it cold
    other = prompt[:64] + rng.integers(0, cfg.vocab_size, 9).tolist()
    warm = eng.generate([other], sp)[0]
    cold_eng, cold_runner = _engine(cfg, graphs=True, chunk=512)
    cold = cold_eng.generate([other], sp)[0]
    cold_runner.ws.check_status()
    assert eng.prefix.hit_tokens == 128
    assert np.mean([a == b for a, b in zip(warm, cold)]) >= 0.8, (warm, cold)
    # two requests at once resuming from the same snapshot, beside a fresh one
    mixed = eng.generate([prompt, prompt, other[:40]], sp)
    assert mixed[0] == mixed[1]
    assert np.mean([a == b for a, b in zip(mixed[0], first)]) >= 0.8, (mixed[0], first)


def test_hybrid_model_speculates_with_the_state_folded_to_the_accepted_prefix():
    """MTP rounds on a model with Gated DeltaNet layers: the review pass leaves the recurrent state alone, the accepted
    rows are folded into it on the device.  Greedy rounds then reproduce plain greedy decoding; with every draft
    rejected or accepted at random (forced), the state must still be the one of the emitted tokens."""
    import numpy as np
    from cubic_serve_b200.executor.spec_executor import SpeculativeGpuExecutor
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.models.mtp import MtpRunner, random_mtp_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = _hybrid_cfg()
    dev = torch.device("cuda")
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (21, 40, 33)]
    sp = SamplingParams(max_tokens=14, ignore_eos=True)
    plain_eng, plain_runner = _engine(cfg, graphs=False, chunk=512)
    plain = plain_eng.generate(prompts, sp)

    def spec_engine(force):
        w = random_decoder_weights(cfg, dev, seed=0, std=0.05)
        runner = DecoderRunner(cfg, w, num_pages=128, max_tokens=512, max_requests=8)
        ex = SpeculativeGpuExecutor(runner, MtpRunner(runner, random_mtp_weights(cfg, dev, std=0.05)), 3,
                                    force_acceptance=force, max_rows=8, max_prefill_tokens=512, max_model_len=256)
        eng = LLMEngine(ex, 128, SchedulerConfig(max_running_requests=8, max_model_len=256, max_batched_tokens=512,
                                                 enable_prefix_cache=False))
        return eng, ex, runner

    eng, ex, runner = spec_engine(None)
    spec = eng.generate(prompts, sp)
    runner.ws.check_status()
    assert ex.stats["rounds"] > 0 and all(len(o) == 14 for o in spec)
    agree = np.mean([a == b for pa, pb in zip(plain, spec) for a, b in zip(pa, pb)])
    assert agree >= 0.9, (agree, plain[0], spec[0])


def test_review_pass_leaves_the_state_and_the_fold_replays_the_accepted_rows():
    """Runner level: after a prefill, four tokens are (a) consumed one decode step at a time, the recurrent state cloned
    after each, and (b) reviewed as one four-row segment without committing, then folded for 1, 2, 3 and 4 accepted
    rows: the folded state is the state (a) had after that many tokens, and the review changed nothing by itself."""
    import numpy as np
    from cubic_serve_b200.executor.gpu_executor import GpuExecutor, Segment
    from cubic_serve_b200.models.decoder import DecoderRunner, random_decoder_weights
    from cubic_serve_b200.ops import kernels as K
    cfg = _hybrid_cfg()
    dev = torch.device("cuda")
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab_size, 37).tolist()
    toks = rng.integers(0, cfg.vocab_size, 4).tolist()
    P, slot, pages = len(prompt), 2, [1, 2, 3]

    def build():
        w = random_decoder_weights(cfg, dev, seed=0, std=0.05)
        runner = DecoderRunner(cfg, w, num_pages=16, max_tokens=256, max_requests=8)
        ex = GpuExecutor(runner, max_rows=8, max_prefill_tokens=256, max_model_len=64, use_graphs=False)
        ex.execute([Segment(slot, prompt, 0, pages, True, uid=1)])
        return runner, ex

    def states(runner):
        return {li: (runner.gdn_state[li][slot].clone(), runner.gdn_conv_state[li][slot].clone()) for li in runner.gdn_state}

    r1, ex1 = build()
    after = []
    for j, t in enumerate(toks):
        ex1.execute([Segment(slot, [t], P + j, pages, True, uid=1)])
        torch.cuda.synchronize()
        after.append(states(r1))
    for accepted_rows in (1, 2, 3, 4):
        r2, ex2 = build()
        before = states(r2)
        b, _ = ex2._fill([Segment(slot, toks, P, pages, True, uid=1)])
        with torch.cuda.stream(ex2.stream):
            ex2.stage.upload()
            r2.begin_gdn_review(4)
            r2.forward_hidden(b)
            ex2.stream.synchronize()
            now = states(r2)
            assert all(torch.equal(now[li][0], before[li][0]) and torch.equal(now[li][1], before[li][1]) for li in now)
            i32 = dict(dtype=torch.int32, device=dev)
            fold = K.GdnSegments(torch.tensor([0], **i32), torch.tensor([accepted_rows], **i32),
                                 torch.tensor([slot], **i32), torch.tensor([P], **i32), 1)
            assert r2.fold_gdn(fold, 4) == 2 * len(r2.gdn_state) and r2.gdn_review is None
            ex2.stream.synchronize()
        r2.ws.check_status()
        got, want = states(r2), after[accepted_rows - 1]
        for li in got:
            assert _rel(got[li][0], want[li][0]) < 2e-2, (accepted_rows, li)
            assert _rel(got[li][1].float(), want[li][1].float()) < 2e-2, (accepted_rows, li)


def test_hybrid_moe_family_decodes_the_same_eagerly_and_in_graphs():
    """The hybrid family with routed experts (Gated DeltaNet / gated attention mixers, mixture-of-experts feed-forward):
    one-shot prefill with eager decode against chunked prefill with CUDA-graph decode."""
    import dataclasses
    import numpy as np
    from cubic_serve_b200.runtime.scheduler import SamplingParams
    cfg = dataclasses.replace(_hybrid_cfg(), name="hybrid-moe-toy", family="qwen3_5_moe", num_experts=8, experts_per_token=2,
                              moe_intermediate_size=128)
    assert cfg.is_hybrid and cfg.is_moe
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in (19, 33, 8)]
    eng_a, run_a = _engine(cfg, graphs=False, chunk=512)
    a = eng_a.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    eng_b, run_b = _engine(cfg, graphs=True, chunk=16)
    b = eng_b.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    run_a.ws.check_status()
    run_b.ws.check_status()
    assert run_b.w.layers[0].moe is not None and run_b.w.layers[0].gdn is not None and run_b.w.layers[3].gdn is None
    assert all(len(o) == 10 for o in b)
    agree = np.mean([x == y for pa, pb in zip(a, b) for x, y in zip(pa, pb)])
    assert agree >= 0.9, (agree, a[0], b[0])
