import torch

from cubic_serve_b200.guardrail.compare import DifferenceClass, compare_tensors, poisoned_padding_preserved, reduction_bound


def test_compare_classes():
    o = torch.randn(8, 16)
    assert compare_tensors(o.clone(), o, 1e-3).klass is DifferenceClass.EXACT
    b = reduction_bound(o, torch.bfloat16, 4096)
    near = o.to(torch.bfloat16).float()
    v = compare_tensors(near, o, b)
    assert v.klass is DifferenceClass.ROUNDING and v.ok and v.rel_l2 < b
    far = o.clone(); far[3, 5] += 10
    v = compare_tensors(far, o, b)
    assert v.klass is DifferenceClass.MISMATCH and v.worst_index == (3, 5) and not v.ok
    nan = o.clone(); nan[1, 2] = float("nan")
    assert compare_tensors(nan, o, b).klass is DifferenceClass.MISMATCH
    assert compare_tensors(o[:4], o, b).klass is DifferenceClass.MISMATCH
    assert poisoned_padding_preserved(o, o.clone()) and not poisoned_padding_preserved(o, far)


def test_trace_record_and_replay(tmp_path):
    """A recorded run replays token for token on a fresh engine (other prefill chunking, look-ahead launches on or
    off); a changed model is reported with the request and position of the first different token."""
    import numpy as np
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.guardrail.replay import TraceRecorder, load_trace, replay_trace
    from cubic_serve_b200.models.config import toy_config
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = toy_config()

    def engine(seed=0, chunk=64):
        return LLMEngine(EagerPagedExecutor(cfg, random_dense_weights(cfg, seed), num_pages=64), num_pages=64,
                         scheduler_config=SchedulerConfig(max_running_requests=4, max_batched_tokens=64,
                                                          prefill_chunk_tokens=chunk, max_model_len=128))

    rng = np.random.default_rng(0)
    rec = TraceRecorder(engine())
    rec.add_request(rng.integers(0, cfg.vocab_size, 21).tolist(), SamplingParams(max_tokens=6))
    rec.add_request(rng.integers(0, cfg.vocab_size, 9).tolist(), SamplingParams(max_tokens=9, temperature=0.7, top_k=8, seed=3))
    for _ in range(3):
        rec.step()
    rec.add_request(rng.integers(0, cfg.vocab_size, 33).tolist(), SamplingParams(max_tokens=4))     # arrives mid-run
    rec.run()
    path = rec.save(tmp_path / "trace.jsonl")
    trace = load_trace(path)
    assert sum(r["kind"] == "request" for r in trace) == 3 and trace[-1]["kind"] == "step"
    rep = replay_trace(path, engine())
    assert rep.ok and rep.tokens == 6 + 9 + 4, rep
    rep2 = replay_trace(trace, engine(chunk=16))                    # same tokens with 16-token prefill chunks
    assert rep2.ok
    bad = replay_trace(trace, engine(seed=1))                       # other weights: a difference is located
    assert not bad.ok and bad.first_difference["position"] >= 0 and "request_id" in bad.first_difference


def test_replay_compares_the_cache_lifecycle(tmp_path):
    """Same tokens, different cache behaviour: the lifecycle records tell a run with prefix sharing from one without,
    and a run on a smaller pool (evictions / preemptions) from the recorded one."""
    import numpy as np
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.guardrail.replay import TraceRecorder, replay_trace
    from cubic_serve_b200.models.config import toy_config
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig
    cfg = toy_config()

    def engine(prefix=True, pages=64):
        return LLMEngine(EagerPagedExecutor(cfg, random_dense_weights(cfg, 0), num_pages=pages), num_pages=pages,
                         scheduler_config=SchedulerConfig(max_running_requests=4, max_batched_tokens=64,
                                                          prefill_chunk_tokens=64, max_model_len=128,
                                                          enable_prefix_cache=prefix))
    rng = np.random.default_rng(1)
    shared = rng.integers(0, cfg.vocab_size, 40).tolist()
    rec = TraceRecorder(engine())
    rec.add_request(shared + [5, 6, 7], SamplingParams(max_tokens=4))
    rec.run()
    rec.add_request(shared + [9, 9], SamplingParams(max_tokens=4))          # resumes from the first request's pages
    rec.run()
    trace = rec.records
    steps = [r for r in trace if r["kind"] == "step"]
    admitted = {}
    for r in steps:
        admitted.update(r["lifecycle"]["admitted"])
    assert sorted(admitted.values()) == [0, 32] and steps[-1]["lifecycle"]["prefix_hit_tokens"] == 32
    assert steps[-1]["lifecycle"]["prefix_blocks"] >= 2
    assert replay_trace(trace, engine(), check_lifecycle=True).ok
    cold = replay_trace(trace, engine(prefix=False))                         # the tokens agree ...
    assert cold.ok
    cold = replay_trace(trace, engine(prefix=False), check_lifecycle=True)   # ... the cache behaviour does not
    assert not cold.ok and ("lifecycle" in cold.first_difference or "reason" in cold.first_difference)
    old = [dict(r, lifecycle=None) if r["kind"] == "step" else r for r in trace]
    rep = replay_trace(old, engine(), check_lifecycle=True)
    assert not rep.ok and "no lifecycle" in rep.first_difference["reason"]


def test_qualification_reports_compare_by_result_digest():
    import torch
    from cubic_serve_b200.guardrail.qualify import compare_reports, tensor_digest
    x = torch.arange(12, dtype=torch.float32).view(3, 4).to(torch.bfloat16)
    assert tensor_digest(x) == tensor_digest(x.clone()) and tensor_digest(x) != tensor_digest(x + 1)
    assert tensor_digest(x.t()) == tensor_digest(x.t().contiguous())                  # values, not strides
    row = lambda k, c, d, e=0.001: {"kernel": k, "shape": [4, 4], "class": c, "rel_l2": e, "digest": d}  # noqa: E731
    old = {"ok": True, "results": [row("gemm", "rounding", "aa"), row("norm", "exact", "bb"), row("attn", "rounding", "cc"),
                                   row("gone", "exact", "dd")]}
    new = {"ok": True, "results": [row("gemm", "rounding", "aa"), row("norm", "rounding", "b2", 0.002),
                                   row("attn", "mismatch", "c2", 0.5), row("fresh", "exact", "ee")]}
    d = compare_reports(old, new)
    assert d["identical"] == ["gemm [4, 4]"] and [c["check"] for c in d["changed"]] == ["norm [4, 4]"]
    assert d["regressed"] == ["attn [4, 4]"] and d["added"] == ["fresh [4, 4]"] and d["removed"] == ["gone [4, 4]"]
    assert not d["ok"]
    assert compare_reports(old, old)["ok"] and len(compare_reports(old, old)["identical"]) == 4
