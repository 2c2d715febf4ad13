"""Multi-GPU paths on real GPUs (skipped below two devices): logits of the fused NVLink path, the NCCL baseline and one
GPU holding the whole model agree within the reduction bound; pipeline stages give the one-GPU tokens."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, module, *args, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", "29671", "-m", module, *args]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert lines, out.stdout[-2000:] + out.stderr[-2000:]
    return json.loads(lines[-1])


def _ranks():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else (2 if n >= 2 else 0))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("model,extra", [("dense-8b", []), ("moe-30b-a3b", ["--experts", "32", "--kv", "4,8"]),
                                         # two key/value heads: on four or more ranks neighbours cache copies of a head
                                         ("moe-30b-a3b", ["--experts", "32", "--kv", "4,8", "--kv-heads", "2"])])
def test_fused_and_nccl_tensor_parallel_logits_match_one_gpu(model, extra):
    rep = _torchrun(_ranks(), "cubic_serve_b200.parallel.tp_check", "--model", model, "--layers", "4", *extra)
    assert rep["ranks_agree"]
    one = rep["vs_one_gpu"]
    if model.startswith("moe"):
        # discrete routing: a row that rounding noise hands another expert moves far; most rows must not
        assert rep["p50_rel_logit_err"] <= rep["bound"] and rep["rows_within_bound"] >= 0.75, rep
        assert one["p50_rel_logit_err"] <= one["bound"] and one["rows_within_bound"] >= 0.75, rep
        assert rep["fused_eq_nccl_tokens"] >= 0.75 and one["token_agreement"] >= 0.75, rep
    else:
        assert rep["max_rel_logit_err"] <= rep["bound"], rep
        assert one["max_rel_logit_err"] <= one["bound"], rep
        assert rep["fused_eq_nccl_tokens"] >= 0.9 and one["token_agreement"] >= 0.9, rep


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_pipeline_stages_give_the_one_gpu_tokens():
    from cubic_serve_b200.parallel import pp_check
    one = pp_check.main(["--pp", "1"])
    two = _torchrun(2, "cubic_serve_b200.parallel.pp_check", "--pp", "2")
    assert two["tokens"] == one["tokens"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_mtp_rounds_under_tensor_parallelism_emit_the_one_gpu_greedy_tokens():
    rep = _torchrun(2, "cubic_serve_b200.parallel.spec_check", "--depth", "3")
    assert rep["rounds"] > 0 and rep["lengths_ok"]
    assert rep["token_agreement_with_plain_greedy"] >= 0.9, rep
