import argparse
import json

import pytest

from cubic_serve_b200 import cli
from cubic_serve_b200.models.config import dense_8b_config
from cubic_serve_b200.runtime.serving import plan_kv_pages


def test_serve_flag_surface():
    a = cli.build_parser().parse_args([
        "serve", "random:toy", "--devices", "0-3", "--tp-size", "4", "--k-cache-dtype", "int4", "--v-cache-dtype", "int8",
        "--no-prefix-cache", "--max-running-requests", "64", "--speculative-config",
        '{"method":"mtp","num_speculative_tokens":3,"mode":"dynamic"}', "--api-key", "k", "--no-thinking"])
    assert cli.parse_devices(a.devices) == [0, 1, 2, 3] and a.tp_size == 4 and a.prefix_cache is False
    assert a.thinking is False and a.k_cache_dtype == "int4"
    spec = cli.parse_speculative_config(a.speculative_config)
    assert (spec.method, spec.num_speculative_tokens, spec.mode) == ("mtp", 3, "dynamic")
    cli.validate_topology([0, 1, 2, 3], 4, 1, 2, cli.SpeculativeConfig())
    cli.validate_topology([0], 1, 1, 1, spec)
    with pytest.raises(SystemExit):                      # rounds run in the single-process executor only
        cli.validate_topology([0, 1, 2, 3], 4, 1, 2, spec)
    ngram = cli.parse_speculative_config('{"method":"ngram","num_speculative_tokens":4}')
    assert (ngram.method, ngram.num_speculative_tokens, ngram.mode) == ("ngram", 4, "fixed")
    with pytest.raises(argparse.ArgumentTypeError):
        cli.parse_speculative_config('{"method":"ngram","num_speculative_tokens":4,"mode":"dynamic"}')


@pytest.mark.parametrize("text", ['{"method":"eagle"}', '{"method":"mtp","num_speculative_tokens":9}', "not json",
                                  '{"method":"mtp","num_speculative_tokens":2,"mode":"x"}'])
def test_bad_speculative_config(text):
    with pytest.raises(argparse.ArgumentTypeError):
        cli.parse_speculative_config(text)


def test_topology_rules():
    none = cli.SpeculativeConfig()
    with pytest.raises(SystemExit):
        cli.validate_topology([0, 1], 2, 3, 1, none)
    with pytest.raises(SystemExit):
        cli.validate_topology([0, 1, 2], 2, 1, 1, none)
    with pytest.raises(SystemExit):
        cli.validate_topology([0, 1, 2, 3], 4, 1, 3, none)
    with pytest.raises(SystemExit):
        cli.validate_topology([0, 1, 2, 3], 2, 2, 1, cli.SpeculativeConfig("mtp", 2))
    assert cli.parse_devices("0,2,5") == [0, 2, 5] and cli.parse_devices("4..7") == [4, 5, 6, 7]
    with pytest.raises(argparse.ArgumentTypeError):
        cli.parse_devices("1,1")


def test_kv_page_planning():
    cfg = dense_8b_config()
    pages = plan_kv_pages(100 << 30, 4 << 30, cfg, 1, 8, 8, 2048, 256)
    per_page = 36 * 8 * 4608
    assert pages == min((96 << 30) // per_page, 256 * 128 + 64)
    assert plan_kv_pages(100 << 30, 4 << 30, cfg, 8, 4, 8, 2048, 256) == 256 * 128 + 64


def test_trace_record_and_replay_between_two_schedules(tmp_path, capsys):
    """``cubic trace``: a trace recorded with four request slots replays token for token on an engine with two."""
    trace = tmp_path / "t.jsonl"
    assert cli.main(["trace", "record", str(trace), "random:toy", "--requests", "5", "--max-tokens", "5",
                     "--serve-args", "--execution-mode eager --max-running-requests 4"]) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["tokens"] == 25 and trace.exists()
    assert cli.main(["trace", "replay", str(trace), "random:toy",
                     "--serve-args", "--execution-mode eager --max-running-requests 2"]) == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["ok"] and rep["tokens"] == 25 and rep["first_difference"] is None
    # a trace that another model produced does not replay: the first difference is located
    lines = trace.read_text().splitlines()
    doctored = []
    for line in lines:
        r = json.loads(line)
        if r["kind"] == "step" and r["emitted"]:
            rid = next(iter(r["emitted"]))
            r["emitted"][rid][0] = (r["emitted"][rid][0] + 1) % 200
            doctored.append(json.dumps(r))
            doctored += lines[len(doctored):]
            break
        doctored.append(line)
    trace.write_text("\n".join(doctored) + "\n")
    assert cli.main(["trace", "replay", str(trace), "random:toy", "--serve-args", "--execution-mode eager"]) == 1
    diff = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["first_difference"]
    assert diff["position"] == 0 and "request_id" in diff


def test_reference_subcommand_decodes_a_written_checkpoint(tmp_path, capsys):
    """``cubic reference``: the eager fp32 decoder on a checkpoint's decoded weights; the eager serving mode loads the
    same weights (``--execution-mode eager`` with a checkpoint directory)."""
    import json

    from cubic_serve_b200 import cli
    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models.config import ModelConfig, QuantSpec
    from cubic_serve_b200.models.reference import EagerDecoder, dense_weights_from_checkpoint
    cfg = ModelConfig(name="tiny", num_layers=2, hidden_size=256, num_q_heads=4, num_kv_heads=2, head_dim=128,
                      intermediate_size=512, vocab_size=320, qk_norm=True, quant=QuantSpec("int", 4, 128))
    path = C.write_random_checkpoint(tmp_path / "ck", cfg, seed=1)
    assert cli.main(["reference", str(path), "--prompt-ids", "1,2,3,4", "--max-tokens", "5"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["prompt_ids"] == [1, 2, 3, 4] and len(out["output_ids"]) == 5
    import torch
    dense = dense_weights_from_checkpoint(C.admit_checkpoint(path))
    tokens, _ = EagerDecoder(cfg, dense).generate(torch.tensor([[1, 2, 3, 4]]), 5)
    assert out["output_ids"] == [int(t) for t in tokens[0]]


def test_wna8_compute_mode_is_refused_not_ignored():
    import pytest

    from cubic_serve_b200 import cli
    with pytest.raises(SystemExit, match="wna8"):
        cli.main(["serve", "random:toy", "--compute-mode", "wna8"])


def test_reference_flag_spellings_are_accepted():
    """Flags of the reference's CLI that name the same thing here parse under their own names too."""
    from cubic_serve_b200.cli import build_parser
    p = build_parser()
    a = p.parse_args(["serve", "random:toy", "--served-model-name", "a", "b", "--allowed-local-media-path", "/srv/m",
                      "--multimodal-memory-gib", "3", "--mm-feature-cache-gib", "0.5", "--mm-preprocess-workers", "4",
                      "--video-max-frames", "64", "--video-fps", "1", "--mamba-ssm-cache-dtype", "float32",
                      "--softmax-dtype", "fp32", "--device", "0"])
    assert a.served_model_name == ["a", "b"] and a.media_file_root == ["/srv/m"] and a.encoder_memory_gib == 3.0
    assert a.mm_feature_cache_gib == 0.5 and a.recurrent_state_dtype == "float32" and a.softmax_dtype == "fp32"
    r = p.parse_args(["reference", "random:toy", "--input-ids", "1,2", "--max-new-tokens", "3"])
    assert r.prompt_ids == "1,2" and r.max_tokens == 3
    import pytest
    with pytest.raises(SystemExit):
        p.parse_args(["--version"])


def test_several_served_names_are_accepted_by_the_server():
    import asyncio
    import json

    from test_api import ScriptedBackend, _call

    from cubic_serve_b200.api.server import CubicASGIApp
    app = CubicASGIApp(ScriptedBackend(), "ckpt", ["public", "alias"])
    body = {"messages": [{"role": "user", "content": "x"}], "max_tokens": 2}
    for name, want in (("public", 200), ("alias", 200), ("ckpt", 200), ("other", 404)):
        st, payload = asyncio.run(_call(app, "POST", "/v1/chat/completions", {**body, "model": name}))
        assert st == want, (name, st, payload[:120])
        if want == 200:
            assert json.loads(payload)["model"] == "public"


def test_qualify_operators_needs_no_gpu(capsys):
    import json
    assert cli.main(["qualify", "--operators", "--quick"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["ok"] and report["checks"] == 18 and report["failed"] == []
