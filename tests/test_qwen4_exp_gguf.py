"""qwen4exp GGUF files: what the exporter's layout stores, and the round trip back to the logical tensors."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from cubic_serve_b200.models import qwen4_exp as Q
from cubic_serve_b200.models import qwen4_exp_gguf as G


def test_round_trip_and_the_exporters_conventions(tmp_path):
    import gguf
    cfg = Q.tiny_config()
    w = Q.random_qwen4_exp_weights(cfg, 4, std=0.1)
    path = G.export_qwen4_exp_gguf(tmp_path / "m.gguf", cfg, w)
    reader = gguf.GGUFReader(str(path))
    stored = {t.name: (tuple(int(x) for x in reversed(t.shape)), np.asarray(t.data)) for t in reader.tensors}
    # what the file holds: stacked experts per projection, two indexer projections, ONE lexical table, 1 + w norms,
    # negative decays, value heads regrouped
    assert stored["blk.0.ffn_gate_exps.weight"][0] == (8, 16, 32) and stored["blk.0.ffn_down_exps.weight"][0] == (8, 32, 16)
    assert stored["blk.1.indexer.q_proj.weight"][0] == (32, 32) and stored["blk.1.indexer.k_proj.weight"][0] == (16, 32)
    assert stored["per_layer_token_embd.weight"][0] == (4 * 512, 8)
    assert not any(n.startswith("blk.1.ple") and "shard" in n for n in stored)
    p0 = "model.language_model.layers.0.linear_attn"
    a = stored["blk.0.ssm_a"][1].reshape(-1)
    assert (a < 0).all()
    order = G.value_head_order(cfg.gdn_k_heads, cfg.gdn_v_heads, 1)
    assert np.allclose(np.log(-a)[order], w[p0 + ".A_log"].numpy(), atol=1e-6)
    qn = stored["blk.1.attn_q_norm.weight"][1].reshape(-1)
    assert np.allclose(qn - 1, w["model.language_model.layers.1.self_attn.q_norm.weight"].numpy(), atol=1e-6)
    gn = stored["blk.0.ssm_norm.weight"][1].reshape(-1)
    assert np.allclose(gn, w[p0 + ".norm.weight"].numpy(), atol=1e-6)              # the DeltaNet output norm is stored as is
    z = stored["blk.0.attn_gate.weight"][1].reshape(stored["blk.0.attn_gate.weight"][0])
    vals = G.value_head_order(cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_v_dim)
    assert np.allclose(z[vals], w[p0 + ".in_proj_z.weight"].numpy(), atol=1e-6) and not np.allclose(z, z[vals])
    # and back
    got_cfg, got = G.load_qwen4_exp_gguf(path)
    assert got_cfg.layer_types == cfg.layer_types and got_cfg.mrope_section == cfg.mrope_section
    assert (got_cfg.ngram_split_parts, got_cfg.ngram_shard_rows) == (1, 2048) and got_cfg.ple_layer_ids == (2,)
    table = torch.cat([w[f"model.language_model.layers.1.ple.ple_embedding.ngram_embedding.shard_{i}.weight"] for i in range(4)])
    for name, t in got.items():
        if "ngram_embedding.shard_0" in name:
            assert torch.allclose(t, table, atol=1e-6)
        else:
            assert t.shape == w[name].shape and torch.allclose(t.float(), w[name].float(), atol=1e-5), name
    assert set(got) == {n for n in w if "ngram_embedding.shard_" not in n or n.endswith("shard_0.weight")}
    # the same logits from the file as from the tensors it was written from
    toks = list(range(3, 30))
    want, _ = Q.Qwen4ExpModel(cfg, w).forward(toks)
    have, _ = Q.Qwen4ExpModel(got_cfg, got).forward(toks)
    assert (want - have).abs().max() < 1e-4


def test_value_head_order_is_the_inverse_of_the_exporters_grouping():
    order = G.value_head_order(2, 6, 1)                     # 2 key heads, 3 value heads each
    assert order.tolist() == [0, 2, 4, 1, 3, 5]            # stored [v0k0 v0k1 v1k0 v1k1 v2k0 v2k1] -> logical k-major
    wide = G.value_head_order(2, 4, 3)
    assert wide[:6].tolist() == [0, 1, 2, 6, 7, 8]


def test_files_with_stray_or_missing_tensors_are_refused(tmp_path):
    import gguf
    cfg = replace(Q.tiny_config(), ple_layer_ids=())
    w = Q.random_qwen4_exp_weights(cfg, 5)
    good = G.export_qwen4_exp_gguf(tmp_path / "ok.gguf", cfg, w)
    got_cfg, got = G.load_qwen4_exp_gguf(good)
    assert got_cfg.ple_layer_ids == () and len(got) == len(w)
    missing = {k: v for k, v in w.items() if not k.endswith("layers.0.linear_attn.dt_bias")}
    with pytest.raises(KeyError):
        G.export_qwen4_exp_gguf(tmp_path / "never.gguf", cfg, {"lm_head.weight": w["lm_head.weight"]})
    bad = G.export_qwen4_exp_gguf(tmp_path / "missing.gguf", cfg, missing)
    with pytest.raises(Q.Qwen4ExpConfigError, match="missing tensor blk.0.ssm_dt.bias"):
        G.load_qwen4_exp_gguf(bad)
    wr = gguf.GGUFWriter(str(tmp_path / "other.gguf"), "llama")
    wr.add_tensor("token_embd.weight", np.zeros((4, 8), np.float32))
    wr.write_header_to_file(); wr.write_kv_data_to_file(); wr.write_tensors_to_file(); wr.close()
    with pytest.raises(Q.Qwen4ExpConfigError, match="architecture"):
        G.load_qwen4_exp_gguf(tmp_path / "other.gguf")


def test_serving_backend_from_a_gguf_file(tmp_path):
    from argparse import Namespace

    from cubic_serve_b200.runtime.serving import build_backend
    cfg = Q.tiny_config()
    path = G.export_qwen4_exp_gguf(tmp_path / "serve.gguf", cfg, Q.random_qwen4_exp_weights(cfg, 6))
    args = Namespace(model=str(path), execution_mode="eager", pp_size=1, seed=0, max_model_len=128, max_running_requests=2,
                     token_budget=64, prefill_chunk_tokens=32, prefix_cache=True, thinking=None, served_model_name=None)
    backend, name = build_backend(args, [0], 1, None, 8, 8)
    assert name == "qwen4exp" and backend.engine.executor.cfg.num_layers == cfg.num_layers
    backend.close()
