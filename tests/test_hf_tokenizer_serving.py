"""The serving path with a HuggingFace tokenizer and its chat template in the checkpoint directory: ``AutoTokenizer`` is
loaded, the template renders the prompt (with ``enable_thinking``), the checkpoint's ``generation_config.json`` gives the
sampling defaults, and a completion streams back as text."""
import asyncio
import json
from argparse import Namespace
from dataclasses import replace

import pytest

TEMPLATE = (
    "{%- for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{%- endfor %}"
    "{%- if add_generation_prompt %}<|im_start|>assistant\n{%- if enable_thinking is defined and enable_thinking is false %}"
    "<think>\n\n</think>\n\n{%- endif %}{%- endif %}")


def _tokenizer(path):
    tokenizers = pytest.importorskip("tokenizers")
    transformers = pytest.importorskip("transformers")
    from tokenizers import models, pre_tokenizers, decoders
    words = ["hello", "world", "tell", "me", "a", "story", "please", "system", "user", "assistant", "be", "brief", "the", "of"]
    specials = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>"]
    alphabet = [chr(c) for c in range(32, 127)] + ["\n"]
    vocab = {t: i for i, t in enumerate(specials + alphabet + words)}
    tok = tokenizers.Tokenizer(models.WordLevel(vocab, unk_token="?"))
    tok.pre_tokenizer = pre_tokenizers.Split(tokenizers.Regex(r"[a-z]+|[\s\S]"), behavior="isolated")
    tok.decoder = decoders.Fuse()
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<|im_end|>", pad_token="<|endoftext|>",
                                                additional_special_tokens=specials)
    fast.chat_template = TEMPLATE
    fast.save_pretrained(str(path))
    return fast


def test_checkpoint_with_a_tokenizer_serves_chat(tmp_path):
    from test_api import _call

    from cubic_serve_b200.api.server import CubicASGIApp
    from cubic_serve_b200.inputs.normalize import sampling_defaults_from_generation_config
    from cubic_serve_b200.models import checkpoint as C
    from cubic_serve_b200.models.config import ModelConfig, QuantSpec
    from cubic_serve_b200.runtime.serving import build_backend
    cfg = replace(ModelConfig(), qk_norm=True, vocab_size=256, quant=QuantSpec("cubic", 4, 128), name="Qwen3ForCausalLM")
    path = C.write_random_checkpoint(tmp_path / "ck", cfg, seed=3, std=0.08)
    tok = _tokenizer(path)
    assert len(tok) <= 256
    (path / "generation_config.json").write_text(json.dumps({"temperature": 0.7, "top_p": 0.8, "top_k": 20, "do_sample": True}))
    args = Namespace(model=str(path), execution_mode="eager", pp_size=1, seed=0, max_model_len=256, max_running_requests=4,
                     token_budget=128, prefill_chunk_tokens=64, prefix_cache=True, thinking=None, served_model_name=None)
    backend, name = build_backend(args, [0], 1, None, 8, 8)
    assert type(backend.tokenizer).__name__.startswith("PreTrainedTokenizer") or hasattr(backend.tokenizer, "apply_chat_template")
    defaults = sampling_defaults_from_generation_config(path / "generation_config.json")
    assert defaults == {"temperature": 0.7, "top_p": 0.8, "top_k": 20}

    async def go():
        app = CubicASGIApp(backend, name, sampling_defaults=defaults)
        body = {"model": name, "max_tokens": 6, "temperature": 0,
                "messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "tell me a story please"}]}
        plain = await _call(app, "POST", "/v1/chat/completions", body)
        stream = await _call(app, "POST", "/v1/chat/completions", {**body, "stream": True})
        nothink = await _call(app, "POST", "/v1/chat/completions", {**body, "chat_template_kwargs": {"enable_thinking": False}})
        backend.close()
        return plain, stream, nothink
    (s1, b1), (s2, b2), (s3, b3) = asyncio.run(go())
    assert s1 == s2 == s3 == 200
    j1, j3 = json.loads(b1), json.loads(b3)
    # the template rendered the prompt: system + user turn + generation prompt, tokenized by the checkpoint's tokenizer
    want = tok.apply_chat_template([{"role": "system", "content": "be brief"}, {"role": "user", "content": "tell me a story please"}],
                                   tokenize=False, add_generation_prompt=True)
    assert j1["usage"]["prompt_tokens"] == len(tok.encode(want, add_special_tokens=False))
    assert j3["usage"]["prompt_tokens"] > j1["usage"]["prompt_tokens"]          # the closed thinking block was appended
    assert j1["usage"]["completion_tokens"] <= 6 and j1["choices"][0]["finish_reason"] in ("length", "stop")
    frames = [f for f in b2.decode().split("\n\n") if f.startswith("data: ") and f != "data: [DONE]"]
    streamed = "".join((json.loads(f[6:])["choices"][0]["delta"].get("content") or "") +
                       (json.loads(f[6:])["choices"][0]["delta"].get("reasoning_content") or "")
                       for f in frames if json.loads(f[6:])["choices"])
    msg = j1["choices"][0]["message"]
    assert streamed == (msg.get("reasoning_content") or "") + (msg.get("content") or "")
