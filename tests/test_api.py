"""HTTP layer: normalisation, projections, SSE framing, auth, strict JSON, cancellation (fake + real backends)."""
import asyncio
import json

import pytest

from cubic_serve_b200.api.projections import (fold_events, project_anthropic_message, project_anthropic_message_stream,
                                              project_openai_chat_completion, project_openai_chat_completion_stream)
from cubic_serve_b200.api.server import CubicASGIApp, ChatBackendError, decode_strict_json
from cubic_serve_b200.contracts.request import EventKind, RequestError, TokenEvent, Usage
from cubic_serve_b200.inputs.normalize import normalize_anthropic_messages, normalize_openai_chat_completions


def _events():
    return [TokenEvent(EventKind.START, usage=Usage(7, 0)), TokenEvent(EventKind.REASONING, "hm"),
            TokenEvent(EventKind.CONTENT, "Hel"), TokenEvent(EventKind.CONTENT, "lo"),
            TokenEvent(EventKind.TOOL_CALL_START, tool_index=0, tool_id="call_1", tool_name="f"),
            TokenEvent(EventKind.TOOL_CALL_ARGS, '{"a":', tool_index=0), TokenEvent(EventKind.TOOL_CALL_ARGS, "1}", tool_index=0),
            TokenEvent(EventKind.FINISH, finish_reason="tool_calls", usage=Usage(7, 5, 0, 1))]


def test_normalize_openai_full():
    req = normalize_openai_chat_completions({
        "model": "m", "messages": [{"role": "developer", "content": "sys"},
                                   {"role": "user", "content": [{"type": "text", "text": "hi"}]},
                                   {"role": "assistant", "content": None, "tool_calls": [
                                       {"id": "c1", "type": "function", "function": {"name": "f", "arguments": "{}"}}]},
                                   {"role": "tool", "tool_call_id": "c1", "content": "42"}],
        "temperature": 0.5, "top_p": 0.9, "top_k": 5, "max_completion_tokens": 9, "stop": "END", "stream": True,
        "stream_options": {"include_usage": True}, "seed": 3,
        "tools": [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}],
        "tool_choice": {"type": "function", "function": {"name": "f"}},
        "chat_template_kwargs": {"enable_thinking": False}})
    assert req.messages[0].role.value == "system" and req.messages[1].text == "hi"
    assert req.messages[2].tool_calls[0].name == "f" and req.messages[3].tool_call_id == "c1"
    assert req.sampling.top_k == 5 and req.sampling.max_tokens == 9 and req.sampling.stop == ("END",)
    assert req.stream and req.include_usage and req.tool_choice.mode == "named" and req.reasoning.enabled is False


@pytest.mark.parametrize("body,param", [
    ({"model": "m", "messages": []}, "messages"),
    ({"model": "m", "messages": [{"role": "user", "content": "x"}], "temperature": 3}, "temperature"),
    ({"model": "m", "messages": [{"role": "user", "content": "x"}], "top_k": 21}, "top_k"),
    ({"model": "m", "messages": [{"role": "user", "content": "x"}], "n": 2}, "n"),
    ({"model": "m", "messages": [{"role": "user", "content": "x"}], "stream_options": {"include_usage": True}}, "stream_options"),
    ({"model": "m", "messages": [{"role": "user", "content": "x"}], "tool_choice": "required"}, "tool_choice"),
    ({"model": "m", "messages": [{"role": "user", "content": "x"}], "response_format": {"type": "json_schema"}}, "response_format"),
    ({"model": "m", "messages": [{"role": "bogus", "content": "x"}]}, "messages"),
])
def test_normalize_openai_rejects(body, param):
    with pytest.raises(RequestError) as e:
        normalize_openai_chat_completions(body)
    assert e.value.param == param


def test_normalize_anthropic():
    req = normalize_anthropic_messages({
        "model": "m", "max_tokens": 100, "system": [{"type": "text", "text": "be brief"}],
        "messages": [{"role": "user", "content": "q"},
                     {"role": "assistant", "content": [{"type": "tool_use", "id": "t1", "name": "f", "input": {"x": 1}}]},
                     {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "t1", "content": "r"}]}],
        "tools": [{"name": "f", "input_schema": {"type": "object"}}], "tool_choice": {"type": "any"},
        "thinking": {"type": "enabled", "budget_tokens": 50}, "stop_sequences": ["X"], "stream": True})
    roles = [m.role.value for m in req.messages]
    assert roles == ["system", "user", "assistant", "tool"]
    assert req.tool_choice.mode == "required" and req.reasoning.budget_tokens == 50 and req.sampling.stop == ("X",)
    with pytest.raises(RequestError):
        normalize_anthropic_messages({"model": "m", "messages": [{"role": "user", "content": "q"}]})
    with pytest.raises(RequestError):
        normalize_anthropic_messages({"model": "m", "max_tokens": 10, "messages": [{"role": "user", "content": "q"}],
                                      "thinking": {"type": "enabled", "budget_tokens": 10}})


def test_projections_roundtrip():
    req = normalize_openai_chat_completions({"model": "m", "messages": [{"role": "user", "content": "x"}], "stream": True,
                                             "stream_options": {"include_usage": True}})
    full = project_openai_chat_completion(req, _events())
    msg = full["choices"][0]["message"]
    assert msg["content"] == "Hello" and msg["reasoning_content"] == "hm"
    assert msg["tool_calls"][0]["function"] == {"name": "f", "arguments": '{"a":1}'}
    assert full["choices"][0]["finish_reason"] == "tool_calls" and full["usage"]["total_tokens"] == 12
    chunks = list(project_openai_chat_completion_stream(req, _events()))
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"]) == "Hello"
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 5
    areq = normalize_anthropic_messages({"model": "m", "max_tokens": 5, "messages": [{"role": "user", "content": "x"}]})
    amsg = project_anthropic_message(areq, _events())
    assert [b["type"] for b in amsg["content"]] == ["thinking", "text", "tool_use"]
    assert amsg["content"][2]["input"] == {"a": 1} and amsg["stop_reason"] == "tool_use"
    names = [n for n, _ in project_anthropic_message_stream(areq, _events())]
    assert names[0] == "message_start" and names[-2:] == ["message_delta", "message_stop"]
    assert names.count("content_block_start") == 3 == names.count("content_block_stop")
    assert fold_events(_events()).usage.reasoning_tokens == 1


def test_strict_json():
    assert decode_strict_json(b'{"a": 1}') == {"a": 1}
    for bad in (b'{"a": 1, "a": 2}', b'{"a": NaN}', b'{"a": Infinity}', b"\xff", b"{"):
        with pytest.raises(ValueError):
            decode_strict_json(bad)


class ScriptedBackend:
    ready = True

    def __init__(self, events=None, error=None, hang=False):
        self.events, self.error, self.hang = events or _events(), error, hang
        self.cancelled = []

    def start(self, req):
        if isinstance(self.error, RequestError):
            raise self.error

        async def gen():
            if self.error:
                raise self.error
            for ev in self.events:
                yield ev
                if self.hang:
                    await asyncio.sleep(3600)
        return gen()

    async def cancel(self, rid):
        self.cancelled.append(rid)


async def _call(app, method, path, body=None, headers=None, disconnect_after=None):
    sent = []
    raw = json.dumps(body).encode() if body is not None else b""
    state = {"sent_body": False}
    gate = asyncio.Event()

    async def receive():
        if not state["sent_body"]:
            state["sent_body"] = True
            return {"type": "http.request", "body": raw, "more_body": False}
        if disconnect_after is not None:
            await gate.wait()
            return {"type": "http.disconnect"}
        await asyncio.sleep(3600)

    async def send(msg):
        sent.append(msg)
        if disconnect_after is not None and sum(1 for m in sent if m["type"] == "http.response.body") >= disconnect_after:
            gate.set()

    scope = {"type": "http", "method": method, "path": path,
             "headers": [(k.encode(), v.encode()) for k, v in (headers or {}).items()]}
    try:
        await asyncio.wait_for(app(scope, receive, send), timeout=5)
    except asyncio.TimeoutError:
        pass
    status = sent[0]["status"] if sent else None
    payload = b"".join(m.get("body", b"") for m in sent if m["type"] == "http.response.body")
    return status, payload


def test_server_routes_auth_errors():
    app = CubicASGIApp(ScriptedBackend(), "model-x", api_key="secret")
    run = asyncio.run
    assert run(_call(app, "GET", "/health"))[0] == 200
    assert run(_call(app, "GET", "/v1/models"))[0] == 401
    st, body = run(_call(app, "GET", "/v1/models", headers={"authorization": "Bearer secret"}))
    assert st == 200 and json.loads(body)["data"][0]["id"] == "model-x"
    assert run(_call(app, "GET", "/v1/models", headers={"x-api-key": "wrong"}))[0] == 401
    h = {"x-api-key": "secret"}
    ok = {"model": "model-x", "messages": [{"role": "user", "content": "hi"}]}
    st, body = run(_call(app, "POST", "/v1/chat/completions", ok, h))
    assert st == 200 and json.loads(body)["choices"][0]["message"]["content"] == "Hello"
    assert run(_call(app, "POST", "/v1/chat/completions", {**ok, "model": "other"}, h))[0] == 404
    assert run(_call(app, "POST", "/v1/chat/completions", {**ok, "temperature": 9}, h))[0] == 400
    assert run(_call(app, "GET", "/v1/chat/completions", None, h))[0] == 405
    assert run(_call(app, "GET", "/nope", None, h))[0] == 404
    assert run(_call(app, "GET", "/metrics"))[0] == 401                      # metrics sit behind the key too
    st, body = run(_call(app, "GET", "/metrics", None, h))
    assert st == 200 and b'cubic_ready{model="model-x"} 1' in body
    st, body = run(_call(app, "POST", "/v1/messages", {"model": "model-x", "max_tokens": 5,
                                                       "messages": [{"role": "user", "content": "hi"}]}, h))
    assert st == 200 and json.loads(body)["type"] == "message"
    busy = CubicASGIApp(ScriptedBackend(error=ChatBackendError(429, "at capacity", "rate_limit_exceeded")), "model-x")
    st, body = run(_call(busy, "POST", "/v1/chat/completions", ok))
    assert st == 429 and json.loads(body)["error"]["message"] == "at capacity"
    st, body = run(_call(busy, "POST", "/v1/chat/completions", {**ok, "stream": True}))
    assert st == 429
    down = ScriptedBackend()
    down.ready = False
    assert run(_call(CubicASGIApp(down, "model-x"), "GET", "/health"))[0] == 503


def test_server_sse_streams_and_disconnect_cancels():
    app = CubicASGIApp(ScriptedBackend(), "model-x")
    body = {"model": "model-x", "messages": [{"role": "user", "content": "hi"}], "stream": True}
    st, payload = asyncio.run(_call(app, "POST", "/v1/chat/completions", body))
    frames = [f for f in payload.decode().split("\n\n") if f]
    assert st == 200 and frames[-1] == "data: [DONE]" and all(f.startswith("data: ") for f in frames)
    text = "".join(json.loads(f[6:])["choices"][0]["delta"].get("content", "") for f in frames[:-1])
    assert text == "Hello"
    st, payload = asyncio.run(_call(app, "POST", "/v1/messages", {"model": "model-x", "max_tokens": 5, "stream": True,
                                                                   "messages": [{"role": "user", "content": "hi"}]}))
    assert st == 200 and payload.decode().startswith("event: message_start\ndata: ")
    assert "event: message_stop" in payload.decode()
    hang = ScriptedBackend(hang=True)
    asyncio.run(_call(CubicASGIApp(hang, "model-x"), "POST", "/v1/chat/completions", body, disconnect_after=1))
    assert len(hang.cancelled) >= 1


def test_real_backend_end_to_end_on_cpu():
    """Byte tokenizer + toy decoder through the async backend and the ASGI app."""
    from cubic_serve_b200.executor.eager_executor import EagerPagedExecutor
    from cubic_serve_b200.inputs.chat import ByteTokenizer
    from cubic_serve_b200.models.config import ModelConfig
    from cubic_serve_b200.models.reference import random_dense_weights
    from cubic_serve_b200.runtime.async_engine import TokenChatBackend
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SchedulerConfig

    tok = ByteTokenizer()
    cfg = ModelConfig(num_layers=1, hidden_size=64, num_q_heads=2, num_kv_heads=1, head_dim=32, intermediate_size=128,
                      vocab_size=tok.vocab_size)
    eng = LLMEngine(EagerPagedExecutor(cfg, random_dense_weights(cfg, 0), 64), 64,
                    SchedulerConfig(max_running_requests=4, max_model_len=512, max_batched_tokens=256))

    async def go():
        backend = TokenChatBackend(eng, tok, default_max_tokens=8)
        app = CubicASGIApp(backend, "toy")
        body = {"model": "toy", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0}
        r1, r2, r3 = await asyncio.gather(
            _call(app, "POST", "/v1/chat/completions", body),
            _call(app, "POST", "/v1/chat/completions", {**body, "stream": True, "stream_options": {"include_usage": True}}),
            _call(app, "POST", "/v1/messages", {**body, "max_tokens": 4}))
        m = await _call(app, "GET", "/metrics")
        backend.close()
        return r1, r2, r3, m

    (s1, b1), (s2, b2), (s3, b3), (sm, bm) = asyncio.run(go())
    assert s1 == s2 == s3 == sm == 200
    metrics = {l.split(" ")[0]: float(l.split(" ")[1]) for l in bm.decode().splitlines() if l and not l.startswith("#")}
    assert metrics['cubic_requests_total{model="toy"}'] == 3 and metrics['cubic_generated_tokens_total{model="toy"}'] == 16
    assert metrics['cubic_ready{model="toy"}'] == 1 and metrics['cubic_requests_running{model="toy"}'] == 0
    assert "# TYPE cubic_kv_cache_usage_ratio gauge" in bm.decode()
    j1 = json.loads(b1)
    assert j1["usage"]["completion_tokens"] == 6 and j1["choices"][0]["finish_reason"] == "length"
    frames = [f for f in b2.decode().split("\n\n") if f]
    assert frames[-1] == "data: [DONE]" and json.loads(frames[-2][6:])["usage"]["completion_tokens"] == 6
    streamed = "".join(json.loads(f[6:])["choices"][0]["delta"].get("content", "") for f in frames[:-2] if json.loads(f[6:])["choices"])
    assert streamed == (j1["choices"][0]["message"]["content"] or "")        # greedy: same text both ways
    assert json.loads(b3)["usage"]["output_tokens"] == 4
    assert eng.pool.num_used == len(eng.prefix)


def test_sampling_defaults_from_generation_config(tmp_path):
    from cubic_serve_b200.inputs.normalize import (normalize_anthropic_messages, normalize_openai_chat_completions,
                                                   sampling_defaults_from_generation_config)
    f = tmp_path / "generation_config.json"
    f.write_text(json.dumps({"temperature": 0.6, "top_p": 0.95, "top_k": 50, "do_sample": True, "eos_token_id": [1, 2]}))
    d = sampling_defaults_from_generation_config(f)
    assert d == {"temperature": 0.6, "top_p": 0.95, "top_k": 20}                     # top_k capped at the sampler's limit
    body = {"model": "m", "messages": [{"role": "user", "content": "hi"}]}
    r = normalize_openai_chat_completions(body, "m", d)
    assert (r.sampling.temperature, r.sampling.top_p, r.sampling.top_k) == (0.6, 0.95, 20)
    r = normalize_openai_chat_completions({**body, "temperature": 0.1, "top_k": 5}, "m", d)   # the request wins
    assert (r.sampling.temperature, r.sampling.top_p, r.sampling.top_k) == (0.1, 0.95, 5)
    assert normalize_openai_chat_completions(body, "m").sampling.temperature == 1.0
    a = normalize_anthropic_messages({**body, "max_tokens": 8}, "m", d)
    assert (a.sampling.temperature, a.sampling.top_k) == (0.6, 20)
    f.write_text(json.dumps({"do_sample": False, "temperature": 5.0, "top_p": 0}))
    assert sampling_defaults_from_generation_config(f) == {"temperature": 0.0}        # greedy; out-of-range values ignored
    assert sampling_defaults_from_generation_config(tmp_path / "missing.json") == {}
    app = CubicASGIApp(ScriptedBackend(), "model-x", sampling_defaults=d)
    assert app.sampling_defaults["top_p"] == 0.95
