"""Wire normalisation: OpenAI ``/v1/chat/completions`` and Anthropic ``/v1/messages`` bodies -> canonical request.

Counterpart of the reference's ``inputs/normalize.py`` (``normalize_openai_chat_completions`` ``:939``,
``normalize_anthropic_messages`` ``:1186``): strict validation with client-facing messages, tools /
tool_choice / response_format / structured outputs / thinking budgets / stream options folded into one
protocol-neutral ``CanonicalChatRequest``.
"""
from __future__ import annotations

import json
import uuid
from typing import Any

from ..contracts.request import (CanonicalChatRequest, ContentPart, Message, ReasoningControl, RequestError, Role,
                                 SamplingMeta, StructuredKind, StructuredOutput, ToolCall, ToolChoice, ToolSpec)

_MAX_STOP = 16


def _require(cond: bool, message: str, param: str | None = None) -> None:
    if not cond:
        raise RequestError(message, param=param)


def _as_number(body: dict, key: str, default, lo=None, hi=None):
    v = body.get(key, default)
    if v is None:
        return default
    _require(isinstance(v, (int, float)) and not isinstance(v, bool), f"{key} must be a number", key)
    if lo is not None:
        _require(v >= lo, f"{key} must be >= {lo}", key)
    if hi is not None:
        _require(v <= hi, f"{key} must be <= {hi}", key)
    return v


def _default(defaults: dict | None, key: str, fallback):
    """The deployment's default for a sampling field (the checkpoint's ``generation_config.json``), else ``fallback``."""
    v = (defaults or {}).get(key)
    return fallback if v is None else v


def sampling_defaults_from_generation_config(path) -> dict:
    """``temperature`` / ``top_p`` / ``top_k`` of a checkpoint's ``generation_config.json`` (reference:
    ``generation/sampler.py:121``).  ``do_sample: false`` means greedy; ``top_k`` is capped at the sampler's 20; values
    out of range are ignored rather than turned into request errors for every client."""
    import json
    from pathlib import Path
    try:
        raw = json.loads(Path(path).read_text())
    except (OSError, ValueError):
        return {}
    out: dict = {}
    t, p, k = raw.get("temperature"), raw.get("top_p"), raw.get("top_k")
    if isinstance(t, (int, float)) and not isinstance(t, bool) and 0.0 <= t <= 2.0:
        out["temperature"] = float(t)
    if isinstance(p, (int, float)) and not isinstance(p, bool) and 0.0 < p <= 1.0:
        out["top_p"] = float(p)
    if isinstance(k, int) and not isinstance(k, bool) and k >= 0:
        out["top_k"] = min(20, k)
    if raw.get("do_sample") is False:
        out["temperature"] = 0.0
    return out


def _stops(v) -> tuple[str, ...]:
    if v is None:
        return ()
    if isinstance(v, str):
        v = [v]
    _require(isinstance(v, list) and all(isinstance(s, str) and s for s in v), "stop must be a string or list of strings", "stop")
    _require(len(v) <= _MAX_STOP, f"at most {_MAX_STOP} stop sequences", "stop")
    return tuple(v)


def _openai_parts(content, role: str) -> tuple[ContentPart, ...]:
    if content is None:
        return ()
    if isinstance(content, str):
        return (ContentPart("text", content),)
    _require(isinstance(content, list), f"{role} message content must be a string or a list of parts", "messages")
    parts = []
    for p in content:
        _require(isinstance(p, dict) and isinstance(p.get("type"), str), "content parts need a type", "messages")
        t = p["type"]
        if t == "text":
            _require(isinstance(p.get("text"), str), "text part needs text", "messages")
            parts.append(ContentPart("text", p["text"]))
        elif t == "image_url":
            url = (p.get("image_url") or {}).get("url") if isinstance(p.get("image_url"), dict) else p.get("image_url")
            _require(isinstance(url, str) and url, "image_url part needs a url", "messages")
            parts.append(ContentPart("image", media_url=url))
        elif t == "video_url":
            url = (p.get("video_url") or {}).get("url") if isinstance(p.get("video_url"), dict) else p.get("video_url")
            _require(isinstance(url, str) and url, "video_url part needs a url", "messages")
            parts.append(ContentPart("video", media_url=url))
        else:
            raise RequestError(f"unsupported content part type {t!r}", param="messages")
    return tuple(parts)


def _openai_tools(body: dict) -> tuple[tuple[ToolSpec, ...], ToolChoice]:
    tools = body.get("tools") or []
    _require(isinstance(tools, list), "tools must be a list", "tools")
    specs = []
    for t in tools:
        _require(isinstance(t, dict) and t.get("type") == "function" and isinstance(t.get("function"), dict),
                 "each tool must be {type: function, function: {...}}", "tools")
        fn = t["function"]
        _require(isinstance(fn.get("name"), str) and fn["name"], "tool function needs a name", "tools")
        params = fn.get("parameters")
        _require(params is None or isinstance(params, dict), "tool parameters must be a JSON schema object", "tools")
        specs.append(ToolSpec(fn["name"], fn.get("description") or "", params, bool(fn.get("strict", False))))
    names = {s.name for s in specs}
    _require(len(names) == len(specs), "tool names must be unique", "tools")
    tc = body.get("tool_choice")
    if tc is None:
        choice = ToolChoice("auto" if specs else "none")
    elif isinstance(tc, str):
        _require(tc in ("auto", "none", "required"), "tool_choice must be auto, none, required or a function", "tool_choice")
        choice = ToolChoice(tc)
    else:
        _require(isinstance(tc, dict) and tc.get("type") == "function" and isinstance(tc.get("function"), dict),
                 "tool_choice object must name a function", "tool_choice")
        name = tc["function"].get("name")
        _require(name in names, f"tool_choice names unknown tool {name!r}", "tool_choice")
        choice = ToolChoice("named", name)
    if choice.mode in ("required", "named"):
        _require(bool(specs), "tool_choice requires tools", "tool_choice")
    return tuple(specs), choice


def _openai_structured(body: dict) -> StructuredOutput:
    rf = body.get("response_format")
    so = body.get("structured_outputs")
    _require(not (rf and so), "response_format and structured_outputs are mutually exclusive", "response_format")
    if so is not None:
        _require(isinstance(so, dict) and len([k for k in so if so[k] is not None]) == 1,
                 "structured_outputs needs exactly one constraint", "structured_outputs")
        key, val = next((k, v) for k, v in so.items() if v is not None)
        mapping = {"json": StructuredKind.JSON_SCHEMA, "regex": StructuredKind.REGEX, "choice": StructuredKind.CHOICE,
                   "grammar": StructuredKind.GRAMMAR, "structural_tag": StructuredKind.STRUCTURAL_TAG}
        _require(key in mapping, f"unknown structured_outputs constraint {key!r}", "structured_outputs")
        if key == "choice":
            _require(isinstance(val, list) and val and all(isinstance(c, str) for c in val),
                     "choice must be a non-empty list of strings", "structured_outputs")
        return StructuredOutput(mapping[key], val)
    if rf is None:
        return StructuredOutput()
    _require(isinstance(rf, dict) and isinstance(rf.get("type"), str), "response_format needs a type", "response_format")
    if rf["type"] == "text":
        return StructuredOutput()
    if rf["type"] == "json_object":
        return StructuredOutput(StructuredKind.JSON_OBJECT)
    if rf["type"] == "json_schema":
        js = rf.get("json_schema")
        _require(isinstance(js, dict) and isinstance(js.get("schema"), dict), "json_schema needs a schema object",
                 "response_format")
        return StructuredOutput(StructuredKind.JSON_SCHEMA, js["schema"], js.get("name"), bool(js.get("strict", False)))
    raise RequestError(f"unsupported response_format type {rf['type']!r}", param="response_format")


def normalize_openai_chat_completions(body: Any, default_model: str | None = None,
                                      sampling_defaults: dict | None = None) -> CanonicalChatRequest:
    _require(isinstance(body, dict), "request body must be a JSON object")
    model = body.get("model") or default_model
    _require(isinstance(model, str) and model, "model is required", "model")
    raw = body.get("messages")
    _require(isinstance(raw, list) and raw, "messages must be a non-empty list", "messages")
    messages = []
    for m in raw:
        _require(isinstance(m, dict) and isinstance(m.get("role"), str), "each message needs a role", "messages")
        role = m["role"]
        if role == "developer":
            role = "system"
        _require(role in ("system", "user", "assistant", "tool"), f"unknown role {m['role']!r}", "messages")
        calls = []
        if role == "assistant" and m.get("tool_calls"):
            _require(isinstance(m["tool_calls"], list), "tool_calls must be a list", "messages")
            for c in m["tool_calls"]:
                fn = c.get("function") if isinstance(c, dict) else None
                _require(isinstance(fn, dict) and isinstance(fn.get("name"), str), "tool_calls entries need a function",
                         "messages")
                args = fn.get("arguments", "{}")
                calls.append(ToolCall(str(c.get("id") or f"call_{uuid.uuid4().hex[:24]}"), fn["name"],
                                      args if isinstance(args, str) else json.dumps(args)))
        if role == "tool":
            _require(isinstance(m.get("tool_call_id"), str), "tool messages need tool_call_id", "messages")
        messages.append(Message(Role(role), _openai_parts(m.get("content"), role), tuple(calls), m.get("tool_call_id"),
                                m.get("name")))
    n = body.get("n", 1)
    _require(n == 1, "only n = 1 is supported", "n")
    max_tokens = body.get("max_completion_tokens", body.get("max_tokens"))
    _require(max_tokens is None or (isinstance(max_tokens, int) and not isinstance(max_tokens, bool)),
             "max_tokens must be an integer", "max_tokens")
    stream = bool(body.get("stream", False))
    so = body.get("stream_options") or {}
    _require(isinstance(so, dict), "stream_options must be an object", "stream_options")
    _require(not so or stream, "stream_options requires stream = true", "stream_options")
    seed = body.get("seed")
    _require(seed is None or (isinstance(seed, int) and not isinstance(seed, bool)), "seed must be an integer", "seed")
    tlp = body.get("top_logprobs") or 0
    _require(isinstance(tlp, int) and 0 <= tlp <= 20, "top_logprobs must be in [0, 20]", "top_logprobs")
    sampling = SamplingMeta(
        temperature=float(_as_number(body, "temperature", _default(sampling_defaults, "temperature", 1.0))),
        top_p=float(_as_number(body, "top_p", _default(sampling_defaults, "top_p", 1.0))),
        top_k=int(_as_number(body, "top_k", _default(sampling_defaults, "top_k", 0))),
        seed=seed, max_tokens=max_tokens, stop=_stops(body.get("stop")),
        stop_token_ids=tuple(int(t) for t in (body.get("stop_token_ids") or [])),
        presence_penalty=float(_as_number(body, "presence_penalty", 0.0, -2.0, 2.0)),
        frequency_penalty=float(_as_number(body, "frequency_penalty", 0.0, -2.0, 2.0)),
        logprobs=bool(body.get("logprobs", False)), top_logprobs=tlp)
    tools, choice = _openai_tools(body)
    structured = _openai_structured(body)
    _require(not (structured.kind != StructuredKind.NONE and choice.mode in ("required", "named")),
             "forced tool calls cannot be combined with a structured output constraint", "tool_choice")
    kw = body.get("chat_template_kwargs") or {}
    _require(isinstance(kw, dict), "chat_template_kwargs must be an object", "chat_template_kwargs")
    enabled = kw.get("enable_thinking")
    effort = body.get("reasoning_effort")
    _require(effort in (None, "none", "low", "medium", "high"), "reasoning_effort must be none, low, medium or high",
             "reasoning_effort")
    if effort == "none":
        enabled = False
    budget = body.get("thinking_token_budget")
    _require(budget is None or (isinstance(budget, int) and budget >= 0), "thinking_token_budget must be >= 0",
             "thinking_token_budget")
    return CanonicalChatRequest(
        protocol="openai", model=model, messages=tuple(messages), sampling=sampling, stream=stream,
        include_usage=bool(so.get("include_usage", False)), tools=tools, tool_choice=choice, structured=structured,
        reasoning=ReasoningControl(enabled if isinstance(enabled, bool) else None, budget, effort),
        user=body.get("user") if isinstance(body.get("user"), str) else None,
        request_id=f"chatcmpl-{uuid.uuid4().hex}", template_kwargs=tuple(sorted(kw.items())))


def _anthropic_parts(content, role: str):
    parts, calls, results = [], [], []
    if isinstance(content, str):
        return (ContentPart("text", content),), (), ()
    _require(isinstance(content, list) and content, "message content must be a string or a non-empty list", "messages")
    for b in content:
        _require(isinstance(b, dict) and isinstance(b.get("type"), str), "content blocks need a type", "messages")
        t = b["type"]
        if t == "text":
            _require(isinstance(b.get("text"), str), "text block needs text", "messages")
            parts.append(ContentPart("text", b["text"]))
        elif t == "image":
            src = b.get("source")
            _require(isinstance(src, dict), "image block needs a source", "messages")
            if src.get("type") == "base64":
                url = f"data:{src.get('media_type', 'image/png')};base64,{src.get('data', '')}"
            else:
                url = src.get("url")
            _require(isinstance(url, str) and url, "image source needs data or url", "messages")
            parts.append(ContentPart("image", media_url=url))
        elif t == "tool_use":
            _require(role == "assistant", "tool_use blocks belong to assistant messages", "messages")
            calls.append(ToolCall(str(b.get("id")), str(b.get("name")), json.dumps(b.get("input") or {})))
        elif t == "tool_result":
            _require(role == "user", "tool_result blocks belong to user messages", "messages")
            c = b.get("content", "")
            if isinstance(c, list):
                c = "".join(x.get("text", "") for x in c if isinstance(x, dict) and x.get("type") == "text")
            results.append((str(b.get("tool_use_id")), str(c)))
        elif t in ("thinking", "redacted_thinking"):
            continue
        else:
            raise RequestError(f"unsupported content block type {t!r}", param="messages")
    return tuple(parts), tuple(calls), tuple(results)


def normalize_anthropic_messages(body: Any, default_model: str | None = None,
                                 sampling_defaults: dict | None = None) -> CanonicalChatRequest:
    _require(isinstance(body, dict), "request body must be a JSON object")
    model = body.get("model") or default_model
    _require(isinstance(model, str) and model, "model is required", "model")
    max_tokens = body.get("max_tokens")
    _require(isinstance(max_tokens, int) and not isinstance(max_tokens, bool) and max_tokens >= 1,
             "max_tokens is required and must be a positive integer", "max_tokens")
    messages = []
    system = body.get("system")
    if system:
        if isinstance(system, list):
            system = "".join(b.get("text", "") for b in system if isinstance(b, dict) and b.get("type") == "text")
        _require(isinstance(system, str), "system must be a string or a list of text blocks", "system")
        messages.append(Message(Role.SYSTEM, (ContentPart("text", system),)))
    raw = body.get("messages")
    _require(isinstance(raw, list) and raw, "messages must be a non-empty list", "messages")
    for m in raw:
        _require(isinstance(m, dict) and m.get("role") in ("user", "assistant"), "message role must be user or assistant",
                 "messages")
        parts, calls, results = _anthropic_parts(m.get("content"), m["role"])
        for tid, text in results:
            messages.append(Message(Role.TOOL, (ContentPart("text", text),), tool_call_id=tid))
        if parts or calls or not results:
            messages.append(Message(Role(m["role"]), parts, calls))
    tools = []
    for t in body.get("tools") or []:
        _require(isinstance(t, dict) and isinstance(t.get("name"), str), "each tool needs a name", "tools")
        schema = t.get("input_schema")
        _require(schema is None or isinstance(schema, dict), "input_schema must be an object", "tools")
        tools.append(ToolSpec(t["name"], t.get("description") or "", schema))
    tc = body.get("tool_choice")
    choice = ToolChoice("auto" if tools else "none")
    if tc is not None:
        _require(isinstance(tc, dict) and tc.get("type") in ("auto", "any", "tool", "none"), "invalid tool_choice",
                 "tool_choice")
        if tc["type"] == "any":
            choice = ToolChoice("required")
        elif tc["type"] == "tool":
            _require(tc.get("name") in {t.name for t in tools}, "tool_choice names an unknown tool", "tool_choice")
            choice = ToolChoice("named", tc["name"])
        else:
            choice = ToolChoice(tc["type"])
    thinking = body.get("thinking")
    reasoning = ReasoningControl()
    if thinking is not None:
        _require(isinstance(thinking, dict) and thinking.get("type") in ("enabled", "disabled"), "invalid thinking block",
                 "thinking")
        if thinking["type"] == "enabled":
            b = thinking.get("budget_tokens")
            _require(isinstance(b, int) and b >= 0, "thinking.budget_tokens must be a non-negative integer", "thinking")
            _require(b < max_tokens, "thinking.budget_tokens must be below max_tokens", "thinking")
            reasoning = ReasoningControl(True, b)
        else:
            reasoning = ReasoningControl(False)
    sampling = SamplingMeta(
        temperature=float(_as_number(body, "temperature", min(1.0, _default(sampling_defaults, "temperature", 1.0)), 0.0, 1.0)),
        top_p=float(_as_number(body, "top_p", _default(sampling_defaults, "top_p", 1.0))),
        top_k=min(20, int(_as_number(body, "top_k", _default(sampling_defaults, "top_k", 0), 0))),
        max_tokens=max_tokens, stop=_stops(body.get("stop_sequences")))
    return CanonicalChatRequest(
        protocol="anthropic", model=model, messages=tuple(messages), sampling=sampling,
        stream=bool(body.get("stream", False)), include_usage=True, tools=tuple(tools), tool_choice=choice,
        reasoning=reasoning, request_id=f"msg_{uuid.uuid4().hex[:24]}")
