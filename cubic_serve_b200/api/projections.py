"""Fold canonical ``TokenEvent`` streams into OpenAI and Anthropic wire objects.

Counterpart of the reference's ``api/_events.py:151`` (``fold_events``),
``api/openai.py:54,88`` and ``api/anthropic.py:42,59``: the same event sequence
renders as a non-streaming response body or as the protocol's SSE chunk
sequence.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Iterable, Iterator

from ..contracts.request import CanonicalChatRequest, EventKind, TokenEvent, Usage


@dataclass
class FoldedToolCall:
    id: str
    name: str
    arguments: str = ""


@dataclass
class Folded:
    content: str = ""
    reasoning: str = ""
    tool_calls: list[FoldedToolCall] = field(default_factory=list)
    finish_reason: str | None = None
    usage: Usage = field(default_factory=Usage)


def fold_events(events: Iterable[TokenEvent]) -> Folded:
    out = Folded()
    for ev in events:
        if ev.kind is EventKind.CONTENT:
            out.content += ev.text
        elif ev.kind is EventKind.REASONING:
            out.reasoning += ev.text
        elif ev.kind is EventKind.TOOL_CALL_START:
            out.tool_calls.append(FoldedToolCall(ev.tool_id, ev.tool_name))
        elif ev.kind is EventKind.TOOL_CALL_ARGS:
            out.tool_calls[ev.tool_index].arguments += ev.text
        elif ev.kind is EventKind.FINISH:
            out.finish_reason = ev.finish_reason
            if ev.usage is not None:
                out.usage = ev.usage
    return out


# ------------------------------------------------------------------ OpenAI
def _openai_usage(u: Usage) -> dict:
    d = {"prompt_tokens": u.prompt_tokens, "completion_tokens": u.completion_tokens,
         "total_tokens": u.prompt_tokens + u.completion_tokens,
         "prompt_tokens_details": {"cached_tokens": u.cached_tokens}}
    if u.reasoning_tokens:
        d["completion_tokens_details"] = {"reasoning_tokens": u.reasoning_tokens}
    return d


def project_openai_chat_completion(req: CanonicalChatRequest, events: Iterable[TokenEvent], created: int | None = None) -> dict:
    f = fold_events(events)
    msg: dict = {"role": "assistant", "content": f.content if (f.content or not f.tool_calls) else None}
    if f.reasoning:
        msg["reasoning_content"] = f.reasoning
    if f.tool_calls:
        msg["tool_calls"] = [{"id": c.id, "type": "function", "function": {"name": c.name, "arguments": c.arguments}}
                             for c in f.tool_calls]
    return {"id": req.request_id, "object": "chat.completion", "created": created or int(time.time()),
            "model": req.model,
            "choices": [{"index": 0, "message": msg, "finish_reason": f.finish_reason or "stop", "logprobs": None}],
            "usage": _openai_usage(f.usage)}


def project_openai_chat_completion_stream(req: CanonicalChatRequest, events: Iterable[TokenEvent],
                                          created: int | None = None) -> Iterator[dict]:
    """Yield ``chat.completion.chunk`` objects (the caller frames them as SSE and appends ``[DONE]``)."""
    created = created or int(time.time())
    base = {"id": req.request_id, "object": "chat.completion.chunk", "created": created, "model": req.model}

    def chunk(delta: dict, finish: str | None = None) -> dict:
        c = dict(base)
        c["choices"] = [{"index": 0, "delta": delta, "finish_reason": finish, "logprobs": None}]
        return c

    for ev in events:
        if ev.kind is EventKind.START:
            yield chunk({"role": "assistant", "content": ""})
        elif ev.kind is EventKind.CONTENT:
            if ev.text:
                yield chunk({"content": ev.text})
        elif ev.kind is EventKind.REASONING:
            if ev.text:
                yield chunk({"reasoning_content": ev.text})
        elif ev.kind is EventKind.TOOL_CALL_START:
            yield chunk({"tool_calls": [{"index": ev.tool_index, "id": ev.tool_id, "type": "function",
                                         "function": {"name": ev.tool_name, "arguments": ""}}]})
        elif ev.kind is EventKind.TOOL_CALL_ARGS:
            if ev.text:
                yield chunk({"tool_calls": [{"index": ev.tool_index, "function": {"arguments": ev.text}}]})
        elif ev.kind is EventKind.FINISH:
            yield chunk({}, ev.finish_reason or "stop")
            if req.include_usage and ev.usage is not None:
                u = dict(base)
                u["choices"] = []
                u["usage"] = _openai_usage(ev.usage)
                yield u


# --------------------------------------------------------------- Anthropic
_ANTHROPIC_STOP = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use", "abort": "end_turn",
                   "stop_sequence": "stop_sequence"}


def _anthropic_usage(u: Usage) -> dict:
    return {"input_tokens": u.prompt_tokens, "output_tokens": u.completion_tokens,
            "cache_read_input_tokens": u.cached_tokens, "cache_creation_input_tokens": 0}


def _parse_args(text: str):
    try:
        v = json.loads(text) if text.strip() else {}
        return v if isinstance(v, dict) else {"value": v}
    except ValueError:
        return {"_raw": text}


def project_anthropic_message(req: CanonicalChatRequest, events: Iterable[TokenEvent]) -> dict:
    f = fold_events(events)
    content: list[dict] = []
    if f.reasoning:
        content.append({"type": "thinking", "thinking": f.reasoning, "signature": ""})
    if f.content:
        content.append({"type": "text", "text": f.content})
    for c in f.tool_calls:
        content.append({"type": "tool_use", "id": c.id, "name": c.name, "input": _parse_args(c.arguments)})
    return {"id": req.request_id, "type": "message", "role": "assistant", "model": req.model, "content": content,
            "stop_reason": _ANTHROPIC_STOP.get(f.finish_reason or "stop", "end_turn"), "stop_sequence": None,
            "usage": _anthropic_usage(f.usage)}


class AnthropicStreamProjector:
    """Incremental Anthropic streaming state machine: ``push(event)`` returns the ``(event name, data)`` frames."""

    def __init__(self, req: CanonicalChatRequest) -> None:
        self.req = req
        self.index = -1
        self.open_kind: str | None = None

    def _close(self, out: list) -> None:
        if self.open_kind is not None:
            self.open_kind = None
            out.append(("content_block_stop", {"type": "content_block_stop", "index": self.index}))

    def push(self, ev: TokenEvent) -> list[tuple[str, dict]]:
        out: list[tuple[str, dict]] = []
        req = self.req
        if ev.kind is EventKind.START:
            out.append(("message_start", {"type": "message_start", "message": {
                "id": req.request_id, "type": "message", "role": "assistant", "model": req.model, "content": [],
                "stop_reason": None, "stop_sequence": None, "usage": _anthropic_usage(ev.usage or Usage())}}))
            return out
        if ev.kind is EventKind.FINISH:
            self._close(out)
            u = ev.usage or Usage()
            out.append(("message_delta", {"type": "message_delta", "delta": {
                "stop_reason": _ANTHROPIC_STOP.get(ev.finish_reason or "stop", "end_turn"), "stop_sequence": None},
                "usage": {"output_tokens": u.completion_tokens}}))
            out.append(("message_stop", {"type": "message_stop"}))
            return out
        want = {EventKind.CONTENT: "text", EventKind.REASONING: "thinking", EventKind.TOOL_CALL_START: "tool_use",
                EventKind.TOOL_CALL_ARGS: "tool_use"}[ev.kind]
        if ev.kind is EventKind.TOOL_CALL_START or self.open_kind != want:
            self._close(out)
            self.index += 1
            self.open_kind = want
            block = {"text": {"type": "text", "text": ""}, "thinking": {"type": "thinking", "thinking": ""},
                     "tool_use": {"type": "tool_use", "id": ev.tool_id, "name": ev.tool_name, "input": {}}}[want]
            out.append(("content_block_start", {"type": "content_block_start", "index": self.index, "content_block": block}))
            if ev.kind is EventKind.TOOL_CALL_START:
                return out
        if ev.text:
            delta = {"text": {"type": "text_delta", "text": ev.text},
                     "thinking": {"type": "thinking_delta", "thinking": ev.text},
                     "tool_use": {"type": "input_json_delta", "partial_json": ev.text}}[want]
            out.append(("content_block_delta", {"type": "content_block_delta", "index": self.index, "delta": delta}))
        return out


def project_anthropic_message_stream(req: CanonicalChatRequest, events: Iterable[TokenEvent]) -> Iterator[tuple[str, dict]]:
    """Yield ``(event name, data)`` pairs of the Anthropic streaming protocol."""
    proj = AnthropicStreamProjector(req)
    for ev in events:
        yield from proj.push(ev)
