"""Generated-token post-processing: incremental detokenisation, reasoning / content / tool-call split, stops.

Counterpart of the reference's ``generation/output.py`` (``GenerationOutputPipeline`` ``:463``,
``TokenPhaseOutputParser`` ``:230``) and ``generation/tool_output.py``: tokens come in one at a time, text
goes out as canonical ``TokenEvent``s as soon as it is unambiguous (a partial UTF-8 sequence, a possible
prefix of a stop string or of a control tag is held back).
"""
from __future__ import annotations

import json
import uuid
from dataclasses import dataclass, field

from ..contracts.request import EventKind, TokenEvent, Usage

THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
TOOL_OPEN, TOOL_CLOSE = "<tool_call>", "</tool_call>"


class IncrementalDetokenizer:
    """Decode a growing id sequence, emitting only text that later tokens cannot change."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True, window: int = 6) -> None:
        self.tok = tokenizer
        self.skip = skip_special_tokens
        self.ids: list[int] = []
        self.prefix_offset = 0
        self.read_offset = 0
        self.window = window

    def _decode(self, ids) -> str:
        try:
            return self.tok.decode(ids, skip_special_tokens=self.skip)
        except TypeError:
            return self.tok.decode(ids)

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        prefix = self._decode(self.ids[self.prefix_offset:self.read_offset])
        full = self._decode(self.ids[self.prefix_offset:])
        if len(full) > len(prefix) and not full.endswith("�"):
            new = full[len(prefix):]
            self.prefix_offset = max(self.read_offset - self.window, self.prefix_offset)
            # keep a few tokens of left context so that merges across the boundary decode the same
            self.prefix_offset = self.read_offset
            self.read_offset = len(self.ids)
            return new
        return ""

    def flush(self) -> str:
        prefix = self._decode(self.ids[self.prefix_offset:self.read_offset])
        full = self._decode(self.ids[self.prefix_offset:])
        self.read_offset = len(self.ids)
        return full[len(prefix):] if len(full) > len(prefix) else ""


def _held_suffix(text: str, needles: tuple[str, ...]) -> int:
    """Length of the longest suffix of ``text`` that is a proper prefix of any needle."""
    best = 0
    for n in needles:
        for k in range(min(len(n) - 1, len(text)), 0, -1):
            if text.endswith(n[:k]):
                best = max(best, k)
                break
    return best


@dataclass
class _ToolState:
    index: int = -1
    buffer: str = ""


class GenerationOutputPipeline:
    """tokens -> TokenEvents for one request."""

    def __init__(self, tokenizer, prompt_tokens: int, stop: tuple[str, ...] = (), reasoning: bool = False,
                 starts_in_reasoning: bool = False, tools_enabled: bool = False, cached_tokens: int = 0,
                 forced_tool: str | None = None) -> None:
        self.detok = IncrementalDetokenizer(tokenizer)
        self.stop = tuple(stop)
        self.reasoning_enabled = reasoning
        self.in_reasoning = starts_in_reasoning
        self.tools_enabled = tools_enabled
        self.prompt_tokens = prompt_tokens
        self.cached_tokens = cached_tokens
        self.completion_tokens = 0
        self.reasoning_tokens = 0
        self.pending = ""
        self.tool = _ToolState()
        self.in_tool = False
        self.saw_tool_call = False
        self.stopped = False
        self.started = False
        self.forced_tool = forced_tool
        if forced_tool:
            # forced tool call: the whole completion is the JSON arguments object
            self.in_tool = True

    # ------------------------------------------------------------------
    def start_events(self) -> list[TokenEvent]:
        self.started = True
        evs = [TokenEvent(EventKind.START, usage=Usage(self.prompt_tokens, 0, self.cached_tokens))]
        if self.forced_tool:
            self.tool.index = 0
            self.saw_tool_call = True
            evs.append(TokenEvent(EventKind.TOOL_CALL_START, tool_index=0, tool_id=f"call_{uuid.uuid4().hex[:24]}",
                                  tool_name=self.forced_tool))
        return evs

    def feed(self, token_id: int) -> list[TokenEvent]:
        """Consume one generated token; returns events and sets ``stopped`` when a stop string completed."""
        if self.stopped:
            return []
        self.completion_tokens += 1
        if self.in_reasoning:
            self.reasoning_tokens += 1
        text = self.detok.push(token_id)
        return self._consume(text, final=False) if text else []

    def finish(self, reason: str) -> list[TokenEvent]:
        evs = []
        if not self.stopped:
            evs.extend(self._consume(self.detok.flush(), final=True))
        if self.saw_tool_call and reason == "stop":
            reason = "tool_calls"
        evs.append(TokenEvent(EventKind.FINISH, finish_reason=reason,
                              usage=Usage(self.prompt_tokens, self.completion_tokens, self.cached_tokens,
                                          self.reasoning_tokens), token_count=self.completion_tokens))
        return evs

    # ------------------------------------------------------------------
    def _emit(self, text: str) -> list[TokenEvent]:
        if not text:
            return []
        if self.forced_tool:
            return [TokenEvent(EventKind.TOOL_CALL_ARGS, text=text, tool_index=0)]
        return [TokenEvent(EventKind.REASONING if self.in_reasoning else EventKind.CONTENT, text=text)]

    def _consume(self, text: str, final: bool) -> list[TokenEvent]:
        self.pending += text
        evs: list[TokenEvent] = []
        while True:
            if self.in_tool and not self.forced_tool:
                end = self.pending.find(TOOL_CLOSE)
                if end < 0:
                    if final:
                        evs.extend(self._finish_tool(self.pending))
                        self.pending = ""
                    return evs
                evs.extend(self._finish_tool(self.pending[:end]))
                self.pending = self.pending[end + len(TOOL_CLOSE):]
                self.in_tool = False
                continue
            # earliest control marker in the pending text
            markers = []
            if self.reasoning_enabled:
                markers.append(THINK_CLOSE if self.in_reasoning else THINK_OPEN)
            if self.tools_enabled and not self.in_reasoning and not self.forced_tool:
                markers.append(TOOL_OPEN)
            stops = self.stop if not self.in_reasoning else ()
            hit_pos, hit = -1, None
            for mk in (*markers, *stops):
                p = self.pending.find(mk)
                if p >= 0 and (hit_pos < 0 or p < hit_pos):
                    hit_pos, hit = p, mk
            if hit is None:
                hold = 0 if final else _held_suffix(self.pending, (*markers, *stops))
                out, self.pending = self.pending[:len(self.pending) - hold], self.pending[len(self.pending) - hold:]
                evs.extend(self._emit(out))
                return evs
            evs.extend(self._emit(self.pending[:hit_pos]))
            self.pending = self.pending[hit_pos + len(hit):]
            if hit in stops:
                self.stopped = True
                self.pending = ""
                return evs
            if hit == THINK_OPEN:
                self.in_reasoning = True
            elif hit == THINK_CLOSE:
                self.in_reasoning = False
                self.pending = self.pending.lstrip("\n")
            elif hit == TOOL_OPEN:
                self.in_tool = True

    def _finish_tool(self, body: str) -> list[TokenEvent]:
        body = body.strip()
        name, args = "", body
        try:
            obj = json.loads(body)
            if isinstance(obj, dict):
                name = str(obj.get("name", ""))
                a = obj.get("arguments", obj.get("parameters", {}))
                args = a if isinstance(a, str) else json.dumps(a, ensure_ascii=False)
        except ValueError:
            pass
        self.tool.index += 1
        self.saw_tool_call = True
        idx = self.tool.index
        return [TokenEvent(EventKind.TOOL_CALL_START, tool_index=idx, tool_id=f"call_{uuid.uuid4().hex[:24]}", tool_name=name),
                TokenEvent(EventKind.TOOL_CALL_ARGS, text=args, tool_index=idx)]
