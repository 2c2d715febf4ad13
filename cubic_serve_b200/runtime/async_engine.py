"""Asynchronous chat backend: HTTP event loop <-> dispatcher thread <-> engine.

Plays the role of the reference's ``TokenChatBackend`` (``runtime/token_chat.py:126``) plus the controller's
dispatcher thread (``runtime/performance.py:10519``): requests are tokenised on the event loop side, queued to
one dispatcher thread that owns the engine and steps it while work exists, and generated tokens travel back
through per-request queues with batched wake-ups (``runtime/token_stream.py:38,206``), one
``call_soon_threadsafe`` per step rather than per token.
"""
from __future__ import annotations

import asyncio
import threading
import time
from collections import deque
from dataclasses import dataclass, field

from ..api.server import ChatBackendError
from ..contracts.request import CanonicalChatRequest, RequestError, StructuredKind, TokenEvent
from ..generation.output import GenerationOutputPipeline
from ..inputs.chat import ChatInputProcessor
from .engine import EnginePoisoned, LLMEngine
from .scheduler import AdmissionError, FinishReason, SamplingParams


class TokenStream:
    """Thread -> asyncio hand-off of one request's events."""

    def __init__(self, loop: asyncio.AbstractEventLoop) -> None:
        self.loop = loop
        self._items: deque = deque()
        self._waiter: asyncio.Future | None = None
        self.closed = False

    def put_threadsafe_nowake(self, item) -> None:
        self._items.append(item)

    def wake(self) -> None:
        """Runs on the event loop thread."""
        w = self._waiter
        if w is not None and not w.done():
            w.set_result(None)

    async def get(self):
        while not self._items:
            self._waiter = self.loop.create_future()
            await self._waiter
            self._waiter = None
        return self._items.popleft()


class TokenWakeBatch:
    """Collects the streams touched by one engine step and wakes them with a single loop call-back."""

    def __init__(self) -> None:
        self._touched: dict[int, TokenStream] = {}

    def defer(self, stream: TokenStream) -> None:
        self._touched[id(stream)] = stream

    def flush(self) -> None:
        if not self._touched:
            return
        streams = list(self._touched.values())
        self._touched.clear()
        loop = streams[0].loop
        loop.call_soon_threadsafe(lambda: [s.wake() for s in streams])


@dataclass
class _Live:
    request: CanonicalChatRequest
    stream: TokenStream
    pipeline: GenerationOutputPipeline
    engine_id: str | None = None
    cancelled: bool = False
    done: bool = False


class TokenChatBackend:
    def __init__(self, engine: LLMEngine, tokenizer, default_thinking: bool | None = None,
                 reasoning_parser: bool = True, default_max_tokens: int = 1024, processor=None) -> None:
        """``processor``: the input processor (default: text only); a ``MultimodalChatProcessor`` makes the backend
        accept image and video parts."""
        self.engine = engine
        self.tokenizer = tokenizer
        self.processor = processor or ChatInputProcessor(tokenizer, default_thinking, engine.cfg.max_model_len)
        self.reasoning_parser = reasoning_parser
        self.default_max_tokens = default_max_tokens
        self.ready = True
        self._lock = threading.Lock()
        self._inbox: deque = deque()
        self._live: dict[str, _Live] = {}
        self._wake = threading.Event()
        self._stop = False
        self._thread = threading.Thread(target=self._dispatch, name="cubic-dispatcher", daemon=True)
        self._thread.start()
        self.stats = {"requests": 0, "tokens": 0, "started": time.time()}

    # ------------------------------------------------------------ front side
    def start(self, req: CanonicalChatRequest):
        if self.engine.poisoned or not self.ready:
            raise ChatBackendError(503, "the server is not ready", "service_unavailable")
        if req.structured.kind not in (StructuredKind.NONE, StructuredKind.JSON_OBJECT):
            from ..generation.constraints import constraint_supported
            if not constraint_supported(req.structured):
                raise RequestError("this structured output constraint is not available in this deployment",
                                   param="response_format")
        plan = None
        if hasattr(self.processor, "plan"):
            # prompts with media: everything but the encoding happens here; the vision tower runs on its own thread and
            # the request reaches the engine when its feature rows exist
            plan = self.processor.plan(req)
            from ..inputs.chat import PreparedInput
            prepared = PreparedInput(list(plan.token_ids), plan.prompt_text, starts_in_reasoning=plan.starts_in_reasoning)
        else:
            prepared = self.processor.build(req)
        loop = asyncio.get_running_loop()
        stream = TokenStream(loop)
        forced = req.tool_choice.name if req.tool_choice.mode == "named" else None
        pipe = GenerationOutputPipeline(
            self.tokenizer, len(prepared.token_ids), stop=req.sampling.stop,
            reasoning=self.reasoning_parser, starts_in_reasoning=prepared.starts_in_reasoning,
            tools_enabled=bool(req.tools) and req.tool_choice.mode != "none", forced_tool=forced)
        live = _Live(req, stream, pipe)
        s = req.sampling
        eos = getattr(self.tokenizer, "eos_token_id", None)
        max_tokens = s.max_tokens or self.default_max_tokens
        matcher = None
        if req.structured.kind is not StructuredKind.NONE and self.engine._mask_words and eos is not None:
            from ..generation.constraints import compile_matcher
            matcher = compile_matcher(req.structured, self.tokenizer, eos, self.engine._mask_words * 32)
            if matcher is not None and prepared.starts_in_reasoning:
                # the constraint describes the answer, not the thinking that precedes it
                from ..generation.constraints import DelayedMatcher
                end = self._reasoning_end_sequence()
                if end:
                    matcher = DelayedMatcher(matcher, end)
        sp = SamplingParams(temperature=s.temperature, top_p=s.top_p, top_k=s.top_k, seed=s.seed, max_tokens=max_tokens,
                            stop_token_ids=tuple(s.stop_token_ids) + ((eos,) if eos is not None else ()),
                            matcher=matcher,
                            thinking_budget=req.reasoning.budget_tokens if prepared.starts_in_reasoning else None)
        with self._lock:
            self._live[req.request_id] = live
            if plan is None or not plan.jobs:
                self._inbox.append((req.request_id, prepared.token_ids, sp, prepared.multimodal))
        if plan is not None and plan.jobs:
            def encoded(fut, rid=req.request_id, ids=prepared.token_ids) -> None:
                try:
                    item = self.processor.assemble(plan, fut.result())
                except BaseException as exc:  # noqa: BLE001 - handed to the request's stream by the dispatcher
                    item = exc
                with self._lock:
                    self._inbox.append((rid, ids, sp, item))
                self._wake.set()
            self.processor.submit(plan).add_done_callback(encoded)
        self._wake.set()
        return self._events(live)

    def _reasoning_end_sequence(self) -> list[int]:
        """Token ids of the marker that closes a reasoning block (empty when the tokenizer cannot encode it)."""
        if not hasattr(self, "_think_end"):
            try:
                try:
                    ids = self.tokenizer.encode("</think>", add_special_tokens=False)
                except TypeError:
                    ids = self.tokenizer.encode("</think>")
                self._think_end = [int(t) for t in ids]
            except Exception:  # noqa: BLE001 - a tokenizer without the marker leaves the constraint undelayed
                self._think_end = []
        return self._think_end

    async def _events(self, live: _Live):
        try:
            while True:
                item = await live.stream.get()
                if isinstance(item, Exception):
                    raise item
                if item is None:
                    return
                yield item
        finally:
            if not live.done:
                await self.cancel(live.request.request_id)

    async def cancel(self, request_id: str) -> None:
        with self._lock:
            live = self._live.get(request_id)
            if live is not None:
                live.cancelled = True
        self._wake.set()

    def close(self) -> None:
        self._stop = True
        self.ready = False
        self._wake.set()
        self._thread.join(timeout=10)

    # ------------------------------------------------------- dispatcher side
    def _publish(self, live: _Live, events, batch: TokenWakeBatch, end: bool = False) -> None:
        for ev in events:
            live.stream.put_threadsafe_nowake(ev)
        if end:
            live.done = True
            live.stream.put_threadsafe_nowake(None)
        batch.defer(live.stream)

    def _dispatch(self) -> None:
        batch = TokenWakeBatch()
        by_engine_id: dict[str, _Live] = {}
        while not self._stop:
            with self._lock:
                inbox = list(self._inbox)
                self._inbox.clear()
                cancelled = [l for l in self._live.values() if l.cancelled and not l.done]
            for rid, ids, sp, mm in inbox:
                live = self._live.get(rid)
                if live is None or live.cancelled:
                    continue
                try:
                    if isinstance(mm, BaseException):          # the encoder refused or failed this request's media
                        raise ValueError(str(mm)) if isinstance(mm, ValueError) else AdmissionError(
                            "the media of this request could not be encoded", status=500)
                    live.engine_id = self.engine.add_request(ids, sp, request_id=rid, multimodal=mm)
                    by_engine_id[rid] = live
                    self.stats["requests"] += 1
                    self._publish(live, live.pipeline.start_events(), batch)
                except AdmissionError as exc:
                    kind = {400: "invalid_request_error", 429: "rate_limit_exceeded"}.get(exc.status, "api_error")
                    err = ChatBackendError(exc.status, str(exc), kind)
                    live.stream.put_threadsafe_nowake(err)
                    live.done = True
                    batch.defer(live.stream)
                except (ValueError, EnginePoisoned) as exc:
                    live.stream.put_threadsafe_nowake(ChatBackendError(400 if isinstance(exc, ValueError) else 503, str(exc)))
                    live.done = True
                    batch.defer(live.stream)
            for live in cancelled:
                if live.engine_id:
                    self.engine.abort(live.engine_id)
                    by_engine_id.pop(live.engine_id, None)
                self._publish(live, live.pipeline.finish("abort"), batch, end=True)
            if not self.engine.has_unfinished:
                batch.flush()
                self._reap()
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            try:
                outs = self.engine.step()
            except Exception as exc:  # noqa: BLE001 - fail closed: every live stream gets a generic 5xx
                self.ready = False
                for live in list(by_engine_id.values()):
                    live.stream.put_threadsafe_nowake(ChatBackendError(500, "generation failed"))
                    live.done = True
                    batch.defer(live.stream)
                batch.flush()
                self._last_error = exc
                return
            # wake the streams of the PREVIOUS step only now: the next GPU step is already queued behind it
            batch.flush()
            for o in outs:
                live = by_engine_id.get(o.request_id)
                if live is None:
                    continue
                self.stats["tokens"] += o.token_id is not None
                evs = []
                hit_stop_token = o.finished and o.finish_reason is FinishReason.STOP
                if not hit_stop_token and o.token_id is not None:
                    evs = live.pipeline.feed(o.token_id)
                if live.pipeline.stopped and not o.finished:
                    self.engine.abort(o.request_id)
                    by_engine_id.pop(o.request_id, None)
                    self._publish(live, evs + live.pipeline.finish("stop"), batch, end=True)
                    continue
                if o.finished:
                    by_engine_id.pop(o.request_id, None)
                    reason = {FinishReason.STOP: "stop", FinishReason.LENGTH: "length"}.get(o.finish_reason, "stop")
                    self._publish(live, evs + live.pipeline.finish(reason), batch, end=True)
                elif evs:
                    self._publish(live, evs, batch)
            if not self.engine.has_unfinished:
                batch.flush()
        batch.flush()

    def _reap(self) -> None:
        with self._lock:
            for rid in [r for r, l in self._live.items() if l.done]:
                del self._live[rid]
