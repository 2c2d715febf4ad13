"""Dependency-free ASGI application: OpenAI and Anthropic compatible streaming HTTP.

Same surface as the reference's ``CubicASGIApp`` (``api/server.py:686-822``):
``POST /v1/chat/completions``, ``POST /v1/messages``, ``GET /v1/models``,
``GET /health``; Bearer / ``x-api-key`` authentication with a constant-time
digest comparison; strict JSON (duplicate keys and NaN/Infinity rejected); a
64 MiB body limit; a disconnect watcher that cancels the generation; SSE
framing; an error taxonomy whose public messages never leak internals.
Run it with any ASGI server (``uvicorn``).
"""
from __future__ import annotations

import asyncio
import hashlib
import hmac
import json
import math
import time
from typing import Any, AsyncIterator, Protocol

from ..contracts.request import CanonicalChatRequest, EventKind, RequestError, TokenEvent
from ..inputs.normalize import normalize_anthropic_messages, normalize_openai_chat_completions
from .projections import (AnthropicStreamProjector, project_anthropic_message, project_openai_chat_completion,
                          project_openai_chat_completion_stream)

MAX_BODY_BYTES = 64 * 1024 * 1024


class ChatBackendError(RuntimeError):
    """Raised by a backend with an HTTP status and a reviewed public message."""

    def __init__(self, status: int, public_message: str, code: str = "server_error") -> None:
        super().__init__(public_message)
        self.status, self.public_message, self.code = status, public_message, code


class ChatBackend(Protocol):
    ready: bool

    def start(self, request: CanonicalChatRequest) -> AsyncIterator[TokenEvent]: ...

    async def cancel(self, request_id: str) -> None: ...


class _StrictJSONError(ValueError):
    pass


def _reject_constant(name: str):
    raise _StrictJSONError(f"non-finite number {name} is not valid JSON")


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise _StrictJSONError(f"duplicate key {k!r}")
        out[k] = v
    return out


def decode_strict_json(raw: bytes) -> Any:
    try:
        text = raw.decode("utf-8")
    except UnicodeDecodeError as exc:
        raise _StrictJSONError("body is not valid UTF-8") from exc
    try:
        value = json.loads(text, object_pairs_hook=_no_duplicates, parse_constant=_reject_constant)
    except _StrictJSONError:
        raise
    except ValueError as exc:
        raise _StrictJSONError("body is not valid JSON") from exc
    return value


def _error_body(protocol: str, status: int, message: str, code: str, param: str | None = None) -> dict:
    if protocol == "anthropic":
        kind = {400: "invalid_request_error", 401: "authentication_error", 404: "not_found_error",
                413: "request_too_large", 429: "rate_limit_error", 503: "overloaded_error"}.get(status, "api_error")
        return {"type": "error", "error": {"type": kind, "message": message}}
    return {"error": {"message": message, "type": code, "param": param, "code": status}}


def render_metrics(backend, model: str) -> str:
    """Engine and scheduler counters in the Prometheus text exposition format (``GET /metrics``, behind the API key
    like every route but ``/health``).  Reads plain counters: no lock is taken and no step is delayed."""
    label = '{model="%s"}' % model.replace("\\", "\\\\").replace('"', '\\"')
    rows: list[tuple[str, str, str, float]] = []
    engine = getattr(backend, "engine", None)
    served = getattr(backend, "stats", None) or {}
    rows.append(("cubic_ready", "gauge", "1 when the backend accepts requests", 1.0 if getattr(backend, "ready", True) else 0.0))
    if isinstance(served, dict):
        rows.append(("cubic_requests_total", "counter", "requests admitted", float(served.get("requests", 0))))
        rows.append(("cubic_streamed_tokens_total", "counter", "tokens handed to response streams", float(served.get("tokens", 0))))
    if engine is not None:
        s = engine.stats()
        for key, name, kind, text in (
                ("running", "cubic_requests_running", "gauge", "requests in the running batch"),
                ("waiting", "cubic_requests_waiting", "gauge", "requests waiting for admission"),
                ("kv_used_frac", "cubic_kv_cache_usage_ratio", "gauge", "fraction of KV pages in use"),
                ("prefix_hit_rate", "cubic_prefix_cache_hit_ratio", "gauge", "prompt tokens served from cached pages"),
                ("steps", "cubic_engine_steps_total", "counter", "engine steps"),
                ("generated_tokens", "cubic_generated_tokens_total", "counter", "tokens sampled"),
                ("prefill_tokens", "cubic_prefill_tokens_total", "counter", "prompt tokens computed")):
            if key in s:
                rows.append((name, kind, text, float(s[key])))
        rows.append(("cubic_last_step_seconds", "gauge", "host time of the last engine step", float(getattr(engine, "last_step_seconds", 0.0))))
        rows.append(("cubic_engine_poisoned", "gauge", "1 after a step failed (the engine refuses work)", 1.0 if getattr(engine, "poisoned", False) else 0.0))
    vision = getattr(getattr(backend, "processor", None), "vision", None)
    if vision is not None:                                   # deployments with a vision tower
        store = vision.store
        rows += [("cubic_media_encode_calls_total", "counter", "calls of the vision tower", float(vision.encode_calls)),
                 ("cubic_media_patches_total", "counter", "patches the tower has encoded", float(vision.encoder.encoded_patches)),
                 ("cubic_media_feature_store_hits_total", "counter", "media items served from encoded features", float(store.hits)),
                 ("cubic_media_feature_store_misses_total", "counter", "media items that had to be encoded", float(store.misses)),
                 ("cubic_media_feature_store_bytes", "gauge", "host memory held by encoded features", float(store.bytes))]
    out = []
    for name, kind, text, value in rows:
        out += [f"# HELP {name} {text}", f"# TYPE {name} {kind}", f"{name}{label} {value:g}"]
    return "\n".join(out) + "\n"


class CubicASGIApp:
    def __init__(self, backend: ChatBackend, model_id: str, served_model_name: str | None = None,
                 api_key: str | None = None, sampling_defaults: dict | None = None) -> None:
        self.sampling_defaults = dict(sampling_defaults or {})      # the checkpoint's generation_config.json
        self.backend = backend
        self.model_id = model_id
        # several public names may be given: requests may use any of them, responses carry the first
        names = [served_model_name] if isinstance(served_model_name, str) else list(served_model_name or ())
        self.served_model_name = names[0] if names else model_id
        self.accepted_names = tuple(dict.fromkeys([*names, model_id]))
        self._key_digest = hashlib.sha256(api_key.encode()).digest() if api_key else None
        self.created = int(time.time())

    # ------------------------------------------------------------------ ASGI
    async def __call__(self, scope, receive, send) -> None:
        if scope["type"] == "lifespan":
            await self._lifespan(receive, send)
            return
        if scope["type"] != "http":
            return
        method, path = scope["method"], scope["path"].rstrip("/") or "/"
        headers = {k.decode("latin1").lower(): v.decode("latin1") for k, v in scope.get("headers", [])}
        protocol = "anthropic" if path == "/v1/messages" else "openai"
        try:
            if path == "/health" and method == "GET":
                ok = bool(getattr(self.backend, "ready", True))
                await self._json(send, 200 if ok else 503, {"status": "ok" if ok else "unavailable"})
                return
            if not self._authorized(headers):
                await self._json(send, 401, _error_body(protocol, 401, "invalid or missing API key", "authentication_error"))
                return
            if path == "/metrics" and method == "GET":
                await self._text(send, 200, render_metrics(self.backend, self.served_model_name),
                                 "text/plain; version=0.0.4; charset=utf-8")
                return
            if path == "/v1/models" and method == "GET":
                await self._json(send, 200, {"object": "list", "data": [
                    {"id": self.served_model_name, "object": "model", "created": self.created, "owned_by": "cubic-serve-b200"}]})
                return
            if path in ("/v1/chat/completions", "/v1/messages"):
                if method != "POST":
                    await self._json(send, 405, _error_body(protocol, 405, "method not allowed", "invalid_request_error"))
                    return
                await self._chat(protocol, receive, send)
                return
            await self._json(send, 404, _error_body(protocol, 404, "unknown route", "not_found_error"))
        except Exception:  # noqa: BLE001 - last-resort guard: never leak internals
            await self._json(send, 500, _error_body(protocol, 500, "internal server error", "server_error"))

    async def _text(self, send, status: int, text: str, content_type: str) -> None:
        body = text.encode()
        await send({"type": "http.response.start", "status": status,
                    "headers": [(b"content-type", content_type.encode()), (b"content-length", str(len(body)).encode())]})
        await send({"type": "http.response.body", "body": body})

    async def _lifespan(self, receive, send) -> None:
        while True:
            msg = await receive()
            if msg["type"] == "lifespan.startup":
                await send({"type": "lifespan.startup.complete"})
            elif msg["type"] == "lifespan.shutdown":
                closer = getattr(self.backend, "close", None)
                if closer:
                    res = closer()
                    if asyncio.iscoroutine(res):
                        await res
                await send({"type": "lifespan.shutdown.complete"})
                return

    def _authorized(self, headers: dict) -> bool:
        if self._key_digest is None:
            return True
        token = headers.get("x-api-key")
        auth = headers.get("authorization", "")
        if token is None and auth.lower().startswith("bearer "):
            token = auth[7:].strip()
        if not token:
            return False
        return hmac.compare_digest(hashlib.sha256(token.encode()).digest(), self._key_digest)

    # ------------------------------------------------------------- plumbing
    async def _json(self, send, status: int, body: dict, extra_headers: list | None = None) -> None:
        raw = json.dumps(body, ensure_ascii=False, separators=(",", ":")).encode()
        await send({"type": "http.response.start", "status": status,
                    "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(raw)).encode()),
                                *(extra_headers or [])]})
        await send({"type": "http.response.body", "body": raw})

    async def _read_body(self, receive) -> bytes | None:
        chunks, total = [], 0
        while True:
            msg = await receive()
            if msg["type"] == "http.disconnect":
                return None
            chunk = msg.get("body", b"")
            total += len(chunk)
            if total > MAX_BODY_BYTES:
                raise ChatBackendError(413, "request body too large", "invalid_request_error")
            chunks.append(chunk)
            if not msg.get("more_body", False):
                return b"".join(chunks)

    async def _chat(self, protocol: str, receive, send) -> None:
        try:
            raw = await self._read_body(receive)
            if raw is None:
                return
            body = decode_strict_json(raw)
            if protocol == "openai":
                req = normalize_openai_chat_completions(body, self.served_model_name, self.sampling_defaults)
            else:
                req = normalize_anthropic_messages(body, self.served_model_name, self.sampling_defaults)
            if req.model not in self.accepted_names:
                raise RequestError(f"model {req.model!r} is not served here", param="model", status=404,
                                   code="model_not_found")
            if req.model != self.served_model_name:
                import dataclasses
                req = dataclasses.replace(req, model=self.served_model_name)      # responses carry the first public name
            if not getattr(self.backend, "ready", True):
                raise ChatBackendError(503, "the server is not ready", "service_unavailable")
            events = self.backend.start(req)
        except _StrictJSONError as exc:
            await self._json(send, 400, _error_body(protocol, 400, str(exc), "invalid_request_error"))
            return
        except RequestError as exc:
            await self._json(send, exc.status, _error_body(protocol, exc.status, exc.public_message, exc.code, exc.param))
            return
        except ChatBackendError as exc:
            await self._json(send, exc.status, _error_body(protocol, exc.status, exc.public_message, exc.code))
            return
        if req.stream:
            await self._stream(protocol, req, events, receive, send)
        else:
            await self._unary(protocol, req, events, receive, send)

    async def _watch_disconnect(self, receive, request_id: str) -> None:
        while True:
            msg = await receive()
            if msg["type"] == "http.disconnect":
                await self.backend.cancel(request_id)
                return

    async def _unary(self, protocol, req, events, receive, send) -> None:
        watcher = asyncio.ensure_future(self._watch_disconnect(receive, req.request_id))
        collected: list[TokenEvent] = []
        try:
            async for ev in events:
                collected.append(ev)
        except RequestError as exc:
            await self._json(send, exc.status, _error_body(protocol, exc.status, exc.public_message, exc.code, exc.param))
            return
        except ChatBackendError as exc:
            await self._json(send, exc.status, _error_body(protocol, exc.status, exc.public_message, exc.code))
            return
        finally:
            watcher.cancel()
        body = (project_openai_chat_completion(req, collected) if protocol == "openai"
                else project_anthropic_message(req, collected))
        await self._json(send, 200, body)

    async def _stream(self, protocol, req, events, receive, send) -> None:
        it = events.__aiter__()
        # the first event decides between an HTTP error and a 200 event stream
        try:
            first = await it.__anext__()
        except StopAsyncIteration:
            first = None
        except RequestError as exc:
            await self._json(send, exc.status, _error_body(protocol, exc.status, exc.public_message, exc.code, exc.param))
            return
        except ChatBackendError as exc:
            await self._json(send, exc.status, _error_body(protocol, exc.status, exc.public_message, exc.code))
            return
        await send({"type": "http.response.start", "status": 200,
                    "headers": [(b"content-type", b"text/event-stream; charset=utf-8"), (b"cache-control", b"no-cache"),
                                (b"x-accel-buffering", b"no")]})
        watcher = asyncio.ensure_future(self._watch_disconnect(receive, req.request_id))

        async def replay():
            if first is not None:
                yield first
            async for ev in it:
                yield ev

        try:
            if protocol == "openai":
                async for ev in replay():
                    for chunk in project_openai_chat_completion_stream(req, [ev], self.created):
                        frame = b"data: " + json.dumps(chunk, ensure_ascii=False, separators=(",", ":")).encode() + b"\n\n"
                        await send({"type": "http.response.body", "body": frame, "more_body": True})
                await send({"type": "http.response.body", "body": b"data: [DONE]\n\n", "more_body": True})
            else:
                projector = AnthropicStreamProjector(req)
                async for ev in replay():
                    for name, data in projector.push(ev):
                        frame = (f"event: {name}\n".encode() + b"data: "
                                 + json.dumps(data, ensure_ascii=False, separators=(",", ":")).encode() + b"\n\n")
                        await send({"type": "http.response.body", "body": frame, "more_body": True})
        except (ChatBackendError, RequestError) as exc:
            err = _error_body(protocol, getattr(exc, "status", 500), exc.public_message, getattr(exc, "code", "server_error"))
            frame = (b"event: error\n" if protocol == "anthropic" else b"") + b"data: " + json.dumps(err).encode() + b"\n\n"
            await send({"type": "http.response.body", "body": frame, "more_body": True})
        except Exception:  # noqa: BLE001
            err = _error_body(protocol, 500, "internal server error", "server_error")
            await send({"type": "http.response.body", "body": b"data: " + json.dumps(err).encode() + b"\n\n",
                        "more_body": True})
        finally:
            watcher.cancel()
            await send({"type": "http.response.body", "body": b"", "more_body": False})
