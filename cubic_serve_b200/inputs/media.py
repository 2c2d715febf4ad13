"""Media resolver: turns the ``media_url`` of an image / video content part into bytes, under an explicit policy.

Three sources, each closed by default except inline data:

* ``data:<mime>;base64,<payload>`` -- decoded in place; the declared type must be an allowed image / video type and
  agree with the payload's magic bytes;
* ``file:///path`` or a bare absolute path -- only below one of the allow-listed roots, after resolving symlinks;
* ``http(s)://host/...`` -- only for allow-listed hosts, fetched with a time limit and a byte limit, no redirects to
  other hosts.

Every result carries the SHA-256 of its bytes; an LRU keyed by the request's URL string keeps the last results so that
a conversation that re-sends its images every turn does not decode or fetch them again.  The text-only model families
served here reject media parts at admission; this module is the boundary a vision encoder consumes.

Reference counterpart: ``inputs/chat.py:57-366`` (media resolver: data / http / file sources with an allow-list).
"""
from __future__ import annotations

import base64
import binascii
import hashlib
import urllib.parse
import urllib.request
from collections import OrderedDict
from dataclasses import dataclass, field
from pathlib import Path

IMAGE_TYPES = ("image/png", "image/jpeg", "image/webp", "image/gif")
VIDEO_TYPES = ("video/mp4", "video/webm")
_MAGIC = ((b"\x89PNG\r\n\x1a\n", "image/png"), (b"\xff\xd8\xff", "image/jpeg"), (b"GIF87a", "image/gif"),
          (b"GIF89a", "image/gif"), (b"\x1aE\xdf\xa3", "video/webm"))


class MediaError(ValueError):
    """The media reference is malformed or outside the policy (a 400 for the client, never a 500)."""


@dataclass(frozen=True)
class MediaPolicy:
    max_bytes: int = 32 << 20
    file_roots: tuple[str, ...] = ()            # directories local files may be read from
    http_hosts: tuple[str, ...] = ()            # host names remote media may be fetched from
    timeout_seconds: float = 10.0
    cache_entries: int = 64


@dataclass(frozen=True)
class ResolvedMedia:
    kind: str          # image | video
    mime: str
    data: bytes = field(repr=False)
    sha256: str = ""
    source: str = ""   # data | file | http


def sniff(data: bytes) -> str | None:
    """Media type by magic bytes (None when unknown)."""
    for magic, mime in _MAGIC:
        if data.startswith(magic):
            return mime
    if data[:4] == b"RIFF" and data[8:12] == b"WEBP":
        return "image/webp"
    if data[4:8] == b"ftyp":
        return "video/mp4"
    return None


class MediaResolver:
    def __init__(self, policy: MediaPolicy | None = None, fetch=None) -> None:
        self.policy = policy or MediaPolicy()
        self._roots = tuple(Path(r).resolve() for r in self.policy.file_roots)
        self._cache: OrderedDict[str, ResolvedMedia] = OrderedDict()
        self._fetch = fetch or self._http_get          # injectable: tests and deployments with their own client
        self.stats = {"resolved": 0, "cache_hits": 0}

    # ------------------------------------------------------------------ public
    def resolve(self, url: str, kind: str = "image") -> ResolvedMedia:
        if kind not in ("image", "video"):
            raise MediaError(f"unknown media kind {kind!r}")
        if not isinstance(url, str) or not url:
            raise MediaError("a media part needs a url")
        key = f"{kind}:{url}" if len(url) < 4096 else f"{kind}:sha256:{hashlib.sha256(url.encode()).hexdigest()}"
        hit = self._cache.get(key)
        if hit is not None:
            self._cache.move_to_end(key)
            self.stats["cache_hits"] += 1
            return hit
        if url.startswith("data:"):
            mime, data, source = *self._from_data(url), "data"
        elif url.startswith(("http://", "https://")):
            mime, data, source = *self._from_http(url), "http"
        elif url.startswith("file://") or url.startswith("/"):
            mime, data, source = *self._from_file(url), "file"
        else:
            raise MediaError("media urls are data:, file: or http(s): references")
        out = self._check(kind, mime, data, source)
        self._cache[key] = out
        while len(self._cache) > self.policy.cache_entries:
            self._cache.popitem(last=False)
        self.stats["resolved"] += 1
        return out

    # ------------------------------------------------------------------ sources
    def _from_data(self, url: str) -> tuple[str | None, bytes]:
        head, sep, payload = url[5:].partition(",")
        if not sep:
            raise MediaError("malformed data: url")
        params = head.split(";")
        if "base64" not in params[1:]:
            raise MediaError("data: urls must be base64 encoded")
        if len(payload) > self.policy.max_bytes * 4 // 3 + 4:
            raise MediaError("media is larger than the configured limit")
        try:
            data = base64.b64decode(payload, validate=True)
        except (binascii.Error, ValueError) as exc:
            raise MediaError("data: url payload is not valid base64") from exc
        return (params[0].strip().lower() or None), data

    def _from_file(self, url: str) -> tuple[str | None, bytes]:
        raw = urllib.parse.unquote(urllib.parse.urlparse(url).path) if url.startswith("file://") else url
        if not self._roots:
            raise MediaError("local files are not enabled in this deployment")
        path = Path(raw).resolve()                      # symlinks resolved before the root check
        if not any(path == r or r in path.parents for r in self._roots):
            raise MediaError("the file is outside the allowed media directories")
        if not path.is_file():
            raise MediaError("no such media file")
        if path.stat().st_size > self.policy.max_bytes:
            raise MediaError("media is larger than the configured limit")
        return None, path.read_bytes()

    def _from_http(self, url: str) -> tuple[str | None, bytes]:
        host = (urllib.parse.urlparse(url).hostname or "").lower()
        if host not in {h.lower() for h in self.policy.http_hosts}:
            raise MediaError("remote media from this host is not enabled in this deployment")
        mime, data = self._fetch(url, self.policy.timeout_seconds, self.policy.max_bytes)
        return (mime.split(";")[0].strip().lower() if mime else None), data

    @staticmethod
    def _http_get(url: str, timeout: float, max_bytes: int) -> tuple[str | None, bytes]:
        class _SameHost(urllib.request.HTTPRedirectHandler):
            def redirect_request(self, req, fp, code, msg, headers, newurl):
                if urllib.parse.urlparse(newurl).hostname != urllib.parse.urlparse(req.full_url).hostname:
                    raise MediaError("remote media redirected to another host")
                return super().redirect_request(req, fp, code, msg, headers, newurl)
        try:
            with urllib.request.build_opener(_SameHost).open(url, timeout=timeout) as resp:
                data = resp.read(max_bytes + 1)
                mime = resp.headers.get("content-type")
        except MediaError:
            raise
        except Exception as exc:  # noqa: BLE001 - network failures are the client's bad reference, not a server fault
            raise MediaError(f"remote media could not be fetched ({type(exc).__name__})") from exc
        if len(data) > max_bytes:
            raise MediaError("media is larger than the configured limit")
        return mime, data

    # ------------------------------------------------------------------ checks
    def _check(self, kind: str, declared: str | None, data: bytes, source: str) -> ResolvedMedia:
        if not data:
            raise MediaError("media is empty")
        if len(data) > self.policy.max_bytes:
            raise MediaError("media is larger than the configured limit")
        actual = sniff(data)
        allowed = IMAGE_TYPES if kind == "image" else VIDEO_TYPES
        if actual is None or actual not in allowed:
            raise MediaError(f"unsupported or unrecognised {kind} format")
        if declared and declared not in ("application/octet-stream", actual):
            raise MediaError(f"declared type {declared} does not match the content ({actual})")
        return ResolvedMedia(kind, actual, data, hashlib.sha256(data).hexdigest(), source)
