"""Serving side of the vision tower: an owned encoder thread, a byte-budgeted store of encoded features, and the
memory plan that bounds one encode call.

* ``EncodedFeatureStore``: feature rows by content digest (the digest of the decoded pixels and the patch geometry),
  least recently used first out, bounded in bytes.  A hit skips the tower entirely; rows are kept on the host so the
  store does not compete with the KV cache for device memory.
* ``EncoderMemoryPlan``: how many patches one ``encode`` call may take so that its transient activations stay inside
  the encoder's memory budget, and the request limits that follow (items above the bound are refused at admission,
  never truncated).  Frames attend only to themselves, so a long clip is cut at frame boundaries into calls that fit
  and the merged rows are concatenated: the result is the same as one call.
* ``VisionService``: owns the tower.  ``submit`` queues a request's media for the encoder thread and returns a future;
  the engine thread never waits on the tower for requests that carry no media.  With tensor parallelism every rank of
  the first pipeline stage runs the same calls in the same order (the service is then driven by ``encode`` directly
  from the rank's command loop, with the tower's ``reduce`` bound to the stage's process group).

Reference counterpart: ``executor/vision.py:223-507`` (``QwenVisionGraph``: memory-bounded buckets, admission limits),
``:576-627`` (``prepare / start / finish_owned_input_encoder``: the owned encoder thread), ``:679-885``
(``InputEncoderGroup``: encoder ranks).
"""
from __future__ import annotations

import hashlib
import queue
import threading
from collections import OrderedDict
from concurrent.futures import Future
from dataclasses import dataclass

import numpy as np
import torch

from ..models.vision import VisionEncoder, feature_rows


class EncoderCapacityError(ValueError):
    """A media item needs more encoder memory than the deployment set aside."""


def media_digest(pixels: np.ndarray, grid: tuple[int, int, int], tag: bytes = b"") -> bytes:
    """Content digest of one item: its pixel rows, grid and the tower / geometry identity ``tag``."""
    h = hashlib.blake2s(tag, digest_size=16)
    h.update(np.asarray(grid, dtype=np.int64).tobytes())
    h.update(np.ascontiguousarray(pixels).view(np.uint8).data)
    return h.digest()


class EncodedFeatureStore:
    def __init__(self, max_bytes: int = 1 << 30) -> None:
        self.max_bytes = int(max_bytes)
        self._rows: OrderedDict[bytes, torch.Tensor] = OrderedDict()
        self._lock = threading.Lock()
        self.bytes = self.hits = self.misses = self.evictions = 0

    def get(self, digest: bytes) -> torch.Tensor | None:
        with self._lock:
            t = self._rows.get(digest)
            if t is None:
                self.misses += 1
                return None
            self._rows.move_to_end(digest)
            self.hits += 1
            return t

    def put(self, digest: bytes, rows: torch.Tensor) -> None:
        rows = rows.detach().to("cpu").contiguous()
        size = rows.numel() * rows.element_size()
        if size > self.max_bytes:
            return                                      # larger than the whole store: served, not kept
        with self._lock:
            old = self._rows.pop(digest, None)
            if old is not None:
                self.bytes -= old.numel() * old.element_size()
            self._rows[digest] = rows
            self.bytes += size
            while self.bytes > self.max_bytes:
                _, gone = self._rows.popitem(last=False)
                self.bytes -= gone.numel() * gone.element_size()
                self.evictions += 1

    def __len__(self) -> int:
        return len(self._rows)


@dataclass(frozen=True)
class EncoderMemoryPlan:
    memory_bytes: int
    max_patches_per_call: int          # transient activations of one encode call stay inside ``memory_bytes``
    max_patches_per_frame: int         # a frame is never cut: larger frames are refused
    max_rows_per_request: int          # decoder rows (placeholder tokens) one request's media may occupy

    @staticmethod
    def build(encoder: VisionEncoder, memory_bytes: int, max_prompt_tokens: int) -> "EncoderMemoryPlan":
        per_patch = max(1, encoder.activation_bytes(1))
        m2 = encoder.cfg.spatial_merge_size ** 2
        # attention of one frame holds a [heads, n, n] score matrix in the worst (non-fused) case
        el = torch.empty((), dtype=encoder.dtype).element_size()
        n = int(memory_bytes // per_patch)
        while n > m2 and n * per_patch + encoder.heads * n * n * el > memory_bytes:
            n = int(n * 0.9)
        n -= n % m2
        if n < m2:
            raise EncoderCapacityError(f"{memory_bytes} bytes of encoder memory hold no merge block")
        return EncoderMemoryPlan(int(memory_bytes), n, n, max_prompt_tokens)

    def calls(self, grid: tuple[int, int, int]) -> list[tuple[int, int]]:
        """Frame ranges ``[first, end)`` of one item, each range one encode call."""
        t, h, w = grid
        if h * w > self.max_patches_per_frame:
            raise EncoderCapacityError(f"a frame of {h * w} patches exceeds the encoder's {self.max_patches_per_frame}")
        per = max(1, self.max_patches_per_call // (h * w))
        return [(f, min(t, f + per)) for f in range(0, t, per)]

    def check_request(self, grids: list[tuple[int, int, int]], merge: int) -> int:
        rows = sum(feature_rows(np.asarray(grids).reshape(-1, 3), merge)) if grids else 0
        if rows > self.max_rows_per_request:
            raise EncoderCapacityError(f"the media expand to {rows} rows; a request may carry {self.max_rows_per_request}")
        for g in grids:
            self.calls(g)
        return rows


class VisionGraphBucket:
    """One captured encode call of ``capacity`` patches: fixed-address inputs, the tower's fixed-shape form recorded in a
    CUDA graph after two eager warm-up runs, replayed for every item that fits.  A small image is bound by the
    launches of the tower's ~16 kernels per layer; a replay issues them as one graph.  On a host without CUDA the
    bucket runs the fixed-shape form eagerly (the arithmetic is the same; tests use this)."""

    def __init__(self, encoder: VisionEncoder, capacity: int) -> None:
        cfg = encoder.cfg
        m2 = cfg.spatial_merge_size ** 2
        if capacity <= 0 or capacity % m2:
            raise ValueError("a bucket holds whole merge blocks")
        self.encoder, self.capacity = encoder, capacity
        dev = encoder.device
        self.px = torch.zeros(capacity, cfg.patch_width, dtype=encoder.dtype, device=dev)
        self.fx = encoder.fixed_inputs(torch.tensor([[1, cfg.spatial_merge_size, cfg.spatial_merge_size]]), capacity)
        self.out: torch.Tensor | None = None
        self.graph = None
        self.replays = 0

    def _capture(self) -> None:
        enc = self.encoder
        if not str(enc.device).startswith("cuda"):
            return
        side = torch.cuda.Stream(enc.device)
        side.wait_stream(torch.cuda.current_stream(enc.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                enc.encode_fixed(self.px, self.fx)
        torch.cuda.current_stream(enc.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        # the capture runs on the encoder's own thread while the engine thread keeps launching: only this thread's
        # calls belong to it
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.out = enc.encode_fixed(self.px, self.fx)

    def encode(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        enc = self.encoder
        n = int(pixel_values.shape[0])
        new = enc.fixed_inputs(grid_thw, self.capacity)
        for k, t in new.items():
            self.fx[k].copy_(t)
        self.px.zero_()
        self.px[:n].copy_(pixel_values.to(enc.device, enc.dtype))
        if self.graph is None and self.out is None:
            self._capture()
        if self.graph is not None:
            self.graph.replay()
            out = self.out
        else:
            out = enc.encode_fixed(self.px, self.fx)
        self.replays += 1
        enc.encoded_patches += n
        rows = n // enc.cfg.spatial_merge_size ** 2
        return out[:rows].clone()


class VisionService:
    """Encodes media items ``(pixels [patches, width] float32, grid)`` to feature rows, through the store."""

    def __init__(self, encoder: VisionEncoder, store: EncodedFeatureStore | None = None,
                 memory_bytes: int = 2 << 30, max_prompt_tokens: int = 1 << 15, identity: bytes = b"",
                 graph_buckets: tuple[int, ...] = ()) -> None:
        """``graph_buckets``: patch capacities of captured encode calls (ascending); a call of at most that many patches
        replays the smallest bucket that holds it, larger calls run eagerly.  Not used by a sharded tower (its
        collectives are not captured)."""
        self.encoder = encoder
        self.buckets = [VisionGraphBucket(encoder, c) for c in sorted(set(graph_buckets))] if encoder.tp_size == 1 else []
        self.store = store if store is not None else EncodedFeatureStore()
        self.plan = EncoderMemoryPlan.build(encoder, memory_bytes, max_prompt_tokens)
        self.identity = identity
        self._queue: queue.Queue = queue.Queue()
        self._thread: threading.Thread | None = None
        self._failure: BaseException | None = None
        self.encode_calls = 0

    # ------------------------------------------------------------------ synchronous path
    def digest(self, pixels: np.ndarray, grid) -> bytes:
        return media_digest(pixels, tuple(int(v) for v in grid), self.identity)

    def encode(self, items: list[tuple[np.ndarray, tuple[int, int, int]]]) -> list[tuple[torch.Tensor, bytes]]:
        """Feature rows and digest per item, in order.  Items already in the store cost nothing."""
        m = self.encoder.cfg.spatial_merge_size
        self.plan.check_request([tuple(g) for _, g in items], m)
        out = []
        for pixels, grid in items:
            grid = tuple(int(v) for v in grid)
            d = self.digest(pixels, grid)
            rows = self.store.get(d)
            if rows is None:
                t, h, w = grid
                parts = []
                for f0, f1 in self.plan.calls(grid):
                    px = torch.from_numpy(np.ascontiguousarray(pixels[f0 * h * w:f1 * h * w]))
                    call_grid = torch.tensor([[f1 - f0, h, w]])
                    bucket = next((b for b in self.buckets if b.capacity >= px.shape[0]), None)
                    if bucket is not None and not self.encoder.cfg.deepstack_visual_indexes:
                        feats = bucket.encode(px, call_grid)
                    else:
                        feats, deep = self.encoder.encode(px, call_grid)
                        if deep:                               # intermediate outputs ride in extra columns of the rows
                            feats = torch.cat([feats] + deep, 1)
                    parts.append(feats)
                    self.encode_calls += 1
                rows = torch.cat(parts, 0) if len(parts) > 1 else parts[0]
                self.store.put(d, rows)
                rows = rows.to("cpu")
            out.append((rows, d))
        return out

    # ------------------------------------------------------------------ owned encoder thread
    def start(self) -> None:
        if self._thread is not None:
            return

        def loop() -> None:
            while True:
                job = self._queue.get()
                if job is None:
                    return
                fut, items = job
                if not fut.set_running_or_notify_cancel():
                    continue
                try:
                    fut.set_result(self.encode(items))
                except BaseException as e:                     # the failure belongs to the request, the thread goes on
                    fut.set_exception(e)
        self._thread = threading.Thread(target=loop, name="vision-encoder", daemon=True)
        self._thread.start()

    def submit(self, items) -> Future:
        """Queue a request's media for the encoder thread (started on first use)."""
        self.start()
        fut: Future = Future()
        self._queue.put((fut, items))
        return fut

    def close(self) -> None:
        if self._thread is not None:
            self._queue.put(None)
            self._thread.join(timeout=30)
            self._thread = None
