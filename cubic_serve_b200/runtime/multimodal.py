"""A request's media after encoding: what the engine and the executors need beside the token ids.

``MultimodalInput`` carries, for a prompt whose media parts were expanded into runs of placeholder tokens:

* ``spans``: ``(first token, feature rows [n, hidden], content digest)`` per media item, in prompt order.  The rows
  take the place of the placeholder tokens' embeddings in the prefill step that covers them;
* ``positions``: int ``[3, prompt length]`` rotary positions (temporal, row, column) and ``delta``: a token generated
  at sequence index ``i`` has position ``i + delta`` on all three axes;
* ``key_tokens``: the token list the prefix cache hashes, with every placeholder replaced by a number derived from
  the item's digest and the row, so cached pages are shared over a media span only between equal media.

Reference counterpart: ``models/qwen3_5/multimodal.py:1360-1727`` (bridge: prompt expansion, M-RoPE positions, cache
keys), ``runtime/README.md`` (feature rows consumed at decoder input layer 0).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import numpy as np


@dataclass
class MultimodalInput:
    spans: list                                  # [(first token, rows tensor [n, hidden], digest bytes)]
    positions: np.ndarray                        # int32 [3, prompt length]
    delta: int
    # width of the decoder's hidden state when the rows carry more than that: the extra columns are the tower's
    # intermediate ("deepstack") outputs, one block of ``hidden`` columns per early decoder layer they are added after
    hidden: int | None = None
    _keys: dict | None = field(default=None, repr=False)   # sequence index -> content key

    def __post_init__(self) -> None:
        self.positions = np.ascontiguousarray(self.positions, dtype=np.int32)
        if self.positions.ndim != 2 or self.positions.shape[0] != 3:
            raise ValueError("positions are [3, prompt length]")
        at = 0
        for first, rows, digest in self.spans:
            if first < at or first + rows.shape[0] > self.positions.shape[1] or not digest:
                raise ValueError("media spans are ordered, disjoint, inside the prompt and carry a content digest")
            at = first + rows.shape[0]

    @property
    def prompt_length(self) -> int:
        return int(self.positions.shape[1])

    @property
    def deep_layers(self) -> int:
        """How many early decoder layers receive an addition at the media positions."""
        if self.hidden is None or not self.spans:
            return 0
        return self.spans[0][1].shape[1] // self.hidden - 1

    def segment_deep(self, start: int, count: int) -> list:
        """``(offset into the segment, rows [n, layers, hidden])`` of the additions that fall into the segment."""
        out = []
        for first, rows, _ in self.spans:
            lo, hi = max(first, start), min(first + rows.shape[0], start + count)
            if lo < hi and self.deep_layers:
                out.append((lo - start, rows[lo - first:hi - first, self.hidden:].reshape(hi - lo, self.deep_layers, self.hidden)))
        return out

    def key_tokens(self, tokens: list[int]) -> list[int]:
        if self._keys is None:
            keys: dict[int, int] = {}
            for first, rows, digest in self.spans:
                for r in range(rows.shape[0]):
                    h = hashlib.blake2s(digest + r.to_bytes(4, "little"), digest_size=7).digest()
                    keys[first + r] = -1 - int.from_bytes(h, "little")
            self._keys = keys
        out = list(tokens)
        for i, k in self._keys.items():
            if i < len(out):
                out[i] = k
        return out

    def segment_inputs(self, start: int, count: int):
        """``(embeds, positions3)`` of the segment ``[start, start + count)``: the feature rows that fall inside it as
        ``(offset into the segment, rows)`` and its int32 ``[3, count]`` positions."""
        end = start + count
        embeds = []
        for first, rows, _ in self.spans:
            lo, hi = max(first, start), min(first + rows.shape[0], end)
            if lo < hi:
                part = rows[lo - first:hi - first]
                embeds.append((lo - start, part if self.hidden is None else part[:, :self.hidden]))
        n = self.prompt_length
        pos = np.empty((3, count), dtype=np.int32)
        inside = max(0, min(end, n) - start)
        if inside:
            pos[:, :inside] = self.positions[:, start:start + inside]
        if inside < count:
            pos[:, inside:] = np.arange(start + inside, end, dtype=np.int32)[None, :] + self.delta
        return embeds, pos
