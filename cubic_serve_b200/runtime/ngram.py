"""N-gram (prompt-lookup) draft proposals: speculative decoding without a draft model.

The proposal for a request is what followed the most recent earlier occurrence of its last ``n`` tokens, longest ``n``
first.  Text that repeats itself -- quoted context, code edits, structured records, a model that loops -- is predicted
for free; text that does not costs nothing, because a request without a match gets no draft and decodes normally.
The index is incremental: every appended token registers the n-grams that end just before it, so a proposal is one
dictionary lookup per ``n``.

Reference counterpart: the n-gram draft oracle among the eager operator references (``ops/eager``) and the
provider-independent draft round of ``executor/draft.py:195`` (proposals may come from any provider).
"""
from __future__ import annotations


class NgramIndex:
    """Positions of the most recent occurrence of every n-gram (``min_n <= n <= max_n``) of one token sequence."""

    def __init__(self, max_n: int = 4, min_n: int = 2) -> None:
        if not 1 <= min_n <= max_n:
            raise ValueError("need 1 <= min_n <= max_n")
        self.max_n, self.min_n = max_n, min_n
        self.tokens: list[int] = []
        # n-gram -> index of the token FOLLOWING its latest occurrence that has a follower
        self._next: dict[tuple, int] = {}

    def extend(self, tokens) -> None:
        for t in tokens:
            pos = len(self.tokens)             # the new token follows every n-gram that ends at pos - 1
            for n in range(self.min_n, self.max_n + 1):
                if pos >= n:
                    self._next[tuple(self.tokens[pos - n:pos])] = pos
            self.tokens.append(int(t))

    def truncate(self, length: int) -> None:
        """Forget tokens beyond ``length`` (a request rolled back); the index is rebuilt."""
        if length < len(self.tokens):
            kept = self.tokens[:length]
            self.tokens, self._next = [], {}
            self.extend(kept)

    def propose(self, k: int) -> list[int]:
        """Up to ``k`` tokens that followed the latest earlier occurrence of the current suffix; [] without a match."""
        L = len(self.tokens)
        if k <= 0:
            return []
        for n in range(min(self.max_n, L), self.min_n - 1, -1):
            pos = self._next.get(tuple(self.tokens[L - n:]))
            if pos is not None and pos < L:
                out = self.tokens[pos:pos + k]
                period = L - pos
                while len(out) < k:            # the match runs into the present: "a b a b" goes on "a b a b ..."
                    out.append(out[len(out) - period])
                return out
        return []


class NgramProposer:
    """Per-request indices, kept in step with the requests' token sequences."""

    def __init__(self, max_n: int = 4, min_n: int = 2) -> None:
        self.max_n, self.min_n = max_n, min_n
        self._index: dict[str, NgramIndex] = {}
        self.stats = {"lookups": 0, "hits": 0, "proposed": 0}

    def propose(self, request_id: str, tokens: list[int], k: int) -> list[int]:
        idx = self._index.get(request_id)
        if idx is None:
            idx = self._index[request_id] = NgramIndex(self.max_n, self.min_n)
        have = len(idx.tokens)
        if have > len(tokens) or (have and idx.tokens[have - 1] != tokens[have - 1]):
            idx.truncate(0)                    # not a continuation of what was indexed (sequences normally only grow)
            have = 0
        idx.extend(tokens[have:])
        out = idx.propose(k)
        self.stats["lookups"] += 1
        self.stats["hits"] += bool(out)
        self.stats["proposed"] += len(out)
        return out

    def forget(self, request_id: str) -> None:
        self._index.pop(request_id, None)
