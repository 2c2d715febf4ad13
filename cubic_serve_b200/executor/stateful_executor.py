"""Executors over eager models that hold a request's whole context themselves (no pages, no prefix sharing), with
optional draft / review rounds when the model has a draft head.

A model for this executor offers

* ``forward(tokens, state, positions3, embeds, last_only) -> (logits, state)``: append ONE request's tokens to its
  state (updated in place); after the call ``model.last_feedback`` holds the hidden rows that feed a draft head;
* ``draft_forward(tokens, feedback, state) -> (logits, feedback, state)`` and ``has_draft_head`` (optional).

Rounds (``speculative_depth`` > 0): the head proposes up to ``depth`` tokens from the root token and the target's
feedback row of the previous position; the target reviews root + drafts in one pass on a COPY of the request's state;
the longest agreeing prefix and the target's own next token are emitted; the committed state is then advanced over the
accepted tokens only.  The head's state follows the committed tokens with the TARGET's feedback rows (its proposal
steps run on a copy), so proposals never depend on rejected drafts.  Greedy, unconstrained requests take part; the
tokens are those of plain greedy decoding.

Reference counterpart: ``executor/draft.py:195-443`` (provider-independent reference of draft rounds) there.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class RequestSlot:
    uid: int
    state: object
    draft: object | None = None                 # the draft head's state: caught up to the position before the last one
    carried: torch.Tensor | None = None         # the target's feedback row of the last position, [1, width]


class StatefulEagerExecutor:
    accepts_features = True
    keeps_request_state = True

    def __init__(self, model, speculative_depth: int = 0) -> None:
        self.model = model
        if speculative_depth and not getattr(model, "has_draft_head", False):
            raise ValueError("speculative rounds need the checkpoint's draft head (mtp.* tensors)")
        self.speculative_depth = int(speculative_depth)
        self._slots: dict[int, RequestSlot] = {}
        self.last_round: dict | None = None
        self.h2d_bytes_last = self.d2h_bytes_last = self.kernel_launches_last = 0

    # hooks of the concrete executor
    def _new_state(self):
        raise NotImplementedError

    def _copy(self, state):
        raise NotImplementedError

    def copy_pages(self, pairs) -> None:
        if pairs:
            raise RuntimeError("this executor keeps no pages: copy-on-write cannot occur with the prefix cache off")

    def _slot(self, s) -> RequestSlot:
        held = self._slots.get(s.request_slot)
        if s.start == 0 or held is None or held.uid != s.uid:
            if s.start != 0:
                raise RuntimeError(f"slot {s.request_slot}: no state for a segment that starts at {s.start}")
            held = RequestSlot(s.uid, self._new_state())
            self._slots[s.request_slot] = held
        if held.state.length != s.start:
            raise RuntimeError(f"slot {s.request_slot}: state holds {held.state.length} tokens, the segment starts at {s.start}")
        return held

    def _advance(self, slot: RequestSlot, tokens: list[int], positions3=None, embeds=None, deep=None) -> torch.Tensor:
        """Run the target over ``tokens`` on the slot's committed state and let the draft head follow: the head sees
        (token i + 1, feedback of position i) for every position whose successor is known."""
        extra = {"deep": deep} if deep else {}
        logits, _ = self.model.forward(tokens, slot.state, positions3, embeds, last_only=True, **extra)
        if self.speculative_depth:
            fb = self.model.last_feedback
            head_tokens = ([tokens[0]] if slot.carried is not None else []) + tokens[1:]
            head_fb = torch.cat(([slot.carried] if slot.carried is not None else []) + [fb[:-1]])
            if head_tokens:
                _, _, slot.draft = self.model.draft_forward(head_tokens, head_fb, slot.draft)
            slot.carried = fb[-1:].clone()
        return logits[0]

    def execute(self, segs: list) -> np.ndarray:
        from .eager_executor import sample_row
        out = []
        for s in segs:
            logits = self._advance(self._slot(s), [int(t) for t in s.token_ids], s.positions3, s.embeds,
                                   getattr(s, "deep_embeds", None))
            if s.sample:
                out.append(sample_row(logits, s))
        return np.asarray(out, dtype=np.int32)

    def execute_speculative(self, segs: list, depths: list[int] | None = None) -> list[list[int]]:
        """One round per decode segment (its root token); returns the emitted tokens of every request."""
        from .eager_executor import sample_row
        outs, accepted, proposed = [], [], []
        for i, s in enumerate(segs):
            K = self.speculative_depth if depths is None else min(self.speculative_depth, int(depths[i]))
            slot = self._slot(s)
            plain = K <= 0 or len(s.token_ids) != 1 or s.temperature > 0 or s.mask is not None or slot.carried is None
            if plain:
                outs.append([sample_row(self._advance(slot, [int(t) for t in s.token_ids], s.positions3, s.embeds), s)])
                accepted.append(0)
                proposed.append(0)
                continue
            root = int(s.token_ids[0])
            # proposals on a copy of the head's state: draft steps feed on the head's own feedback
            dstate = self._copy(slot.draft) if slot.draft is not None else None
            drafts, tok, fb = [], root, slot.carried
            for _ in range(K):
                lg, fb, dstate = self.model.draft_forward([tok], fb, dstate)
                tok = int(lg[0].argmax())
                drafts.append(tok)
            # review: root + drafts in one pass on a copy of the committed state
            pos3 = None
            if s.positions3 is not None:
                pos3 = np.asarray(s.positions3)[:, :1] + np.arange(K + 1)[None, :]
            logits, _ = self.model.forward([root] + drafts, self._copy(slot.state), pos3)
            target = logits.argmax(-1).tolist()
            a = 0
            while a < K and drafts[a] == target[a]:
                a += 1
            # commit the accepted prefix (the head follows with the target's feedback)
            self._advance(slot, [root] + drafts[:a], None if pos3 is None else pos3[:, :a + 1])
            outs.append([int(t) for t in target[:a + 1]])
            accepted.append(a)
            proposed.append(K)
        self.last_round = {"depth": max(proposed, default=0), "accepted": accepted, "proposed": proposed,
                           "proposal_ms": 0.0, "target_ms": 0.0}
        return outs
