"""Structured-output constraints: request-local ``mask -> apply -> accept`` boundary.

The reference routes json_schema / regex / choice / grammar / structural_tag constraints through xgrammar
(``generation/constraints.py:46-531``, ``generation/xgrammar.py:280``): a matcher per request fills a token
bitmask before sampling, the sampler applies it, and the accepted token advances (or, for speculative
rounds, rolls back) the matcher.  The sampler kernel here takes exactly that bitmask (``mask`` argument of
``ops.kernels.sample``).  This module owns the matcher life cycle; it works without xgrammar for the
constraint kinds that need no grammar engine (``choice``) and reports the others as unavailable when the
optional dependency is missing.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..contracts.request import StructuredKind, StructuredOutput

try:  # optional extra
    import xgrammar as _xgr
except Exception:  # pragma: no cover
    _xgr = None


def constraint_supported(s: StructuredOutput) -> bool:
    if s.kind in (StructuredKind.NONE, StructuredKind.JSON_OBJECT, StructuredKind.CHOICE):
        return True
    return _xgr is not None


class ChoiceMatcher:
    """Rewindable matcher for ``choice`` constraints: the output must be exactly one of the given strings."""

    def __init__(self, choices: list[str], tokenizer, eos_token_id: int) -> None:
        self.seqs = [list(tokenizer.encode(c, add_special_tokens=False)) for c in choices]
        self.eos = eos_token_id
        self.pos = 0
        self.alive = list(range(len(self.seqs)))
        self._history: list[list[int]] = []

    def fill_bitmask(self, bitmask: np.ndarray) -> None:
        """``bitmask``: uint32 words of one row, bit set = token allowed."""
        bitmask[:] = 0
        for i in self.alive:
            seq = self.seqs[i]
            tok = seq[self.pos] if self.pos < len(seq) else self.eos
            bitmask[tok >> 5] |= np.uint32(1 << (tok & 31))

    def accept(self, token: int) -> bool:
        nxt = [i for i in self.alive if (self.seqs[i][self.pos] if self.pos < len(self.seqs[i]) else self.eos) == token]
        if not nxt:
            return False
        self._history.append(self.alive)
        self.alive = nxt
        self.pos += 1
        return True

    def rollback(self, n: int) -> None:
        for _ in range(n):
            self.alive = self._history.pop()
            self.pos -= 1

    @property
    def finished(self) -> bool:
        return any(self.pos > len(self.seqs[i]) for i in self.alive)


@dataclass
class GrammarTransaction:
    """Per-round view used by speculative decoding: accept draft tokens tentatively, roll back the rejected tail."""
    matcher: object
    accepted: int = 0

    def try_accept(self, token: int) -> bool:
        ok = self.matcher.accept(token)
        if ok:
            self.accepted += 1
        return ok

    def commit(self, keep: int) -> None:
        if keep < self.accepted:
            self.matcher.rollback(self.accepted - keep)
        self.accepted = 0


class DelayedMatcher:
    """A constraint that starts after the reasoning block: while the model is thinking every token is allowed; once
    the closing sequence (``</think>``, one or several token ids) has been emitted the inner matcher rules.  Rewindable
    across the boundary, like the matchers it wraps (reference: delayed constraints of ``generation/constraints.py``)."""

    def __init__(self, inner, end_sequence: list[int]) -> None:
        if not end_sequence:
            raise ValueError("a delayed constraint needs the token sequence that ends the reasoning block")
        self.inner = inner
        self.end = [int(t) for t in end_sequence]
        self.free: list[int] = []          # tokens accepted while unconstrained (only the tail is ever looked at)
        self.active = False
        self._log: list[bool] = []         # per accepted token: did the inner matcher consume it?

    def fill_bitmask(self, bitmask: np.ndarray) -> None:
        if self.active:
            self.inner.fill_bitmask(bitmask)
        else:
            bitmask[:] = np.uint32(0xFFFFFFFF)

    def accept(self, token: int) -> bool:
        if self.active:
            ok = self.inner.accept(token)
            if ok:
                self._log.append(True)
            return ok
        self.free.append(int(token))
        self._log.append(False)
        if self.free[-len(self.end):] == self.end:
            self.active = True
        return True

    def rollback(self, n: int) -> None:
        for _ in range(n):
            if self._log.pop():
                self.inner.rollback(1)
            else:
                self.free.pop()
                self.active = False        # the token that completed the closing sequence is among those taken back

    @property
    def finished(self) -> bool:
        return self.active and self.inner.finished


class GrammarEngineMatcher:
    """Adapter giving an xgrammar ``GrammarMatcher`` the ``fill_bitmask / accept / rollback`` interface."""

    def __init__(self, matcher, vocab_size: int) -> None:
        self.m = matcher
        self.vocab_size = vocab_size
        self._bitmask = _xgr.allocate_token_bitmask(1, vocab_size)      # int32 torch tensor [1, words]

    def fill_bitmask(self, bitmask: np.ndarray) -> None:
        self.m.fill_next_token_bitmask(self._bitmask, 0)
        words = self._bitmask[0].numpy().view(np.uint32)
        bitmask[:len(words)] = words[:len(bitmask)]

    def accept(self, token: int) -> bool:
        return bool(self.m.accept_token(int(token)))

    def rollback(self, n: int) -> None:
        self.m.rollback(n)

    @property
    def finished(self) -> bool:
        return bool(self.m.is_terminated())


def _tokenizer_info(tokenizer, eos_token_id: int, vocab_size: int):
    """The grammar engine's view of the vocabulary.  HuggingFace tokenizers are read by the engine itself; a tokenizer
    that only offers ``decode`` (the built-in byte tokenizer) is described token by token as a raw vocabulary (ids
    above the tokenizer's own range are padding of the model's vocabulary and never allowed)."""
    if hasattr(tokenizer, "get_vocab") and hasattr(tokenizer, "convert_ids_to_tokens"):
        return _xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=vocab_size)
    own = int(getattr(tokenizer, "vocab_size", vocab_size))
    vocab: list = []
    for i in range(vocab_size):
        if i < 256 and own >= 256:
            vocab.append(bytes([i]))                       # byte-level ids
        elif i < own:
            vocab.append(tokenizer.decode([i], skip_special_tokens=False) or f"<special_{i}>")
        else:
            vocab.append(f"<unused_{i}>")
    return _xgr.TokenizerInfo(vocab, vocab_type=_xgr.VocabType.RAW, vocab_size=vocab_size, stop_token_ids=[int(eos_token_id)])


def _compile_structural_tag(compiler, spec):
    """Structural tags: free text in which every occurrence of a trigger opens a tagged region whose body follows a
    JSON schema (tool calls written inline).  Both wire forms are taken: the engine's own
    ``{"type": "structural_tag", "format": {...}}`` and the older ``{"structures": [{"begin", "schema", "end"}],
    "triggers": [...]}`` of the OpenAI-compatible servers."""
    import json
    if isinstance(spec, str):
        spec = json.loads(spec)
    if not isinstance(spec, dict):
        raise ValueError("a structural tag is a JSON object")
    if "structures" in spec:
        structures, triggers = spec.get("structures"), spec.get("triggers")
        if not isinstance(structures, list) or not structures or not isinstance(triggers, list) or not triggers:
            raise ValueError("structural_tag needs non-empty 'structures' and 'triggers'")
        tags = []
        for item in structures:
            if not isinstance(item, dict) or not isinstance(item.get("begin"), str) or not isinstance(item.get("end"), str):
                raise ValueError("every structure needs 'begin' and 'end' strings")
            if not any(item["begin"].startswith(t) for t in triggers):
                raise ValueError(f"no trigger is a prefix of the tag {item['begin']!r}")
            schema = item.get("schema", {})
            tags.append(_xgr.StructuralTagItem(begin=item["begin"], schema=schema if isinstance(schema, str) else json.dumps(schema),
                                               end=item["end"]))
        return compiler.compile_structural_tag(tags, [str(t) for t in triggers])
    return compiler.compile_structural_tag(spec)


def compile_matcher(s: StructuredOutput, tokenizer, eos_token_id: int, vocab_size: int):
    """Build a matcher for a constraint, or ``None`` when the request is unconstrained."""
    if s.kind is StructuredKind.NONE:
        return None
    if s.kind is StructuredKind.CHOICE:
        return ChoiceMatcher(list(s.schema), tokenizer, eos_token_id)
    if _xgr is None:
        if s.kind is StructuredKind.JSON_OBJECT:
            return None            # without a grammar engine json_object stays a prompt-level instruction
        raise RuntimeError("xgrammar is not installed")
    compiler = _xgr.GrammarCompiler(_tokenizer_info(tokenizer, eos_token_id, vocab_size))
    if s.kind is StructuredKind.JSON_OBJECT:
        compiled = compiler.compile_builtin_json_grammar()
    elif s.kind in (StructuredKind.JSON_SCHEMA, StructuredKind.TOOL_SCHEMA):
        import json
        compiled = compiler.compile_json_schema(json.dumps(s.schema))
    elif s.kind is StructuredKind.REGEX:
        compiled = compiler.compile_regex(s.schema)
    elif s.kind is StructuredKind.GRAMMAR:
        compiled = compiler.compile_grammar(s.schema)
    elif s.kind is StructuredKind.STRUCTURAL_TAG:
        compiled = _compile_structural_tag(compiler, s.schema)
    else:
        raise RuntimeError(f"unsupported constraint kind {s.kind}")
    return GrammarEngineMatcher(_xgr.GrammarMatcher(compiled), vocab_size)
