"""Grammar masks of a speculative round (``LLMEngine._review_masks_of``): row j allows what the grammar allows after
the first j drafts; the matcher is left where it was; rows behind a refused draft stay open."""
import numpy as np

from cubic_serve_b200.generation.constraints import ChoiceMatcher
from cubic_serve_b200.models.config import kv_heads_of_rank
from cubic_serve_b200.runtime.engine import LLMEngine
from cubic_serve_b200.runtime.scheduler import SchedulerConfig


class _Tok:
    def encode(self, text, add_special_tokens=False):
        return [ord(c) for c in text]


class _Exec:
    cfg = type("C", (), {"vocab_size": 256, "is_hybrid": False})()

    def execute(self, segs):
        return np.zeros(len(segs), dtype=np.int32)

    def copy_pages(self, pairs):
        pass


def _allowed(row):
    return {i for i in range(256) if (int(row[i >> 5]) >> (i & 31)) & 1}


def test_review_rows_follow_the_grammar_and_the_matcher_is_restored():
    eng = LLMEngine(_Exec(), num_pages=8, scheduler_config=SchedulerConfig(max_running_requests=2, max_model_len=64))
    eng._mask_words = 8
    m = ChoiceMatcher(["cat", "car", "dog"], _Tok(), eos_token_id=3)
    fn = eng._review_masks_of(m)
    rows = fn([ord("c"), ord("a"), ord("x"), ord("y")])
    assert rows.shape == (5, 8)
    assert _allowed(rows[0]) == {ord("c"), ord("d")}
    assert _allowed(rows[1]) == {ord("a")}
    assert _allowed(rows[2]) == {ord("t"), ord("r")}
    assert len(_allowed(rows[3])) == 256 and len(_allowed(rows[4])) == 256     # behind the refused draft 'x': never reached
    assert m.pos == 0 and not m.finished                                       # rolled back
    # a full accepted chain up to the end token
    rows = fn([ord("d"), ord("o"), ord("g"), 3])
    assert _allowed(rows[3]) == {3} and m.pos == 0
    # the matcher advanced for real: the next round starts from there
    assert m.accept(ord("c")) and m.accept(ord("a"))
    assert _allowed(fn([ord("r")])[0]) == {ord("t"), ord("r")} and m.pos == 2


def test_kv_heads_of_rank_shares_heads_between_neighbouring_ranks():
    assert [kv_heads_of_rank(8, r, 4) for r in range(4)] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert [kv_heads_of_rank(4, r, 8) for r in range(8)] == [(0, 1), (0, 1), (1, 1), (1, 1), (2, 1), (2, 1), (3, 1), (3, 1)]
    assert kv_heads_of_rank(1, 5, 8) == (0, 1)
    import pytest
    with pytest.raises(ValueError):
        kv_heads_of_rank(3, 0, 2)
    with pytest.raises(ValueError):
        kv_heads_of_rank(3, 0, 8)
