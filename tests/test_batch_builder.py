"""Host-side batch staging: decode fast path, prefill row blocks, padding rows, incremental page-table rows."""
import numpy as np

from cubic_serve_b200.executor.gpu_executor import BatchBuilder, Segment


def test_decode_fast_path_and_padding():
    bb = BatchBuilder(max_rows=8, max_tokens=256, max_model_len=256, group=4, kv_heads=2, device="cpu")
    segs = [Segment(i, [10 + i], 33 + i, list(range(i * 10, i * 10 + 4)), True, 0.5, 0.9, 3, 7, 2, uid=i) for i in range(3)]
    b, rows = bb.fill(segs, pad_rows_to=8)
    h = bb.stage.h
    assert (rows, b.num_tokens, b.num_row_blocks, b.num_logit_rows) == (3, 8, 8, 8)
    assert h["token_ids"][:3].tolist() == [10, 11, 12] and h["positions"][:3].tolist() == [33, 34, 35]
    # slot = page * 16 + offset with page = pages[pos >> 4]
    assert h["slots"][:3].tolist() == [2 * 16 + 1, 12 * 16 + 2, 22 * 16 + 3]
    assert h["slots"][3:8].tolist() == [-1] * 5 and h["rb_qcount"][:8].tolist() == [1, 1, 1, 0, 0, 0, 0, 0]
    assert h["rb_ctx"][:3].tolist() == [34, 35, 36] and h["rb_req"][:3].tolist() == [0, 1, 2]
    assert h["page_table"][1, :4].tolist() == [10, 11, 12, 13]
    assert np.allclose(h["temperature"][:3], 0.5) and h["temperature"][3] == 0 and h["top_k"][:3].tolist() == [3, 3, 3]
    assert b.attn_splits == min(32, -(-296 // (8 * 2)))
    # request segments (recurrent layers): one row each, padding segments have no rows
    assert b.segments.num == 8 and h["seg_count"][:8].tolist() == [1, 1, 1, 0, 0, 0, 0, 0]
    assert h["seg_row0"][:8].tolist() == list(range(8)) and h["seg_slot"][:3].tolist() == [0, 1, 2]
    assert h["seg_pos0"][:3].tolist() == [33, 34, 35]


def test_prefill_blocks_and_incremental_page_rows():
    bb = BatchBuilder(max_rows=4, max_tokens=256, max_model_len=256, group=8, kv_heads=1, device="cpu")   # 2 positions per block
    seg = Segment(2, list(range(100, 105)), 16, [7, 8], True, uid=5)
    b, rows = bb.fill([seg, Segment(0, [1, 2], 0, [3], False, uid=6)])
    h = bb.stage.h
    assert (b.num_tokens, b.num_row_blocks, rows) == (7, 4, 1)
    assert h["rb_qstart"][:4].tolist() == [0, 2, 4, 5] and h["rb_qcount"][:4].tolist() == [2, 2, 1, 2]
    assert h["rb_ctx"][:4].tolist() == [17, 19, 21, 1] and h["rb_req"][:4].tolist() == [2, 2, 2, 0]
    assert h["logit_rows"][0] == 4 and h["slots"][:5].tolist() == [8 * 16 + i for i in range(5)]
    assert b.segments.num == 2 and h["seg_row0"][:2].tolist() == [0, 5] and h["seg_count"][:2].tolist() == [5, 2]
    assert h["seg_slot"][:2].tolist() == [2, 0] and h["seg_pos0"][:2].tolist() == [16, 0]
    # the request grows by one page: only the new entry is written
    h["page_table"][2, 0] = 99                        # would be overwritten by a full rewrite
    seg2 = Segment(2, [1], 32, [7, 8, 9], True, uid=5)
    bb.fill([seg2])
    assert h["page_table"][2, :3].tolist() == [99, 8, 9]
    # a different request reusing the slot rewrites the row; so does an explicit invalidation
    bb.fill([Segment(2, [1], 0, [4], True, uid=6)])
    assert h["page_table"][2, 0] == 4
    h["page_table"][2, 0] = 55
    bb.invalidate_page_rows([2])
    bb.fill([Segment(2, [1], 1, [4], True, uid=6)])
    assert h["page_table"][2, 0] == 4


def test_page_rows_follow_a_request_through_preemption_and_readmission():
    """Scheduler + batch builder under tight memory: after every planned step the staged page-table row of each
    scheduled request equals the request's pages, also when a preempted request gets its old slot back with other
    pages (the row's identity changes with every admission)."""
    from cubic_serve_b200.runtime.engine import LLMEngine
    from cubic_serve_b200.runtime.scheduler import SamplingParams, SchedulerConfig

    class Ex:
        vocab_size = 97

        def __init__(self):
            self.bb = BatchBuilder(max_rows=6, max_tokens=128, max_model_len=128, group=4, kv_heads=2, device="cpu")
            self.invalidate_page_rows = self.bb.invalidate_page_rows
            self.checked = 0

        def copy_pages(self, pairs):
            pass

        def execute(self, segs):
            self.bb.fill(segs)
            table = self.bb.stage.h["page_table"]
            for s in segs:
                assert table[s.request_slot, :len(s.pages)].tolist() == list(s.pages), (s.request_slot, s.uid)
                self.checked += 1
            return np.asarray([(int(s.token_ids[-1]) * 31 + s.start) % 97 for s in segs if s.sample], dtype=np.int32)

    ex = Ex()
    eng = LLMEngine(ex, num_pages=14, scheduler_config=SchedulerConfig(
        max_running_requests=6, max_model_len=96, max_batched_tokens=96, prefill_chunk_tokens=48, enable_prefix_cache=False))
    reqs = [eng.requests[eng.add_request([(7 * r + i) % 97 for i in range(30 + r)],
                                         SamplingParams(max_tokens=30, ignore_eos=True), f"p{r}")] for r in range(6)]
    for _ in range(3000):
        if not eng.has_unfinished:
            break
        eng.step()
    assert not eng.has_unfinished and ex.checked > 100
    assert sum(r.preemptions for r in reqs) > 0


def test_same_slot_same_arrival_new_admission_rewrites_the_row():
    bb = BatchBuilder(max_rows=2, max_tokens=64, max_model_len=128, group=4, kv_heads=2, device="cpu")
    bb.fill([Segment(1, [5], 48, [7, 8, 9, 7], True, uid=(3 << 16) | 0)])
    # the same request (arrival 3) re-admitted after a preemption: same slot, same page count, other pages
    bb.fill([Segment(1, [5], 48, [4, 5, 6, 7], True, uid=(3 << 16) | 1)])
    assert bb.stage.h["page_table"][1, :4].tolist() == [4, 5, 6, 7]


def test_three_axis_positions_and_feature_rows_are_staged():
    import numpy as np
    import torch

    from cubic_serve_b200.executor.gpu_executor import BatchBuilder, Segment
    bb = BatchBuilder(max_rows=4, max_tokens=64, max_model_len=128, group=4, kv_heads=2, device="cpu")
    p3 = np.stack([np.arange(6), np.arange(6) + 2, np.arange(6) * 3]).astype(np.int32)
    feats = torch.ones(2, 8)
    segs = [Segment(0, list(range(6)), 0, [3], embeds=[(1, feats)], positions3=p3),
            Segment(1, [7, 8, 9], 16, [4, 5])]
    b, rows = bb.fill(segs)
    h = bb.stage.h
    assert b.positions_hw is not None and rows == 2
    assert h["positions"][:9].tolist() == [0, 1, 2, 3, 4, 5, 16, 17, 18]
    assert h["positions_h"][:9].tolist() == [2, 3, 4, 5, 6, 7, 16, 17, 18]
    assert h["positions_w"][:9].tolist() == [0, 3, 6, 9, 12, 15, 16, 17, 18]
    assert [(f, tuple(r.shape), r.dtype) for f, r in b.embeds] == [(1, (2, 8), torch.bfloat16)]
    assert h["slots"][6:9].tolist() == [5 * 16, 5 * 16 + 1, 5 * 16 + 2]       # cache slots follow the sequence index
    # equal axes: the one-axis kernel path; a decode row of a request with media sits at index + offset
    same = np.stack([np.arange(4) + 10] * 3).astype(np.int32)
    b2, _ = bb.fill([Segment(0, [1, 2, 3, 4], 10, [3])])
    assert b2.positions_hw is None and b2.embeds is None
    b3, _ = bb.fill([Segment(0, [1, 2, 3, 4], 10, [3], positions3=same)])
    assert b3.positions_hw is None
    b4, _ = bb.fill([Segment(0, [5], 40, [3, 4, 5], positions3=np.full((3, 1), 33, np.int32)), Segment(1, [6], 20, [6, 7])])
    assert h["positions"][:2].tolist() == [33, 20] and h["rb_ctx"][:2].tolist() == [41, 21]
