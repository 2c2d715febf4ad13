"""Per-rank GPU executor: batch metadata staging, CUDA-graph buckets, replay.

Mirrors the reference worker's replay path (``runtime/quantized_graph.py:1566``
command loop -> ``executor.replay_batch`` -> fill pinned metadata -> H2D ->
``graph.replay()`` -> sample) with one difference in structure: all per-step
metadata lives in ONE pinned byte buffer mirrored by ONE device buffer, so a
step is a single ``cudaMemcpyAsync`` followed by a graph launch and a single
D2H read of the sampled ids.

Decode steps replay graphs captured per power-of-two row capacity; prefill
chunks (variable token counts) launch the same kernels eagerly.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass

import numpy as np
import torch

from ..models.decoder import DecoderRunner, StepBatch
from ..ops import kernels as K
from .graph_runtime import CudaGraphRuntime, GraphState

log = logging.getLogger(__name__)


@dataclass
class Segment:
    """One request's slice of a step: ``count`` new tokens starting at ``start`` (its position)."""
    request_slot: int            # row of the persistent page table owned by the request
    token_ids: np.ndarray | list  # the new tokens (len == count)
    start: int                   # position of the first new token
    pages: np.ndarray | list     # physical page ids of the request, covering start + count tokens
    sample: bool = True          # whether the last token's logits are sampled
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = 0
    draw: int = 0
    uid: int = -1                # identity of the request owning the slot (page-table row reuse detection)
    mask: np.ndarray | None = None   # allowed-token bitmask of the sampled row (uint32 words, bit set = allowed)
    budget_init: int = -2        # thinking budget of the sampled row's request: -2 keep, -1 none, >= 0 (re)start with it
    # speculative rounds of a constrained request: callable(drafts) -> uint32 [len(drafts) + 1, words], row j = the
    # allowed tokens after the request's grammar has accepted drafts[:j] (the matcher is left where it was)
    mask_fn: object = None
    # multimodal prefill: ``embeds`` = [(offset into this segment's tokens, rows [n, hidden])] replace the embedding of
    # those tokens with encoder features; ``positions3`` = int [3, count] rotary positions (None: all axes = position)
    embeds: object = None
    positions3: object = None
    # [(offset, rows [n, layers, hidden])]: additions to the hidden state at media positions after the first decoder
    # layers (towers with intermediate outputs; executors that state ``accepts_deepstack``)
    deep_embeds: object = None


class _Staging:
    """Typed views over one pinned host buffer and its device mirror."""

    def __init__(self, max_tokens: int, max_rows: int, max_row_blocks: int, max_pages: int, device) -> None:
        self.max_tokens, self.max_rows, self.max_row_blocks, self.max_pages = max_tokens, max_rows, max_row_blocks, max_pages
        fields = [
            ("token_ids", np.int32, max_tokens), ("positions", np.int32, max_tokens), ("slots", np.int32, max_tokens),
            ("rb_req", np.int32, max_row_blocks), ("rb_qstart", np.int32, max_row_blocks),
            ("rb_qcount", np.int32, max_row_blocks), ("rb_ctx", np.int32, max_row_blocks),
            ("top_k", np.int32, max_rows), ("temperature", np.float32, max_rows), ("top_p", np.float32, max_rows),
            ("logit_rows", np.int64, max_rows), ("seeds", np.int64, max_rows), ("draws", np.int64, max_rows),
            # the step's rows grouped by request (recurrent layers walk a request's rows in order)
            ("seg_row0", np.int32, max_rows), ("seg_count", np.int32, max_rows), ("seg_slot", np.int32, max_rows),
            ("seg_pos0", np.int32, max_rows),
            # per sampled row: the request's slot and its thinking-budget command (device-side budget state machine)
            ("row_slot", np.int32, max_rows), ("budget_init", np.int32, max_rows),
            ("page_table", np.int32, max_rows * max_pages),
            # row- and column-axis rotary positions of multimodal prefill steps (``positions`` is the temporal axis)
            ("positions_h", np.int32, max_tokens), ("positions_w", np.int32, max_tokens),
        ]
        off = 0
        self.offsets = {}
        for name, dt, n in fields:
            off = (off + 15) & ~15
            self.offsets[name] = (off, dt, n)
            off += np.dtype(dt).itemsize * n
        self.nbytes = (off + 15) & ~15
        self.host = torch.empty(self.nbytes, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        self.dev = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.h_np = self.host.numpy()
        self.h = {}
        self.d = {}
        tmap = {np.int32: torch.int32, np.float32: torch.float32, np.int64: torch.int64}
        for name, (o, dt, n) in self.offsets.items():
            size = np.dtype(dt).itemsize * n
            self.h[name] = self.h_np[o:o + size].view(dt)
            self.d[name] = self.dev[o:o + size].view(tmap[dt])
        self.d["page_table"] = self.d["page_table"].view(max_rows, max_pages)
        self.h["page_table"] = self.h["page_table"].reshape(max_rows, max_pages)

    def upload(self, nbytes: int | None = None) -> int:
        n = self.nbytes if nbytes is None else nbytes
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        return n


class BatchBuilder:
    """Host side of a step: turns segments into the staged metadata arrays (no CUDA calls except the upload)."""

    def __init__(self, max_rows: int, max_tokens: int, max_model_len: int, group: int, kv_heads: int, device) -> None:
        self.qb = 16 // group                                   # query positions per attention row block
        self.kv_heads = kv_heads
        self.max_rows = max_rows
        self.max_tokens = max_tokens
        self.max_pages = -(-max_model_len // K.PAGE_TOKENS)
        max_rb = max(max_rows, max_tokens // self.qb + max_rows)
        self.stage = _Staging(max_tokens, max_rows, max_rb, self.max_pages, device)
        self.device = device
        self._page_rows: list[tuple[int, int]] = [(-2, 0)] * max_rows

    def _splits(self, row_blocks: int) -> int:
        from ..ops.strategies import active
        a = active().attention
        ctas = max(1, row_blocks * self.kv_heads)
        return int(min(a.max_splits, max(1, -(-a.target_ctas // ctas))))

    def fill(self, segs: list[Segment], pad_rows_to: int | None = None):
        return self._fill(segs, pad_rows_to)

    def _sync_page_row(self, s: Segment) -> None:
        """Bring row ``request_slot`` of the host page table up to date (only the new tail is written)."""
        slot = s.request_slot
        known_uid, known_len = self._page_rows[slot]
        pages = s.pages
        n = len(pages)
        if known_uid != s.uid or s.uid < 0 or n < known_len:
            self.stage.h["page_table"][slot, :n] = pages
        elif n > known_len:
            self.stage.h["page_table"][slot, known_len:n] = pages[known_len:]
        else:
            return
        self._page_rows[slot] = (s.uid, n)

    def invalidate_page_rows(self, slots) -> None:
        """Force a full rewrite of these page-table rows (used after copy-on-write replaced a page)."""
        for slot in slots:
            self._page_rows[slot] = (-2, 0)

    def _fill(self, segs: list[Segment], pad_rows_to: int | None = None) -> StepBatch:
        st = self.stage
        h = st.h
        qb = self.qb
        axes, embeds = False, []
        for s in segs:
            self._sync_page_row(s)
        if all(len(s.token_ids) == 1 for s in segs):
            # decode fast path: one token, one row block and one sampled row per segment
            n = len(segs)
            h["token_ids"][:n] = [s.token_ids[0] for s in segs]
            starts = np.fromiter((s.start for s in segs), dtype=np.int32, count=n)
            h["positions"][:n] = starts
            for i, s in enumerate(segs):
                if s.positions3 is not None:               # a request with media decodes at sequence index + its offset
                    h["positions"][i] = int(np.asarray(s.positions3)[0, 0])
            h["slots"][:n] = [s.pages[s.start >> 4] * 16 + (s.start & 15) for s in segs]
            h["rb_req"][:n] = [s.request_slot for s in segs]
            ar = np.arange(n, dtype=np.int32)
            h["rb_qstart"][:n] = ar
            h["rb_qcount"][:n] = 1
            h["rb_ctx"][:n] = starts + 1
            h["seg_row0"][:n] = ar
            h["seg_count"][:n] = 1
            h["seg_slot"][:n] = h["rb_req"][:n]
            h["seg_pos0"][:n] = starts
            t = rb = nseg = n
            rows = 0
            if all(s.sample for s in segs):
                h["row_slot"][:n] = h["rb_req"][:n]
                h["budget_init"][:n] = [s.budget_init for s in segs]
                h["logit_rows"][:n] = ar
                h["temperature"][:n] = [s.temperature for s in segs]
                h["top_p"][:n] = [s.top_p for s in segs]
                h["top_k"][:n] = [s.top_k for s in segs]
                h["seeds"][:n] = [s.seed for s in segs]
                h["draws"][:n] = [s.draw for s in segs]
                rows = n
            else:
                for i, s in enumerate(segs):
                    if s.sample:
                        h["logit_rows"][rows] = i
                        h["row_slot"][rows], h["budget_init"][rows] = s.request_slot, s.budget_init
                        h["temperature"][rows], h["top_p"][rows], h["top_k"][rows] = s.temperature, s.top_p, s.top_k
                        h["seeds"][rows], h["draws"][rows] = s.seed, s.draw
                        rows += 1
        else:
            t = rb = rows = 0
            nseg = len(segs)
            # three-axis rotary positions are staged only for steps in which some row's axes differ
            axes = any(s.positions3 is not None and not (np.asarray(s.positions3)[0] == np.asarray(s.positions3)[1:]).all()
                       for s in segs)
            for i, s in enumerate(segs):
                n = len(s.token_ids)
                h["seg_row0"][i], h["seg_count"][i], h["seg_slot"][i], h["seg_pos0"][i] = t, n, s.request_slot, s.start
                h["token_ids"][t:t + n] = s.token_ids
                pos = np.arange(s.start, s.start + n, dtype=np.int32)
                if s.positions3 is None:
                    h["positions"][t:t + n] = pos
                    if axes:
                        h["positions_h"][t:t + n] = pos
                        h["positions_w"][t:t + n] = pos
                else:
                    p3 = np.asarray(s.positions3, dtype=np.int32)
                    h["positions"][t:t + n], h["positions_h"][t:t + n], h["positions_w"][t:t + n] = p3[0], p3[1], p3[2]
                for off, feat in (s.embeds or ()):
                    embeds.append((t + off, feat))
                pages = np.asarray(s.pages, dtype=np.int32)
                h["slots"][t:t + n] = pages[pos >> 4] * 16 + (pos & 15)
                nb = -(-n // qb)
                starts = np.arange(nb, dtype=np.int32) * qb
                h["rb_req"][rb:rb + nb] = s.request_slot
                h["rb_qstart"][rb:rb + nb] = t + starts
                h["rb_qcount"][rb:rb + nb] = np.minimum(n - starts, qb)
                h["rb_ctx"][rb:rb + nb] = s.start + starts + 1
                rb += nb
                if s.sample:
                    h["logit_rows"][rows] = t + n - 1
                    h["row_slot"][rows], h["budget_init"][rows] = s.request_slot, s.budget_init
                    h["temperature"][rows], h["top_p"][rows], h["top_k"][rows] = s.temperature, s.top_p, s.top_k
                    h["seeds"][rows], h["draws"][rows] = s.seed, s.draw
                    rows += 1
                t += n
        if pad_rows_to is not None and pad_rows_to > t:
            # decode bucket padding: rows that write nothing and attend to nothing
            p = pad_rows_to
            h["token_ids"][t:p] = 0
            h["positions"][t:p] = 0
            h["slots"][t:p] = -1
            h["rb_req"][rb:p] = 0
            h["rb_qstart"][rb:p] = np.arange(rb, p, dtype=np.int32)
            h["rb_qcount"][rb:p] = 0
            h["rb_ctx"][rb:p] = 0
            h["logit_rows"][rows:p] = np.arange(rows, p)
            h["row_slot"][rows:p] = -1
            h["temperature"][rows:p] = 0
            h["seg_row0"][nseg:p] = np.arange(nseg, p, dtype=np.int32)
            h["seg_count"][nseg:p] = 0
            h["seg_slot"][nseg:p] = 0
            h["seg_pos0"][nseg:p] = 0
            t, rb, rows_cap, nseg = p, p, p, p
        else:
            rows_cap = rows
        d = st.d
        splits = self._splits(rb)
        return StepBatch(num_tokens=t, num_row_blocks=rb, num_logit_rows=rows_cap, token_ids=d["token_ids"],
                         positions=d["positions"], slots=d["slots"], page_table=d["page_table"], rb_req=d["rb_req"],
                         rb_qstart=d["rb_qstart"], rb_qcount=d["rb_qcount"], rb_ctx=d["rb_ctx"],
                         logit_rows=d["logit_rows"], attn_splits=splits,
                         segments=K.GdnSegments(d["seg_row0"], d["seg_count"], d["seg_slot"], d["seg_pos0"], nseg),
                         positions_hw=(d["positions_h"], d["positions_w"]) if axes else None,
                         embeds=[(first, feat.to(self.device, torch.bfloat16, non_blocking=True))
                                 for first, feat in embeds] or None), rows


class GpuExecutor:
    def __init__(self, runner: DecoderRunner, max_rows: int = 256, max_prefill_tokens: int = 8192,
                 max_model_len: int = 4096, use_graphs: bool = True, rows_per_request: int = 1) -> None:
        """``rows_per_request`` > 1 sizes the sampled-row staging for speculative review (K + 1 rows per request)."""
        self.runner = runner
        # encoder feature rows and three-axis positions are taken on one GPU by the plain executor (the speculative
        # executors and the tensor-parallel embedding path do not carry them)
        self.accepts_features = type(self) is GpuExecutor and runner.tp is None and getattr(runner, "pp", None) is None \
            and runner.cfg.mrope_section is not None
        self.cfg = runner.cfg
        self.device = runner.device
        self.max_rows = max_rows
        self.max_tokens = max(max_prefill_tokens, max_rows)
        assert self.max_tokens <= runner.max_tokens
        if runner.cfg.is_hybrid and max_rows > runner.max_requests:
            raise ValueError("the runner's recurrent state has fewer rows than the executor has request slots")
        self.builder = BatchBuilder(max_rows * rows_per_request, self.max_tokens, max_model_len,
                                    runner.hq // runner.hkv, runner.hkv, self.device)
        self.stage = self.builder.stage
        self._fill = self.builder._fill
        self.invalidate_page_rows = self.builder.invalidate_page_rows
        v_local = runner.w.lm_head.n
        self.logits = torch.empty(max_rows, v_local, dtype=torch.bfloat16, device=self.device)
        self.out_ids = torch.zeros(max_rows * rows_per_request, dtype=torch.int32, device=self.device)
        # two result buffers: a step may be launched before the previous step's ids have been read (``launch`` / ``collect``)
        self.out_host = torch.zeros(2, max_rows * rows_per_request, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.use_graphs = use_graphs
        self.graph_masks = False         # True once decode graphs were captured with the mask buffer as an input
        self.graph_rt = CudaGraphRuntime(resources=(0, 1))      # capture -> qualify -> seal -> replay; result-buffer leases
        self._leases: list = [None, None]
        self.stream = torch.cuda.Stream(device=self.device)
        self.h2d_bytes_last = 0
        self.d2h_bytes_last = 0
        self.kernel_launches_last = 0
        self.timing = False              # record device time of the compute part of every step
        self.device_ms: list[float] = []
        self._ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(2)]
        self._done = [torch.cuda.Event(), torch.cuda.Event()]
        self._uploaded = torch.cuda.Event()
        self._upload_pending = False
        self._launches = 0

    @property
    def reasoning_end_id(self) -> int | None:
        """Closing token of a reasoning block when thinking budgets are enforced on the device, else None."""
        r = self.runner.reasoning
        return None if r is None else r.end_token_id

    # ----------------------------------------------------------------- batches
    # ------------------------------------------------------------------- run
    def _body(self, b: StepBatch) -> None:
        self.runner.run_step(b, self.stage.d, self.logits, self.out_ids)

    def _mask_buffers(self) -> None:
        if getattr(self, "_mask_host", None) is None:
            words = -(-self.cfg.vocab_size // 32)
            rows = self.out_ids.numel()
            self._mask_host = torch.empty(rows, words, dtype=torch.int32, pin_memory=torch.cuda.is_available())
            self._mask_dev = torch.full((rows, words), -1, dtype=torch.int32, device=self.device)     # everything allowed
            self._mask_rows_dirty = 0

    def _stage_masks(self, segs: list[Segment]) -> bool:
        """Upload the allowed-token bitmasks of this step's sampled rows; rows without one allow everything.

        With ``graph_masks`` (set by ``capture_decode_graphs``) the sampler ALWAYS reads the device mask buffer, in
        graphs and eagerly: it holds all-ones rows except where a constrained step wrote masks, and those rows are
        reset by one fill when the next unconstrained step comes.  Constrained decode steps then replay the same
        graphs as any other.  Without it the mask is a step input only when a segment is constrained, and such steps
        run eagerly.  Returns whether this step carries masks.
        """
        sampled = [s for s in segs if s.sample]
        constrained = any(s.mask is not None for s in sampled)
        if not constrained:
            if self.graph_masks:
                if self._mask_rows_dirty:
                    with torch.cuda.stream(self.stream):
                        self._mask_dev[:self._mask_rows_dirty].fill_(-1)
                    self._mask_rows_dirty = 0
            else:
                self.stage.d.pop("mask", None)
            return False
        self._mask_buffers()
        words = self._mask_host.shape[1]
        hm = self._mask_host.numpy().view(np.uint32)
        for i, s in enumerate(sampled):
            if s.mask is None:
                hm[i] = 0xFFFFFFFF
            else:
                hm[i] = s.mask
        n = len(sampled)
        with torch.cuda.stream(self.stream):
            self._mask_dev[:n].copy_(self._mask_host[:n], non_blocking=True)
        self._mask_rows_dirty = max(self._mask_rows_dirty, n)
        self.stage.d["mask"] = self._mask_dev
        self.h2d_mask_bytes_last = n * words * 4
        return True

    def capture_decode_graphs(self, capacities: list[int] | None = None) -> list[int]:
        """Capture one graph per decode row capacity (largest first, like the reference)."""
        caps = capacities or [c for c in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512) if c <= self.max_rows]
        # the captured sampler reads the mask buffer (all-ones rows unless a constrained step wrote masks), so that
        # structured-output requests decode in the same graphs; 4 bytes per 32 vocabulary entries and row
        self._mask_buffers()
        self.graph_masks = True
        self.stage.d["mask"] = self._mask_dev
        rt = CudaGraphRuntime(resources=(0, 1))
        if isinstance(getattr(self.runner, "attn", None), torch.Tensor):
            with torch.cuda.stream(self.stream):
                self.runner.attn.zero_()     # padding rows are not written by attention: give the comparison defined values
        for cap in sorted(caps, reverse=True):
            dummy = [Segment(0, [0], 0, [0])]
            b, _ = self._fill(dummy, pad_rows_to=cap)
            self.invalidate_page_rows([0])
            # the warm-up run below must not touch real cache pages: the single real row is turned into padding too
            self.stage.h["slots"][:cap] = -1
            self.stage.h["rb_qcount"][:cap] = 0
            self.stage.upload()
            with torch.cuda.stream(self.stream):
                for _ in range(2):
                    self._body(b)
                self.stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self._body(b)
                rt.add(cap, g, self.runner.launches_per_step)
                rt.qualify(cap, lambda slot: self._replay_equals_eager(slot, b, cap))
        torch.cuda.synchronize(self.device)
        ready = rt.seal()
        self.graph_rt = rt
        for c, why in rt.poison_log:
            log.error("decode graph for %d rows is out of service: %s", c, why)
        self.execution_plan = self._describe_execution(sorted(ready.sealed))
        return list(ready.sealed)

    def _describe_execution(self, capacities):
        """The sealed execution plan of this rank: topology, replayable capacities and the operator signatures of a
        decode step at the largest one, sealed with the implementation identity and the device (what the ranks of a
        deployment compare before they declare themselves ready)."""
        from ..contracts.implementation import identity
        from ..contracts.plan import ExecutionPlan, decoder_step_operators
        if not capacities:
            return None
        tp = self.runner.tp_size
        topo = f"tp{tp}" + (f"pp{self.runner.pp.stages}" if self.runner.pp is not None and hasattr(self.runner.pp, "stages") else "")
        try:
            impl = identity().digest
        except Exception:  # noqa: BLE001 - identity is evidence, not a precondition of serving
            impl = "unknown"
        plan = ExecutionPlan(topo, tuple(capacities), decoder_step_operators(self.cfg, max(capacities), tp, topo))
        return plan.seal(impl, torch.cuda.get_device_name(self.device))

    def _replay_equals_eager(self, slot, b: StepBatch, cap: int):
        """Qualification of a captured decode graph: the eager step on the capture inputs and one replay must sample
        the same ids and produce the same logits (to rounding of differently ordered partial sums).  Runs on
        ``self.stream``, inside ``capture_decode_graphs``."""
        self.logits[:cap].zero_()              # rows a step does not write (another pipeline stage samples) compare equal
        self.out_ids[:cap].fill_(-7)
        self._body(b)
        self.stream.synchronize()
        want_ids, want = self.out_ids[:cap].clone(), self.logits[:cap].float()
        self.logits[:cap].zero_()
        self.out_ids[:cap].fill_(-7)
        slot.graph.replay()
        self.stream.synchronize()
        got = self.logits[:cap].float()
        # the capture inputs are padding rows: what attention leaves unwritten for them may be anything, non-finite
        # included, but it is the same memory for both runs
        finite = torch.isfinite(want)
        if not torch.equal(finite, torch.isfinite(got)):
            return "the replay's logits are non-finite where the eager step's are finite (or the reverse)"
        got, want = torch.where(finite, got, 0.0), torch.where(finite, want, 0.0)
        err = ((got - want).norm() / want.norm().clamp_min(1e-12)).item()
        if err > 1e-3:
            return f"replayed logits differ from the eager step's (relative L2 {err:.3g})"
        if not torch.equal(self.out_ids[:cap], want_ids):
            return "the replay sampled other ids than the eager step"
        return True

    @property
    def graphs(self) -> dict:
        """Sealed decode graphs by capacity (read-only view)."""
        return {c: s.graph for c, s in self.graph_rt.slots.items() if s.state is GraphState.SEALED}

    @property
    def state_checkpoint_rows(self) -> tuple[int, ...]:
        return tuple(getattr(self.runner, "state_checkpoint_rows", ()))

    def copy_state(self, pairs) -> None:
        """Recurrent-state row copies ``(src row, dst row)`` in stream order with the steps: a snapshot taken after the
        step that ended on a page boundary, or a snapshot restored into the row of a request that resumes there."""
        if not pairs:
            return
        src = torch.tensor([p[0] for p in pairs], dtype=torch.int32, device=self.device)
        dst = torch.tensor([p[1] for p in pairs], dtype=torch.int32, device=self.device)
        with torch.cuda.stream(self.stream):
            self.runner.copy_state(src, dst)

    def copy_pages(self, pairs) -> None:
        """Copy-on-write page copies (all layers) ahead of a step."""
        if not pairs:
            return
        src = torch.tensor([p[0] for p in pairs], dtype=torch.int32, device=self.device)
        dst = torch.tensor([p[1] for p in pairs], dtype=torch.int32, device=self.device)
        with torch.cuda.stream(self.stream):
            for cache in self.runner.kv:
                K.copy_pages(cache, src, dst)

    def execute(self, segs: list[Segment]) -> np.ndarray:
        """Run one step and return the sampled token id of every sampling segment (host array)."""
        return self.collect(self.launch(segs))

    def launch(self, segs: list[Segment], feedback_rows: int = 0) -> dict:
        """Enqueue one step without waiting for it: stage + upload the inputs, replay the graph (or run eagerly),
        enqueue the device -> host copy of the sampled ids.  ``collect`` waits and returns them.

        ``feedback_rows`` > 0: the input token of row ``i < feedback_rows`` is the id the PREVIOUS launch sampled for
        its row ``i`` (copied on the device, the host does not know it yet): the engine uses it to launch a decode
        step while it still processes the previous step's results.  At most two launches may be outstanding.
        """
        total = sum(len(s.token_ids) for s in segs)
        masked = self._stage_masks(segs)
        decode = (all(len(s.token_ids) == 1 for s in segs) and self.use_graphs and (self.graph_masks or not masked))
        cap = self.graph_rt.dispatch(total) if decode else None
        if self._upload_pending:
            # the pinned staging buffer is rewritten below: the previous launch's upload must have left it
            self._uploaded.synchronize()
            self._upload_pending = False
        b, rows = self._fill(segs, pad_rows_to=cap)
        if cap is not None and getattr(self, "audit_poison_padding", False):
            self._poison_padding(total, cap)
        k = self._launches & 1
        # the result buffer of this launch must have been collected: a third outstanding launch is an error, not an overwrite
        self._leases[k] = self.graph_rt.leases.acquire(k, f"launch {self._launches}")
        self._launches += 1
        with torch.cuda.stream(self.stream):
            h2d = self.stage.upload()
            self._uploaded.record(self.stream)
            self._upload_pending = True
            if feedback_rows:
                self.stage.d["token_ids"][:feedback_rows].copy_(self.out_ids[:feedback_rows], non_blocking=True)
            if self.timing:
                self._ev[k][0].record(self.stream)
            if cap is not None:
                launches = self.graph_rt.replay(cap, self._leases[k]).launches
            else:
                self._body(b)
                launches = self.runner.launches_per_step
            if self.timing:
                self._ev[k][1].record(self.stream)
            if rows:
                self.out_host[k, :rows].copy_(self.out_ids[:rows], non_blocking=True)
            self._done[k].record(self.stream)
        return {"k": k, "rows": rows, "h2d": h2d, "launches": launches}

    def _poison_padding(self, rows: int, cap: int) -> None:
        """Audit facility (``guardrail/graph_audit.py``): the padding rows ``[rows, cap)`` of a decode bucket get random
        token ids and positions, and the activations that a step leaves unwritten for them (the attention output) are
        filled with NaN, so that any path from a padding row into a real row shows up in the real rows' logits.  The
        rows still write no cache slot and attend to nothing."""
        rng = np.random.default_rng(rows * 7919 + cap)
        h = self.stage.h
        h["token_ids"][rows:cap] = rng.integers(0, self.cfg.vocab_size, cap - rows)
        h["positions"][rows:cap] = rng.integers(0, 1 << 12, cap - rows)
        attn = getattr(self.runner, "attn", None)
        if isinstance(attn, torch.Tensor):
            with torch.cuda.stream(self.stream):
                attn[rows:cap].fill_(float("nan"))

    def collect(self, handle: dict) -> np.ndarray:
        """Wait for a launched step and return its sampled ids (host array)."""
        k, rows = handle["k"], handle["rows"]
        self._done[k].synchronize()
        self.graph_rt.leases.release(self._leases[k])
        self._leases[k] = None
        self.h2d_bytes_last = handle["h2d"]
        self.kernel_launches_last = handle["launches"]
        self.d2h_bytes_last = rows * 4
        if self.timing:
            self.device_ms.append(self._ev[k][0].elapsed_time(self._ev[k][1]))
        return self.out_host[k, :rows].numpy().copy()
