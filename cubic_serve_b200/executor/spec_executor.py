"""Speculative decoding round on the GPU: MTP proposals -> target review -> verification (greedy, or p / q rejection
sampling when a request of the round samples).

One round, in the order of the reference's ``execute_draft_batch`` (``runtime/performance.py:7189-7556`` there):
(1) proposal passes of the MTP head, depth by depth, chaining draft tokens and hidden states on the device;
(2) ONE target pass over ``[root, d1 .. dK]`` per request (segment length K + 1, every row sampled);
(3) verification on the device: greedy requests keep the longest matching prefix (bonus token = the target's choice
    after it); with a sampling request in the round every draft is DRAWN from the head's shaped distribution q and
    accepted with probability min(1, p / q) against the target's p, the first rejected position is redrawn from
    normalise(max(0, p - q)) (``csrc/sampling.cu::verify_sampled_kernel``; reference
    ``generation/tp_sampling.py:154-217``), so the emitted tokens are distributed as plain sampling from p;
(4) the hidden state of the last accepted position becomes the head's input for the next round.
Rejected positions need no repair: their KV slots are simply rewritten by the next round.

``force_acceptance`` replaces natural agreement by a seeded per-depth Bernoulli draw -- only meaningful for
benchmarks with random weights, where a draft never matches on its own.
"""
from __future__ import annotations

import numpy as np
import torch

from ..models.mtp import MtpRunner
from ..ops import kernels as K
from .gpu_executor import GpuExecutor, Segment


class SpeculativeGpuExecutor(GpuExecutor):
    speculative_sampling = True      # rounds also serve requests with temperature > 0 (p / q rejection sampling)
    speculative_grammar = True       # ... and constrained requests: every review row is sampled under the grammar's mask

    def __init__(self, runner, mtp: MtpRunner, depth: int, force_acceptance: float | None = None, seed: int = 0,
                 round_graphs: bool = True, **kw) -> None:
        # models with Gated DeltaNet layers: the review pass leaves the recurrent state untouched and the accepted
        # prefix is folded into it afterwards (DecoderRunner.begin_gdn_review / fold_gdn)
        super().__init__(runner, rows_per_request=depth + 1, use_graphs=False, **kw)
        self.mtp = mtp
        if runner.tp is not None:
            # vocabulary-sharded logits: drafts and review rows are sampled by the candidate exchange + merge of the
            # tensor-parallel sampler (greedy requests; p / q verification needs merged candidate lists)
            self.speculative_sampling = False
        self.speculative_depth = depth
        self.force_acceptance = force_acceptance
        self._rng = np.random.default_rng(seed)
        dev, H = self.device, runner.cfg.hidden_size
        rows = self.max_rows
        self.last_hidden = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)      # by request slot
        self.hidden_rows = torch.empty(runner.max_tokens, H, dtype=torch.bfloat16, device=dev)
        self.draft_ids = torch.zeros(rows, depth, dtype=torch.int32, device=dev)
        self.target_ids = torch.zeros(rows, depth + 1, dtype=torch.int32, device=dev)
        self.accepted = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.bonus = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.depth_t = torch.full((rows,), depth, dtype=torch.int32, device=dev)
        self.forced = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.mtp_logits = torch.empty(rows, runner.w.lm_head.n, dtype=torch.bfloat16, device=dev)
        # candidate distributions of a sampled round: the head's (q) per draft, the target's (p) per review row
        C = K.SAMPLE_CANDIDATES
        self.q_val = torch.zeros(rows * depth, C, dtype=torch.float32, device=dev)
        self.q_id = torch.zeros(rows * depth, C, dtype=torch.int32, device=dev)
        self.p_val = torch.zeros(rows * (depth + 1), C, dtype=torch.float32, device=dev)
        self.p_id = torch.zeros(rows * (depth + 1), C, dtype=torch.int32, device=dev)
        self.cand_tmp = (torch.zeros(rows, C, dtype=torch.float32, device=dev), torch.zeros(rows, C, dtype=torch.int32, device=dev))
        self.stats = {"rounds": 0, "accepted": 0, "proposed": 0, "emitted": 0, "graphed_rounds": 0}
        # captured rounds (greedy requests of models without recurrent layers on one GPU): one graph per row capacity
        # for a proposal pass of the head, one per (capacity, depth) for review + verification; see _round_graphed
        self.round_graphs = bool(round_graphs) and runner.tp is None and not runner.gdn_state and runner.pp is None
        self._round_graph: dict = {}
        self.g_prev = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)       # hidden that precedes a proposal row
        self.g_tok = torch.zeros(rows, dtype=torch.int32, device=dev)              # proposal input token / sampled draft
        self.g_hid_sel = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)    # target hidden of the last accepted row
        self._rl = torch.empty(rows * (depth + 1), runner.w.lm_head.n, dtype=torch.bfloat16, device=dev)

    # ------------------------------------------------------------- plain steps
    def execute(self, segs):
        """Prefill / non-speculative steps also feed the MTP head (its KV cache and ``last_hidden``)."""
        ids = self._execute_with_hidden(segs)
        return ids

    def _execute_with_hidden(self, segs):
        total = sum(len(s.token_ids) for s in segs)
        masked = self._stage_masks(segs)                # allowed-token masks of constrained requests' sampled rows
        b, rows = self._fill(segs)
        r = self.runner
        with torch.cuda.stream(self.stream):
            self.h2d_bytes_last = self.stage.upload()
            hidden = r.forward_hidden(b)
            d = self.stage.d
            if rows:
                logits = r.forward_logits(b, hidden, self.logits)
                mask = d["mask"][:rows, r.w.vocab_start // 32:] if masked else None
                if r.tp is None:
                    K.sample(logits, self.out_ids[:rows], temperature=d["temperature"][:rows], top_p=d["top_p"][:rows],
                             top_k=d["top_k"][:rows], seeds=d["seeds"][:rows], counters=d["draws"][:rows],
                             vocab=logits.shape[1], mask=mask)
                else:
                    r.tp.sample_sharded_nccl(logits, rows, self.out_ids, d, r.w.vocab_start, mask)
            # MTP pass over the same rows: row i is preceded by the target hidden of row i - 1 (the first row of a
            # segment by the request's carried hidden)
            prev = self.hidden_rows[:total]
            prev[1:].copy_(hidden[:total - 1])
            first, last, slots = [], [], []
            t = 0
            for s in segs:
                first.append(t)
                t += len(s.token_ids)
                last.append(t - 1)
                slots.append(s.request_slot)
            fi = torch.tensor(first, device=self.device)
            la = torch.tensor(last, device=self.device)
            sl = torch.tensor(slots, device=self.device)
            prev.index_copy_(0, fi, self.last_hidden.index_select(0, sl))
            self.mtp.forward(b, prev)
            self.last_hidden.index_copy_(0, sl, hidden.index_select(0, la))
            if rows:
                self.out_host[0, :rows].copy_(self.out_ids[:rows], non_blocking=True)
            self.stream.synchronize()
        self.kernel_launches_last = r.launches_per_step + self.mtp.launches + 3
        self.d2h_bytes_last = rows * 4
        return self.out_host[0, :rows].numpy().copy()

    # ------------------------------------------------------- speculative round
    def execute_speculative(self, segs: list[Segment], depths: list[int] | None = None):
        """``segs``: one decode segment per request (its root token).  Returns per request the emitted tokens.

        ``depths`` (dynamic draft length, one entry per request, each <= the configured depth): the round runs
        ``max(depths)`` proposal passes and a review of that length; a request with a smaller depth only has
        that many of its drafts verified.  All zero = a plain decode step.
        """
        R = len(segs)
        Kd = self.speculative_depth if depths is None else min(self.speculative_depth, max(depths, default=0))
        if Kd == 0:
            ids = self.execute(segs)
            self.last_round = {"depth": 0, "accepted": [0] * R, "proposed": [0] * R, "proposal_ms": 0.0,
                               "target_ms": self.device_ms[-1] if (self.timing and self.device_ms) else 0.0}
            return [[int(t)] for t in ids]
        per_req = [Kd] * R if depths is None else [min(int(d), Kd) for d in depths]
        r, dev = self.runner, self.device
        if (self.round_graphs and not any(s.temperature > 0 or s.mask_fn is not None for s in segs)):
            return self._round_graphed(segs, Kd, per_req)
        sl = torch.tensor([s.request_slot for s in segs], device=dev)
        launches = 0
        # compact [R, Kd] / [R, Kd + 1] views: the verification kernel's row strides follow the round's depth
        draft_ids = self.draft_ids.view(-1)[:R * Kd].view(R, Kd)
        target_ids = self.target_ids.view(-1)[:R * (Kd + 1)].view(R, Kd + 1)
        self.depth_t[:R].copy_(torch.tensor(per_req, dtype=torch.int32), non_blocking=True)
        # a round with a sampling request draws its drafts and verifies by rejection sampling; forced acceptance is a
        # benchmark device of the greedy path
        self._sampling = None
        if any(s.temperature > 0 for s in segs) and self.force_acceptance is None:
            self._sampling = {
                "temperature": torch.tensor([s.temperature for s in segs], dtype=torch.float32, device=dev),
                "top_p": torch.tensor([s.top_p for s in segs], dtype=torch.float32, device=dev),
                "top_k": torch.tensor([s.top_k for s in segs], dtype=torch.int32, device=dev),
                "seeds": torch.tensor([s.seed for s in segs], dtype=torch.int64, device=dev),
                "draws": torch.tensor([s.draw for s in segs], dtype=torch.int64, device=dev)}
        sm = self._sampling
        with torch.cuda.stream(self.stream):
            ev0, ev1 = self._ev[0]
            if not hasattr(self, "_ev_mid"):
                self._ev_mid = torch.cuda.Event(enable_timing=True)
            if self.timing:
                ev0.record(self.stream)
            prev = self.last_hidden.index_select(0, sl)
            # ---- proposals: depth d consumes the token at position start + d - 1
            for d in range(Kd):
                step = [Segment(s.request_slot, [s.token_ids[0] if d == 0 else 0], s.start + d, s.pages, True, uid=s.uid)
                        for s in segs]
                b, _ = self._fill(step)
                self.h2d_bytes_last = self.stage.upload()
                if d > 0:
                    self.stage.d["token_ids"][:R].copy_(draft_ids[:, d - 1])
                hid = self.mtp.forward(b, prev)
                lg = self.mtp.logits(hid, R, self.mtp_logits)
                tmp = self.out_ids[:R]
                if sm is None:
                    self._sample_greedy(lg, R, tmp)
                else:
                    # the draft is drawn from the head's shaped distribution; its candidates are kept as q.  Draft draws
                    # live in their own part of the request's Philox stream (sub-stream 0x4000 + depth)
                    cv, ci = self.cand_tmp[0][:R], self.cand_tmp[1][:R]
                    K.sample_candidates(lg, cv, ci, temperature=sm["temperature"], top_k=sm["top_k"], vocab=lg.shape[1])
                    self.q_val[:R * Kd].view(R, Kd, -1)[:, d].copy_(cv)
                    self.q_id[:R * Kd].view(R, Kd, -1)[:, d].copy_(ci)
                    K.sample(lg, tmp, temperature=sm["temperature"], top_p=sm["top_p"], top_k=sm["top_k"],
                             seeds=sm["seeds"], counters=sm["draws"] | ((0x4000 + d) << 40), vocab=lg.shape[1])
                    launches += 3
                draft_ids[:, d].copy_(tmp)
                prev = hid[:R].clone()
                launches += self.mtp.launches + 4
            if self.timing:
                self._ev_mid.record(self.stream)
            self._review_mask = self._grammar_masks(segs, Kd, draft_ids)
            hidden = self._review_and_verify(segs, Kd, draft_ids, target_ids)
            launches += r.launches_per_step + 1
            rows = torch.arange(R, device=dev) * (Kd + 1) + self.accepted[:R].long()
            self.last_hidden.index_copy_(0, sl, hidden.index_select(0, rows))
            if self.timing:
                ev1.record(self.stream)
            acc = self.accepted[:R].cpu()
            tg = target_ids.cpu()
            self.stream.synchronize()
        prop_ms = tgt_ms = 0.0
        if self.timing:
            self.device_ms.append(ev0.elapsed_time(ev1))
            prop_ms, tgt_ms = ev0.elapsed_time(self._ev_mid), self._ev_mid.elapsed_time(ev1)
        out = []
        for i in range(R):
            a = int(acc[i])
            out.append([int(t) for t in tg[i, :a + 1]])
            self.stats["accepted"] += a
            self.stats["emitted"] += a + 1
        self.stats["rounds"] += 1
        self.stats["proposed"] += sum(per_req)
        self.last_round = {"depth": Kd, "accepted": [int(a) for a in acc], "proposed": per_req, "proposal_ms": prop_ms,
                           "target_ms": tgt_ms}
        self.kernel_launches_last = launches + 2
        self.d2h_bytes_last = R * (Kd + 2) * 4
        return out

    # ---------------------------------------------------------- captured rounds
    @staticmethod
    def _capacity(n: int) -> int:
        c = 1
        while c < n:
            c *= 2
        return c

    def _staged(self, segs, pad_rows_to=None):
        """``_fill`` + upload, after the previous upload has left the pinned staging buffer (with captured passes the
        host runs far ahead of the device)."""
        if self._upload_pending:
            self._uploaded.synchronize()
        b, _ = self._fill(segs, pad_rows_to=pad_rows_to)
        return b

    def _upload(self) -> int:
        n = self.stage.upload()
        self._uploaded.record(self.stream)
        self._upload_pending = True
        return n

    def _proposal_body(self, b, cap: int) -> None:
        self.stage.d["token_ids"][:cap].copy_(self.g_tok[:cap])
        hid = self.mtp.forward(b, self.g_prev)
        lg = self.mtp.logits(hid, cap, self.mtp_logits)
        K.sample(lg, self.g_tok[:cap], vocab=lg.shape[1])
        self.g_prev[:cap].copy_(hid[:cap])

    def _review_body(self, b, cap: int, Kd: int, draft_ids: torch.Tensor, target_ids: torch.Tensor) -> None:
        r, T = self.runner, cap * (Kd + 1)
        self.stage.d["token_ids"][:T].view(cap, Kd + 1)[:, 1:].copy_(draft_ids)
        hidden = r.forward_hidden(b)
        logits = r.forward_logits(b, hidden, self._rl)
        K.sample(logits, target_ids.view(-1), vocab=logits.shape[1])
        forced = None
        if self.force_acceptance is not None:
            # forced acceptance: the draft is *declared* equal to the target up to the depth drawn on the host
            forced = self.forced
            keep = torch.arange(Kd, device=self.device)[None, :] < self.forced[:cap, None]
            draft_ids.copy_(torch.where(keep, target_ids[:, :Kd], draft_ids))
        K.verify_greedy(target_ids, draft_ids, self.depth_t[:cap], Kd, self.accepted, self.bonus, forced)
        rows = torch.arange(cap, device=self.device) * (Kd + 1) + self.accepted[:cap].long()
        self.g_hid_sel[:cap].copy_(hidden.index_select(0, rows))

    def _captured(self, key, body, restore) -> "torch.cuda.CUDAGraph":
        """The graph for ``key``, captured on first use from the staged inputs of the current round: two eager runs, the
        capture, and ``restore()`` before each so that every run (and the first replay) starts from the same inputs."""
        g = self._round_graph.get(key)
        if g is None:
            for _ in range(2):
                body()
                restore()
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                body()
            restore()
            self._round_graph[key] = g
        return g

    def _round_graphed(self, segs: list[Segment], Kd: int, per_req: list[int]):
        """A round of greedy requests on captured graphs: per proposal pass one replay of the head's graph for the row
        capacity, then one replay of the review + verification graph for (capacity, depth).  The host stages the
        inputs of each pass (positions, cache slots, page tables; tokens and hidden states chain on the device) and
        reads back accepted counts and tokens once.  Reference: one captured graph per (review capacity, depth),
        ``executor/draft_graph.py:574`` there; here the proposal passes are graphs of their own so that one capture
        serves every depth."""
        R, dev, r = len(segs), self.device, self.runner
        cap = self._capacity(R)
        draft_ids = self.draft_ids.view(-1)[:cap * Kd].view(cap, Kd)
        target_ids = self.target_ids.view(-1)[:cap * (Kd + 1)].view(cap, Kd + 1)
        depth_host = torch.zeros(cap, dtype=torch.int32)
        depth_host[:R] = torch.tensor(per_req, dtype=torch.int32)
        sl = torch.tensor([s.request_slot for s in segs], device=dev)
        if not hasattr(self, "_ev_mid"):
            self._ev_mid = torch.cuda.Event(enable_timing=True)
        launches = 0
        with torch.cuda.stream(self.stream):
            ev0, ev1 = self._ev[0]
            if self.timing:
                ev0.record(self.stream)
            self.depth_t[:cap].copy_(depth_host, non_blocking=True)
            self.g_prev[:R].copy_(self.last_hidden.index_select(0, sl))
            for d in range(Kd):
                step = [Segment(s.request_slot, [s.token_ids[0] if d == 0 else 0], s.start + d, s.pages, True, uid=s.uid)
                        for s in segs]
                b = self._staged(step, pad_rows_to=cap)
                self.h2d_bytes_last = self._upload()
                if d == 0:
                    self.g_tok[:cap].copy_(self.stage.d["token_ids"][:cap])
                restore = None
                if ("proposal", cap) not in self._round_graph:
                    keep_tok, keep_prev = self.g_tok[:cap].clone(), self.g_prev[:cap].clone()

                    def restore():
                        self.g_tok[:cap].copy_(keep_tok)
                        self.g_prev[:cap].copy_(keep_prev)
                self._captured(("proposal", cap), lambda: self._proposal_body(b, cap), restore).replay()
                draft_ids[:, d].copy_(self.g_tok[:cap])
                launches += 4
            if self.timing:
                self._ev_mid.record(self.stream)
            # review rows: the requests' [root, d1 .. dK], then whole dummy requests up to the capacity; their rows
            # write no cache slot and attend to nothing
            pad_slot = self.max_rows                       # a page-table row no request uses
            review = [Segment(s.request_slot, [s.token_ids[0]] + [0] * Kd, s.start, s.pages, True, uid=s.uid) for s in segs]
            review += [Segment(pad_slot, [0] * (Kd + 1), 0, [0], True, uid=-1) for _ in range(cap - R)]
            b = self._staged(review)
            T, Tr = cap * (Kd + 1), R * (Kd + 1)
            h = self.stage.h
            nb = -(-(Kd + 1) // self.builder.qb)
            h["slots"][Tr:T] = -1
            h["rb_qcount"][R * nb:cap * nb] = 0
            h["logit_rows"][:T] = np.arange(T)
            h["temperature"][:T] = 0
            b.num_logit_rows = T
            self.h2d_bytes_last += self._upload()
            if self.force_acceptance is not None:
                draws = self._rng.random((R, Kd)) < self.force_acceptance
                first_fail = np.zeros(cap, dtype=np.int32)
                first_fail[:R] = np.where(draws.all(1), Kd, draws.argmin(1))
                self.forced[:cap].copy_(torch.from_numpy(first_fail), non_blocking=False)
            restore_review = None
            if ("review", cap, Kd) not in self._round_graph:
                keep_drafts = draft_ids.clone()

                def restore_review():
                    draft_ids.copy_(keep_drafts)
            self._captured(("review", cap, Kd), lambda: self._review_body(b, cap, Kd, draft_ids, target_ids),
                           restore_review).replay()
            self.last_hidden.index_copy_(0, sl, self.g_hid_sel[:R])
            launches += 6
            if self.timing:
                ev1.record(self.stream)
            acc = self.accepted[:R].cpu()
            tg = target_ids[:R].cpu()
            self.stream.synchronize()
        prop_ms = tgt_ms = 0.0
        if self.timing:
            self.device_ms.append(ev0.elapsed_time(ev1))
            prop_ms, tgt_ms = ev0.elapsed_time(self._ev_mid), self._ev_mid.elapsed_time(ev1)
        out = []
        for i in range(R):
            a = int(acc[i])
            out.append([int(t) for t in tg[i, :a + 1]])
            self.stats["accepted"] += a
            self.stats["emitted"] += a + 1
        self.stats["rounds"] += 1
        self.stats["graphed_rounds"] += 1
        self.stats["proposed"] += sum(per_req)
        self.last_round = {"depth": Kd, "accepted": [int(a) for a in acc], "proposed": per_req, "proposal_ms": prop_ms,
                           "target_ms": tgt_ms}
        # kernels inside the replayed graphs count as launched kernels of this step
        self.kernel_launches_last = launches + Kd * (self.mtp.launches + 3) + r.launches_per_step + 6
        self.d2h_bytes_last = R * (Kd + 2) * 4
        return out

    def _grammar_masks(self, segs: list[Segment], Kd: int, draft_ids: torch.Tensor):
        """Allowed-token masks of the review rows when a request of the round is constrained: row j of a request is
        sampled under its grammar's state after drafts[:j] (reference: the per-round grammar transactions of
        ``generation/constraints.py`` there).  The drafts are read back for this, so a constrained round pays one
        synchronisation between proposals and review; rounds without constraints do not.  Returns a device tensor
        ``[R (Kd + 1), words]`` or None."""
        if not any(s.mask_fn is not None for s in segs):
            return None
        R, T = len(segs), len(segs) * (Kd + 1)
        drafts = draft_ids.cpu().numpy()                   # synchronises with the proposal passes on this stream
        words = -(-self.cfg.vocab_size // 32)
        if getattr(self, "_rm_host", None) is None or self._rm_host.shape[0] < T:
            self._rm_host = torch.empty(max(T, self.max_rows * (self.speculative_depth + 1)), words, dtype=torch.int32,
                                        pin_memory=True)
            self._rm_dev = torch.empty_like(self._rm_host, device=self.device)
        hm = self._rm_host.numpy().view(np.uint32)
        hm[:T] = 0xFFFFFFFF
        for i, s in enumerate(segs):
            if s.mask_fn is not None:
                hm[i * (Kd + 1):(i + 1) * (Kd + 1)] = s.mask_fn([int(t) for t in drafts[i]])
        self._rm_dev[:T].copy_(self._rm_host[:T], non_blocking=True)
        return self._rm_dev[:T]

    def _review_and_verify(self, segs: list[Segment], Kd: int, draft_ids: torch.Tensor, target_ids: torch.Tensor) -> torch.Tensor:
        """ONE target pass over ``[root, d1 .. dK]`` of every request (greedy ids of all rows into ``target_ids``) and
        the device-side verification (``self.accepted``, ``self.bonus``; per-request depths in ``self.depth_t``).
        Runs on ``self.stream``; returns the hidden states of the review rows."""
        r, dev = self.runner, self.device
        R = len(segs)
        review = [Segment(s.request_slot, [s.token_ids[0]] + [0] * Kd, s.start, s.pages, True, uid=s.uid) for s in segs]
        b, _ = self._fill(review)
        T = R * (Kd + 1)
        self.stage.h["logit_rows"][:T] = np.arange(T)
        self.stage.h["temperature"][:T] = 0
        self.h2d_bytes_last = self.stage.upload()
        toks = torch.cat([torch.tensor([s.token_ids[0] for s in segs], dtype=torch.int32, device=dev)[:, None],
                          draft_ids], 1).reshape(-1)
        self.stage.d["token_ids"][:T].copy_(toks)
        b.num_logit_rows = T
        r.begin_gdn_review(T)
        hidden = r.forward_hidden(b)
        logits = r.forward_logits(b, hidden, self._review_logits(T))
        hidden = self._verify(segs, Kd, draft_ids, target_ids, logits, hidden)
        if r.gdn_review is not None:
            # recurrent layers: replay the accepted rows (root + accepted drafts) into the state, all on the device
            i32 = dict(dtype=torch.int32, device=dev)
            fold = K.GdnSegments(torch.arange(R, **i32) * (Kd + 1), (self.accepted[:R] + 1).to(torch.int32),
                                 torch.tensor([s.request_slot for s in segs], **i32),
                                 torch.tensor([s.start for s in segs], **i32), R)
            self._fold_launches = r.fold_gdn(fold, T)
        return hidden

    def _verify(self, segs, Kd: int, draft_ids: torch.Tensor, target_ids: torch.Tensor, logits: torch.Tensor,
                hidden: torch.Tensor) -> torch.Tensor:
        r, dev = self.runner, self.device
        R, T = len(segs), len(segs) * (Kd + 1)
        sm = getattr(self, "_sampling", None)
        mask = getattr(self, "_review_mask", None)          # grammar masks of the review rows (constrained requests)
        if sm is not None:
            # p / q rejection sampling over the candidate distributions; `target_ids` receives the emitted tokens
            rep = lambda t: t.repeat_interleave(Kd + 1)                                # noqa: E731
            K.sample_candidates(logits, self.p_val[:T], self.p_id[:T], temperature=rep(sm["temperature"]),
                                top_k=rep(sm["top_k"]), vocab=logits.shape[1], mask=mask)
            K.verify_sampled(self.q_val, self.q_id, self.p_val, self.p_id, draft_ids, self.depth_t[:R], Kd,
                             sm["temperature"], sm["top_p"], sm["top_k"], sm["seeds"], sm["draws"], self.accepted,
                             self.bonus, target_ids)
            return hidden
        self._sample_greedy(logits, T, target_ids.view(-1), mask)
        forced = None
        if self.force_acceptance is not None:
            draws = self._rng.random((R, Kd)) < self.force_acceptance
            first_fail = np.where(draws.all(1), Kd, draws.argmin(1)).astype(np.int32)
            self.forced[:R].copy_(torch.from_numpy(first_fail), non_blocking=True)
            forced = self.forced
            # forced acceptance: the draft is *declared* equal to the target up to the drawn depth
            agree = target_ids[:, :Kd].clone()
            keep = torch.arange(Kd, device=dev)[None, :] < self.forced[:R, None]
            draft_ids.copy_(torch.where(keep, agree, draft_ids))
        K.verify_greedy(target_ids, draft_ids, self.depth_t[:R], Kd, self.accepted, self.bonus, forced)
        return hidden

    def _sample_greedy(self, logits: torch.Tensor, rows: int, out_ids: torch.Tensor, mask=None) -> None:
        """Greedy ids of ``rows`` rows: over the whole vocabulary, or (tensor parallel) merged over the ranks' shards."""
        r = self.runner
        if r.tp is None:
            K.sample(logits, out_ids, vocab=logits.shape[1], mask=mask)
            return
        if getattr(self, "_greedy_d", None) is None or self._greedy_d["temperature"].shape[0] < rows:
            n = max(rows, self.max_rows * (self.speculative_depth + 1))
            z = lambda dt: torch.zeros(n, dtype=dt, device=self.device)          # noqa: E731
            self._greedy_d = {"temperature": z(torch.float32), "top_p": torch.ones(n, device=self.device),
                              "top_k": z(torch.int32), "seeds": z(torch.int64), "draws": z(torch.int64)}
        if mask is not None:
            mask = mask[:rows, r.w.vocab_start // 32:]
        r.tp.sample_sharded_nccl(logits, rows, out_ids, self._greedy_d, r.w.vocab_start, mask)

    def _review_logits(self, rows: int) -> torch.Tensor:
        if getattr(self, "_rl", None) is None or self._rl.shape[0] < rows:
            self._rl = torch.empty(rows, self.runner.w.lm_head.n, dtype=torch.bfloat16, device=self.device)
        return self._rl


class NgramSpeculativeGpuExecutor(SpeculativeGpuExecutor):
    speculative_sampling = False     # prompt-lookup drafts are verified against the target's greedy choice only
    speculative_grammar = False      # and a constrained request makes its step a plain one

    """Speculative rounds whose drafts come from the host (n-gram / prompt lookup, ``runtime/ngram.py``): no draft
    model, no proposal passes, no carried hidden state -- a round is the target review over ``[root, d1 .. dk]`` plus
    the device-side verification.  Requests without a draft take part with depth 0 (their row is a plain decode row);
    a step in which nobody has a draft is a plain decode step and replays the captured decode graphs."""

    draft_source = "ngram"

    def __init__(self, runner, depth: int, **kw) -> None:
        if runner.cfg.is_hybrid:
            raise NotImplementedError("speculative decoding is not available for models with Gated DeltaNet layers")
        kw.setdefault("use_graphs", True)
        GpuExecutor.__init__(self, runner, rows_per_request=depth + 1, **kw)
        self.mtp = None
        self.speculative_depth = depth
        self.force_acceptance = None
        dev, rows = self.device, self.max_rows
        self.draft_ids = torch.zeros(rows, depth, dtype=torch.int32, device=dev)
        self.target_ids = torch.zeros(rows, depth + 1, dtype=torch.int32, device=dev)
        self.accepted = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.bonus = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.depth_t = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.forced = torch.zeros(rows, dtype=torch.int32, device=dev)
        self._draft_host = torch.zeros(rows, depth, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.stats = {"rounds": 0, "accepted": 0, "proposed": 0, "emitted": 0, "graphed_rounds": 0}
        self.round_graphs = False          # host-drafted rounds run eagerly
        self._round_graph = {}

    def execute(self, segs):
        return GpuExecutor.execute(self, segs)

    def execute_speculative(self, segs: list[Segment], depths: list[int] | None = None, drafts: list[list[int]] | None = None):
        """``drafts[i]``: the host's proposal for request ``i`` (possibly empty, at most the configured depth;
        ``depths`` may shorten it further).  Returns per request the emitted tokens."""
        R = len(segs)
        drafts = [list(d)[:self.speculative_depth] for d in (drafts or [[]] * R)]
        if depths is not None:
            drafts = [d[:max(0, int(k))] for d, k in zip(drafts, depths)]
        per_req = [len(d) for d in drafts]
        Kd = max(per_req, default=0)
        if Kd == 0:
            ids = self.execute(segs)
            self.last_round = {"depth": 0, "accepted": [0] * R, "proposed": [0] * R, "proposal_ms": 0.0,
                               "target_ms": self.device_ms[-1] if (self.timing and self.device_ms) else 0.0}
            return [[int(t)] for t in ids]
        dev = self.device
        draft_ids = self.draft_ids.view(-1)[:R * Kd].view(R, Kd)
        target_ids = self.target_ids.view(-1)[:R * (Kd + 1)].view(R, Kd + 1)
        host = self._draft_host.view(-1)[:R * Kd].view(R, Kd)
        host.zero_()
        for i, d in enumerate(drafts):
            if d:
                host[i, :len(d)] = torch.tensor(d, dtype=torch.int32)
        if self._upload_pending:
            self._uploaded.synchronize()                    # a plain step's staging upload may still be in flight
            self._upload_pending = False
        with torch.cuda.stream(self.stream):
            ev0, ev1 = self._ev[0]
            if self.timing:
                ev0.record(self.stream)
            draft_ids.copy_(host, non_blocking=True)
            self.depth_t[:R].copy_(torch.tensor(per_req, dtype=torch.int32), non_blocking=True)
            self._review_and_verify(segs, Kd, draft_ids, target_ids)
            if self.timing:
                ev1.record(self.stream)
            acc = self.accepted[:R].cpu()
            tg = target_ids.cpu()
            self.stream.synchronize()
        tgt_ms = 0.0
        if self.timing:
            tgt_ms = ev0.elapsed_time(ev1)
            self.device_ms.append(tgt_ms)
        out = []
        for i in range(R):
            a = int(acc[i])
            out.append([int(t) for t in tg[i, :a + 1]])
            self.stats["accepted"] += a
            self.stats["emitted"] += a + 1
        self.stats["rounds"] += 1
        self.stats["proposed"] += sum(per_req)
        self.last_round = {"depth": Kd, "accepted": [int(a) for a in acc], "proposed": per_req, "proposal_ms": 0.0,
                           "target_ms": tgt_ms}
        self.kernel_launches_last = self.runner.launches_per_step + 3
        self.h2d_bytes_last += R * Kd * 4
        self.d2h_bytes_last = R * (Kd + 2) * 4
        return out
