"""Tensor parallelism: NCCL baseline and the fused NVLink path.

Two interchangeable back ends behind the decoder runner:

``mode="nccl"`` -- the baseline.  Hidden states stay replicated; every
row-parallel GEMM is followed by an NCCL all-reduce (captured inside the CUDA
graph), as in the reference (``executor/model_runner.py:3088`` ``_tp_sum``).

``mode="fused"`` -- the product.  No NCCL on the hot path: the row-parallel GEMM
pushes partial rows to their owner over P2P stores (reduce-scatter in the
epilogue), ``tp_reduce_norm`` sums them in rank order, adds the row-sharded
residual, normalises and pushes the rows to every rank (all-gather), and the
next column-parallel GEMM waits for the rows inside its producer warp.  Buffers
are symmetric (same offsets on every rank); peer addresses come from
``torch.distributed._symmetric_memory`` (CUDA VMM + handle exchange) or, for
single-GPU tests, from ``local_fabric`` which places all "ranks" on one device.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from ..ops import kernels as K
from ..ops import native

MODE_GATHER_WAIT = 1
MODE_SCATTER_PUSH = 2
FLAG_WORDS = 64          # per rank: [set(2)][kind(2: rs, ag)][8 sources] + argmax [8] + candidates [8] + pad
CAND = K.SAMPLE_CANDIDATES


def rows_per_rank(m: int, size: int) -> int:
    return -(-(-(-m // size)) // 16) * 16


@dataclass
class TpBuffers:
    """One rank's view: local tensors plus every rank's base addresses (same layout on all ranks)."""
    rank: int
    size: int
    hidden: int
    max_tokens: int
    recv: torch.Tensor            # bf16 [2, size * rpr_max * hidden]   (rpr_max = rows_per_rank(max_tokens))
    xfull: torch.Tensor           # bf16 [2, max_tokens_pad, hidden]
    flags: torch.Tensor           # int32 [FLAG_WORDS]
    xchg_val: torch.Tensor        # fp32 [size, rows_max]
    xchg_id: torch.Tensor         # int32 [size, rows_max]
    cand: torch.Tensor            # int32 [size, 2 * rows_max * CAND]  per source: values (fp32 bits) then ids
    recv_mc: int = 0              # NVLS multicast mappings of recv / xfull (0 = none: plain peer loads and stores)
    xfull_mc: int = 0
    recv_ptrs: list[int] = field(default_factory=list)
    xfull_ptrs: list[int] = field(default_factory=list)
    flags_ptrs: list[int] = field(default_factory=list)
    xval_ptrs: list[int] = field(default_factory=list)
    xid_ptrs: list[int] = field(default_factory=list)
    cand_ptrs: list[int] = field(default_factory=list)


def _alloc_local(rank: int, size: int, hidden: int, max_tokens: int, rows_max: int, device, alloc) -> TpBuffers:
    rpr_max = rows_per_rank(max_tokens, size)
    pad_tokens = rpr_max * size
    return TpBuffers(
        rank, size, hidden, max_tokens,
        recv=alloc((2, size * rpr_max * hidden), torch.bfloat16),
        xfull=alloc((2, pad_tokens, hidden), torch.bfloat16),
        flags=alloc((FLAG_WORDS,), torch.int32),
        xchg_val=alloc((size, rows_max), torch.float32),
        xchg_id=alloc((size, rows_max), torch.int32),
        cand=alloc((size, 2 * rows_max * CAND), torch.int32),
    )


def local_fabric(size: int, hidden: int, max_tokens: int, rows_max: int, device) -> list[TpBuffers]:
    """All ranks on ONE device (tests / emulation): peers are just other tensors of the same process."""
    bufs = [_alloc_local(r, size, hidden, max_tokens, rows_max, device,
                         lambda shape, dt: torch.zeros(shape, dtype=dt, device=device)) for r in range(size)]
    for b in bufs:
        b.recv_ptrs = [o.recv.data_ptr() for o in bufs]
        b.xfull_ptrs = [o.xfull.data_ptr() for o in bufs]
        b.flags_ptrs = [o.flags.data_ptr() for o in bufs]
        b.xval_ptrs = [o.xchg_val.data_ptr() for o in bufs]
        b.xid_ptrs = [o.xchg_id.data_ptr() for o in bufs]
        b.cand_ptrs = [o.cand.data_ptr() for o in bufs]
    return bufs


def symmetric_buffers(group, hidden: int, max_tokens: int, rows_max: int, device) -> TpBuffers:
    """Allocate the buffers in symmetric memory and exchange peer addresses over ``group``."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    rank, size = dist.get_rank(group), dist.get_world_size(group)
    handles = []

    def alloc(shape, dt):
        t = symm.empty(shape, dtype=dt, device=device)
        t.zero_()
        handles.append((t, symm.rendezvous(t, group)))
        return t

    b = _alloc_local(rank, size, hidden, max_tokens, rows_max, device, alloc)
    torch.cuda.synchronize(device)
    dist.barrier(group)
    ptrs = [[int(p) for p in h.buffer_ptrs] for _, h in handles]
    b.recv_ptrs, b.xfull_ptrs, b.flags_ptrs, b.xval_ptrs, b.xid_ptrs, b.cand_ptrs = ptrs
    # NVLS: the multicast mappings of the two big buffers, when the fabric offers them (NVSwitch)
    b.recv_mc = int(getattr(handles[0][1], "multicast_ptr", 0) or 0)
    b.xfull_mc = int(getattr(handles[1][1], "multicast_ptr", 0) or 0)
    b._handles = handles  # keep the mappings alive
    return b


class FusedTp:
    """Launch helpers of the fused path for one rank."""

    def __init__(self, bufs: TpBuffers, device, ws: K.Workspace | None = None) -> None:
        self.b = bufs
        self.rank, self.size = bufs.rank, bufs.size
        self.device = device
        self.ws = ws or K.workspace(device)
        self.state = torch.zeros(16, dtype=torch.int32, device=device)   # [set][kind]{epoch, done} + argmax epoch
        self.rpr_max = rows_per_rank(bufs.max_tokens, self.size)
        self.h_local = torch.zeros(self.rpr_max, bufs.hidden, dtype=torch.bfloat16, device=device)
        self.rpr = self.rpr_max
        self.m = 0
        self._links: dict = {}
        self.rows_max = bufs.xchg_val.shape[1]
        self.cand_local = torch.zeros(2, self.rows_max, CAND, dtype=torch.int32, device=device)
        # NVLS forms of the two collectives of a site (CUBIC_SERVE_NVLS: "0" off, "gather" only the all-gather store,
        # "1" / unset both where the fabric has multicast).  The reduction inside the switch sums in an order of its
        # choosing: results are no longer bit-identical from run to run, the all-gather store changes no bit.
        import os
        mode = os.environ.get("CUBIC_SERVE_NVLS", "gather")
        self.nvls_gather = mode != "0" and bufs.xfull_mc != 0
        self.nvls_reduce = mode == "1" and bufs.recv_mc != 0 and bufs.xfull_mc != 0

    # ---------------------------------------------------------------- helpers
    def begin_step(self, m: int) -> None:
        assert m <= self.b.max_tokens
        self.m = m
        self.rpr = rows_per_rank(m, self.size)

    def _flag_off(self, s: int, kind: int) -> int:
        return ((s * 2 + kind) * 8) * 4                               # bytes

    def _state_ptr(self, s: int, kind: int) -> int:
        return self.state.data_ptr() + ((s * 2 + kind) * 2) * 4

    def _recv_off(self, s: int) -> int:
        return s * self.b.recv.stride(0) * 2

    def _x_off(self, s: int) -> int:
        return s * self.b.xfull.stride(0) * 2

    def x_view(self, s: int, m: int | None = None) -> torch.Tensor:
        return self.b.xfull[s, : (self.m if m is None else m)]

    # ---------------------------------------------------------------- launches
    def gemm_scatter(self, x: torch.Tensor, w, s: int) -> None:
        """Row-parallel GEMM whose epilogue pushes partial rows to their owners (set ``s``)."""
        link = native.TpLinkStruct()
        link.mode, link.rank, link.size, link.rows_per_rank = MODE_SCATTER_PUSH, self.rank, self.size, self.rpr
        for r in range(self.size):
            if self.nvls_reduce:
                # partial rows stay in THIS rank's buffer, laid out by global row: owner r's "slot of this rank" is
                # made to start at row r * rpr of the local buffer; the owner sums all ranks' copies in the switch
                link.recv[r] = self.b.recv.data_ptr() + self._recv_off(s) + (r - self.rank) * self.rpr * w.n * 2
            else:
                link.recv[r] = self.b.recv_ptrs[r] + self._recv_off(s)
            link.rs_flag[r] = self.b.flags_ptrs[r] + self._flag_off(s, 0)
        K.wq_gemm(x, w, out=None, ws=self.ws, link=link)

    def n_tiles_expected(self, n: int, m: int) -> int:
        """Arrivals per source rank at one owner: (n tiles) x (m tiles overlapping the owner's rows)."""
        mb = 256 if m >= 256 else -(-m // 16) * 16
        lo, hi = self.rank * self.rpr, min(m, (self.rank + 1) * self.rpr) - 1
        m_tiles = 0 if hi < lo else hi // mb - lo // mb + 1
        return -(-n // 128) * m_tiles

    def reduce_norm(self, norm_w: torch.Tensor, s: int, n_out: int, eps: float, zero_centered: bool = False,
                    reduce: bool = True, local_only: bool = False) -> None:
        """Owner-side rank-ordered sum + residual + RMSNorm, then all-gather push into set ``s``.

        ``local_only`` keeps the normalised rows on this rank (its own rows of set ``s``, no counters): the
        consumer is the expert-parallel dispatch on the same stream.
        """
        a = native.ReduceNormStruct()
        a.recv = self.b.recv.data_ptr() + self._recv_off(s)
        a.rs_flag = self.b.flags.data_ptr() + self._flag_off(s, 0)
        a.rs_state = self._state_ptr(s, 0)
        a.rs_expected = self.n_tiles_expected(n_out, self.m) if reduce else 0
        a.h = self.h_local.data_ptr()
        a.norm_w = norm_w.data_ptr()
        for r in range(self.size):
            a.x_peer[r] = self.b.xfull_ptrs[r] + self._x_off(s)
            a.ag_flag_peer[r] = self.b.flags_ptrs[r] + self._flag_off(s, 1)
        a.status = self.ws.status.data_ptr()
        a.rank, a.size, a.rows_per_rank, a.H, a.M = self.rank, self.size, self.rpr, self.b.hidden, self.m
        a.eps, a.zero_centered, a.local_only = float(eps), int(zero_centered), int(local_only)
        a.recv_mc = (self.b.recv_mc + self._recv_off(s)) if (self.nvls_reduce and reduce) else None
        a.x_mc = (self.b.xfull_mc + self._x_off(s)) if (self.nvls_gather and not local_only) else None
        native.check(native.lib().cb_tp_reduce_norm(ctypes.byref(a), K._stream()), "cb_tp_reduce_norm")

    def _gather_link(self, s: int):
        link = native.TpLinkStruct()
        link.mode, link.rank, link.size, link.rows_per_rank = MODE_GATHER_WAIT, self.rank, self.size, self.rpr
        link.ag_flag = self.b.flags.data_ptr() + self._flag_off(s, 1)
        link.ag_state = self._state_ptr(s, 1)
        link.ag_expected = self.rpr
        return link

    def gemm_gather(self, w, out: torch.Tensor, s: int) -> torch.Tensor:
        """Column-parallel GEMM on the gathered activations of set ``s`` (waits for them in-kernel)."""
        return K.wq_gemm(self.x_view(s), w, out=out, ws=self.ws, link=self._gather_link(s))

    def gate_up_act(self, w, gu: torch.Tensor, act: torch.Tensor, s: int) -> int:
        """Column-parallel gate/up projection + SwiGLU on the gathered activations of set ``s``; returns the launches."""
        return K.gate_up_act(self.x_view(s), w, gu, act, ws=self.ws, link=self._gather_link(s))

    def wait_gather(self, s: int) -> torch.Tensor:
        native.check(native.lib().cb_tp_wait(self.b.flags.data_ptr() + self._flag_off(s, 1), self._state_ptr(s, 1),
                                             self.rpr, self.size, self.ws.status.data_ptr(), K._stream()), "cb_tp_wait")
        return self.x_view(s)

    def argmax_merge(self, local_val: torch.Tensor, local_id: torch.Tensor, out_id: torch.Tensor, rows: int) -> None:
        """Agree on the global greedy token of every row (also acts as the end-of-step barrier)."""
        a = native.ArgmaxMergeStruct()
        a.local_val, a.local_id = local_val.data_ptr(), local_id.data_ptr()
        off = 32 * 4
        for r in range(self.size):
            a.slot_val[r], a.slot_id[r] = self.b.xval_ptrs[r], self.b.xid_ptrs[r]
            a.flag_peer[r] = self.b.flags_ptrs[r] + off
        a.my_val, a.my_id = self.b.xchg_val.data_ptr(), self.b.xchg_id.data_ptr()
        a.my_flag = self.b.flags.data_ptr() + off
        a.my_state = self.state.data_ptr() + 8 * 4
        a.out_id, a.status = out_id.data_ptr(), self.ws.status.data_ptr()
        a.rank, a.size, a.rows, a.rows_max = self.rank, self.size, rows, self.b.xchg_val.shape[1]
        native.check(native.lib().cb_tp_argmax_merge(ctypes.byref(a), K._stream()), "cb_tp_argmax_merge")


    def sample_sharded(self, logits: torch.Tensor, rows: int, out_ids: torch.Tensor, d: dict, vocab_start: int,
                       mask: torch.Tensor | None = None) -> None:
        """Vocab-sharded sampling: local candidates -> push to every rank -> identical merge + draw everywhere.

        Replaces the reference's gather-to-root + broadcast (``generation/tp_sampling.py:681``): every rank runs
        the same draw on the same gathered candidates, so no broadcast is needed; the exchange doubles as the
        end-of-step barrier.  Greedy rows carry one candidate, sampled rows up to 20.
        """
        val, ids = self.cand_local[0].view(torch.float32), self.cand_local[1]
        K.sample_candidates(logits, val, ids, temperature=d["temperature"][:rows], top_k=d["top_k"][:rows], mask=mask,
                            vocab=logits.shape[1], id_offset=vocab_start)
        a = native.ExchangeStruct()
        a.local = self.cand_local.data_ptr()
        off = 40 * 4
        for r in range(self.size):
            a.area_peer[r] = self.b.cand_ptrs[r]
            a.flag_peer[r] = self.b.flags_ptrs[r] + off
        a.my_flag = self.b.flags.data_ptr() + off
        a.my_state = self.state.data_ptr() + 10 * 4
        a.status = self.ws.status.data_ptr()
        a.rank, a.size, a.segments = self.rank, self.size, 2
        a.seg_words, a.seg_stride, a.area_words = rows * CAND, self.rows_max * CAND, 2 * self.rows_max * CAND
        native.check(native.lib().cb_tp_exchange(ctypes.byref(a), K._stream()), "cb_tp_exchange")
        area = self.b.cand
        K.sample_merge(area.view(torch.float32), area.view(-1)[self.rows_max * CAND:], self.size, area.stride(0), rows,
                       out_ids, temperature=d["temperature"][:rows], top_p=d["top_p"][:rows], top_k=d["top_k"][:rows],
                       seeds=d["seeds"][:rows], counters=d["draws"][:rows])


class TensorParallel:
    """What the decoder runner sees: ``size``, ``rank``, ``mode`` and the collective entry points."""

    def __init__(self, group, device, mode: str = "fused", hidden: int = 4096, max_tokens: int = 8192,
                 rows_max: int = 512) -> None:
        import torch.distributed as dist
        self.group = group
        self.device = device
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.mode = mode
        self.fused: FusedTp | None = None
        if mode == "fused":
            self.fused = FusedTp(symmetric_buffers(group, hidden, max_tokens, rows_max, device), device)
        self._gather_val = torch.empty(self.size, rows_max, dtype=torch.float32, device=device)
        self._gather_id = torch.empty(self.size, rows_max, dtype=torch.int32, device=device)
        self.rows_max = rows_max

    def all_reduce(self, t: torch.Tensor) -> None:
        import torch.distributed as dist
        dist.all_reduce(t, group=self.group)

    def all_reduce_max(self, t: torch.Tensor) -> None:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)

    def sample_sharded_nccl(self, logits: torch.Tensor, rows: int, out_ids: torch.Tensor, d: dict, vocab_start: int,
                            mask: torch.Tensor | None = None) -> None:
        """Baseline of ``FusedTp.sample_sharded``: NCCL all-gather of the candidates, same merge kernel."""
        import torch.distributed as dist
        if not hasattr(self, "_cand_local"):
            self._cand_local = torch.zeros(2, self.rows_max, CAND, dtype=torch.int32, device=self.device)
            self._cand_all = torch.zeros(self.size, 2, self.rows_max, CAND, dtype=torch.int32, device=self.device)
        val, ids = self._cand_local[0].view(torch.float32), self._cand_local[1]
        K.sample_candidates(logits, val, ids, temperature=d["temperature"][:rows], top_k=d["top_k"][:rows], mask=mask,
                            vocab=logits.shape[1], id_offset=vocab_start)
        dist.all_gather_into_tensor(self._cand_all, self._cand_local, group=self.group)
        flat = self._cand_all.view(self.size, -1)
        K.sample_merge(flat.view(torch.float32), flat.view(-1)[self.rows_max * CAND:], self.size, flat.stride(0), rows,
                       out_ids, temperature=d["temperature"][:rows], top_p=d["top_p"][:rows], top_k=d["top_k"][:rows],
                       seeds=d["seeds"][:rows], counters=d["draws"][:rows])

    def argmax_merge_nccl(self, local_val: torch.Tensor, local_id: torch.Tensor, out_id: torch.Tensor, rows: int) -> None:
        """Baseline: all_gather of (value, id) and a small torch reduction (reference ``tp_sampling.py:1225``)."""
        import torch.distributed as dist
        gv, gi = self._gather_val[:, :rows].contiguous(), self._gather_id[:, :rows].contiguous()
        dist.all_gather_into_tensor(gv, local_val[:rows].contiguous(), group=self.group)
        dist.all_gather_into_tensor(gi, local_id[:rows].contiguous(), group=self.group)
        best = gv.max(0, keepdim=True).values
        cand = torch.where(gv == best, gi, torch.full_like(gi, 0x7FFFFFFF))
        out_id[:rows].copy_(cand.min(0).values)
