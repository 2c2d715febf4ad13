"""Expert parallelism with fused dispatch / combine over NVLink peer memory.

Host side of ``csrc/ep_comm.cu``: symmetric receive / return regions, the launch sequence of one MoE block, and a
single-device fabric for tests.  The residual stream is row-sharded (rank ``r`` owns token rows
``[r * rows_per_rank, ...)``, the layout of the fused tensor-parallel path in ``parallel/tp.py``); expert ``e``
lives on rank ``e // experts_per_rank``.

    logits  = router GEMM on the rank's own normalised rows                (tcgen05 GEMM, bf16 weights)
    ep_dispatch : top-k + slot claim + P2P push of rows and {ids, weights}  (one kernel)
    ep_unpack   : wait for every source, build the permutation inputs
    moe_permute -> grouped gate/up GEMM -> SwiGLU -> grouped down GEMM      (same kernels as without EP)
    ep_combine_push : per received token, weighted sum of its local routes, one row pushed home
    ep_finish   : ordered sum over ranks + residual into the rank's rows

Reference counterpart: NCCL ``ep_dispatch`` / ``ep_combine`` of the eager partition
(``executor/parallel/nccl.py:43``) and the eager EP MoE (``models/qwen3_5_moe/distributed.py:191``).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from ..ops import kernels as K
from ..ops import native
from .tp import rows_per_rank

EP_FLAG_WORDS = 32          # [dispatch arrivals: 8][return arrivals: 8][pad]


@dataclass
class EpBuffers:
    """One rank's regions plus every rank's base addresses (same layout everywhere)."""
    rank: int
    size: int
    hidden: int
    top_k: int
    cap: int                      # rows one source may send = rows_per_rank(max_tokens)
    xin: torch.Tensor             # bf16 [size, cap, H]   rows received from each source
    ids_in: torch.Tensor          # int32 [size, cap, k]
    w_in: torch.Tensor            # fp32 [size, cap, k]
    cnt_in: torch.Tensor          # int32 [size]
    yin: torch.Tensor             # bf16 [size, cap, H]   rows returned by each expert owner
    flags: torch.Tensor           # int32 [EP_FLAG_WORDS]
    ptrs: dict = field(default_factory=dict)     # name -> list of per-rank base addresses


_NAMES = ("xin", "ids_in", "w_in", "cnt_in", "yin", "flags")


def _alloc(rank: int, size: int, hidden: int, top_k: int, max_tokens: int, alloc) -> EpBuffers:
    cap = rows_per_rank(max_tokens, size)
    return EpBuffers(rank, size, hidden, top_k, cap,
                     xin=alloc((size, cap, hidden), torch.bfloat16), ids_in=alloc((size, cap, top_k), torch.int32),
                     w_in=alloc((size, cap, top_k), torch.float32), cnt_in=alloc((size,), torch.int32),
                     yin=alloc((size, cap, hidden), torch.bfloat16), flags=alloc((EP_FLAG_WORDS,), torch.int32))


def local_ep_fabric(size: int, hidden: int, top_k: int, max_tokens: int, device) -> list[EpBuffers]:
    """All ranks on ONE device (tests): peers are other tensors of the same process."""
    bufs = [_alloc(r, size, hidden, top_k, max_tokens, lambda shape, dt: torch.zeros(shape, dtype=dt, device=device))
            for r in range(size)]
    for b in bufs:
        b.ptrs = {n: [getattr(o, n).data_ptr() for o in bufs] for n in _NAMES}
    return bufs


def symmetric_ep_buffers(group, hidden: int, top_k: int, max_tokens: int, device) -> EpBuffers:
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    rank, size = dist.get_rank(group), dist.get_world_size(group)
    handles = []

    def alloc(shape, dt):
        t = symm.empty(shape, dtype=dt, device=device)
        t.zero_()
        handles.append((t, symm.rendezvous(t, group)))
        return t

    b = _alloc(rank, size, hidden, top_k, max_tokens, alloc)
    torch.cuda.synchronize(device)
    dist.barrier(group)
    b.ptrs = {n: [int(p) for p in h.buffer_ptrs] for n, (_, h) in zip(_NAMES, handles)}
    b._handles = handles
    return b


class FusedEp:
    """Launch sequence of one expert-parallel MoE block for one rank."""

    def __init__(self, bufs: EpBuffers, device, num_experts: int, inter2: int, ws: K.Workspace | None = None) -> None:
        self.b = bufs
        self.rank, self.size = bufs.rank, bufs.size
        self.device = device
        self.ws = ws or K.workspace(device)
        assert num_experts % self.size == 0
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.size
        virt = self.size * bufs.cap                                   # received records are the permutation's "tokens"
        mb = 64 if virt * bufs.top_k >= 32 * self.experts_per_rank else 32
        self.sc = K.MoeScratch(virt, bufs.top_k, bufs.hidden, inter2, self.experts_per_rank, mb, device)
        i32 = dict(dtype=torch.int32, device=device)
        self.local_cnt = torch.zeros(self.size, **i32)
        self.sent = torch.full((bufs.cap, self.size), -1, **i32)
        self.done = torch.zeros(2, **i32)                              # CTA counters of dispatch / combine_push
        self.state = torch.zeros(4, **i32)                             # {consumed, done CTAs} x {dispatch, return}
        self.logits = torch.empty(bufs.cap, num_experts, dtype=torch.bfloat16, device=device)
        self.launches = 9

    def forward(self, layer, x_rows: torch.Tensor, cnt: int, h_rows: torch.Tensor) -> None:
        """``x_rows``: this rank's normalised rows ``[>= cnt, H]``; ``h_rows``: its residual rows, updated in place.

        The three phases wait on one another ACROSS ranks, so a single-device emulation of several ranks has to
        run phase by phase over all ranks (``dispatch`` of every rank, then ``experts``, then ``finish``); with one
        process per GPU the phases simply follow each other on the stream.
        """
        self.dispatch(layer, x_rows, cnt)
        self.experts(layer)
        self.finish(cnt, h_rows)

    def dispatch(self, layer, x_rows: torch.Tensor, cnt: int) -> None:
        b, lib = self.b, native.lib()
        H, k = b.hidden, b.top_k
        st = K._stream()
        if cnt:
            K.wq_gemm(x_rows[:cnt], layer.router, out=self.logits[:cnt], ws=self.ws)
        d = native.EpDispatchStruct()
        d.logits, d.x, d.ld, d.cnt = self.logits.data_ptr(), x_rows.data_ptr(), self.logits.stride(0), cnt
        d.E, d.k, d.H, d.normalize = self.num_experts, k, H, int(layer.normalize)
        d.experts_per_rank, d.rank, d.size, d.cap = self.experts_per_rank, self.rank, self.size, b.cap
        for r in range(self.size):
            d.xin_peer[r], d.ids_peer[r], d.w_peer[r] = b.ptrs["xin"][r], b.ptrs["ids_in"][r], b.ptrs["w_in"][r]
            d.cnt_peer[r], d.flag_peer[r] = b.ptrs["cnt_in"][r], b.ptrs["flags"][r]
        d.local_cnt, d.sent, d.done = self.local_cnt.data_ptr(), self.sent.data_ptr(), self.done.data_ptr()
        native.check(lib.cb_ep_dispatch(ctypes.byref(d), st), "cb_ep_dispatch")

    def experts(self, layer) -> None:
        b, sc, lib = self.b, self.sc, native.lib()
        H, k = b.hidden, b.top_k
        st = K._stream()
        lo = self.rank * self.experts_per_rank
        native.check(lib.cb_ep_unpack(b.ids_in.data_ptr(), b.w_in.data_ptr(), b.cnt_in.data_ptr(), b.flags.data_ptr(),
                                      self.state.data_ptr(), self.size, b.cap, k, lo, self.experts_per_rank,
                                      sc.topk_ids.data_ptr(), sc.topk_w.data_ptr(), sc.counts.data_ptr(),
                                      self.ws.status.data_ptr(), st), "cb_ep_unpack")
        virt = self.size * b.cap
        native.check(lib.cb_moe_permute(b.xin.data_ptr(), sc.topk_ids.data_ptr(), virt, k, H, lo, self.experts_per_rank,
                                        sc.mb, sc.counts.data_ptr(), sc.offsets.data_ptr(), sc.cursors.data_ptr(),
                                        sc.total.data_ptr(), sc.tiles.data_ptr(), sc.route_pos.data_ptr(),
                                        sc.xs.data_ptr(), st), "cb_moe_permute")
        rows = virt * k
        layer.experts(sc, rows, self.ws)

        c = native.EpCombineStruct()
        c.y, c.route_pos, c.topk_w, c.cnt_in = sc.y.data_ptr(), sc.route_pos.data_ptr(), sc.topk_w.data_ptr(), b.cnt_in.data_ptr()
        c.size, c.cap, c.k, c.H, c.rank = self.size, b.cap, k, H, self.rank
        for r in range(self.size):
            c.yin_peer[r], c.flag_peer[r] = b.ptrs["yin"][r], b.ptrs["flags"][r] + 8 * 4
        c.done = self.done.data_ptr() + 4
        native.check(lib.cb_ep_combine_push(ctypes.byref(c), st), "cb_ep_combine_push")

    def finish(self, cnt: int, h_rows: torch.Tensor) -> None:
        b, lib = self.b, native.lib()
        H, st = b.hidden, K._stream()
        native.check(lib.cb_ep_finish(b.yin.data_ptr(), self.sent.data_ptr(), b.flags.data_ptr() + 8 * 4,
                                      self.state.data_ptr() + 8, h_rows.data_ptr(), self.size, b.cap, H, cnt,
                                      self.ws.status.data_ptr(), st), "cb_ep_finish")
