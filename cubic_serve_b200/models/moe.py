"""Mixture-of-experts FFN on the native kernels (router -> permute -> grouped expert GEMMs -> combine).

Semantics of the reference's fused MoE (``ops/cuda/moe/fused.py``): stable top-k over router logits, softmax
over the selected logits, SwiGLU experts, weighted combine in fixed route order.  Expert parallelism follows
the reference's serving path (``runtime/README.md:140-160`` there): tokens are replicated, a rank computes only
the experts it owns (routes to other experts contribute +0) and the per-rank partial outputs are summed like any
row-parallel partial.  The expert GEMMs are ONE grouped launch each (gate/up and down) over a device-side work
list, so variable routing needs no host round trip and is CUDA-graph safe.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import kernels as K
from ..ops import wq_pack
from .config import ModelConfig


def stack_experts(packed: list[wq_pack.PackedWeight]) -> tuple[wq_pack.PackedWeight, int, int]:
    """Stack per-expert packed weights along a leading axis; returns (stacked, code stride, meta stride) in bytes."""
    first = packed[0]
    alpha = first.alpha
    if first.fmt == wq_pack.FMT_NVFP4 and any(p.alpha != alpha for p in packed):
        # every expert carries its own global scale, the grouped GEMM applies ONE: the largest becomes the stack's and
        # each expert's ratio to it is folded into its block scales (bf16 pairs in the metadata)
        alpha = max(p.alpha for p in packed)
        packed = [p if p.alpha == alpha else _rescaled_nvfp4(p, p.alpha / alpha) for p in packed]
    codes = torch.stack([p.codes for p in packed])
    meta = torch.stack([p.meta for p in packed]) if first.meta is not None else None
    stacked = wq_pack.PackedWeight(first.fmt, first.n, first.k, first.group_k, codes, meta, alpha)
    cs = codes[0].numel() * codes.element_size()
    ms = meta[0].numel() if meta is not None else 0
    return stacked, cs, ms


def _rescaled_nvfp4(p: wq_pack.PackedWeight, ratio: float) -> wq_pack.PackedWeight:
    """The same NVFP4 matrix with its block scales multiplied by ``ratio`` (and its global scale divided by it)."""
    scales = p.meta.contiguous().view(torch.bfloat16).float() * ratio
    meta = scales.to(torch.bfloat16).view(torch.uint8).reshape(p.meta.shape)
    return wq_pack.PackedWeight(p.fmt, p.n, p.k, p.group_k, p.codes, meta, p.alpha / ratio, p.act_interleaved)


@dataclass
class MoeLayer:
    router: wq_pack.PackedWeight          # bf16 [E, H]
    gate_up: wq_pack.PackedWeight         # stacked [E_local] x [2I, H]
    down: wq_pack.PackedWeight            # stacked [E_local] x [H, I]
    strides: tuple[int, int, int, int]    # code / meta strides of gate_up and down
    num_experts: int
    top_k: int
    expert_lo: int
    expert_count: int
    normalize: bool = True
    scratch: K.MoeScratch | None = None
    launches: int = 7
    # shared expert (Qwen2-MoE / Qwen3.5-MoE): a dense SwiGLU feed-forward over every token whose output is scaled by
    # sigmoid(x . gate) and added to the routed experts' sum.  Under tensor parallelism a rank holds its share of the
    # intermediate features (a partial sum like the routed part); the gate vector is replicated.
    shared_gate_up: wq_pack.PackedWeight | None = None    # [2 Is(/tp), H]
    shared_down: wq_pack.PackedWeight | None = None       # [H, Is(/tp)]
    shared_gate: wq_pack.PackedWeight | None = None       # bf16 [8, H]: row 0 is the gate vector, the others zero

    def fuse_activation(self) -> None:
        """Re-order every expert's ``[gate; up]`` rows so that the grouped GEMM applies SwiGLU in its epilogue."""
        self.gate_up = wq_pack.swiglu_interleave(self.gate_up, stacked=True)
        if self.shared_gate_up is not None and (self.shared_gate_up.n // 2) % 16 == 0 \
                and self.shared_gate_up.fmt != wq_pack.FMT_FP8_BLOCK:
            self.shared_gate_up = wq_pack.swiglu_interleave(self.shared_gate_up)

    def _shared(self, x: torch.Tensor, out: torch.Tensor, ws) -> None:
        """``out += sigmoid(x . gate) * shared_expert(x)`` (fixed buffers: the step may be captured in a CUDA graph)."""
        t = x.shape[0]
        act = self.sh_act[:t]
        if self.shared_gate_up.act_interleaved:
            K.wq_gemm_act(x, self.shared_gate_up, out=act, ws=ws)
        else:
            K.wq_gemm(x, self.shared_gate_up, out=self.sh_gu[:t], ws=ws)
            K.swiglu(self.sh_gu[:t], out=act)
        K.wq_gemm(act, self.shared_down, out=self.sh_out[:t], ws=ws)
        K.wq_gemm(x, self.shared_gate, out=self.sh_logit[:t], ws=ws)
        torch.sigmoid(self.sh_logit[:t, :1], out=self.sh_sig[:t])
        out.addcmul_(self.sh_out[:t], self.sh_sig[:t])

    def experts(self, sc: K.MoeScratch, rows: int, ws) -> None:
        """Grouped gate/up GEMM, SwiGLU, grouped down GEMM over the sorted rows ``sc.xs`` -> ``sc.y``."""
        if self.gate_up.act_interleaved:
            K.wq_gemm_grouped(sc.xs, self.gate_up, sc.act, rows, sc, self.strides[0], self.strides[1], ws, swiglu=True)
        else:
            K.wq_gemm_grouped(sc.xs, self.gate_up, sc.gu, rows, sc, self.strides[0], self.strides[1], ws)
            K.swiglu(sc.gu[:rows], out=sc.act[:rows])
        K.wq_gemm_grouped(sc.act, self.down, sc.y, rows, sc, self.strides[2], self.strides[3], ws)

    def ensure_scratch(self, max_tokens: int, hidden: int, device) -> K.MoeScratch:
        if self.scratch is None or self.scratch.topk_ids.shape[0] < max_tokens:
            from ..ops.strategies import active
            pol = active().moe
            big = max_tokens * self.top_k >= pol.large_routes_per_expert * self.expert_count
            mb = pol.rows_per_item_large if big else pol.rows_per_item_small
            self.scratch = K.MoeScratch(max_tokens, self.top_k, hidden, self.gate_up.n, self.expert_count, mb, device)
            self.logits = torch.empty(max_tokens, self.num_experts, dtype=torch.bfloat16, device=device)
            self.out = torch.empty(max_tokens, hidden, dtype=torch.bfloat16, device=device)
            if self.shared_gate_up is not None:
                bf = dict(dtype=torch.bfloat16, device=device)
                self.sh_gu = torch.empty(max_tokens, self.shared_gate_up.n, **bf)
                self.sh_act = torch.empty(max_tokens, self.shared_gate_up.n // 2, **bf)
                self.sh_out = torch.empty(max_tokens, hidden, **bf)
                self.sh_logit = torch.empty(max_tokens, self.shared_gate.n, **bf)
                self.sh_sig = torch.empty(max_tokens, 1, **bf)
        return self.scratch

    def forward(self, x: torch.Tensor, runner=None, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
        """``x``: normalised activations ``[T, H]``; returns this rank's (partial) FFN output ``[T, H]``.

        With ``residual`` the combine adds it (``out`` may alias ``residual``: the residual stream is updated in place).
        """
        t, h = x.shape
        sc = self.ensure_scratch(runner.max_tokens if runner is not None else t, h, x.device)
        ws = runner.ws if runner is not None else None
        logits = K.wq_gemm(x, self.router, out=self.logits[:t], ws=ws)
        K.moe_route(logits, x, self.top_k, sc, self.normalize, self.expert_lo, self.expert_count)
        rows = t * self.top_k
        self.experts(sc, rows, ws)
        res = K.moe_combine(sc.y, sc, t, self.out[:t] if out is None else out, residual)
        if self.shared_gate_up is not None:
            self._shared(x, res, ws)
        return res


def expert_coordinates(tp_rank: int, tp_size: int, ep_size: int | None) -> tuple[int, int, int]:
    """``(expert owner, lane, lanes)`` of a tensor rank: the ``tp_size`` ranks of a stage are ``ep_size`` expert owners
    times ``tp_size / ep_size`` lanes; the lanes of one owner hold the same experts and divide every expert's
    intermediate features among them (reference: ``contracts/execution.py:238-248``).  ``ep_size`` None = ``tp_size``
    (every rank owns whole experts)."""
    ep = tp_size if ep_size is None else ep_size
    if ep < 1 or tp_size % ep:
        raise ValueError("the expert-parallel size divides the tensor-parallel size")
    lanes = tp_size // ep
    return tp_rank // lanes, tp_rank % lanes, lanes


def random_moe_weights(cfg: ModelConfig, device, gen, tp_rank: int = 0, tp_size: int = 1, std: float = 0.02,
                       layer_seed: int = 0, ep_size: int | None = None) -> MoeLayer:
    """Random experts, router replicated.  Rank ``(owner, lane)`` holds the contiguous expert ids of its owner and, of
    each, the gate / up rows and down columns of its lane (``ep_size`` None: whole experts, one owner per rank).
    Expert ``e`` of a layer draws from a generator seeded by (layer, e) only, so every partition holds slices of the
    same model."""
    from .decoder import quantize_linear
    H, I, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts
    owner, lane, lanes = expert_coordinates(tp_rank, tp_size, ep_size)
    if E % (tp_size // lanes) or I % lanes or (I // lanes) % 128:
        raise ValueError("experts divide over the owners and every lane keeps whole 128-feature groups of an expert")
    local, il = E // (tp_size // lanes), I // lanes
    shared = torch.Generator(device=device).manual_seed(12345 + layer_seed)
    router = (torch.randn(E, H, device=device, generator=shared) * std).to(torch.bfloat16)
    gus, downs = [], []
    for e in range(owner * local, (owner + 1) * local):
        gen.manual_seed(layer_seed * 1024 + e + 1)
        gu_full = torch.randn(2 * I, H, device=device, generator=gen) * std
        dn_full = torch.randn(H, I, device=device, generator=gen) * std
        if lanes > 1:
            gu_full = torch.cat([gu_full[lane * il:(lane + 1) * il], gu_full[I + lane * il:I + (lane + 1) * il]])
            dn_full = dn_full[:, lane * il:(lane + 1) * il].contiguous()
        gus.append(quantize_linear(gu_full, cfg))
        downs.append(quantize_linear(dn_full, cfg))
    gu, gcs, gms = stack_experts(gus)
    dn, dcs, dms = stack_experts(downs)
    layer = MoeLayer(wq_pack.pack_bf16(router), gu, dn, (gcs, gms, dcs, dms), E, cfg.experts_per_token,
                     owner * local, local, cfg.norm_topk_prob)
    if cfg.shared_intermediate_size:
        Is = cfg.shared_intermediate_size
        if Is % tp_size or (Is // tp_size) % 128:
            raise ValueError("every rank keeps whole 128-feature groups of the shared expert")
        sl = Is // tp_size
        sgu = torch.randn(2 * Is, H, device=device, generator=shared) * std
        sdn = torch.randn(H, Is, device=device, generator=shared) * std
        gate = torch.randn(1, H, device=device, generator=shared) * std
        lo = tp_rank * sl
        layer.shared_gate_up = quantize_linear(torch.cat([sgu[lo:lo + sl], sgu[Is + lo:Is + lo + sl]]), cfg)
        layer.shared_down = quantize_linear(sdn[:, lo:lo + sl].contiguous(), cfg)
        layer.shared_gate = shared_gate_matrix(gate)
        layer.launches += 5
    return layer


def shared_gate_matrix(gate: torch.Tensor) -> wq_pack.PackedWeight:
    """The shared expert's gate vector ``[1, H]`` as a bf16 GEMM operand of 8 rows (row 0 = the vector)."""
    m = torch.zeros(8, gate.shape[-1], dtype=torch.bfloat16, device=gate.device)
    m[0] = gate.reshape(-1).to(torch.bfloat16)
    return wq_pack.pack_bf16(m)


def load_moe_layer(ck, layer: int, device, tp_rank: int = 0, tp_size: int = 1) -> MoeLayer:
    """Experts of decoder layer ``layer`` from an admitted checkpoint.  Expert parallelism over the tensor-parallel
    ranks: rank ``r`` owns the contiguous expert ids ``[r E / tp, (r + 1) E / tp)`` whole; the router is replicated.
    Payloads keep the checkpoint's quantization (``pack_logical`` re-tiles, it does not re-quantize)."""
    from .checkpoint import CheckpointError, logical_inventory, pack_logical
    cfg, q = ck.cfg, ck.cfg.quant
    E = cfg.num_experts
    if E % tp_size:
        raise CheckpointError(f"{E} experts do not split over {tp_size} ranks")
    local = E // tp_size
    shapes, _ = logical_inventory(cfg)
    gus, downs = [], []
    for e in range(tp_rank * local, (tp_rank + 1) * local):
        ep = f"model.layers.{layer}.mlp.experts.{e}"
        gate, up, down = f"{ep}.gate_proj", f"{ep}.up_proj", f"{ep}.down_proj"
        gus.append(pack_logical(q.method, [(ck.payload(gate), shapes[gate]), (ck.payload(up), shapes[up])], q))
        downs.append(pack_logical(q.method, [(ck.payload(down), shapes[down])], q))
    gu, gcs, gms = stack_experts(gus)
    dn, dcs, dms = stack_experts(downs)
    router = ck.store.get(f"model.layers.{layer}.mlp.gate.weight").to(torch.bfloat16)
    out = MoeLayer(wq_pack.pack_bf16(router).to(device), gu.to(device), dn.to(device), (gcs, gms, dcs, dms), E,
                   cfg.experts_per_token, tp_rank * local, local, cfg.norm_topk_prob)
    if cfg.shared_intermediate_size:
        from .checkpoint import _slice_rows
        Is = cfg.shared_intermediate_size
        if Is % tp_size or (Is // tp_size) % 128:
            raise CheckpointError("every rank keeps whole 128-feature groups of the shared expert")
        lo, hi = tp_rank * (Is // tp_size), (tp_rank + 1) * (Is // tp_size)
        sp = f"model.layers.{layer}.mlp.shared_expert"
        parts = [(_slice_rows(ck.payload(f"{sp}.{m}"), q.method, lo, hi, Is, q.bits), (hi - lo, cfg.hidden_size))
                 for m in ("gate_proj", "up_proj")]
        out.shared_gate_up = pack_logical(q.method, parts, q).to(device)
        out.shared_down = pack_logical(q.method, [(ck.payload(f"{sp}.down_proj"), shapes[f"{sp}.down_proj"])], q,
                                       (lo, hi)).to(device)
        out.shared_gate = shared_gate_matrix(ck.store.get(f"model.layers.{layer}.mlp.shared_expert_gate.weight")).to(device)
        out.launches += 5
    return out


def moe_reference(x: torch.Tensor, router: torch.Tensor, gate_up: list[torch.Tensor], down: list[torch.Tensor],
                  top_k: int, normalize: bool = True, expert_lo: int = 0) -> torch.Tensor:
    """Independent fp32 oracle: dense per-token loop over the selected experts (local experts only)."""
    xf = x.float()
    logits = (xf @ router.float().t()).to(torch.bfloat16).float()
    t, e = logits.shape
    out = torch.zeros(t, x.shape[1], device=x.device)
    # stable top-k with lowest id on ties: sort by (-value, id)
    order = torch.argsort(-logits, dim=-1, stable=True)[:, :top_k]
    sel = torch.gather(logits, 1, order)
    w = torch.softmax(sel, -1) if normalize else torch.softmax(logits, -1).gather(1, order)
    for ti in range(t):
        for r in range(top_k):
            le = int(order[ti, r]) - expert_lo
            if not 0 <= le < len(gate_up):
                continue
            gu = (xf[ti] @ gate_up[le].float().t()).to(torch.bfloat16).float()
            i = gu.shape[0] // 2
            act = (torch.nn.functional.silu(gu[:i]) * gu[i:]).to(torch.bfloat16).float()
            y = (act @ down[le].float().t()).to(torch.bfloat16).float()
            out[ti] += w[ti, r] * y
    return out
