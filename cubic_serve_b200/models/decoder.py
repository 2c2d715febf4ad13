"""GQA decoder executed with the native sm_100a kernels (dense FFN or MoE).

One ``DecoderRunner`` is the per-rank model body: it owns the rank-local packed
weights, fixed-address activation buffers and the quantized paged KV cache, and
exposes ``forward(batch)`` which is safe to capture in a CUDA graph (no host
synchronisation, no allocation).  It corresponds to the reference's captured
stage body (``executor/quantized_model_runner.py:213``,
``executor/text_graph.py:126``): norm -> QKV GEMM -> RoPE + KV quantize-on-write
-> paged attention -> o_proj (+collective) -> norm -> gate/up -> SwiGLU -> down
(+collective) -> final norm -> lm_head -> sampler.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops import kernels as K
from ..ops import wq_pack
from ..ops.eager import rope_inv_freq
from ..quantization import cubic
from .config import ModelConfig


@dataclass
class GdnWeights:
    """Gated DeltaNet mixer of one layer (rank-local heads).  ``in_proj`` rows: q [Hk 128] | k [Hk 128] | v [Hv 128] |
    z [Hv 128]; ``in_ba`` rows: b [Hv] | a [Hv], kept in bf16 (64 rows: too small to quantize; reference modules
    ``in_proj_qkvz`` and ``in_proj_ba``, ``models/qwen3_5/model.py:498``)."""
    in_proj: wq_pack.PackedWeight
    in_ba: wq_pack.PackedWeight
    conv_w: torch.Tensor                 # fp32 [2 Hk 128 + Hv 128, 4]
    a_log: torch.Tensor                  # fp32 [Hv]
    dt_bias: torch.Tensor                # fp32 [Hv]
    norm_w: torch.Tensor                 # fp32 [128]
    out: wq_pack.PackedWeight            # [H, Hv 128]
    hk: int = 0
    hv: int = 0


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    qkv: wq_pack.PackedWeight | None = None     # None for Gated DeltaNet layers
    o: wq_pack.PackedWeight | None = None
    gdn: GdnWeights | None = None
    attn_gate: wq_pack.PackedWeight | None = None   # [hq D, H]: output gate of the hybrid family's attention layers
    gate_up: wq_pack.PackedWeight | None = None
    down: wq_pack.PackedWeight | None = None
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    moe: object | None = None
    qkv_bias: torch.Tensor | None = None            # bf16 [(hq + 2 hkv) D]: q / k / v projection biases of this rank's heads


@dataclass
class DecoderWeights:
    embed: torch.Tensor                     # [V(/tp), H] bf16
    layers: list[LayerWeights]
    final_norm: torch.Tensor
    lm_head: wq_pack.PackedWeight           # [V(/tp), H]
    vocab_start: int = 0
    extras: dict = field(default_factory=dict)

    def nbytes(self) -> int:
        total = self.embed.numel() * 2 + self.lm_head.nbytes
        for l in self.layers:
            ws = [l.qkv, l.o, l.gate_up, l.down, l.attn_gate]
            if l.gdn is not None:
                ws += [l.gdn.in_proj, l.gdn.in_ba, l.gdn.out]
            if l.moe is not None:
                ws += [l.moe.router, l.moe.gate_up, l.moe.down, l.moe.shared_gate_up, l.moe.shared_down]
            for w in ws:
                if w is not None:
                    total += w.nbytes
        return total


def quantize_linear(w: torch.Tensor, cfg: ModelConfig, amax: float | None = None,
                    row_amax: torch.Tensor | None = None) -> wq_pack.PackedWeight:
    """Quantize a dense ``[N, K]`` matrix with the config's weight format and re-tile it for the GEMM.  ``amax``: the
    largest magnitude of the matrix ``w`` is a shard of (formats with one scale per tensor, i.e. NVFP4); ``row_amax``:
    the largest magnitude of every row of that matrix (formats with one scale per row, i.e. FP8), so that a column
    shard carries the codes and scales of the whole rows."""
    q = cfg.quant
    if q.method == "none":
        return wq_pack.pack_bf16(w)
    if q.method == "cubic":
        if q.bits != 4:
            raise NotImplementedError("the tcgen05 GEMM consumes 4-bit Cubic codes")
        scheme = cubic.CubicScheme(bits=4, group_in=q.group_size)
        out_codes, sc, aa, bb = [], [], [], []
        for r0 in range(0, w.shape[0], 8192):  # bounded temporaries
            p = cubic.quantize(w[r0:r0 + 8192], scheme)
            out_codes.append(cubic.unpack_codes(p["weight_packed"], 4, w.shape[1]))
            sc.append(p["weight_scale"]); aa.append(p["weight_a"]); bb.append(p["weight_b"])
        return wq_pack.pack_cubic4(torch.cat(out_codes), torch.cat(sc), torch.cat(aa), torch.cat(bb), q.group_size)
    if q.method in ("int", "awq", "gguf"):
        g = q.group_size if q.method != "gguf" else 32
        n, k = w.shape
        wg = w.float().reshape(n, k // g, g)
        lo, hi = wg.amin(-1), wg.amax(-1)
        scale = ((hi - lo) / 15.0).clamp_min(1e-8)
        qv = torch.round((wg - lo[..., None]) / scale[..., None]).clamp(0, 15).to(torch.uint8).reshape(n, k)
        return wq_pack.pack_affine4(qv, scale, lo, g)
    if q.method == "fp8":
        from ..quantization import formats
        if row_amax is None:
            payload = formats.fp8_quantize(w, block=False)
            return wq_pack.pack_fp8(payload["weight"], payload["weight_scale"])
        scale = (row_amax.float().reshape(-1, 1) / 448.0).clamp_min(1e-12)
        return wq_pack.pack_fp8((w.float() / scale).to(torch.float8_e4m3fn), scale)
    if q.method == "fp8_block":
        from ..quantization import formats
        payload = formats.fp8_quantize(w, block=True)
        return wq_pack.pack_fp8_block(payload["weight"], payload["weight_scale_inv"])
    if q.method == "nvfp4":
        from ..quantization import nvfp4
        payload = nvfp4.quantize(w, amax)
        return wq_pack.pack_nvfp4(payload["weight_packed"], payload["weight_scale"].float(),
                                  1.0 / float(payload["weight_global_scale"]))
    raise NotImplementedError(f"weight format {q.method}")


def random_decoder_weights(cfg: ModelConfig, device, seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                           std: float = 0.02, layer_range: tuple[int, int] | None = None,
                           ep_size: int | None = None) -> DecoderWeights:
    """Random-init N(0, std) weights, quantized offline into the config's format, rank-local TP shards.
    ``ep_size`` (mixture-of-experts models): expert owners among the ``tp_size`` ranks; the ``tp_size / ep_size`` lanes
    of an owner divide every owned expert's intermediate features (None: every rank owns whole experts).

    Column-parallel: QKV (whole heads per rank), gate/up; row-parallel: o_proj,
    down; vocab-sharded embedding and lm_head (reference ownership planners:
    ``models/parallel_weights.py:72-352``).  ``layer_range`` keeps only the layers ``[lo, hi)`` of one pipeline
    stage; every layer draws from its own generator, so a stage holds exactly the weights the whole model would.

    The model does not depend on the partition: every rank draws the FULL matrix of a projection from a generator
    seeded by (seed, layer) only and keeps its rows / columns, so the shards of any ``tp_size`` are slices of the
    one-GPU model (quantization groups lie along K in multiples of the shard widths, so quantizing a slice equals
    slicing the quantized matrix).  Outputs of different partitions can therefore be compared with each other.
    """
    from .config import kv_heads_of_rank
    assert cfg.num_q_heads % tp_size == 0
    kv_first, kv_count = kv_heads_of_rank(cfg.num_kv_heads, tp_rank, tp_size)
    gen = torch.Generator(device=device)
    H, D = cfg.hidden_size, cfg.head_dim
    hq, hkv = cfg.num_q_heads // tp_size, kv_count
    inter = cfg.intermediate_size // tp_size

    def qkv_rows(full):
        """This rank's query heads and its key/value heads (a copy of a shared head when ranks outnumber them) out of
        the full [q | k | v] projection."""
        kb = cfg.num_q_heads * D
        vb = kb + cfg.num_kv_heads * D
        return torch.cat([full[tp_rank * hq * D:(tp_rank + 1) * hq * D],
                          full[kb + kv_first * D:kb + (kv_first + hkv) * D],
                          full[vb + kv_first * D:vb + (kv_first + hkv) * D]])

    def rnd(n, k):
        return torch.randn(n, k, device=device, generator=gen, dtype=torch.float32) * std

    r = tp_rank

    def rows_of(full, width):
        """This rank's ``width`` rows of a matrix whose rows are owned in rank order."""
        return full[r * width:(r + 1) * width]

    def shard_q(full, pick):
        """Quantized shard ``pick(full)`` of a matrix, with the per-tensor scale (if the format has one) of the whole."""
        if cfg.quant.method == "fp8":
            # which rows the shard keeps: a row pick maps the probe's row numbers, a column pick keeps every row
            probe = torch.arange(full.shape[0], device=full.device).view(-1, 1)
            kept = pick(probe)
            rows = probe[:, 0] if kept.shape[1] == 0 else kept[:, 0]
            return quantize_linear(pick(full).contiguous(), cfg, row_amax=full.abs().amax(1)[rows])
        return quantize_linear(pick(full).contiguous(), cfg, float(full.abs().amax()) if cfg.quant.method == "nvfp4" else None)

    def cols_of(width):
        return lambda full: full[:, r * width:(r + 1) * width]

    def sections(full, widths):
        """``full`` is a stack of sections of ``tp_size * w`` rows each; this rank keeps rows ``[r w, (r + 1) w)`` of
        every section (q | k | v heads, gate | up features, ...)."""
        out, base = [], 0
        for w in widths:
            out.append(full[base + r * w:base + (r + 1) * w])
            base += w * tp_size
        return torch.cat(out)

    def norm_w():
        # zero-centred norms multiply by (1 + w)
        return torch.full((H,), 0.0 if cfg.zero_centered_norm else 1.0, device=device, dtype=torch.bfloat16)

    layers = []
    lo, hi = layer_range or (0, cfg.num_layers)
    for li in range(lo, hi):
        gen.manual_seed(seed * 4096000 + li)
        if cfg.layer_is_gdn(li):
            gk, gv = cfg.gdn_k_heads // tp_size, cfg.gdn_v_heads // tp_size
            f32 = dict(device=device, dtype=torch.float32)
            lw = LayerWeights(ln1=norm_w(), ln2=norm_w(), gdn=GdnWeights(
                in_proj=shard_q(rnd(2 * gk * 128 * tp_size + 2 * gv * 128 * tp_size, H),
                                lambda f: sections(f, [gk * 128, gk * 128, gv * 128, gv * 128])),
                in_ba=wq_pack.pack_bf16(sections(rnd(2 * gv * tp_size, H), [gv, gv])),
                conv_w=sections(torch.randn((2 * gk + gv) * 128 * tp_size, 4, generator=gen, **f32) * 0.3,
                                [gk * 128, gk * 128, gv * 128]),
                a_log=rows_of(torch.randn(gv * tp_size, generator=gen, **f32) * 0.5, gv),
                dt_bias=rows_of(torch.randn(gv * tp_size, generator=gen, **f32) * 0.5, gv),
                norm_w=torch.ones(128, **f32),
                out=shard_q(rnd(H, gv * 128 * tp_size), cols_of(gv * 128)),
                hk=gk, hv=gv))
        else:
            lw = LayerWeights(
                ln1=norm_w(), ln2=norm_w(),
                qkv=shard_q(rnd((cfg.num_q_heads + 2 * cfg.num_kv_heads) * D, H), qkv_rows),
                o=shard_q(rnd(H, hq * D * tp_size), cols_of(hq * D)),
            )
            if cfg.attn_output_gate:
                lw.attn_gate = shard_q(rnd(hq * D * tp_size, H), lambda f: rows_of(f, hq * D))
        if cfg.qk_norm and lw.gdn is None:
            lw.q_norm = torch.ones(D, device=device, dtype=torch.bfloat16)
            lw.k_norm = torch.ones(D, device=device, dtype=torch.bfloat16)
        if cfg.qkv_bias and lw.gdn is None:
            full = torch.randn((cfg.num_q_heads + 2 * cfg.num_kv_heads) * D, 1, device=device, generator=gen) * std
            lw.qkv_bias = qkv_rows(full).flatten().to(torch.bfloat16).contiguous()
        if cfg.is_moe:
            from .moe import random_moe_weights
            lw.moe = random_moe_weights(cfg, device, gen, tp_rank, tp_size, std, layer_seed=seed * 4096000 + li,
                                        ep_size=ep_size)
        else:
            lw.gate_up = shard_q(rnd(2 * inter * tp_size, H), lambda f: sections(f, [inter, inter]))
            lw.down = shard_q(rnd(H, inter * tp_size), cols_of(inter))
        layers.append(lw)
    gen.manual_seed(seed * 4096000 + 4095)
    v_local = cfg.vocab_size // tp_size
    # the embedding table is generated identically on every rank (rank-independent stream), kept whole
    # for the fused path (each rank embeds only the rows it owns) and sliced for the vocab-sharded baseline
    shared = torch.Generator(device=device).manual_seed(seed * 1000 + 999)
    embed_full = (torch.randn(cfg.vocab_size, H, device=device, generator=shared) * std).to(torch.bfloat16)
    embed = embed_full[tp_rank * v_local:(tp_rank + 1) * v_local]
    if cfg.tie_embeddings:
        head = embed
    else:
        head = rows_of((torch.randn(v_local * tp_size, H, device=device, generator=gen) * std).to(torch.bfloat16), v_local)
    lm_head = quantize_linear(head.float(), cfg) if cfg.quant.lm_head_quantized else wq_pack.pack_bf16(head)
    return DecoderWeights(embed=embed, layers=layers, final_norm=norm_w(), lm_head=lm_head,
                          vocab_start=tp_rank * v_local, extras={"embed_full": embed_full})


@dataclass
class StepBatch:
    """Device-side, fixed-address inputs of one forward step (filled by the executor)."""
    num_tokens: int
    num_row_blocks: int
    num_logit_rows: int
    token_ids: torch.Tensor      # int32 [T]
    positions: torch.Tensor      # int32 [T]
    slots: torch.Tensor          # int32 [T]  page*16 + offset, -1 = padding row
    page_table: torch.Tensor     # int32 [R, max_pages]
    rb_req: torch.Tensor         # int32 [RB]
    rb_qstart: torch.Tensor
    rb_qcount: torch.Tensor
    rb_ctx: torch.Tensor
    logit_rows: torch.Tensor     # int64 [R] rows of the hidden state that feed lm_head
    attn_splits: int = 1
    segments: object | None = None   # K.GdnSegments: the step's rows grouped by request (Gated DeltaNet layers)
    # multimodal prefill steps (one GPU): row- and column-axis rotary positions int32 [T] each (``positions`` is then
    # the temporal axis) and encoder feature rows ``[(first row, bf16 [n, H])]`` that replace token embeddings
    positions_hw: tuple | None = None
    embeds: list | None = None


class DecoderRunner:
    def __init__(self, cfg: ModelConfig, weights: DecoderWeights, num_pages: int, max_tokens: int,
                 k_bits: int = 8, v_bits: int = 8, tp=None, device=None, pp=None, max_requests: int = 256,
                 state_checkpoints: int = 0,
                 kv_rotation: bool = False) -> None:
        """``max_requests``: rows of the per-request recurrent state of Gated DeltaNet layers (= page-table rows).
        ``kv_rotation``: q / k / v head vectors are Walsh-Hadamard transformed before the cache write (smoother
        channels for INT4 / INT6 codes); the attention output is transformed back."""
        self.cfg = cfg
        self.w = weights            # ``weights.layers`` holds only the layers of this pipeline stage
        self.device = device or weights.embed.device
        self.tp = tp
        self.pp = pp                # parallel.pp.PipelineStage or None
        if pp is not None and tp is not None and tp.fused is not None:
            raise ValueError("pipeline stages use the NCCL tensor-parallel collectives (tp mode 'nccl')")
        if tp is not None and tp.fused is not None and any(
                pw is not None and pw.fmt in (wq_pack.FMT_FP8, wq_pack.FMT_FP8_BLOCK) for lw in weights.layers for pw in (lw.qkv, lw.o, lw.gate_up, lw.down)):
            # the fp8 GEMM's activation operand is quantized per token by a kernel of its own, which would read rows
            # that the fused all-gather has not delivered yet
            raise ValueError("FP8 weights run with the NCCL tensor-parallel collectives (tp mode 'nccl')")
        self.tp_size = tp.size if tp is not None else 1
        self.k_bits, self.v_bits = k_bits, v_bits
        self.kv_rotation = kv_rotation
        self.reasoning = None        # K.ReasoningBudget once enable_reasoning_budget() was called
        self.hq = cfg.num_q_heads // self.tp_size
        from .config import kv_heads_of_rank
        self.hkv = kv_heads_of_rank(cfg.num_kv_heads, 0, self.tp_size)[1]     # a shared head is held whole by its ranks
        self.D = cfg.head_dim
        self.max_tokens = max_tokens
        H = cfg.hidden_size
        dev = self.device
        blob = K.kv_blob_bytes(self.D, k_bits, v_bits)
        self.num_pages = num_pages
        # one cache tensor per layer: [pages, kv_heads, blob]; zero-filled so that
        # never-written slots hold finite scales
        self.kv = [torch.zeros(0 if lw.gdn is not None else num_pages, self.hkv, blob, dtype=torch.uint8, device=dev)
                   for lw in weights.layers]
        # Gated DeltaNet layers: per request the last three conv inputs of every channel and one 128 x 128 fp32 state
        # per value head; a request's row is its page-table row, reset implicitly when it starts at position 0
        self.max_requests = max_requests
        # rows [max_requests, max_requests + state_checkpoints) of the recurrent-state arrays hold snapshots taken at
        # page boundaries of prompts, so that cached prefixes of models with recurrent layers can be resumed
        self.state_checkpoint_rows = tuple(range(max_requests, max_requests + state_checkpoints))
        self.gdn_conv_state, self.gdn_state = {}, {}
        self.gdn_review = None       # set by begin_gdn_review(): the record of a speculative review pass
        self._gdn_record = None
        gdn_first = next((lw.gdn for lw in weights.layers if lw.gdn is not None), None)
        if gdn_first is not None:
            if tp is not None and tp.fused is not None:
                raise ValueError("Gated DeltaNet layers use the NCCL tensor-parallel collectives (tp mode 'nccl')")
            gk, gv = gdn_first.hk, gdn_first.hv
            C = (2 * gk + gv) * 128
            for li, lw in enumerate(weights.layers):
                if lw.gdn is not None:
                    rows = max_requests + state_checkpoints
                    self.gdn_conv_state[li] = torch.zeros(rows, 3, C, dtype=torch.bfloat16, device=dev)
                    self.gdn_state[li] = torch.zeros(rows, gv, 128, 128, dtype=torch.float32, device=dev)
            self.gdn_in = torch.empty(max_tokens, gdn_first.in_proj.n, dtype=torch.bfloat16, device=dev)
            self.gdn_ba = torch.empty(max_tokens, 2 * gv, dtype=torch.bfloat16, device=dev)
            self.gdn_mix = torch.empty(max_tokens, C, dtype=torch.bfloat16, device=dev)
            self.gdn_out = torch.empty(max_tokens, gv * 128, dtype=torch.bfloat16, device=dev)
        if any(lw.attn_gate is not None for lw in weights.layers):
            self.gate = torch.empty(max_tokens, self.hq * self.D, dtype=torch.bfloat16, device=dev)
        self.inv_freq = rope_inv_freq(cfg.rotary_dim or self.D, cfg.rope_theta, dev, scaling=cfg.rope_scaling)
        bf = torch.bfloat16
        T = max_tokens
        self.h = torch.empty(T, H, dtype=bf, device=dev)           # residual stream
        self.x = torch.empty(T, H, dtype=bf, device=dev)           # normed activations
        self.qkv = torch.empty(T, (self.hq + 2 * self.hkv) * self.D, dtype=bf, device=dev)
        self.q = torch.empty(T, self.hq * self.D, dtype=bf, device=dev)
        self.attn = torch.empty(T, self.hq * self.D, dtype=bf, device=dev)
        self.part = torch.empty(T, H, dtype=bf, device=dev)        # row-parallel partial sums (TP > 1)
        inter = (cfg.intermediate_size // self.tp_size) if not cfg.is_moe else 0
        self.gu = torch.empty(T, 2 * inter, dtype=bf, device=dev) if inter else None
        self.act = torch.empty(T, inter, dtype=bf, device=dev) if inter else None
        self.ws = K.workspace(dev)
        self.launches_per_step = 0
        from ..ops.strategies import active
        if active().gemm.fuse_swiglu and torch.device(dev).type == "cuda":
            # gate / up rows interleaved once, so that the GEMM epilogue applies the activation (no [T, 2I] round trip)
            for lw in weights.layers:
                if lw.moe is not None:
                    lw.moe.fuse_activation()
                elif lw.gate_up is not None and (lw.gate_up.n // 2) % 16 == 0:
                    lw.gate_up = wq_pack.swiglu_interleave(lw.gate_up)
        self.ep = None
        if cfg.is_moe and tp is not None and tp.fused is not None:
            # expert parallelism over the tensor-parallel group: fused dispatch / combine on the row-sharded stream
            if any(lw.moe is not None and lw.moe.shared_gate_up is not None for lw in weights.layers):
                raise ValueError("shared experts use the NCCL tensor-parallel collectives (tp mode 'nccl')")
            if any(lw.moe is not None and lw.moe.expert_count * self.tp_size != cfg.num_experts for lw in weights.layers):
                raise ValueError("experts divided into feature lanes use the NCCL tensor-parallel collectives "
                                 "(tp mode 'nccl'): the fused dispatch moves rows to owners of WHOLE experts")
            from ..parallel.ep import FusedEp, symmetric_ep_buffers
            bufs = symmetric_ep_buffers(tp.group, H, cfg.experts_per_token, tp.fused.b.max_tokens, dev)
            self.ep = FusedEp(bufs, dev, cfg.num_experts, 2 * cfg.moe_intermediate_size, ws=self.ws)

    def copy_state(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """Bit-preserving copies of whole recurrent-state rows ``src[i] -> dst[i]`` (int32 device tensors) in every
        Gated DeltaNet layer: delta-rule state and convolution history (reference: the captured owner-row copies of
        ``executor/state_transfer.py:140``).  Rows are request rows or snapshot rows."""
        for li, st in self.gdn_state.items():
            K.copy_rows(st, src, dst)
            K.copy_rows(self.gdn_conv_state[li], src, dst)

    # ---------------------------------------------------------------- forward
    def forward_hidden(self, b: StepBatch) -> torch.Tensor:
        """Run this stage's layers for ``b.num_tokens`` rows; returns the residual stream view ``[T, H]``.

        With pipeline parallelism the rows are processed in wavefront lanes: a later stage receives a lane's
        rows from its predecessor, an earlier stage sends them on, and the next lane's compute overlaps the
        successor's work on the previous one (reference: ``runtime/performance.py:199-211``).
        """
        T = b.num_tokens
        pp = self.pp
        self.launches_per_step = 0
        if pp is None:
            self._run_layers(b, 0, T, 0, b.num_row_blocks, embed=True)
            return self.h[:T]
        from ..parallel.pp import split_lanes
        for t0, t1, rb0, rb1 in split_lanes(T, b.num_row_blocks, pp.lanes):
            if not pp.is_first:
                pp.recv(self.h[t0:t1])
            self._run_layers(b, t0, t1, rb0, rb1, embed=pp.is_first)
            if not pp.is_last:
                pp.send(self.h[t0:t1])
        return self.h[:T]

    def _gdn_mixer(self, li: int, g: GdnWeights, x: torch.Tensor, b: StepBatch, t0: int, t1: int) -> torch.Tensor:
        """Gated DeltaNet token mixer of layer ``li`` over rows ``[t0, t1)``: projection, causal conv + SiLU, gated
        delta rule + gated norm.  Returns the ``[rows, Hv 128]`` input of the output projection."""
        if b.segments is None:
            raise RuntimeError("Gated DeltaNet layers need the step's request segments (StepBatch.segments)")
        if t0 != 0 or t1 != b.num_tokens:
            raise NotImplementedError("pipeline lanes split a step's rows; Gated DeltaNet layers take whole steps")
        rec = self.gdn_review
        if rec is None:
            proj, ba = self.gdn_in[t0:t1], self.gdn_ba[t0:t1]
        else:
            # speculative review pass: the layer's projections are kept (the fold replays the accepted prefix from
            # them) and the recurrent state is read but not written
            proj, ba = rec["proj"][li][t0:t1], rec["ba"][li][t0:t1]
        K.wq_gemm(x, g.in_proj, out=proj, ws=self.ws)
        K.wq_gemm(x, g.in_ba, out=ba, ws=self.ws)
        C = (2 * g.hk + g.hv) * 128
        mix, out = self.gdn_mix[t0:t1], self.gdn_out[t0:t1]
        K.gdn_conv(proj, g.conv_w, self.gdn_conv_state[li], b.segments, mix, commit=rec is None)
        z = proj[:, C:C + g.hv * 128]
        K.gdn_delta(mix, z, ba, g.a_log, g.dt_bias, g.norm_w, self.gdn_state[li], b.segments, out, g.hk, g.hv,
                    eps_norm=self.cfg.rms_eps, commit=rec is None)
        return out

    def begin_gdn_review(self, rows: int) -> None:
        """The next ``forward_hidden`` is a speculative review pass over ``rows`` token rows: Gated DeltaNet layers
        leave their state untouched and keep their projections for ``fold_gdn``."""
        if not self.gdn_state:
            return
        if self._gdn_record is None or self._gdn_record["rows"] < rows:
            first = next(lw.gdn for lw in self.w.layers if lw.gdn is not None)
            dev = self.device
            self._gdn_record = {"rows": rows,
                                "proj": {li: torch.empty(rows, first.in_proj.n, dtype=torch.bfloat16, device=dev)
                                         for li in self.gdn_state},
                                "ba": {li: torch.empty(rows, 2 * first.hv, dtype=torch.bfloat16, device=dev)
                                       for li in self.gdn_state}}
        self.gdn_review = self._gdn_record

    def fold_gdn(self, segments: "K.GdnSegments", rows: int) -> int:
        """Bring the recurrent state of every Gated DeltaNet layer to the accepted position of a reviewed round:
        ``segments`` describes, per request, the first row of its review rows and HOW MANY of them were accepted
        (a device tensor, so no host round trip); the conv and delta kernels replay exactly those rows from the
        projections kept by the review pass, this time writing the state.  Returns the launches made.
        (Reference: ``ops/cuda/linear_attention/gated_delta_fold.cu:22``, a kernel of its own there.)"""
        rec, self.gdn_review = self.gdn_review, None
        if rec is None:
            return 0
        n = 0
        for li, lw in enumerate(self.w.layers):
            g = lw.gdn
            if g is None:
                continue
            C = (2 * g.hk + g.hv) * 128
            proj, ba = rec["proj"][li][:rows], rec["ba"][li][:rows]
            mix, out = self.gdn_mix[:rows], self.gdn_out[:rows]
            K.gdn_conv(proj, g.conv_w, self.gdn_conv_state[li], segments, mix)
            K.gdn_delta(mix, proj[:, C:C + g.hv * 128], ba, g.a_log, g.dt_bias, g.norm_w, self.gdn_state[li], segments,
                        out, g.hk, g.hv, eps_norm=self.cfg.rms_eps)
            n += 2
        return n

    def _run_layers(self, b: StepBatch, t0: int, t1: int, rb0: int, rb1: int, embed: bool) -> None:
        """Layers of this stage over rows ``[t0, t1)`` whose attention row blocks are ``[rb0, rb1)``."""
        cfg, w = self.cfg, self.w
        T = b.num_tokens
        h, x = self.h[t0:t1], self.x[t0:t1]
        qkv, q, attn = self.qkv[t0:t1], self.q[t0:t1], self.attn[t0:t1]
        # attention addresses query rows by their absolute index, so it gets the whole q / out buffers
        q_all, attn_all = self.q[:T].view(T, self.hq, self.D), self.attn[:T].view(T, self.hq, self.D)
        n = 0
        if embed:
            K.embedding(b.token_ids[t0:t1], w.embed, out=h, vocab_start=w.vocab_start)
            n += 1
            if self.tp is not None:
                self.tp.all_reduce(h)
            for first, rows in (b.embeds or ()):               # encoder features take the place of the embeddings
                lo, hi = max(first, t0), min(first + rows.shape[0], t1)
                if lo < hi:
                    h[lo - t0:hi - t0].copy_(rows[lo - first:hi - first])
        pending = None  # partial sum waiting to be folded into h by the next norm (TP > 1)
        fp8s = (wq_pack.FMT_FP8, wq_pack.FMT_FP8_BLOCK)

        def norm(src, weight, residual, consumers):
            """RMSNorm into ``x``; when every consumer of the result is an fp8 GEMM the norm kernel quantizes its own
            output per token and the e4m3 operand is returned instead (no bf16 round trip, no extra launch)."""
            if consumers and all(c is not None and c.fmt in fp8s for c in consumers):
                return K.rmsnorm_fp8(src, weight, cfg.rms_eps, residual=residual, zero_centered=cfg.zero_centered_norm,
                                     ws=self.ws)
            return K.rmsnorm(src, weight, cfg.rms_eps, out=x, residual=residual, zero_centered=cfg.zero_centered_norm)

        def row_in(t, weight):
            """Input of a row-parallel projection under tensor parallelism: an fp8 projection's operand is quantized
            with the MAX over the ranks of the per-token scales, i.e. with the scale of the unsharded row, so that
            the partition does not change the codes (the reference's scale collective)."""
            if weight.fmt not in fp8s:
                return t
            return K.fp8_quantize(t, self.ws, scale_max=self.tp.all_reduce_max)

        for li, lw in enumerate(w.layers):
            xin = norm(pending if pending is not None else h, lw.ln1, h if pending is not None else None,
                       [] if lw.gdn is not None else [lw.qkv] + ([lw.attn_gate] if lw.attn_gate is not None else []))
            if lw.gdn is not None:
                mixed, o_w = self._gdn_mixer(li, lw.gdn, x, b, t0, t1), lw.gdn.out
                n += 5
            else:
                K.wq_gemm(xin, lw.qkv, out=qkv, ws=self.ws)
                hw = None if b.positions_hw is None else (b.positions_hw[0][t0:t1], b.positions_hw[1][t0:t1])
                K.rope_kv_write(qkv, q, self.kv[li], b.positions[t0:t1], b.slots[t0:t1], self.inv_freq, self.hq, self.hkv,
                                self.D, self.k_bits, self.v_bits, q_norm=lw.q_norm, k_norm=lw.k_norm, eps=cfg.rms_eps,
                                rotary_dim=cfg.rotary_dim, rotate=self.kv_rotation, positions_hw=hw,
                                mrope_section=cfg.mrope_section if hw is not None else None, qkv_bias=lw.qkv_bias)
                K.paged_attention(q_all, attn_all, self.kv[li], b.page_table, b.rb_req[rb0:rb1], b.rb_qstart[rb0:],
                                  b.rb_qcount[rb0:], b.rb_ctx[rb0:], self.hq, self.hkv, self.D, self.k_bits, self.v_bits,
                                  scale=cfg.attention_scale, splits=b.attn_splits, ws=self.ws)
                n += 4
                if self.kv_rotation:
                    K.hadamard(attn)
                    n += 1
                if lw.attn_gate is not None:
                    gate = self.gate[t0:t1]
                    K.wq_gemm(xin, lw.attn_gate, out=gate, ws=self.ws)
                    K.sigmoid_gate(attn, gate)
                    n += 2
                mixed, o_w = attn, lw.o
            ffn_in = [] if lw.moe is not None else [lw.gate_up]
            if self.tp is None:
                K.wq_gemm(mixed, o_w, out=h, residual=h, ws=self.ws)
                xin = norm(h, lw.ln2, None, ffn_in)
            else:
                part = self.part[t0:t1]
                K.wq_gemm(row_in(mixed, o_w), o_w, out=part, ws=self.ws)
                self.tp.all_reduce(part)
                xin = norm(part, lw.ln2, h, ffn_in)
            # fp8 projections whose input is not a norm's output (attention output, activation) quantize it first
            per_quant = 1 if self.tp is None else 3          # sharded operands: scale, MAX over ranks, quantize
            n += 2 + per_quant * ((o_w.fmt in fp8s) + (lw.moe is None and lw.down.fmt in fp8s))
            if lw.moe is not None:
                n += lw.moe.launches
                if self.tp is None:
                    lw.moe.forward(x, self, residual=h, out=h)     # combine adds into the residual stream
                    pending = None
                else:
                    out = lw.moe.forward(x, self)                  # this rank's experts only: a partial sum
                    self.tp.all_reduce(out)
                    pending = out
            else:
                gu, act = self.gu[t0:t1], self.act[t0:t1]
                n += 1 + K.gate_up_act(xin, lw.gate_up, gu, act, ws=self.ws)
                if self.tp is None:
                    K.wq_gemm(act, lw.down, out=h, residual=h, ws=self.ws)
                else:
                    part = self.part[t0:t1]
                    K.wq_gemm(row_in(act, lw.down), lw.down, out=part, ws=self.ws)
                    self.tp.all_reduce(part)
                    pending = part
        if pending is not None:
            h.add_(pending)
        self.launches_per_step += n

    def forward_logits(self, b: StepBatch, hidden: torch.Tensor, logits_out: torch.Tensor) -> torch.Tensor:
        """Final norm + lm_head for the selected rows -> bf16 logits ``[R, V(/tp)]``."""
        R = b.num_logit_rows
        # the normed-activation buffer is free once the last layer has run: it takes the gathered + normed rows
        xn = K.rmsnorm_rows(hidden, b.logit_rows[:R], self.w.final_norm, self.cfg.rms_eps, out=self.x[:R],
                            zero_centered=self.cfg.zero_centered_norm)
        K.wq_gemm(xn, self.w.lm_head, out=logits_out[:R], ws=self.ws)
        self.launches_per_step += 2
        return logits_out[:R]

    # ------------------------------------------------------- fused tensor parallel
    def forward_hidden_fused(self, b: StepBatch) -> int:
        """All layers on the fused NVLink path; returns the buffer set that holds the final normalised rows.

        The residual stream is sharded by ROWS (each rank keeps the rows it owns), activations that feed a
        column-parallel GEMM are all-gathered by push, partial sums of row-parallel GEMMs are
        reduce-scattered by push; see ``parallel/tp.py``.
        """
        cfg, w, f = self.cfg, self.w, self.tp.fused
        T, H = b.num_tokens, cfg.hidden_size
        f.begin_step(T)
        lo = f.rank * f.rpr
        cnt = max(0, min(T, lo + f.rpr) - lo)
        n = 0
        if cnt:
            K.embedding(b.token_ids[lo:lo + cnt], w.extras["embed_full"], out=f.h_local[:cnt])
            n += 1
        qkv, q, attn = self.qkv[:T], self.q[:T], self.attn[:T]
        s = 0
        f.reduce_norm(w.layers[0].ln1, s, 0, cfg.rms_eps, cfg.zero_centered_norm, reduce=False)
        n += 1
        for li, lw in enumerate(w.layers):
            f.gemm_gather(lw.qkv, qkv, s)
            K.rope_kv_write(qkv, q, self.kv[li], b.positions, b.slots, self.inv_freq, self.hq, self.hkv, self.D,
                            self.k_bits, self.v_bits, q_norm=lw.q_norm, k_norm=lw.k_norm, eps=cfg.rms_eps,
                            rotary_dim=cfg.rotary_dim, rotate=self.kv_rotation, qkv_bias=lw.qkv_bias)
            K.paged_attention(q.view(T, self.hq, self.D), attn.view(T, self.hq, self.D), self.kv[li], b.page_table,
                              b.rb_req[:b.num_row_blocks], b.rb_qstart, b.rb_qcount, b.rb_ctx, self.hq, self.hkv,
                              self.D, self.k_bits, self.v_bits, scale=cfg.attention_scale, splits=b.attn_splits, ws=self.ws)
            if self.kv_rotation:
                K.hadamard(attn)
                n += 1
            s ^= 1
            f.gemm_scatter(attn, lw.o, s)
            nxt = w.layers[li + 1].ln1 if li + 1 < len(w.layers) else w.final_norm
            if lw.moe is not None:
                # MoE block on the row-sharded stream: the normalised rows stay on their home rank, the
                # expert-parallel kernels move each row only to the ranks that own one of its experts and add
                # the combined result into h_local; the next norm then gathers for the attention GEMM
                f.reduce_norm(lw.ln2, s, H, cfg.rms_eps, cfg.zero_centered_norm, local_only=True)
                self.ep.forward(lw.moe, f.b.xfull[s, lo:lo + f.rpr], cnt, f.h_local)
                s ^= 1
                f.reduce_norm(nxt, s, 0, cfg.rms_eps, cfg.zero_centered_norm, reduce=False)
                n += 7 + self.ep.launches
                continue
            f.reduce_norm(lw.ln2, s, H, cfg.rms_eps, cfg.zero_centered_norm)
            gu, act = self.gu[:T], self.act[:T]
            fused = 2 - f.gate_up_act(lw.gate_up, gu, act, s)
            s ^= 1
            f.gemm_scatter(act, lw.down, s)
            f.reduce_norm(nxt, s, H, cfg.rms_eps, cfg.zero_centered_norm)
            n += 9 - fused
        self.launches_per_step = n
        return s

    def _dummy_val(self) -> torch.Tensor:
        if not hasattr(self, "_cand_val"):
            self._cand_val = torch.zeros(1, dtype=torch.float32, device=self.device)
            self._cand_id = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._cand_val

    def _dummy_id(self) -> torch.Tensor:
        self._dummy_val()
        return self._cand_id

    def enable_reasoning_budget(self, end_token_id: int, forced_tokens: list[int]) -> None:
        """Enforce thinking-token budgets on the device (before the decode graphs are captured): after the budget of
        a request is used up its sampled ids are replaced by ``forced_tokens`` (1-4 tokens, ending the reasoning
        block); sampling ``end_token_id`` on its own ends the phase.  Every rank and stage runs the same state
        machine on the same ids."""
        self.reasoning = K.ReasoningBudget(self.max_requests, end_token_id, forced_tokens, self.device)

    def run_step(self, b: StepBatch, d: dict, logits_buf: torch.Tensor, out_ids: torch.Tensor) -> None:
        """Whole step: layers, final norm, lm_head, sampling (and the cross-rank token agreement under TP), then the
        thinking-budget state machine on the sampled ids when it is enabled."""
        self._run_step(b, d, logits_buf, out_ids)
        if self.reasoning is not None and b.num_logit_rows:
            self.reasoning.apply(out_ids, d["row_slot"], d["budget_init"], b.num_logit_rows)
            self.launches_per_step += 1

    def _run_step(self, b: StepBatch, d: dict, logits_buf: torch.Tensor, out_ids: torch.Tensor) -> None:
        R = b.num_logit_rows
        fused = self.tp is not None and self.tp.fused is not None
        pp = self.pp
        if not fused:
            hidden = self.forward_hidden(b)
            if not R:
                return
            if pp is not None and not pp.is_last:
                pp.share_token_ids(out_ids[:R])        # receive what the last stage sampled
                return
            logits = self.forward_logits(b, hidden, logits_buf)
        else:
            f = self.tp.fused
            s = self.forward_hidden_fused(b)
            if R == b.num_tokens:
                logits = f.gemm_gather(self.w.lm_head, logits_buf[:R], s)
            else:
                x = f.wait_gather(s)
                if R:
                    rows = torch.index_select(x, 0, b.logit_rows[:R])
                    logits = K.wq_gemm(rows, self.w.lm_head, out=logits_buf[:R], ws=self.ws)
            self.launches_per_step += 2
        mask = d.get("mask")             # allowed-token bitmask rows [R, ceil(V / 32)] (structured output) or None
        if mask is not None:
            mask = mask[:R, self.w.vocab_start // 32:]       # this rank's vocabulary shard starts at a word boundary
        if self.tp is None:
            K.sample(logits, out_ids[:R], temperature=d["temperature"][:R], top_p=d["top_p"][:R], top_k=d["top_k"][:R],
                     seeds=d["seeds"][:R], counters=d["draws"][:R], vocab=logits.shape[1], mask=mask)
            self.launches_per_step += 1
            if pp is not None:
                pp.share_token_ids(out_ids[:R])
            return
        # vocab-sharded: rank-local candidates (one for a greedy row, up to 20 for a sampled one), exchanged
        # between the ranks, then the same merge + draw on every rank
        if fused:
            if R:
                self.tp.fused.sample_sharded(logits, R, out_ids, d, self.w.vocab_start, mask)
            else:
                self.tp.fused.argmax_merge(self._dummy_val(), self._dummy_id(), out_ids, 0)   # step barrier only
        elif R:
            self.tp.sample_sharded_nccl(logits, R, out_ids, d, self.w.vocab_start, mask)
        self.launches_per_step += 3
        if pp is not None and R:
            pp.share_token_ids(out_ids[:R])
