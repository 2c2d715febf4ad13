"""Vision tower of the multimodal families: patches -> feature rows of the decoder's width.

The tower is a pre-norm ViT over ``[patches, C * Tp * p * p]`` pixel rows that arrive in merge-block order (the
``m x m`` patches that the merger folds into one decoder row are consecutive):

* patch embedding: the strided 3-D convolution of the checkpoint is one GEMM over the flattened patch;
* learned positions: the ``side x side`` table is read at ``linspace(0, side - 1, h) x linspace(0, side - 1, w)``
  with bilinear weights, so any grid maps onto the trained table;
* blocks: LayerNorm -> attention (bias, rotate-half rotary over the (row, column) of the patch, every frame attends
  only to itself) -> LayerNorm -> GELU(tanh) MLP;
* merger: LayerNorm, fold ``m x m`` neighbours into one row, two linear layers with an exact GELU between; optional
  "deepstack" mergers read intermediate layers (their norm runs after the fold).

Tensor parallelism shards attention heads and the MLP's hidden features over the ranks of the first pipeline stage;
the two row-parallel projections of a block are completed by the ``reduce`` callable (an all-reduce of the partial
rows).  GEMMs and attention are library calls: the encoder runs once per image, outside the decode loop.

Tensor names are the checkpoint's (``model.visual.`` prefix stripped).  Reference counterpart:
``models/qwen3_5/multimodal.py:646-983`` (reference encoder), ``models/qwen4_exp/weights.py:589-656`` (tensor
inventory), ``executor/vision.py:223-507`` (serving graph).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Mapping

import torch
import torch.nn.functional as F


class VisionConfigError(ValueError):
    pass


@dataclass(frozen=True)
class VisionConfig:
    depth: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    out_hidden_size: int
    in_channels: int = 3
    patch_size: int = 16
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    num_position_embeddings: int = 2304
    hidden_act: str = "gelu_pytorch_tanh"
    deepstack_visual_indexes: tuple[int, ...] = ()
    rope_theta: float = 10000.0
    norm_eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_width(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def merge_width(self) -> int:
        return self.hidden_size * self.spatial_merge_size ** 2

    @property
    def side(self) -> int:
        return math.isqrt(self.num_position_embeddings)

    @staticmethod
    def from_hf(raw: Mapping[str, object]) -> "VisionConfig":
        """``vision_config`` of a checkpoint's ``config.json``; unknown keys are refused."""
        known = {"depth", "hidden_size", "intermediate_size", "num_heads", "out_hidden_size", "in_channels", "patch_size",
                 "spatial_merge_size", "temporal_patch_size", "num_position_embeddings", "hidden_act",
                 "deepstack_visual_indexes", "model_type", "initializer_range", "dtype", "torch_dtype"}
        extra = sorted(set(raw) - known)
        if extra:
            raise VisionConfigError(f"vision_config has unknown keys {extra}")
        try:
            cfg = VisionConfig(
                depth=int(raw["depth"]), hidden_size=int(raw["hidden_size"]), intermediate_size=int(raw["intermediate_size"]),
                num_heads=int(raw["num_heads"]), out_hidden_size=int(raw["out_hidden_size"]),
                in_channels=int(raw.get("in_channels", 3)), patch_size=int(raw.get("patch_size", 16)),
                spatial_merge_size=int(raw.get("spatial_merge_size", 2)),
                temporal_patch_size=int(raw.get("temporal_patch_size", 2)),
                num_position_embeddings=int(raw.get("num_position_embeddings", 2304)),
                hidden_act=str(raw.get("hidden_act", "gelu_pytorch_tanh")),
                deepstack_visual_indexes=tuple(int(i) for i in raw.get("deepstack_visual_indexes", ())))
        except KeyError as e:
            raise VisionConfigError(f"vision_config lacks {e.args[0]!r}") from None
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if min(self.depth, self.hidden_size, self.intermediate_size, self.num_heads, self.out_hidden_size, self.in_channels,
               self.patch_size, self.spatial_merge_size, self.temporal_patch_size) <= 0:
            raise VisionConfigError("vision sizes are positive")
        if self.hidden_size % self.num_heads or self.head_dim % 4:
            raise VisionConfigError("the head width is hidden / heads and a multiple of 4 (two rotary axes)")
        if self.side * self.side != self.num_position_embeddings:
            raise VisionConfigError("the position table is square")
        if self.hidden_act not in ("gelu_pytorch_tanh", "gelu", "silu"):
            raise VisionConfigError(f"unknown activation {self.hidden_act!r}")
        idx = self.deepstack_visual_indexes
        if len(set(idx)) != len(idx) or any(not 0 <= i < self.depth for i in idx):
            raise VisionConfigError("deepstack indexes are distinct layers of the tower")


# ------------------------------------------------------------------ weights
def vision_tensor_shapes(cfg: VisionConfig) -> dict[str, tuple[int, ...]]:
    """Every tensor of the tower by checkpoint name (without the ``model.visual.`` prefix)."""
    h, i, mw = cfg.hidden_size, cfg.intermediate_size, cfg.merge_width
    s: dict[str, tuple[int, ...]] = {
        "patch_embed.proj.weight": (h, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size),
        "patch_embed.proj.bias": (h,), "pos_embed.weight": (cfg.num_position_embeddings, h)}
    for l in range(cfg.depth):
        p = f"blocks.{l}"
        s.update({f"{p}.norm1.weight": (h,), f"{p}.norm1.bias": (h,), f"{p}.norm2.weight": (h,), f"{p}.norm2.bias": (h,),
                  f"{p}.attn.qkv.weight": (3 * h, h), f"{p}.attn.qkv.bias": (3 * h,),
                  f"{p}.attn.proj.weight": (h, h), f"{p}.attn.proj.bias": (h,),
                  f"{p}.mlp.linear_fc1.weight": (i, h), f"{p}.mlp.linear_fc1.bias": (i,),
                  f"{p}.mlp.linear_fc2.weight": (h, i), f"{p}.mlp.linear_fc2.bias": (h,)})

    def merger(p: str, norm_width: int) -> None:
        s.update({f"{p}.norm.weight": (norm_width,), f"{p}.norm.bias": (norm_width,),
                  f"{p}.linear_fc1.weight": (mw, mw), f"{p}.linear_fc1.bias": (mw,),
                  f"{p}.linear_fc2.weight": (cfg.out_hidden_size, mw), f"{p}.linear_fc2.bias": (cfg.out_hidden_size,)})
    merger("merger", h)
    for j in range(len(cfg.deepstack_visual_indexes)):
        merger(f"deepstack_merger_list.{j}", mw)
    return s


def random_vision_weights(cfg: VisionConfig, seed: int = 0, dtype=torch.float32, device="cpu", std: float = 0.05):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in vision_tensor_shapes(cfg).items():
        if name.endswith("norm.weight") or ".norm1.weight" in name or ".norm2.weight" in name:
            t = 1 + 0.1 * torch.randn(shape, generator=g)
        else:
            t = std * torch.randn(shape, generator=g)
        out[name] = t.to(dtype).to(device)
    return out


def check_vision_weights(cfg: VisionConfig, weights: Mapping[str, torch.Tensor]) -> None:
    """The closed inventory: every expected tensor present with its shape, nothing else."""
    want = vision_tensor_shapes(cfg)
    missing = sorted(set(want) - set(weights))
    extra = sorted(set(weights) - set(want))
    if missing or extra:
        raise VisionConfigError(f"vision tensors missing {missing[:4]} unexpected {extra[:4]}")
    for n, shape in want.items():
        if tuple(weights[n].shape) != shape:
            raise VisionConfigError(f"{n}: shape {tuple(weights[n].shape)}, expected {shape}")


def shard_vision_weights(cfg: VisionConfig, weights: Mapping[str, torch.Tensor], rank: int, size: int) -> dict:
    """The tensors rank ``rank`` of ``size`` keeps: attention heads and MLP features are divided, the biases of the
    row-parallel projections stay whole (added once, after the partial rows are summed), everything else is
    replicated."""
    if size == 1:
        return dict(weights)
    if cfg.num_heads % size or cfg.intermediate_size % size:
        raise VisionConfigError(f"{cfg.num_heads} heads / {cfg.intermediate_size} features do not divide over {size} ranks")
    h, hl, il = cfg.hidden_size, cfg.hidden_size // size, cfg.intermediate_size // size
    out = {}
    for n, t in weights.items():
        if n.endswith("attn.qkv.weight") or n.endswith("attn.qkv.bias"):
            parts = t.reshape(3, h, *t.shape[1:])[:, rank * hl:(rank + 1) * hl]
            t = parts.reshape(3 * hl, *t.shape[1:])
        elif n.endswith("attn.proj.weight"):
            t = t[:, rank * hl:(rank + 1) * hl]
        elif n.startswith("blocks.") and (n.endswith("linear_fc1.weight") or n.endswith("linear_fc1.bias")):
            t = t[rank * il:(rank + 1) * il]
        elif n.startswith("blocks.") and n.endswith("linear_fc2.weight"):
            t = t[:, rank * il:(rank + 1) * il]
        out[n] = t.contiguous()
    return out


def group_reduce(group=None) -> Callable[[torch.Tensor], torch.Tensor]:
    """The ``reduce`` of a sharded tower bound to a ``torch.distributed`` group: the partial rows of a row-parallel
    projection summed over the ranks of the first pipeline stage (every rank gets the same bits)."""
    import torch.distributed as dist

    def reduce(t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=group)
        return t
    return reduce


# ------------------------------------------------------------------ geometry of a request's grids
def _grids(grid_thw) -> list[tuple[int, int, int]]:
    g = torch.as_tensor(grid_thw).reshape(-1, 3).tolist()
    return [(int(t), int(h), int(w)) for t, h, w in g]


def merge_order(h: int, w: int, m: int, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """(row, column) of every patch of an ``h x w`` frame in merge-block order."""
    r, c = torch.meshgrid(torch.arange(h, device=device), torch.arange(w, device=device), indexing="ij")
    shape = (h // m, m, w // m, m)
    return r.reshape(shape).transpose(1, 2).flatten(), c.reshape(shape).transpose(1, 2).flatten()


def patch_positions(grid_thw, m: int, device=None) -> torch.Tensor:
    """``[patches, 2]`` (row, column) for the rotary embedding; frames of one item repeat the frame's pattern."""
    out = []
    for t, h, w in _grids(grid_thw):
        r, c = merge_order(h, w, m, device)
        out.append(torch.stack((r, c), -1).repeat(t, 1))
    return torch.cat(out, 0)


def bilinear_table_reads(grid_thw, side: int, m: int, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """Four table rows and weights per patch: ``(indices [4, patches] int64, weights [4, patches] fp32)``."""
    idx, wts = [], []
    for t, h, w in _grids(grid_thw):
        ys = torch.linspace(0, side - 1, h, device=device)
        xs = torch.linspace(0, side - 1, w, device=device)
        y0, x0 = ys.long(), xs.long()
        y1, x1 = (y0 + 1).clamp_max(side - 1), (x0 + 1).clamp_max(side - 1)
        fy, fx = ys - y0, xs - x0
        i4 = torch.stack([(y0[:, None] * side + x0[None, :]), (y0[:, None] * side + x1[None, :]),
                          (y1[:, None] * side + x0[None, :]), (y1[:, None] * side + x1[None, :])]).reshape(4, h * w)
        w4 = torch.stack([((1 - fy)[:, None] * (1 - fx)[None, :]), ((1 - fy)[:, None] * fx[None, :]),
                          (fy[:, None] * (1 - fx)[None, :]), (fy[:, None] * fx[None, :])]).reshape(4, h * w)
        r, c = merge_order(h, w, m, device)
        order = r * w + c
        idx.append(i4[:, order].repeat(1, t))
        wts.append(w4[:, order].repeat(1, t))
    return torch.cat(idx, 1), torch.cat(wts, 1)


def frame_lengths(grid_thw) -> list[int]:
    """Patches per attention segment (one per frame)."""
    return [h * w for t, h, w in _grids(grid_thw) for _ in range(t)]


def feature_rows(grid_thw, m: int) -> list[int]:
    """Decoder rows each item yields."""
    return [t * h * w // (m * m) for t, h, w in _grids(grid_thw)]


def validate_patches(cfg: VisionConfig, pixel_values: torch.Tensor, grid_thw) -> None:
    if pixel_values.dim() != 2 or pixel_values.shape[1] != cfg.patch_width or not pixel_values.is_floating_point():
        raise ValueError(f"pixel rows are floating point [patches, {cfg.patch_width}]")
    grids = _grids(grid_thw)
    m = cfg.spatial_merge_size
    if not grids or any(min(g) <= 0 or g[1] % m or g[2] % m for g in grids):
        raise ValueError("grids are positive (t, h, w) with h and w whole numbers of merge blocks")
    if sum(t * h * w for t, h, w in grids) != pixel_values.shape[0]:
        raise ValueError("the grids do not account for the pixel rows supplied")


# ------------------------------------------------------------------ the encoder
class VisionEncoder:
    """``encode(pixel_values, grid_thw) -> (rows [n, out_hidden], [deepstack rows...])``."""

    def __init__(self, cfg: VisionConfig, weights: Mapping[str, torch.Tensor], tp_rank: int = 0, tp_size: int = 1,
                 reduce: Callable[[torch.Tensor], torch.Tensor] | None = None, segment_rows: int = 1 << 14) -> None:
        cfg.validate()
        if tp_size > 1 and reduce is None:
            raise ValueError("a sharded tower needs the reduction of its partial rows")
        self.cfg, self.tp_rank, self.tp_size, self.reduce = cfg, tp_rank, tp_size, reduce
        self.w = dict(weights)
        first = self.w["patch_embed.proj.weight"]
        self.dtype, self.device = first.dtype, first.device
        self.patch_w = first.reshape(cfg.hidden_size, cfg.patch_width)
        self.heads = cfg.num_heads // tp_size
        quarter = cfg.head_dim // 4
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(quarter, dtype=torch.float32, device=self.device) / quarter))
        self.segment_rows = segment_rows
        self.encoded_patches = 0

    # row-parallel projection: partial rows summed over the ranks, the bias once
    def _row(self, x: torch.Tensor, name: str) -> torch.Tensor:
        if self.tp_size == 1:
            return F.linear(x, self.w[name + ".weight"], self.w[name + ".bias"])
        return self.reduce(F.linear(x, self.w[name + ".weight"])) + self.w[name + ".bias"]

    def _act(self, x: torch.Tensor) -> torch.Tensor:
        a = self.cfg.hidden_act
        return F.gelu(x, approximate="tanh") if a == "gelu_pytorch_tanh" else F.gelu(x) if a == "gelu" else F.silu(x)

    def _norm(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.layer_norm(x, (x.shape[-1],), self.w[name + ".weight"], self.w[name + ".bias"], self.cfg.norm_eps)

    def _attention(self, x: torch.Tensor, p: str, cos: torch.Tensor, sin: torch.Tensor, lengths: list[int]) -> torch.Tensor:
        n, d = x.shape[0], self.cfg.head_dim
        qkv = F.linear(x, self.w[p + ".attn.qkv.weight"], self.w[p + ".attn.qkv.bias"]).view(n, 3, self.heads, d)
        q, k, v = qkv.unbind(1)

        def rot(t: torch.Tensor) -> torch.Tensor:
            tf = t.float()
            half = torch.cat((-tf[..., d // 2:], tf[..., :d // 2]), -1)
            return (tf * cos + half * sin).to(t.dtype)
        q, k = rot(q), rot(k)
        out = torch.empty_like(q)
        at = 0
        for ln in lengths:                                            # every frame attends to itself only
            sl = slice(at, at + ln)
            o = F.scaled_dot_product_attention(q[sl].transpose(0, 1)[None], k[sl].transpose(0, 1)[None],
                                               v[sl].transpose(0, 1)[None])
            out[sl] = o[0].transpose(0, 1)
            at += ln
        return self._row(out.reshape(n, self.heads * d), p + ".attn.proj")

    def _merge(self, x: torch.Tensor, p: str, norm_after_fold: bool) -> torch.Tensor:
        mw = self.cfg.merge_width
        x = self._norm(x.view(-1, mw), p + ".norm") if norm_after_fold else self._norm(x, p + ".norm").view(-1, mw)
        x = F.gelu(F.linear(x, self.w[p + ".linear_fc1.weight"], self.w[p + ".linear_fc1.bias"]))
        return F.linear(x, self.w[p + ".linear_fc2.weight"], self.w[p + ".linear_fc2.bias"])

    @torch.no_grad()
    def encode(self, pixel_values: torch.Tensor, grid_thw) -> tuple[torch.Tensor, list[torch.Tensor]]:
        cfg = self.cfg
        validate_patches(cfg, pixel_values, grid_thw)
        dev, m = self.device, cfg.spatial_merge_size
        x = F.linear(pixel_values.to(dev, self.dtype), self.patch_w, self.w["patch_embed.proj.bias"])
        idx, wts = bilinear_table_reads(grid_thw, cfg.side, m, dev)
        table = self.w["pos_embed.weight"]
        x = x + (table[idx] * wts[:, :, None].to(table.dtype)).sum(0).to(x.dtype)
        pos = patch_positions(grid_thw, m, dev).float()                           # [n, 2]
        ang = (pos[:, :, None] * self.inv_freq[None, None, :]).flatten(1)         # [n, d / 2]: row angles, column angles
        ang = torch.cat((ang, ang), -1)[:, None, :]                               # [n, 1, d]
        cos, sin = ang.cos(), ang.sin()
        lengths = frame_lengths(grid_thw)
        deep = []
        for l in range(cfg.depth):
            p = f"blocks.{l}"
            x = x + self._attention(self._norm(x, p + ".norm1"), p, cos, sin, lengths)
            hmid = self._act(F.linear(self._norm(x, p + ".norm2"), self.w[p + ".mlp.linear_fc1.weight"],
                                      self.w[p + ".mlp.linear_fc1.bias"]))
            x = x + self._row(hmid, p + ".mlp.linear_fc2")
            if l in cfg.deepstack_visual_indexes:
                deep.append(self._merge(x, f"deepstack_merger_list.{cfg.deepstack_visual_indexes.index(l)}", True))
        self.encoded_patches += int(pixel_values.shape[0])
        return self._merge(x, "merger", False), deep

    # ------------------------------------------------------------------ fixed-shape form (CUDA-graph buckets)
    def fixed_inputs(self, grid_thw, capacity: int) -> dict[str, torch.Tensor]:
        """Everything of ``encode`` that depends on the grids, padded to ``capacity`` patches: table reads and weights,
        rotary cosines / sines, and the attention mask (a patch sees the patches of its own frame; a padding row sees
        itself, so no row of the softmax is empty)."""
        cfg, dev, m = self.cfg, self.device, self.cfg.spatial_merge_size
        lengths = frame_lengths(grid_thw)
        n = sum(lengths)
        if n > capacity or capacity % (m * m):
            raise ValueError("the bucket holds whole merge blocks and at least the patches given")
        idx = torch.zeros(4, capacity, dtype=torch.long, device=dev)
        wts = torch.zeros(4, capacity, dtype=torch.float32, device=dev)
        idx[:, :n], wts[:, :n] = bilinear_table_reads(grid_thw, cfg.side, m, dev)
        pos = torch.zeros(capacity, 2, dtype=torch.float32, device=dev)
        pos[:n] = patch_positions(grid_thw, m, dev).float()
        ang = (pos[:, :, None] * self.inv_freq[None, None, :]).flatten(1)
        ang = torch.cat((ang, ang), -1)[:, None, :]
        frame = torch.arange(capacity, device=dev) + len(lengths)                  # padding rows: one frame each
        frame[:n] = torch.repeat_interleave(torch.arange(len(lengths), device=dev),
                                            torch.tensor(lengths, device=dev))
        return {"idx": idx, "wts": wts, "cos": ang.cos(), "sin": ang.sin(), "mask": frame[:, None] == frame[None, :]}

    @torch.no_grad()
    def encode_fixed(self, pixel_values: torch.Tensor, fx: dict[str, torch.Tensor]) -> torch.Tensor:
        """``encode`` on a full bucket: the same arithmetic with the frames separated by the mask instead of by slicing,
        so every shape is fixed and the call can be captured in a CUDA graph.  Rows of real patches equal ``encode``'s;
        rows of padding are finite and ignored by the caller."""
        cfg = self.cfg
        d = cfg.head_dim
        x = F.linear(pixel_values.to(self.dtype), self.patch_w, self.w["patch_embed.proj.bias"])
        table = self.w["pos_embed.weight"]
        x = x + (table[fx["idx"]] * fx["wts"][:, :, None].to(table.dtype)).sum(0).to(x.dtype)
        cos, sin, mask = fx["cos"], fx["sin"], fx["mask"]
        n = x.shape[0]
        for l in range(cfg.depth):
            p = f"blocks.{l}"
            h = self._norm(x, p + ".norm1")
            qkv = F.linear(h, self.w[p + ".attn.qkv.weight"], self.w[p + ".attn.qkv.bias"]).view(n, 3, self.heads, d)
            q, k, v = qkv.unbind(1)

            def rot(t: torch.Tensor) -> torch.Tensor:
                tf = t.float()
                return (tf * cos + torch.cat((-tf[..., d // 2:], tf[..., :d // 2]), -1) * sin).to(t.dtype)
            o = F.scaled_dot_product_attention(rot(q).transpose(0, 1)[None], rot(k).transpose(0, 1)[None],
                                               v.transpose(0, 1)[None], attn_mask=mask)
            x = x + self._row(o[0].transpose(0, 1).reshape(n, self.heads * d), p + ".attn.proj")
            hmid = self._act(F.linear(self._norm(x, p + ".norm2"), self.w[p + ".mlp.linear_fc1.weight"],
                                      self.w[p + ".mlp.linear_fc1.bias"]))
            x = x + self._row(hmid, p + ".mlp.linear_fc2")
        return self._merge(x, "merger", False)

    def activation_bytes(self, patches: int) -> int:
        """Upper bound of the transient memory one ``encode`` of ``patches`` rows holds: the residual, the normalised
        copy, q / k / v and the attention output, the MLP's hidden features, in the tower's dtype; rotary tables in
        fp32."""
        c = self.cfg
        el = torch.empty((), dtype=self.dtype).element_size()
        per_row = (2 * c.hidden_size + 4 * c.hidden_size // self.tp_size + c.intermediate_size // self.tp_size) * el \
            + 2 * c.head_dim * 4 + c.patch_width * el
        return patches * per_row


def mrope_positions(token_ids, grids_of_spans: list[tuple[int, int, tuple[int, int, int]]], m: int) -> tuple[list, int]:
    """Three-axis positions of a prompt whose media spans are given as ``(first token, rows, (t, h, w))``.

    Text tokens advance all three axes together.  A row of an item sits at (frame, merged row, merged column) relative to the
    item's first position; the text behind the item continues one past the largest coordinate the item used.  Returns ``([t, h, w] lists over the prompt, delta)`` where a token generated at
    sequence index ``i`` has position ``i + delta`` on every axis."""
    n = len(token_ids)
    pos = [[0] * n for _ in range(3)]
    at, nxt = 0, 0
    for first, rows, (t, h, w) in sorted(grids_of_spans):
        if first < at or first + rows > n or rows != t * (h // m) * (w // m):
            raise ValueError("media spans overlap, leave the prompt or disagree with their grids")
        for i in range(at, first):
            pos[0][i] = pos[1][i] = pos[2][i] = nxt
            nxt += 1
        hh, ww = h // m, w // m
        for r in range(rows):
            f, rem = divmod(r, hh * ww)
            pos[0][first + r] = nxt + f
            pos[1][first + r] = nxt + rem // ww
            pos[2][first + r] = nxt + rem % ww
        at, nxt = first + rows, nxt + max(t, hh, ww)
    for i in range(at, n):
        pos[0][i] = pos[1][i] = pos[2][i] = nxt
        nxt += 1
    return pos, nxt - n
