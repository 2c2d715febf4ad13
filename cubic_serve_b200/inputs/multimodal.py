"""Chat requests with image / video parts -> prompt tokens, placeholder runs, feature rows and positions.

``MultimodalChatProcessor`` extends the text processor:

1. every media part is resolved (``inputs/media.py``: data / file / http under the deployment's policy), decoded and
   cut into patches (``inputs/vision_patches.py``); a video part may also carry already decoded frames in
   ``ContentPart.data`` (container decoding needs a codec library that this build does not ship: mp4 / webm urls are
   refused with a 400);
2. the prompt is rendered with ``<|vision_start|><|image_pad|><|vision_end|>`` (``<|video_pad|>`` for clips) where
   the part stood, tokenized, and each pad token is expanded into as many copies as the item has feature rows;
3. the vision service encodes the items (or finds them in its store) and the three-axis rotary positions of the
   expanded prompt are computed (``models/vision.py::mrope_positions``).

The result is a ``PreparedInput`` whose ``multimodal`` field (``runtime/multimodal.py::MultimodalInput``) the engine
takes with the token ids.

Reference counterpart: ``models/qwen3_5/multimodal.py:1148-1358`` (processor: decode, resize, patchify),
``:1360-1727`` (bridge: expand the prompt, positions, encode, cache keys).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np

from ..contracts.request import (CanonicalChatRequest, ContentPart, EncoderJob, InputPlan, MediaPlacement,
                                 RequestError)
from ..models.vision import mrope_positions
from ..runtime.multimodal import MultimodalInput
from .chat import ChatInputProcessor, PreparedInput
from .media import MediaError, MediaResolver
from .vision_patches import (MediaPatches, PatchGeometry, VisionInputError, decode_image, patchify_image,
                             patchify_video)


@dataclass(frozen=True)
class VisionTokens:
    """Token ids of the checkpoint's ``config.json`` (``image_token_id`` ...) and the strings the template emits."""
    image: int
    video: int
    start: int
    end: int
    image_text: str = "<|image_pad|>"
    video_text: str = "<|video_pad|>"
    start_text: str = "<|vision_start|>"
    end_text: str = "<|vision_end|>"

    @staticmethod
    def from_hf(cfg: dict) -> "VisionTokens":
        try:
            return VisionTokens(int(cfg["image_token_id"]), int(cfg["video_token_id"]),
                                int(cfg["vision_start_token_id"]), int(cfg["vision_end_token_id"]))
        except KeyError as e:
            raise ValueError(f"config.json lacks {e.args[0]!r}") from None


class MultimodalChatProcessor(ChatInputProcessor):
    def __init__(self, tokenizer, vision_service, tokens: VisionTokens, geometry: PatchGeometry | None = None,
                 resolver: MediaResolver | None = None, default_thinking: bool | None = None,
                 max_model_len: int | None = None, max_items: int = 16, video_max_frames: int = 768,
                 preprocess_workers: int = 2) -> None:
        super().__init__(tokenizer, default_thinking, max_model_len)
        self.vision, self.tokens = vision_service, tokens
        cfg = vision_service.encoder.cfg
        self.geometry = geometry or PatchGeometry(cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size)
        if (self.geometry.patch_size, self.geometry.merge_size, self.geometry.temporal_patch_size) != \
                (cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size):
            raise ValueError("the patch geometry differs from the vision tower's")
        self.resolver = resolver or MediaResolver()
        self.max_items = max_items
        self.video_max_frames = video_max_frames
        # media of one request are fetched, decoded and cut into patches concurrently (I/O, Pillow and the resize release
        # the interpreter lock)
        self._pool = None
        if preprocess_workers > 1:
            from concurrent.futures import ThreadPoolExecutor
            self._pool = ThreadPoolExecutor(max_workers=preprocess_workers, thread_name_prefix="media-prep")

    # ------------------------------------------------------------------ media parts -> patches
    def _patches(self, part: ContentPart) -> MediaPatches:
        try:
            if part.kind == "image":
                if part.data is not None:
                    return patchify_image(part.data, self.geometry)
                media = self.resolver.resolve(part.media_url, "image")
                return patchify_image(decode_image(media.data), self.geometry)
            if part.data is not None:
                return patchify_video(list(part.data), self.geometry, max_frames=self.video_max_frames)
            self.resolver.resolve(part.media_url, "video")          # policy and type checks still apply
            raise RequestError("video containers cannot be decoded by this deployment; send frames as images",
                               param="messages")
        except (MediaError, VisionInputError) as e:
            raise RequestError(str(e), param="messages") from None

    def plan(self, req: CanonicalChatRequest) -> InputPlan:
        """Everything except the encoding: media resolved, decoded and cut into patches, the prompt rendered and its
        placeholders expanded, positions computed, the encoder's capacity limits checked."""
        t = self.tokens
        media = [p for m in req.messages for p in m.parts if p.kind in ("image", "video")]
        if len(media) > self.max_items:
            raise RequestError(f"a request may carry {self.max_items} media items", param="messages")
        patches = iter(list(self._pool.map(self._patches, media)) if self._pool is not None and len(media) > 1
                       else [self._patches(p) for p in media])
        items: list[tuple[str, MediaPatches]] = []
        msgs = []
        for m in req.messages:
            parts = []
            for p in m.parts:
                if p.kind in ("image", "video"):
                    items.append((p.kind, next(patches)))
                    pad = t.image_text if p.kind == "image" else t.video_text
                    parts.append(ContentPart("text", t.start_text + pad + t.end_text))
                else:
                    parts.append(p)
            msgs.append(replace(m, parts=tuple(parts)))
        if not items:
            base = super().build(req)
            return InputPlan(tuple(base.token_ids), base.prompt_text, base.starts_in_reasoning)
        base = super().build(replace(req, messages=tuple(msgs)))
        merge = self.geometry.merge_size
        ids: list[int] = []
        spans_at: list[int] = []
        k = 0
        for tok in base.token_ids:                                    # expand every pad token into the item's rows
            if tok in (t.image, t.video):
                if k >= len(items) or (tok == t.image) != (items[k][0] == "image"):
                    raise RequestError("the rendered prompt's media placeholders do not match the media parts",
                                       param="messages")
                spans_at.append(len(ids))
                ids.extend([tok] * items[k][1].rows(merge))
                k += 1
            else:
                ids.append(tok)
        if k != len(items):
            raise RequestError("the chat template dropped a media part", param="messages")
        if self.max_model_len is not None and len(ids) + 1 > self.max_model_len:
            raise RequestError(f"the prompt has {len(ids)} tokens with its media; the context limit is "
                               f"{self.max_model_len}", param="messages")
        try:
            self.vision.plan.check_request([mp.grid for _, mp in items], merge)
        except ValueError as e:                                       # capacity limits of the encoder
            raise RequestError(str(e), param="messages") from None
        placements, jobs = [], []
        for at, (kind, mp) in zip(spans_at, items):
            d = self.vision.digest(mp.pixels, mp.grid)
            placements.append(MediaPlacement(kind, at, mp.rows(merge), tuple(mp.grid), d))
            jobs.append(EncoderJob(d, kind, tuple(mp.grid), mp.pixels))
        pos, delta = mrope_positions(ids, [(p.first_token, p.rows, p.grid) for p in placements], merge)
        return InputPlan(tuple(ids), base.prompt_text, base.starts_in_reasoning, np.asarray(pos, dtype=np.int32), delta,
                         tuple(placements), tuple(jobs))

    def assemble(self, plan: InputPlan, encoded: list) -> MultimodalInput | None:
        """The engine's view of a plan whose jobs were encoded (``encoded``: ``(rows, digest)`` per job, in order)."""
        if not plan.placements:
            return None
        spans = []
        for p, (rows, digest) in zip(plan.placements, encoded):
            if rows.shape[0] != p.rows or digest != p.digest:
                raise ValueError("the encoder's rows do not match the plan's placement")
            spans.append((p.first_token, rows, digest))
        cfg = self.vision.encoder.cfg
        return MultimodalInput(spans, plan.positions, plan.position_delta,
                               hidden=cfg.out_hidden_size if cfg.deepstack_visual_indexes else None)

    def encode(self, plan: InputPlan) -> list:
        return self.vision.encode([(j.patches, j.grid) for j in plan.jobs])

    def submit(self, plan: InputPlan):
        """Future of ``encode(plan)`` on the vision service's own thread."""
        return self.vision.submit([(j.patches, j.grid) for j in plan.jobs])

    def build(self, req: CanonicalChatRequest) -> PreparedInput:
        """``plan`` + encoding on the calling thread (library use; the serving backend encodes on the encoder thread)."""
        plan = self.plan(req)
        out = PreparedInput(list(plan.token_ids), plan.prompt_text, starts_in_reasoning=plan.starts_in_reasoning)
        if plan.jobs:
            try:
                out.multimodal = self.assemble(plan, self.encode(plan))
            except ValueError as e:
                raise RequestError(str(e), param="messages") from None
        return out
