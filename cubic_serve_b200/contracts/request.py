"""Canonical request, plan and event types shared by both wire protocols.

Protocol-neutral core of the API layer, matching the reference's frozen
contracts (``contracts/request.py:668`` ``CanonicalChatRequest``, ``:599``
``SamplingMeta``, ``:989`` ``TokenEvent``): the HTTP layer normalises OpenAI and
Anthropic bodies into ``CanonicalChatRequest``; the backend answers with a
stream of ``TokenEvent``; the projections fold those back into wire objects.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any


class Role(str, enum.Enum):
    SYSTEM = "system"
    USER = "user"
    ASSISTANT = "assistant"
    TOOL = "tool"


class StructuredKind(str, enum.Enum):
    NONE = "none"
    JSON_OBJECT = "json_object"
    JSON_SCHEMA = "json_schema"
    REGEX = "regex"
    CHOICE = "choice"
    GRAMMAR = "grammar"
    STRUCTURAL_TAG = "structural_tag"
    TOOL_SCHEMA = "tool_schema"


@dataclass(frozen=True)
class ContentPart:
    kind: str                 # text | image | video | tool_use | tool_result
    text: str = ""
    media_url: str | None = None
    data: Any = None


@dataclass(frozen=True)
class ToolCall:
    id: str
    name: str
    arguments: str            # JSON text


@dataclass(frozen=True)
class Message:
    role: Role
    parts: tuple[ContentPart, ...]
    tool_calls: tuple[ToolCall, ...] = ()
    tool_call_id: str | None = None
    name: str | None = None

    @property
    def text(self) -> str:
        return "".join(p.text for p in self.parts if p.kind == "text")


@dataclass(frozen=True)
class ToolSpec:
    name: str
    description: str = ""
    parameters: dict | None = None
    strict: bool = False


@dataclass(frozen=True)
class ToolChoice:
    mode: str = "auto"        # auto | none | required | named
    name: str | None = None


@dataclass(frozen=True)
class StructuredOutput:
    kind: StructuredKind = StructuredKind.NONE
    schema: Any = None        # JSON schema / regex / choices / grammar text
    name: str | None = None
    strict: bool = False


@dataclass(frozen=True)
class SamplingMeta:
    """Sampling controls; ranges follow the reference (T in [0, 2], top_k <= 20)."""
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int | None = None
    max_tokens: int | None = None
    stop: tuple[str, ...] = ()
    stop_token_ids: tuple[int, ...] = ()
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logprobs: bool = False
    top_logprobs: int = 0

    def __post_init__(self) -> None:
        if not 0.0 <= self.temperature <= 2.0:
            raise RequestError("temperature must be between 0 and 2", param="temperature")
        if not 0.0 < self.top_p <= 1.0:
            raise RequestError("top_p must be in (0, 1]", param="top_p")
        if not 0 <= self.top_k <= 20:
            raise RequestError("top_k must be between 0 and 20", param="top_k")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise RequestError("max_tokens must be at least 1", param="max_tokens")


@dataclass(frozen=True)
class ReasoningControl:
    enabled: bool | None = None       # None = model default
    budget_tokens: int | None = None
    effort: str | None = None


@dataclass(frozen=True)
class CanonicalChatRequest:
    protocol: str                      # openai | anthropic
    model: str
    messages: tuple[Message, ...]
    sampling: SamplingMeta = field(default_factory=SamplingMeta)
    stream: bool = False
    include_usage: bool = False
    tools: tuple[ToolSpec, ...] = ()
    tool_choice: ToolChoice = field(default_factory=ToolChoice)
    structured: StructuredOutput = field(default_factory=StructuredOutput)
    reasoning: ReasoningControl = field(default_factory=ReasoningControl)
    n: int = 1
    user: str | None = None
    request_id: str = ""
    template_kwargs: tuple[tuple[str, Any], ...] = ()


@dataclass(frozen=True)
class MediaPlacement:
    """Where a media item sits in the expanded prompt: ``rows`` placeholder tokens from ``first_token`` on are replaced
    by the item's encoder features; ``grid`` = (t, h, w) in patches; ``digest`` identifies the content."""
    kind: str                  # image | video
    first_token: int
    rows: int
    grid: tuple[int, int, int]
    digest: bytes = field(repr=False, default=b"")


@dataclass(frozen=True)
class EncoderJob:
    """One item for the vision tower: ``patches`` is a float32 array [t h w, patch width] in merge-block order."""
    digest: bytes = field(repr=False)
    kind: str = "image"
    grid: tuple[int, int, int] = (1, 0, 0)
    patches: Any = field(repr=False, default=None)


@dataclass(frozen=True)
class InputPlan:
    """A prepared prompt before its media are encoded: token ids with placeholder runs, rotary positions on the three
    axes (None for text-only prompts: the sequence index), media placements in prompt order and the encoder jobs
    that will produce their feature rows (one per placement, same order)."""
    token_ids: tuple[int, ...]
    prompt_text: str = ""
    starts_in_reasoning: bool = False
    positions: Any = None                       # int [3, len(token_ids)] or None
    position_delta: int = 0                     # position of a generated token = its sequence index + delta
    placements: tuple[MediaPlacement, ...] = ()
    jobs: tuple[EncoderJob, ...] = field(default=(), repr=False)

    def __post_init__(self) -> None:
        if len(self.placements) != len(self.jobs):
            raise ValueError("one encoder job per media placement")
        at = 0
        for p in self.placements:
            t, h, w = p.grid
            if p.first_token < at or p.rows <= 0 or p.first_token + p.rows > len(self.token_ids) or min(t, h, w) <= 0:
                raise ValueError("media placements are ordered, disjoint and inside the prompt")
            at = p.first_token + p.rows
        if self.placements and self.positions is None:
            raise ValueError("a prompt with media carries its positions")


class EventKind(str, enum.Enum):
    START = "start"
    REASONING = "reasoning"
    CONTENT = "content"
    TOOL_CALL_START = "tool_call_start"
    TOOL_CALL_ARGS = "tool_call_args"
    FINISH = "finish"


@dataclass(frozen=True)
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0
    reasoning_tokens: int = 0


@dataclass(frozen=True)
class TokenEvent:
    kind: EventKind
    text: str = ""
    tool_index: int = 0
    tool_id: str = ""
    tool_name: str = ""
    finish_reason: str | None = None   # stop | length | tool_calls | content_filter | abort
    usage: Usage | None = None
    token_count: int = 0


class RequestError(ValueError):
    """A client error with a reviewed public message (HTTP 400 family)."""

    def __init__(self, message: str, *, param: str | None = None, status: int = 400,
                 code: str = "invalid_request_error") -> None:
        super().__init__(message)
        self.public_message = message
        self.param = param
        self.status = status
        self.code = code
