"""Chat input processing: messages + tools -> prompt token ids.

Counterpart of the reference's ``ChatInputProcessor`` (``inputs/chat.py:390``).  A HuggingFace tokenizer's own
chat template is used when it has one; otherwise a ChatML template (the Qwen family's format, including the
Hermes-style ``<tool_call>`` convention and ``<think>`` reasoning blocks) is rendered here.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..contracts.request import CanonicalChatRequest, Message, RequestError, Role


class ByteTokenizer:
    """Self-contained byte-level tokenizer (ids 0..255 = bytes, then specials) for tests and toy models."""

    SPECIALS = ("<|im_start|>", "<|im_end|>", "<|endoftext|>")

    def __init__(self) -> None:
        self.special_ids = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.eos_token_id = self.special_ids["<|im_end|>"]
        self.vocab_size = 256 + len(self.SPECIALS)
        self.chat_template = None

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        out: list[int] = []
        i = 0
        while i < len(text):
            for s, sid in self.special_ids.items():
                if text.startswith(s, i):
                    out.append(sid)
                    i += len(s)
                    break
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        rev = {v: k for k, v in self.special_ids.items()}
        buf = bytearray()
        parts: list[str] = []
        for t in ids:
            if t < 256:
                buf.append(t)
            else:
                if buf:
                    parts.append(buf.decode("utf-8", errors="replace"))
                    buf = bytearray()
                if not skip_special_tokens and t in rev:
                    parts.append(rev[t])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)


def render_chatml(req: CanonicalChatRequest, enable_thinking: bool | None) -> str:
    out: list[str] = []
    msgs = list(req.messages)
    system = ""
    if msgs and msgs[0].role is Role.SYSTEM:
        system = msgs.pop(0).text
    if req.tools and req.tool_choice.mode != "none":
        tools = "\n".join(json.dumps({"type": "function", "function": {
            "name": t.name, "description": t.description, "parameters": t.parameters or {"type": "object", "properties": {}}}},
            ensure_ascii=False) for t in req.tools)
        system = (system + "\n\n" if system else "") + (
            "# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
            "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n" + tools +
            "\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
            "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call>")
    if system:
        out.append(f"<|im_start|>system\n{system}<|im_end|>\n")
    for m in msgs:
        if m.role is Role.TOOL:
            out.append(f"<|im_start|>user\n<tool_response>\n{m.text}\n</tool_response><|im_end|>\n")
            continue
        body = m.text
        if m.role is Role.ASSISTANT and m.tool_calls:
            calls = "\n".join("<tool_call>\n" + json.dumps({"name": c.name, "arguments": json.loads(c.arguments or "{}")},
                                                              ensure_ascii=False) + "\n</tool_call>" for c in m.tool_calls)
            body = (body + "\n" if body else "") + calls
        out.append(f"<|im_start|>{m.role.value}\n{body}<|im_end|>\n")
    out.append("<|im_start|>assistant\n")
    if enable_thinking is False:
        out.append("<think>\n\n</think>\n\n")
    return "".join(out)


@dataclass
class PreparedInput:
    token_ids: list[int]
    prompt_text: str
    starts_in_reasoning: bool = False
    multimodal: object = None        # ``runtime.multimodal.MultimodalInput`` when the prompt carries media


class ChatInputProcessor:
    def __init__(self, tokenizer, default_thinking: bool | None = None, max_model_len: int | None = None) -> None:
        self.tokenizer = tokenizer
        self.default_thinking = default_thinking
        self.max_model_len = max_model_len

    def build(self, req: CanonicalChatRequest) -> PreparedInput:
        for m in req.messages:
            if any(p.kind in ("image", "video") for p in m.parts):
                raise RequestError("this deployment serves text only; image and video parts are not accepted",
                                   param="messages")
        thinking = req.reasoning.enabled if req.reasoning.enabled is not None else self.default_thinking
        template = getattr(self.tokenizer, "chat_template", None)
        if template and hasattr(self.tokenizer, "apply_chat_template"):
            msgs = [self._hf_message(m) for m in req.messages]
            tools = [{"type": "function", "function": {"name": t.name, "description": t.description,
                                                        "parameters": t.parameters or {}}} for t in req.tools] or None
            kwargs = dict(req.template_kwargs)
            if thinking is not None:
                kwargs.setdefault("enable_thinking", thinking)
            text = self.tokenizer.apply_chat_template(msgs, tools=tools, tokenize=False, add_generation_prompt=True, **kwargs)
        else:
            text = render_chatml(req, thinking)
        ids = list(self.tokenizer.encode(text, add_special_tokens=False))
        if self.max_model_len is not None and len(ids) + 1 > self.max_model_len:
            raise RequestError(f"the prompt has {len(ids)} tokens; the context limit is {self.max_model_len}",
                               param="messages")
        return PreparedInput(ids, text, starts_in_reasoning=text.rstrip().endswith("<think>"))

    @staticmethod
    def _hf_message(m: Message) -> dict:
        d: dict = {"role": m.role.value, "content": m.text}
        if m.tool_calls:
            d["tool_calls"] = [{"id": c.id, "type": "function",
                                "function": {"name": c.name, "arguments": json.loads(c.arguments or "{}")}} for c in m.tool_calls]
        if m.tool_call_id:
            d["tool_call_id"] = m.tool_call_id
        return d
