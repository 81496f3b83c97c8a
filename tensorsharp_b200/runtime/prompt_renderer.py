"""Prompt renderers: the plain GGUF-template renderer and the KV-cache-aware renderer that
splices earlier assistant turns back in as the exact token ids the model generated.

Parity: TensorSharp.Runtime/PromptRenderer.cs:14-34 (GgufPromptRenderer) and
KVCachePromptRenderer.cs: placeholder ``\\uE000R{index:D4}\\uE000`` (:294-300),
architecture-specific generation suffix injected before each placeholder (:85-117),
whitespace before a placeholder trimmed when the renderer right-trims its output, token-span
replacement from the highest placeholder down (:139-240).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

from .chat import ChatMessage, ToolFunction
from .chat_template import QWEN35_FAMILY, render_from_gguf_template

PLACEHOLDER_SENTINEL = "\ue000"   # private-use character: never occurs in real text


class GgufPromptRenderer:
    def render(self, chat_template, messages, add_generation_prompt=True, architecture=None, tools=None,
               enable_thinking=False) -> str:
        return render_from_gguf_template(chat_template, messages, add_generation_prompt, architecture, tools,
                                         enable_thinking)


def assistant_generation_suffix(architecture: Optional[str], enable_thinking: bool) -> str:
    if not architecture:
        return ""
    if architecture == "gemma4" and not enable_thinking:
        return "<|channel>thought\n<channel|>"
    if architecture in QWEN35_FAMILY and enable_thinking:
        return "<think>\n"
    return ""


def make_placeholder(index: int) -> str:
    return f"{PLACEHOLDER_SENTINEL}R{index:04d}{PLACEHOLDER_SENTINEL}"


def _walk_placeholders(text: str, before) -> str:
    out, pos = [], 0
    while pos < len(text):
        s = text.find(PLACEHOLDER_SENTINEL, pos)
        if s < 0:
            out.append(text[pos:])
            break
        out.append(before(text[pos:s]))
        e = text.find(PLACEHOLDER_SENTINEL, s + 1)
        if e < 0:
            raise ValueError("Malformed KV-cache placeholder: opening sentinel without matching close.")
        out.append(text[s:e + 1])
        pos = e + 1
    return "".join(out)


def _find_subsequence(hay: Sequence[int], needle: Sequence[int]) -> int:
    n, m = len(hay), len(needle)
    if m == 0 or n < m:
        return -1
    for i in range(n - m + 1):
        if hay[i] == needle[0] and list(hay[i:i + m]) == list(needle):
            return i
    return -1


class KVCachePromptRenderer:
    def __init__(self, inner_renderer):
        if inner_renderer is None:
            raise ValueError("inner_renderer is required")
        self.inner = inner_renderer

    def render_to_tokens(self, tokenizer, chat_template, messages: List[ChatMessage], architecture,
                         add_generation_prompt: bool, tools: Optional[List[ToolFunction]] = None,
                         enable_thinking: bool = False) -> List[int]:
        if tokenizer is None or messages is None:
            raise ValueError("tokenizer and messages are required")
        rendered: Optional[List[ChatMessage]] = None
        raws: List[List[int]] = []
        for i, m in enumerate(messages):
            has_raw = m is not None and m.role == "assistant" and bool(m.raw_output_tokens)
            if not has_raw:
                if rendered is not None:
                    rendered.append(m)
                continue
            if rendered is None:
                rendered = list(messages[:i])
            rendered.append(ChatMessage(role=m.role, content=make_placeholder(len(raws)), thinking=None, tool_calls=None,
                                        image_paths=m.image_paths, audio_paths=m.audio_paths, is_video=m.is_video))
            raws.append(list(m.raw_output_tokens))
        text = self.inner.render(chat_template, rendered if rendered is not None else messages,
                                 add_generation_prompt=add_generation_prompt, architecture=architecture, tools=tools,
                                 enable_thinking=enable_thinking)
        if not raws:
            return tokenizer.encode(text, add_special=True)
        suffix = assistant_generation_suffix(architecture, enable_thinking)
        if suffix:
            text = _walk_placeholders(text, lambda seg: seg + suffix)
        if text and not text[-1].isspace():
            text = _walk_placeholders(text, lambda seg: seg.rstrip())
        tokens = list(tokenizer.encode(text, add_special=True))
        for i in range(len(raws) - 1, -1, -1):
            ph = tokenizer.encode(make_placeholder(i), add_special=False)
            at = _find_subsequence(tokens, ph)
            if at < 0:
                raise RuntimeError(f"Could not locate placeholder #{i} in the tokenized prompt: the tokenizer treats "
                                   "the placeholder differently in context than in isolation")
            tokens[at:at + len(ph)] = raws[i]
        return tokens
