"""Streaming output parsers: split generated text into content, thinking and tool calls.

Observable behaviour follows TensorSharp.Runtime/OutputParser.cs: Qwen3 ``<think>`` /
``<tool_call>{json}</tool_call>`` (:75-333), Gemma 4 ``<|channel>thought ... <channel|>`` and
``<|tool_call>call:NAME{...}<tool_call|>`` with ``<|"|>`` string quotes (:348-582), Harmony
``<|start|>...<|channel|>X<|message|>...<|end|>`` framing with the ``analysis`` channel as
thinking (:590-758), passthrough, and the per-architecture factory (:782-801).  Text that
could be the beginning of a tag is held back until the next chunk decides.  In addition to
the reference, the Qwen parser also accepts the XML-style ``<function=NAME><parameter=K>``
body that the Qwen3.5 template instructs the model to emit.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .chat import ToolCall, ToolFunction


@dataclass
class ParsedOutput:
    content: str = ""
    thinking: str = ""
    tool_calls: Optional[List[ToolCall]] = None


def hold_back(buf: str, *tags: str) -> int:
    """Length of the longest suffix of ``buf`` that is a proper prefix of one of ``tags``."""
    best = 0
    for tag in tags:
        for n in range(min(len(tag), len(buf)), 0, -1):
            if buf.endswith(tag[:n]):
                best = max(best, n)
                break
    return best


class _StreamParser:
    has_thinking_support = False
    has_tool_support = False
    always_required = False

    def __init__(self):
        self.buf = ""

    def init(self, enable_thinking: bool, tools: Optional[List[ToolFunction]] = None) -> None:
        self.buf = ""

    def add(self, text: str, done: bool) -> ParsedOutput:
        raise NotImplementedError

    # split `self.buf` at a held-back boundary: emit the safe part, keep the possible tag prefix
    def _emit_safe(self, sink: List[str], *tags: str) -> None:
        h = hold_back(self.buf, *tags)
        if h:
            if len(self.buf) > h:
                sink.append(self.buf[:-h])
            self.buf = self.buf[-h:]
        else:
            sink.append(self.buf)
            self.buf = ""


class PassthroughOutputParser(_StreamParser):
    def add(self, text: str, done: bool) -> ParsedOutput:
        return ParsedOutput(content=text)


_FUNC_RE = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


class Qwen3OutputParser(_StreamParser):
    has_thinking_support = True
    has_tool_support = True

    THINKING, THINKING_DONE, CONTENT, TOOL = range(4)

    def init(self, enable_thinking: bool, tools=None) -> None:
        self.buf = ""
        self.call_index = 0
        self.state = self.THINKING if enable_thinking else self.CONTENT
        self.strip_open_tag = bool(enable_thinking)

    def _parse_tool(self, raw: str) -> Optional[ToolCall]:
        raw = raw.strip()
        if not raw:
            return None
        try:
            obj = json.loads(raw)
            name = obj.get("name") if isinstance(obj, dict) else None
            if not name:
                return None
            args = obj.get("arguments")
            tc = ToolCall(name=name, arguments=dict(args) if isinstance(args, dict) else {}, index=self.call_index)
        except (ValueError, AttributeError):
            m = _FUNC_RE.search(raw)
            if not m:
                return None
            args: Dict[str, Any] = {}
            for pm in _PARAM_RE.finditer(m.group(2)):
                v = pm.group(2)
                try:
                    args[pm.group(1)] = json.loads(v)
                except ValueError:
                    args[pm.group(1)] = v
            tc = ToolCall(name=m.group(1), arguments=args, index=self.call_index)
        self.call_index += 1
        return tc

    def add(self, text: str, done: bool) -> ParsedOutput:
        self.buf += text
        think: List[str] = []
        content: List[str] = []
        calls: List[ToolCall] = []
        again = True
        while again:
            again = False
            buf = self.buf
            if self.state == self.THINKING:
                if self.strip_open_tag:
                    t = buf.lstrip()
                    if t.startswith("<think>"):
                        self.buf = t[7:].lstrip()
                        self.strip_open_tag = False
                        again = bool(self.buf)
                        continue
                    if "<think>".startswith(t) and not done:
                        break
                    self.strip_open_tag = False
                close, tool = buf.find("</think>"), buf.find("<tool_call>")
                if tool >= 0 and (close < 0 or tool < close):
                    before = buf[:tool].rstrip()
                    self.buf = buf[tool + 11:].lstrip()
                    if before:
                        think.append(before)
                    self.state = self.TOOL
                    again = True
                elif close >= 0:
                    th = buf[:close].rstrip()
                    self.buf = buf[close + 8:].lstrip()
                    if th:
                        think.append(th)
                    self.state = self.CONTENT if self.buf else self.THINKING_DONE
                    again = bool(self.buf)
                elif done:
                    if buf:
                        think.append(buf)
                    self.buf = ""
                else:
                    self._emit_safe(think, "</think>", "<tool_call>")
            elif self.state == self.THINKING_DONE:
                self.buf = buf.lstrip()
                if self.buf:
                    self.state = self.CONTENT
                    again = True
            elif self.state == self.CONTENT:
                tool = buf.find("<tool_call>")
                if tool >= 0:
                    before = buf[:tool].rstrip()
                    self.buf = buf[tool + 11:].lstrip()
                    if before:
                        content.append(before)
                    self.state = self.TOOL
                    again = True
                elif done:
                    if buf:
                        content.append(buf)
                    self.buf = ""
                else:
                    self._emit_safe(content, "<tool_call>")
            else:  # TOOL
                end = buf.find("</tool_call>")
                if end >= 0:
                    tc = self._parse_tool(buf[:end])
                    self.buf = buf[end + 12:].lstrip()
                    if tc:
                        calls.append(tc)
                    self.state = self.CONTENT
                    again = bool(self.buf)
                elif done and buf:
                    tc = self._parse_tool(buf)
                    if tc:
                        calls.append(tc)
                    self.buf = ""
                    self.state = self.CONTENT
        return ParsedOutput("".join(content), "".join(think), calls or None)


class Qwen35OutputParser(Qwen3OutputParser):
    pass


_G4_QUOTED = re.compile(r'<\|"\|>(.*?)<\|"\|>', re.S)
_G4_BARE_KEY = re.compile(r"([,{])(\w+):")


def gemma4_args_to_json(s: str) -> str:
    """``{city:<|"|>Paris<|"|>,n:3}`` -> ``{"city":"Paris","n":3}``."""
    strings: List[str] = []

    def stash(m):
        strings.append(m.group(1))
        return f"\x00{len(strings) - 1}\x00"
    text = _G4_QUOTED.sub(stash, s)
    text = _G4_BARE_KEY.sub(r'\1"\2":', text)
    for i, val in enumerate(strings):
        text = text.replace(f"\x00{i}\x00", json.dumps(val))
    return text


class Gemma4OutputParser(_StreamParser):
    has_thinking_support = True
    has_tool_support = True
    always_required = True

    CONTENT, THINKING, TOOL = range(3)

    def init(self, enable_thinking: bool, tools=None) -> None:
        self.buf = ""
        self.thinking_enabled = bool(enable_thinking)
        self.strip_channel_name = False
        self.state = self.CONTENT

    @staticmethod
    def _parse_tool(raw: str) -> Optional[ToolCall]:
        raw = raw.strip()
        if not raw.startswith("call:"):
            return None
        raw = raw[5:]
        brace = raw.find("{")
        if brace < 0:
            return None
        try:
            args = json.loads(gemma4_args_to_json(raw[brace:]))
        except ValueError:
            return None
        if not isinstance(args, dict):
            return None
        return ToolCall(name=raw[:brace].strip(), arguments=args)

    def add(self, text: str, done: bool) -> ParsedOutput:
        self.buf += text
        think: List[str] = []
        content: List[str] = []
        calls: List[ToolCall] = []
        again = True
        while again:
            again = False
            buf = self.buf
            if not buf:
                break
            if self.state == self.CONTENT:
                ch, tc = buf.find("<|channel>"), buf.find("<|tool_call>")
                if ch >= 0 and (tc < 0 or ch < tc):
                    before = buf[:ch].rstrip()
                    self.buf = buf[ch + 10:]
                    if before:
                        content.append(before)
                    self.state, self.strip_channel_name, again = self.THINKING, True, True
                elif tc >= 0:
                    before = buf[:tc].rstrip()
                    self.buf = buf[tc + 12:]
                    if before:
                        content.append(before)
                    self.state, again = self.TOOL, True
                elif not done:
                    self._emit_safe(content, "<|channel>", "<|tool_call>")
                else:
                    content.append(buf)
                    self.buf = ""
            elif self.state == self.THINKING:
                if self.strip_channel_name:
                    if buf.startswith("thought\n"):
                        self.buf = buf[8:]
                        self.strip_channel_name = False
                        again = bool(self.buf)
                        continue
                    if not done and ("thought\n".startswith(buf) or buf.startswith("thought")):
                        break
                    self.strip_channel_name = False
                close = buf.find("<channel|>")
                sink = think if self.thinking_enabled else []
                if close >= 0:
                    th = buf[:close].rstrip()
                    self.buf = buf[close + 10:].lstrip()
                    if th:
                        sink.append(th)
                    self.state = self.CONTENT
                    again = bool(self.buf)
                elif not done:
                    self._emit_safe(sink, "<channel|>")
                else:
                    sink.append(buf)
                    self.buf = ""
            else:
                end = buf.find("<tool_call|>")
                if end >= 0:
                    tc_ = self._parse_tool(buf[:end])
                    self.buf = buf[end + 12:].lstrip()
                    if tc_:
                        calls.append(tc_)
                    self.state = self.CONTENT
                    again = bool(self.buf)
                elif done and buf:
                    tc_ = self._parse_tool(buf)
                    if tc_:
                        calls.append(tc_)
                    self.buf = ""
                    self.state = self.CONTENT
        return ParsedOutput("".join(content), "".join(think), calls or None)


class HarmonyOutputParser(_StreamParser):
    has_thinking_support = True
    has_tool_support = False
    always_required = True

    START, HEADER, BODY = range(3)
    T_START, T_END, T_MSG, T_CHANNEL = "<|start|>", "<|end|>", "<|message|>", "<|channel|>"

    def init(self, enable_thinking: bool, tools=None) -> None:
        # generation continues the "<|start|>assistant" the prompt ended with
        self.buf = "<|start|>assistant"
        self.thinking_enabled = bool(enable_thinking)
        self.state = self.START
        self.channel: Optional[str] = None

    def add(self, text: str, done: bool) -> ParsedOutput:
        self.buf += text
        think: List[str] = []
        content: List[str] = []
        again = True
        while again:
            again = False
            buf = self.buf
            if not buf:
                break
            if self.state == self.START:
                i = buf.find(self.T_START)
                if i >= 0:
                    self.buf = buf[i + len(self.T_START):]
                    self.state, again = self.HEADER, True
                elif not done:
                    h = hold_back(buf, self.T_START)
                    if h:
                        self.buf = buf[-h:]
            elif self.state == self.HEADER:
                i = buf.find(self.T_MSG)
                if i >= 0:
                    header = buf[:i]
                    self.buf = buf[i + len(self.T_MSG):]
                    c = header.find(self.T_CHANNEL)
                    if c >= 0:
                        part = header[c + len(self.T_CHANNEL):]
                        m = re.search(r"[ \t\n\r]", part)
                        self.channel = part[:m.start()] if m else part
                    else:
                        self.channel = "final"
                    self.state = self.BODY
                    again = bool(self.buf)
                # else: keep the partial header whole until "<|message|>" arrives (the reference
                # trims it to the held-back tag prefix, which loses the channel name when the
                # tag itself is split across pieces)
            else:
                sink = think if self.channel == "analysis" else content
                i = buf.find(self.T_END)
                if i >= 0:
                    if buf[:i]:
                        sink.append(buf[:i])
                    self.buf = buf[i + len(self.T_END):]
                    self.state = self.START
                    again = bool(self.buf)
                elif not done:
                    self._emit_safe(sink, self.T_END, self.T_START)
                else:
                    sink.append(buf)
                    self.buf = ""
        return ParsedOutput("".join(content), "".join(think), None)


_QWEN35 = ("qwen35", "qwen35moe", "qwen3next", "qwen3vl", "qwen3vlmoe")


def create_output_parser(architecture: Optional[str]) -> _StreamParser:
    a = architecture or ""
    if a == "gemma4":
        return Gemma4OutputParser()
    if a == "qwen3":
        return Qwen3OutputParser()
    if a in _QWEN35:
        return Qwen35OutputParser()
    if a in ("gptoss", "gpt-oss"):
        return HarmonyOutputParser()
    if a in ("nemotron_h", "nemotron_h_moe"):
        return Qwen3OutputParser()
    return PassthroughOutputParser()


def is_always_required(architecture: Optional[str]) -> bool:
    return architecture in ("gptoss", "gpt-oss", "gemma4")
