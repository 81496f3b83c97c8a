"""Chat data types shared by templates, parsers, the CLI and the server.

Parity: TensorSharp.Runtime/ChatTemplate.cs:18-62 (ChatMessage), OutputParser.cs:22-51
(ToolFunction, ToolParameter, ToolCall).  ``dotnet_json`` reproduces System.Text.Json's
default output (compact separators, its escaping of ``" & ' + < > ` `` and of non-ASCII
characters as ``\\uXXXX``), which the hardcoded templates embed into prompts, so prompt text
and therefore token ids match the reference byte for byte.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional


@dataclass
class ToolParameter:
    type: Optional[str] = None
    description: Optional[str] = None
    enum: Optional[List[str]] = None


@dataclass
class ToolFunction:
    name: str = ""
    description: Optional[str] = None
    parameters: Optional[Dict[str, ToolParameter]] = None
    required: Optional[List[str]] = None

    def to_dotnet(self) -> Dict[str, Any]:
        params = None
        if self.parameters is not None:
            params = {k: {"Type": p.type, "Description": p.description, "Enum": p.enum}
                      for k, p in self.parameters.items()}
        return {"Name": self.name, "Description": self.description, "Parameters": params, "Required": self.required}


@dataclass
class ToolCall:
    name: str = ""
    arguments: Optional[Dict[str, Any]] = None
    index: int = 0

    def __str__(self) -> str:
        return f"{self.name}({dotnet_json(self.arguments) if self.arguments is not None else '{}'})"


@dataclass
class ChatMessage:
    role: str = "user"
    content: Optional[str] = None
    image_paths: Optional[List[str]] = None
    audio_paths: Optional[List[str]] = None
    text_file_paths: Optional[List[str]] = None
    is_video: bool = False
    tool_calls: Optional[List[ToolCall]] = None
    thinking: Optional[str] = None
    raw_output_tokens: Optional[List[int]] = None


_ESC = {'"': "\\u0022", "&": "\\u0026", "'": "\\u0027", "+": "\\u002B", "<": "\\u003C", ">": "\\u003E",
        "`": "\\u0060", "\\": "\\\\", "\n": "\\n", "\r": "\\r", "\t": "\\t", "\b": "\\b", "\f": "\\f"}


def _esc_str(s: str) -> str:
    out = []
    for ch in s:
        e = _ESC.get(ch)
        if e is not None:
            out.append(e)
        elif ord(ch) < 0x20 or ord(ch) > 0x7E:
            cp = ord(ch)
            if cp > 0xFFFF:
                cp -= 0x10000
                out.append("\\u%04X\\u%04X" % (0xD800 + (cp >> 10), 0xDC00 + (cp & 0x3FF)))
            else:
                out.append("\\u%04X" % cp)
        else:
            out.append(ch)
    return '"' + "".join(out) + '"'


def _fmt_num(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if v != v or v in (float("inf"), float("-inf")):
        raise ValueError("NaN / infinity are not valid JSON numbers")
    if v == int(v) and abs(v) < 1e15:
        return str(int(v))
    return repr(float(v))


def dotnet_json(obj: Any, indented: bool = False, _level: int = 0) -> str:
    """Serialise like ``System.Text.Json.JsonSerializer.Serialize`` with default options."""
    if obj is None:
        return "null"
    if isinstance(obj, bool) or isinstance(obj, (int, float)):
        return _fmt_num(obj)
    if isinstance(obj, str):
        return _esc_str(obj)
    if hasattr(obj, "to_dotnet"):
        return dotnet_json(obj.to_dotnet(), indented, _level)
    nl = "\n" + "  " * (_level + 1) if indented else ""
    end = "\n" + "  " * _level if indented else ""
    if isinstance(obj, dict):
        if not obj:
            return "{}"
        sep = ": " if indented else ":"
        items = [f"{nl}{_esc_str(str(k))}{sep}{dotnet_json(v, indented, _level + 1)}" for k, v in obj.items()]
        return "{" + ",".join(items) + end + "}"
    if isinstance(obj, (list, tuple)):
        if not obj:
            return "[]"
        items = [f"{nl}{dotnet_json(v, indented, _level + 1)}" for v in obj]
        return "[" + ",".join(items) + end + "]"
    return _esc_str(str(obj))
