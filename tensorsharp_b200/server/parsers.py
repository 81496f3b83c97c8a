"""Request-body parsers for the three protocols.

Parity: TensorSharp.Server/RequestParsers/SamplingConfigParser.cs (web UI accepts snake_case
and camelCase at the top level; Ollama reads ``options.*`` with ``repeat_penalty``; OpenAI
reads temperature / top_p / penalties / seed / stop-as-string-or-array), ToolFunctionParser.cs,
ChatMessageParser.cs (Ollama ``images`` and OpenAI ``image_url`` data URLs are written to the
upload directory as PNG files), OpenAIResponseFormatParser.cs.
"""
from __future__ import annotations

import base64
import json
import os
import uuid
from typing import Any, Dict, List, Optional, Tuple

from ..runtime.chat import ChatMessage, ToolFunction, ToolParameter
from ..runtime.sampling import SamplingConfig
from ..runtime.structured import StructuredOutputFormat


def _seed(defaults: Optional[SamplingConfig]) -> SamplingConfig:
    return defaults.clone() if defaults is not None else SamplingConfig()


def _strs(arr) -> List[str]:
    return [s for s in arr if isinstance(s, str)]


def parse_sampling_webui(body: Dict[str, Any], defaults: Optional[SamplingConfig] = None) -> SamplingConfig:
    cfg = _seed(defaults)
    for keys, attr, conv in ((("temperature",), "temperature", float), (("top_k", "topK"), "top_k", int),
                             (("top_p", "topP"), "top_p", float), (("min_p", "minP"), "min_p", float),
                             (("repetition_penalty", "repetitionPenalty"), "repetition_penalty", float),
                             (("presence_penalty", "presencePenalty"), "presence_penalty", float),
                             (("frequency_penalty", "frequencyPenalty"), "frequency_penalty", float),
                             (("seed",), "seed", int)):
        for k in keys:
            if k in body:
                setattr(cfg, attr, conv(body[k]))
    if isinstance(body.get("stop"), list):
        cfg.stop_sequences = _strs(body["stop"])
    return cfg


def parse_sampling_ollama(body: Dict[str, Any], defaults: Optional[SamplingConfig] = None) -> SamplingConfig:
    cfg = _seed(defaults)
    o = body.get("options")
    if isinstance(o, dict):
        for k, attr, conv in (("temperature", "temperature", float), ("top_k", "top_k", int), ("top_p", "top_p", float),
                              ("min_p", "min_p", float), ("repeat_penalty", "repetition_penalty", float),
                              ("presence_penalty", "presence_penalty", float),
                              ("frequency_penalty", "frequency_penalty", float), ("seed", "seed", int)):
            if k in o:
                setattr(cfg, attr, conv(o[k]))
        if isinstance(o.get("stop"), list):
            cfg.stop_sequences = _strs(o["stop"])
    return cfg


def parse_sampling_openai(body: Dict[str, Any], defaults: Optional[SamplingConfig] = None) -> SamplingConfig:
    cfg = _seed(defaults)
    for k, attr, conv in (("temperature", "temperature", float), ("top_p", "top_p", float),
                          ("presence_penalty", "presence_penalty", float),
                          ("frequency_penalty", "frequency_penalty", float), ("seed", "seed", int)):
        if k in body:
            setattr(cfg, attr, conv(body[k]))
    if "stop" in body:
        s = body["stop"]
        cfg.stop_sequences = _strs(s) if isinstance(s, list) else ([s] if isinstance(s, str) else [])
    return cfg


# ---------------------------------------------------------------------------- tools
def _parse_function(fn: Dict[str, Any]) -> ToolFunction:
    tf = ToolFunction(name=fn.get("name", ""), description=fn.get("description", ""))
    params = fn.get("parameters")
    if isinstance(params, dict):
        props = params.get("properties")
        if isinstance(props, dict):
            tf.parameters = {}
            for name, p in props.items():
                p = p if isinstance(p, dict) else {}
                tp = ToolParameter(type=p.get("type", "string"), description=p.get("description"))
                if isinstance(p.get("enum"), list):
                    tp.enum = [e if isinstance(e, str) else None for e in p["enum"]]
                tf.parameters[name] = tp
        if isinstance(params.get("required"), list):
            tf.required = [r if isinstance(r, str) else None for r in params["required"]]
    return tf


def parse_tools_ollama(body: Dict[str, Any]) -> Optional[List[ToolFunction]]:
    tools = body.get("tools")
    if not isinstance(tools, list):
        return None
    out = [_parse_function(t["function"]) for t in tools if isinstance(t, dict) and isinstance(t.get("function"), dict)]
    return out or None


def parse_tools_openai(body: Dict[str, Any]) -> Optional[List[ToolFunction]]:
    tools = body.get("tools")
    if not isinstance(tools, list):
        return None
    out = []
    for t in tools:
        if not isinstance(t, dict) or t.get("type", "function") != "function":
            continue
        if isinstance(t.get("function"), dict):
            out.append(_parse_function(t["function"]))
    return out or None


# ---------------------------------------------------------------------------- messages
def write_base64_image(b64: str, upload_dir: str) -> str:
    data = base64.b64decode(b64, validate=False)
    os.makedirs(upload_dir, exist_ok=True)
    path = os.path.join(upload_dir, f"{uuid.uuid4().hex}.png")
    with open(path, "wb") as f:
        f.write(data)
    return path


def parse_messages_webui(messages: List[Dict[str, Any]]) -> List[ChatMessage]:
    out = []
    for m in messages:
        msg = ChatMessage(role=m["role"], content=m["content"])
        for key, attr in (("imagePaths", "image_paths"), ("audioPaths", "audio_paths"), ("textFilePaths", "text_file_paths")):
            if isinstance(m.get(key), list) and m[key]:
                setattr(msg, attr, list(m[key]))
        if "isVideo" in m:
            msg.is_video = bool(m["isVideo"])
        out.append(msg)
    return out


def parse_messages_ollama(messages: List[Dict[str, Any]], upload_dir: str) -> List[ChatMessage]:
    out = []
    for m in messages:
        msg = ChatMessage(role=m.get("role", "user"), content=m.get("content", ""))
        if isinstance(m.get("images"), list):
            msg.image_paths = [write_base64_image(b, upload_dir) for b in m["images"] if isinstance(b, str) and b]
        out.append(msg)
    return out


def parse_messages_openai(messages: List[Dict[str, Any]], upload_dir: str) -> List[ChatMessage]:
    out = []
    for m in messages:
        msg = ChatMessage(role=m.get("role", "user"), content=None)
        c = m.get("content")
        if isinstance(c, str):
            msg.content = c
        elif isinstance(c, list):
            texts, images = [], []
            for part in c:
                if not isinstance(part, dict):
                    continue
                t = part.get("type", "")
                if t == "text" and "text" in part:
                    texts.append(part["text"] if part["text"] is not None else "")
                elif t == "image_url" and isinstance(part.get("image_url"), dict):
                    url = part["image_url"].get("url", "") or ""
                    if url.startswith("data:"):
                        comma = url.find(",")
                        if comma > 0:
                            images.append(write_base64_image(url[comma + 1:], upload_dir))
            msg.content = "\n".join(texts)
            msg.image_paths = images or None
        out.append(msg)
    return out


def decode_base64_images(body: Dict[str, Any], upload_dir: str) -> Optional[List[str]]:
    imgs = body.get("images")
    if not isinstance(imgs, list):
        return None
    out = [write_base64_image(b, upload_dir) for b in imgs if isinstance(b, str) and b]
    return out or None


# ---------------------------------------------------------------------------- response_format
def parse_response_format(body: Dict[str, Any]) -> Tuple[Optional[StructuredOutputFormat], Optional[str]]:
    """Returns ``(format or None, error or None)``."""
    rf = body.get("response_format")
    if rf is None:
        return None, None
    if not isinstance(rf, dict):
        return None, "response_format must be an object."
    t = rf.get("type")
    if not isinstance(t, str):
        return None, "response_format.type is required."
    if t == "text":
        return None, None
    if t == "json_object":
        return StructuredOutputFormat.json_object(), None
    if t != "json_schema":
        return None, f"Unsupported response_format.type '{t}'."
    wrap = rf
    if "json_schema" in rf:
        if not isinstance(rf["json_schema"], dict):
            return None, "response_format.json_schema must be an object."
        wrap = rf["json_schema"]
    name = wrap.get("name")
    if not isinstance(name, str) or not name.strip():
        return None, "response_format.json_schema.name is required."
    schema = wrap.get("schema")
    if not isinstance(schema, dict):
        return None, "response_format.json_schema.schema must be an object."
    strict = wrap.get("strict") is True
    desc = wrap.get("description") if isinstance(wrap.get("description"), str) else None
    return StructuredOutputFormat.json_schema(name, json.dumps(schema, ensure_ascii=False), strict, desc), None
