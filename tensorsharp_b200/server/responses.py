"""Wire payloads of the three protocols, as ordered dicts, and their serialiser.

Parity: TensorSharp.Server/ResponseSerializers/OllamaResponseFactory.cs,
OpenAIResponseFactory.cs, WebUiSseEvents.cs, JsonOptions.cs and StreamingWriters/*.  Field
order is the reference's declaration order; ``serialize(..., ignore_nulls=True)`` drops null
members the way its ``IgnoreNulls`` options do; text is escaped like System.Text.Json's default
encoder (non-ASCII and ``< > & ' +`` as ``\\uXXXX``) so byte-level clients see the same stream.
"""
from __future__ import annotations

import time
import uuid
from typing import Any, Dict, Optional, Sequence

from ..runtime.chat import ToolCall, dotnet_json
from .sessions import _utcnow, iso_o


def _strip_nulls(o):
    if isinstance(o, dict):
        return {k: _strip_nulls(v) for k, v in o.items() if v is not None}
    if isinstance(o, (list, tuple)):
        return [_strip_nulls(v) for v in o]
    return o


def serialize(payload: Any, ignore_nulls: bool = False) -> str:
    return dotnet_json(_strip_nulls(payload) if ignore_nulls else payload)


def ndjson_line(payload: Any, ignore_nulls: bool = False) -> bytes:
    return (serialize(payload, ignore_nulls) + "\n").encode("utf-8")


def sse_event(payload: Any, ignore_nulls: bool = False) -> bytes:
    return ("data: " + serialize(payload, ignore_nulls) + "\n\n").encode("utf-8")


SSE_DONE = b"data: [DONE]\n\n"


def _now() -> str:
    return iso_o(_utcnow())


def _ratio(reused: int, total: int) -> float:
    return reused / total if total > 0 else 0.0


def _metrics(prompt_tokens, eval_tokens, reused, total_ns, prompt_ns, eval_ns) -> Dict[str, Any]:
    return {"total_duration": int(total_ns), "prompt_eval_count": prompt_tokens, "prompt_eval_duration": int(prompt_ns),
            "eval_count": eval_tokens, "eval_duration": int(eval_ns), "prompt_cache_hit_tokens": reused,
            "prompt_cache_hit_ratio": _ratio(reused, prompt_tokens)}


# ---------------------------------------------------------------------------- Ollama
class Ollama:
    @staticmethod
    def queue_generate_chunk(model, position, pending):
        return {"model": model, "created_at": _now(), "response": "", "done": False,
                "queue_position": position, "queue_pending": pending}

    @staticmethod
    def generate_token_chunk(model, piece):
        return {"model": model, "created_at": _now(), "response": piece, "done": False}

    @staticmethod
    def generate_final_chunk(model, *m):
        return {"model": model, "created_at": _now(), "response": "", "done": True, "done_reason": "stop", **_metrics(*m)}

    @staticmethod
    def generate_error(model, error):
        return {"model": model, "created_at": _now(), "response": "", "done": True, "done_reason": "error", "error": error}

    @staticmethod
    def generate_non_streaming(model, content, *m):
        return {"model": model, "created_at": _now(), "response": content, "done": True, "done_reason": "stop", **_metrics(*m)}

    @staticmethod
    def queue_chat_chunk(model, position, pending):
        return {"model": model, "created_at": _now(), "message": {"role": "assistant", "content": ""}, "done": False,
                "queue_position": position, "queue_pending": pending}

    @staticmethod
    def chat_raw_token_chunk(model, piece):
        return {"model": model, "created_at": _now(), "message": {"role": "assistant", "content": piece}, "done": False}

    @staticmethod
    def chat_parsed_chunk(model, content, thinking):
        return {"model": model, "created_at": _now(),
                "message": {"role": "assistant", "content": content, "thinking": thinking}, "done": False}

    @staticmethod
    def chat_raw_final_chunk(model, *m):
        return {"model": model, "created_at": _now(), "message": {"role": "assistant", "content": ""}, "done": True,
                "done_reason": "stop", **_metrics(*m)}

    @staticmethod
    def chat_parsed_final_chunk(model, tool_calls: Optional[Sequence[ToolCall]], *m):
        return {"model": model, "created_at": _now(),
                "message": {"role": "assistant", "content": "", "tool_calls": Ollama.convert_tool_calls(tool_calls)},
                "done": True, "done_reason": "tool_calls" if tool_calls is not None else "stop", **_metrics(*m)}

    @staticmethod
    def chat_error_chunk(model, error):
        return {"model": model, "created_at": _now(), "message": {"role": "assistant", "content": ""}, "done": True,
                "done_reason": "error", "error": error}

    @staticmethod
    def chat_non_streaming(model, message, done_reason, *m):
        return {"model": model, "created_at": _now(), "message": message, "done": True, "done_reason": done_reason,
                **_metrics(*m)}

    @staticmethod
    def chat_non_streaming_message(content, thinking, tool_calls):
        return {"role": "assistant", "content": content or "", "thinking": thinking,
                "tool_calls": Ollama.convert_tool_calls(tool_calls)}

    @staticmethod
    def chat_plain_message(content):
        return {"role": "assistant", "content": content}

    @staticmethod
    def convert_tool_calls(tool_calls):
        if not tool_calls:
            return None
        return [{"function": {"name": tc.name, "arguments": tc.arguments}} for tc in tool_calls]


# ---------------------------------------------------------------------------- OpenAI
CHUNK_OBJECT = "chat.completion.chunk"
COMPLETION_OBJECT = "chat.completion"


def _unix_now() -> int:
    return int(time.time())


class OpenAI:
    @staticmethod
    def new_request_id() -> str:
        return ("chatcmpl-" + uuid.uuid4().hex)[:30]

    @staticmethod
    def usage(prompt_tokens, eval_tokens, reused):
        return {"prompt_tokens": prompt_tokens, "completion_tokens": eval_tokens,
                "total_tokens": prompt_tokens + eval_tokens, "prompt_tokens_details": {"cached_tokens": reused}}

    @staticmethod
    def queue_chunk(rid, model, position, pending):
        return {"id": rid, "object": CHUNK_OBJECT, "model": model, "created": _unix_now(),
                "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}],
                "queue_position": position, "queue_pending": pending}

    @staticmethod
    def content_chunk(rid, model, content):
        return {"id": rid, "object": CHUNK_OBJECT, "created": _unix_now(), "model": model,
                "choices": [{"index": 0, "delta": {"role": None, "content": content}, "finish_reason": None}]}

    @staticmethod
    def structured_content_chunk(rid, model, content):
        return {"id": rid, "object": CHUNK_OBJECT, "created": _unix_now(), "model": model,
                "choices": [{"index": 0, "delta": {"role": "assistant", "content": content}, "finish_reason": None}]}

    @staticmethod
    def end_chunk(rid, model, finish_reason, prompt_tokens, eval_tokens, reused):
        return {"id": rid, "object": CHUNK_OBJECT, "created": _unix_now(), "model": model,
                "choices": [{"index": 0, "delta": {"role": None, "content": None}, "finish_reason": finish_reason}],
                "usage": OpenAI.usage(prompt_tokens, eval_tokens, reused)}

    @staticmethod
    def error_content_chunk(rid, model, message):
        return {"id": rid, "object": CHUNK_OBJECT, "model": model, "created": _unix_now(),
                "choices": [{"index": 0, "delta": {"content": f"Error: {message}"}, "finish_reason": "stop"}]}

    @staticmethod
    def completion(rid, model, message, finish_reason, prompt_tokens, eval_tokens, reused):
        return {"id": rid, "object": COMPLETION_OBJECT, "created": _unix_now(), "model": model,
                "choices": [{"index": 0, "message": message, "finish_reason": finish_reason}],
                "usage": OpenAI.usage(prompt_tokens, eval_tokens, reused)}

    @staticmethod
    def parsed_assistant_message(content, thinking, tool_calls):
        return {"role": "assistant", "content": content or "", "thinking": thinking,
                "tool_calls": OpenAI.build_tool_calls(tool_calls)}

    @staticmethod
    def plain_assistant_message(content):
        return {"role": "assistant", "content": content}

    structured_assistant_message = plain_assistant_message

    @staticmethod
    def build_tool_calls(tool_calls):
        if not tool_calls:
            return None
        return [{"id": ("call_" + uuid.uuid4().hex)[:24], "type": "function",
                 "function": {"name": tc.name, "arguments": dotnet_json(tc.arguments)}} for tc in tool_calls]

    @staticmethod
    def error(message, type_="invalid_request_error", details=None):
        e = {"message": message, "type": type_}
        if details is not None:
            e["details"] = details
        return {"error": e}


# ---------------------------------------------------------------------------- web UI
class WebUi:
    @staticmethod
    def queue_progress(position, pending):
        return {"queue_position": position, "queue_pending": pending}

    @staticmethod
    def token(token):
        return {"token": token}

    @staticmethod
    def thinking(thinking):
        return {"thinking": thinking}

    @staticmethod
    def tool_calls(tool_calls):
        return {"tool_calls": [{"name": tc.name, "arguments": tc.arguments} for tc in tool_calls]}

    @staticmethod
    def done(token_count, elapsed_s, tok_per_sec, aborted, error, session_id, prompt_tokens, reused):
        return {"done": True, "tokenCount": token_count, "elapsed": float(elapsed_s), "tokPerSec": float(tok_per_sec),
                "aborted": bool(aborted), "error": error, "sessionId": session_id, "promptTokens": prompt_tokens,
                "kvReusedTokens": reused,
                "kvReusePercent": 100.0 * reused / prompt_tokens if prompt_tokens > 0 else 0.0}
