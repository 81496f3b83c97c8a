"""HTTP front end: routes, protocol adapters, request logging, static web UI.

Parity: TensorSharp.Server/Program.cs and Endpoints/* (the fifteen routes below),
ProtocolAdapters/OllamaAdapter.cs, OpenAIChatAdapter.cs, WebUiAdapter.cs,
Logging/RequestLoggingMiddleware.cs (``X-TensorSharp-Request-Id`` echo / 12-hex-digit id, client
label by path, 4xx -> Warning, 5xx -> Error), WebUiChatPolicy.cs, TextUploadHelper.cs.

    GET  /                      GET  /api/version         GET  /api/tags
    POST /api/show              POST /api/generate        POST /api/chat/ollama
    POST /v1/chat/completions   GET  /v1/models           POST /api/sessions
    DELETE /api/sessions/{id}   POST /api/upload          GET  /api/queue/status
    GET  /api/models            POST /api/models/load     POST /api/chat
    GET  /metrics  (totals in the Prometheus text format; not in the reference)
    (anything else: the web UI's index.html)

Built on the standard library's threading HTTP server: one thread per connection, responses
streamed with chunked transfer encoding.  Inference itself is serialised by ``InferenceQueue``;
waiting clients get their queue position once a second in their protocol's framing.
"""
from __future__ import annotations

import email
import email.policy
import json
import os
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Callable, Dict, List, Optional, Tuple
from urllib.parse import unquote, urlsplit

from ..runtime import media
from ..runtime.logging import Ev, FileLoggerProvider, Logger, NULL_LOGGER, log_scope
from ..runtime.output_parser import create_output_parser, is_always_required
from ..runtime.structured import apply_to_messages, normalize_output, validate_schema
from . import parsers as P
from .inference_queue import CancellationToken, InferenceQueue
from .model_service import ModelService
from .metrics import METRICS
from .options import (ServerHostingOptions, try_ensure_hosted_model_loaded, try_resolve_hosted_model_request,
                      try_resolve_supported_backend, try_validate_hosted_mmproj_request)
from .responses import SSE_DONE, Ollama, OpenAI, WebUi, ndjson_line, serialize, sse_event
from .sessions import DEFAULT_SESSION_ID, SessionManager, iso_o

REQUEST_ID_HEADER = "X-TensorSharp-Request-Id"
MODEL_SELECTION_LOCKED = ("Use /api/models/load to choose a model before chatting. Changing models during chat is "
                          "not supported.")
VERSION = "0.1.0"

_EXT_KIND = {}
for _k, _exts in (("image", "png jpg jpeg gif webp bmp heic heif"), ("video", "mp4 mov avi mkv webm"),
                  ("audio", "mp3 wav ogg flac m4a"),
                  ("text", "txt csv json xml md log py js ts cs java cpp c h html css yaml yml toml ini cfg sh bat ps1 rb "
                           "go rs swift kt sql r m tex rtf")):
    for _e in _exts.split():
        _EXT_KIND["." + _e] = _k


def classify_extension(ext: str) -> str:
    return _EXT_KIND.get(ext.lower(), "unknown")


def classify_client(path: str) -> Optional[str]:
    p = (path or "").lower()
    if p.startswith("/v1/"):
        return "openai"
    if p == "/api/chat/ollama" or p.startswith(("/api/generate", "/api/show", "/api/tags", "/api/version")):
        return "ollama"
    if p.startswith("/api/"):
        return "webui"
    return None


def validate_webui_chat_request(model: Optional[str], backend: Optional[str]) -> Optional[str]:
    if not (model and model.strip()) and not (backend and backend.strip()):
        return None
    return MODEL_SELECTION_LOCKED


def prepare_text_content(text: Optional[str], tokenizer, model_context_limit: int, fallback_char_limit: int) -> Dict[str, Any]:
    """Clip an uploaded text file to half the context (in tokens) or, with no model loaded, to
    a character limit."""
    if tokenizer is not None and model_context_limit > 0:
        limit = max(1, model_context_limit // 2)
        toks = tokenizer.encode(text or "", add_special=False)
        truncated = len(toks) > limit
        if truncated:
            text = tokenizer.decode(toks[:limit])
        returned = tokenizer.encode(text or "", add_special=False)
        return {"textContent": text, "truncated": truncated, "truncateLimit": limit, "truncateUnit": "tokens",
                "modelContextLimit": model_context_limit, "originalTokenCount": len(toks), "returnedTokenCount": len(returned)}
    safe = text or ""
    truncated = len(safe) > fallback_char_limit
    return {"textContent": safe[:fallback_char_limit] if truncated else safe, "truncated": truncated,
            "truncateLimit": fallback_char_limit, "truncateUnit": "characters", "modelContextLimit": None,
            "originalTokenCount": None, "returnedTokenCount": None}


class ClientDisconnected(Exception):
    pass


class HttpError(Exception):
    def __init__(self, status: int, payload: Any):
        self.status, self.payload = status, payload


class Exchange:
    """One request/response pair, independent of the socket layer (tests drive it directly)."""

    def __init__(self, method: str, target: str, headers: Dict[str, str], body: bytes, writer=None):
        self.method = method.upper()
        parts = urlsplit(target)
        self.path = unquote(parts.path) or "/"
        self.headers = {k.lower(): v for k, v in headers.items()}
        self.body = body
        self.cancel = CancellationToken()
        self.status = 200
        self.response_headers: Dict[str, str] = {}
        self.content_type: Optional[str] = None
        self.started = False
        self.streaming = False
        self.chunks: List[bytes] = []
        self._writer = writer               # socket-backed sink or None (in-memory)

    # -- request side
    def json(self) -> Any:
        try:
            return json.loads(self.body.decode("utf-8") if self.body else "null")
        except (ValueError, UnicodeDecodeError) as e:
            raise HttpError(400, {"error": f"invalid JSON body: {e}"}) from None

    def json_object(self) -> Dict[str, Any]:
        b = self.json()
        if not isinstance(b, dict):
            raise HttpError(400, {"error": "request body must be a JSON object"})
        return b

    # -- response side
    def send_json(self, payload: Any, status: int = 200, ignore_nulls: bool = False) -> None:
        self.send_bytes(serialize(payload, ignore_nulls).encode("utf-8"), "application/json; charset=utf-8", status)

    def send_bytes(self, data: bytes, content_type: str, status: int = 200) -> None:
        self.status, self.content_type = status, content_type
        self.started = True
        self.chunks.append(data)
        if self._writer is not None:
            self._writer.send_full(self, data)

    def begin_stream(self, content_type: str, extra: Optional[Dict[str, str]] = None) -> None:
        if self.started:
            return
        self.content_type = content_type
        self.response_headers.update(extra or {})
        self.started = self.streaming = True
        if self._writer is not None:
            self._writer.begin_stream(self)

    def write(self, data: bytes) -> None:
        if self.cancel.cancelled:
            raise ClientDisconnected()
        self.chunks.append(data)
        if self._writer is not None:
            self._writer.write_chunk(self, data)

    @property
    def text(self) -> str:
        return b"".join(self.chunks).decode("utf-8")


NDJSON_HEADERS = {"Cache-Control": "no-cache"}
SSE_HEADERS = {"Cache-Control": "no-cache", "Connection": "keep-alive"}


class ServerApp:
    def __init__(self, options: ServerHostingOptions, svc: Optional[ModelService] = None,
                 queue: Optional[InferenceQueue] = None, sessions: Optional[SessionManager] = None,
                 log_provider: Optional[FileLoggerProvider] = None, queue_poll_s: float = 1.0):
        self.options = options
        self._provider = log_provider
        n_batch = max(1, int(getattr(options, "max_batch", 1) or 1))
        self.queue = queue or InferenceQueue(self.logger("TensorSharp.Server.InferenceQueue"), capacity=n_batch)
        if svc is None and n_batch > 1:
            # concurrent requests: one service per running slot over one loaded model, model calls merged per step
            from .service_pool import ServicePool
            svc = ServicePool(self.logger("TensorSharp.Server.ModelService"), self.queue, n_batch, max_context=options.max_context)
        self.svc = svc or ModelService(self.logger("TensorSharp.Server.ModelService"), max_context=options.max_context,
                                       max_sessions=options.max_sessions)
        self.sessions = sessions or SessionManager(self.logger("TensorSharp.Server.SessionManager"))
        self.queue_poll_s = queue_poll_s
        self._http_log = self.logger("TensorSharp.Server.Logging.RequestLoggingMiddleware")
        self.low_noise_paths = {"/api/queue/status", "/metrics"}
        self.web_root = options.web_root or os.path.join(os.path.dirname(__file__), "wwwroot")
        self._routes: List[Tuple[str, str, Callable]] = [
            ("GET", "/", self.root), ("GET", "/api/version", self.version), ("GET", "/api/tags", self.ollama_tags),
            ("POST", "/api/show", self.ollama_show), ("POST", "/api/generate", self.ollama_generate),
            ("POST", "/api/chat/ollama", self.ollama_chat), ("POST", "/v1/chat/completions", self.openai_chat),
            ("GET", "/v1/models", self.openai_models), ("POST", "/api/sessions", self.create_session),
            ("DELETE", "/api/sessions/{id}", self.dispose_session), ("POST", "/api/upload", self.upload),
            ("GET", "/api/queue/status", self.queue_status), ("GET", "/metrics", self.metrics), ("GET", "/api/models", self.webui_models),
            ("POST", "/api/models/load", self.webui_load_model), ("POST", "/api/chat", self.webui_chat)]

    def logger(self, category: str) -> Logger:
        return self._provider.get_logger(category) if self._provider is not None else NULL_LOGGER

    # ------------------------------------------------------------------ dispatch + request logging
    def _match(self, method: str, path: str):
        for m, pat, fn in self._routes:
            if m != method:
                continue
            if "{id}" in pat:
                prefix = pat[:pat.index("{id}")]
                if path.startswith(prefix) and "/" not in path[len(prefix):] and path[len(prefix):]:
                    return fn, path[len(prefix):]
            elif path == pat or (pat != "/" and path.rstrip("/") == pat):
                return fn, None
        return None, None

    def handle(self, ex: Exchange) -> None:
        rid = (ex.headers.get(REQUEST_ID_HEADER.lower()) or "").strip() or uuid.uuid4().hex[:12]
        ex.request_id = rid
        ex.response_headers[REQUEST_ID_HEADER] = rid
        scope = {"RequestId": rid, "Operation": f"{ex.method} {ex.path}"}
        client = classify_client(ex.path)
        if client:
            scope["Client"] = client
        low = ex.path.lower() in self.low_noise_paths
        with log_scope(**scope):
            self._http_log.log("Debug" if low else "Information", Ev.HttpRequestStarted,
                               "HTTP {Method} {Path} (content-type={ContentType}, content-length={ContentLength})",
                               Method=ex.method, Path=ex.path, ContentType=ex.headers.get("content-type", ""),
                               ContentLength=ex.headers.get("content-length", "(none)"))
            t0 = time.perf_counter()
            try:
                fn, arg = self._match(ex.method, ex.path)
                if fn is None:
                    self.fallback(ex)
                elif arg is not None:
                    fn(ex, arg)
                else:
                    fn(ex)
            except HttpError as he:
                if not ex.started:
                    ex.send_json(he.payload, he.status)
            except ClientDisconnected:
                ex.cancel.cancel()
            except Exception as e:
                self._http_log.log("Error", Ev.HttpRequestFailed, "HTTP {Method} {Path} threw {ExceptionType} after "
                                   "{ElapsedMs:.1f} ms", exc=e, Method=ex.method, Path=ex.path,
                                   ExceptionType=type(e).__name__, ElapsedMs=(time.perf_counter() - t0) * 1e3)
                if not ex.started:
                    ex.send_json({"error": str(e)}, 500)
                METRICS.record_http(client, 500)
                return
            METRICS.record_http(client, ex.status)
            level = "Error" if ex.status >= 500 else "Warning" if ex.status >= 400 else "Debug" if low else "Information"
            self._http_log.log(level, Ev.HttpRequestRejected if ex.status >= 400 else Ev.HttpRequestCompleted,
                               "HTTP {Method} {Path} -> {StatusCode} in {ElapsedMs:.1f} ms (response content-type="
                               "{ResponseContentType})", Method=ex.method, Path=ex.path, StatusCode=ex.status,
                               ElapsedMs=(time.perf_counter() - t0) * 1e3, ResponseContentType=ex.content_type or "(none)")

    # ------------------------------------------------------------------ small routes
    def root(self, ex: Exchange) -> None:
        ex.send_json("TensorSharp.Server is running")

    def version(self, ex: Exchange) -> None:
        ex.send_json({"version": VERSION})

    def fallback(self, ex: Exchange) -> None:
        index = os.path.join(self.web_root, "index.html") if self.web_root else None
        if ex.method == "GET" and self.web_root:
            rel = os.path.normpath(ex.path.lstrip("/"))
            cand = os.path.join(self.web_root, rel)
            if rel and not rel.startswith("..") and os.path.isfile(cand):
                ctype = {".html": "text/html", ".js": "text/javascript", ".css": "text/css", ".png": "image/png",
                         ".svg": "image/svg+xml", ".ico": "image/x-icon"}.get(os.path.splitext(cand)[1].lower(),
                                                                              "application/octet-stream")
                with open(cand, "rb") as f:
                    ex.send_bytes(f.read(), ctype)
                return
        if index and os.path.isfile(index):
            with open(index, "rb") as f:
                ex.send_bytes(f.read(), "text/html")
            return
        ex.send_bytes(("index.html not found. WebRootPath: " + (self.web_root or "(null)")).encode(), "text/plain", 404)

    def queue_status(self, ex: Exchange) -> None:
        s = self.queue.get_status()
        ex.send_json({"busy": s.busy, "pending_requests": s.pending_requests, "total_processed": s.total_processed})

    def metrics(self, ex: Exchange) -> None:
        text = METRICS.render(self.queue, getattr(self.svc, "gather", None))
        ex.send_bytes(text.encode("utf-8"), "text/plain; version=0.0.4; charset=utf-8")

    def create_session(self, ex: Exchange) -> None:
        s = self.sessions.create_session()
        ex.send_json({"sessionId": s.id, "createdAt": iso_o(s.created_at)})

    def dispose_session(self, ex: Exchange, sid: str) -> None:
        if sid == DEFAULT_SESSION_ID:
            ex.send_json({"ok": False, "error": "Cannot dispose the default session."}, 400)
            return
        removed = self.sessions.try_remove(sid)
        if removed is None:
            ex.send_json({"ok": False, "error": f"Session '{sid}' not found."}, 404)
            return
        with self.queue.enqueue(ex.cancel, ex.request_id) as ticket:
            ticket.wait_until_ready()
            self.svc.dispose_session(removed)
        ex.send_json({"ok": True, "sessionId": sid})

    # ------------------------------------------------------------------ shared plumbing
    def _ensure_loaded(self, model_name: str) -> Optional[str]:
        o = self.options
        return try_ensure_hosted_model_loaded(self.svc, model_name, o.startup_model_path, o.startup_mmproj_path,
                                              o.default_backend)

    def _wait_with_progress(self, ex: Exchange, ticket, make_chunk: Callable[[int, int], bytes]) -> None:
        while not ticket.is_ready:
            if ex.cancel.cancelled:
                raise ClientDisconnected()
            ex.write(make_chunk(ticket.position, self.queue.pending_count))
            ticket.wait(self.queue_poll_s)

    @staticmethod
    def _use_parser(think: bool, tools, arch) -> bool:
        return bool(think) or bool(tools) or is_always_required(arch)

    # ------------------------------------------------------------------ Ollama
    def ollama_tags(self, ex: Exchange) -> None:
        models = []
        p = self.options.startup_model_path
        if p and p.strip():
            exists = os.path.isfile(p)
            fn = os.path.basename(p)
            import datetime as _dt
            mod = iso_o(_dt.datetime.fromtimestamp(os.path.getmtime(p), _dt.timezone.utc)) if exists else ""
            models.append({"name": os.path.splitext(fn)[0], "model": fn, "size": os.path.getsize(p) if exists else 0,
                           "modified_at": mod})
        ex.send_json({"models": models})

    @staticmethod
    def _require_model(body: Dict[str, Any]) -> Optional[str]:
        m = body.get("model")
        return m if isinstance(m, str) and m.strip() else None

    def ollama_show(self, ex: Exchange) -> None:
        body = ex.json_object()
        name = self._require_model(body)
        if name is None:
            ex.send_json({"error": "model is required"}, 400)
            return
        path, err = try_resolve_hosted_model_request(name, self.options.startup_model_path)
        if err:
            ex.send_json({"error": err}, 404)
            return
        fam = self.svc.architecture if self.svc.is_loaded and self.svc.loaded_model_name == os.path.basename(path) else ""
        ex.send_json({"modelfile": "", "parameters": "", "template": "", "details": {"format": "gguf", "family": fam},
                      "model_info": {"file": os.path.basename(path), "size": os.path.getsize(path)}})

    @staticmethod
    def _num_predict(body: Dict[str, Any], default: int = 200) -> int:
        o = body.get("options")
        if isinstance(o, dict) and "num_predict" in o:
            return int(o["num_predict"])
        return default

    def ollama_generate(self, ex: Exchange) -> None:
        body = ex.json_object()
        name = self._require_model(body)
        if name is None:
            ex.send_json({"error": "model is required"}, 400)
            return
        prompt = body.get("prompt") or ""
        stream = bool(body.get("stream", True))
        max_tokens = self._num_predict(body)
        cfg = P.parse_sampling_ollama(body, self.options.default_sampling_config)
        images = P.decode_base64_images(body, self.options.upload_directory)
        with self.queue.enqueue(ex.cancel, ex.request_id) as ticket:
            if stream:
                ex.begin_stream("application/x-ndjson", NDJSON_HEADERS)
                self._wait_with_progress(ex, ticket, lambda p, n: ndjson_line(Ollama.queue_generate_chunk(name, p, n)))
                err = self._ensure_loaded(name)
                if err:
                    ex.write(ndjson_line(Ollama.generate_error(name, err)))
                    return
                for it in self.svc.generate_stream(prompt, images, max_tokens, ex.cancel, cfg):
                    m = self.svc.loaded_model_name
                    ex.write(ndjson_line(Ollama.generate_final_chunk(m, *it[2:]) if it.done
                                         else Ollama.generate_token_chunk(m, it.piece)))
                return
            ticket.wait_until_ready()
            err = self._ensure_loaded(name)
            if err:
                ex.send_json({"error": err}, 404)
                return
            pieces, final = [], None
            for it in self.svc.generate_stream(prompt, images, max_tokens, ex.cancel, cfg):
                if it.done:
                    final = it
                else:
                    pieces.append(it.piece)
            ex.send_json(Ollama.generate_non_streaming(self.svc.loaded_model_name, "".join(pieces), *final[2:]))

    def ollama_chat(self, ex: Exchange) -> None:
        body = ex.json_object()
        name = self._require_model(body)
        if name is None:
            ex.send_json({"error": "model is required"}, 400)
            return
        if not isinstance(body.get("messages"), list):
            ex.send_json({"error": "messages is required"}, 400)
            return
        stream = bool(body.get("stream", True))
        max_tokens = self._num_predict(body)
        cfg = P.parse_sampling_ollama(body, self.options.default_sampling_config)
        messages = P.parse_messages_ollama(body["messages"], self.options.upload_directory)
        tools = P.parse_tools_ollama(body)
        think = body.get("think") is True
        with self.queue.enqueue(ex.cancel, ex.request_id) as ticket:
            if stream:
                self._ollama_chat_stream(ex, ticket, name, messages, max_tokens, cfg, tools, think)
            else:
                self._ollama_chat_complete(ex, ticket, name, messages, max_tokens, cfg, tools, think)

    def _ollama_chat_stream(self, ex, ticket, name, messages, max_tokens, cfg, tools, think) -> None:
        ex.begin_stream("application/x-ndjson", NDJSON_HEADERS)
        self._wait_with_progress(ex, ticket, lambda p, n: ndjson_line(Ollama.queue_chat_chunk(name, p, n)))
        err = self._ensure_loaded(name)
        if err:
            ex.write(ndjson_line(Ollama.chat_error_chunk(name, err)))
            return
        parser = create_output_parser(self.svc.architecture)
        parser.init(think, tools)
        use_parser = self._use_parser(think, tools, self.svc.architecture)
        collected = None
        for it in self.svc.chat_stream_with_metrics(messages, max_tokens, ex.cancel, cfg, tools, think):
            m = self.svc.loaded_model_name
            if not it.done:
                if not use_parser:
                    ex.write(ndjson_line(Ollama.chat_raw_token_chunk(m, it.piece), True))
                    continue
                parsed = parser.add(it.piece, False)
                if parsed.tool_calls is not None:
                    collected = parsed.tool_calls
                thinking = parsed.thinking or None
                content = parsed.content or ""
                if thinking is None and not content:
                    continue
                ex.write(ndjson_line(Ollama.chat_parsed_chunk(m, content, thinking), True))
                continue
            if use_parser:
                fin = parser.add("", True)
                if fin.tool_calls is not None:
                    collected = fin.tool_calls
                if fin.thinking or fin.content:
                    ex.write(ndjson_line(Ollama.chat_parsed_chunk(m, fin.content or "", fin.thinking or None), True))
                ex.write(ndjson_line(Ollama.chat_parsed_final_chunk(m, collected, *it[2:]), True))
            else:
                ex.write(ndjson_line(Ollama.chat_raw_final_chunk(m, *it[2:]), True))

    def _ollama_chat_complete(self, ex, ticket, name, messages, max_tokens, cfg, tools, think) -> None:
        ticket.wait_until_ready()
        err = self._ensure_loaded(name)
        if err:
            ex.send_json({"error": err}, 404)
            return
        pieces, final = [], None
        for it in self.svc.chat_stream_with_metrics(messages, max_tokens, ex.cancel, cfg, tools, think):
            if it.done:
                final = it
            else:
                pieces.append(it.piece)
        raw = "".join(pieces)
        done_reason = "stop"
        if self._use_parser(think, tools, self.svc.architecture):
            parser = create_output_parser(self.svc.architecture)
            parser.init(think, tools)
            parsed = parser.add(raw, True)
            msg = Ollama.chat_non_streaming_message(parsed.content, parsed.thinking if think and parsed.thinking else None,
                                                    parsed.tool_calls)
            if parsed.tool_calls:
                done_reason = "tool_calls"
        else:
            msg = Ollama.chat_plain_message(raw)
        ex.send_json(Ollama.chat_non_streaming(self.svc.loaded_model_name, msg, done_reason, *final[2:]), ignore_nulls=True)

    # ------------------------------------------------------------------ OpenAI
    def openai_models(self, ex: Exchange) -> None:
        p = self.options.startup_model_path
        data = [{"id": os.path.splitext(os.path.basename(p))[0], "object": "model", "owned_by": "local"}] if p and p.strip() else []
        ex.send_json({"object": "list", "data": data})

    def openai_chat(self, ex: Exchange) -> None:
        body = ex.json_object()
        name = self._require_model(body)
        if name is None:
            ex.send_json(OpenAI.error("model is required"), 400)
            return
        if not isinstance(body.get("messages"), list):
            ex.send_json(OpenAI.error("messages is required"), 400)
            return
        stream = body.get("stream") is True
        max_tokens = int(body["max_tokens"]) if "max_tokens" in body else 200
        cfg = P.parse_sampling_openai(body, self.options.default_sampling_config)
        messages = P.parse_messages_openai(body["messages"], self.options.upload_directory)
        rid = OpenAI.new_request_id()
        tools = P.parse_tools_openai(body)
        think = body.get("think") is True
        fmt, fmt_err = P.parse_response_format(body)
        if fmt_err:
            ex.send_json(OpenAI.error(fmt_err), 400)
            return
        if fmt is not None:
            if think:
                ex.send_json(OpenAI.error("response_format cannot be combined with think=true"), 400)
                return
            if tools:
                ex.send_json(OpenAI.error("response_format cannot be combined with tools"), 400)
                return
            v = validate_schema(fmt)
            if not v.is_valid:
                ex.send_json(OpenAI.error(v.error_message, details=v.errors), 400)
                return
        inference_messages = apply_to_messages(messages, fmt)
        with self.queue.enqueue(ex.cancel, ex.request_id) as ticket:
            if stream:
                self._openai_stream(ex, ticket, rid, name, inference_messages, max_tokens, cfg, tools, think, fmt)
            else:
                self._openai_complete(ex, ticket, rid, name, inference_messages, max_tokens, cfg, tools, think, fmt)

    def _openai_stream(self, ex, ticket, rid, name, messages, max_tokens, cfg, tools, think, fmt) -> None:
        structured = fmt is not None
        if not structured:
            ex.begin_stream("text/event-stream", SSE_HEADERS)
            self._wait_with_progress(ex, ticket, lambda p, n: sse_event(OpenAI.queue_chunk(rid, name, p, n)))
        else:
            ticket.wait_until_ready()
        err = self._ensure_loaded(name)
        if err:
            if structured:
                ex.send_json(OpenAI.error(err), 404)
            else:
                ex.write(sse_event(OpenAI.error_content_chunk(rid, name, err)))
                ex.write(SSE_DONE)
            return
        arch = self.svc.architecture
        use_parser = self._use_parser(think, tools, arch)
        buffer: List[str] = []
        parser = None
        collected = None
        if use_parser and not structured:
            parser = create_output_parser(arch)
            parser.init(think, tools)
        for it in self.svc.chat_stream_with_metrics(messages, max_tokens, ex.cancel, cfg, tools, think):
            m = self.svc.loaded_model_name
            if not it.done:
                if structured:
                    buffer.append(it.piece)
                elif parser is not None:
                    parsed = parser.add(it.piece, False)
                    if parsed.tool_calls is not None:
                        collected = parsed.tool_calls
                    content = parsed.content or ""
                    if not content and not parsed.thinking:
                        continue
                    ex.write(sse_event(OpenAI.content_chunk(rid, m, content or None)))
                else:
                    ex.write(sse_event(OpenAI.content_chunk(rid, m, it.piece)))
                continue
            if structured:
                raw = "".join(buffer)
                if use_parser:
                    sp = create_output_parser(arch)
                    sp.init(think, tools)
                    raw = sp.add(raw, True).content or ""
                norm = normalize_output(raw, fmt)
                if not norm.is_valid:
                    ex.send_json(OpenAI.error(norm.error_message, "invalid_response_error", norm.errors), 422)
                    return
                ex.begin_stream("text/event-stream", SSE_HEADERS)
                ex.write(sse_event(OpenAI.structured_content_chunk(rid, m, norm.normalized_content)))
                ex.write(sse_event(OpenAI.end_chunk(rid, m, "stop", it.prompt_tokens, it.eval_tokens, it.kv_reused_tokens)))
                ex.write(SSE_DONE)
                continue
            finish = "stop"
            if parser is not None:
                fin = parser.add("", True)
                if fin.tool_calls is not None:
                    collected = fin.tool_calls
                if fin.content:
                    ex.write(sse_event(OpenAI.content_chunk(rid, m, fin.content)))
                if collected:
                    finish = "tool_calls"
            ex.write(sse_event(OpenAI.end_chunk(rid, m, finish, it.prompt_tokens, it.eval_tokens, it.kv_reused_tokens)))
            ex.write(SSE_DONE)

    def _openai_complete(self, ex, ticket, rid, name, messages, max_tokens, cfg, tools, think, fmt) -> None:
        ticket.wait_until_ready()
        err = self._ensure_loaded(name)
        if err:
            ex.send_json(OpenAI.error(err), 404)
            return
        pieces, final = [], None
        for it in self.svc.chat_stream_with_metrics(messages, max_tokens, ex.cancel, cfg, tools, think):
            if it.done:
                final = it
            else:
                pieces.append(it.piece)
        raw = "".join(pieces)
        finish = "stop"
        if fmt is not None:
            norm = normalize_output(raw, fmt)
            if not norm.is_valid:
                ex.send_json(OpenAI.error(norm.error_message, "invalid_response_error", norm.errors), 422)
                return
            msg = OpenAI.structured_assistant_message(norm.normalized_content)
        elif self._use_parser(think, tools, self.svc.architecture):
            parser = create_output_parser(self.svc.architecture)
            parser.init(think, tools)
            parsed = parser.add(raw, True)
            msg = OpenAI.parsed_assistant_message(parsed.content, parsed.thinking if think and parsed.thinking else None,
                                                  parsed.tool_calls)
            if parsed.tool_calls:
                finish = "tool_calls"
        else:
            msg = OpenAI.plain_assistant_message(raw)
        ex.send_json(OpenAI.completion(rid, self.svc.loaded_model_name, msg, finish, final.prompt_tokens,
                                       final.eval_tokens, final.kv_reused_tokens), ignore_nulls=True)

    # ------------------------------------------------------------------ web UI
    def webui_models(self, ex: Exchange) -> None:
        o = self.options
        ex.send_json({
            "models": [os.path.basename(o.startup_model_path)] if o.startup_model_path else [],
            "mmProjModels": [os.path.basename(o.startup_mmproj_path)] if o.startup_mmproj_path else [],
            "loaded": self.svc.loaded_model_name, "loadedMmProj": self.svc.loaded_mmproj_name,
            "loadedBackend": self.svc.loaded_backend, "defaultBackend": o.default_backend,
            "supportedBackends": o.supported_backends, "architecture": self.svc.architecture,
            "hostedModelPath": o.startup_model_path, "hostedMmProjPath": o.startup_mmproj_path,
            "defaultMaxTokens": o.default_web_max_tokens})

    def webui_load_model(self, ex: Exchange) -> None:
        body = ex.json_object()
        if "model" not in body:
            raise HttpError(400, {"ok": False, "error": "model is required"})
        model_name, requested_backend, mmproj = body.get("model"), body.get("backend"), body.get("mmproj")
        backend, err = try_resolve_supported_backend(self.options, requested_backend)
        if err:
            ex.send_json({"ok": False, "error": err}, 400)
            return
        path, err = try_resolve_hosted_model_request(model_name, self.options.startup_model_path)
        if err:
            ex.send_json({"ok": False, "error": err}, 400)
            return
        err = try_validate_hosted_mmproj_request(mmproj, self.options.startup_mmproj_path)
        if err:
            ex.send_json({"ok": False, "error": err}, 400)
            return
        with self.queue.enqueue(ex.cancel, ex.request_id) as ticket:
            ticket.wait_until_ready()
            try:
                self.svc.load_model(path, self.options.startup_mmproj_path, backend)
            except Exception as e:
                ex.send_json({"ok": False, "error": str(e)}, 500)
                return
            ex.send_json({"ok": True, "model": self.svc.loaded_model_name, "loadedMmProj": self.svc.loaded_mmproj_name,
                          "architecture": self.svc.architecture})

    def upload(self, ex: Exchange) -> None:
        log = self.logger("TensorSharp.Server.Upload")
        ctype = ex.headers.get("content-type", "")
        if not ctype.lower().startswith("multipart/form-data"):
            log.warning(Ev.UploadRejected, "Upload rejected: missing multipart form data")
            ex.send_json({"error": "Expected multipart form data"}, 400)
            return
        msg = email.message_from_bytes(b"Content-Type: " + ctype.encode() + b"\r\nMIME-Version: 1.0\r\n\r\n" + ex.body,
                                       policy=email.policy.HTTP)
        file_part = None
        if msg.is_multipart():
            for part in msg.iter_parts():
                if part.get_filename() is not None:
                    file_part = part
                    break
        if file_part is None:
            log.warning(Ev.UploadRejected, "Upload rejected: no file in request")
            ex.send_json({"error": "No file uploaded"}, 400)
            return
        file_name = file_part.get_filename()
        data = file_part.get_payload(decode=True) or b""
        ext = os.path.splitext(file_name)[1].lower()
        os.makedirs(self.options.upload_directory, exist_ok=True)
        save_path = os.path.join(self.options.upload_directory, uuid.uuid4().hex + ext)
        with open(save_path, "wb") as f:
            f.write(data)
        kind = classify_extension(ext)
        log.info(Ev.UploadReceived, "Upload received: name={FileName} ext={Extension} mediaType={MediaType} bytes={Length} "
                 "savedPath={SavedPath}", FileName=file_name, Extension=ext, MediaType=kind, Length=len(data), SavedPath=save_path)
        if kind == "video":
            frames = media.extract_video_frames(save_path)
            ex.send_json({"ok": True, "path": save_path, "mediaType": kind, "fileName": file_name,
                          "frames": [os.path.basename(f) for f in frames], "framePaths": frames})
            return
        if kind == "text":
            model = self.svc.model
            prepared = prepare_text_content(data.decode("utf-8", errors="replace"),
                                            model.tokenizer if model is not None else None,
                                            int(getattr(model, "max_context", 0) or 0) if model is not None else 0,
                                            self.options.max_text_file_chars)
            ex.send_json({"ok": True, "path": save_path, "mediaType": kind, "fileName": file_name, **prepared})
            return
        ex.send_json({"ok": True, "path": save_path, "mediaType": kind, "fileName": file_name})

    def webui_chat(self, ex: Exchange) -> None:
        log = self.logger("TensorSharp.Server.WebUI.Chat")
        body = ex.json_object()
        err = validate_webui_chat_request(body.get("model"), body.get("backend"))
        if err:
            ex.send_json({"error": err}, 400)
            return
        sid = body.get("sessionId")
        if isinstance(sid, str) and sid.strip():
            session = self.sessions.get_session(sid)
            if session is None or session.is_disposed:
                ex.send_json({"error": f"Session '{sid}' not found or has been disposed."}, 404)
                return
        else:
            session = self.sessions.default_session
        if body.get("newChat") is True:
            self.svc.reset_session(session)
        if not self.svc.is_loaded:
            ex.send_json({"error": "No model loaded"}, 400)
            return
        if not isinstance(body.get("messages"), list):
            raise HttpError(400, {"error": "messages is required"})
        max_tokens = int(body["maxTokens"]) if "maxTokens" in body else self.options.default_web_max_tokens
        cfg = P.parse_sampling_webui(body, self.options.default_sampling_config)
        think = body.get("think") is True
        tools = P.parse_tools_ollama(body) if isinstance(body.get("tools"), list) else None
        messages = P.parse_messages_webui(body["messages"])
        ex.begin_stream("text/event-stream", SSE_HEADERS)
        prefer = getattr(self.svc, "preferred_slot", None)
        with self.queue.enqueue(ex.cancel, ex.request_id, prefer_slot=prefer(session) if prefer else -1) as ticket:
            self._wait_with_progress(ex, ticket, lambda p, n: sse_event(WebUi.queue_progress(p, n)))
            t0 = time.perf_counter()
            count = 0
            parser = None
            if self._use_parser(think, tools, self.svc.architecture):
                parser = create_output_parser(self.svc.architecture)
                parser.init(think, tools)
            aborted, error = False, None
            prompt_tokens = reused = 0

            def emit(parsed) -> None:
                if parsed.thinking:
                    ex.write(sse_event(WebUi.thinking(parsed.thinking)))
                if parsed.content:
                    ex.write(sse_event(WebUi.token(parsed.content)))
                if parsed.tool_calls is not None:
                    ex.write(sse_event(WebUi.tool_calls(parsed.tool_calls)))

            try:
                for it in self.svc.chat_stream_with_metrics(messages, max_tokens, ex.cancel, cfg, tools, think, session=session):
                    if it.done:
                        prompt_tokens, reused = it.prompt_tokens, it.kv_reused_tokens
                        continue
                    if not it.piece:
                        continue
                    count += 1
                    if parser is not None:
                        emit(parser.add(it.piece, False))
                    else:
                        ex.write(sse_event(WebUi.token(it.piece)))
            except ClientDisconnected:
                aborted = True
                ex.cancel.cancel()
                log.warning(Ev.ChatAborted, "Web UI chat aborted by client (sessionId={SessionId}, partialTokens={PartialTokens})",
                            SessionId=session.id, PartialTokens=count)
            except Exception as e:
                log.error(Ev.ChatFailed, "Web UI chat failed (sessionId={SessionId}, partialTokens={PartialTokens})", exc=e,
                          SessionId=session.id, PartialTokens=count)
                error = str(e)
            try:
                if parser is not None and not aborted:
                    emit(parser.add("", True))
                dt = time.perf_counter() - t0
                ex.write(sse_event(WebUi.done(count, dt, count / dt if count > 0 and dt > 0 else 0.0, aborted, error,
                                              session.id, prompt_tokens, reused)))
            except ClientDisconnected:
                pass


# ---------------------------------------------------------------------------- socket layer
class _SocketWriter:
    def __init__(self, handler: BaseHTTPRequestHandler):
        self.h = handler

    def _head(self, ex: Exchange, extra: Dict[str, str]) -> None:
        h = self.h
        h.send_response(ex.status)
        if ex.content_type:
            h.send_header("Content-Type", ex.content_type)
        for k, v in {**ex.response_headers, **extra}.items():
            h.send_header(k, v)
        h.end_headers()

    def send_full(self, ex: Exchange, data: bytes) -> None:
        try:
            self._head(ex, {"Content-Length": str(len(data))})
            self.h.wfile.write(data)
            self.h.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, TimeoutError):
            ex.cancel.cancel()

    def begin_stream(self, ex: Exchange) -> None:
        try:
            self._head(ex, {"Transfer-Encoding": "chunked"})
            self.h.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, TimeoutError):
            ex.cancel.cancel()
            raise ClientDisconnected() from None

    def write_chunk(self, ex: Exchange, data: bytes) -> None:
        if not data:
            return
        try:
            self.h.wfile.write(b"%x\r\n" % len(data) + data + b"\r\n")
            self.h.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, TimeoutError):
            ex.cancel.cancel()
            raise ClientDisconnected() from None

    def end_stream(self, ex: Exchange) -> None:
        try:
            self.h.wfile.write(b"0\r\n\r\n")
            self.h.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, TimeoutError):
            ex.cancel.cancel()


def make_handler(app: ServerApp, max_body_bytes: int = 512 * 1024 * 1024):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "TensorSharpB200/" + VERSION

        def log_message(self, fmt, *args):          # request logging goes to the JSONL log instead
            pass

        def _serve(self) -> None:
            n = int(self.headers.get("Content-Length") or 0)
            if n > max_body_bytes:
                self.send_error(413)
                return
            body = self.rfile.read(n) if n > 0 else b""
            writer = _SocketWriter(self)
            ex = Exchange(self.command, self.path, dict(self.headers.items()), body, writer)
            app.handle(ex)
            if ex.streaming:
                writer.end_stream(ex)
            elif not ex.started:
                ex.send_bytes(b"", "text/plain", 204)

        do_GET = do_POST = do_DELETE = do_PUT = _serve

    return Handler


class TensorSharpHTTPServer(ThreadingHTTPServer):
    daemon_threads = True
    allow_reuse_address = True
    request_queue_size = 128


def serve(app: ServerApp, host: Optional[str] = None, port: Optional[int] = None) -> TensorSharpHTTPServer:
    """Bind and return the server; the caller runs ``serve_forever()`` (or a thread does)."""
    return TensorSharpHTTPServer((host or app.options.host, app.options.port if port is None else port), make_handler(app))
