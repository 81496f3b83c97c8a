"""The hosted model and its chat / generate streams.

Parity: TensorSharp.Server/ModelService.cs — LoadModel :160, ActivateSession :124,
ChatStreamInternalAsync :300 (render with cached raw tokens, truncate to the context, plan KV
reuse, sample, emit UTF-8-safe pieces, stop sequences, track history), AugmentWithCachedRawTokens
:497, UpdateTrackedHistory :564, PrepareForGeneration :614 (exact match / partial reuse / reset),
ForwardPromptPrefill :729 with ResolvePrefillChunkSize :777 (5120 tokens on the GPU backend, 2048
on the CPU one), TruncatePromptToContext :803, GenerateStreamAsync :865, FindValidUtf8Length
:1034, PrepareHistoryForInference :1056 (Gemma 4 video-frame downsampling).

Streams are plain generators of ``StreamItem``; the HTTP layer runs them on the request thread
while it holds the inference queue's ticket.  Unlike the reference, a session keeps its own
sequence in the paged KV pool when the model was created with ``max_seqs > 1``, so switching
sessions costs nothing until the pool is full (then the least recently used one is evicted).
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Iterator, List, NamedTuple, Optional, Sequence

from ..runtime import media
from ..runtime.chat import ChatMessage, ToolFunction
from ..runtime.kv_cache import ReusePlanKind
from ..runtime.logging import Ev, NULL_LOGGER, log_scope
from ..runtime.prompt_renderer import GgufPromptRenderer, KVCachePromptRenderer
from ..runtime.sampling import SamplingConfig, TokenSampler
from .metrics import METRICS
from .options import backend_device, canonicalize_backend
from .sessions import ChatSession, _utcnow


class StreamItem(NamedTuple):
    piece: str
    done: bool
    prompt_tokens: int = 0
    eval_tokens: int = 0
    kv_reused_tokens: int = 0
    total_ns: int = 0
    prompt_ns: int = 0
    eval_ns: int = 0


class PromptTooLongError(RuntimeError):
    pass


def find_valid_utf8_length(b: bytes) -> int:
    """Length of the longest prefix of ``b`` that does not end inside a multi-byte sequence."""
    n = len(b)
    for i in range(1, min(4, n) + 1):
        c = b[n - i]
        if c & 0x80 == 0:
            return n
        if c & 0xE0 == 0xC0:
            return n if i >= 2 else n - i
        if c & 0xF0 == 0xE0:
            return n if i >= 3 else n - i
        if c & 0xF8 == 0xF0:
            return n if i >= 4 else n - i
        if c & 0xC0 == 0x80:
            continue
        return n
    return n


def resolve_prefill_chunk_size(backend: Optional[str], token_count: int) -> int:
    if token_count <= 0:
        return 0
    return min(token_count, 5120 if canonicalize_backend(backend) == "b200" else 2048)


def sanitize_for_log(s: Optional[str]) -> str:
    return (s or "").replace("\r", "\\r").replace("\n", "\\n")


def _clone_with(m: ChatMessage, **kw) -> ChatMessage:
    d = dict(role=m.role, content=m.content, image_paths=m.image_paths, audio_paths=m.audio_paths,
             text_file_paths=m.text_file_paths, is_video=m.is_video, tool_calls=m.tool_calls, thinking=m.thinking,
             raw_output_tokens=m.raw_output_tokens)
    d.update(kw)
    return ChatMessage(**d)


def augment_with_cached_raw_tokens(incoming: Optional[List[ChatMessage]],
                                   tracked: Optional[Sequence[ChatMessage]]) -> Optional[List[ChatMessage]]:
    """Give assistant turns that match the tracked history their originally sampled token ids,
    so re-rendering the conversation reproduces the cached token sequence exactly."""
    if incoming is None:
        return None
    match_until = 0
    if tracked is not None:
        for i in range(min(len(incoming), len(tracked))):
            src, tr = incoming[i], tracked[i]
            if src.role != tr.role:
                break
            if src.role != "assistant" and (src.content or "") != (tr.content or ""):
                break
            match_until = i + 1
    out: List[ChatMessage] = []
    for i, src in enumerate(incoming):
        use = (tracked is not None and i < match_until and tracked[i].role == "assistant"
               and bool(tracked[i].raw_output_tokens) and not src.raw_output_tokens)
        out.append(_clone_with(src, raw_output_tokens=tracked[i].raw_output_tokens) if use else src)
    return out


def prepare_history_for_inference(history: Optional[List[ChatMessage]], arch: Optional[str], logger=None):
    if not history:
        return history
    prepared = None
    max_frames = media.get_configured_max_video_frames()
    for i, m in enumerate(history):
        if arch != "gemma4" or not m.is_video or m.image_paths is None or len(m.image_paths) <= max_frames:
            continue
        sampled = [m.image_paths[j] for j in media.select_evenly_spaced_indices(len(m.image_paths), max_frames)]
        if logger is not None:
            logger.info(Ev.VideoFrameDownsample, "Downsampled video frames {Original}->{Kept} for {Architecture}",
                        Original=len(m.image_paths), Kept=len(sampled), Architecture=arch)
        if prepared is None:
            prepared = list(history)
        prepared[i] = _clone_with(m, image_paths=sampled,
                                  audio_paths=list(m.audio_paths) if m.audio_paths is not None else None,
                                  text_file_paths=list(m.text_file_paths) if m.text_file_paths is not None else None)
    return prepared if prepared is not None else history


def has_multimodal_content(x) -> bool:
    if x is None:
        return False
    if isinstance(x, ChatMessage):
        return bool(x.image_paths) or bool(x.audio_paths)
    return any(has_multimodal_content(m) for m in x)


def get_image_paths_in_prompt_order(history: Optional[List[ChatMessage]]) -> List[str]:
    return [p for m in (history or []) if m.image_paths for p in m.image_paths if p]


def _path_list(src):
    out = [p for p in (src or []) if p]
    return out or None


def _relaxed_json(obj) -> str:
    import json
    return json.dumps(obj, ensure_ascii=False, separators=(",", ":"))


def serialize_messages_for_log(messages: Optional[List[ChatMessage]]) -> str:
    if not messages:
        return "[]"
    entries = []
    for m in messages:
        if m is None:
            continue
        e = {"role": m.role or "", "content": m.content or ""}
        for key, val in (("images", _path_list(m.image_paths)), ("audios", _path_list(m.audio_paths)),
                         ("textFiles", _path_list(m.text_file_paths)), ("isVideo", True if m.is_video else None),
                         ("thinking", m.thinking or None), ("toolCallCount", len(m.tool_calls) if m.tool_calls else None)):
            if val is not None:
                e[key] = val
        entries.append(e)
    return _relaxed_json(entries)


def serialize_uploads_for_log(message: Optional[ChatMessage]) -> str:
    if message is None:
        return "[]"
    entries = []
    for paths, kind in ((message.image_paths, "video_frame" if message.is_video else "image"),
                        (message.audio_paths, "audio"), (message.text_file_paths, "text")):
        for p in paths or []:
            if p:
                entries.append({"path": p, "name": os.path.basename(p), "mediaType": kind})
    return _relaxed_json(entries) if entries else "[]"


class ModelService:
    def __init__(self, logger=None, model_factory=None, max_context: Optional[int] = None, max_sessions: int = 1):
        """``model_factory(path, device, **kw)`` defaults to ``ModelBase.create``; tests inject
        a recording fake."""
        self._log = logger or NULL_LOGGER
        self._prompt_renderer = GgufPromptRenderer()
        self._kv_renderer = KVCachePromptRenderer(self._prompt_renderer)
        self._model = None
        self._loaded_model_path: Optional[str] = None
        self._loaded_mmproj_path: Optional[str] = None
        self._backend: Optional[str] = None
        self._active: Optional[ChatSession] = None
        self._intrinsic = ChatSession("__svc_intrinsic__")
        self._factory = model_factory
        self._max_context = max_context
        self._max_sessions = max(1, int(max_sessions))
        self._resident: List[ChatSession] = []          # sessions holding a KV sequence, LRU first

    # ------------------------------------------------------------------ state
    @property
    def is_loaded(self) -> bool:
        return self._model is not None

    @property
    def loaded_model_name(self) -> Optional[str]:
        return os.path.basename(self._loaded_model_path) if self._loaded_model_path else None

    @property
    def loaded_model_path(self) -> Optional[str]:
        return self._loaded_model_path

    @property
    def loaded_mmproj_name(self) -> Optional[str]:
        return os.path.basename(self._loaded_mmproj_path) if self._loaded_mmproj_path else None

    @property
    def loaded_mmproj_path(self) -> Optional[str]:
        return self._loaded_mmproj_path

    @property
    def loaded_backend(self) -> Optional[str]:
        return self._backend if self._model is not None else None

    @property
    def architecture(self) -> Optional[str]:
        return self._model.arch if self._model is not None else None

    @property
    def model(self):
        return self._model

    @property
    def active_session(self) -> Optional[ChatSession]:
        return self._active

    @property
    def kv_cache(self):
        return (self._active or self._intrinsic).kv_cache

    @property
    def tracked_history(self) -> List[ChatMessage]:
        return list((self._active or self._intrinsic).tracked_history)

    def is_model_already_loaded(self, name: str) -> bool:
        return self._model is not None and (self.loaded_model_name or "").lower() == (name or "").lower()

    # ------------------------------------------------------------------ sessions
    def invalidate_kv_cache(self) -> None:
        self.reset_session(self._active or self._intrinsic)

    def _multi(self) -> bool:
        return self._max_sessions > 1 and self._model is not None and hasattr(self._model, "bind_sequence")

    def _drop_residency(self, session: ChatSession) -> None:
        if session.seq is not None and self._model is not None:
            try:
                self._model.free_sequence(session.seq)
            except Exception:
                pass
        session.seq = None
        if session in self._resident:
            self._resident.remove(session)

    def reset_session(self, session: Optional[ChatSession]) -> None:
        if session is None:
            return
        session.tracked_history.clear()
        session.kv_cache.reset()
        if session is self._active and self._model is not None:
            self._model.reset_kv_cache()
        elif self._multi() and session.seq is not None:
            self._drop_residency(session)
        self._log.debug(Ev.SessionReset, "Session {SessionId} reset", SessionId=session.id)

    def dispose_session(self, session: Optional[ChatSession]) -> None:
        if session is None or session.is_disposed:
            return
        was_active = session is self._active
        session.dispose()
        if self._multi():
            if was_active:
                self._model.bind_sequence(None)
            self._drop_residency(session)
            if was_active:
                self._active = None
        elif was_active:
            self._active = None
            if self._model is not None:
                self._model.reset_kv_cache()
        self._log.info(Ev.SessionDisposed, "Session {SessionId} disposed", SessionId=session.id)

    def activate_session(self, session: ChatSession) -> None:
        if session is None:
            raise ValueError("session")
        if session.is_disposed:
            raise RuntimeError(f"Session {session.id} has been disposed.")
        session.last_used_at = _utcnow()
        if session is self._active:
            if self._multi() and session in self._resident:
                self._resident.remove(session)
                self._resident.append(session)
            return
        prev = self._active.id if self._active is not None else None
        if self._multi():
            if session.seq is None:
                while len(self._resident) >= self._max_sessions:
                    victim = self._resident[0]
                    victim.kv_cache.reset()
                    self._drop_residency(victim)
                session.kv_cache.reset()
                session.seq = self._model.new_sequence()
            if session in self._resident:
                self._resident.remove(session)
            self._resident.append(session)
            self._model.bind_sequence(session.seq)
        else:
            if self._active is not None:
                self._active.kv_cache.reset()
            if self._model is not None:
                self._model.reset_kv_cache()
            session.kv_cache.reset()
        self._active = session
        self._log.info(Ev.SessionActivated, "Activated session {SessionId} (previous={PreviousSessionId})",
                       SessionId=session.id, PreviousSessionId=prev or "(none)")

    # ------------------------------------------------------------------ model
    def load_model(self, model_path: str, mmproj_path: Optional[str], backend: Optional[str]) -> None:
        self._log.info(Ev.ModelLoadStarted, "Loading model {Model} (mmproj={MmProj}, backend={Backend})",
                       Model=os.path.basename(model_path), MmProj=os.path.basename(mmproj_path or ""),
                       Backend=backend or "(default)")
        previous = self.loaded_model_name
        if self._model is not None:
            self._model.close()
        self._model = None
        self._loaded_model_path = self._loaded_mmproj_path = None
        self._active = None
        for s in list(self._resident):
            s.seq = None
            s.kv_cache.reset()
        self._resident.clear()
        self._intrinsic.tracked_history.clear()
        self._intrinsic.kv_cache.reset()
        self._intrinsic.seq = None
        if previous:
            self._log.info(Ev.ModelUnloaded, "Unloaded previous model {PreviousModel}", PreviousModel=previous)
        self._backend = canonicalize_backend(backend) or "cpu"
        if self._backend not in ("b200", "cpu"):
            self._backend = "cpu"
        t0 = time.perf_counter()
        try:
            factory = self._factory
            if factory is None:
                from ..models.base import ModelBase
                factory = ModelBase.create
            kw = {}
            if self._max_context:
                kw["max_context"] = self._max_context
            if self._max_sessions > 1:
                kw["max_seqs"] = self._max_sessions
            self._model = factory(model_path, backend_device(self._backend), **kw)
            self._loaded_model_path = model_path
            if mmproj_path and os.path.exists(mmproj_path):
                mm = getattr(self._model, "multimodal", None)
                if mm is not None:
                    mm.load_projectors(mmproj_path)
                self._loaded_mmproj_path = mmproj_path
            self._log.info(Ev.ModelLoadCompleted, "Loaded {Model} arch={Architecture} backend={Backend} in {ElapsedMs:.1f} ms",
                           Model=self.loaded_model_name, Architecture=self.architecture or "(unknown)",
                           Backend=self.loaded_backend or "(unknown)", ElapsedMs=(time.perf_counter() - t0) * 1e3)
        except Exception as ex:
            self._log.error(Ev.ModelLoadFailed, "Model load failed: {Model} backend={Backend}", exc=ex,
                            Model=os.path.basename(model_path), Backend=backend or "(default)")
            raise

    # ------------------------------------------------------------------ multimodal hooks
    def _mm(self):
        return getattr(self._model, "multimodal", None)

    def _mm_queue(self, reused_prefix: int) -> bool:
        mm = self._mm()
        return bool(mm.queue_prompt_embeddings(reused_prefix)) if mm is not None else False

    # ------------------------------------------------------------------ prefill
    def _forward_prompt_prefill(self, tokens: Sequence[int], allow_chunking: bool = True):
        if not tokens:
            raise ValueError("Prompt token list cannot be null or empty.")
        n = len(tokens)
        chunk = resolve_prefill_chunk_size(self._backend, n) if allow_chunking else n
        if chunk >= n:
            return self._model.forward_refill(list(tokens), n)
        self._log.info(Ev.PromptChunking, "Prefilling {PromptTokens} tokens in chunks of {ChunkSize} on {Backend}",
                       PromptTokens=n, ChunkSize=chunk, Backend=self.loaded_backend)
        return self._model.forward_refill(list(tokens), chunk)

    def _prepare_for_generation(self, session: ChatSession, input_tokens: List[int]):
        cache = session.kv_cache
        plan = cache.plan_reuse(input_tokens, bool(getattr(self._model, "supports_kv_truncation", True)))
        n = len(input_tokens)
        if plan.kind == ReusePlanKind.EXACT_MATCH:
            self._log.info(Ev.KvCacheReusePlan, "kv.reuse exact match {Reused}/{PromptTokens} tokens", Reused=n, PromptTokens=n)
            self._mm_queue(n)
            return plan.cached_logits, n
        if plan.kind == ReusePlanKind.PARTIAL_REUSE:
            prefix, suffix_len = plan.reused_prefix_length, plan.tokens_to_forward
            self._model.truncate_kv_cache(prefix)
            cache.truncate_to(prefix)
            queued = self._mm_queue(prefix)
            suffix = list(input_tokens[prefix:prefix + suffix_len])
            self._log.info(Ev.KvCacheReusePlan, "kv.reuse partial {Reused}/{PromptTokens} tokens, forwarding {Suffix} "
                           "({Percent:.1f}% reused)", Reused=prefix, PromptTokens=n, Suffix=suffix_len, Percent=100.0 * prefix / n)
            logits = self._forward_prompt_prefill(suffix, allow_chunking=not queued)
            cache.record_append(suffix, logits)
            return logits, prefix
        if not cache.is_empty:
            self._log.info(Ev.KvCacheReusePlan, "kv.reuse reset: cached {Cached} tokens diverge, full prefill of "
                           "{PromptTokens}", Cached=cache.count, PromptTokens=n)
        else:
            self._log.info(Ev.KvCacheReusePlan, "kv.reuse full prefill {PromptTokens} tokens", PromptTokens=n)
        self._model.reset_kv_cache()
        cache.reset()
        queued = self._mm_queue(0)
        logits = self._forward_prompt_prefill(list(input_tokens), allow_chunking=not queued)
        cache.record_append(list(input_tokens), logits)
        return logits, 0

    def _truncate_prompt_to_context(self, session: ChatSession, tokens: List[int], max_tokens: int) -> List[int]:
        max_ctx = int(getattr(self._model, "max_context", 0) or 0)
        if max_ctx <= 0 or tokens is None or len(tokens) + max_tokens <= max_ctx:
            return tokens
        msg = (f"Prompt ({len(tokens)} tokens) exceeds the model's context limit ({max_ctx} tokens). "
               "Please shorten the input or reduce attached file size.")
        available = max_ctx - max_tokens
        if available < 1:
            raise PromptTooLongError(msg)
        trim = len(tokens) - available
        mm = self._mm()
        if mm is not None:
            trim = mm.clamp_trim_start(trim)
        kept = len(tokens) - trim
        if kept < 1:
            raise PromptTooLongError(msg)
        self._log.warning(Ev.PromptTruncated, "Prompt truncated {Original}->{Kept} tokens (context={Context}, "
                          "maxTokens={MaxTokens}, session={SessionId})", Original=len(tokens), Kept=kept, Context=max_ctx,
                          MaxTokens=max_tokens, SessionId=session.id if session else "(none)")
        if mm is not None:
            mm.trim_prepared_prompt(trim)
        session.tracked_history.clear()
        session.kv_cache.reset()
        self._model.reset_kv_cache()
        return tokens[trim:trim + kept]

    # ------------------------------------------------------------------ recovery
    @contextlib.contextmanager
    def _exchange_guard(self):
        """A bounded device-side wait that gave up surfaces as ``ExchangeTimeoutError`` from a model call.  The request
        fails (the caller sees the error), and before the next one the in-kernel exchanges are torn down and rebuilt
        on every rank, the caches emptied and the sessions' bookkeeping reset; the weights stay loaded."""
        from ..parallel.errors import ExchangeTimeoutError
        try:
            yield
        except ExchangeTimeoutError as ex:
            self.recover_after_exchange_failure(ex)
            raise

    def recover_after_exchange_failure(self, ex=None) -> None:
        self._log.warning(Ev.ChatFailed, "exchange failure ({Error}): rebuilding the exchanges, resetting caches", Error=str(ex))
        METRICS.record_exchange_recovery()
        for session in {id(x): x for x in [self._active, self._intrinsic, *self._resident] if x is not None}.values():
            session.kv_cache.reset()
            session.tracked_history.clear()
            if session.seq is not None:
                self._drop_residency(session)
        recover = getattr(self._model, "recover_exchanges", None)
        if recover is not None:
            try:
                closed = recover()
                self._log.info(Ev.SessionReset, "exchanges dropped: {Closed}; they are set up again on next use", Closed=closed)
            except Exception as err:                       # a rank that cannot rebuild leaves the failure for the watchdog
                self._log.error(Ev.ChatFailed, "recovery failed: {Error}", Error=str(err))

    # ------------------------------------------------------------------ token loop
    def _token_loop(self, session: ChatSession, logits, max_tokens: int, cfg: SamplingConfig, cancel,
                    stop_before_emit: bool, state: dict) -> Iterator[StreamItem]:
        tok = self._model.tokenizer
        sampler = TokenSampler(cfg)
        generated: List[int] = state["generated"]
        raw = bytearray()
        state["raw"] = raw
        prev_len = 0
        state["finish"] = "max_tokens"
        t_eval = time.perf_counter_ns()
        for _ in range(max_tokens):
            if cancel is not None and cancel.cancelled:
                state["cancelled"] = True
                state["finish"] = "cancelled"
                break
            nxt = sampler.sample(logits, generated)
            if tok.is_eos(nxt):
                state["finish"] = "eos"
                break
            generated.append(nxt)
            raw += tok.token_bytes(nxt)
            decoded = bytes(raw[:find_valid_utf8_length(raw)]).decode("utf-8", errors="replace")
            piece = decoded[prev_len:] if prev_len < len(decoded) else ""
            prev_len = len(decoded)
            stop = False
            if cfg.stop_sequences:
                _, stop = sampler.check_stop_sequences(decoded)
                if stop:
                    state["finish"] = "stop_sequence"
                    if stop_before_emit:
                        break
            if "ttft_ns" not in state:
                state["ttft_ns"] = time.perf_counter_ns() - t_eval
            if piece:
                yield StreamItem(piece, False)
            if stop:
                break
            logits = self._model.forward([nxt])
            session.kv_cache.record_append(nxt, logits)
        state["eval_ns"] = time.perf_counter_ns() - t_eval

    # ------------------------------------------------------------------ chat
    def chat_stream(self, history: List[ChatMessage], max_tokens: int, cancel=None,
                    sampling: Optional[SamplingConfig] = None, tools: Optional[List[ToolFunction]] = None,
                    enable_thinking: bool = False, session: Optional[ChatSession] = None) -> Iterator[str]:
        for it in self.chat_stream_with_metrics(history, max_tokens, cancel, sampling, tools, enable_thinking,
                                                session=session, with_metrics=False):
            if it.piece:
                yield it.piece

    def chat_stream_with_metrics(self, history: List[ChatMessage], max_tokens: int, cancel=None,
                                 sampling: Optional[SamplingConfig] = None, tools: Optional[List[ToolFunction]] = None,
                                 enable_thinking: bool = False, session: Optional[ChatSession] = None,
                                 with_metrics: bool = True) -> Iterator[StreamItem]:
        self.activate_session(session or self._intrinsic)
        active = self._active
        arch = self._model.arch
        prepared = prepare_history_for_inference(history, arch, self._log)
        render_history = augment_with_cached_raw_tokens(prepared, active.tracked_history)
        with log_scope(SessionId=active.id, Model=self.loaded_model_name or "(none)",
                       Backend=self.loaded_backend or "(none)", Operation="chat.stream"):
            last_user = next((m for m in reversed(prepared or []) if m is not None and m.role == "user"), None)
            cfg = sampling or SamplingConfig.default()
            self._log.info(Ev.ChatStarted, "chat.start arch={Architecture} maxTokens={MaxTokens} thinking={EnableThinking} "
                           "tools={ToolCount} messages={Messages} uploads={Uploads} sampling(temp={Temperature},topK={TopK},"
                           "topP={TopP},minP={MinP},seed={Seed}) userInput=\"{LastUserContent}\" fullInput={FullInput}",
                           Architecture=arch, MaxTokens=max_tokens, EnableThinking=enable_thinking, ToolCount=len(tools or []),
                           Messages=len(prepared or []), Uploads=serialize_uploads_for_log(last_user),
                           Temperature=cfg.temperature, TopK=cfg.top_k, TopP=cfg.top_p, MinP=cfg.min_p, Seed=cfg.seed,
                           LastUserContent=sanitize_for_log(last_user.content if last_user else ""),
                           FullInput=serialize_messages_for_log(prepared))
            tokens = self._kv_renderer.render_to_tokens(self._model.tokenizer, self._model.cfg.chat_template, render_history,
                                                        arch, add_generation_prompt=True, tools=tools,
                                                        enable_thinking=enable_thinking)
            mm = self._mm()
            if mm is not None:
                tokens = mm.process_prompt_tokens(render_history, tokens)
            tokens = self._truncate_prompt_to_context(active, tokens, max_tokens)
            n_prompt = len(tokens)
            t0 = time.perf_counter_ns()
            state = {"generated": []}
            with self._exchange_guard():
                logits, reused = self._prepare_for_generation(active, tokens)
                prompt_ns = time.perf_counter_ns() - t0
                yield from self._token_loop(active, logits, max_tokens, cfg, cancel, False, state)
            total_ns = time.perf_counter_ns() - t0
            generated = state["generated"]
            text = bytes(state.get("raw", b"")).decode("utf-8", errors="replace")
            active.tracked_history[:] = [_clone_with(m) for m in (render_history or [])]
            active.tracked_history.append(ChatMessage(role="assistant", content=text, raw_output_tokens=generated))
            eval_s = state.get("eval_ns", 0) / 1e9
            pct = 100.0 * reused / n_prompt if n_prompt else 0.0
            if state.get("cancelled"):
                self._log.warning(Ev.ChatAborted, "chat.cancelled tokens={Tokens} promptTokens={PromptTokens} kvReused="
                                  "{KvReusedTokens} kvReusePercent={KvReusePercent:.1f} ttftMs={TimeToFirstTokenMs} elapsedMs="
                                  "{ElapsedMs:.1f} assistantOutput=\"{AssistantContent}\"", Tokens=len(generated),
                                  PromptTokens=n_prompt, KvReusedTokens=reused, KvReusePercent=pct,
                                  TimeToFirstTokenMs=state.get("ttft_ns", 0) // 1_000_000, ElapsedMs=total_ns / 1e6,
                                  AssistantContent=sanitize_for_log(text))
            else:
                self._log.info(Ev.ChatCompleted, "chat.complete tokens={Tokens} promptTokens={PromptTokens} kvReused="
                               "{KvReusedTokens} kvReusePercent={KvReusePercent:.1f} ttftMs={TimeToFirstTokenMs} elapsedMs="
                               "{ElapsedMs:.1f} tokensPerSec={TokensPerSec:.2f} finishReason={FinishReason} "
                               "assistantOutput=\"{AssistantContent}\"", Tokens=len(generated), PromptTokens=n_prompt,
                               KvReusedTokens=reused, KvReusePercent=pct,
                               TimeToFirstTokenMs=state.get("ttft_ns", 0) // 1_000_000, ElapsedMs=total_ns / 1e6,
                               TokensPerSec=(len(generated) / eval_s if eval_s > 0 and generated else 0.0),
                               FinishReason=state["finish"], AssistantContent=sanitize_for_log(text))
            METRICS.record_generation(n_prompt, len(generated), reused, prompt_ns, state.get("eval_ns", 0),
                                      bool(state.get("cancelled")))
            if with_metrics:
                yield StreamItem("", True, n_prompt, len(generated), reused, total_ns, prompt_ns, state.get("eval_ns", 0))

    # ------------------------------------------------------------------ generate
    def generate_stream(self, prompt: str, image_paths: Optional[List[str]], max_tokens: int, cancel=None,
                        sampling: Optional[SamplingConfig] = None, session: Optional[ChatSession] = None) -> Iterator[StreamItem]:
        self.activate_session(session or self._intrinsic)
        active = self._active
        arch = self._model.arch
        messages = [ChatMessage(role="user", content=prompt, image_paths=image_paths)]
        with log_scope(SessionId=active.id, Model=self.loaded_model_name or "(none)",
                       Backend=self.loaded_backend or "(none)", Operation="generate.stream"):
            cfg = sampling or SamplingConfig.default()
            self._log.info(Ev.ChatStarted, "generate.start arch={Architecture} maxTokens={MaxTokens} imageAttachments="
                           "{ImageCount} uploads={Uploads} sampling(temp={Temperature},topK={TopK},topP={TopP},seed={Seed}) "
                           "prompt=\"{Prompt}\"", Architecture=arch, MaxTokens=max_tokens, ImageCount=len(image_paths or []),
                           Uploads=serialize_uploads_for_log(messages[0]), Temperature=cfg.temperature, TopK=cfg.top_k,
                           TopP=cfg.top_p, Seed=cfg.seed, Prompt=sanitize_for_log(prompt))
            prepared = prepare_history_for_inference(messages, arch, self._log)
            tokens = self._kv_renderer.render_to_tokens(self._model.tokenizer, self._model.cfg.chat_template, prepared, arch,
                                                        add_generation_prompt=True)
            mm = self._mm()
            if mm is not None:
                tokens = mm.process_prompt_tokens(prepared, tokens)
            tokens = self._truncate_prompt_to_context(active, tokens, max_tokens)
            self.reset_session(active)
            t0 = time.perf_counter_ns()
            queued = self._mm_queue(0)
            state = {"generated": []}
            with self._exchange_guard():
                logits = self._forward_prompt_prefill(list(tokens), allow_chunking=not queued)
                active.kv_cache.record_append(list(tokens), logits)
                prompt_ns = time.perf_counter_ns() - t0
                yield from self._token_loop(active, logits, max_tokens, cfg, cancel, True, state)
            total_ns = time.perf_counter_ns() - t0
            generated = state["generated"]
            text = bytes(state.get("raw", b"")).decode("utf-8", errors="replace")
            eval_s = state.get("eval_ns", 0) / 1e9
            if state.get("cancelled"):
                self._log.warning(Ev.ChatAborted, "generate.cancelled tokens={Tokens} promptTokens={PromptTokens} elapsedMs="
                                  "{ElapsedMs:.1f} completion=\"{Completion}\"", Tokens=len(generated), PromptTokens=len(tokens),
                                  ElapsedMs=total_ns / 1e6, Completion=sanitize_for_log(text))
            else:
                self._log.info(Ev.ChatCompleted, "generate.complete tokens={Tokens} promptTokens={PromptTokens} elapsedMs="
                               "{ElapsedMs:.1f} tokensPerSec={TokensPerSec:.2f} finishReason={FinishReason} completion="
                               "\"{Completion}\"", Tokens=len(generated), PromptTokens=len(tokens), ElapsedMs=total_ns / 1e6,
                               TokensPerSec=(len(generated) / eval_s if eval_s > 0 and generated else 0.0),
                               FinishReason=state["finish"], Completion=sanitize_for_log(text))
            METRICS.record_generation(len(tokens), len(generated), 0, prompt_ns, state.get("eval_ns", 0), bool(state.get("cancelled")))
            yield StreamItem("", True, len(tokens), len(generated), 0, total_ns, prompt_ns, state.get("eval_ns", 0))

    # ------------------------------------------------------------------ misc
    @staticmethod
    def _is_mmproj(name: str) -> bool:
        return "mmproj" in name.lower()

    def scan_models(self, directory: str) -> List[str]:
        if not os.path.isdir(directory):
            return []
        return sorted(f for f in os.listdir(directory) if f.endswith(".gguf") and not self._is_mmproj(f))

    def scan_mmproj_models(self, directory: str) -> List[str]:
        if not os.path.isdir(directory):
            return []
        return sorted(f for f in os.listdir(directory) if f.endswith(".gguf") and self._is_mmproj(f))

    def close(self) -> None:
        if self._model is not None:
            self._model.close()
        self._model = None
        self._active = None
        self._resident.clear()
        self._intrinsic.dispose()
