"""Structured JSONL logging with a background writer.

Schema and behaviour follow TensorSharp.Runtime/Logging: one JSON object per line with
``ts, level, category, event{id,name}, message, exception, template, props, scope``
(LogEntryFormatter.cs), files ``{prefix}-yyyyMMdd[-NNNN].jsonl`` rotated daily (UTC) and at
25 MB, a bounded queue of 16384 entries that drops the oldest when full, a 500 ms flush
interval (FileLoggerOptions.cs:27-68, FileLoggerProvider.cs), the event ids of
LogEventIds.cs and the scope keys of LogScopes.cs.
"""
from __future__ import annotations

import collections
import contextlib
import contextvars
import datetime as _dt
import json
import os
import threading
import traceback
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

LEVELS = {"Trace": 0, "Debug": 1, "Information": 2, "Warning": 3, "Error": 4, "Critical": 5, "None": 6}


class Ev:
    """(id, name) pairs of every event the engine emits."""
    HostStarting = (1000, "HostStarting")
    HostStarted = (1001, "HostStarted")
    HostStopping = (1002, "HostStopping")
    HostStopped = (1003, "HostStopped")
    HostConfiguration = (1010, "HostConfiguration")
    BackendDetected = (1020, "BackendDetected")
    BackendUnavailable = (1021, "BackendUnavailable")
    LoggingInitialized = (1030, "LoggingInitialized")
    HttpRequestStarted = (1100, "HttpRequestStarted")
    HttpRequestCompleted = (1101, "HttpRequestCompleted")
    HttpRequestFailed = (1102, "HttpRequestFailed")
    HttpRequestRejected = (1103, "HttpRequestRejected")
    QueueEnqueued = (1200, "QueueEnqueued")
    QueueReady = (1201, "QueueReady")
    QueueReleased = (1202, "QueueReleased")
    QueueCancelled = (1203, "QueueCancelled")
    SessionCreated = (1300, "SessionCreated")
    SessionRemoved = (1301, "SessionRemoved")
    SessionReset = (1302, "SessionReset")
    SessionDisposed = (1303, "SessionDisposed")
    SessionActivated = (1304, "SessionActivated")
    ModelLoadStarted = (1400, "ModelLoadStarted")
    ModelLoadCompleted = (1401, "ModelLoadCompleted")
    ModelLoadFailed = (1402, "ModelLoadFailed")
    ModelUnloaded = (1403, "ModelUnloaded")
    ChatStarted = (1500, "ChatStarted")
    ChatCompleted = (1501, "ChatCompleted")
    ChatFailed = (1502, "ChatFailed")
    ChatAborted = (1503, "ChatAborted")
    KvCacheReusePlan = (1510, "KvCacheReusePlan")
    PromptChunking = (1511, "PromptChunking")
    PromptTruncated = (1512, "PromptTruncated")
    VideoFrameDownsample = (1513, "VideoFrameDownsample")
    GenerationProgress = (1520, "GenerationProgress")
    UploadReceived = (1600, "UploadReceived")
    UploadRejected = (1601, "UploadRejected")
    CliStarted = (1700, "CliStarted")
    CliCompleted = (1701, "CliCompleted")
    CliFailed = (1702, "CliFailed")
    CliBenchmark = (1710, "CliBenchmark")
    CliBatchProgress = (1711, "CliBatchProgress")


SCOPE_KEYS = ("RequestId", "Operation", "SessionId", "Model", "Backend", "Client", "CorrelationId")
_scope: contextvars.ContextVar = contextvars.ContextVar("tsb_log_scope", default=())


@contextlib.contextmanager
def log_scope(**kv):
    """Attach key/value pairs (see SCOPE_KEYS) to every entry logged inside the block."""
    tok = _scope.set(_scope.get() + tuple(kv.items()))
    try:
        yield
    finally:
        _scope.reset(tok)


@dataclass
class FileLoggerOptions:
    directory: str = "logs"
    file_prefix: str = "tensorsharp"
    minimum_level: str = "Information"
    max_file_size_bytes: int = 25 * 1024 * 1024
    max_queued_entries: int = 16 * 1024
    flush_interval_s: float = 0.5
    use_json_format: bool = True
    include_scopes: bool = True


def format_entry(ts: _dt.datetime, level: str, category: str, event: Optional[Tuple[int, str]], message: str,
                 exception: Optional[str], template: Optional[str], props: Dict[str, Any], scopes, include_scopes=True) -> str:
    d: Dict[str, Any] = {"ts": ts.astimezone(_dt.timezone.utc).strftime("%Y-%m-%dT%H:%M:%S.%f") + "0Z",
                         "level": level, "category": category}
    if event is not None and (event[0] != 0 or event[1]):
        d["event"] = {"id": event[0], "name": event[1]} if event[1] else {"id": event[0]}
    d["message"] = message or ""
    if exception:
        d["exception"] = exception
    if template is not None:
        d["template"] = template
    if props:
        d["props"] = props
    if include_scopes and scopes:
        d["scope"] = dict(scopes)
    return json.dumps(d, ensure_ascii=False, default=str)


_LABEL = {"Trace": "TRC", "Debug": "DBG", "Information": "INF", "Warning": "WRN", "Error": "ERR", "Critical": "CRT"}


def format_text_line(ts: _dt.datetime, level: str, category: str, event: Optional[Tuple[int, str]], message: str,
                     exception: Optional[str], scopes, include_scopes=True) -> str:
    """The plain-text alternative (LogEntryFormatter.cs ToTextLine):
    ``2026-01-01T00:00:00.000Z INF [1500:ChatStarted] Category: message => Key=value``."""
    t = ts.astimezone(_dt.timezone.utc)
    out = [t.strftime("%Y-%m-%dT%H:%M:%S.") + "%03dZ" % (t.microsecond // 1000), " ", _LABEL.get(level, "NON"), " "]
    if event is not None and event[0] != 0:
        out.append(f"[{event[0]}:{event[1]}] " if event[1] else f"[{event[0]}] ")
    out += [category, ": ", message or ""]
    if include_scopes and scopes:
        out.append(" =>" + "".join(f" {k}={v}" for k, v in scopes))
    if exception:
        out.append("\n    " + exception)
    return "".join(out)


class FileLoggerProvider:
    """Owns the writer thread and the current log file."""

    def __init__(self, options: Optional[FileLoggerOptions] = None, clock=None):
        self.options = options or FileLoggerOptions()
        self._clock = clock or (lambda: _dt.datetime.now(_dt.timezone.utc))
        self._q: collections.deque = collections.deque()
        self._cv = threading.Condition()
        self.dropped = 0
        self._stop = False
        self._file = None
        self._file_path: Optional[str] = None
        self._date = None
        self._suffix = 0
        os.makedirs(self.options.directory, exist_ok=True)
        self._thread = threading.Thread(target=self._run, name="tsb-log-writer", daemon=True)
        self._thread.start()

    # -------------------------------------------------------------- producer side
    def get_logger(self, category: str) -> "Logger":
        return Logger(self, category)

    def enqueue(self, line: str) -> None:
        with self._cv:
            if len(self._q) >= self.options.max_queued_entries:
                self._q.popleft()            # drop the oldest entry: never block the request path
                self.dropped += 1
            self._q.append(line)
            self._cv.notify()

    # -------------------------------------------------------------- writer side
    def _path_for(self, date, suffix) -> str:
        sfx = "" if suffix == 0 else f"-{suffix:04d}"
        return os.path.join(self.options.directory, f"{self.options.file_prefix}-{date:%Y%m%d}{sfx}.jsonl")

    def _ensure_file(self) -> None:
        today = self._clock().date()
        if self._file is not None and today == self._date and self._file.tell() < self.options.max_file_size_bytes:
            return
        if self._file is not None:
            self._file.close()
            self._file = None
            if today != self._date:
                self._suffix = 0
            else:
                self._suffix += 1
        elif today != self._date:
            self._suffix = 0
        self._date = today
        path = self._path_for(today, self._suffix)
        while os.path.exists(path) and os.path.getsize(path) >= self.options.max_file_size_bytes:
            self._suffix += 1
            path = self._path_for(today, self._suffix)
        self._file_path = path
        self._file = open(path, "a", encoding="utf-8")

    def _drain(self) -> None:
        while True:
            with self._cv:
                if not self._q:
                    break
                batch = list(self._q)
                self._q.clear()
            for line in batch:
                self._ensure_file()
                self._file.write(line + "\n")
            if self._file is not None:
                self._file.flush()

    def _run(self) -> None:
        while True:
            with self._cv:
                if not self._q and not self._stop:
                    self._cv.wait(self.options.flush_interval_s)
                stop = self._stop
            try:
                self._drain()
            except OSError:
                pass
            if stop:
                return

    def flush(self) -> None:
        self._drain()

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify()
        self._thread.join(timeout=5)
        self._drain()
        if self._file is not None:
            self._file.close()
            self._file = None

    @property
    def current_file(self) -> Optional[str]:
        return self._file_path


class Logger:
    def __init__(self, provider: Optional[FileLoggerProvider], category: str):
        self.provider, self.category = provider, category

    def is_enabled(self, level: str) -> bool:
        return self.provider is not None and LEVELS[level] >= LEVELS[self.provider.options.minimum_level]

    def log(self, level: str, event: Optional[Tuple[int, str]], template: str, exc: Optional[BaseException] = None, **props):
        if not self.is_enabled(level):
            return
        try:
            message = template.format(**props)
        except (KeyError, IndexError, ValueError):
            message = template
        exc_text = "".join(traceback.format_exception(type(exc), exc, exc.__traceback__)) if exc is not None else None
        o = self.provider.options
        if o.use_json_format:
            line = format_entry(self.provider._clock(), level, self.category, event, message, exc_text, template, props,
                                _scope.get(), o.include_scopes)
        else:
            line = format_text_line(self.provider._clock(), level, self.category, event, message, exc_text, _scope.get(),
                                    o.include_scopes)
        self.provider.enqueue(line)

    def info(self, event, template, **props):
        self.log("Information", event, template, **props)

    def warning(self, event, template, **props):
        self.log("Warning", event, template, **props)

    def error(self, event, template, exc=None, **props):
        self.log("Error", event, template, exc=exc, **props)

    def debug(self, event, template, **props):
        self.log("Debug", event, template, **props)


NULL_LOGGER = Logger(None, "null")


def setup_file_logging(directory: Optional[str] = None, level: Optional[str] = None, prefix: str = "tensorsharp",
                       enabled: bool = True) -> Optional[FileLoggerProvider]:
    """Create the provider from flags / environment (TENSORSHARP_LOG_DIR, TENSORSHARP_LOG_FILE=0
    disables the file, TENSORSHARP_LOG_LEVEL; TensorSharp.Server/Hosting/LoggingSetup.cs:28)."""
    env = os.environ
    if env.get("TENSORSHARP_LOG_FILE", "1").lower() in ("0", "false", "off", "no") or not enabled:
        return None
    lvl = (level or env.get("TENSORSHARP_LOG_LEVEL") or "Information").capitalize()
    lvl = {"Info": "Information", "Warn": "Warning"}.get(lvl, lvl)
    if lvl not in LEVELS:
        lvl = "Information"
    return FileLoggerProvider(FileLoggerOptions(directory=directory or env.get("TENSORSHARP_LOG_DIR") or "logs",
                                                file_prefix=prefix, minimum_level=lvl))
