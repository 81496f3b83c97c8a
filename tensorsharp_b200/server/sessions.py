"""Chat sessions: each owns the token-level KV bookkeeping and the tracked history of one chat.

Parity: TensorSharp.Server/ChatSession.cs:23-68, SessionManager.cs:21-105 (default session
``__default__`` that cannot be removed, ids are 32 hex digits).  ``seq`` is this build's
addition: the session's sequence in the paged KV pool, so that with ``max_seqs > 1`` several
sessions stay resident on the device and switching between them forwards nothing.
"""
from __future__ import annotations

import datetime as _dt
import threading
import uuid
from typing import Dict, List, Optional

from ..runtime.chat import ChatMessage
from ..runtime.kv_cache import KVCache
from ..runtime.logging import Ev, NULL_LOGGER

DEFAULT_SESSION_ID = "__default__"


def _utcnow() -> _dt.datetime:
    return _dt.datetime.now(_dt.timezone.utc)


def iso_o(t: _dt.datetime) -> str:
    """.NET's round-trip ("o") format for a UTC time: seven fractional digits and ``Z``."""
    t = t.astimezone(_dt.timezone.utc)
    return t.strftime("%Y-%m-%dT%H:%M:%S.") + "%06d0Z" % t.microsecond


class ChatSession:
    def __init__(self, session_id: Optional[str] = None):
        if session_id is not None and not session_id.strip():
            raise ValueError("Session id cannot be null or empty.")
        self.id = session_id or uuid.uuid4().hex
        self.kv_cache = KVCache()
        self.tracked_history: List[ChatMessage] = []
        self.created_at = _utcnow()
        self.last_used_at = self.created_at
        self.is_disposed = False
        self.seq = None                     # paged-KV sequence while resident on the device

    def dispose(self) -> None:
        if self.is_disposed:
            return
        self.is_disposed = True
        self.tracked_history.clear()
        self.kv_cache.reset()


class SessionManager:
    def __init__(self, logger=None):
        self._log = logger or NULL_LOGGER
        self._lock = threading.Lock()
        self._sessions: Dict[str, ChatSession] = {DEFAULT_SESSION_ID: ChatSession(DEFAULT_SESSION_ID)}

    @property
    def default_session(self) -> ChatSession:
        return self._sessions[DEFAULT_SESSION_ID]

    @property
    def session_ids(self) -> List[str]:
        with self._lock:
            return list(self._sessions)

    @property
    def session_count(self) -> int:
        return len(self._sessions)

    def create_session(self) -> ChatSession:
        with self._lock:
            while True:
                s = ChatSession()
                if s.id not in self._sessions:
                    self._sessions[s.id] = s
                    break
        self._log.info(Ev.SessionCreated, "Created chat session {SessionId} (total sessions={SessionCount})",
                       SessionId=s.id, SessionCount=len(self._sessions))
        return s

    def get_session(self, session_id: Optional[str]) -> Optional[ChatSession]:
        if session_id is None or not session_id.strip():
            return self.default_session
        return self._sessions.get(session_id)

    def try_remove(self, session_id: Optional[str]) -> Optional[ChatSession]:
        if session_id is None or not session_id.strip():
            return None
        if session_id == DEFAULT_SESSION_ID:
            self._log.warning(Ev.SessionRemoved, "Refusing to remove default session {SessionId}", SessionId=session_id)
            return None
        with self._lock:
            s = self._sessions.pop(session_id, None)
        if s is not None:
            self._log.info(Ev.SessionRemoved, "Removed chat session {SessionId} (remaining sessions={SessionCount})",
                           SessionId=session_id, SessionCount=len(self._sessions))
        return s
