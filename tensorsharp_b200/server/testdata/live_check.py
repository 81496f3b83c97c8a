#!/usr/bin/env python3
"""Checks a running server over HTTP: the three API styles, several turns with KV reuse, streaming framing,
structured outputs, thinking and tools, error answers, the queue and concurrent clients, a client that hangs up.

    python tensorsharp_b200/server/testdata/live_check.py --url http://127.0.0.1:5000 [--model NAME]
                                                          [--max-tokens 24] [--content-checks] [--only NAME,...]

Needs nothing but the standard library.  By default the checks are about the protocol (status codes, fields,
token accounting, framing) and hold for any model, random weights included; ``--content-checks`` adds the ones
that need a model able to follow instructions (valid JSON for a schema, a recalled fact).  Exit code 0 when no
check failed.  Plays the part of TensorSharp.Server/testdata/test_multiturn.py of the reference.
"""
from __future__ import annotations

import argparse
import http.client
import json
import sys
import threading
import time
import urllib.parse
from typing import Any, Callable, Dict, List, Optional, Tuple


class Client:
    """One connection per call; knows the three stream framings."""

    def __init__(self, url: str, timeout: float = 300.0):
        u = urllib.parse.urlparse(url if "//" in url else "http://" + url)
        self.host, self.port, self.timeout = u.hostname or "127.0.0.1", u.port or 80, timeout

    def _conn(self) -> http.client.HTTPConnection:
        return http.client.HTTPConnection(self.host, self.port, timeout=self.timeout)

    def request(self, method: str, path: str, body: Any = None, raw: Optional[bytes] = None) -> Tuple[int, Dict[str, str], str]:
        c = self._conn()
        try:
            data = raw if raw is not None else (json.dumps(body).encode() if body is not None else None)
            c.request(method, path, data, {"Content-Type": "application/json"} if data is not None else {})
            r = c.getresponse()
            return r.status, {k.lower(): v for k, v in r.getheaders()}, r.read().decode("utf-8", "replace")
        finally:
            c.close()

    def get_json(self, path: str):
        st, _, text = self.request("GET", path)
        return st, (json.loads(text) if text else None)

    def post_json(self, path: str, body: Any):
        st, _, text = self.request("POST", path, body)
        try:
            return st, json.loads(text)
        except ValueError:
            return st, {"_raw": text}

    def post_sse(self, path: str, body: Any):
        """Server-sent events: the ``data:`` payloads in order (JSON-decoded unless ``[DONE]``)."""
        st, hdr, text = self.request("POST", path, body)
        out: List[Any] = []
        for block in text.split("\n\n"):
            for line in block.splitlines():
                if line.startswith("data: "):
                    p = line[6:]
                    out.append(p if p == "[DONE]" else json.loads(p))
        return st, hdr, out, text

    def post_ndjson(self, path: str, body: Any):
        st, hdr, text = self.request("POST", path, body)
        items = []
        for line in text.splitlines():
            if line.strip():
                try:
                    items.append(json.loads(line))
                except ValueError:
                    items.append({"_raw": line})
        return st, hdr, items

    def post_and_hang_up(self, path: str, body: Any, after_bytes: int = 1) -> int:
        """Start a streaming request, read a little, close the socket; returns the number of bytes seen."""
        c = self._conn()
        c.request("POST", path, json.dumps(body).encode(), {"Content-Type": "application/json"})
        r = c.getresponse()
        got = len(r.read1(max(1, after_bytes)) if hasattr(r, "read1") else r.read(after_bytes))
        c.close()
        return got


class Report:
    def __init__(self, out=None):
        self.rows: List[Tuple[str, str, str]] = []            # (check, outcome, detail)
        self.out = out or sys.stdout
        self._group = ""

    def group(self, name: str) -> None:
        self._group = name
        print(f"\n== {name}", file=self.out, flush=True)

    def _add(self, outcome: str, what: str, detail: str = "") -> None:
        self.rows.append((f"{self._group}: {what}", outcome, detail))
        print(f"  [{outcome:4}] {what}" + (f"  ({detail})" if detail else ""), file=self.out, flush=True)

    def expect(self, cond: bool, what: str, detail: Any = "") -> bool:
        self._add("ok" if cond else "FAIL", what, "" if cond else str(detail)[:300])
        return bool(cond)

    def skip(self, what: str, why: str) -> None:
        self._add("skip", what, why)

    @property
    def failed(self) -> int:
        return sum(1 for _, o, _ in self.rows if o == "FAIL")

    def summary(self) -> str:
        n_ok = sum(1 for _, o, _ in self.rows if o == "ok")
        n_skip = sum(1 for _, o, _ in self.rows if o == "skip")
        return f"{n_ok} passed, {self.failed} failed, {n_skip} skipped"


class LiveCheck:
    def __init__(self, url: str, model: Optional[str] = None, max_tokens: int = 24, content_checks: bool = False, out=None):
        self.c = Client(url)
        self.model, self.max_tokens, self.content = model, max_tokens, content_checks
        self.r = Report(out)
        self.arch = ""

    # ------------------------------------------------------------------ discovery
    def check_discovery(self) -> None:
        r = self.r
        r.group("discovery")
        st, v = self.c.get_json("/api/version")
        r.expect(st == 200 and isinstance(v, dict) and v.get("version"), "GET /api/version names a version", v)
        st, tags = self.c.get_json("/api/tags")
        names = [m.get("name") for m in (tags or {}).get("models", [])] if st == 200 else []
        r.expect(st == 200 and names, "GET /api/tags lists hosted models", tags)
        st, models = self.c.get_json("/v1/models")
        r.expect(st == 200 and models.get("object") == "list" and models.get("data"), "GET /v1/models lists them the OpenAI way", models)
        st, ui = self.c.get_json("/api/models")
        r.expect(st == 200 and isinstance(ui, dict), "GET /api/models answers for the web UI", ui)
        if self.model is None and names:
            self.model = names[0]
        r.expect(bool(self.model), "a model to talk to", "none hosted and none given")
        if self.model:
            st, show = self.c.post_json("/api/show", {"model": self.model})
            r.expect(st == 200 and isinstance(show, dict), "POST /api/show describes it", show)
            info = show.get("model_info", {}) if isinstance(show, dict) else {}
            self.arch = str(info.get("general.architecture", "") or show.get("details", {}).get("family", ""))
        st, _, text = self.c.request("GET", "/")
        r.expect(st == 200 and text, "GET / serves the front page")
        if self.model and isinstance(ui, dict) and not ui.get("loaded"):
            # the web UI route talks to the loaded model only; load the hosted one as the page's model picker would
            st, a = self.c.post_json("/api/models/load", {"model": self.model, "backend": ui.get("defaultBackend")})
            r.expect(st == 200 and a.get("ok"), "POST /api/models/load loads the hosted model", (st, a))

    # ------------------------------------------------------------------ web UI style
    def check_webui_turns(self, turns: int = 3) -> None:
        r = self.r
        r.group("web UI chat, several turns in one session")
        st, s = self.c.post_json("/api/sessions", None)
        sid = s.get("sessionId") if st == 200 else None
        if not r.expect(bool(sid), "POST /api/sessions opens a session", s):
            return
        msgs: List[Dict[str, str]] = []
        prev_prompt = prev_count = 0
        for t in range(turns):
            msgs.append({"role": "user", "content": f"Turn {t + 1}: please say something short."})
            st, hdr, ev, _ = self.c.post_sse("/api/chat", {"sessionId": sid, "messages": msgs, "maxTokens": self.max_tokens})
            if not r.expect(st == 200 and ev and isinstance(ev[-1], dict) and ev[-1].get("done"), f"turn {t + 1} streams to a done event", ev[-1:] or st):
                return
            d = ev[-1]
            r.expect(hdr.get("content-type", "").startswith("text/event-stream"), f"turn {t + 1} is an event stream", hdr)
            r.expect(d.get("error") is None and d.get("sessionId") == sid, f"turn {t + 1} ends without error in the same session", d)
            r.expect(0 <= d.get("tokenCount", -1) <= self.max_tokens, f"turn {t + 1} respects maxTokens", d)
            if t > 0:
                r.expect(d.get("kvReusedTokens", 0) >= prev_prompt, f"turn {t + 1} re-uses the cache of turn {t} "
                         f"({d.get('kvReusedTokens')} of {d.get('promptTokens')} prompt tokens)", d)
            reply = "".join(e.get("token", "") for e in ev[:-1] if isinstance(e, dict))
            msgs.append({"role": "assistant", "content": reply})
            prev_prompt, prev_count = d.get("promptTokens", 0), d.get("tokenCount", 0)
        st, _, ev, _ = self.c.post_sse("/api/chat", {"sessionId": sid, "newChat": True, "maxTokens": 4,
                                                      "messages": [{"role": "user", "content": "Fresh start."}]})
        r.expect(st == 200 and ev and ev[-1].get("kvReusedTokens") == 0, "newChat drops the session's cache", ev[-1:] or st)
        st, _, _ = self.c.request("DELETE", f"/api/sessions/{sid}")
        r.expect(st in (200, 204), "DELETE /api/sessions/{id} closes it", st)
        st, _ = self.c.post_json("/api/chat", {"sessionId": sid, "messages": [{"role": "user", "content": "x"}]})
        r.expect(st == 404, "a closed session is unknown afterwards", st)

    # ------------------------------------------------------------------ Ollama style
    def check_ollama(self) -> None:
        r, m, n = self.r, self.model, self.max_tokens
        r.group("Ollama style: /api/generate and /api/chat/ollama")
        st, g = self.c.post_json("/api/generate", {"model": m, "prompt": "Hello.", "stream": False, "options": {"num_predict": n}})
        ok = r.expect(st == 200 and g.get("done") is True, "generate (one answer) completes", g)
        if ok:
            r.expect(0 <= g.get("eval_count", -1) <= n and g.get("prompt_eval_count", 0) > 0, "token counts are reported and bounded", g)
            r.expect(g.get("total_duration", 0) >= g.get("eval_duration", 0) >= 0 and g.get("prompt_eval_duration", -1) >= 0,
                     "durations are reported in nanoseconds and add up", g)
            r.expect(g.get("done_reason") in ("stop", "length"), "done_reason is stop or length", g.get("done_reason"))
        st, hdr, items = self.c.post_ndjson("/api/generate", {"model": m, "prompt": "Hello.", "options": {"num_predict": n}})
        r.expect(st == 200 and "ndjson" in hdr.get("content-type", ""), "generate streams newline-delimited JSON", hdr.get("content-type"))
        r.expect(bool(items) and items[-1].get("done") is True and all(not x.get("done") for x in items[:-1]),
                 "only the last line is marked done", items[-1:] or st)
        if ok and items and self.content:
            r.expect("".join(x.get("response", "") for x in items) == g.get("response"),
                     "streamed pieces join to the one-answer text (greedy server settings assumed)", "differs")
        msgs = [{"role": "system", "content": "You are terse."}, {"role": "user", "content": "My code word is heron. Remember it."}]
        st, a = self.c.post_json("/api/chat/ollama", {"model": m, "messages": msgs, "stream": False, "options": {"num_predict": n}})
        if r.expect(st == 200 and a.get("message", {}).get("role") == "assistant", "chat turn 1 answers as the assistant", a):
            msgs += [{"role": "assistant", "content": a["message"].get("content", "")}, {"role": "user", "content": "What was the code word?"}]
            st, b = self.c.post_json("/api/chat/ollama", {"model": m, "messages": msgs, "stream": False, "options": {"num_predict": n}})
            r.expect(st == 200 and b.get("prompt_cache_hit_tokens", 0) > 0, "chat turn 2 re-uses cached prompt tokens "
                     f"({b.get('prompt_cache_hit_tokens')} hit, ratio {b.get('prompt_cache_hit_ratio')})", b)
            if self.content:
                r.expect("heron" in b.get("message", {}).get("content", "").lower(), "turn 2 recalls the fact of turn 1", b.get("message"))
        st, hdr, items = self.c.post_ndjson("/api/chat/ollama", {"model": m, "messages": msgs[:2], "options": {"num_predict": n}})
        r.expect(st == 200 and items and items[-1].get("done") and "message" in items[0], "chat streams message pieces and a final record", items[-1:] or st)

    # ------------------------------------------------------------------ OpenAI style
    def check_openai(self) -> None:
        r, m, n = self.r, self.model, self.max_tokens
        r.group("OpenAI style: /v1/chat/completions")
        msgs = [{"role": "system", "content": "Answer briefly."}, {"role": "user", "content": "Name a colour."}]
        st, a = self.c.post_json("/v1/chat/completions", {"model": m, "messages": msgs, "max_tokens": n})
        if r.expect(st == 200 and a.get("object") == "chat.completion" and a.get("choices"), "a completion object comes back", a):
            u = a.get("usage", {})
            r.expect(u.get("total_tokens") == u.get("prompt_tokens", 0) + u.get("completion_tokens", 0) and u.get("completion_tokens", 99999) <= n,
                     "usage adds up and respects max_tokens", u)
            r.expect(a["choices"][0].get("finish_reason") in ("stop", "length"), "finish_reason is stop or length", a["choices"][0])
            msgs += [{"role": "assistant", "content": a["choices"][0]["message"].get("content") or ""}, {"role": "user", "content": "Another one."}]
        st, hdr, ev, _ = self.c.post_sse("/v1/chat/completions", {"model": m, "messages": msgs, "max_tokens": n, "stream": True})
        r.expect(st == 200 and ev and ev[-1] == "[DONE]", "the stream ends with [DONE]", ev[-1:] or st)
        chunks = [e for e in ev if isinstance(e, dict)]
        r.expect(bool(chunks) and all(c.get("object") == "chat.completion.chunk" for c in chunks), "every event is a chunk object", chunks[:1])
        if chunks:
            r.expect(chunks[-1]["choices"][0].get("finish_reason") in ("stop", "length"), "the last chunk carries the finish reason", chunks[-1])
            cached = (chunks[-1].get("usage") or {}).get("prompt_tokens_details", {}).get("cached_tokens", 0)
            r.expect(cached > 0, f"the second turn's usage reports cached prompt tokens ({cached})", chunks[-1].get("usage"))

    def check_structured(self) -> None:
        r, m = self.r, self.model
        r.group("structured outputs")
        schema = {"type": "object", "properties": {"city": {"type": "string"}, "population": {"type": "integer"}},
                  "required": ["city", "population"], "additionalProperties": False}
        base = {"model": m, "messages": [{"role": "user", "content": "Give a city and its population as JSON."}], "max_tokens": max(64, self.max_tokens)}
        for label, rf, keys in (("json_object", {"type": "json_object"}, None),
                                ("json_schema", {"type": "json_schema", "json_schema": {"name": "city", "strict": True, "schema": schema}}, ["city", "population"])):
            st, a = self.c.post_json("/v1/chat/completions", {**base, "response_format": rf})
            if st == 200:
                try:
                    obj = json.loads(a["choices"][0]["message"]["content"])
                    good = isinstance(obj, (dict, list)) and (keys is None or list(obj) == keys)
                except (ValueError, KeyError, TypeError):
                    good = False
                r.expect(good, f"{label}: the content is JSON in the requested shape", a)
            elif st == 422 and not self.content:
                r.expect(a.get("error", {}).get("type") == "invalid_response_error", f"{label}: a reply that is not valid JSON is refused with 422", a)
            else:
                r.expect(False, f"{label}: 200 with JSON" + ("" if self.content else " or 422"), (st, a))
        st, a = self.c.post_json("/v1/chat/completions", {**base, "think": True, "response_format": {"type": "json_object"}})
        r.expect(st == 400, "response_format with think=true is rejected", (st, a))
        bad = {"type": "json_schema", "json_schema": {"name": "x", "strict": True, "schema": {"anyOf": []}}}
        st, a = self.c.post_json("/v1/chat/completions", {**base, "response_format": bad})
        r.expect(st == 400, "an unsupported schema is rejected before any generation", (st, a))

    # ------------------------------------------------------------------ thinking and tools
    def check_thinking_and_tools(self) -> None:
        r, m, n = self.r, self.model, self.max_tokens
        r.group("thinking and tool calls")
        msgs = [{"role": "user", "content": "What is 17 + 25?"}]
        st, a = self.c.post_json("/api/chat/ollama", {"model": m, "messages": msgs, "think": True, "stream": False, "options": {"num_predict": n}})
        if r.expect(st == 200 and "message" in a, "think=true is accepted by the Ollama chat route", (st, a)):
            msg = a["message"]
            r.expect(isinstance(msg.get("content", ""), str) and isinstance(msg.get("thinking", ""), str),
                     "thinking (when the model has a thinking mode) is separate from the content", msg)
            if self.content:
                r.expect("42" in msg.get("content", "") + msg.get("thinking", ""), "the sum is right", msg)
        tools = [{"type": "function", "function": {"name": "get_weather", "description": "Current weather of a city",
                                                    "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}}]
        ask = [{"role": "user", "content": "What is the weather in Paris? Use the tool."}]
        st, a = self.c.post_json("/v1/chat/completions", {"model": m, "messages": ask, "tools": tools, "max_tokens": max(64, n)})
        if r.expect(st == 200 and a.get("choices"), "tools are accepted by the OpenAI route", (st, a)):
            ch = a["choices"][0]
            calls = ch["message"].get("tool_calls") or []
            r.expect(ch.get("finish_reason") in ("stop", "length", "tool_calls") and (bool(calls) == (ch.get("finish_reason") == "tool_calls")),
                     "finish_reason is tool_calls exactly when calls were parsed", ch)
            for tc in calls:
                args_ok = True
                try:
                    json.loads(tc["function"]["arguments"])
                except (ValueError, KeyError, TypeError):
                    args_ok = False
                r.expect(tc.get("type") == "function" and str(tc.get("id", "")).startswith("call_") and args_ok,
                         "a call has an id, a name and JSON arguments in a string", tc)
            if self.content:
                r.expect(bool(calls) and calls[0]["function"]["name"] == "get_weather", "the model called the tool", ch)
            if calls:
                follow = ask + [{"role": "assistant", "content": ch["message"].get("content") or "", "tool_calls": calls},
                                {"role": "tool", "tool_call_id": calls[0]["id"], "content": "{\"temp_c\": 21}"}]
                st, b = self.c.post_json("/v1/chat/completions", {"model": m, "messages": follow, "tools": tools, "max_tokens": n})
                r.expect(st == 200, "the tool's result can be sent back", (st, b))
        st, a = self.c.post_json("/api/chat/ollama", {"model": m, "messages": ask, "tools": tools, "stream": False, "options": {"num_predict": max(64, n)}})
        if r.expect(st == 200, "tools are accepted by the Ollama route", (st, a)):
            calls = a.get("message", {}).get("tool_calls") or []
            r.expect(all(isinstance(c.get("function", {}).get("arguments"), dict) for c in calls), "Ollama calls carry arguments as an object", calls)

    # ------------------------------------------------------------------ errors
    def check_errors(self) -> None:
        r, m = self.r, self.model
        r.group("error answers")
        for what, path, body, code in (
                ("generate without a model", "/api/generate", {"prompt": "x"}, 400),
                ("generate with an unknown model", "/api/generate", {"model": "no-such-model.gguf", "prompt": "x", "stream": False}, 404),
                ("Ollama chat without messages", "/api/chat/ollama", {"model": m}, 400),
                ("OpenAI chat without a model", "/v1/chat/completions", {"messages": []}, 400),
                ("OpenAI chat without messages", "/v1/chat/completions", {"model": m}, 400),
                ("OpenAI chat with an unknown model", "/v1/chat/completions", {"model": "no-such-model.gguf", "messages": []}, 404),
                ("web UI chat with an unknown session", "/api/chat", {"sessionId": "no-such-session", "messages": []}, 404)):
            st, a = self.c.post_json(path, body)
            r.expect(st == code, f"{what} -> {code}", (st, a))
        st, _, text = self.c.request("POST", "/v1/chat/completions", raw=b"{not json")
        r.expect(st == 400, "a body that is not JSON -> 400", (st, text[:120]))
        st, a = self.c.post_json("/v1/chat/completions", {"messages": []})
        r.expect(isinstance(a.get("error"), dict) and a["error"].get("type") == "invalid_request_error", "OpenAI errors use the error object", a)
        st, hdr, _ = self.c.request("GET", "/no-such-page")
        r.expect(st == 404 or (st == 200 and "html" in hdr.get("content-type", "")), "an unknown path falls back to the front page (or 404)", st)
        st, g = self.c.post_json("/api/generate", {"model": m, "prompt": "still alive?", "stream": False, "options": {"num_predict": 2}})
        r.expect(st == 200 and g.get("done"), "the server still answers after the bad requests", (st, g))

    # ------------------------------------------------------------------ queue, concurrent clients, a client that leaves
    def _queue(self) -> Dict[str, Any]:
        st, q = self.c.get_json("/api/queue/status")
        return q if st == 200 and isinstance(q, dict) else {}

    def _wait_idle(self, seconds: float = 60.0) -> Dict[str, Any]:
        end = time.monotonic() + seconds
        q = self._queue()
        while (q.get("busy") or q.get("pending_requests")) and time.monotonic() < end:
            time.sleep(0.1)
            q = self._queue()
        return q

    def check_queue_and_concurrency(self, clients: int = 4) -> None:
        r, m = self.r, self.model
        r.group("queue status, concurrent clients, a client that hangs up")
        q0 = self._wait_idle()
        r.expect({"busy", "pending_requests", "total_processed"} <= set(q0), "GET /api/queue/status has busy, pending_requests, total_processed", q0)
        results: List[Tuple[int, Any]] = []
        lock = threading.Lock()

        def one(i: int) -> None:
            out = self.c.post_json("/api/generate", {"model": m, "prompt": f"Client {i} says hello.", "stream": False,
                                                      "options": {"num_predict": min(8, self.max_tokens)}})
            with lock:
                results.append(out)
        th = [threading.Thread(target=one, args=(i,)) for i in range(clients)]
        [t.start() for t in th]
        [t.join(600) for t in th]
        r.expect(len(results) == clients and all(st == 200 and g.get("done") for st, g in results), f"{clients} clients at once are all answered",
                 [(st, g.get("error")) for st, g in results])
        q1 = self._wait_idle()
        r.expect(q1.get("total_processed", 0) >= q0.get("total_processed", 0) + clients and not q1.get("busy"),
                 f"the queue counted them ({q0.get('total_processed')} -> {q1.get('total_processed')}) and is idle again", q1)
        seen = self.c.post_and_hang_up("/api/generate", {"model": m, "prompt": "Count slowly to one hundred.", "options": {"num_predict": 512}})
        r.expect(seen > 0, "a stream was started and the client hung up in the middle")
        q2 = self._wait_idle(120.0)
        r.expect(not q2.get("busy") and not q2.get("pending_requests"), "the abandoned generation is cancelled: the queue drains", q2)
        st, g = self.c.post_json("/api/generate", {"model": m, "prompt": "next", "stream": False, "options": {"num_predict": 2}})
        r.expect(st == 200 and g.get("done"), "the next client is served", (st, g))
        st, _, text = self.c.request("GET", "/metrics")
        if st == 200:
            r.expect("# TYPE" in text and "_total" in text, "GET /metrics is in the Prometheus text format", text[:200])
        else:
            r.skip("GET /metrics", f"status {st}")

    # ------------------------------------------------------------------ driver
    CHECKS = ("discovery", "webui", "ollama", "openai", "structured", "thinking_tools", "errors", "queue")

    def run(self, only: Optional[List[str]] = None) -> int:
        table: Dict[str, Callable[[], None]] = {
            "discovery": self.check_discovery, "webui": self.check_webui_turns, "ollama": self.check_ollama, "openai": self.check_openai,
            "structured": self.check_structured, "thinking_tools": self.check_thinking_and_tools, "errors": self.check_errors,
            "queue": self.check_queue_and_concurrency}
        names = [n for n in self.CHECKS if not only or n in only or n == "discovery"]
        for name in names:
            try:
                table[name]()
            except Exception as e:                               # a check that cannot even talk to the server is a failure, not a crash
                self.r.expect(False, f"{name} ran to its end", f"{type(e).__name__}: {e}")
            if name == "discovery" and not self.model:
                break
        print(f"\n{self.r.summary()}", file=self.r.out, flush=True)
        return 1 if self.r.failed else 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Protocol checks against a running server")
    ap.add_argument("--url", default="http://127.0.0.1:5000")
    ap.add_argument("--model", default=None, help="hosted model name (default: the first one the server lists)")
    ap.add_argument("--max-tokens", type=int, default=24)
    ap.add_argument("--content-checks", action="store_true", help="also check what the model says (needs real weights)")
    ap.add_argument("--only", default="", help="comma-separated subset of: " + ", ".join(LiveCheck.CHECKS))
    a = ap.parse_args(argv)
    only = [x.strip() for x in a.only.split(",") if x.strip()]
    unknown = [x for x in only if x not in LiveCheck.CHECKS]
    if unknown:
        ap.error(f"unknown checks: {unknown}")
    return LiveCheck(a.url, a.model, a.max_tokens, a.content_checks).run(only or None)


if __name__ == "__main__":
    sys.exit(main())
