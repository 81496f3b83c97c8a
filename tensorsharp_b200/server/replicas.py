"""Data-parallel serving: N copies of the server, one per GPU, behind one address.

``python -m tensorsharp_b200.server --model m.gguf --replicas N --port 5000`` starts N ordinary server
processes (replica ``i`` sees GPU ``i`` only and listens on a private loopback port) and a small front end on
the public port that hands each request to a replica:

* a request that names a web-UI chat session goes to the replica that owns the session (its KV cache is there);
  new sessions are opened on the least busy replica;
* any other generation request goes to the replica with the fewest requests in flight;
* ``GET /api/queue/status`` and ``GET /metrics`` are gathered from all replicas (status summed, metrics labelled
  ``replica="i"``); ``POST /api/models/load`` is sent to every replica; everything else is answered by replica 0.

Responses are passed through as they arrive (streams stay streams); when the client hangs up the upstream
connection is closed, which cancels the generation on the replica.  One process per GPU keeps every replica's
CUDA context, graphs and allocator to itself.  The reference has no counterpart: it serves one request at a
time from one process (TensorSharp.Server/InferenceQueue.cs).
"""
from __future__ import annotations

import http.client
import json
import os
import re
import subprocess
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional, Sequence, Tuple

GENERATION_PATHS = ("/api/generate", "/api/chat/ollama", "/v1/chat/completions", "/api/chat")
PASS_HEADERS = ("content-type", "cache-control", "x-tensorsharp-request-id")


class Replica:
    def __init__(self, index: int, host: str, port: int, process: Optional[subprocess.Popen] = None):
        self.index, self.host, self.port, self.process = index, host, port, process
        self.in_flight = 0
        self.served = 0
        self.down_until = 0.0             # monotonic time until which the router avoids this replica
        self.restarts = 0
        self.launch = None                # () -> Popen: how to start this replica's process again

    @property
    def up(self) -> bool:
        return time.monotonic() >= self.down_until

    def mark_down(self, seconds: float = 5.0) -> None:
        self.down_until = time.monotonic() + seconds

    def connect(self, timeout: float = 600.0) -> http.client.HTTPConnection:
        return http.client.HTTPConnection(self.host, self.port, timeout=timeout)

    def get_json(self, path: str, timeout: float = 10.0):
        c = self.connect(timeout)
        try:
            c.request("GET", path)
            r = c.getresponse()
            return r.status, json.loads(r.read() or b"null")
        finally:
            c.close()

    def get_text(self, path: str, timeout: float = 10.0) -> Tuple[int, str]:
        c = self.connect(timeout)
        try:
            c.request("GET", path)
            r = c.getresponse()
            return r.status, r.read().decode("utf-8", "replace")
        finally:
            c.close()


class Router:
    """Which replica serves a request (thread-safe)."""

    def __init__(self, replicas: Sequence[Replica]):
        self.replicas = list(replicas)
        self._lock = threading.Lock()
        self._session_owner: Dict[str, int] = {}
        self._rr = 0

    def _least_busy(self) -> Replica:
        n = len(self.replicas)
        best = min(range(n), key=lambda i: (not self.replicas[i].up, self.replicas[i].in_flight, (i - self._rr) % n))
        self._rr = (best + 1) % n
        return self.replicas[best]

    def pick(self, method: str, path: str, body: bytes) -> Replica:
        sid = None
        if method == "DELETE" and path.startswith("/api/sessions/"):
            sid = path[len("/api/sessions/"):]
        elif method == "POST" and path.rstrip("/") == "/api/chat" and body:
            try:
                obj = json.loads(body)
                sid = obj.get("sessionId") if isinstance(obj, dict) else None
            except ValueError:
                sid = None
        with self._lock:
            if isinstance(sid, str) and sid in self._session_owner:
                r = self.replicas[self._session_owner[sid]]
            elif method == "POST" and (path.rstrip("/") in GENERATION_PATHS or path.rstrip("/") == "/api/sessions"):
                r = self._least_busy()
            else:
                r = next((x for x in self.replicas if x.up), self.replicas[0])
            r.in_flight += 1
            return r

    def another(self, failed: Replica) -> Optional[Replica]:
        """A different replica that is up, for one more try of a request that is not tied to a session."""
        with self._lock:
            rest = [x for x in self.replicas if x is not failed and x.up]
            if not rest:
                return None
            r = min(rest, key=lambda x: x.in_flight)
            r.in_flight += 1
            return r

    def done(self, r: Replica) -> None:
        with self._lock:
            r.in_flight = max(0, r.in_flight - 1)
            r.served += 1

    def bind_session(self, sid: str, r: Replica) -> None:
        with self._lock:
            self._session_owner[sid] = r.index

    def drop_session(self, sid: str) -> None:
        with self._lock:
            self._session_owner.pop(sid, None)

    def forget_sessions_of(self, r: Replica) -> None:
        with self._lock:
            for sid in [k for k, v in self._session_owner.items() if v == r.index]:
                del self._session_owner[sid]

    def owner(self, sid: str) -> int:
        with self._lock:
            return self._session_owner.get(sid, -1)


_SAMPLE = re.compile(r"^([A-Za-z_:][A-Za-z0-9_:]*)(\{[^}]*\})?\s+(\S+)\s*$")


def merge_metrics(texts: Sequence[str]) -> str:
    """Prometheus text of every replica in one exposition: HELP / TYPE lines once, samples labelled ``replica="i"``."""
    meta: List[str] = []
    seen_meta = set()
    samples: List[str] = []
    for i, text in enumerate(texts):
        for line in text.splitlines():
            if not line.strip():
                continue
            if line.startswith("#"):
                if line not in seen_meta:
                    seen_meta.add(line)
                    meta.append(line)
                continue
            m = _SAMPLE.match(line)
            if not m:
                continue
            name, labels, value = m.group(1), m.group(2), m.group(3)
            inner = labels[1:-1].strip() if labels else ""
            inner = f'{inner},replica="{i}"' if inner else f'replica="{i}"'
            samples.append(f"{name}{{{inner}}} {value}")
    # keep each metric's samples under its own HELP / TYPE block
    out: List[str] = []
    by_name: Dict[str, List[str]] = {}
    for s in samples:
        by_name.setdefault(_SAMPLE.match(s).group(1), []).append(s)
    emitted = set()
    for line in meta:
        out.append(line)
        parts = line.split()
        if len(parts) >= 3 and parts[1] == "TYPE":
            out.extend(by_name.get(parts[2], []))
            emitted.add(parts[2])
    for name, rows in by_name.items():
        if name not in emitted:
            out.extend(rows)
    return "\n".join(out) + "\n"


def merged_status(replicas: Sequence[Replica]) -> Dict[str, object]:
    rows = []
    for r in replicas:
        try:
            st, q = r.get_json("/api/queue/status")
            q = q if st == 200 and isinstance(q, dict) else {}
        except (OSError, ValueError, http.client.HTTPException):
            q = {"unreachable": True}
        rows.append({"replica": r.index, "in_flight": r.in_flight, "up": r.up and not q.get("unreachable", False),
                     "restarts": r.restarts, **q})
    return {"busy": any(x.get("busy") for x in rows),
            "pending_requests": sum(int(x.get("pending_requests", 0) or 0) for x in rows),
            "total_processed": sum(int(x.get("total_processed", 0) or 0) for x in rows),
            "replicas": rows}


def make_front_handler(router: Router):
    class Front(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):
            pass

        def _send(self, status: int, ctype: str, data: bytes) -> None:
            self.send_response(status)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def _relay(self) -> None:
            n = int(self.headers.get("Content-Length") or 0)
            body = self.rfile.read(n) if n > 0 else b""
            path = self.path.split("?", 1)[0]
            if self.command == "GET" and path.rstrip("/") == "/api/queue/status":
                return self._send(200, "application/json", json.dumps(merged_status(router.replicas)).encode())
            if self.command == "GET" and path.rstrip("/") == "/metrics":
                texts = []
                for r in router.replicas:
                    try:
                        texts.append(r.get_text("/metrics")[1])
                    except (OSError, http.client.HTTPException):
                        texts.append("")
                return self._send(200, "text/plain; version=0.0.4; charset=utf-8", merge_metrics(texts).encode())
            if self.command == "POST" and path.rstrip("/") == "/api/models/load":
                return self._broadcast(path, body)
            replica = router.pick(self.command, path, body)
            try:
                reached = self._forward(replica, path, body)
            finally:
                router.done(replica)
            if reached is False:
                # nothing was sent to the client yet: a request that no session ties to the dead replica goes to another
                replica.mark_down()
                sticky = path.startswith("/api/sessions/") or (path.rstrip("/") == "/api/chat" and b'"sessionId"' in body)
                other = None if sticky else router.another(replica)
                if other is None:
                    return self._send(502, "application/json", json.dumps({"error": f"replica {replica.index} is not reachable"}).encode())
                try:
                    if self._forward(other, path, body) is False:
                        other.mark_down()
                        self._send(502, "application/json", json.dumps({"error": "no replica is reachable"}).encode())
                finally:
                    router.done(other)

        def _headers_out(self) -> Dict[str, str]:
            keep = ("content-type", "x-tensorsharp-request-id", "accept", "authorization")
            return {k: v for k, v in self.headers.items() if k.lower() in keep}

        def _broadcast(self, path: str, body: bytes) -> None:
            first = None
            for r in router.replicas:
                c = r.connect()
                try:
                    c.request("POST", path, body, self._headers_out())
                    resp = c.getresponse()
                    got = (resp.status, resp.getheader("Content-Type") or "application/json", resp.read())
                finally:
                    c.close()
                if first is None or (got[0] >= 400 and first[0] < 400):
                    first = got                      # the first failure wins, else replica 0's answer
            self._send(*first)

        def _forward(self, replica: Replica, path: str, body: bytes) -> Optional[bool]:
            """Relay to ``replica``; False when it could not be reached (and nothing has been sent to the client)."""
            up = replica.connect()
            try:
                try:
                    up.request(self.command, self.path, body if body else None, self._headers_out())
                    resp = up.getresponse()
                except (OSError, http.client.HTTPException):
                    return False
                streamed = (resp.getheader("Transfer-Encoding") or "").lower() == "chunked"
                self.send_response(resp.status)
                for k, v in resp.getheaders():
                    if k.lower() in PASS_HEADERS:
                        self.send_header(k, v)
                if not streamed:
                    data = resp.read()
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    self.wfile.write(data)
                    self._track_session(replica, path, resp.status, data)
                    return
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()
                try:
                    while True:
                        piece = resp.read1(65536)
                        if not piece:
                            break
                        self.wfile.write(b"%x\r\n" % len(piece) + piece + b"\r\n")
                        self.wfile.flush()
                    self.wfile.write(b"0\r\n\r\n")
                    self.wfile.flush()
                except (BrokenPipeError, ConnectionResetError, TimeoutError):
                    self.close_connection = True     # the client left: closing ``up`` below cancels the generation
            finally:
                up.close()

        def _track_session(self, replica: Replica, path: str, status: int, data: bytes) -> None:
            p = path.rstrip("/")
            if self.command == "POST" and p == "/api/sessions" and status == 200:
                try:
                    sid = json.loads(data).get("sessionId")
                except (ValueError, AttributeError):
                    sid = None
                if isinstance(sid, str):
                    router.bind_session(sid, replica)
            elif self.command == "DELETE" and p.startswith("/api/sessions/"):
                router.drop_session(p[len("/api/sessions/"):])

        do_GET = do_POST = do_DELETE = do_PUT = _relay

    return Front


class FrontServer(ThreadingHTTPServer):
    daemon_threads = True
    allow_reuse_address = True
    request_queue_size = 128


def serve_front(router: Router, host: str, port: int) -> FrontServer:
    return FrontServer((host, port), make_front_handler(router))


# ---------------------------------------------------------------------------------------------------
# starting and stopping the replica processes

def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def replica_argv(argv: Sequence[str], port: int) -> List[str]:
    """The front end's own arguments for one replica: no ``--replicas``, loopback host, private port."""
    out: List[str] = []
    skip = False
    for a in argv:
        if skip:
            skip = False
            continue
        name = a.split("=", 1)[0]
        if name in ("--replicas", "--port", "--host"):
            skip = "=" not in a
            continue
        out.append(a)
    return out + ["--host", "127.0.0.1", "--port", str(port)]


def replica_env(base, gpu: Optional[str]) -> Dict[str, str]:
    """The environment of one replica process: a plain single-process server (no rank variables, no replica count of
    its own, which would make it start replicas in turn) that sees ``gpu`` only."""
    env = dict(base)
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK", "TENSORSHARP_REPLICAS"):
        env.pop(k, None)
    if gpu is not None:
        env["CUDA_VISIBLE_DEVICES"] = gpu
    return env


def spawn_replicas(argv: Sequence[str], n: int, *, use_gpus: bool, ready_timeout_s: float = 600.0,
                   log_dir: Optional[str] = None) -> List[Replica]:
    """Start ``n`` server processes and wait until each answers ``GET /api/version``.  With ``use_gpus`` replica ``i``
    is given GPU ``i`` of the GPUs this process may see (``CUDA_VISIBLE_DEVICES`` is narrowed, never widened)."""
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    gpu_ids = [x for x in visible.split(",") if x.strip()] if visible else [str(i) for i in range(n)]
    if use_gpus and len(gpu_ids) < n:
        raise ValueError(f"--replicas {n} needs {n} GPUs, {len(gpu_ids)} visible")
    replicas: List[Replica] = []
    try:
        for i in range(n):
            port = _free_port()
            env = replica_env(os.environ, gpu_ids[i] if use_gpus else None)
            def launch(i=i, port=port, env=env):
                out = open(os.path.join(log_dir, f"replica-{i}.log"), "ab") if log_dir else subprocess.DEVNULL
                return subprocess.Popen([sys.executable, "-m", "tensorsharp_b200.server", *replica_argv(argv, port)], env=env,
                                        stdout=out, stderr=subprocess.STDOUT)
            r = Replica(i, "127.0.0.1", port, launch())
            r.launch = launch
            replicas.append(r)
        deadline = time.monotonic() + ready_timeout_s
        for r in replicas:
            while True:
                if r.process.poll() is not None:
                    raise RuntimeError(f"replica {r.index} exited with code {r.process.returncode} before it was ready")
                try:
                    if r.get_json("/api/version", timeout=2.0)[0] == 200:
                        break
                except (OSError, ValueError, http.client.HTTPException):
                    pass
                if time.monotonic() > deadline:
                    raise TimeoutError(f"replica {r.index} did not answer within {ready_timeout_s:.0f} s")
                time.sleep(0.2)
        return replicas
    except BaseException:
        stop_replicas(replicas)
        raise


class Supervisor:
    """Restarts replica processes that exited (a crash, an out-of-memory kill): checks once a second, keeps the replica
    out of the rotation until it answers again.  Sessions that lived on it are gone (their caches were its memory); the
    front end then opens them anew on whichever replica the next request reaches."""

    def __init__(self, router: "Router", poll_s: float = 1.0, ready_timeout_s: float = 600.0):
        self.router, self.poll_s, self.ready_timeout_s = router, poll_s, ready_timeout_s
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="tsb-replica-supervisor", daemon=True)

    def start(self) -> "Supervisor":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=5)

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            for r in self.router.replicas:
                if r.process is None or r.launch is None or r.process.poll() is None:
                    continue
                if time.monotonic() < getattr(r, "next_restart", 0.0):
                    continue                         # it died again right after the last restart: wait before the next try
                r.next_restart = time.monotonic() + min(60.0, 2.0 ** min(r.restarts, 6))
                r.mark_down(self.ready_timeout_s)
                self.router.forget_sessions_of(r)
                r.process = r.launch()
                r.restarts += 1
                deadline = time.monotonic() + self.ready_timeout_s
                while not self._stop.is_set() and time.monotonic() < deadline and r.process.poll() is None:
                    try:
                        if r.get_json("/api/version", timeout=2.0)[0] == 200:
                            r.down_until = 0.0
                            break
                    except (OSError, ValueError, http.client.HTTPException):
                        pass
                    time.sleep(0.2)


def stop_replicas(replicas: Sequence[Replica], grace_s: float = 10.0) -> None:
    """Ask every replica process that this module started to end (SIGTERM to its own pid), then make sure."""
    for r in replicas:
        if r.process is not None and r.process.poll() is None:
            r.process.terminate()
    end = time.monotonic() + grace_s
    for r in replicas:
        if r.process is None:
            continue
        try:
            r.process.wait(max(0.1, end - time.monotonic()))
        except subprocess.TimeoutExpired:
            r.process.kill()
            r.process.wait(5)
