"""Host-side fault injection against the HTTP server: truncated and malformed bodies, a client that
disconnects in the middle of a stream, and a model file that fails to load.  After each fault the
queue must be free and the next request must succeed."""
import http.client
import json
import os
import socket
import threading
import time

import pytest

from tensorsharp_b200.server.app import ServerApp, serve
from tensorsharp_b200.server.options import build_options


@pytest.fixture()
def live(tmp_path, tiny_qwen3_path):
    opts = build_options(["--model", tiny_qwen3_path, "--backend", "cpu", "--port", "0", "--temperature", "0", "--top-k", "0",
                          "--top-p", "1", "--repeat-penalty", "1"], str(tmp_path), env={"TENSORSHARP_LOG_FILE": "0"})
    app = ServerApp(opts)
    httpd = serve(app, "127.0.0.1", 0)
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    yield app, httpd.server_address[1], os.path.basename(tiny_qwen3_path)
    httpd.shutdown()
    httpd.server_close()
    app.svc.close()


def _post(port, path, body, timeout=120):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=timeout)
    c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    return r.status, data


def _queue(port):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request("GET", "/api/queue/status")
    q = json.loads(c.getresponse().read())
    c.close()
    return q


def _wait_idle(port, seconds=30):
    t0 = time.time()
    while time.time() - t0 < seconds:
        q = _queue(port)
        if not q["busy"] and q["pending_requests"] == 0:
            return q
        time.sleep(0.05)
    raise AssertionError(f"queue still busy: {q}")


def test_truncated_body_then_healthy(live):
    app, port, name = live
    s = socket.create_connection(("127.0.0.1", port), timeout=10)
    body = json.dumps({"model": name, "prompt": "Hello", "stream": False})
    s.sendall((f"POST /api/generate HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\n"
               f"Content-Length: {len(body) + 50}\r\n\r\n{body[:10]}").encode())
    s.shutdown(socket.SHUT_WR)                       # the promised bytes never come
    s.settimeout(10)
    try:
        s.recv(4096)
    except OSError:
        pass
    s.close()
    _wait_idle(port)
    st, data = _post(port, "/api/generate", {"model": name, "prompt": "Hello", "stream": False, "options": {"num_predict": 3}})
    assert st == 200 and json.loads(data)["done"]


def test_malformed_json_is_a_client_error(live):
    app, port, name = live
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request("POST", "/v1/chat/completions", "{not json", {"Content-Type": "application/json"})
    r = c.getresponse()
    r.read()
    assert 400 <= r.status < 500
    assert not _queue(port)["busy"]


def test_client_disconnect_mid_stream_frees_the_queue(live):
    app, port, name = live
    st, _ = _post(port, "/api/generate", {"model": name, "prompt": "Hi", "stream": False, "options": {"num_predict": 1}})
    assert st == 200                                  # loads the model; /api/chat needs one loaded
    s = socket.create_connection(("127.0.0.1", port), timeout=30)
    body = json.dumps({"messages": [{"role": "user", "content": "Tell me a long story"}], "maxTokens": 400})
    s.sendall((f"POST /api/chat HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\n"
               f"Content-Length: {len(body)}\r\n\r\n{body}").encode())
    got = b""
    while b"data: " not in got:                      # first event arrived: generation is running
        chunk = s.recv(4096)
        assert chunk
        got += chunk
    s.setsockopt(socket.SOL_SOCKET, socket.SO_LINGER, b"\x01\x00\x00\x00\x00\x00\x00\x00")   # reset, not FIN
    s.close()
    q = _wait_idle(port)
    st, data = _post(port, "/api/generate", {"model": name, "prompt": "Hi", "stream": False, "options": {"num_predict": 2}})
    assert st == 200 and json.loads(data)["done"]
    assert _queue(port)["total_processed"] >= q["total_processed"] + 1


def test_load_of_corrupt_model_keeps_server_usable(live, tmp_path):
    app, port, name = live
    st, data = _post(port, "/api/models/load", {"model": "does-not-exist.gguf"})
    assert st >= 400 or "error" in data.lower()
    st, data = _post(port, "/api/generate", {"model": name, "prompt": "Hi", "stream": False, "options": {"num_predict": 2}})
    assert st == 200 and json.loads(data)["done"]


def test_concurrent_requests_share_steps_and_match_sequential(tmp_path, tiny_qwen3_path):
    """--max-batch 3: three clients at once are served together (the stepper's mean batch exceeds one), every
    answer equals what the one-at-a-time server gives, a fourth request waits in the queue, and a follow-up
    turn of a web-UI session still finds its KV cache."""
    name = os.path.basename(tiny_qwen3_path)
    args = ["--model", tiny_qwen3_path, "--backend", "cpu", "--port", "0", "--temperature", "0", "--top-k", "0", "--top-p", "1",
            "--repeat-penalty", "1"]
    prompts = ["Hello", "Tell me about the sea", "One two three", "What is this?", "Again and again"]

    def run_all(extra, concurrent):
        opts = build_options(args + extra, str(tmp_path), env={"TENSORSHARP_LOG_FILE": "0"})
        app = ServerApp(opts)
        httpd = serve(app, "127.0.0.1", 0)
        port = httpd.server_address[1]
        threading.Thread(target=httpd.serve_forever, daemon=True).start()
        out = {}
        try:
            st, _ = _post(port, "/api/generate", {"model": name, "prompt": "warm", "stream": False, "options": {"num_predict": 1}})
            assert st == 200

            def one(i):
                st, data = _post(port, "/api/generate", {"model": name, "prompt": prompts[i], "stream": False,
                                                         "options": {"num_predict": 6 + i}})
                out[i] = (st, json.loads(data)["response"])
            if concurrent:
                ths = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
                for t in ths:
                    t.start()
                for t in ths:
                    t.join(timeout=120)
            else:
                for i in range(len(prompts)):
                    one(i)
            gather = getattr(app.svc, "gather", None)
            mean = gather.step_rows / max(1, gather.steps) if gather is not None else 1.0
            q = _wait_idle(port)
            return out, mean, q
        finally:
            httpd.shutdown()
            httpd.server_close()
            app.svc.close()

    seq, _, _ = run_all([], False)
    par, mean, q = run_all(["--max-batch", "3"], True)
    assert all(st == 200 for st, _ in par.values())
    assert {i: r for i, (_, r) in par.items()} == {i: r for i, (_, r) in seq.items()}
    assert mean > 1.2, mean
    assert q["total_processed"] == len(prompts) + 1


def test_pool_reload_and_web_session_turns(tmp_path, tiny_qwen3_path):
    """With --max-batch the hosted model can be reloaded through /api/models/load (every slot moves to the
    new model, the old one gives its memory back) and a web-UI session's second turn is answered."""
    name = os.path.basename(tiny_qwen3_path)
    opts = build_options(["--model", tiny_qwen3_path, "--backend", "cpu", "--port", "0", "--max-batch", "2", "--temperature", "0",
                          "--top-k", "0", "--top-p", "1", "--repeat-penalty", "1"], str(tmp_path), env={"TENSORSHARP_LOG_FILE": "0"})
    app = ServerApp(opts)
    httpd = serve(app, "127.0.0.1", 0)
    port = httpd.server_address[1]
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        st, data = _post(port, "/api/models/load", {"model": name})
        assert st == 200 and json.loads(data)["ok"] is True
        first = app.svc.gather
        st, data = _post(port, "/api/models/load", {"model": name})
        assert st == 200 and app.svc.gather is not first and first._stop
        st, data = _post(port, "/api/chat", {"messages": [{"role": "user", "content": "Hello"}], "maxTokens": 4})
        ev = [json.loads(l[6:]) for l in data.split("\n\n") if l.startswith("data: ")]
        assert st == 200 and ev[-1]["done"] and ev[-1]["error"] is None
        reply = "".join(e.get("token", "") for e in ev)
        st, data = _post(port, "/api/chat", {"messages": [{"role": "user", "content": "Hello"}, {"role": "assistant", "content": reply},
                                                          {"role": "user", "content": "again"}], "maxTokens": 3})
        ev2 = [json.loads(l[6:]) for l in data.split("\n\n") if l.startswith("data: ")]
        assert st == 200 and ev2[-1]["done"] and ev2[-1]["error"] is None and ev2[-1]["promptTokens"] > ev[-1]["promptTokens"]
        # the session went back to the slot that holds its cache: the second turn re-used the first turn's tokens
        assert ev2[-1]["kvReusedTokens"] >= ev[-1]["promptTokens"]
    finally:
        httpd.shutdown()
        httpd.server_close()
        app.svc.close()
