"""Data-parallel serving: two server processes (CPU, a tiny random model) behind the routing front end."""
import http.client
import importlib.util
import io
import json
import os
import threading

import pytest

from tensorsharp_b200.server import replicas as R

HERE = os.path.dirname(os.path.abspath(__file__))


def test_router_prefers_idle_replicas_and_keeps_sessions_where_they_are():
    reps = [R.Replica(i, "127.0.0.1", 1) for i in range(3)]
    router = R.Router(reps)
    a = router.pick("POST", "/api/generate", b"{}")
    b = router.pick("POST", "/v1/chat/completions", b"{}")
    c = router.pick("POST", "/api/chat/ollama", b"{}")
    assert sorted(x.index for x in (a, b, c)) == [0, 1, 2]          # three requests in flight: one each
    router.done(b)
    assert router.pick("POST", "/api/generate", b"{}") is b          # the idle one
    router.bind_session("s1", reps[2])
    body = json.dumps({"sessionId": "s1", "messages": []}).encode()
    assert router.pick("POST", "/api/chat", body) is reps[2] and router.pick("DELETE", "/api/sessions/s1", b"") is reps[2]
    router.drop_session("s1")
    assert router.owner("s1") == -1
    assert router.pick("GET", "/api/tags", b"") is reps[0]           # everything else: replica 0
    assert R.replica_argv(["--model", "m", "--replicas", "2", "--port=5000", "--host", "0.0.0.0"], 7001) == \
        ["--model", "m", "--host", "127.0.0.1", "--port", "7001"]
    env = R.replica_env({"TENSORSHARP_REPLICAS": "4", "WORLD_SIZE": "2", "RANK": "1", "HOME": "/h", "CUDA_VISIBLE_DEVICES": "0,1"}, "1")
    assert env == {"HOME": "/h", "CUDA_VISIBLE_DEVICES": "1"}                 # a replica must not start replicas of its own
    assert R.replica_env({"CUDA_VISIBLE_DEVICES": "0,1"}, None) == {"CUDA_VISIBLE_DEVICES": "0,1"}


def test_merge_metrics_labels_samples_by_replica():
    a = "# HELP x_total n\n# TYPE x_total counter\nx_total 3\ny{k=\"v\"} 1\n"
    out = R.merge_metrics([a, a.replace(" 3", " 4")])
    assert out.count("# TYPE x_total counter") == 1
    assert 'x_total{replica="0"} 3' in out and 'x_total{replica="1"} 4' in out and 'y{k="v",replica="1"} 1' in out


@pytest.fixture(scope="module")
def front(tmp_path_factory, tiny_qwen3_path):
    base = tmp_path_factory.mktemp("replicas")
    argv = ["--model", tiny_qwen3_path, "--backend", "cpu", "--temperature", "0", "--top-k", "0", "--top-p", "1",
            "--repeat-penalty", "1", "--replicas", "2"]
    env_before = dict(os.environ)
    os.environ.update(TENSORSHARP_BASE_DIR=str(base), TENSORSHARP_LOG_FILE="0")
    try:
        reps = R.spawn_replicas(argv, 2, use_gpus=False, ready_timeout_s=300, log_dir=str(base))
    finally:
        os.environ.clear()
        os.environ.update(env_before)
    router = R.Router(reps)
    httpd = R.serve_front(router, "127.0.0.1", 0)
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    try:
        yield f"http://127.0.0.1:{httpd.server_address[1]}", router
    finally:
        httpd.shutdown()
        httpd.server_close()
        R.stop_replicas(reps)
        assert all(r.process.poll() is not None for r in reps)


def _post(url, path, body, timeout=300):
    host, port = url[7:].split(":")
    c = http.client.HTTPConnection(host, int(port), timeout=timeout)
    c.request("POST", path, json.dumps(body).encode() if body is not None else None, {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    return r.status, data


def test_concurrent_requests_spread_over_the_replicas_and_sessions_stay_put(front, tiny_qwen3_path):
    url, router = front
    name = os.path.basename(tiny_qwen3_path)
    results = []

    def one(i):
        results.append(_post(url, "/api/generate", {"model": name, "prompt": f"hello {i}", "stream": False, "options": {"num_predict": 12}}))
    host, port = url[7:].split(":")
    for burst in range(3):            # on a loaded machine one replica can finish a request before the next one is sent
        th = [threading.Thread(target=one, args=(i,)) for i in range(4)]
        [t.start() for t in th]
        [t.join(300) for t in th]
        assert len(results) == 4 * (burst + 1) and all(st == 200 and json.loads(d)["done"] for st, d in results)
        c = http.client.HTTPConnection(host, int(port), timeout=30)
        c.request("GET", "/api/queue/status")
        q = json.loads(c.getresponse().read())
        c.close()
        per = [x["total_processed"] for x in q["replicas"]]
        assert q["total_processed"] == sum(per) >= 4 * (burst + 1), q
        if all(n >= 1 for n in per):
            break
    assert all(n >= 1 for n in per), q                                                # both replicas did some of the work
    # a chat session lives on one replica: the second turn finds the first one's cache there
    st, d = _post(url, "/api/sessions", None)
    sid = json.loads(d)["sessionId"]
    owner = router.owner(sid)
    assert st == 200 and owner in (0, 1)
    msgs = [{"role": "user", "content": "Hello there"}]
    st, d = _post(url, "/api/models/load", {"model": name, "backend": "cpu"})
    assert st == 200 and json.loads(d)["ok"]                                          # sent to every replica
    st, d = _post(url, "/api/chat", {"sessionId": sid, "messages": msgs, "maxTokens": 4})
    ev = [json.loads(l[6:]) for l in d.split("\n\n") if l.startswith("data: ")]
    assert st == 200 and ev[-1]["done"] and ev[-1]["error"] is None
    reply = "".join(e.get("token", "") for e in ev[:-1])
    msgs += [{"role": "assistant", "content": reply}, {"role": "user", "content": "again"}]
    st, d = _post(url, "/api/chat", {"sessionId": sid, "messages": msgs, "maxTokens": 3})
    ev2 = [json.loads(l[6:]) for l in d.split("\n\n") if l.startswith("data: ")]
    assert ev2[-1]["kvReusedTokens"] >= ev[-1]["promptTokens"] and router.owner(sid) == owner
    c = http.client.HTTPConnection(host, int(port), timeout=30)
    c.request("GET", "/metrics")
    text = c.getresponse().read().decode()
    c.close()
    assert 'replica="0"' in text and 'replica="1"' in text


def test_live_checks_pass_through_the_front_end(front):
    url, _ = front
    spec = importlib.util.spec_from_file_location(
        "live_check", os.path.join(os.path.dirname(HERE), "tensorsharp_b200", "server", "testdata", "live_check.py"))
    lc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lc)
    out = io.StringIO()
    check = lc.LiveCheck(url, max_tokens=5, out=out)
    assert check.run(["webui", "ollama", "openai", "errors", "queue"]) == 0, out.getvalue()


def test_the_server_entry_point_starts_and_stops_its_replicas(tmp_path, tiny_qwen3_path):
    """``python -m tensorsharp_b200.server --replicas 2``: one public port, SIGTERM ends the front end and both replicas."""
    import signal
    import subprocess
    import sys
    import time
    port = R._free_port()
    env = dict(os.environ, TENSORSHARP_BASE_DIR=str(tmp_path), TENSORSHARP_LOG_FILE="0", PYTHONPATH=os.path.dirname(HERE))
    p = subprocess.Popen([sys.executable, "-m", "tensorsharp_b200.server", "--model", tiny_qwen3_path, "--backend", "cpu",
                          "--replicas", "2", "--port", str(port)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        line = ""
        deadline = time.monotonic() + 300
        while "replicas ready" not in line and time.monotonic() < deadline and p.poll() is None:
            line = p.stdout.readline()
        assert "2 replicas ready" in line, line
        child_ports = [int(x) for x in line.split("(")[1].split(")")[0].split(",")]
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/api/queue/status")
        q = json.loads(c.getresponse().read())
        c.close()
        assert len(q["replicas"]) == 2 and not q["busy"]
        p.send_signal(signal.SIGTERM)
        assert p.wait(60) == 0
        for cp in child_ports:                                   # the replicas are gone with it
            with pytest.raises(OSError):
                http.client.HTTPConnection("127.0.0.1", cp, timeout=2).request("GET", "/api/version")
    finally:
        if p.poll() is None:
            p.kill()


def test_a_dead_replica_is_avoided_and_started_again(tmp_path, tiny_qwen3_path):
    """A replica process that dies: requests that reach it before the front end knows are retried on the other one,
    the supervisor starts it again, and it takes work again once it answers."""
    import time
    argv = ["--model", tiny_qwen3_path, "--backend", "cpu", "--temperature", "0", "--replicas", "2"]
    env_before = dict(os.environ)
    os.environ.update(TENSORSHARP_BASE_DIR=str(tmp_path), TENSORSHARP_LOG_FILE="0")
    try:
        reps = R.spawn_replicas(argv, 2, use_gpus=False, ready_timeout_s=300)
    finally:
        os.environ.clear()
        os.environ.update(env_before)
    router = R.Router(reps)
    sup = R.Supervisor(router, poll_s=0.2, ready_timeout_s=300).start()
    httpd = R.serve_front(router, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{httpd.server_address[1]}"
    name = os.path.basename(tiny_qwen3_path)
    ask = {"model": name, "prompt": "hello", "stream": False, "options": {"num_predict": 4}}
    try:
        first_pid = reps[1].process.pid
        reps[1].process.terminate()
        reps[1].process.wait(30)
        for _ in range(3):                                    # some of these are dealt to the dead replica first
            st, d = _post(url, "/api/generate", ask)
            assert st == 200 and json.loads(d)["done"]
        deadline = time.monotonic() + 300
        while not (reps[1].restarts >= 1 and reps[1].up) and time.monotonic() < deadline:
            time.sleep(0.2)
        assert reps[1].restarts == 1 and reps[1].up and reps[1].process.pid != first_pid and reps[1].process.poll() is None
        for _ in range(4):
            assert _post(url, "/api/generate", ask)[0] == 200
        st, q = reps[1].get_json("/api/queue/status")
        assert st == 200 and q["total_processed"] >= 1         # the new process is in the rotation again
        # a session that lived on a replica that is gone is forgotten by the router
        router.bind_session("s-old", reps[1])
        router.forget_sessions_of(reps[1])
        assert router.owner("s-old") == -1
    finally:
        sup.stop()
        httpd.shutdown()
        httpd.server_close()
        R.stop_replicas(reps)
