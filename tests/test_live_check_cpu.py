"""The live-server checker (server/testdata/live_check.py) run against a loopback server with a tiny random model:
every protocol check passes, and the checker notices a server that misbehaves."""
import importlib.util
import io
import os
import threading

import pytest

from tensorsharp_b200.server.app import ServerApp, serve
from tensorsharp_b200.server.options import build_options

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(os.path.dirname(HERE), "tensorsharp_b200", "server", "testdata", "live_check.py")


def _load():
    spec = importlib.util.spec_from_file_location("live_check", SCRIPT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture()
def live_server(tmp_path, tiny_qwen3_path):
    opts = build_options(["--model", tiny_qwen3_path, "--backend", "cpu", "--port", "0", "--temperature", "0", "--top-k", "0",
                          "--top-p", "1", "--repeat-penalty", "1"], str(tmp_path), env={"TENSORSHARP_LOG_FILE": "0"})
    app = ServerApp(opts)
    httpd = serve(app, "127.0.0.1", 0)
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    try:
        yield f"http://127.0.0.1:{httpd.server_address[1]}"
    finally:
        httpd.shutdown()
        httpd.server_close()
        app.svc.close()


def test_every_protocol_check_passes_against_a_loopback_server(live_server):
    lc = _load()
    out = io.StringIO()
    check = lc.LiveCheck(live_server, max_tokens=6, out=out)
    rc = check.run()
    failed = [row for row in check.r.rows if row[1] == "FAIL"]
    assert rc == 0 and not failed, out.getvalue()
    assert len(check.r.rows) > 50                            # every group ran


def test_the_checker_reports_failures_and_bad_arguments(live_server):
    lc = _load()
    out = io.StringIO()
    check = lc.LiveCheck(live_server, model="not-hosted.gguf", max_tokens=4, out=out)
    assert check.run(["ollama"]) == 1 and check.r.failed > 0 and "FAIL" in out.getvalue()
    dead = lc.LiveCheck("http://127.0.0.1:9", max_tokens=4, out=io.StringIO())
    assert dead.run(["errors"]) == 1                         # nothing listens there: reported, not raised
    with pytest.raises(SystemExit):
        lc.main(["--only", "nonsense"])
