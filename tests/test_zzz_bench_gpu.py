"""bench.py on tiny models: the JSON contract, and the long-context configuration's second turn on a kept prefix."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench(tmp_path, *flags):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "4", "--warmup", "3", "--prefill-repeats", "1",
                        "--cache-dir", str(tmp_path), *flags], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    return json.loads(p.stdout.strip().splitlines()[-1])


def test_contract_fields_on_the_tiny_model(tmp_path):
    r = _bench(tmp_path, "--model", "qwen3-tiny")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "dtype", "data",
                "config", "e2e", "gpu_launches", "clocks"):
        assert key in r, key
    assert r["steps"] == 4 and r["value"] > 0 and r["gpu_launches"] > 0 and r["e2e"]["value"] > 0 and r["kernel_status"] == 0


def test_second_turn_keeps_a_prefix_of_the_cache(tmp_path):
    r = _bench(tmp_path, "--model", "gemma-tiny")
    t2 = r["second_turn"]
    assert t2["kv_reused_tokens"] == 80 and t2["new_tokens"] > 16 and t2["ttft_ms"] > 0 and r["kernel_status"] == 0
