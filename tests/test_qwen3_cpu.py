"""Tiny Qwen3 on the CPU oracle path: cache consistency, truncation, chunked prefill."""
import pytest
import torch

from tensorsharp_b200.models.base import ModelBase
from tensorsharp_b200.runtime.engine import DecodeGraph, generate, run_benchmark, synthetic_prompt
from tensorsharp_b200.runtime.sampling import SamplingConfig, TokenSampler


def test_incremental_equals_full(tiny_qwen3_path):
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=256)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 4096, (40,), generator=g).tolist()
    full = m.forward(ids)
    m.reset_kv_cache()
    m.forward(ids[:25])
    inc = m.forward(ids[25:])
    assert torch.allclose(full, inc, atol=5e-3)
    # truncate to a prefix and replay the suffix (multi-turn reuse)
    m.truncate_kv_cache(10)
    assert m.cache_length == 10
    again = m.forward(ids[10:])
    assert torch.allclose(full, again, atol=5e-3)
    m.reset_kv_cache()
    assert torch.allclose(m.forward_refill(ids, chunk=7), full, atol=5e-3)


def test_batched_equals_single(tiny_qwen3_path):
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128, max_seqs=4)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (3, 11, 20)]
    seqs = [m.kv.new_seq() for _ in prompts]
    lb = m.forward_batch(m.kv.build_batch(seqs, prompts))
    for i, p in enumerate(prompts):
        m.reset_kv_cache()
        assert torch.allclose(m.forward(p), lb[i], atol=5e-3)
    # batched greedy decode through the step runner equals per-sequence decode
    dg = DecodeGraph(m, seqs, 4)
    dg.set_tokens([int(x) for x in lb.argmax(-1)])
    got = [dg.step().tolist() for _ in range(3)]
    m.reset_kv_cache()
    l = m.forward(prompts[1])
    t = int(l.argmax())
    for s in range(3):
        l = m.forward([t])
        t = int(l.argmax())
        assert got[s][1] == t
    # the step runner refuses to go past the context it reserved (longest prompt 20 + 4 new tokens + 1)
    dg.step(); dg.step()
    with pytest.raises(RuntimeError, match="sized for a context"):
        dg.step()


def test_generate_and_benchmark(tiny_qwen3_path):
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=256)
    out = generate(m, synthetic_prompt(16, m.cfg.vocab), 5, TokenSampler(SamplingConfig.greedy()))
    assert len(out) == 5
    r = run_benchmark(m, prefill=8, decode=4, runs=2)
    assert len(r) == 2 and r[0].decode_tokens == 4 and r[0].prefill_tps > 0
    assert synthetic_prompt(20, 50)[:3] == [49, 49, 49] and synthetic_prompt(3, 4096) == [100, 101, 102]


def test_bench_cpu_configuration_prints_one_json_line(tmp_path):
    """``bench.py --model qwen3-tiny --device cpu``: the tiny configuration on the CPU backend (prompt 64, 32 greedy tokens)."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--model", "qwen3-tiny", "--device", "cpu",
                        "--cache-dir", str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.loads(p.stdout.strip().splitlines()[-1])
    assert r["device"] == "cpu" and r["steps"] == 32 and r["config"]["seq_len"] == 64 and r["value"] > 0 and r["prefill_tok_s"] > 0
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--model", "qwen3-tiny", "--device", "cpu", "--impl", "reference"],
                       capture_output=True, text=True, timeout=600)
    assert json.loads(p.stdout.strip().splitlines()[-1])["impl"] == "reference"
