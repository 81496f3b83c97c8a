"""The 8-bit (e4m3) KV cache on the CPU oracle path: a model that keeps its keys and values in one byte each follows
the float32-cache model closely, prefix reuse and truncation behave the same, and saved sessions convert between the
two cache types."""
import pytest
import torch

from tensorsharp_b200.models.base import ModelBase
from tensorsharp_b200.ops import functional as F


def test_scatter_and_gather_round_to_e4m3():
    cache = torch.zeros((8, 2, 16), dtype=torch.float8_e4m3fn)
    rows = torch.randn(3, 2, 16) * 3
    slots = torch.tensor([5, 0, 7])
    F.kv_scatter(cache, slots, rows)
    back = F.kv_gather(cache, slots)
    assert back.dtype == torch.float32 and torch.equal(back, rows.to(torch.float8_e4m3fn).float())
    assert float((back - rows).abs().max()) <= 0.0625 * float(rows.abs().max()) + 1e-3        # three mantissa bits
    assert float(F.kv_gather(cache, torch.tensor([1, 2])).abs().max()) == 0.0


def test_fp8_cache_follows_the_float_cache(tiny_qwen3_path, monkeypatch):
    ref = ModelBase.create(tiny_qwen3_path, "cpu", max_context=256)
    monkeypatch.setenv("TSB_KV_DTYPE", "fp8")
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=256)
    assert m.kv_dtype == torch.float8_e4m3fn and m.kv.k[0].dtype == torch.float8_e4m3fn
    assert m.kv.k[0].element_size() == 1
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 4096, (48,), generator=g).tolist()
    want = ref.forward(ids)
    full = m.forward(ids)
    rel = float((full - want).abs().max() / want.abs().max())
    assert rel < 0.08, rel                                 # the rounding of K and V, nothing structural
    # the cache is consistent with itself: incremental steps, truncation and replay give what one pass gives
    m.reset_kv_cache()
    m.forward(ids[:30])
    inc = m.forward(ids[30:])
    assert torch.allclose(full, inc, atol=5e-3)
    m.truncate_kv_cache(12)
    assert torch.allclose(m.forward(ids[12:]), full, atol=5e-3)


def test_sessions_move_between_cache_types(tiny_qwen3_path, tmp_path, monkeypatch):
    from tensorsharp_b200.runtime.kv_cache import KVCache
    from tensorsharp_b200.runtime.session_store import load_session, save_session
    prompt = [5, 9, 33, 7, 21, 40, 2, 18, 77, 91]
    monkeypatch.setenv("TSB_KV_DTYPE", "fp8")
    m8 = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    cache = KVCache()
    lg = m8.forward(prompt)
    cache.record_append(prompt, lg)
    nxt = int(lg.argmax())
    want = m8.forward([nxt]).clone()
    m8.truncate_kv_cache(len(prompt))
    path = str(tmp_path / "chat8.tsbkv")
    assert save_session(path, m8, cache) == len(prompt)
    # into a second 8-bit cache: the bytes come back as they were
    again = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    c2 = KVCache()
    assert load_session(path, again, c2) == len(prompt)
    assert torch.allclose(again.forward([nxt]), want, atol=1e-4, rtol=1e-4)
    # into a float32 cache: the e4m3 values are exactly representable there
    monkeypatch.delenv("TSB_KV_DTYPE")
    m32 = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    assert m32.kv_dtype == torch.float32
    c3 = KVCache()
    assert load_session(path, m32, c3) == len(prompt)
    got = m32.forward([nxt])
    assert float((got - want).abs().max() / want.abs().max()) < 0.05      # only the new token's K / V differ in rounding


def test_fp8_cache_is_refused_where_it_has_no_path(tiny_qwen3_path, monkeypatch):
    class FakeComm:
        size = 2
        rank = 0
    monkeypatch.setenv("TSB_KV_DTYPE", "fp8")
    with pytest.raises(ValueError, match="8-bit KV cache"):
        ModelBase.create(tiny_qwen3_path, "cpu", max_context=64, cp_comm=FakeComm())


def test_kv_dtype_option_of_the_cli_and_the_server(monkeypatch, tmp_path):
    from tensorsharp_b200.cli.args import parse_cli_args
    from tensorsharp_b200.server import options as O
    assert parse_cli_args(["--model", "m.gguf", "--kv-dtype", "FP8"]).kv_dtype == "fp8"
    assert parse_cli_args(["--model", "m.gguf"]).kv_dtype is None
    with pytest.raises(ValueError, match="--kv-dtype"):
        parse_cli_args(["--kv-dtype", "int3"])
    monkeypatch.setenv("TSB_KV_DTYPE", "bf16")          # registered with monkeypatch, so the export below is undone afterwards
    assert O.parse_args(["--kv-dtype", "e4m3", "--port", "5001"])["kv_dtype"] == "e4m3"
    O.build_options(["--kv-dtype", "e4m3"], str(tmp_path), env={})
    import os
    assert os.environ.get("TSB_KV_DTYPE") == "fp8"


@pytest.mark.parametrize("name", ["gptoss", "gemma3", "gemma4", "gemma4_wide_heads", "mistral3", "qwen35_dense", "nemotron_h"])
def test_every_family_runs_on_the_fp8_cache(name, tmp_path, monkeypatch):
    """Sliding windows, sinks, shared KV layers, wide heads and the attention layers of the hybrid models read the 8-bit
    pages through the same helpers: logits stay close to the float32-cache model, and prefix + suffix equals one pass."""
    from tests.test_model_families_cpu import FAMILIES
    fn, kw = FAMILIES[name]
    p = str(tmp_path / f"{name}.gguf")
    fn(p, device="cpu", **kw)
    ref = ModelBase.create(p, "cpu", max_context=256)
    monkeypatch.setenv("TSB_KV_DTYPE", "fp8")
    m = ModelBase.create(p, "cpu", max_context=256)
    assert all(k is None or k.dtype == torch.float8_e4m3fn for k in m.kv.k)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 4096, (70,), generator=g).tolist()
    want, full = ref.forward(ids), m.forward(ids)
    assert torch.isfinite(full).all()
    rel = float((full - want).abs().max() / want.abs().max())
    assert rel < 0.15, rel
    m.reset_kv_cache()
    m.forward(ids[:40], want_logits=False)
    inc = m.forward(ids[40:])
    assert float((inc - full).abs().max()) < 2e-2 * max(1.0, float(full.abs().max()))
