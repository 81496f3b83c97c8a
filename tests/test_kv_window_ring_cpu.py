"""Sliding-window layers on a ring of pages (TSB_KV_WINDOW_RING=1): same logits as the pool that keeps every page, for
prompts that wrap the ring several times, chunked prefill, decode steps, a cut within the ring's slack and one beyond it;
and the memory the window layers then hold."""
import pytest
import torch

from tensorsharp_b200.models import synth
from tensorsharp_b200.models.base import ModelBase
from tensorsharp_b200.runtime.paged_kv import PagedKV


def _make(path, monkeypatch, ring, chunk=32, **kw):
    monkeypatch.setenv("TSB_KV_WINDOW_RING", "1" if ring else "0")
    monkeypatch.setenv("TSB_KV_RING_CHUNK", str(chunk))
    return ModelBase.create(path, "cpu", max_context=512, page_size=16, **kw)


@pytest.mark.parametrize("family", ["gemma3", "gptoss"])
def test_ring_gives_the_full_pool_logits(tmp_path, monkeypatch, family):
    p = str(tmp_path / "m.gguf")
    if family == "gemma3":
        synth.write_gemma(p, arch="gemma3", window=16, device="cpu")
    else:
        synth.write_gptoss(p, n_layers=2, window=16, device="cpu")
    full = _make(p, monkeypatch, False)
    ring = _make(p, monkeypatch, True)
    assert ring.kv.ring and not full.kv.ring
    # window 16 + chunk 32 -> 3 pages of 16, + 1: a ring of 4 pages = 64 tokens per window layer and sequence
    assert ring.kv.ring_pages == 4
    wl = ring.kv_window_layers()
    assert wl and all(ring.kv.k[l].shape[0] < full.kv.k[l].shape[0] for l in wl)
    assert all(ring.kv.k[l].shape[0] == full.kv.k[l].shape[0] for l in range(len(ring.kv.k)) if l not in wl and ring.kv.k[l] is not None)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 4096, (300,), generator=g).tolist()          # wraps the 64-token ring more than four times
    for i in range(0, 288, 32):                                          # the same chunks the ring model cuts the prompt into
        full.forward(toks[i:i + 32], want_logits=False)
    a, b = full.forward(toks[288:]), ring.forward(toks)
    assert torch.allclose(a, b, atol=1e-5), float((a - b).abs().max())
    t = int(a.argmax())
    for _ in range(20):                                                  # decode across a page boundary of the ring
        a, b = full.forward([t]), ring.forward([t])
        assert torch.allclose(a, b, atol=1e-5)
        t = int(a.argmax())
    # a cut within the slack (ring capacity 64 - window 16 = 48 tokens back) keeps the cache; the logits still agree
    keep = full.cache_length - 30
    full.truncate_kv_cache(keep)
    ring.truncate_kv_cache(keep)
    assert ring.cache_length == keep
    a, b = full.forward(toks[:7]), ring.forward(toks[:7])
    assert torch.allclose(a, b, atol=1e-5)
    # a cut further back than the ring remembers starts the sequence over instead of attending to overwritten keys
    ring.truncate_kv_cache(100)
    assert ring.cache_length == 0


def test_ring_bookkeeping():
    kv = PagedKV([(2, 8), (2, 8)], n_pages=64, page_size=16, window_layers={0: 16}, ring_chunk=32, max_seqs=2)
    assert kv.ring_pages == 4 and kv.n_wpages == 8 and kv.k[0].shape[0] == 8 * 16 and kv.k[1].shape[0] == 64 * 16
    s = kv.new_seq()
    b = kv.build_batch([s], [list(range(20))])
    assert len(s.wpages) == 2 and b.slots_w.tolist() == [kv.wslot(s, p) for p in range(20)]
    with pytest.raises(ValueError):
        kv.build_batch([s], [list(range(33))])                           # more than the ring was sized for
    for _ in range(5):
        b = kv.build_batch([s], [list(range(32))])
    assert s.length == 180 and len(s.wpages) == 4 and len(s.pages) == 12
    row = b.block_table_w[0].tolist()
    assert row[:12] == [s.wpages[j % 4] for j in range(12)]
    w = b.windowed()
    assert w.block_table is b.block_table_w and w.slots is b.slots_w and w.tokens is b.tokens
    assert kv.can_truncate(s, 180 - 48) and not kv.can_truncate(s, 180 - 49)
    free_before = len(kv._wfree)
    kv.free_seq(s)
    assert len(kv._wfree) == free_before + 4 and kv.free_pages == 64


def test_decode_graph_bookkeeping_on_a_ring_pool(tmp_path, monkeypatch):
    """DecodeGraph (eager on CPU: the same static batch and advance arithmetic as the captured step) keeps the ring's
    slots in step with the positions: greedy tokens equal those of the pool that keeps every page."""
    from tensorsharp_b200.ops import functional as F
    from tensorsharp_b200.runtime.engine import DecodeGraph
    p = str(tmp_path / "m.gguf")
    synth.write_gemma(p, arch="gemma3", window=16, device="cpu")
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 4096, (30,), generator=g).tolist()
    outs = []
    for ring in (False, True):
        m = _make(p, monkeypatch, ring)
        seq = m.new_sequence()
        first = int(F.argmax(m.forward_batch(m.kv.build_batch([seq], [prompt])))[0])
        dg = DecodeGraph(m, [seq], 90)
        dg.set_tokens([first])
        dg.capture()
        outs.append([first] + [int(dg.step()[0]) for _ in range(80)])     # 110 positions: the 64-token ring wraps
    assert outs[0] == outs[1]
