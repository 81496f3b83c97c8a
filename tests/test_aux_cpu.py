"""Auxiliary subsystems: phase timing, rank liveness (failures injected on the host), session
persistence, typed errors, and a CPU model of the tagged-word exchange protocol."""
import multiprocessing as mp
import os
import time

import pytest
import torch

from tensorsharp_b200.parallel.errors import ExchangeTimeoutError, RankFailureError
from tensorsharp_b200.parallel.watchdog import Heartbeat, Watchdog
from tensorsharp_b200.runtime.profiling import PhaseTimer


def test_phase_timer_table():
    t = PhaseTimer("cpu", enabled=True)
    for _ in range(3):
        with t.phase("decode"):
            time.sleep(0.001)
    with t.phase("prefill"):
        time.sleep(0.002)
    s = t.stats()
    assert s["decode"]["calls"] == 3 and s["prefill"]["calls"] == 1
    assert s["decode"]["total_ms"] >= 3 * 0.9
    assert "share" in t.table() and "prefill" in t.table()
    t.reset()
    assert t.stats() == {}


def test_phase_timer_off_is_free():
    t = PhaseTimer("cpu", enabled=False)
    with t.phase("x"):
        pass
    assert t.stats() == {}


class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode()

    def get(self, k):
        return self.d[k]

    def check(self, ks):
        return all(k in self.d for k in ks)


def test_heartbeat_detects_silent_and_departed_rank():
    store, now = DictStore(), [0.0]
    hb = [Heartbeat(store, r, 3, clock=lambda: now[0]) for r in range(3)]
    assert hb[0].stale_ranks(1.0) == set()
    now[0] = 0.5
    hb[1].beat(); hb[2].beat()
    assert hb[0].stale_ranks(1.0) == set()
    now[0] = 2.0
    hb[1].beat()                                   # rank 2 stays silent
    assert hb[0].stale_ranks(1.0) == {2}
    hb[1].leave()
    with pytest.raises(RankFailureError) as e:
        hb[0].check(1.0)
    assert e.value.stale == [1, 2]


def test_watchdog_thread_reports_once():
    store = DictStore()
    a, b = Heartbeat(store, 0, 2), Heartbeat(store, 1, 2)
    seen = []
    w = Watchdog(a, timeout_s=0.15, interval_s=0.03, on_failure=lambda s: seen.append(set(s))).start()
    t0 = time.time()
    while time.time() - t0 < 0.1:
        b.beat(); time.sleep(0.02)
    assert not seen
    time.sleep(0.4)                                # b stops beating
    w.stop()
    assert seen == [{1}]


def _rank_main(rank, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from datetime import timedelta
    store = dist.TCPStore("127.0.0.1", port, 2, rank == 0, timeout=timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=2, timeout=timedelta(seconds=20))
    hb = Heartbeat(store, rank, 2)
    x = torch.ones(4)
    dist.all_reduce(x)                             # step 1: both ranks alive
    if rank == 1:
        hb.leave()                                 # leaves between steps, nothing in flight
        q.put(("left", float(x[0])))
        time.sleep(1.0)                            # keep the store's client socket open while rank 0 checks
        return
    deadline = time.time() + 10
    err = None
    while time.time() < deadline and err is None:
        try:
            hb.check(0.5)                          # before launching step 2
            time.sleep(0.05)
        except RankFailureError as e:
            err = e.stale
    q.put(("detected", err))


def test_rank_departure_detected_before_next_collective():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    ps = [ctx.Process(target=_rank_main, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    assert got["left"] == 2.0
    assert got["detected"] == [1]


def test_exchange_timeout_error_fields():
    e = ExchangeTimeoutError("x", 3)
    assert e.code == 3 and "status 3" in str(e)


# ---- CPU model of the tagged-word exchange: a word is valid only when its tag matches the reader's
# epoch; slots are reused every SLOTS epochs, so a writer may run at most SLOTS - 1 epochs ahead.
SLOTS = 4


class Mailbox:
    def __init__(self, ranks, words):
        self.val = [[[0.0] * words for _ in range(ranks)] for _ in range(SLOTS)]
        self.tag = [[[0] * words for _ in range(ranks)] for _ in range(SLOTS)]


def _push(boxes, src, epoch, vals):
    for mb in boxes:
        for i, v in enumerate(vals):
            mb.val[epoch % SLOTS][src][i] = v
            mb.tag[epoch % SLOTS][src][i] = epoch + 1


def _try_reduce(mb, epoch, ranks, words):
    s = epoch % SLOTS
    if any(mb.tag[s][r][i] != epoch + 1 for r in range(ranks) for i in range(words)):
        return None
    return [sum(mb.val[s][r][i] for r in range(ranks)) for i in range(words)]


def test_tagged_word_protocol_model_interleavings():
    import random
    rng = random.Random(0)
    ranks, words, epochs = 3, 2, 12
    for trial in range(50):
        boxes = [Mailbox(ranks, words) for _ in range(ranks)]
        pushed = [0] * ranks                        # next epoch each rank will push
        reduced = [0] * ranks                       # next epoch each rank will reduce
        while min(reduced) < epochs:
            r = rng.randrange(ranks)
            # a rank pushes epoch e only after reducing e - 1 (one exchange per kernel pair), so it is
            # never more than one epoch ahead of itself and at most two ahead of the slowest peer
            if pushed[r] == reduced[r] and pushed[r] < epochs:
                _push(boxes, r, pushed[r], [float(pushed[r] * 10 + r + i) for i in range(words)])
                pushed[r] += 1
            elif reduced[r] < pushed[r]:
                out = _try_reduce(boxes[r], reduced[r], ranks, words)
                if out is not None:
                    e = reduced[r]
                    assert out == [float(sum(e * 10 + q + i for q in range(ranks))) for i in range(words)]
                    reduced[r] += 1
            assert max(pushed) - min(reduced) < SLOTS


def test_tagged_word_stale_slot_is_not_accepted():
    boxes = [Mailbox(2, 1)]
    _push(boxes, 0, 0, [1.0]); _push(boxes, 1, 0, [2.0])
    assert _try_reduce(boxes[0], 0, 2, 1) == [3.0]
    _push(boxes, 0, SLOTS, [5.0])                  # same slot, later epoch, peer 1 not yet there
    assert _try_reduce(boxes[0], SLOTS, 2, 1) is None


def test_session_store_round_trip(tiny_qwen3_path, tmp_path):
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.kv_cache import KVCache
    from tensorsharp_b200.runtime.session_store import load_session, save_session
    m = ModelBase.create(tiny_qwen3_path, device="cpu", max_context=128)
    prompt = [5, 9, 33, 7, 21, 40, 2, 18]
    cache = KVCache()
    lg = m.forward(prompt)
    cache.record_append(prompt, lg)
    nxt = int(lg.argmax())
    want = m.forward([nxt]).clone()
    m.truncate_kv_cache(len(prompt))
    path = str(tmp_path / "chat.tsbkv")
    assert save_session(path, m, cache) == len(prompt)

    m2 = ModelBase.create(tiny_qwen3_path, device="cpu", max_context=128)
    cache2 = KVCache()
    assert load_session(path, m2, cache2) == len(prompt)
    assert list(cache2.tokens) == prompt and m2.cache_length == len(prompt)
    assert torch.allclose(cache2.next_logits.float(), lg.float())
    got = m2.forward([nxt])
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    plan = cache2.plan_reuse(prompt + [nxt], True)
    assert plan.reused_prefix == len(prompt) if hasattr(plan, "reused_prefix") else True


def test_model_timing_table(tiny_qwen3_path, monkeypatch, capsys):
    from tensorsharp_b200.models.base import ModelBase
    monkeypatch.setenv("TSB_PROFILE", "1")
    m = ModelBase.create(tiny_qwen3_path, device="cpu", max_context=64)
    m.forward([1, 2, 3, 4])
    m.forward([5]); m.forward([6])
    s = m.timer.stats()
    assert s["prefill"]["calls"] == 1 and s["decode"]["calls"] == 2
    m.print_timing_stats()
    assert "decode" in capsys.readouterr().err


def test_gathered_model_merges_threads_and_propagates_errors(tiny_qwen3_path):
    import threading

    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import generate
    from tensorsharp_b200.runtime.gather import GatheredModel
    real = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128, max_seqs=5)
    g = GatheredModel(real, 4, window_s=0.05)
    gen = torch.Generator().manual_seed(6)
    prompts = [torch.randint(5, 4000, (n,), generator=gen).tolist() for n in (9, 17, 4, 12)]
    eos = [t for t in range(real.cfg.vocab) if real.tokenizer.is_eos(t)]
    got = {}

    def worker(i):
        with g.slot(i) as m:                                  # the bracket tells the stepper how many callers to expect
            got[i] = generate(m, prompts[i], 6, eos_ids=eos, prefill_chunk=8)
    ths = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(timeout=120)
    assert g.step_rows / g.steps > 1.5                        # steps were shared
    for i, p in enumerate(prompts):
        real.reset_kv_cache()
        assert got[i] == generate(real, p, 6, eos_ids=eos)
    # slot state is per slot: truncation and reset act on that slot's sequence only
    s0, s1 = g.slot(0), g.slot(1)
    l0, l1 = s0.cache_length, s1.cache_length
    s0.truncate_kv_cache(3)
    assert s0.cache_length == 3 and s1.cache_length == l1 and l0 > 3
    s1.reset_kv_cache()
    assert s1.cache_length == 0
    # a failing step reaches the caller as an exception, and the stepper keeps running
    with pytest.raises(Exception):
        s0.forward([10 ** 9])                                 # token id outside the vocabulary
    assert s1.forward([5]) is not None
    free_before = real.kv.free_pages
    g.close()
    assert real.kv.free_pages > free_before                   # slots gave their sequences back
    with pytest.raises(RuntimeError):
        s1.forward([5])


def test_batch_stepper_follows_changing_membership(tiny_qwen3_path, monkeypatch):
    """Single-token steps of several sequences through the static batch of ``BatchGraphStepper`` (eager on CPU) give the
    logits of the ordinary batched step while sequences join, leave and cross a page boundary; with TSB_GATHER_GRAPH=1
    the merged steps of concurrent callers go through it."""
    import threading

    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import BatchGraphStepper, generate
    from tensorsharp_b200.runtime.gather import GatheredModel
    a = ModelBase.create(tiny_qwen3_path, "cpu", max_context=256, max_seqs=4, page_size=16)
    b = ModelBase.create(tiny_qwen3_path, "cpu", max_context=256, max_seqs=4, page_size=16)
    st = BatchGraphStepper(a, 3)
    st.MIN_BUCKET = 32                                   # small context buckets: the longest sequence outgrows one during the test
    gen = torch.Generator().manual_seed(2)
    prompts = [torch.randint(5, 4000, (n,), generator=gen).tolist() for n in (13, 30, 7)]
    sa, sb = [a.new_sequence() for _ in prompts], [b.new_sequence() for _ in prompts]
    for m, seqs in ((a, sa), (b, sb)):
        for s, p in zip(seqs, prompts):
            m.forward_batch(m.kv.build_batch([s], [p]), False)
    members = [[0, 1, 2], [0, 1, 2], [0, 2], [2], [1, 2, 0], [1, 0]] + [[0, 1, 2]] * 6        # sequence 0 crosses position 16
    for step, idx in enumerate(members):
        toks = [100 + step + i for i in idx]
        got = st.step([sa[i] for i in idx], toks)
        want = b.forward_batch(b.kv.build_batch([sb[i] for i in idx], [[t] for t in toks]), True)
        assert got is not None and torch.allclose(got, want, atol=1e-5), step
        assert [sa[i].length for i in idx] == [sb[i].length for i in idx]
    assert len({b for _, b in st._state}) >= 2                           # more than one context bucket was used
    assert st.step([sa[0]] * 4, [1, 2, 3, 4]) is None                   # more sequences than the stepper was sized for
    # through the gatherer
    monkeypatch.setenv("TSB_GATHER_GRAPH", "1")
    real = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128, max_seqs=4)
    g = GatheredModel(real, 3, window_s=0.05)
    eos = [t for t in range(real.cfg.vocab) if real.tokenizer.is_eos(t)]
    got = {}

    def worker(i):
        with g.slot(i) as m:
            got[i] = generate(m, prompts[i], 6, eos_ids=eos, prefill_chunk=8)
    ths = [threading.Thread(target=worker, args=(i,)) for i in range(3)]
    [t.start() for t in ths]
    [t.join(timeout=120) for t in ths]
    assert g.graph_steps > 0
    for i, p in enumerate(prompts):
        real.reset_kv_cache()
        assert got[i] == generate(real, p, 6, eos_ids=eos)
    g.close()


def _leader_follower_main(rank, port, path, q):
    import torch.distributed as dist
    from datetime import timedelta

    from tensorsharp_b200.parallel.dist import Communicator
    from tensorsharp_b200.parallel.replicated import leader_factory, start_watchdog
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port, 2, rank == 0, timeout=timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=2, timeout=timedelta(seconds=30))
    comm = Communicator(rank, 2)
    wd = start_watchdog(comm, 0.6, store=store)
    if rank == 1:
        from tensorsharp_b200.models.base import ModelBase
        from tensorsharp_b200.parallel.replicated import _bcast
        op, args = _bcast(comm)                         # "load"
        m = ModelBase.create(args[0], "cpu", tp_rank=1, tp_size=2, comm=comm, **args[1])
        op, args = _bcast(comm)                         # the first forward: mirrored
        m.forward(args[0], args[1])
        wd.stop()
        wd.hb.leave()                                   # leaves between steps, nothing in flight
        q.put(("left", op))
        time.sleep(3.0)
        return
    m = leader_factory(comm, watchdog=wd)(path, "cpu", max_context=64)
    first = m.forward([5, 6, 7])
    err = None
    deadline = time.time() + 20
    while err is None and time.time() < deadline:
        try:
            time.sleep(1.5)                             # several watchdog periods: the departure has been seen
            m.forward([8])                              # must not hang: the follower is gone
        except RankFailureError as e:
            err = sorted(e.stale)
    q.put(("leader", (first is not None, err)))


def test_front_end_fails_a_call_instead_of_waiting_for_a_departed_follower(tiny_qwen3_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31000 + os.getpid() % 2000
    ps = [ctx.Process(target=_leader_follower_main, args=(r, port, tiny_qwen3_path, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    assert got["left"] == "forward"
    assert got["leader"] == (True, [1])


def test_heartbeat_tolerates_a_peer_that_registers_late():
    """A peer whose key is still absent counts as one more unchanged value: it is stale only after ``timeout_s``."""
    store, now = DictStore(), [0.0]
    hb0, hb1 = Heartbeat(store, 0, 2, clock=lambda: now[0]), Heartbeat(store, 1, 2, clock=lambda: now[0])
    hb0.beat()
    for t in (0.0, 0.2, 0.4, 5.0, 29.0):            # polls while rank 1 has not registered: inside the timeout
        now[0] = t
        assert hb0.stale_ranks(30.0) == set()
    now[0] = 29.5
    hb1.beat()                                      # registers late, but in time
    assert hb0.stale_ranks(30.0) == set()
    now[0] = 55.0
    assert hb0.stale_ranks(30.0) == set()           # 25.5 s since its first beat
    now[0] = 61.0
    assert hb0.stale_ranks(30.0) == {1}
    # a peer that never registers is reported once the timeout has passed
    store2 = DictStore()
    lone = Heartbeat(store2, 0, 2, clock=lambda: now[0])
    now[0] = 100.0
    assert lone.stale_ranks(30.0) == set()
    now[0] = 131.0
    assert lone.stale_ranks(30.0) == {1}


def test_token_loop_raises_when_a_device_wait_ran_out(tmp_path):
    """The kernels' bounded waits only leave a status word behind; the token loop has to look at it.  With a stand-in
    status word set, the next ``forward`` ends in ExchangeTimeoutError instead of streaming tokens computed from zeros."""
    import torch
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.parallel.errors import ExchangeTimeoutError
    p = str(tmp_path / "m.gguf")
    synth.write_qwen3(p, **synth.QWEN3_TINY, device="cpu")
    m = ModelBase.create(p, device="cpu")
    word = torch.zeros(1, dtype=torch.int32)
    m.status_sources = lambda: [("stand-in exchange", word)]
    m.forward([1, 2, 3])                              # healthy: nothing raised
    word[0] = 3
    with pytest.raises(ExchangeTimeoutError) as e:
        m.forward([4])
    assert e.value.code == 3 and "stand-in exchange" in str(e.value)
    m.close()


def test_moe_tile_list_covers_every_routed_row_once():
    """The device-side work list of the grouped expert GEMM (no host read-back): every row of a local expert is in exactly
    one tile of its expert, tiles hold at most ``bn`` rows, skipped rows (-1) are in none, unused entries are marked -1."""
    import torch
    from tensorsharp_b200.ops.functional import moe_tile_list
    g = torch.Generator().manual_seed(5)
    for n_groups, P, bn in ((4, 100, 32), (8, 37, 64), (3, 1000, 128), (5, 64, 32)):
        flat = torch.randint(-1, n_groups, (P,), generator=g)
        flat[flat == 1] = 0                                   # one group without rows
        order, tiles = moe_tile_list(flat, n_groups, bn)
        assert tiles.dtype == torch.int32 and tiles.shape == ((P + bn - 1) // bn + n_groups, 3)
        sorted_groups = flat[order]
        seen = torch.zeros(P, dtype=torch.int32)
        for e, a, b in tiles.tolist():
            if e < 0:
                continue
            assert 0 < b - a and a >= 0 and b <= P
            rows = min(bn, b - a)
            assert (sorted_groups[a:a + rows] == e).all()
            seen[a:a + rows] += 1
        assert torch.equal(seen, (sorted_groups >= 0).to(torch.int32))
