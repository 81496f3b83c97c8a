"""Recovery after an in-kernel exchange gave up waiting for a peer, without a GPU: the failure is a stand-in status
word or an exception raised on the host.  The request fails with a typed error; the model drops its exchange objects
(closing their symmetric buffers) so the next use rebuilds them, forgets its captured-graph steppers, clears the status
words and resets its cache; the serving layer resets its sessions and keeps serving with the weights still loaded."""
import pytest
import torch

from tensorsharp_b200.models.base import ModelBase
from tensorsharp_b200.parallel.errors import ExchangeTimeoutError
from tensorsharp_b200.runtime.chat import ChatMessage

from tests.test_server_cpu import GREEDY, make_service, run_chat


class FakeExchange:
    def __init__(self):
        self.closed = 0

    def close(self):
        self.closed += 1


def test_model_drops_its_exchanges_and_resets(tiny_qwen3_path):
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    want = m.forward([5, 9, 33, 7]).clone()
    a, b, c, d = FakeExchange(), FakeExchange(), FakeExchange(), FakeExchange()
    m._tpx, m._tpseq = a, b
    m.__dict__["_cpa"], m.__dict__["_mega"] = c, d
    m.__dict__["_steppers"] = {1: object()}
    word = torch.tensor([7], dtype=torch.int32)
    m.status_sources = lambda: [("stand-in exchange", word)]
    with pytest.raises(ExchangeTimeoutError, match="stand-in exchange"):
        m.poll_status(force=True)
    assert m.cache_length == 4
    assert m.recover_exchanges() == 4
    assert (a.closed, b.closed, c.closed, d.closed) == (1, 1, 1, 1)
    assert m.tp_exchange() is None and getattr(m, "_tpseq", None) is None and "_steppers" not in m.__dict__
    assert int(word) == 0 and m.cache_length == 0
    m.poll_status(force=True)                                  # nothing pending any more
    assert torch.allclose(m.forward([5, 9, 33, 7]), want, atol=1e-5)     # weights untouched, cache rebuilt from nothing
    assert m.recover_exchanges() == 0                          # nothing to close: harmless to call again


def test_a_disabled_exchange_marker_is_not_closed(tiny_qwen3_path):
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=64)
    m._tpx = False                                             # "no fused exchange for this model" marker
    m.__dict__["_mega"] = False
    assert m.recover_exchanges() == 0


def test_service_fails_the_request_recovers_and_serves_the_next_one():
    svc, model = make_service()
    recovered = []
    model.recover_exchanges = lambda: recovered.append(1) or 2
    hist = [ChatMessage(role="user", content="hello")]
    text, _ = run_chat(svc, hist, "fine")
    assert text == "fine" and svc._intrinsic.kv_cache.count > 0
    # the third decode step of the next turn reports a wait that ran out
    calls = {"n": 0}
    plain_forward = model.forward

    def failing_forward(tokens, want_logits=True):
        calls["n"] += 1
        if calls["n"] == 3:
            raise ExchangeTimeoutError("tensor-parallel mailbox exchange", 12)
        return plain_forward(tokens, want_logits)
    model.forward = failing_forward
    model.say("this reply is cut short")
    hist2 = hist + [ChatMessage(role="assistant", content="fine"), ChatMessage(role="user", content="again")]
    with pytest.raises(ExchangeTimeoutError):
        list(svc.chat_stream_with_metrics(hist2, 32, sampling=GREEDY))
    assert recovered == [1]
    from tensorsharp_b200.server.metrics import METRICS
    assert METRICS.exchange_recoveries >= 1 and "tensorsharp_exchange_recoveries_total" in METRICS.render()
    assert svc._intrinsic.kv_cache.count == 0 and not svc._intrinsic.tracked_history       # nothing of the failed turn is trusted
    # the service keeps serving: same weights, fresh cache (a full prefill, no prefix reuse)
    model.forward = plain_forward
    text, last = run_chat(svc, hist, "back again")
    assert text == "back again" and last.done
    assert not any(op[0] == "truncate" for op in model.ops)


def test_leader_tells_the_followers_to_recover(monkeypatch):
    """The front end's model announces the recovery like every other state-changing call, and a follower carries it out
    on its own shard (the broadcast itself is replaced by a list here; the gloo ranks are covered elsewhere)."""
    from tensorsharp_b200.parallel import replicated as R

    class Shard:
        def __init__(self):
            self.calls = []

        def recover_exchanges(self):
            self.calls.append("recover")
            return 3

        def reset_kv_cache(self):
            self.calls.append("reset")

    sent = []
    monkeypatch.setattr(R, "_bcast", lambda comm, obj=None: sent.append(obj))
    leader_shard = Shard()
    leader = R.LeaderModel(leader_shard, comm=object())
    assert leader.recover_exchanges() == 3
    assert sent == [("recover", ())] and leader_shard.calls == ["recover"]
    # the follower side: replay the leader's commands
    follower_shard = Shard()
    script = iter([("load", ("m.gguf", {})), ("recover", ()), ("reset", ()), ("stop", ())])
    monkeypatch.setattr(R, "_bcast", lambda comm, obj=None: next(script))

    class Comm:
        rank, size = 1, 2
        device = torch.device("cpu")
    n = R.follower_main(Comm(), create=lambda path, dev, **kw: follower_shard)
    assert n == 4 and follower_shard.calls == ["recover", "reset"]


def test_cli_helper_recovers_only_after_an_exchange_failure():
    from tensorsharp_b200.cli.main import recover_if_exchange_failed
    from tensorsharp_b200.runtime.logging import NULL_LOGGER

    class M:
        n = 0

        def recover_exchanges(self):
            self.n += 1
            return 1
    m = M()
    assert recover_if_exchange_failed(m, ValueError("bad request"), NULL_LOGGER) is False and m.n == 0
    assert recover_if_exchange_failed(m, ExchangeTimeoutError("sequence-parallel prefill exchange", 10), NULL_LOGGER) is True and m.n == 1
