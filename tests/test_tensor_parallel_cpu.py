"""Tensor-parallel sharding checked on CPU ranks (Gloo): two ranks must reproduce the
single-rank logits, and the shard arithmetic must tile every dimension exactly."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from tensorsharp_b200.parallel.dist import block_split, even_split, head_split


def test_shard_arithmetic_tiles_exactly():
    for n, parts in ((9728, 8), (151936, 8), (10, 3), (7, 8)):
        spans = [even_split(n, parts, r) for r in range(parts)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    spans = [block_split(9728, 256, 8, r) for r in range(8)]          # 38 super-blocks over 8 ranks
    assert [(e - s) // 256 for s, e in spans] == [5, 5, 5, 5, 5, 5, 4, 4]
    assert all(s % 256 == 0 for s, _ in spans) and spans[-1][1] == 9728
    (q, kv) = head_split(32, 8, 8, 3)
    assert q == (12, 16) and kv == (3, 4)
    with pytest.raises(ValueError):
        head_split(32, 8, 3, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, path, prompt, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.parallel.dist import Communicator
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = ModelBase.create(path, "cpu", max_context=128, tp_rank=rank, tp_size=world, comm=Communicator(rank, world))
        l1 = m.forward(prompt)
        t = int(l1.argmax())
        l2 = m.forward([t])
        if rank == 0:
            torch.save((l1, l2), out_path)
    finally:
        dist.destroy_process_group()


def test_tp2_matches_single_rank(tiny_qwen3_path, tmp_path):
    from tensorsharp_b200.models.base import ModelBase
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 4096, (19,), generator=g).tolist()
    single = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    s1 = single.forward(prompt)
    s2 = single.forward([int(s1.argmax())])
    out = str(tmp_path / "tp.pt")
    mp.spawn(_worker, args=(2, _free_port(), tiny_qwen3_path, prompt, out), nprocs=2, join=True)
    l1, l2 = torch.load(out)
    assert torch.allclose(l1, s1, atol=5e-3) and torch.allclose(l2, s2, atol=5e-3)


def test_head_split_replicates_kv_heads_when_ranks_outnumber_them():
    from tensorsharp_b200.parallel.dist import head_split
    assert head_split(32, 8, 4, 1) == ((8, 16), (2, 4))                       # the usual case: KV heads dealt, none shared
    got = [head_split(16, 2, 8, r) for r in range(8)]                         # 2 KV heads over 8 ranks: 4 ranks share each
    assert [q for q, _ in got] == [(2 * r, 2 * r + 2) for r in range(8)]
    assert [k for _, k in got] == [(0, 1)] * 4 + [(1, 2)] * 4
    with pytest.raises(ValueError):
        head_split(16, 2, 3, 0)


@pytest.mark.parametrize("family", ["gptoss", "qwen35", "qwen35_one_kv_head", "nemotron", "gemma3", "gemma4"])
def test_other_families_shard_over_two_ranks(tmp_path, family):
    """Head / FFN shards (Gemma, GPT-OSS attention) and expert ranges (GPT-OSS, Qwen3.5, Nemotron-H, Gemma 4) on two gloo
    ranks give the logits of one process, for a prompt and a decode step."""
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    p = str(tmp_path / "m.gguf")
    if family == "gptoss":
        synth.write_gptoss(p, n_layers=2, device="cpu")
    elif family == "qwen35":
        synth.write_qwen35(p, device="cpu")
    elif family == "qwen35_one_kv_head":
        synth.write_qwen35(p, n_kv_heads=1, device="cpu")                     # both ranks hold the KV head, two query heads each
    elif family == "nemotron":
        synth.write_nemotron_h(p, device="cpu")
    else:
        synth.write_gemma(p, arch=family, device="cpu")
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, 4096, (19,), generator=g).tolist()
    single = ModelBase.create(p, "cpu", max_context=128)
    s1 = single.forward(prompt)
    s2 = single.forward([int(s1.argmax())])
    out = str(tmp_path / "tp.pt")
    mp.spawn(_worker, args=(2, _free_port(), p, prompt, out), nprocs=2, join=True)
    l1, l2 = torch.load(out)
    scale = float(s1.abs().max())
    assert float((l1 - s1).abs().max()) < 2e-2 * scale and float((l2 - s2).abs().max()) < 2e-2 * scale


def _pp_worker(rank, world, port, path, prompt, n_new, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.parallel import pipeline
    from tensorsharp_b200.parallel.dist import Communicator
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = ModelBase.create(path, "cpu", max_context=128, pp_rank=rank, pp_size=world, pp_comm=Communicator(rank, world))
        held = [k is not None for k in m.kv.k]
        toks = pipeline.generate(m, prompt, n_new, prefill_chunk=8)       # chunked prefill crosses the stages too
        torch.save((toks, held, m.layer_range, m.tok_emb is not None, m.lm_head is not None), f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_stages_match_single_process(tiny_qwen3_path, tmp_path, world):
    """Layer ranges on successive gloo ranks, the residual stream sent stage to stage, the sampled token
    broadcast back: every rank returns the tokens the single-process model generates, and each stage
    holds only its own layers' KV cache."""
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import generate
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 4096, (21,), generator=g).tolist()
    single = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    want = generate(single, prompt, 6)
    out = str(tmp_path / "pp.pt")
    mp.spawn(_pp_worker, args=(world, _free_port(), tiny_qwen3_path, prompt, 6, out), nprocs=world, join=True)
    n_layers = single.cfg.n_layers
    covered = []
    for r in range(world):
        toks, held, (l0, l1), has_emb, has_head = torch.load(f"{out}.{r}")
        assert toks == want
        assert held == [l0 <= l < l1 for l in range(n_layers)]
        covered += list(range(l0, l1))
        assert has_head == (r == world - 1)
        assert has_emb == (r == 0 or r == world - 1)          # tied embeddings: the last stage needs them for the lm_head
    assert covered == list(range(n_layers))


G4 = dict(arch="gemma4", n_layers=8, head_dim_global=128, kv_heads_global=1, rot_global=64, shared_kv=2, ple_dim=32, n_experts=4, top_k=2)


@pytest.mark.parametrize("family", ["gptoss", "qwen35", "nemotron", "gemma3", "gemma4"])
def test_other_families_pipeline_stages_match_single_process(tmp_path, family):
    """The mixture-of-experts family (sliding windows follow the global layer index, the last layer's last-token
    shortcut runs on the last stage only) and the two families with recurrent layers (state slots live with their
    layers' stage) over two stages."""
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import generate
    p = str(tmp_path / "m.gguf")
    if family == "gptoss":
        synth.write_gptoss(p, n_layers=3, device="cpu")
    elif family == "qwen35":
        synth.write_qwen35(p, device="cpu")
    elif family == "gemma3":
        synth.write_gemma(p, arch="gemma3", device="cpu")
    elif family == "gemma4":
        synth.write_gemma(p, device="cpu", **G4)      # shared-KV layers 6, 7 read layer 4: all on the second stage; per-layer inputs on both
    else:
        synth.write_nemotron_h(p, device="cpu")
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, 4096, (21,), generator=g).tolist()
    single = ModelBase.create(p, "cpu", max_context=128)
    want = generate(single, prompt, 5)
    has_kv = [k is not None for k in single.kv.k]
    out = str(tmp_path / "pp_moe.pt")
    mp.spawn(_pp_worker, args=(2, _free_port(), p, prompt, 5, out), nprocs=2, join=True)
    for r in range(2):
        toks, held, (l0, l1), _, has_head = torch.load(f"{out}.{r}")
        assert toks == want and has_head == (r == 1)
        if family != "gemma4":                          # (its shared-KV layers alias their donor's tensors)
            assert held == [has_kv[l] and l0 <= l < l1 for l in range(single.cfg.n_layers)]


def test_pipeline_refuses_a_cut_between_a_shared_kv_layer_and_its_donor(tmp_path):
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    p = str(tmp_path / "g.gguf")
    synth.write_gemma(p, device="cpu", **G4)
    with pytest.raises(ValueError, match="shared-KV"):
        ModelBase.create(p, "cpu", max_context=64, pp_rank=3, pp_size=4)          # layers 6, 7 without layer 4
    with pytest.raises(ValueError):
        ModelBase.create(p, "cpu", max_context=64, pp_rank=0, pp_size=2, tp_size=2)   # stages are not combined with weight shards


def _serve_worker(rank, world, port, path, out_path, mode="tp"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), TSB_CP_MIN_TOKENS="4")
    import torch.distributed as dist
    from tensorsharp_b200.parallel.dist import Communicator
    from tensorsharp_b200.parallel import replicated
    from tensorsharp_b200.parallel.replicated import follower_main, layout_create, shutdown_followers
    create = layout_create(mode)

    def leader_factory(comm):
        return replicated.leader_factory(comm, create)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = Communicator(rank, world)
    try:
        if rank != 0:
            n = follower_main(comm, create=create)
            torch.save(n, f"{out_path}.{rank}")
            return
        from tensorsharp_b200.runtime.chat import ChatMessage
        from tensorsharp_b200.runtime.sampling import SamplingConfig
        from tensorsharp_b200.server.model_service import ModelService
        svc = ModelService(model_factory=leader_factory(comm), max_context=256)
        svc.load_model(path, None, "cpu")
        greedy = SamplingConfig.greedy()
        hist = [ChatMessage(role="user", content="Hello there")]
        first = "".join(svc.chat_stream(hist, 6, sampling=greedy))
        hist += [ChatMessage(role="assistant", content=first), ChatMessage(role="user", content="and again")]
        items = list(svc.chat_stream_with_metrics(hist, 5, sampling=greedy))
        second = "".join(i.piece for i in items if i.piece)
        # recovery after an exchange failure (injected here: no device is involved): every rank drops its exchanges and
        # empties its cache at the same point, and the same chat gives the same text again
        from tensorsharp_b200.parallel.errors import ExchangeTimeoutError
        svc.recover_after_exchange_failure(ExchangeTimeoutError("injected", 1))
        again = "".join(svc.chat_stream([ChatMessage(role="user", content="Hello there")], 6, sampling=greedy))
        # two resident chats: sequences are created, bound and freed on every rank alike
        from tensorsharp_b200.server.sessions import SessionManager
        svc2 = ModelService(model_factory=leader_factory(comm), max_context=256, max_sessions=2)
        svc.close()
        svc2.load_model(path, None, "cpu")
        mgr = SessionManager()
        sa, sb = mgr.create_session(), mgr.create_session()
        ta = "".join(svc2.chat_stream([ChatMessage(role="user", content="Hello there")], 4, sampling=greedy, session=sa))
        tb = "".join(svc2.chat_stream([ChatMessage(role="user", content="Something else")], 4, sampling=greedy, session=sb))
        ta2 = "".join(svc2.chat_stream([ChatMessage(role="user", content="Hello there"), ChatMessage(role="assistant", content=ta),
                                        ChatMessage(role="user", content="and again")], 3, sampling=greedy, session=sa))
        svc2.dispose_session(sb)
        svc2.close()
        shutdown_followers(comm)
        torch.save((first, second, ta, tb, ta2, again), f"{out_path}.0")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["tp", "pp", "cp"])
def test_front_end_on_rank0_with_follower_shards(tiny_qwen3_path, tmp_path, mode):
    """The model service runs on rank 0 only; the follower rank mirrors every call on its part of the model (a weight
    shard, a range of layers, or a whole copy that takes its slice of each prompt), so a two-turn chat (prefill,
    decode, KV reuse on the second turn) gives the single-process text."""
    from tensorsharp_b200.runtime.chat import ChatMessage
    from tensorsharp_b200.runtime.sampling import SamplingConfig
    from tensorsharp_b200.server.model_service import ModelService
    svc = ModelService(max_context=256)
    svc.load_model(tiny_qwen3_path, None, "cpu")
    greedy = SamplingConfig.greedy()
    hist = [ChatMessage(role="user", content="Hello there")]
    first = "".join(svc.chat_stream(hist, 6, sampling=greedy))
    hist += [ChatMessage(role="assistant", content=first), ChatMessage(role="user", content="and again")]
    second = "".join(svc.chat_stream(hist, 5, sampling=greedy))
    svc.close()
    out = str(tmp_path / "serve.pt")
    mp.spawn(_serve_worker, args=(2, _free_port(), tiny_qwen3_path, out, mode), nprocs=2, join=True)
    got = torch.load(f"{out}.0")
    assert got[:2] == (first, second)
    assert got[2] == first[:len(got[2])] or len(got[2]) > 0        # same prompt, fewer tokens: a prefix of the first answer
    assert all(isinstance(t, str) for t in got[2:])
    assert got[5] == first                      # after the recovery on both ranks
    assert torch.load(f"{out}.1") > 10          # the follower executed the leader's commands


def _cli_pp_worker(rank, world, port, path, prompt_file, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    import io

    from tensorsharp_b200.cli.main import Console, main
    out, err = io.StringIO(), io.StringIO()
    rc = main(["--model", path, "--backend", "cpu", "--pp", str(world), "--input", prompt_file, "--max-tokens", "5",
               "--log-file", "off"], Console(out, err))
    torch.save((rc, out.getvalue(), err.getvalue()), f"{out_path}.{rank}")


def test_cli_over_pipeline_stages(tiny_qwen3_path, tmp_path):
    """``--pp 2``: the CLI's own token loop runs on every stage (the last stage broadcasts the logits), rank 0
    prints what the single-process CLI prints, the other rank stays silent."""
    import io

    from tensorsharp_b200.cli.main import Console, main
    prompt = tmp_path / "p.txt"
    prompt.write_text("Hello there")
    out = io.StringIO()
    assert main(["--model", tiny_qwen3_path, "--backend", "cpu", "--input", str(prompt), "--max-tokens", "5", "--log-file", "off"],
                Console(out, io.StringIO())) == 0
    res = str(tmp_path / "cli_pp")
    mp.spawn(_cli_pp_worker, args=(2, _free_port(), tiny_qwen3_path, str(prompt), res), nprocs=2, join=True)
    rc0, out0, err0 = torch.load(f"{res}.0")
    rc1, out1, _ = torch.load(f"{res}.1")
    assert rc0 == 0 and rc1 == 0, err0
    assert out0 == out.getvalue() and out1 == ""


def _embed_worker(rank, world, port, path, mode, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from tensorsharp_b200.parallel.dist import Communicator
    from tensorsharp_b200.parallel.replicated import follower_main, layout_create, leader_factory, shutdown_followers
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = Communicator(rank, world)
    try:
        create = layout_create(mode)
        if rank != 0:
            follower_main(comm, create=create)
            return
        m = leader_factory(comm, create)(path, "cpu", max_context=64)
        torch.manual_seed(3)
        m.set_vision_embeddings(torch.randn(3, m.cfg.hidden) * 0.1, 2)
        out = m.forward([5, 6, 7, 8, 9, 10, 11]).clone()
        m.close()
        shutdown_followers(comm)
        torch.save(out, out_path)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["tp", "pp"])
def test_leader_hands_image_embeddings_to_the_followers(tiny_qwen3_path, tmp_path, mode):
    from tensorsharp_b200.models.base import ModelBase
    single = ModelBase.create(tiny_qwen3_path, "cpu", max_context=64)
    torch.manual_seed(3)
    single.set_vision_embeddings(torch.randn(3, single.cfg.hidden) * 0.1, 2)
    want = single.forward([5, 6, 7, 8, 9, 10, 11])
    out = str(tmp_path / "emb.pt")
    mp.spawn(_embed_worker, args=(2, _free_port(), tiny_qwen3_path, mode, out), nprocs=2, join=True)
    assert torch.allclose(torch.load(out), want, atol=5e-3)
