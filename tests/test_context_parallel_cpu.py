"""Context-parallel prefill over gloo ranks: a prompt dealt to 2 and 3 ranks gives the logits of one process, every
rank ends with the whole cache (so decode steps agree), and a second prompt on a non-empty sequence works too."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_bounds_and_shard_batch(tiny_qwen3_path):
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.parallel.context import shard_batch, shard_bounds
    for T, n in ((19, 3), (8, 4), (5, 5), (100, 7)):
        b = [shard_bounds(T, n, r) for r in range(n)]
        assert b[0][0] == 0 and b[-1][1] == T and all(b[i][1] == b[i + 1][0] for i in range(n - 1))
        assert max(y - x for x, y in b) - min(y - x for x, y in b) <= 1
    from tensorsharp_b200.parallel.context import balanced_ranges
    for T, n in ((64, 4), (45, 2), (1000, 8)):
        pieces = sorted(r for k in range(n) for r in balanced_ranges(T, n, k))
        assert pieces[0][0] == 0 and pieces[-1][1] == T and all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
        # keys seen under a causal mask: every rank within a few percent of the mean
        work = [sum((b - a) * (a + b) / 2 for a, b in balanced_ranges(T, n, k)) for k in range(n)]
        assert max(work) / (sum(work) / n) < 1.1
    assert balanced_ranges(5, 4, 3) == [(4, 5)]                           # too short to cut twice per rank: one slice each
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    seq = m.new_sequence()
    m.kv.build_batch([seq], [[1, 2, 3]])
    batch = m.kv.build_batch([seq], [list(range(10, 20))])
    sub = shard_batch(batch, 4, 7)
    assert sub.tokens.tolist() == [14, 15, 16] and sub.positions.tolist() == [7, 8, 9]
    assert sub.h_kv_lens == (10,) and sub.max_q_len == 3 and not sub.is_decode
    assert sub.slots.tolist() == batch.slots[4:7].tolist()
    two = shard_batch(batch, [(0, 2), (8, 10)])                           # two pieces: two packed rows over one block table
    assert two.tokens.tolist() == [10, 11, 18, 19] and two.h_cu_q == (0, 2, 4) and two.h_kv_lens == (5, 13)
    assert two.last_idx.tolist() == [1, 3] and two.block_table.shape[0] == 2 and two.max_q_len == 2


def _worker(rank, world, port, path, prompt, more, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      TSB_CP_MIN_TOKENS="4")
    import torch.distributed as dist
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.parallel.dist import Communicator
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = ModelBase.create(path, "cpu", max_context=128, cp_comm=Communicator(rank, world))
        l1 = m.forward(prompt)
        l2 = m.forward([int(l1.argmax())])                 # decode on every rank from its own, now complete, cache
        l3 = m.forward(more)                               # a further prompt on the non-empty sequence
        torch.save((l1, l2, l3), f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_prefill_matches_single_process(tiny_qwen3_path, tmp_path, world):
    from tensorsharp_b200.models.base import ModelBase
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 4096, (23,), generator=g).tolist()
    more = torch.randint(0, 4096, (9,), generator=g).tolist()
    single = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128)
    s1 = single.forward(prompt)
    s2 = single.forward([int(s1.argmax())])
    s3 = single.forward(more)
    out = str(tmp_path / "cp.pt")
    mp.spawn(_worker, args=(world, _free_port(), tiny_qwen3_path, prompt, more, out), nprocs=world, join=True)
    for r in range(world):
        l1, l2, l3 = torch.load(f"{out}.{r}")
        assert torch.allclose(l1, s1, atol=5e-3), r
        assert torch.allclose(l2, s2, atol=5e-3), r
        assert torch.allclose(l3, s3, atol=5e-3), r


@pytest.mark.parametrize("family", ["gptoss", "gemma3", "gemma4"])
def test_families_with_windows_sinks_and_shared_caches(tmp_path, family):
    """The general route (each rank runs its slice through the model's ordinary layers, the cache of every layer is
    completed between the cache write and the attention): sliding windows, attention sinks, experts, layers that read
    another layer's cache and per-layer inputs all behave as in one process."""
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    path = str(tmp_path / "m.gguf")
    if family == "gptoss":
        synth.write_gptoss(path, n_layers=3, device="cpu")
    else:
        synth.write_gemma(path, arch=family, device="cpu")
    g = torch.Generator().manual_seed(12)
    prompt = torch.randint(0, 4096, (45,), generator=g).tolist()
    more = torch.randint(0, 4096, (7,), generator=g).tolist()
    single = ModelBase.create(path, "cpu", max_context=128)
    s1 = single.forward(prompt)
    s2 = single.forward([int(s1.argmax())])
    s3 = single.forward(more)
    out = str(tmp_path / "cp.pt")
    mp.spawn(_worker, args=(2, _free_port(), path, prompt, more, out), nprocs=2, join=True)
    for r in range(2):
        l1, l2, l3 = torch.load(f"{out}.{r}")
        assert torch.allclose(l1, s1, atol=2e-2) and torch.allclose(l2, s2, atol=2e-2) and torch.allclose(l3, s3, atol=2e-2), r


def test_models_without_the_path_refuse_the_group(tmp_path):
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.parallel.dist import Communicator
    path = str(tmp_path / "g.gguf")
    synth.write_qwen35(path, device="cpu")
    with pytest.raises(ValueError, match="context-parallel"):
        ModelBase.create(path, "cpu", max_context=64, cp_comm=Communicator(0, 2))


def _cli_worker(rank, world, port, path, prompt_file, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      TSB_CP_MIN_TOKENS="4")
    import io

    from tensorsharp_b200.cli.main import Console, main
    out, err = io.StringIO(), io.StringIO()
    rc = main(["--model", path, "--backend", "cpu", "--cp", str(world), "--input", prompt_file, "--max-tokens", "5",
               "--log-file", "off"], Console(out, err))
    torch.save((rc, out.getvalue(), err.getvalue()), f"{out_path}.{rank}")


def test_cli_with_context_parallel_ranks(tiny_qwen3_path, tmp_path):
    """``--cp 2``: both processes run the CLI's loop, the prompt is dealt to them, rank 0 prints what one process prints."""
    import io

    from tensorsharp_b200.cli.main import Console, main
    prompt = tmp_path / "p.txt"
    prompt.write_text("Hello there, this prompt is long enough to be dealt to two ranks.")
    out = io.StringIO()
    assert main(["--model", tiny_qwen3_path, "--backend", "cpu", "--input", str(prompt), "--max-tokens", "5", "--log-file", "off"],
                Console(out, io.StringIO())) == 0
    res = str(tmp_path / "cli_cp")
    mp.spawn(_cli_worker, args=(2, _free_port(), tiny_qwen3_path, str(prompt), res), nprocs=2, join=True)
    rc0, out0, err0 = torch.load(f"{res}.0")
    rc1, out1, _ = torch.load(f"{res}.1")
    assert rc0 == 0 and rc1 == 0, err0
    assert out0 == out.getvalue() and out1 == ""
    with pytest.raises(ValueError, match="needs 2 processes"):
        from tensorsharp_b200.cli.args import parse_cli_args
        from tensorsharp_b200.cli.main import load_model
        from tensorsharp_b200.runtime.logging import NULL_LOGGER
        load_model(parse_cli_args(["--model", tiny_qwen3_path, "--backend", "cpu", "--cp", "2"]), NULL_LOGGER)   # one process only
