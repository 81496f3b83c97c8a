"""End-to-end: the tiny Qwen3 graph on the CUDA kernels against the CPU oracle path."""
import pytest
import torch

from tensorsharp_b200.models.base import ModelBase

pytestmark = pytest.mark.gpu


def test_tiny_qwen3_cuda_matches_cpu(tiny_qwen3_path):
    cpu = ModelBase.create(tiny_qwen3_path, "cpu", max_context=512)
    gpu = ModelBase.create(tiny_qwen3_path, "cuda", max_context=512)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 4096, (64,), generator=g).tolist()
    lc, lg = cpu.forward(prompt), gpu.forward(prompt).cpu()
    assert float((lc - lg).norm() / lc.norm()) < 3e-2
    # decode steps (GEMV path) stay close to the oracle when both follow the oracle's tokens
    t = int(lc.argmax())
    for _ in range(6):
        lc, lg = cpu.forward([t]), gpu.forward([t]).cpu()
        assert float((lc - lg).norm() / lc.norm()) < 3e-2
        t = int(lc.argmax())
    # chunked prefill == one-shot prefill
    gpu.reset_kv_cache()
    l2 = gpu.forward_refill(prompt, chunk=24).cpu()
    gpu.reset_kv_cache()
    l1 = gpu.forward(prompt).cpu()
    assert float((l1 - l2).norm() / l1.norm()) < 2e-2


def test_batched_decode_matches_single(tiny_qwen3_path):
    m = ModelBase.create(tiny_qwen3_path, "cuda", max_context=256, max_seqs=4)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (5, 17, 33)]
    seqs = [m.kv.new_seq() for _ in prompts]
    lb = m.forward_batch(m.kv.build_batch(seqs, prompts)).cpu()
    for i, p in enumerate(prompts):
        m.reset_kv_cache()
        ls = m.forward(p).cpu()
        assert float((ls - lb[i]).norm() / ls.norm()) < 2e-2


def test_sampled_decode_inside_the_graph(tiny_qwen3_path):
    """Sampling runs inside the captured step: the same seed reproduces the run, another seed does not,
    every drawn id is inside the vocabulary, and the penalty table counts exactly the drawn tokens."""
    from tensorsharp_b200.ops import functional as F
    from tensorsharp_b200.runtime.engine import DecodeGraph
    from tensorsharp_b200.runtime.sampling import SamplingConfig

    def run(seed):
        m = ModelBase.create(tiny_qwen3_path, "cuda", max_context=256, max_seqs=4)
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (9, 21)]
        seqs = [m.kv.new_seq() for _ in prompts]
        first = F.argmax(m.forward_batch(m.kv.build_batch(seqs, prompts)))
        cfg = SamplingConfig(temperature=0.9, top_k=50, top_p=0.95, min_p=0.0, repetition_penalty=1.1, seed=seed)
        dg = DecodeGraph(m, seqs, 40, sampling=cfg)
        dg.set_tokens(first.tolist())
        dg.capture()
        out = [dg.step().clone() for _ in range(24)]
        torch.cuda.synchronize()
        return torch.stack(out).cpu(), dg.counts.cpu(), dg.ngen.cpu()

    a, ca, na = run(5)
    b, _, _ = run(5)
    c, _, _ = run(6)
    assert torch.equal(a, b)
    assert not torch.equal(a, c)
    assert int(a.min()) >= 0 and int(a.max()) < 4096
    assert na.tolist() == [24, 24]
    for r in range(2):
        assert torch.equal(torch.bincount(a[:, r].long(), minlength=ca.shape[1])[:ca.shape[1]].int(), ca[r])


def test_single_token_forward_replays_a_graph(tiny_qwen3_path, monkeypatch):
    """``forward([t])`` goes through a captured graph: same logits as the eager step, across a truncation,
    a further prefill and the growth of the context past the captured bucket."""
    from tensorsharp_b200.runtime import engine
    monkeypatch.setattr(engine.GraphStepper, "MIN_BUCKET", 64)
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 4096, (40,), generator=g).tolist()

    def run(graph: bool):
        monkeypatch.setenv("TSB_GRAPH_FORWARD", "1" if graph else "0")
        m = ModelBase.create(tiny_qwen3_path, "cuda", max_context=512)
        out = [m.forward(prompt).clone()]
        t = int(out[-1].argmax())
        for _ in range(40):                                   # 40 + 40 tokens: crosses the 64-position bucket
            out.append(m.forward([t]).clone())
            t = int(out[-1].argmax())
        m.truncate_kv_cache(30)                               # an edited turn: shorter cache, then new tokens
        out.append(m.forward(prompt[30:36]).clone())
        t = int(out[-1].argmax())
        for _ in range(5):
            out.append(m.forward([t]).clone())
            t = int(out[-1].argmax())
        m.reset_kv_cache()
        out.append(m.forward([7]).clone())                    # a single-token prompt on an empty cache
        return torch.stack(out).cpu(), ("_steppers" in m.__dict__)

    eager, used0 = run(False)
    graph, used1 = run(True)
    assert used1 and not used0
    err = (eager - graph).norm(dim=1) / eager.norm(dim=1)
    assert float(err.max()) < 2e-2, err
