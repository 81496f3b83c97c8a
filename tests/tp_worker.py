"""One rank of the multi-GPU tensor-parallel checks (launched by test_tp_fused_gpu.py through
``python -m torch.distributed.run``; not collected by pytest).  Prints one ``TPCHECK`` JSON line
on rank 0."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main():
    from tensorsharp_b200.parallel.dist import init_from_env
    comm = init_from_env()
    if os.environ.get("TSB_WORKER_MODE") == "pipeline":
        check_pipeline(sys.argv[1], comm)
        comm.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    if os.environ.get("TSB_WORKER_MODE") == "mega":
        check_mega(sys.argv[1], comm)
        comm.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    if os.environ.get("TSB_WORKER_MODE") == "families":
        for path in sys.argv[1:]:
            check_family(path, comm)
        comm.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    if os.environ.get("TSB_WORKER_MODE") == "cp_model":
        check_context_parallel_model(sys.argv[1], comm)
        comm.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    check_context_parallel(comm)
    for path in sys.argv[1:]:
        check_model(path, comm)
    comm.barrier()
    torch.cuda.synchronize()
    os._exit(0)          # skip NCCL teardown: it can block while captured graphs still hold its kernels


def check_pipeline(path, comm):
    """Layer ranges on successive GPUs with NCCL point-to-point hand-off: every rank must produce the
    tokens one GPU generates."""
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.parallel import pipeline
    from tensorsharp_b200.runtime.engine import generate
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, 4096, (150,), generator=g).tolist()
    single = ModelBase.create(path, comm.device, max_context=256)
    want = generate(single, prompt, 8)
    del single
    m = ModelBase.create(path, comm.device, max_context=256, pp_rank=comm.rank, pp_size=comm.size, pp_comm=comm)
    got = pipeline.generate(m, prompt, 8, prefill_chunk=64)
    same = torch.tensor([int(got == want)], device=comm.device)
    comm.all_reduce(same)
    if comm.rank == 0:
        print("PPCHECK " + json.dumps({"world": comm.size, "ranks_agree": int(same[0]), "tokens": got, "want": want}), flush=True)


def check_context_parallel(comm):
    """Sequence-sharded causal attention against plain attention over the whole sequence."""
    from tensorsharp_b200.ops import reference as ref
    from tensorsharp_b200.parallel.context import ContextParallelAttention
    n, Hq, Hkv, Dh = 160, 4, 2, 64
    world, rank, dev = comm.size, comm.rank, comm.device
    g = torch.Generator().manual_seed(5)
    q = torch.randn(world * n, Hq, Dh, generator=g).to(dev).bfloat16()
    k = torch.randn(world * n, Hkv, Dh, generator=g).to(dev).bfloat16()
    v = torch.randn(world * n, Hkv, Dh, generator=g).to(dev).bfloat16()
    cp = ContextParallelAttention(comm, 256, Hkv, Dh)
    sl = slice(rank * n, (rank + 1) * n)
    worst = 0.0
    for rep in range(4):                                           # several calls: both staging halves and the back-pressure
        out = cp.attention(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), Dh ** -0.5)
        want = ref.attention(q, k, v, torch.arange(world * n, device=dev), scale=Dh ** -0.5)[sl]
        worst = max(worst, float((out.float() - want.reshape(out.shape)).abs().max()))
    t = torch.tensor([worst, float(cp.status())], device=dev)
    import torch.distributed as dist
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print("CPCHECK " + json.dumps({"world": world, "max_err": float(t[0]), "status": int(t[1])}), flush=True)
    cp.close()


def check_context_parallel_model(path, comm):
    """A prompt dealt to the ranks of a context-parallel group against one GPU running it whole: the first prompt
    takes the peer-memory attention (new sequence, equal slices), the second one the exchange + local attention
    (sequence not empty, slices of unequal length); decode steps run on every rank from its own cache."""
    from tensorsharp_b200.models.base import ModelBase
    os.environ["TSB_CP_MIN_TOKENS"] = "64"
    g = torch.Generator().manual_seed(21)
    world = comm.size
    prompt = torch.randint(0, 4096, (256 * world,), generator=g).tolist()
    more = torch.randint(0, 4096, (100 * world + 1,), generator=g).tolist()
    single = ModelBase.create(path, comm.device, max_context=2048)
    want = [single.forward(prompt).float().clone()]
    want.append(single.forward([int(want[0].argmax())]).float().clone())
    want.append(single.forward(more).float().clone())
    del single
    m = ModelBase.create(path, comm.device, max_context=2048, cp_comm=comm)
    got = [m.forward(prompt).float().clone()]
    got.append(m.forward([int(want[0].argmax())]).float().clone())
    got.append(m.forward(more).float().clone())
    errs = [float((a - b).abs().max() / b.abs().max()) for a, b in zip(got, want)]
    cpa = m.__dict__.get("_cpa")
    t = torch.tensor(errs + [float(cpa.status()) if cpa is not None else -1.0], device=comm.device)
    import torch.distributed as dist
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if comm.rank == 0:
        print("CPMODEL " + json.dumps({"world": world, "rel_err": [float(x) for x in t[:3]], "status": int(t[3])}), flush=True)


def check_mega(path, comm):
    """The one-kernel decode step with tensor parallelism: the row-parallel projections store their tagged partial
    sums into every rank's buffer from inside the kernel.  Logits against one GPU (per-op path and fused step),
    bit-equality across ranks, and the same tokens through a captured graph."""
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import DecodeGraph
    rank, world = comm.rank, comm.size
    os.environ["TSB_GRAPH_FORWARD"] = "0"
    g = torch.Generator().manual_seed(13)
    prompt = torch.randint(0, 8192, (70,), generator=g).tolist()

    follow = [int(t) for t in torch.randint(0, 8192, (6,), generator=g)]     # every run is fed the same tokens

    def run(model):
        model.reset_kv_cache()
        out = [model.forward(prompt).float().clone()]
        for t in follow:
            out.append(model.forward([t]).float().clone())
        return torch.stack(out)

    model = ModelBase.create(path, comm.device, max_context=512, max_seqs=2, tp_rank=rank, tp_size=world, comm=comm)
    md = model.mega_decoder()
    tp = run(model)
    status = md.status() if md is not None else -1
    # every rank must hold the same logits bit for bit (same sums in the same order everywhere)
    lo, hi = tp.clone(), tp.clone()
    import torch.distributed as dist
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    spread = float((hi - lo).abs().max())
    model.reset_kv_cache()
    first = int(model.forward(prompt).argmax())
    dg = DecodeGraph(model, [model._seq()], 8)
    dg.set_tokens([first])
    dg.capture()
    graph_tokens = [first] + [int(dg.step()[0]) for _ in range(5)]
    model.reset_kv_cache()                                    # the same greedy run, one eager step at a time
    eager_tokens = [int(model.forward(prompt).argmax())]
    for _ in range(5):
        eager_tokens.append(int(model.forward([eager_tokens[-1]]).argmax()))
    status |= md.status() if md is not None else 0
    res = {"world": world, "engaged": md is not None, "status": status, "spread": spread, "graph_tokens": graph_tokens,
           "eager_tokens": eager_tokens, "launches_per_step": dg.launches_per_step}
    if rank == 0:
        os.environ["TSB_MEGA"] = "1"
        single = ModelBase.create(path, comm.device, max_context=512)
        ref_mega = run(single)
        single.__dict__["_mega"] = False
        ref_plain = run(single)
        rel = lambda a, b: float((a - b).norm() / b.norm())
        res["tp_vs_single_mega"] = rel(tp[1:], ref_mega[1:])
        res["tp_vs_single_plain"] = rel(tp[1:], ref_plain[1:])
        res["mega_vs_plain"] = rel(ref_mega[1:], ref_plain[1:])
        print("MEGACHECK " + json.dumps(res), flush=True)
    comm.barrier()


def check_family(path, comm):
    """Families whose row-parallel projections are summed by the mailbox all-reduce kernel (Gemma, Qwen3.5, Nemotron-H):
    decode-sized batches through the mailboxes against the NCCL path and one GPU, eagerly and inside a captured graph."""
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import DecodeGraph
    rank, world = comm.rank, comm.size
    os.environ["TSB_TP_FUSED"] = "1"
    g = torch.Generator().manual_seed(12)
    prompt = torch.randint(0, 4096, (9,), generator=g).tolist()

    def run(model, steps=5):
        model.reset_kv_cache()
        out = [model.forward(prompt).float().clone()]
        for _ in range(steps):
            out.append(model.forward([int(out[-1].argmax())]).float().clone())
        return torch.stack(out)

    model = ModelBase.create(path, comm.device, max_context=256, max_seqs=2, tp_rank=rank, tp_size=world, comm=comm)
    fused = run(model)
    tpx = model.tp_exchange()
    status, exchanges = tpx.status(), tpx.exchanges
    model.reset_kv_cache()
    first = int(model.forward(prompt).argmax())
    dg = DecodeGraph(model, [model._seq()], 8)
    dg.set_tokens([first])
    dg.capture()
    graph_tokens = [first] + [int(dg.step()[0]) for _ in range(4)]
    eager_tokens = [int(x.argmax()) for x in fused[:5]]
    status |= tpx.status()
    model._tpx = False
    os.environ["TSB_TP_FUSED"] = "0"
    nccl = run(model)
    res = {"world": world, "arch": model.arch, "status": status, "exchanges": exchanges,
           "fused_vs_nccl": float((fused - nccl).abs().max()), "graph_tokens": graph_tokens, "eager_tokens": eager_tokens}
    if rank == 0:
        single = ModelBase.create(path, comm.device, max_context=256)
        ref = run(single)
        res["fused_vs_single"] = float((fused - ref).abs().max())
        res["scale"] = float(ref.abs().max())
        print("TPCHECK " + json.dumps(res), flush=True)
    comm.barrier()


def check_model(path, comm):
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.engine import DecodeGraph
    rank, world = comm.rank, comm.size
    os.environ["TSB_TP_FUSED"] = "1"
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 4096, (9,), generator=g).tolist()

    def run(model, steps=6):
        model.reset_kv_cache()
        out = [model.forward(prompt).float().clone()]          # 9 tokens: the small-batch (exchange) path
        for _ in range(steps):
            out.append(model.forward([int(out[-1].argmax())]).float().clone())
        return torch.stack(out)

    model = ModelBase.create(path, comm.device, max_context=512, max_seqs=2, tp_rank=rank, tp_size=world, comm=comm)
    fused = run(model)
    tpx = model.tp_exchange()
    status = tpx.status()
    exchanges = tpx.exchanges
    # the same steps captured as a CUDA graph: the exchange keeps its epoch in device memory
    model.reset_kv_cache()
    first = int(model.forward(prompt).argmax())
    dg = DecodeGraph(model, [model._seq()], 8)
    dg.set_tokens([first])
    dg.capture()
    graph_tokens = [first]
    for _ in range(5):
        graph_tokens.append(int(dg.step()[0]))
    eager_tokens = [int(x.argmax()) for x in fused[:6]]
    status |= tpx.status()
    # long prompt: the sequence-parallel prefill (GEMM -> reduce-scatter, all-gather -> GEMM)
    long_prompt = torch.randint(0, 4096, (300,), generator=g).tolist()
    model.reset_kv_cache()
    seq_logits = model.forward(long_prompt).float().clone()
    seq_next = model.forward([int(seq_logits.argmax())]).float().clone()     # decode on the cache the prefill wrote
    sp = getattr(model, "_tpseq", None)
    seq_status = sp.status() if sp is not None else -1
    # expert dispatch by destination against the all-gather form of the same exchange (mixture-of-experts models only)
    routed_diff = None
    if model.arch == "gpt-oss" or hasattr(model, "n_experts"):
        os.environ["TSB_EP_ROUTED"] = "0"
        model.reset_kv_cache()
        routed_diff = float((model.forward(long_prompt).float() - seq_logits).abs().max())
        os.environ["TSB_EP_ROUTED"] = "1"
        seq_status |= sp.status() if sp is not None else -1
    model._tpx = False                                          # NCCL all-reduce path on the same weights
    os.environ["TSB_TP_FUSED"] = "0"
    nccl = run(model)
    model.reset_kv_cache()
    nccl_long = model.forward(long_prompt).float().clone()
    # the same token as the fused run took (random-init logits are nearly flat: each path's own arg-max can differ)
    nccl_next = model.forward([int(seq_logits.argmax())]).float().clone()
    res = {"world": world, "arch": model.arch, "status": status, "exchanges": exchanges,
           "fused_vs_nccl": float((fused - nccl).abs().max()), "graph_tokens": graph_tokens, "eager_tokens": eager_tokens,
           "seq_status": seq_status, "seq_vs_nccl": float((seq_logits - nccl_long).abs().max()),
           "seq_next_vs_nccl": float((seq_next - nccl_next).abs().max()), "routed_vs_allgather": routed_diff}
    if rank == 0:
        single = ModelBase.create(path, comm.device, max_context=512)
        ref = run(single)
        res["fused_vs_single"] = float((fused - ref).abs().max())
        single.reset_kv_cache()
        res["seq_vs_single"] = float((seq_logits - single.forward(long_prompt).float()).abs().max())
        res["scale"] = float(ref.abs().max())
        print("TPCHECK " + json.dumps(res), flush=True)
    comm.barrier()


if __name__ == "__main__":
    main()
