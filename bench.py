#!/usr/bin/env python
"""Headline benchmark: decode (and prefill) tokens/s of a Qwen3-4B-shaped Q4_K_M model.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N ...            # the reference's own GGML-CUDA library
    python bench.py --model gptoss-20b | qwen35-35b-a3b | gemma4-31b   # the other named configurations
    python bench.py --model qwen3-tiny --device cpu          # the tiny configuration on the CPU backend

A *step* is one greedy decode step of the whole batch (batch 1 by default, as the
reference benchmark is; ``--batch 16`` gives the batched config).  The model is random-init
N(0, 0.02) weights written to GGUF as Q4_K_M and loaded back through the normal loader;
the prompt is 2048 synthetic token ids.  K steps are timed with CUDA events between two
barriers + synchronisations, max over ranks; rank 0 prints one JSON line.  The weights
(2.4 GB) are far larger than the 126 MB L2, so every step streams them from HBM and no
explicit L2 flush is needed.  The end-to-end number repeats the measurement through the
public API with a pinned-host → device copy of the step's input ids and a device → host
read of the sampled ids in every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from baseline import METRIC  # noqa: E402  (the metric string both arms print)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="sequences decoded together (default: 1; gptoss-20b: 64)")
    ap.add_argument("--prefill", type=int, default=None, help="prompt tokens per sequence (default: 2048; gptoss-20b: 1024)")
    ap.add_argument("--model", default="qwen3-4b", choices=["qwen3-4b", "qwen3-tiny", "gptoss-20b", "gptoss-tiny", "qwen35-35b-a3b",
                                                           "gemma4-31b", "gemma-tiny"])
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: the tiny Qwen3 config on the CPU backend (prompt 64, 32 greedy tokens, wall clock)")
    ap.add_argument("--reuse-prefix", type=int, default=None,
                    help="gemma configs: tokens of the first turn's cache that the second turn keeps (default 30000 of 32768 + 512)")
    ap.add_argument("--prefill-repeats", type=int, default=3, help="timed prefill repetitions (median reported)")
    ap.add_argument("--also-batch", type=int, default=None,
                    help="qwen3-4b at batch 1: measure this batch size as well and report it under \"batch16\"-style extra keys "
                         "(default 16, the other half of the configuration; 0 = skip)")
    ap.add_argument("--no-graph", action="store_true", help="run decode steps eagerly (for kernel-level profiling)")
    ap.add_argument("--trace-prefill", default=None, metavar="FILE",
                    help="one GPU: write the kernel timeline of one prefill to FILE and print the per-kernel table to stderr")
    ap.add_argument("--trace", default=None, metavar="FILE",
                    help="after the timed runs, record three more graph replays with the CUDA activity tracer, write the "
                         "kernel events of the middle one to FILE (JSON) and print its per-kernel table to stderr")
    ap.add_argument("--cache-dir", default=os.environ.get("TSB_BENCH_CACHE", os.path.join(tempfile.gettempdir(), "tsb_bench")))
    a = ap.parse_args()
    if a.batch is None:
        a.batch = {"gptoss-20b": 64, "qwen35-35b-a3b": 8}.get(a.model, 1)
    if a.prefill is None:
        a.prefill = {"gptoss-20b": 1024, "qwen35-35b-a3b": 8192, "gemma4-31b": 32768, "gemma-tiny": 96}.get(a.model, 2048)
    if a.also_batch is None:
        a.also_batch = 16 if (a.model == "qwen3-4b" and a.batch == 1 and a.device == "cuda") else 0
    if a.reuse_prefix is None:
        a.reuse_prefix = {"gemma4-31b": 30000, "gemma-tiny": 80}.get(a.model)
    return a


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


MODEL_SHAPES = {
    "qwen3-4b": dict(n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, ffn=9728, vocab=151936,
                     scheme="Q4_K_M", rope_base=1e6, tied=True),
    "qwen3-tiny": dict(n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=768, vocab=4096,
                       scheme="Q8_0", rope_base=1e6, tied=True),
    "gptoss-20b": dict(n_layers=24, hidden=2880, n_heads=64, n_kv_heads=8, head_dim=64, n_experts=32, top_k=4,
                       expert_ffn=2880, vocab=201088, window=128),
    "gptoss-tiny": dict(n_layers=2, hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, n_experts=8, top_k=2,
                        expert_ffn=256, vocab=4096, window=16),
    "qwen35-35b-a3b": dict(n_layers=40, hidden=2048, n_heads=16, n_kv_heads=2, head_dim=256, rope_dims=64, interval=4,
                           hk=16, hv=32, dk=128, dv=128, conv_k=4, n_experts=256, top_k=8, expert_ffn=512, shared_ffn=512,
                           ffn=6144, vocab=151936, scheme="Q4_K_M"),
    "gemma4-31b": dict(arch="gemma3", n_layers=60, hidden=5376, n_heads=32, n_kv_heads=16, head_dim=128, ffn=21504, vocab=262144,
                       window=1024, scheme="Q8_0", softcap=30.0),
    "gemma-tiny": dict(arch="gemma3", n_layers=6, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=4096,
                       window=16, scheme="Q8_0", softcap=30.0),
}
MODEL_TEXT = {
    "qwen3-4b": ("Qwen3-4B-shaped Q4_K_M (36L, hidden 2560, 32q/8kv x128, ffn 9728, vocab 151936), random-init",
                 "bf16 activations / f32 accumulate, Q4_K_M weights as stored",
                 "weights (2.4 GB) exceed the 126 MB L2; no flush needed"),
    "qwen3-tiny": ("tiny Qwen3 Q8_0 (4L, hidden 256), random-init", "bf16 activations / f32 accumulate, Q8_0 weights as stored",
                   "tiny model: fits L2, smoke configuration only"),
    "gptoss-20b": ("gpt-oss-20b-shaped (24L, hidden 2880, 64q/8kv x64, 32 experts top-4, expert ffn 2880, vocab 201088, "
                   "window 128), MXFP4 experts + bf16 attention, random-init",
                   "bf16 activations / f32 accumulate, MXFP4 expert weights as stored",
                   "weights (12.5 GB) exceed the 126 MB L2; no flush needed"),
    "qwen35-35b-a3b": ("Qwen3.5-35B-A3B-shaped Q4_K_M (40L, hidden 2048, GatedDeltaNet 16 QK / 32 V heads x128 on 3 of 4 layers, "
                       "attention 16q/2kv x256, 256 experts top-8 + shared, expert ffn 512, vocab 151936), random-init",
                       "bf16 activations / f32 accumulate, Q4_K_M weights as stored",
                       "weights (about 20 GB) exceed the 126 MB L2; no flush needed"),
    "gemma4-31b": ("Gemma-4-31B-class dense Q8_0 (60L, hidden 5376, 32q/16kv x128, GeGLU 21504, 5 sliding(1024) : 1 global, "
                   "logit softcap, vocab 262144), random-init",
                   "bf16 activations / f32 accumulate, Q8_0 weights as stored", "weights (about 28 GB) exceed the 126 MB L2; no flush needed"),
    "gemma-tiny": ("tiny Gemma 3 Q8_0 (6L, hidden 256, window 16), random-init", "bf16 activations / f32 accumulate, Q8_0 weights as stored",
                   "tiny model: smoke configuration only"),
    "gptoss-tiny": ("tiny gpt-oss (2L, hidden 256, 8 experts top-2), random-init",
                    "bf16 activations / f32 accumulate, MXFP4 expert weights as stored", "tiny model: smoke configuration only"),
}


def ensure_model(args, rank: int, world: int) -> str:
    """Write the synthetic GGUF once per box (rank 0) and let the other ranks wait for it."""
    import torch
    os.makedirs(args.cache_dir, exist_ok=True)
    path = os.path.join(args.cache_dir, f"{args.model}.gguf")
    done = path + ".done"
    if rank == 0 and not os.path.exists(done):
        from tensorsharp_b200.models import synth
        writer = (synth.write_gptoss if args.model.startswith("gptoss") else
                  synth.write_qwen35 if args.model.startswith("qwen35") else
                  synth.write_gemma if args.model.startswith("gemma") else synth.write_qwen3)
        writer(path, **MODEL_SHAPES[args.model], seed=0, device="cuda" if torch.cuda.is_available() else "cpu")
        open(done, "w").write("ok")
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    return path


def trace_step(dg, path: str, run=None, what: str = "decode step") -> None:
    """Kernel timeline of one decode step inside the captured graph (or of one call of ``run``: a prefill).  Kernels
    overlap under programmatic dependent launch (a kernel is resident and waiting before its predecessor ends), so
    besides each kernel's own duration the table gives its *exclusive* time: the part of it after every earlier
    kernel had finished, which is what it adds to the step."""
    import collections
    import re

    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            run() if run is not None else dg.step()
        torch.cuda.synchronize()
    ev = sorted(((e.name, e.time_range.start, e.time_range.end) for e in prof.events()
                 if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda x: x[1])
    n = len(ev) // 3
    step = ev[n:2 * n]
    with open(path, "w") as f:
        json.dump(step, f)
    t0, prev = step[0][1], step[0][1]
    rows = collections.OrderedDict()
    for name, s, e in step:
        k = re.sub(r"\(.*", "", name)[:48]
        r = rows.setdefault(k, [0, 0.0, 0.0])
        r[0] += 1
        r[1] += e - s
        r[2] += max(0.0, e - max(prev, s))
        prev = max(prev, e)
    print(f"{what}: {n} kernels, {prev - t0:.1f} us", file=sys.stderr)
    print(f"{'kernel':50s}{'n':>4s}{'sum us':>9s}{'excl us':>9s}{'excl/n':>8s}", file=sys.stderr)
    for k, (c, du, ex) in sorted(rows.items(), key=lambda kv: -kv[1][2]):
        print(f"{k:50s}{c:4d}{du:9.1f}{ex:9.1f}{ex / c:8.2f}", file=sys.stderr)


def run_ours(args) -> dict:
    import torch
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.ops import functional as F
    from tensorsharp_b200.ops import kernels
    from tensorsharp_b200.runtime.engine import DecodeGraph

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from tensorsharp_b200.parallel.dist import Communicator
        comm = Communicator(rank, world, dev)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    path = ensure_model(args, rank, world)
    B, P, K, W = args.batch, args.prefill, args.steps, args.warmup
    ctx = P + 2 * (K + W) + 64
    model = ModelBase.create(path, dev, max_context=ctx, max_seqs=max(B, args.also_batch) + 1, tp_rank=rank, tp_size=world, comm=comm)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, model.cfg.vocab, (P,), generator=g).tolist() for _ in range(B)]

    # ---- prefill (time to first token) ------------------------------------------------------
    def prefill_once(B=B, prompts=prompts):
        seqs = [model.kv.new_seq() for _ in range(B)]
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        first = None
        per = 4 if P >= 2048 else max(4, 16384 // P)     # 8 k to 16 k tokens per forward keeps activations modest
        rc = model.kv.ring_chunk or P                  # window layers on a ring of pages: the prompt goes in by chunks
        for i in range(0, B, per):
            chunk = seqs[i:i + per]
            for j in range(0, P, rc):
                last = j + rc >= P
                logits = model.forward_batch(model.kv.build_batch(chunk, [p[j:j + rc] for p in prompts[i:i + per]]), want_logits=last)
            t = F.argmax(logits)
            first = t if first is None else torch.cat([first, t])
        e1.record()
        barrier()
        return seqs, first, e0.elapsed_time(e1)

    seqs, first, _ = prefill_once()              # warm-up (allocations, attribute set-up)
    for s in seqs:
        model.kv.free_seq(s)
    ttfts = []
    for _ in range(args.prefill_repeats):
        seqs, first, ms = prefill_once()
        ttfts.append(ms)
        if _ < args.prefill_repeats - 1:
            for s in seqs:
                model.kv.free_seq(s)
    ttfts.sort()
    prefill_ms = ttfts[len(ttfts) // 2]

    # ---- decode: K timed steps of the whole batch -------------------------------------------
    dg = DecodeGraph(model, seqs, 2 * (K + W) + 8, use_graph=not args.no_graph)
    dg.set_tokens(first.tolist())
    dg.capture()
    n0 = kernels.LAUNCHES
    for _ in range(W):
        dg.step()
    launches_eager = (kernels.LAUNCHES - n0) // max(1, W)
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prof_range = os.environ.get("TSB_BENCH_PROFILE_RANGE") == "1"     # lets a profiler started with its capture off see only the timed steps
    if prof_range:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(K):
        dg.step()
    e1.record()
    barrier()
    if prof_range:
        torch.cuda.profiler.stop()
    dev_ms = e0.elapsed_time(e1)

    # ---- end to end: ids in from pinned host memory, sampled ids back to the host, every step
    toks = dg.sampled.tolist()
    for _ in range(W):
        toks = dg.step_host(toks)
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for _ in range(K):
        toks = dg.step_host(toks)
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 0.0)
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    clock_info = clocks.stop() if rank == 0 else {}

    if args.trace and rank == 0:
        trace_step(dg, args.trace)
    if args.trace_prefill and rank == 0 and world == 1:
        def one_prefill():
            ss, _, _ = prefill_once()
            for s_ in ss:
                model.kv.free_seq(s_)
        trace_step(None, args.trace_prefill, run=one_prefill, what="prefill")

    # ---- second turn (long-context configs): keep a prefix of the first turn's cache, prefill what follows it
    turn2_ms, turn2_new = 0.0, 0
    if args.reuse_prefix and B == 1:
        seq = seqs[0]
        total = seq.length
        keep = min(args.reuse_prefix, total - 1)
        tail = (prompts[0] + [int(t) % model.cfg.vocab for t in range(total)])[keep:total]      # same length as the turn it replaces
        turn2_new = len(tail)
        dg.graph = None                                # the captured steps hold this sequence's pages
        model.kv.truncate(seq, keep)
        barrier()
        e0.record()
        rc = model.kv.ring_chunk or len(tail)
        for j in range(0, len(tail), rc):
            lg = model.forward_batch(model.kv.build_batch([seq], [tail[j:j + rc]]), want_logits=j + rc >= len(tail))
        F.argmax(lg)
        e1.record()
        barrier()
        turn2_ms = e0.elapsed_time(e1)

    # ---- the batched half of the configuration (qwen3-4b: 16 sequences x the same prompt length), same timing rules
    extra_ms = [0.0, 0.0]
    Bx = args.also_batch if not turn2_new else 0
    if Bx:
        dg.graph = None
        for s_ in seqs:
            model.kv.free_seq(s_)
        prompts_x = [torch.randint(0, model.cfg.vocab, (P,), generator=g).tolist() for _ in range(Bx)]
        seqs_x, first_x, _ = prefill_once(Bx, prompts_x)
        for s_ in seqs_x:
            model.kv.free_seq(s_)
        seqs_x, first_x, extra_ms[1] = prefill_once(Bx, prompts_x)
        dgx = DecodeGraph(model, seqs_x, K + W + 8, use_graph=not args.no_graph)
        dgx.set_tokens(first_x.tolist())
        dgx.capture()
        for _ in range(W):
            dgx.step()
        barrier()
        e0.record()
        for _ in range(K):
            dgx.step()
        e1.record()
        barrier()
        extra_ms[0] = e0.elapsed_time(e1)
        dgx.graph = None

    vals = torch.tensor([dev_ms, e2e_ms, prefill_ms, e2e_wall_ms, turn2_ms] + extra_ms, dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, prefill_ms, e2e_wall_ms, turn2_ms, bx_dec_ms, bx_pre_ms = vals.tolist()
    status = int(kernels.gemm_status(dev).item())
    res = {
        "metric": METRIC if B == 1 else f"decode tok/s (batch {B}, greedy); prefill tok/s and p50 TTFT alongside",
        "timing": "CUDA events on the launching stream between barriers, max over ranks",
        "value": B * K / (dev_ms / 1e3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": MODEL_TEXT[args.model][1], "data": "synthetic",
        "impl": "ours",
        "config": {"model": MODEL_TEXT[args.model][0], "global_batch": B, "seq_len": P, "decode_steps": K,
                   "parallelism": (f"tp{world}" if args.model.startswith(("qwen3-", "gemma")) else f"tp{world} attention + ep{world} experts"),
                   "l2": MODEL_TEXT[args.model][2],
                   "prefill_weights": "GEMMs of the prefill read a bf16 copy of each quantised matrix, decoded once at first use "
                                      "and kept in spare HBM (TSB_BF16_WEIGHT_CACHE_GB); decode streams the GGUF blocks"},
        "prefill_tok_s": B * P / (prefill_ms / 1e3), "ttft_ms_p50": prefill_ms,
        "e2e": {"value": B * K / (max(e2e_ms, e2e_wall_ms) / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B, "ms_per_step_device": e2e_ms / K, "ms_per_step_wall": e2e_wall_ms / K},
        "gpu_launches": (dg.launches_per_step or launches_eager) * K,
        "kv_cache": {"gb": round(sum(t.numel() * t.element_size() for t in {id(t): t for t in list(model.kv.k) + list(model.kv.v) if t is not None}.values()) / 1e9, 3),
                     "window_ring_pages": model.kv.ring_pages or None},
        "second_turn": ({"kv_reused_tokens": int(args.reuse_prefix), "new_tokens": turn2_new, "ttft_ms": turn2_ms}
                        if turn2_new else None),
        "kernel_status": status,
        "clocks": clock_info,
    }
    if Bx:
        res[f"batch{Bx}"] = {"decode_tok_s": Bx * K / (bx_dec_ms / 1e3), "ms_per_step": bx_dec_ms / K,
                              "prefill_tok_s": Bx * P / (bx_pre_ms / 1e3), "ttft_ms": bx_pre_ms, "global_batch": Bx, "seq_len": P}
    if world > 1:
        # Tearing an NCCL communicator down while CUDA graphs that captured its kernels are still
        # alive blocks for ever in destroy_process_group(); print first, drop the graphs, then
        # leave without the collective teardown (process exit releases everything).
        import gc

        import torch.distributed as dist
        if rank == 0:
            print(json.dumps(res), flush=True)
        dg.graph = None
        del dg
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)
    return res if rank == 0 else None


def run_cpu(args) -> dict:
    """The tiny Qwen3 configuration on the CPU backend (the fp32 oracle of every op): batch 1, a 64-token prompt,
    32 greedy decode tokens, wall clock.  No GPU is touched."""
    import torch
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    if args.model != "qwen3-tiny":
        raise SystemExit("--device cpu runs the qwen3-tiny configuration only")
    os.makedirs(args.cache_dir, exist_ok=True)
    path = os.path.join(args.cache_dir, "qwen3-tiny-cpu.gguf")
    if not os.path.exists(path + ".done"):
        synth.write_qwen3(path, **MODEL_SHAPES["qwen3-tiny"], seed=0, device="cpu")
        open(path + ".done", "w").write("ok")
    P, K, W = 64, 32, max(3, args.warmup)
    model = ModelBase.create(path, "cpu", max_context=P + K + W + 8)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, model.cfg.vocab, (P,), generator=g).tolist()

    def one_run():
        model.reset_kv_cache()
        t0 = time.perf_counter()
        logits = model.forward(prompt)
        t1 = time.perf_counter()
        ids = []
        for _ in range(K):
            ids.append(int(logits.argmax()))
            logits = model.forward([ids[-1]])
        return (t1 - t0) * 1e3, (time.perf_counter() - t1) * 1e3, ids
    for _ in range(W):
        one_run()
    runs = sorted(one_run()[:2] for _ in range(3))
    prefill_ms, decode_ms = runs[1]
    return {"metric": "decode tok/s (CPU backend, wall clock); prefill tok/s alongside", "value": K / (decode_ms / 1e3), "unit": "tok/s",
            "n_gpus": 0, "steps": K, "warmup": W, "ms_per_step": decode_ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp32 oracle, Q8_0 weights as stored", "data": "synthetic", "impl": "ours", "device": "cpu",
            "config": {"model": MODEL_TEXT["qwen3-tiny"][0], "global_batch": 1, "seq_len": P, "decode_steps": K, "parallelism": "none"},
            "prefill_tok_s": P / (prefill_ms / 1e3), "ttft_ms_p50": prefill_ms, "gpu_launches": 0}


def run_reference(args) -> dict:
    try:
        from baseline.ref_harness import run as ref_run
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference harness not importable: {exc}"}
    if int(os.environ.get("RANK", "0")) != 0 and not args.model.startswith("qwen3-"):
        return None
    if args.model.startswith("qwen35"):
        return {"impl": "reference", "unavailable": "no export covers the Qwen3.5 step: TSGgml_GatedDeltaNetChunkedF32 is the prefill scan only; the "
                                                    "single-token GatedDeltaNet step, its conv state and the MoE routing run in the C# graph "
                                                    "(Qwen35Model.GatedDeltaNet.cs:1449-1500, Qwen35Model.cs:1931-2402), for which this box has no runtime"}
    if args.model.startswith("gemma"):
        return {"impl": "reference", "unavailable": "this configuration is written as the gemma3 architecture, which the reference runs op by op from "
                                                    "its C# graph (Gemma3Model.cs); its whole-model exports TSGgml_Gemma4ModelDecode / "
                                                    "TSGgml_Gemma4LayerPrefill take the gemma4 tensor set (per-layer embeddings, shared-KV map) that "
                                                    "this file does not have; the per-op restatement is not written"}
    if args.model.startswith("gptoss"):
        return {"impl": "reference", "unavailable": "the GPT-OSS step needs the sink-aware attention and the biased router of GptOssModel.cs:591-865, "
                                                    "which exist only in the C# graph: TSGgml_FlashAttnDecodeF32 takes no sinks and "
                                                    "TSGgml_MoEExpertsSwiGLUResidualF32 has neither expert biases nor the clamped SwiGLU"}
    return ref_run(args, MODEL_SHAPES[args.model])


def main():
    args = parse_args()
    dump = os.environ.get("TSB_BENCH_STACK_DUMP_AFTER")
    if dump:          # diagnostics: print every thread's Python stack if the run is still going after N seconds
        import faulthandler
        faulthandler.dump_traceback_later(float(dump), repeat=False, exit=True)
    if args.device == "cpu" and args.impl == "reference":
        res = {"impl": "reference", "unavailable": "the reference's CPU backend is its C# code; no .NET SDK exists on this box"}
    elif args.device == "cpu":
        res = run_cpu(args)
    else:
        res = run_reference(args) if args.impl == "reference" else run_ours(args)
    if res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
