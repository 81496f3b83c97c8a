#!/usr/bin/env python
"""Kernel micro-benchmarks: one hot kernel in isolation, device-timed, on weights that do not fit L2.

    python bench_kernels.py gemv --type Q4_K --n 19456 --k 2560 --glu --m 1
    python bench_kernels.py gemv --type Q4_K --n 2560 --k 9728
    python bench_kernels.py gemm --t 2048 --n 19456 --k 2560         # bf16 tensor-core GEMM; TSB_GEMM_WIDE=0 / 2 picks the tile
    python bench_kernels.py attn --t 2048 --hq 32 --hkv 8 --dh 128   # causal flash prefill over the paged cache
    python bench_kernels.py attn_decode --b 16 --t 2048 [--kv fp8]   # split-KV decode attention, bf16 or e4m3 pages
    python bench_kernels.py recurrent --op gdn --t 2048
    python bench_kernels.py recurrent --op mamba2 --t 2048

Each call cycles through enough copies of the weight matrix to exceed the 126 MB L2, so every launch
streams from HBM; the figure printed is the mean over ``--iters`` launches between two CUDA events,
after ``--warmup`` launches, with the achieved bandwidth as a fraction of the measured copy
bandwidth in MEASURED_PEAKS.json when that file is present.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def time_us(fn, iters: int, warmup: int) -> float:
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def recurrent(args):
    """The token-by-token scan kernel against the chunked form (tensor ops) on one prompt of ``--t`` tokens, at the
    Qwen3.5-35B-A3B GatedDeltaNet shape (16 QK / 32 V heads x 128) or the Nemotron-H Mamba2 shape (64 heads x 64,
    8 groups, state 128).  Prints both times and the distance between the two outputs, then the chunked form with its
    chunk-after-chunk part as one kernel and with the chunk-parallel part as a kernel too (csrc/gdn_chunk.cu)."""
    import torch
    from tensorsharp_b200.ops import kernels
    from tensorsharp_b200.ops import reference as ref
    dev, T = "cuda", args.t
    torch.manual_seed(0)
    cu_q = torch.tensor([0, T], dtype=torch.int32, device=dev)
    slots = torch.zeros(1, dtype=torch.int32, device=dev)
    if args.op == "gdn":
        Hk, Hv, Dk, Dv = 16, 32, 128, 128
        qkv = torch.randn(T, 2 * Hk * Dk + Hv * Dv, device=dev)
        z = torch.randn(T, Hv * Dv, device=dev)
        beta, alpha = torch.randn(T, Hv, device=dev), torch.randn(T, Hv, device=dev)
        dt_bias, a_log = torch.randn(Hv, device=dev) * 0.1, -torch.rand(Hv, device=dev)
        norm_w = torch.ones(Dv, device=dev)
        kw = dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=1e-6)
        s0 = torch.zeros(1, Hv, Dv, Dk, device=dev)
        s1 = torch.zeros(Hv, Dv, Dk, device=dev)

        def scan():
            s0.zero_()
            return kernels.gdn_recurrent(qkv, z, beta, alpha, dt_bias, a_log, norm_w, s0, cu_q, slots, **kw)

        def chunked():
            s1.zero_()
            return ref.gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, s1, chunk=args.chunk, **kw)
    else:
        H, P, G, N = 64, 64, 8, 128
        xbc = torch.randn(T, H * P + 2 * G * N, device=dev)
        dt = torch.randn(T, H, device=dev)
        dt_bias, A, D = torch.randn(H, device=dev) * 0.1, -torch.rand(H, device=dev), torch.randn(H, device=dev)
        kw = dict(H=H, P=P, G=G, N=N)
        s0 = torch.zeros(1, H, P, N, device=dev)
        s1 = torch.zeros(H, P, N, device=dev)

        def scan():
            s0.zero_()
            return kernels.mamba2_recurrent(xbc, dt, dt_bias, A, D, s0, cu_q, slots, **kw)

        def chunked():
            s1.zero_()
            return ref.mamba2_chunked(xbc, dt, dt_bias, A, D, s1, chunk=args.chunk, **kw)
    fused = None
    if args.op == "mamba2":
        s2 = torch.zeros_like(s1)

        def fused():
            s2.zero_()
            return ref.mamba2_chunked(xbc, dt, dt_bias, A, D, s2, chunk=64, carry=kernels.gdn_chunk_carry, **kw)
    if args.op == "gdn":
        s2 = torch.zeros_like(s1)

        def fused():
            s2.zero_()
            return ref.gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, s2, chunk=64, carry=kernels.gdn_chunk_carry, **kw)
    kern3 = None
    if args.op == "gdn":
        s3 = torch.zeros(1, Hv, Dv, Dk, device=dev)

        def kern3():
            s3.zero_()
            return kernels.gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, s3, cu_q, [0, T], [0], **kw)
    if args.op == "mamba2":
        s3 = torch.zeros(1, H, P, N, device=dev)

        def kern3():
            s3.zero_()
            return kernels.mamba2_chunked(xbc, dt, dt_bias, A, D, s3, cu_q, [0, T], [0], **kw)
    a, b = scan().float(), chunked().float()
    rel = float((a - b).norm() / b.norm())
    srel = float((s0[0] - s1).norm() / s1.norm())
    print(json.dumps({"kernel": "recurrent", "op": args.op, "T": T, "chunk": args.chunk,
                      "scan_us": time_us(scan, args.iters, args.warmup),
                      "chunked_us": time_us(chunked, args.iters, args.warmup),
                      "chunked_carry_kernel_us": time_us(fused, args.iters, args.warmup) if fused else None,
                      "rel_diff_out_carry_kernel": float((fused().float() - b).norm() / b.norm()) if fused else None,
                      "chunk_kernels_us": time_us(kern3, args.iters, args.warmup) if kern3 else None,
                      "rel_diff_out_chunk_kernels": float((kern3().float() - b).norm() / b.norm()) if kern3 else None,
                      "rel_diff_out": rel, "rel_diff_state": srel}))


def gemm(args):
    """The bf16 tcgen05 GEMM on [t, k] x [n, k]^T against torch.matmul (cuBLAS), cycling through weight copies larger
    than L2.  TSB_GEMM_WIDE=0 keeps 128 x 256 tiles, 2 forces 256 x 256 (default: by tile count)."""
    import torch
    from tensorsharp_b200.ops import kernels
    dev = "cuda"
    torch.manual_seed(0)
    copies = max(2, int(300e6 // (args.n * args.k * 2)) + 1)
    ws = [(torch.randn(args.n, args.k, device=dev) * 0.05).bfloat16() for _ in range(copies)]
    x = torch.randn(args.t, args.k, device=dev).bfloat16()
    state = {"i": 0}

    odt = torch.float32 if args.f32 else torch.bfloat16
    res = torch.randn(args.t, args.n, device=dev).to(odt) if args.residual else None
    outb = torch.empty(args.t, args.n, device=dev, dtype=odt)

    def ours():
        state["i"] += 1
        return kernels.gemm_bf16(ws[state["i"] % copies], x, out_dtype=odt, residual=res, out=outb)

    def lib():
        state["i"] += 1
        return x @ ws[state["i"] % copies].t()
    want = (x @ ws[0].t()).float()
    err = float((kernels.gemm_bf16(ws[0], x, out_dtype=torch.bfloat16).float() - want).norm() / want.norm())
    flop = 2.0 * args.t * args.n * args.k
    us_o, us_l = time_us(ours, args.iters, args.warmup), time_us(lib, args.iters, args.warmup)
    peak = None
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:  # noqa: BLE001
        pass
    print(json.dumps({"kernel": "gemm_bf16", "T": args.t, "N": args.n, "K": args.k, "f32_out": args.f32, "residual": args.residual, "wide": os.environ.get("TSB_GEMM_WIDE", "0"), "persistent": os.environ.get("TSB_GEMM_PERSISTENT", "1"),
                      "us": us_o, "tflops": flop / us_o / 1e6, "cublas_us": us_l, "cublas_tflops": flop / us_l / 1e6,
                      "of_measured_cublas_peak": (flop / us_o / 1e6 / peak) if peak else None, "rel_diff": err,
                      "status": int(kernels.gemm_status(torch.device(dev)).item())}))


def attn(args):
    """Causal prefill attention of one sequence of ``--t`` tokens against the paged bf16 cache (pages of 64 in shuffled
    order), ``--hq`` query / ``--hkv`` KV heads of ``--dh``; FLOPs counted as 4 * T^2 / 2 * Dh * Hq."""
    import torch
    from tensorsharp_b200.ops import kernels
    dev, T, Hq, Hkv, Dh, ps = "cuda", args.t, args.hq, args.hkv, args.dh, 64
    torch.manual_seed(0)
    n_pages = (T + ps - 1) // ps
    kc = torch.randn(n_pages * ps, Hkv, Dh, device=dev).bfloat16()
    vc = torch.randn(n_pages * ps, Hkv, Dh, device=dev).bfloat16()
    table = torch.randperm(n_pages, device=dev).to(torch.int32).view(1, n_pages)
    q = torch.randn(T, Hq, Dh, device=dev).bfloat16()
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    lens = torch.tensor([T], dtype=torch.int32, device=dev)
    out = torch.empty_like(q)

    def run():
        return kernels.attn_prefill(q, kc, vc, table, lens, cu, T, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps,
                                    window=args.window, out=out)
    us = time_us(run, args.iters, args.warmup)
    span = T if not args.window else min(T, args.window)
    flop = 4.0 * T * (span if args.window else T / 2.0) * Dh * Hq
    print(json.dumps({"kernel": "attn_prefill", "T": T, "Hq": Hq, "Hkv": Hkv, "Dh": Dh, "window": args.window, "us": us,
                      "tflops": flop / us / 1e6}))


def attn_decode(args):
    """Decode attention (one query per sequence) of ``--b`` sequences at context ``--t`` against the paged cache, bf16 pages
    or e4m3 bytes (``--kv fp8``), with the split factor the model path would pick; reports the K / V bytes per second."""
    import torch
    from tensorsharp_b200.ops import functional as F
    from tensorsharp_b200.ops import kernels
    dev, T, B, Hq, Hkv, Dh, ps = "cuda", args.t, args.b, args.hq, args.hkv, args.dh, 64
    torch.manual_seed(0)
    pages_per = (T + ps - 1) // ps
    n_pages = pages_per * B
    layers = max(2, int(300e6 // (n_pages * ps * Hkv * Dh * 2 * (1 if args.kv == "fp8" else 2))) + 1)     # cycle: larger than L2
    caches = []
    for _ in range(layers):
        kc = torch.randn(n_pages * ps, Hkv, Dh, device=dev).bfloat16()
        vc = torch.randn(n_pages * ps, Hkv, Dh, device=dev).bfloat16()
        caches.append((kc.to(torch.float8_e4m3fn), vc.to(torch.float8_e4m3fn)) if args.kv == "fp8" else (kc, vc))
    table = torch.randperm(n_pages, device=dev).to(torch.int32).view(B, pages_per)
    q = torch.randn(B, Hq, Dh, device=dev).bfloat16()
    lens = torch.full((B,), T, dtype=torch.int32, device=dev)

    class Shape:                         # what decode_splits reads of a batch
        pass
    sh = Shape()
    sh.B, sh.max_kv_len = B, T
    splits = F.decode_splits(sh, Hkv, 0)
    split_len = F.decode_split_len(sh, splits, 0)
    state = {"i": 0}

    def run():
        kc, vc = caches[state["i"] % layers]
        state["i"] += 1
        return kernels.attn_decode(q, kc, vc, table, lens, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps, splits=splits,
                                   split_len=split_len)
    us = time_us(run, args.iters, args.warmup)
    nbytes = 2.0 * B * T * Hkv * Dh * (1 if args.kv == "fp8" else 2)
    print(json.dumps({"kernel": "attn_decode", "kv": args.kv, "B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "Dh": Dh, "splits": splits,
                      "us": us, "kv_mb": nbytes / 1e6, "gb_s": nbytes / us / 1e3}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "recurrent", "gemm", "attn", "attn_decode"])
    ap.add_argument("--b", type=int, default=16, help="attn_decode: sequences")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8"], help="attn_decode: element type of the cache")
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--dh", type=int, default=128)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--op", default="gdn", choices=["gdn", "mamba2"])
    ap.add_argument("--t", type=int, default=2048)
    ap.add_argument("--chunk", type=int, default=64)
    ap.add_argument("--type", default="Q4_K")
    ap.add_argument("--n", type=int, default=19456)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--glu", action="store_true")
    ap.add_argument("--f32", action="store_true", help="gemm: float32 output")
    ap.add_argument("--residual", action="store_true", help="gemm: add a residual of the output's type in the epilogue")
    ap.add_argument("--iters", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    args = ap.parse_args()
    if args.what == "recurrent":
        return recurrent(args)
    if args.what == "gemm":
        return gemm(args)
    if args.what == "attn":
        return attn(args)
    if args.what == "attn_decode":
        return attn_decode(args)
    import torch
    from tensorsharp_b200.gguf.constants import GGMLType
    from tensorsharp_b200.ops import kernels
    from tensorsharp_b200.quant.qweight import QuantWeight
    dev = "cuda"
    torch.manual_seed(0)
    t = GGMLType[args.type]
    base = QuantWeight.from_float(torch.randn(args.n, args.k, device=dev) * 0.05, t)
    nbytes = sum(p.numel() * p.element_size() for p in base.planes)
    copies = max(2, int(300e6 // nbytes) + 1)
    ws = [base] + [QuantWeight(base.ggml_type, base.N, base.K, [p.clone() for p in base.planes], 1, f"copy{i}")
                   for i in range(copies - 1)]
    x = torch.randn(args.m, args.k, device=dev).bfloat16()
    kw = dict(M=args.m, act="swiglu" if args.glu else None, out_dtype=torch.bfloat16 if args.glu else torch.float32)
    if base.uses_q8_activations:
        xq, xds = kernels.quantize_q8(x)
        kw.update(xq=xq, xds=xds)
    else:
        kw.update(xb=x)
    for i in range(args.warmup):
        kernels.gemv(ws[i % copies], **kw)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.iters):
        kernels.gemv(ws[i % copies], **kw)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.iters
    gbs = nbytes / us / 1e3
    peak = None
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:  # noqa: BLE001
        pass
    print(json.dumps({"kernel": "gemv", "type": args.type, "N": args.n, "K": args.k, "M": args.m, "glu": args.glu,
                      "weight_bytes": nbytes, "copies": copies, "us": us, "GBps": gbs,
                      "of_measured_copy": (gbs / peak) if peak else None}))


if __name__ == "__main__":
    main()
