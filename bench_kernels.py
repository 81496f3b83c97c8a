#!/usr/bin/env python
"""Kernel micro-benchmarks: one hot kernel in isolation, device-timed, on weights that do not fit L2.

    python bench_kernels.py gemv --type Q4_K --n 19456 --k 2560 --glu --m 1
    python bench_kernels.py gemv --type Q4_K --n 2560 --k 9728

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv"])
    ap.add_argument("--type", default="Q4_K")
    ap.add_argument("--n", type=int, default=19456)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--glu", action="store_true")
    ap.add_argument("--iters", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    args = ap.parse_args()
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
