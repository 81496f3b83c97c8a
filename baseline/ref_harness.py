"""Reference arm of bench.py: the unmodified TensorSharp native bridge (libGgmlOps.so, built
from TensorSharp.GGML.Native + vendored ggml with CUDA for sm_100) driven through its own C
exports in the order the C# model code calls them.

The C# layers cannot run here (no .NET SDK), so this file restates only the *call sequence*
of the reference's fastest stock decode path, Qwen3Model.Forward for one token on a ggml
backend (TensorSharp.Models/Models/Qwen3/Qwen3Model.cs:175-236):

    host embedding row dequant            (ModelBase.cs:826-873)
    TSGgml_TransformerModelDecode         (GgmlBasicOps.cs:719 -> ggml_ops_transformer.cpp:1012)
    TSGgml_NormF32 (output_norm)          (ModelBase.cs:1174 RMSNormOp)
    TSGgml_AddmmQuantF32 (lm_head)        (ModelBase.cs:875 LinearForward)
    logits download + host arg-max        (Program.cs:1515-1607)

None of this repository's kernels, models or engine is on that path; only the GGUF container
reader and writer are shared, to produce and parse the weight file.

The whole-model decode export takes ONE ggml type per matrix class and needs fused QKV, which
the C# code only builds when q, k and v share a type (Qwen3Model.cs:67-78).  A stock Q4_K_M
mixture (Q6_K for some attn_v / ffn_down) therefore cannot take this path in the reference
at all; the harness gives the reference a uniform-Q4_K variant of the same shape (token
embedding Q6_K as in Q4_K_M), which has slightly *fewer* bytes to stream than the Q4_K_M file
this engine is measured on, i.e. the substitution favours the reference.

Timing is the reference's own method, host wall clock around the calls (every call ends with
a backend synchronise and a download), so device time is included.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
try:
    from . import METRIC
except ImportError:                      # run as a script
    import sys
    sys.path.insert(0, ROOT)
    from baseline import METRIC
LIB = os.path.join(ROOT, "baseline", "_ref", "libGgmlOps.so")
BACKEND_CUDA = 3


class View2D(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dim0", C.c_int), ("dim1", C.c_int), ("stride0", C.c_int),
                ("stride1", C.c_int), ("raw_bytes", C.c_int64)]


class View4D(C.Structure):
    _fields_ = [("data", C.c_void_p), ("ne0", C.c_int), ("ne1", C.c_int), ("ne2", C.c_int), ("ne3", C.c_int),
                ("nb1", C.c_int64), ("nb2", C.c_int64), ("nb3", C.c_int64), ("raw_bytes", C.c_int64)]


def _v4(a: np.ndarray) -> View4D:
    """A contiguous 1-D / 2-D float array as the bridge's 4-D view (ne0 innermost)."""
    a2 = a.reshape(1, -1) if a.ndim == 1 else a
    rows, cols = a2.shape
    return View4D(a.ctypes.data, cols, rows, 1, 1, cols * 4, rows * cols * 4, rows * cols * 4, a.nbytes)


def _v2(a: np.ndarray) -> View2D:
    rows, cols = a.shape
    return View2D(a.ctypes.data, rows, cols, cols, 1, a.nbytes)


def _aligned(n_bytes: int, align: int = 16384) -> np.ndarray:
    buf = np.zeros(n_bytes + align, dtype=np.uint8)
    off = (-buf.ctypes.data) % align
    return buf[off:off + n_bytes]


def unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def run(args, shape: dict) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return None          # the reference is single-GPU (ggml_ops_core.cpp:136-149): extra ranks idle
    if not os.path.exists(LIB):
        return unavailable("baseline/_ref/libGgmlOps.so is missing (reference native bridge not built on this box)")
    try:
        lib = C.CDLL(LIB)
    except OSError as exc:
        return unavailable(f"cannot load reference library: {exc}")
    lib.TSGgml_GetLastError.restype = C.c_char_p
    lib.TSGgml_IsBackendAvailable.argtypes = [C.c_int]
    if not lib.TSGgml_IsBackendAvailable(BACKEND_CUDA):
        return unavailable("reference ggml-cuda backend failed to initialise: "
                           + (lib.TSGgml_GetLastError() or b"").decode("utf-8", "replace"))

    import torch
    from tensorsharp_b200.gguf.constants import GGMLType
    from tensorsharp_b200.gguf.reader import GGUFFile
    from tensorsharp_b200.models import synth

    os.makedirs(args.cache_dir, exist_ok=True)
    path = os.path.join(args.cache_dir, f"{args.model}-ref-uniform.gguf")
    if not os.path.exists(path + ".done"):
        s = dict(shape)
        s["scheme"] = "Q4_K_UNIFORM" if shape["scheme"] == "Q4_K_M" else shape["scheme"]
        synth.write_qwen3(path, **s, seed=0, device="cuda" if torch.cuda.is_available() else "cpu")
        open(path + ".done", "w").write("ok")
    g = GGUFFile(path)
    L, D = shape["n_layers"], shape["hidden"]
    Hq, Hkv, Dh, F = shape["n_heads"], shape["n_kv_heads"], shape["head_dim"], shape["ffn"]
    P, K, W = args.prefill, args.steps, args.warmup
    max_seq = P + K + W + 8

    lib.TSGgml_PreloadQuantizedWeight.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64]
    keep = []

    def fused(names):
        infos = [g.tensors[n] for n in names]
        t = infos[0].ggml_type
        if any(i.ggml_type != t for i in infos):
            raise RuntimeError(f"{names}: mixed ggml types; the reference cannot fuse them")
        raw = np.concatenate([np.asarray(g.tensor_bytes_view(n)) for n in names])
        buf = _aligned(raw.nbytes)
        buf[:] = raw
        keep.append(buf)
        ne0 = infos[0].ne[0]
        ne1 = sum(i.ne[1] for i in infos)
        ok = lib.TSGgml_PreloadQuantizedWeight(buf.ctypes.data, buf.ctypes.data, int(t), ne0, ne1, buf.nbytes)
        if not ok:
            raise RuntimeError("PreloadQuantizedWeight: " + lib.TSGgml_GetLastError().decode())
        return buf.ctypes.data, int(t), ne0, ne1, buf.nbytes

    def f32(name):
        ti = g.tensors[name]
        a = _aligned(ti.nbytes).view(np.float32)
        a[:] = np.frombuffer(g.tensor_bytes_view(name), dtype=np.float32)
        keep.append(a)
        return a

    try:
        qkv, o, gu, down, an, fn, qn, kn, kc, vc = ([] for _ in range(10))
        for l in range(L):
            p = f"blk.{l}."
            qkv.append(fused([p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"]))
            o.append(fused([p + "attn_output.weight"]))
            gu.append(fused([p + "ffn_gate.weight", p + "ffn_up.weight"]))
            down.append(fused([p + "ffn_down.weight"]))
            an.append(f32(p + "attn_norm.weight"))
            fn.append(f32(p + "ffn_norm.weight"))
            qn.append(f32(p + "attn_q_norm.weight"))
            kn.append(f32(p + "attn_k_norm.weight"))
            kc.append(_aligned(Hkv * max_seq * Dh * 4).view(np.float32))
            vc.append(_aligned(Hkv * max_seq * Dh * 4).view(np.float32))
        keep.extend(kc + vc)
    except RuntimeError as exc:
        return unavailable(str(exc))

    def parr(items):
        return (C.c_void_p * L)(*[x[0] if isinstance(x, tuple) else x.ctypes.data for x in items])

    arrs = [parr(x) for x in (an, qkv, qn, kn, o, fn, gu, down, kc, vc)]
    out_norm = f32("output_norm.weight")
    emb_info = g.tensors["token_embd.weight"]
    emb_raw = np.asarray(g.tensor_bytes_view("token_embd.weight"))
    emb_buf = _aligned(emb_raw.nbytes)
    emb_buf[:] = emb_raw
    keep.append(emb_buf)
    V = emb_info.ne[1]
    row_bytes = emb_info.nbytes // V

    lib.TSGgml_DequantizeToF32.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
    lib.TSGgml_TransformerModelDecode.argtypes = (
        [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 10
        + [C.c_int, C.c_int64, C.c_int64, C.c_int64] * 4
        + [C.c_int] * 3 + [C.c_int] * 2 + [C.c_float] * 3 + [C.c_int] * 2)
    lib.TSGgml_NormF32.argtypes = [C.c_int, View4D, View4D, View4D, View4D, C.c_int, C.c_float]
    lib.TSGgml_AddmmQuantF32.argtypes = [View2D, View2D, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64]

    hidden = _aligned(D * 4).view(np.float32)
    normed = _aligned(D * 4).view(np.float32).reshape(1, D)
    logits = _aligned(V * 4).view(np.float32).reshape(1, V)
    eps, rope_base = float(g.get_float("qwen3.attention.layer_norm_rms_epsilon", 1e-6)), float(shape["rope_base"])

    def step(token: int, position: int) -> int:
        lib.TSGgml_DequantizeToF32(int(emb_info.ggml_type), emb_buf.ctypes.data + token * row_bytes, D,
                                   hidden.ctypes.data)
        ok = lib.TSGgml_TransformerModelDecode(
            hidden.ctypes.data, D, L, *arrs,
            qkv[0][1], qkv[0][2], qkv[0][3], qkv[0][4], o[0][1], o[0][2], o[0][3], o[0][4],
            gu[0][1], gu[0][2], gu[0][3], gu[0][4], down[0][1], down[0][2], down[0][3], down[0][4],
            Dh, Hq, Hkv, max_seq, position, eps, rope_base, 1.0, F, 2)
        if not ok:
            raise RuntimeError("TransformerModelDecode: " + lib.TSGgml_GetLastError().decode())
        h2 = hidden.reshape(1, D)
        if not lib.TSGgml_NormF32(2, _v4(normed), _v4(h2), _v4(out_norm), _v4(out_norm), 0, eps):
            raise RuntimeError("NormF32: " + lib.TSGgml_GetLastError().decode())
        if not lib.TSGgml_AddmmQuantF32(_v2(logits), _v2(normed), emb_buf.ctypes.data, int(emb_info.ggml_type), D, V,
                                        emb_buf.nbytes):
            raise RuntimeError("AddmmQuantF32: " + lib.TSGgml_GetLastError().decode())
        return int(np.argmax(logits[0]))

    # The KV cache starts as zeros for positions [0, P): the reference's prefill runs through a
    # different (per-op, host round trip) path that is not restated here; decode cost depends on the
    # number of cached positions, not on their values.
    try:
        tok, pos = 100, P
        for _ in range(W):
            tok = step(tok, pos)
            pos += 1
        per_step = []
        t0 = time.perf_counter()
        for _ in range(K):
            t1 = time.perf_counter()
            tok = step(tok, pos)
            pos += 1
            per_step.append((time.perf_counter() - t1) * 1e3)
        dt = time.perf_counter() - t0
    except RuntimeError as exc:
        return unavailable(str(exc))
    ms = dt * 1e3 / K
    return {
        "impl": "reference",
        "metric": METRIC,
        "timing": "host wall clock around the reference's own calls, as its --benchmark does (every call ends with a backend "
                  "synchronise and a download, so device time is included)",
        "value": 1e3 / ms, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 activations, Q4_K weights (uniform; see module docstring), f32 KV cache", "data": "synthetic",
        "config": {"model": "Qwen3-4B-shaped, uniform Q4_K (Q6_K token embedding)", "global_batch": 1, "seq_len": P,
                   "decode_steps": K, "parallelism": "single GPU (the reference has no multi-GPU path)",
                   "path": "TSGgml_TransformerModelDecode + TSGgml_NormF32 + TSGgml_AddmmQuantF32"},
        "prefill_tok_s": None,
        # spread of the timed steps: the path is host-bound (a 36-layer ggml graph is rebuilt, allocated and scheduled
        # on the host for every token), so the mean moves with the box's CPU and with what else runs on it
        "ms_per_step_min": min(per_step), "ms_per_step_median": sorted(per_step)[len(per_step) // 2],
        "e2e": {"value": 1e3 / ms, "unit": "tok/s", "h2d_bytes_per_step": D * 4 + 4, "d2h_bytes_per_step": D * 4 + V * 4},
    }


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--cache-dir", default="/tmp/tsb_bench")
    a = ap.parse_args()
    import sys
    sys.path.insert(0, ROOT)
    from bench import MODEL_SHAPES
    print(json.dumps(run(a, MODEL_SHAPES[a.model])))
