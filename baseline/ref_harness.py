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

Prefill goes through the reference's fused per-layer exports, in the order of its prefill block
(Qwen3Model.cs:287-421: norm, QKV, per-head QK norm, RoPE, cache write, causal attention, output
projection, FFN):

    TSGgml_FusedRmsNormMatMulQuantF32     attn_norm + fused QKV   (ggml_ops_fused.cpp:1375)
    TSGgml_NormF32                        per-head RMSNorm of Q, K (ggml_ops_norm_attn.cpp:1568)
    TSGgml_RoPEExF32                      NeoX RoPE of Q, K        (ggml_ops_norm_attn.cpp:1644)
    host copies into the f32 KV cache     (CopyToCache, ModelBase.cs:1340)
    TSGgml_FusedPrefillAttentionF32       causal attention         (ggml_ops_norm_attn.cpp:1699)
    TSGgml_FusedOutProjFFNQuantF32        o_proj + residual + ffn_norm + SwiGLU FFN + residual (ggml_ops_fused.cpp:1538)

The cache the timed decode steps read is the one this prefill wrote.

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


class Contig(C.Structure):
    _fields_ = [("data", C.c_void_p), ("count", C.c_int64), ("etype", C.c_int)]


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


class RefUnavailable(RuntimeError):
    pass


def load_library():
    """The reference's native bridge, or RefUnavailable with the reason."""
    if not os.path.exists(LIB):
        raise RefUnavailable("baseline/_ref/libGgmlOps.so is missing (reference native bridge not built on this box)")
    try:
        lib = C.CDLL(LIB)
    except OSError as exc:
        raise RefUnavailable(f"cannot load reference library: {exc}")
    lib.TSGgml_GetLastError.restype = C.c_char_p
    lib.TSGgml_IsBackendAvailable.argtypes = [C.c_int]
    if not lib.TSGgml_IsBackendAvailable(BACKEND_CUDA):
        raise RefUnavailable("reference ggml-cuda backend failed to initialise: "
                             + (lib.TSGgml_GetLastError() or b"").decode("utf-8", "replace"))
    lib.TSGgml_PreloadQuantizedWeight.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64]
    lib.TSGgml_DequantizeToF32.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
    lib.TSGgml_TransformerModelDecode.argtypes = (
        [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 10
        + [C.c_int, C.c_int64, C.c_int64, C.c_int64] * 4
        + [C.c_int] * 3 + [C.c_int] * 2 + [C.c_float] * 3 + [C.c_int] * 2)
    lib.TSGgml_NormF32.argtypes = [C.c_int, View4D, View4D, View4D, View4D, C.c_int, C.c_float]
    lib.TSGgml_AddmmQuantF32.argtypes = [View2D, View2D, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64]
    lib.TSGgml_FusedRmsNormMatMulQuantF32.argtypes = [View2D, View2D, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_int64,
                                                      C.c_int64, C.c_int64]
    lib.TSGgml_RoPEExF32.argtypes = [View4D, View4D, Contig, C.c_int, C.c_int, C.c_int] + [C.c_float] * 6 + [C.c_int, C.c_int]
    lib.TSGgml_FusedPrefillAttentionF32.argtypes = [C.c_void_p] * 4 + [C.c_int] * 7 + [C.c_float, C.c_int]
    lib.TSGgml_FusedOutProjFFNQuantF32.argtypes = ([View2D, View2D, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int,
                                                    C.c_float] + [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64] * 2 + [C.c_int])
    return lib


class RefQwen3:
    """A Qwen3-architecture GGUF file driven through the reference library: ``prefill(tokens)`` and
    ``decode(token, position)`` return the next-token logits (numpy f32 ``[vocab]``).  The file must let the
    reference fuse Q/K/V and gate/up (one ggml type per fused group)."""

    def __init__(self, lib, path: str, max_seq: int):
        from tensorsharp_b200.gguf.reader import GGUFFile
        self.lib, self.max_seq = lib, int(max_seq)
        g = self.g = GGUFFile(path)
        arch = g.get_str("general.architecture", "qwen3")
        gi = lambda k, d=0: int(g.get_int(f"{arch}.{k}", d))
        self.L, self.D = gi("block_count"), gi("embedding_length")
        self.Hq, self.Hkv = gi("attention.head_count"), gi("attention.head_count_kv")
        self.Dh = gi("attention.key_length", self.D // max(1, self.Hq))
        self.F = gi("feed_forward_length")
        self.eps = float(g.get_float(f"{arch}.attention.layer_norm_rms_epsilon", 1e-6))
        self.rope_base = float(g.get_float(f"{arch}.rope.freq_base", 10000.0))
        self.keep = []
        L, Hkv, Dh = self.L, self.Hkv, self.Dh
        self.qkv, self.o, self.gu, self.down, self.an, self.fn, self.qn, self.kn, self.kc, self.vc = ([] for _ in range(10))
        for l in range(L):
            p = f"blk.{l}."
            self.qkv.append(self._fused([p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"]))
            self.o.append(self._fused([p + "attn_output.weight"]))
            self.gu.append(self._fused([p + "ffn_gate.weight", p + "ffn_up.weight"]))
            self.down.append(self._fused([p + "ffn_down.weight"]))
            self.an.append(self._f32(p + "attn_norm.weight"))
            self.fn.append(self._f32(p + "ffn_norm.weight"))
            self.qn.append(self._f32(p + "attn_q_norm.weight"))
            self.kn.append(self._f32(p + "attn_k_norm.weight"))
            self.kc.append(_aligned(Hkv * self.max_seq * Dh * 4).view(np.float32))
            self.vc.append(_aligned(Hkv * self.max_seq * Dh * 4).view(np.float32))
        parr = lambda items: (C.c_void_p * L)(*[x[0] if isinstance(x, tuple) else x.ctypes.data for x in items])
        self.arrs = [parr(x) for x in (self.an, self.qkv, self.qn, self.kn, self.o, self.fn, self.gu, self.down, self.kc, self.vc)]
        self.out_norm = self._f32("output_norm.weight")
        head = "output.weight" if "output.weight" in g.tensors else "token_embd.weight"
        self.emb_info, self.emb_buf = self._raw("token_embd.weight")
        self.head_info, self.head_buf = (self.emb_info, self.emb_buf) if head == "token_embd.weight" else self._raw(head)
        self.V = self.emb_info.ne[1]
        self.row_bytes = self.emb_info.nbytes // self.V
        self.hidden = _aligned(self.D * 4).view(np.float32)
        self.normed = _aligned(self.D * 4).view(np.float32).reshape(1, self.D)
        self.logits = _aligned(self.V * 4).view(np.float32).reshape(1, self.V)

    # ------------------------------------------------------------------ weights
    def _raw(self, name):
        ti = self.g.tensors[name]
        raw = np.asarray(self.g.tensor_bytes_view(name))
        buf = _aligned(raw.nbytes)
        buf[:] = raw
        self.keep.append(buf)
        return ti, buf

    def _fused(self, names):
        g = self.g
        infos = [g.tensors[n] for n in names]
        t = infos[0].ggml_type
        if any(i.ggml_type != t for i in infos):
            raise RefUnavailable(f"{names}: mixed ggml types; the reference cannot fuse them")
        raw = np.concatenate([np.asarray(g.tensor_bytes_view(n)) for n in names])
        buf = _aligned(raw.nbytes)
        buf[:] = raw
        self.keep.append(buf)
        ne0 = infos[0].ne[0]
        ne1 = sum(i.ne[1] for i in infos)
        if not self.lib.TSGgml_PreloadQuantizedWeight(buf.ctypes.data, buf.ctypes.data, int(t), ne0, ne1, buf.nbytes):
            raise RuntimeError("PreloadQuantizedWeight: " + self.lib.TSGgml_GetLastError().decode())
        return buf.ctypes.data, int(t), ne0, ne1, buf.nbytes

    def _f32(self, name):
        ti = self.g.tensors[name]
        a = _aligned(ti.nbytes).view(np.float32)
        a[:] = np.frombuffer(self.g.tensor_bytes_view(name), dtype=np.float32)
        self.keep.append(a)
        return a

    def _check(self, ok, what):
        if not ok:
            raise RuntimeError(what + ": " + (self.lib.TSGgml_GetLastError() or b"").decode("utf-8", "replace"))

    def _head(self, row: np.ndarray) -> np.ndarray:
        lib = self.lib
        self._check(lib.TSGgml_NormF32(2, _v4(self.normed), _v4(row), _v4(self.out_norm), _v4(self.out_norm), 0, self.eps), "NormF32")
        self._check(lib.TSGgml_AddmmQuantF32(_v2(self.logits), _v2(self.normed), self.head_buf.ctypes.data, int(self.head_info.ggml_type),
                                             self.D, self.V, self.head_buf.nbytes), "AddmmQuantF32")
        return self.logits[0]

    # ------------------------------------------------------------------ the two passes
    def prefill(self, tokens) -> np.ndarray:
        """The prompt (from position 0) through the reference's fused per-layer exports; fills the KV cache."""
        lib, T, D, Hq, Hkv, Dh, eps = self.lib, len(tokens), self.D, self.Hq, self.Hkv, self.Dh, self.eps
        h = _aligned(T * D * 4).view(np.float32).reshape(T, D)
        for i, t in enumerate(tokens):
            lib.TSGgml_DequantizeToF32(int(self.emb_info.ggml_type), self.emb_buf.ctypes.data + int(t) * self.row_bytes, D, h[i].ctypes.data)
        nq, nkv = Hq * Dh, Hkv * Dh
        qkv_out = _aligned(T * (nq + 2 * nkv) * 4).view(np.float32).reshape(T, nq + 2 * nkv)
        attn = _aligned(T * nq * 4).view(np.float32).reshape(T, nq)
        tmp = _aligned(T * nq * 4).view(np.float32)

        def heads_view(a, H):            # [T, H * Dh] as the bridge's 4-D view (1, T, H, Dh)
            return View4D(a.ctypes.data, Dh, H, T, 1, Dh * 4, H * Dh * 4, T * H * Dh * 4, a.nbytes)

        for l in range(self.L):
            w = self.qkv[l]
            self._check(lib.TSGgml_FusedRmsNormMatMulQuantF32(_v2(qkv_out), _v2(h), self.an[l].ctypes.data, D, eps, *w), "FusedRmsNormMatMulQuant")
            q = np.ascontiguousarray(qkv_out[:, :nq])
            k = np.ascontiguousarray(qkv_out[:, nq:nq + nkv])
            v = np.ascontiguousarray(qkv_out[:, nq + nkv:])
            for x, H, wn in ((q, Hq, self.qn[l]), (k, Hkv, self.kn[l])):
                ps = np.repeat(np.arange(T, dtype=np.int32), H)
                rows, out = x.reshape(T * H, Dh), tmp[:T * H * Dh].reshape(T * H, Dh)
                self._check(lib.TSGgml_NormF32(2, _v4(out), _v4(rows), _v4(wn), _v4(wn), 0, eps), "NormF32")
                normed_rows = out.reshape(T, H * Dh)
                self._check(lib.TSGgml_RoPEExF32(heads_view(x, H), heads_view(normed_rows, H), Contig(ps.ctypes.data, ps.size, 3), Dh, 2, 0,
                                                 self.rope_base, 1.0, 0.0, 1.0, 0.0, 0.0, 0, 0), "RoPEExF32")
            self.kc[l].reshape(Hkv, self.max_seq, Dh)[:, :T] = k.reshape(T, Hkv, Dh).transpose(1, 0, 2)
            self.vc[l].reshape(Hkv, self.max_seq, Dh)[:, :T] = v.reshape(T, Hkv, Dh).transpose(1, 0, 2)
            self._check(lib.TSGgml_FusedPrefillAttentionF32(q.ctypes.data, k.ctypes.data, v.ctypes.data, attn.ctypes.data, Hq, Hkv, Dh, T, T, 0, 0,
                                                            float(Dh) ** -0.5, 1), "FusedPrefillAttention")
            self._check(lib.TSGgml_FusedOutProjFFNQuantF32(_v2(h), _v2(attn), *self.o[l], self.fn[l].ctypes.data, D, eps, *self.gu[l],
                                                           *self.down[l], self.F), "FusedOutProjFFNQuant")
        return self._head(h[T - 1:T])

    def decode(self, token: int, position: int) -> np.ndarray:
        """One token at ``position`` through the whole-model decode export (the cache must hold ``position`` tokens)."""
        lib, q0, o0, g0, d0 = self.lib, self.qkv[0], self.o[0], self.gu[0], self.down[0]
        lib.TSGgml_DequantizeToF32(int(self.emb_info.ggml_type), self.emb_buf.ctypes.data + int(token) * self.row_bytes, self.D,
                                   self.hidden.ctypes.data)
        self._check(lib.TSGgml_TransformerModelDecode(
            self.hidden.ctypes.data, self.D, self.L, *self.arrs,
            q0[1], q0[2], q0[3], q0[4], o0[1], o0[2], o0[3], o0[4], g0[1], g0[2], g0[3], g0[4], d0[1], d0[2], d0[3], d0[4],
            self.Dh, self.Hq, self.Hkv, self.max_seq, position, self.eps, self.rope_base, 1.0, self.F, 2), "TransformerModelDecode")
        return self._head(self.hidden.reshape(1, self.D))


def run(args, shape: dict) -> dict:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return None          # the reference is single-GPU (ggml_ops_core.cpp:136-149): extra ranks idle
    import torch
    from tensorsharp_b200.models import synth
    try:
        lib = load_library()
        os.makedirs(args.cache_dir, exist_ok=True)
        path = os.path.join(args.cache_dir, f"{args.model}-ref-uniform.gguf")
        if not os.path.exists(path + ".done"):
            s = dict(shape)
            s["scheme"] = "Q4_K_UNIFORM" if shape["scheme"] == "Q4_K_M" else shape["scheme"]
            synth.write_qwen3(path, **s, seed=0, device="cuda" if torch.cuda.is_available() else "cpu")
            open(path + ".done", "w").write("ok")
        P, K, W = args.prefill, args.steps, args.warmup
        m = RefQwen3(lib, path, P + K + W + 8)
    except RefUnavailable as exc:
        return unavailable(str(exc))
    D, V = m.D, m.V
    prefill_ms = None
    try:
        rng = np.random.default_rng(1)
        prompt = rng.integers(0, V, size=P).tolist()
        if os.environ.get("TSB_REF_PREFILL", "1") != "0":
            m.prefill(prompt[:min(P, 64)])                     # warm-up: context pools, weight uploads
            t0 = time.perf_counter()
            tok = int(np.argmax(m.prefill(prompt)))
            prefill_ms = (time.perf_counter() - t0) * 1e3
        else:
            tok = 100
        pos = P
        for _ in range(W):
            tok = int(np.argmax(m.decode(tok, pos)))
            pos += 1
        per_step = []
        t0 = time.perf_counter()
        for _ in range(K):
            t1 = time.perf_counter()
            tok = int(np.argmax(m.decode(tok, pos)))
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
                   "path": "decode: TSGgml_TransformerModelDecode + TSGgml_NormF32 + TSGgml_AddmmQuantF32; prefill: "
                           "TSGgml_FusedRmsNormMatMulQuantF32, TSGgml_NormF32, TSGgml_RoPEExF32, TSGgml_FusedPrefillAttentionF32, "
                           "TSGgml_FusedOutProjFFNQuantF32 per layer"},
        "prefill_tok_s": (P / (prefill_ms / 1e3)) if prefill_ms else None, "ttft_ms_p50": prefill_ms,
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
