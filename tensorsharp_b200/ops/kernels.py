"""ctypes bindings for the sm_100a kernels in ``libtsb200.so``.

Each function takes torch CUDA tensors, passes their raw pointers and the current
stream, and raises on a non-zero status.  There is no fallback here: if the library
is missing the call fails loudly.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from ..quant.qweight import QuantWeight
from . import native

ACT = {None: 0, "none": 0, "swiglu": 1, "geglu": 2, "geglu_tanh": 2, "geglu_erf": 3, "swiglu_oai": 4,
       "relu2": 5, "silu": 6, "sigmoid_mul": 7}

_vp = C.c_void_p


def _p(t: Optional[torch.Tensor]):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


def _stream():
    return _vp(torch.cuda.current_stream().cuda_stream)


# Debug mode TSB_CHECK_INDICES=1: before a launch, every index tensor that the kernel will use to address memory (token
# ids, KV slots, block-table pages, cache lengths, expert ids, state slots) is checked on the host against the size of
# what it indexes, and an IndexError names the kernel and the offending value instead of the kernel reading or writing out
# of bounds.  Each check synchronises the stream, so the mode is for debugging only (and cannot be used while a CUDA
# graph is being captured).  The kernels themselves index unchecked.
CHECK_INDICES = os.environ.get("TSB_CHECK_INDICES", "0") not in ("", "0")


def check_index(kernel: str, what: str, t: Optional[torch.Tensor], limit: int, low: int = 0) -> None:
    """Raise IndexError unless every element of ``t`` lies in ``[low, limit)``.  No-op unless TSB_CHECK_INDICES=1."""
    if not CHECK_INDICES or t is None or t.numel() == 0:
        return
    if t.is_cuda and torch.cuda.is_current_stream_capturing():
        return
    lo, hi = int(t.min().item()), int(t.max().item())
    if lo < low or hi >= limit:
        raise IndexError(f"{kernel}: {what} out of range: values span [{lo}, {hi}], allowed [{low}, {limit})")


def _planes(w: QuantWeight):
    ps = [_vp(p.data_ptr()) for p in w.planes]
    while len(ps) < 4:
        ps.append(_vp(0))
    return ps


class RopeParams(C.Structure):
    _fields_ = [("theta_base", C.c_float), ("freq_scale", C.c_float), ("ext_factor", C.c_float),
                ("attn_factor", C.c_float), ("corr_lo", C.c_float), ("corr_hi", C.c_float),
                ("rot_dim", C.c_int), ("mode", C.c_int)]


class QkvArgs(C.Structure):
    _fields_ = [("q", _vp), ("k", _vp), ("v", _vp),
                ("q_tok", C.c_long), ("q_head", C.c_long), ("k_tok", C.c_long), ("k_head", C.c_long),
                ("v_tok", C.c_long), ("v_head", C.c_long),
                ("in_f32", C.c_int), ("qn", _vp), ("kn", _vp), ("v_norm", C.c_int), ("eps", C.c_float),
                ("pos", _vp), ("slot", _vp), ("freq_factors", _vp), ("cs_table", _vp), ("q_out", _vp), ("k_cache", _vp),
                ("v_cache", _vp), ("q_scale", C.c_float),
                ("T", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("Dh", C.c_int), ("rp", RopeParams)]


class AttnArgs(C.Structure):
    _fields_ = [("q", _vp), ("k_cache", _vp), ("v_cache", _vp), ("out", _vp), ("block_table", _vp),
                ("kv_lens", _vp), ("cu_q", _vp), ("sinks", _vp), ("part_o", _vp), ("part_ml", _vp),
                ("scale", C.c_float), ("softcap", C.c_float), ("window", C.c_int),
                ("B", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("Dh", C.c_int), ("page_size", C.c_int),
                ("max_pages", C.c_int), ("splits", C.c_int), ("q_pos0", _vp), ("lse_out", _vp),
                ("out_q", _vp), ("out_ds", _vp), ("ticket", _vp), ("split_len", C.c_int)]


_configured = False
LAUNCHES = 0          # kernels launched through this module (eager mode; graph replays add theirs)


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def _lib():
    global _configured
    lib = native.lib()
    if not _configured:
        for name in ("tsb_quantize_q8", "tsb_gemv", "tsb_rmsnorm", "tsb_qkv_rope", "tsb_glu", "tsb_gather_rows",
                     "tsb_argmax", "tsb_rope_table", "tsb_fused_gemv", "tsb_gemv_push", "tsb_tp_reduce_norm", "tsb_tpseq_push_rows", "tsb_decode_advance", "tsb_attn_decode", "tsb_attn_prefill", "tsb_gemm_bf16", "tsb_causal_conv1d", "tsb_gdn_recurrent",
                     "tsb_mamba2_recurrent"):
            getattr(lib, name).restype = C.c_int
        _configured = True
    return lib


# --------------------------------------------------------------------------------------------
def quantize_q8(x: torch.Tensor):
    """x [rows, K] (bf16 or f32) -> (int8 [rows, K], float32 [rows, K/32, 2])."""
    assert x.is_cuda and x.is_contiguous()
    rows, K = x.shape
    xq = torch.empty((rows, K), dtype=torch.int8, device=x.device)
    xds = torch.empty((rows, K // 32, 2), dtype=torch.float32, device=x.device)
    native.check(_lib().tsb_quantize_q8(_p(x), C.c_int(x.dtype == torch.float32), _p(xq), _p(xds), C.c_long(rows),
                                        C.c_int(K), _stream()), "quantize_q8")
    _count(1)
    return xq, xds


def gemv(w: QuantWeight, *, xq=None, xds=None, xb=None, M: int, out_dtype=torch.float32, bias=None, residual=None,
         act=None, ids=None, row_scale=None, x_div: int = 1, out: Optional[torch.Tensor] = None,
         push: Optional[int] = None) -> Optional[torch.Tensor]:
    """Small-batch matvec over quantised weights.  With ``ids`` ([P] int32) each problem p
    uses expert ids[p], activation row p // x_div and output row p.  ``push`` (device address of a
    tensor-parallel exchange descriptor) sends the f32 result to every rank's mailbox instead of
    ``out``."""
    a = ACT[act]
    glu = 1 <= a <= 4
    n_out = w.N // 2 if glu else w.N
    problems = int(ids.numel()) if ids is not None else 1
    rows = problems if ids is not None else M
    dev = w.device
    if out is None and push is None:
        out = torch.empty((rows, n_out), dtype=out_dtype, device=dev)
    ps = _planes(w)
    native.check(_lib().tsb_gemv_push(ps[0], ps[1], ps[2], ps[3], C.c_int(int(w.ggml_type)), C.c_int(w.N), C.c_int(w.K),
                                      _p(xq), _p(xds), _p(xb), _p(out), _p(bias), _p(residual), _p(ids), _p(row_scale),
                                      C.c_int(M), C.c_int(problems), C.c_int(x_div),
                                      C.c_int(1 if (out is None or out.dtype == torch.float32) else 0), C.c_int(a),
                                      C.c_void_p(push) if push else None, _stream()), "gemv")
    _count(1)
    return out


def gemv_multi(ws, *, xq=None, xds=None, xb=None, M: int, out_dtype=torch.float32) -> torch.Tensor:
    """Two or three weight matrices over the same activations in one launch -> [M, sum of rows]."""
    n = len(ws)
    planes = (C.c_void_p * (4 * n))()
    for i, w in enumerate(ws):
        for j, p in enumerate(_planes(w)):
            planes[4 * i + j] = p.value if hasattr(p, "value") else p
    types = (C.c_int * n)(*[int(w.ggml_type) for w in ws])
    rows = (C.c_int * n)(*[w.N for w in ws])
    total = sum(w.N for w in ws)
    out = torch.empty((M, total), dtype=out_dtype, device=ws[0].device)
    native.check(_lib().tsb_gemv_multi(planes, types, rows, C.c_int(n), C.c_int(ws[0].K), _p(xq), _p(xds), _p(xb), _p(out),
                                       C.c_int(M), C.c_int(1 if out_dtype == torch.float32 else 0), _stream()), "gemv_multi")
    _count(1)
    return out


def moe_route(logits: torch.Tensor, k: int, *, mode: int = 0, sel_bias=None, normalize: bool = False, scale: float = 1.0):
    """Router on the device: f32 logits [T, E] -> (ids int32 [T, k], weights f32 [T, k]).  mode 0: top-k
    then softmax over the selected; mode 1: sigmoid, selection on p + sel_bias, optional renormalise, scale."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous()
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    native.check(_lib().tsb_moe_route(_p(logits), _p(sel_bias), C.c_int(T), C.c_int(E), C.c_int(k), C.c_int(mode),
                                      C.c_int(1 if normalize else 0), C.c_float(scale), _p(ids), _p(w), _stream()), "moe_route")
    _count(1)
    return ids, w


def moe_grouped(*, xq=None, xds=None, xb=None, ids: torch.Tensor, weights: torch.Tensor, gate_up: QuantWeight,
                down: QuantWeight, act, gate_up_bias=None, down_bias=None, expert_offset: int = 0) -> torch.Tensor:
    """Grouped expert projections with the routing kept on the device (no host read-back, fixed launch
    sequence): group the (token, slot) pairs by local expert, gather activations into that order, run
    gate/up and down as tile GEMVs (each tile streams its expert's rows once for up to 8 pairs), and
    sum every token's slots.  ``ids`` are global expert ids [T, k]; pairs whose expert is not in
    ``[expert_offset, expert_offset + gate_up.experts)`` contribute nothing.  Returns f32 [T, D]."""
    lib = _lib()
    T, k = ids.shape
    P = T * k
    dev = ids.device
    E_local = gate_up.experts
    a = ACT[act]
    glu = 1 <= a <= 4
    F_out = gate_up.N // 2 if glu else gate_up.N
    D, K = down.N, gate_up.K
    ids = ids.contiguous()
    pos = torch.empty((P,), dtype=torch.int32, device=dev)
    max_tiles = int(lib.tsb_moe_max_tiles(C.c_int(P), C.c_int(E_local)))
    tiles = torch.empty((max_tiles, 4), dtype=torch.int32, device=dev)
    meta = torch.empty((2,), dtype=torch.int32, device=dev)
    native.check(lib.tsb_moe_group(_p(ids), C.c_int(P), C.c_int(expert_offset), C.c_int(E_local), _p(pos), _p(tiles), _p(meta),
                                   _stream()), "moe_group")
    sq = sds = sb = None
    if xq is not None:
        sq = torch.zeros((P, K), dtype=torch.int8, device=dev)
        sds = torch.zeros((P, K // 32, 2), dtype=torch.float32, device=dev)
    else:
        sb = torch.zeros((P, K), dtype=torch.bfloat16, device=dev)
    sw = torch.zeros((P,), dtype=torch.float32, device=dev)
    wflat = weights.reshape(-1).float().contiguous()
    native.check(lib.tsb_moe_gather(_p(pos), C.c_int(P), C.c_int(k), C.c_int(K), _p(xq), _p(xds), _p(xb), _p(wflat), _p(sq),
                                    _p(sds), _p(sb), _p(sw), _stream()), "moe_gather")
    gu = torch.zeros((P, F_out), dtype=torch.bfloat16, device=dev)
    ps = _planes(gate_up)
    native.check(lib.tsb_moe_gemv_tiles(ps[0], ps[1], ps[2], ps[3], C.c_int(int(gate_up.ggml_type)), C.c_int(gate_up.N), C.c_int(K),
                                        _p(sq), _p(sds), _p(sb), _p(gu), _p(gate_up_bias), None, _p(tiles), _p(meta),
                                        C.c_int(max_tiles), C.c_int(0), C.c_int(a), _stream()), "moe_gemv_tiles(gate_up)")
    y = torch.empty((P, D), dtype=torch.float32, device=dev)
    ps = _planes(down)
    if down.uses_q8_activations:
        gq, gds = quantize_q8(gu)
        gb = None
    else:
        gq = gds = None
        gb = gu
    native.check(lib.tsb_moe_gemv_tiles(ps[0], ps[1], ps[2], ps[3], C.c_int(int(down.ggml_type)), C.c_int(D), C.c_int(F_out),
                                        _p(gq), _p(gds), _p(gb), _p(y), _p(down_bias), _p(sw), _p(tiles), _p(meta),
                                        C.c_int(max_tiles), C.c_int(1), C.c_int(0), _stream()), "moe_gemv_tiles(down)")
    out = torch.empty((T, D), dtype=torch.float32, device=dev)
    native.check(lib.tsb_moe_combine(_p(y), _p(pos), C.c_int(T), C.c_int(k), C.c_int(D), _p(out), _stream()), "moe_combine")
    _count(5)
    return out


def moe_combine_weighted(y: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, T: int, k: int) -> torch.Tensor:
    """out[t] = sum_j w[t, j] * y[pos[t * k + j]] (f32 rows; pos < 0 = no row): each token gathers its own rows, so the
    sum has a fixed order and needs no atomics."""
    D = y.shape[1]
    assert y.dtype == torch.float32 and y.is_contiguous() and pos.dtype == torch.int32 and w.dtype == torch.float32
    out = torch.empty((T, D), dtype=torch.float32, device=y.device)
    lib = _lib()
    lib.tsb_moe_combine_weighted.restype = C.c_int
    native.check(lib.tsb_moe_combine_weighted(_p(y), _p(pos.contiguous()), _p(w.contiguous()), C.c_int(T), C.c_int(k), C.c_int(D),
                                              _p(out), _stream()), "moe_combine_weighted")
    _count(1)
    return out


def sample(logits: torch.Tensor, ngen: torch.Tensor, *, temperature: float, top_k: int, top_p: float, min_p: float,
           repetition_penalty: float = 1.0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0, seed: int = 0,
           counts: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Draw one token per row of f32 logits [B, V] on the device (reference order of transformations).
    ``ngen`` [B] int32 counts the tokens drawn so far per row and keys the random stream; ``counts``
    [B, V] int32 holds the occurrences of each id for the penalties.  Both are advanced by the kernel."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous()
    B, V = logits.shape
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    native.check(_lib().tsb_sample(_p(logits), _p(counts), _p(ngen), _p(out), C.c_int(B), C.c_int(V), C.c_float(temperature),
                                   C.c_int(top_k), C.c_float(top_p), C.c_float(min_p), C.c_float(repetition_penalty),
                                   C.c_float(presence_penalty), C.c_float(frequency_penalty),
                                   C.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _stream()), "sample")
    _count(1)
    return out


def device_sampler_supports(cfg) -> bool:
    """Settings the device sampler reproduces exactly (the rest stay with the host sampler)."""
    if cfg.temperature <= 0:
        return True
    return (1 <= cfg.top_k <= 1024) or (cfg.top_k <= 0 and cfg.top_p >= 1.0)


def fused_gemv(w: QuantWeight, *, x_f32=None, x_bf16=None, norm_w=None, eps: float = 0.0, do_norm: bool = False,
               out_dtype=torch.float32, bias=None, residual=None, act=None, out: Optional[torch.Tensor] = None,
               push: Optional[int] = None) -> Optional[torch.Tensor]:
    """Decode GEMV (at most 4 rows) with RMSNorm / cast + int8 quantisation of the input done
    inside the kernel.  ``push`` is the device address of a tensor-parallel exchange descriptor:
    the result then goes to the mailboxes and nothing is returned."""
    x = x_f32 if x_f32 is not None else x_bf16
    assert x.is_cuda and x.is_contiguous() and x.shape[-1] == w.K
    M = x.numel() // w.K
    a = ACT[act]
    glu = 1 <= a <= 4
    n_out = w.N // 2 if glu else w.N
    if push is None and out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=w.device)
    ps = _planes(w)
    lib = _lib()
    native.check(lib.tsb_fused_gemv(ps[0], ps[1], ps[2], ps[3], C.c_int(int(w.ggml_type)), C.c_int(w.N), C.c_int(w.K),
                                    _p(x_f32), _p(x_bf16), _p(norm_w), C.c_float(eps), C.c_int(1 if do_norm else 0),
                                    _p(out), _p(bias), _p(residual), C.c_int(M),
                                    C.c_int(1 if (out is None or out.dtype == torch.float32) else 0), C.c_int(a),
                                    C.c_void_p(push) if push else None, _stream()), "fused_gemv")
    _count(1)
    return out


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, *, delta=None, want_bf16=True, want_q8=False,
            want_f32=False, add=None, l2=False):
    """Fused (x += delta) -> RMSNorm -> {bf16, f32 (+add), q8}.  Returns (y_bf16, y_f32, yq, yds)."""
    assert x.is_cuda and x.is_contiguous()
    D = x.shape[-1]
    rows = x.numel() // D
    dev = x.device
    yb = torch.empty(x.shape, dtype=torch.bfloat16, device=dev) if want_bf16 else None
    yf = torch.empty(x.shape, dtype=torch.float32, device=dev) if (want_f32 or add is not None) else None
    yq = yds = None
    if want_q8:
        yq = torch.empty((rows, D), dtype=torch.int8, device=dev)
        yds = torch.empty((rows, D // 32, 2), dtype=torch.float32, device=dev)
    native.check(_lib().tsb_rmsnorm(_p(x), C.c_int(x.dtype == torch.float32), _p(delta), _p(w), C.c_float(eps),
                                    C.c_long(rows), C.c_int(D), _p(yb), _p(yf), _p(add), _p(yq), _p(yds),
                                    C.c_int(1 if l2 else 0), _stream()), "rmsnorm")
    _count(1)
    return yb, yf, yq, yds


def yarn_corr_dims(n_dims: int, n_ctx_orig: int, freq_base: float, beta_fast: float, beta_slow: float):
    """ggml's rope_yarn_corr_dims: the pair-index range over which YaRN blends."""
    def corr(n_rot):
        return n_dims * math.log(n_ctx_orig / (n_rot * 2 * math.pi)) / (2 * math.log(freq_base))
    lo = max(0.0, math.floor(corr(beta_fast)))
    hi = min(n_dims - 1.0, math.ceil(corr(beta_slow)))
    return lo, hi


def qkv_rope(*, q, k, v, q_strides, k_strides, v_strides, Hq, Hkv, Dh, pos, slot, q_out, k_cache, v_cache,
             qn=None, kn=None, v_norm=False, eps=1e-6, rope: RopeParams, freq_factors=None, q_scale=1.0,
             cs_table=None):
    T = int(pos.numel())
    check_index("qkv_rope", "KV slot", slot, k_cache.shape[0] if k_cache is not None else 1 << 62)
    check_index("qkv_rope", "position", pos, 1 << 31)
    a = QkvArgs()
    a.q, a.k, a.v = _p(q), _p(k), _p(v)
    a.q_tok, a.q_head = q_strides
    a.k_tok, a.k_head = k_strides
    a.v_tok, a.v_head = v_strides
    a.in_f32 = int(q.dtype == torch.float32)
    a.qn, a.kn = _p(qn), _p(kn)
    a.v_norm = int(v_norm)
    a.eps = eps
    a.pos, a.slot, a.freq_factors = _p(pos), _p(slot), _p(freq_factors)
    a.cs_table = _p(cs_table)
    a.q_out, a.k_cache, a.v_cache = _p(q_out), _p(k_cache), _p(v_cache)
    a.q_scale = q_scale
    a.T, a.Hq, a.Hkv, a.Dh = T, Hq, Hkv, Dh
    a.rp = rope
    native.check(_lib().tsb_qkv_rope(C.byref(a), _stream()), "qkv_rope")
    _count(1)


def rope_table(pos: torch.Tensor, rope: RopeParams, freq_factors=None) -> torch.Tensor:
    """(cos, sin) for every (token, rotary pair): float32 [T, rot_dim / 2, 2]."""
    T = int(pos.numel())
    out = torch.empty((T, rope.rot_dim // 2, 2), dtype=torch.float32, device=pos.device)
    native.check(_lib().tsb_rope_table(_p(pos), C.byref(rope), _p(freq_factors), _p(out), C.c_int(T), _stream()),
                 "rope_table")
    _count(1)
    return out


def glu(gate: torch.Tensor, up: Optional[torch.Tensor], act: str, F: int, g_stride: int, u_stride: int, rows: int,
        want_bf16=True, want_q8=False):
    dev = gate.device
    out = torch.empty((rows, F), dtype=torch.bfloat16, device=dev) if want_bf16 else None
    yq = yds = None
    if want_q8:
        yq = torch.empty((rows, F), dtype=torch.int8, device=dev)
        yds = torch.empty((rows, F // 32, 2), dtype=torch.float32, device=dev)
    native.check(_lib().tsb_glu(_p(gate), _p(up), C.c_int(gate.dtype == torch.float32), C.c_long(g_stride),
                                C.c_long(u_stride), C.c_long(rows), C.c_int(F), C.c_int(ACT[act]), _p(out), _p(yq),
                                _p(yds), _stream()), "glu")
    _count(1)
    return out, yq, yds


def gather_rows(w: QuantWeight, ids: Optional[torch.Tensor], scale: float = 1.0, out_dtype=torch.bfloat16,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Embedding lookup (ids given) or whole-matrix decode to ``out_dtype`` (ids None)."""
    n = int(ids.numel()) if ids is not None else w.rows
    check_index("gather_rows", "row id", ids, w.rows)
    if out is None:
        out = torch.empty((n, w.K), dtype=out_dtype, device=w.device)
    ps = _planes(w)
    native.check(_lib().tsb_gather_rows(ps[0], ps[1], ps[2], ps[3], C.c_int(int(w.ggml_type)), C.c_int(w.rows),
                                        C.c_int(w.K), _p(ids), C.c_long(n), C.c_float(scale), _p(out),
                                        C.c_int(out.dtype == torch.float32), _stream()), "gather_rows")
    _count(1)
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    native.check(_lib().tsb_argmax(_p(logits), C.c_long(logits.stride(0)), C.c_long(rows), C.c_int(V), _p(out), _vp(0),
                                   _stream()), "argmax")
    _count(1)
    return out


def decode_advance(sampled, batch) -> None:
    """In-place, on the device: next tokens = sampled, positions / kv_lens += 1, new KV slots."""
    B = batch.tokens.shape[0]
    native.check(_lib().tsb_decode_advance(_p(sampled), _p(batch.tokens), _p(batch.positions), _p(batch.kv_lens),
                                           _p(batch.slots), _p(batch.block_table), C.c_int(batch.block_table.shape[1]),
                                           C.c_int(batch.page_size), C.c_int(B), _stream()), "decode_advance")
    _count(1)


def _attn_args(q, k_cache, v_cache, out, block_table, kv_lens, cu_q, sinks, scale, softcap, window, Hq, Hkv, Dh,
               page_size, B):
    check_index("attention", "block-table page", block_table, k_cache.shape[0] // page_size)
    check_index("attention", "cache length", kv_lens, block_table.shape[1] * page_size + 1)
    a = AttnArgs()
    a.q, a.k_cache, a.v_cache, a.out = _p(q), _p(k_cache), _p(v_cache), _p(out)
    a.block_table, a.kv_lens, a.cu_q, a.sinks = _p(block_table), _p(kv_lens), _p(cu_q), _p(sinks)
    a.scale, a.softcap, a.window = scale, softcap or 0.0, int(window or 0)
    a.B, a.Hq, a.Hkv, a.Dh, a.page_size = B, Hq, Hkv, Dh, page_size
    a.max_pages = block_table.shape[1]
    a.splits = 1
    return a


def attn_decode(q, k_cache, v_cache, block_table, kv_lens, *, scale, Hq, Hkv, Dh, page_size, splits, sinks=None,
                softcap=0.0, window=0, out=None, want_q8=False, split_len=0):
    """q [B, Hq, Dh] bf16; one query per sequence against the paged cache.  ``want_q8`` also returns the
    output as int8 groups of 32 with (scale, sum) written by the combine kernel: (out, q, ds)."""
    B = q.shape[0]
    if out is None:
        out = torch.empty_like(q)
    a = _attn_args(q, k_cache, v_cache, out, block_table, kv_lens, None, sinks, scale, softcap, window, Hq, Hkv, Dh,
                   page_size, B)
    a.splits = splits
    a.split_len = split_len
    part_o = torch.empty((B, Hq, splits, Dh), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((B, Hq, splits, 2), dtype=torch.float32, device=q.device)
    a.part_o, a.part_ml = _p(part_o), _p(part_ml)
    oq = ods = None
    if want_q8 and Dh % 32 == 0:
        oq = torch.empty((B, Hq * Dh), dtype=torch.int8, device=q.device)
        ods = torch.empty((B, Hq * Dh // 32, 2), dtype=torch.float32, device=q.device)
        a.out_q, a.out_ds = oq.data_ptr(), ods.data_ptr()
    if k_cache.dtype in FP8_DTYPES:           # e4m3 pages: the split kernel that reads bytes, the same merge kernel
        lib = _lib()
        lib.tsb_attn_decode_fp8.restype = C.c_int
        native.check(lib.tsb_attn_decode_fp8(C.byref(a), _stream()), "attn_decode_fp8")
    else:
        native.check(_lib().tsb_attn_decode(C.byref(a), _stream()), "attn_decode")
    _count(2)
    return (out, oq, ods) if want_q8 else out


FP8_DTYPES = (torch.float8_e4m3fn,)


def kv_store_fp8(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor) -> None:
    """Dense bf16 rows ``k`` / ``v`` ``[T, Hkv, Dh]`` -> e4m3 bytes at ``slots`` (int64 ``[T]``) of the paged caches."""
    assert k.dtype == v.dtype == torch.bfloat16 and k.is_contiguous() and v.is_contiguous() and slots.dtype == torch.int64
    assert k_cache.dtype in FP8_DTYPES and v_cache.dtype in FP8_DTYPES and k_cache.is_contiguous() and v_cache.is_contiguous()
    T, Hkv, Dh = k.shape
    check_index("kv_store_fp8", "cache slot", slots, k_cache.shape[0])
    lib = _lib()
    lib.tsb_kv_store_fp8.restype = C.c_int
    native.check(lib.tsb_kv_store_fp8(_p(k), _p(v), _p(k_cache), _p(v_cache), _p(slots), C.c_long(T), C.c_int(Hkv), C.c_int(Dh),
                                      _stream()), "kv_store_fp8")
    _count(1)


def kv_load_fp8(k_cache: torch.Tensor, v_cache: torch.Tensor, idx: torch.Tensor):
    """Rows ``idx`` (int64 ``[n]``) of the e4m3 caches as dense bf16 ``[n, Hkv, Dh]`` tensors (K, V)."""
    assert k_cache.dtype in FP8_DTYPES and v_cache.dtype in FP8_DTYPES and idx.dtype == torch.int64 and idx.is_contiguous()
    n, (_, Hkv, Dh) = idx.numel(), k_cache.shape
    check_index("kv_load_fp8", "cache slot", idx, k_cache.shape[0])
    ko = torch.empty((n, Hkv, Dh), dtype=torch.bfloat16, device=idx.device)
    vo = torch.empty_like(ko)
    lib = _lib()
    lib.tsb_kv_load_fp8.restype = C.c_int
    native.check(lib.tsb_kv_load_fp8(_p(k_cache), _p(v_cache), _p(idx), _p(ko), _p(vo), C.c_long(n), C.c_int(Hkv), C.c_int(Dh),
                                     _stream()), "kv_load_fp8")
    _count(1)
    return ko, vo


def attn_prefill(q, k_cache, v_cache, block_table, kv_lens, cu_q, max_q_len, *, scale, Hq, Hkv, Dh, page_size,
                 sinks=None, softcap=0.0, window=0, out=None, q_pos0=None, lse_out=None):
    """q [T, Hq, Dh] bf16 packed over sequences (cu_q [B+1]).  ``q_pos0`` [B] int32 overrides the cache
    position of each sequence's first query (default kv_len - q_len); ``lse_out`` [T, Hq] f32 receives the
    log-sum-exp of the scores, for merging partial results over KV shards."""
    B = kv_lens.shape[0]
    if out is None:
        out = torch.empty_like(q)
    a = _attn_args(q, k_cache, v_cache, out, block_table, kv_lens, cu_q, sinks, scale, softcap, window, Hq, Hkv, Dh,
                   page_size, B)
    a.q_pos0 = q_pos0.data_ptr() if q_pos0 is not None else None
    a.lse_out = lse_out.data_ptr() if lse_out is not None else None
    native.check(_lib().tsb_attn_prefill(C.byref(a), C.c_int(max_q_len), _stream()), "attn_prefill")
    _count(1)
    return out


_status_words = {}


def gemm_status(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


_SPLITK_WS: dict = {}


def _splitk_workspace(device) -> Optional[torch.Tensor]:
    """Per-device float32 scratch (16 MB) for the partial tiles of split-K GEMMs; launches on one stream reuse it in order."""
    if os.environ.get("TSB_GEMM_SPLITK", "1") == "0":
        return None
    key = torch.device(device).index or 0
    ws = _SPLITK_WS.get(key)
    if ws is None:
        ws = _SPLITK_WS[key] = torch.empty(4 << 20, dtype=torch.float32, device=device)
    return ws


def gemm_bf16(W: torch.Tensor, X: torch.Tensor, *, out_dtype=torch.bfloat16, bias=None, residual=None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[T, N] = X[T, K] @ W[N, K]^T on tcgen05 tensor cores (bf16 in, f32 accumulate)."""
    assert W.dtype == torch.bfloat16 and X.dtype == torch.bfloat16
    assert W.stride(1) == 1 and X.stride(1) == 1
    N, K = W.shape
    T = X.shape[0]
    if out is None:
        out = torch.empty((T, N), dtype=out_dtype, device=X.device)
    ws = _splitk_workspace(X.device) if T <= 64 else None       # few tiles, long K: the library may split K over CTAs
    lib = _lib()
    lib.tsb_gemm_bf16_ws.restype = C.c_int
    native.check(lib.tsb_gemm_bf16_ws(_p(W), C.c_long(W.stride(0)), _p(X), C.c_long(X.stride(0)), _p(out),
                                      C.c_long(out.stride(0)), C.c_int(out.dtype == torch.float32), _p(bias),
                                      _p(residual), C.c_int(T), C.c_int(N), C.c_int(K), _p(gemm_status(X.device)),
                                      _stream(), _p(ws), C.c_long(ws.numel() * 4 if ws is not None else 0)), "gemm_bf16")
    _count(1)
    return out


def gemm_bf16_grouped(W: torch.Tensor, E: int, X: torch.Tensor, tiles: torch.Tensor, bn: int, *, out_dtype=torch.bfloat16,
                      bias=None) -> torch.Tensor:
    """Grouped GEMM over a stack of ``E`` matrices: W [E * N, K] bf16, X [P, K] bf16 with each group's rows contiguous,
    ``tiles`` int32 [n_tiles, 3] on the device = (matrix index or -1, first row, end row) with at most ``bn`` rows per
    tile -> out [P, N], zero where no tile covers a row."""
    assert W.dtype == torch.bfloat16 and X.dtype == torch.bfloat16 and W.stride(1) == 1 and X.stride(1) == 1
    assert tiles.dtype == torch.int32 and tiles.is_contiguous() and tiles.shape[1] == 3
    N, K = W.shape[0] // E, W.shape[1]
    P = X.shape[0]
    out = torch.zeros((P, N), dtype=out_dtype, device=X.device)
    lib = _lib()
    lib.tsb_gemm_bf16_grouped.restype = C.c_int
    native.check(lib.tsb_gemm_bf16_grouped(_p(W), C.c_long(W.stride(0)), C.c_int(E), _p(X), C.c_long(X.stride(0)), _p(out),
                                           C.c_long(out.stride(0)), C.c_int(out.dtype == torch.float32), _p(bias), C.c_int(P),
                                           C.c_int(N), C.c_int(K), _p(tiles), C.c_int(tiles.shape[0]), C.c_int(bn),
                                           _p(gemm_status(X.device)), _stream()), "gemm_bf16_grouped")
    _count(1)
    return out


# --------------------------------------------------------------------------------------------
class ConvArgs(C.Structure):
    _fields_ = [("x", _vp), ("xs", C.c_long), ("x_f32", C.c_int), ("w", _vp), ("bias", _vp), ("state", _vp),
                ("cu_q", _vp), ("seq_slots", _vp), ("out", _vp), ("os", C.c_long),
                ("C", C.c_int), ("K", C.c_int), ("B", C.c_int), ("act", C.c_int)]


class GdnArgs(C.Structure):
    _fields_ = [("qkv", _vp), ("qkv_s", C.c_long), ("z", _vp), ("z_s", C.c_long), ("z_f32", C.c_int),
                ("beta", _vp), ("alpha", _vp), ("ba_s", C.c_long), ("ba_f32", C.c_int),
                ("dt_bias", _vp), ("a", _vp), ("norm_w", _vp), ("state", _vp), ("cu_q", _vp), ("seq_slots", _vp),
                ("out", _vp), ("out_s", C.c_long), ("eps", C.c_float),
                ("Hk", C.c_int), ("Hv", C.c_int), ("Dk", C.c_int), ("Dv", C.c_int), ("B", C.c_int)]


class GdnCarryArgs(C.Structure):
    _fields_ = [("U0", _vp), ("W", _vp), ("Qd", _vp), ("Kd", _vp), ("P", _vp), ("gamma", _vp), ("state", _vp), ("out", _vp),
                ("Hv", C.c_int), ("nc", C.c_int), ("Dk", C.c_int), ("Dv", C.c_int)]


class GdnPrepArgs(C.Structure):
    _fields_ = [("qkv", _vp), ("qkv_s", C.c_long), ("beta", _vp), ("alpha", _vp), ("ba_s", C.c_long), ("ba_f32", C.c_int),
                ("dt_bias", _vp), ("a_log", _vp), ("cu_q", _vp),
                ("U0", _vp), ("W", _vp), ("Qd", _vp), ("Kd", _vp), ("P", _vp), ("gamma", _vp),
                ("Hk", C.c_int), ("Hv", C.c_int), ("Dk", C.c_int), ("Dv", C.c_int), ("B", C.c_int), ("nc", C.c_int),
                ("eps", C.c_float)]


class GdnFinishArgs(C.Structure):
    _fields_ = [("core", _vp), ("z", _vp), ("z_s", C.c_long), ("z_f32", C.c_int), ("norm_w", _vp), ("cu_q", _vp),
                ("out", _vp), ("out_s", C.c_long), ("Hv", C.c_int), ("Dv", C.c_int), ("B", C.c_int), ("nc", C.c_int),
                ("eps", C.c_float)]


class MambaArgs(C.Structure):
    _fields_ = [("xbc", _vp), ("xbc_s", C.c_long), ("dt", _vp), ("dt_s", C.c_long), ("dt_f32", C.c_int),
                ("dt_bias", _vp), ("A", _vp), ("D", _vp), ("state", _vp), ("cu_q", _vp), ("seq_slots", _vp),
                ("y", _vp), ("y_s", C.c_long),
                ("H", C.c_int), ("P", C.c_int), ("G", C.c_int), ("N", C.c_int), ("B", C.c_int)]


def causal_conv1d(x, w, bias, state, cu_q, seq_slots, max_q, act_silu=True) -> torch.Tensor:
    """x [T, C] view (row stride allowed) -> f32 [T, C]; the per-slot tail ``state`` is updated."""
    T, Cc = x.shape
    check_index("causal_conv1d", "state slot", seq_slots, state.shape[0])
    out = torch.empty((T, Cc), dtype=torch.float32, device=x.device)
    a = ConvArgs()
    a.x, a.xs, a.x_f32 = _p(x), x.stride(0), int(x.dtype == torch.float32)
    a.w, a.bias, a.state = _p(w), _p(bias), _p(state)
    a.cu_q, a.seq_slots, a.out, a.os = _p(cu_q), _p(seq_slots), _p(out), Cc
    a.C, a.K, a.B, a.act = Cc, w.shape[1], cu_q.numel() - 1, 1 if act_silu else 0
    native.check(_lib().tsb_causal_conv1d(C.byref(a), C.c_int(max_q), _stream()), "causal_conv1d")
    _count(2)
    return out


def gdn_recurrent(qkv, z, beta, alpha, dt_bias, a_log, norm_w, state, cu_q, seq_slots, *, Hk, Hv, Dk, Dv, eps):
    T = qkv.shape[0]
    check_index("gdn_recurrent", "state slot", seq_slots, state.shape[0])
    check_index("gdn_recurrent", "row offset", cu_q, T + 1)
    out = torch.empty((T, Hv * Dv), dtype=torch.bfloat16, device=qkv.device)
    assert qkv.dtype == torch.float32 and beta.dtype == alpha.dtype and beta.stride(0) == alpha.stride(0)
    a = GdnArgs()
    a.qkv, a.qkv_s = _p(qkv), qkv.stride(0)
    a.z, a.z_s, a.z_f32 = _p(z), z.stride(0), int(z.dtype == torch.float32)
    a.beta, a.alpha, a.ba_s, a.ba_f32 = _p(beta), _p(alpha), beta.stride(0), int(beta.dtype == torch.float32)
    a.dt_bias, a.a, a.norm_w, a.state = _p(dt_bias), _p(a_log), _p(norm_w), _p(state)
    a.cu_q, a.seq_slots, a.out, a.out_s, a.eps = _p(cu_q), _p(seq_slots), _p(out), Hv * Dv, eps
    a.Hk, a.Hv, a.Dk, a.Dv, a.B = Hk, Hv, Dk, Dv, cu_q.numel() - 1
    native.check(_lib().tsb_gdn_recurrent(C.byref(a), _stream()), "gdn_recurrent")
    _count(1)
    return out


def gdn_chunk_carry_supported(Dk: int, Dv: int, chunk: int) -> bool:
    return chunk == 64 and Dk in (64, 128) and Dv % 32 == 0


def gdn_chunked_supported(Dk: int, Dv: int) -> bool:
    return Dk in (64, 128) and Dv % 32 == 0 and Dv <= 128


def gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, state, cu_q, h_cu_q, slots, *, Hk, Hv, Dk, Dv, eps) -> torch.Tensor:
    """Chunked GatedDeltaNet prefill of a packed batch in three kernels (csrc/gdn_chunk.cu): the chunk-parallel algebra
    (normalisation, decay, Gram products, the triangular solve) per (sequence, head, chunk); the state carried chunk
    after chunk per (sequence, head, value slice); the gated output norm.  ``state`` [slots, Hv, Dv, Dk] f32 is updated
    for the sequences' slots (host list ``slots``); ``cu_q`` int32 [B + 1] on the device, ``h_cu_q`` its host copy.
    Returns bf16 [T, Hv * Dv]."""
    T = qkv.shape[0]
    B = len(h_cu_q) - 1
    nc = (max(h_cu_q[i + 1] - h_cu_q[i] for i in range(B)) + 63) // 64
    dev = qkv.device
    assert qkv.dtype == torch.float32 and qkv.stride(1) == 1 and beta.dtype == alpha.dtype and beta.stride(0) == alpha.stride(0)
    BH = B * Hv
    f32 = dict(dtype=torch.float32, device=dev)
    U0, W = torch.empty((BH, nc, 64, Dv), **f32), torch.empty((BH, nc, 64, Dk), **f32)
    Qd, Kd = torch.empty((BH, nc, 64, Dk), **f32), torch.empty((BH, nc, 64, Dk), **f32)
    P, gamma = torch.empty((BH, nc, 64, 64), **f32), torch.empty((BH, nc), **f32)
    a = GdnPrepArgs()
    a.qkv, a.qkv_s = _p(qkv), qkv.stride(0)
    a.beta, a.alpha, a.ba_s, a.ba_f32 = _p(beta), _p(alpha), beta.stride(0), int(beta.dtype == torch.float32)
    a.dt_bias, a.a_log, a.cu_q = _p(dt_bias), _p(a_log), _p(cu_q)
    a.U0, a.W, a.Qd, a.Kd, a.P, a.gamma = _p(U0), _p(W), _p(Qd), _p(Kd), _p(P), _p(gamma)
    a.Hk, a.Hv, a.Dk, a.Dv, a.B, a.nc, a.eps = Hk, Hv, Dk, Dv, B, nc, eps
    lib = _lib()
    native.check(lib.tsb_gdn_chunk_prep(C.byref(a), _stream()), "gdn_chunk_prep")
    _count(1)
    if B == 1:
        S = state[slots[0]]
    else:
        idx = torch.tensor(slots, dtype=torch.long, device=dev)
        S = state[idx].reshape(BH, Dv, Dk)
    core = gdn_chunk_carry(U0, W, Qd, Kd, P, gamma, S)
    if B > 1:
        state[idx] = S.view(B, Hv, Dv, Dk)
    out = torch.empty((T, Hv * Dv), dtype=torch.bfloat16, device=dev)
    f = GdnFinishArgs()
    f.core, f.z, f.z_s, f.z_f32 = _p(core), _p(z), z.stride(0), int(z.dtype == torch.float32)
    f.norm_w, f.cu_q, f.out, f.out_s = _p(norm_w), _p(cu_q), _p(out), Hv * Dv
    f.Hv, f.Dv, f.B, f.nc, f.eps = Hv, Dv, B, nc, eps
    native.check(lib.tsb_gdn_chunk_finish(C.byref(f), _stream()), "gdn_chunk_finish")
    _count(1)
    return out


class MambaPrepArgs(C.Structure):
    _fields_ = [("xbc", _vp), ("xbc_s", C.c_long), ("dt", _vp), ("dt_s", C.c_long), ("dt_f32", C.c_int),
                ("dt_bias", _vp), ("A", _vp), ("cu_q", _vp),
                ("U0", _vp), ("Qd", _vp), ("Kd", _vp), ("P", _vp), ("gamma", _vp),
                ("H", C.c_int), ("Pd", C.c_int), ("G", C.c_int), ("N", C.c_int), ("B", C.c_int), ("nc", C.c_int)]


def mamba2_chunked_supported(N: int, P: int) -> bool:
    return N in (64, 128) and P % 32 == 0


def mamba2_chunked(xbc, dt, dt_bias, A, D, state, cu_q, h_cu_q, slots, *, H, P, G, N) -> torch.Tensor:
    """Chunked Mamba2 prefill of a packed batch in two kernels (csrc/gdn_chunk.cu): the chunk-parallel algebra per
    (sequence, head, chunk) - step sizes, running decay, C B^T with its decay mask, decayed reads and writes - and the
    chunk-carry kernel of the delta rule with nothing to correct.  ``xbc`` f32 [T, H P + 2 G N] (after the convolution),
    ``state`` [slots, H, P, N] f32 updated for the sequences' slots.  Returns y f32 [T, H * P] (skip term included)."""
    T = xbc.shape[0]
    B = len(h_cu_q) - 1
    nc = (max(h_cu_q[i + 1] - h_cu_q[i] for i in range(B)) + 63) // 64
    dev = xbc.device
    assert xbc.dtype == torch.float32 and xbc.stride(1) == 1 and dt.stride(1) == 1 and state.dtype == torch.float32
    BH = B * H
    f32 = dict(dtype=torch.float32, device=dev)
    U0 = torch.empty((BH, nc, 64, P), **f32)
    Qd, Kd = torch.empty((BH, nc, 64, N), **f32), torch.empty((BH, nc, 64, N), **f32)
    Pm, gamma = torch.empty((BH, nc, 64, 64), **f32), torch.empty((BH, nc), **f32)
    a = MambaPrepArgs()
    a.xbc, a.xbc_s = _p(xbc), xbc.stride(0)
    a.dt, a.dt_s, a.dt_f32 = _p(dt), dt.stride(0), int(dt.dtype == torch.float32)
    a.dt_bias, a.A, a.cu_q = _p(dt_bias.float().contiguous() if dt_bias is not None else None), _p(A.float().contiguous()), _p(cu_q)
    a.U0, a.Qd, a.Kd, a.P, a.gamma = _p(U0), _p(Qd), _p(Kd), _p(Pm), _p(gamma)
    a.H, a.Pd, a.G, a.N, a.B, a.nc = H, P, G, N, B, nc
    lib = _lib()
    lib.tsb_mamba2_chunk_prep.restype = C.c_int
    native.check(lib.tsb_mamba2_chunk_prep(C.byref(a), _stream()), "mamba2_chunk_prep")
    _count(1)
    if B == 1:
        S = state[slots[0]]
    else:
        idx = torch.tensor(slots, dtype=torch.long, device=dev)
        S = state[idx].reshape(BH, P, N)
    core = gdn_chunk_carry(U0, None, Qd, Kd, Pm, gamma, S)           # [BH, nc, 64, P]; W = 0: nothing to correct
    if B > 1:
        state[idx] = S.view(B, H, P, N)
    y = torch.empty((T, H, P), **f32)
    for b in range(B):
        q0, n = h_cu_q[b], h_cu_q[b + 1] - h_cu_q[b]
        y[q0:q0 + n] = core[b * H:(b + 1) * H].reshape(H, nc * 64, P)[:, :n].transpose(0, 1)
    if D is not None:
        y = y + D.float().view(1, H, 1) * xbc[:, :H * P].view(T, H, P)
    return y.view(T, H * P)


def gdn_chunk_carry(U0, W, Qd, Kd, P, gamma, state) -> torch.Tensor:
    """The sequential part of the chunked GatedDeltaNet prefill for one sequence: ``state`` [Hv, Dv, Dk] f32 (contiguous,
    updated in place) carried through the chunks of U0 [Hv, nc, 64, Dv], W / Qd / Kd [Hv, nc, 64, Dk], P [Hv, nc, 64, 64],
    gamma [Hv, nc] -> outputs [Hv, nc, 64, Dv] f32.  ``W`` None stands for zeros (no correction term)."""
    U0, Qd, Kd, P, gamma = (t.float().contiguous() for t in (U0, Qd, Kd, P, gamma))
    W = W.float().contiguous() if W is not None else None              # None: nothing to correct (the Mamba2 form)
    Hv, nc, Cn, Dv = U0.shape
    Dk = Qd.shape[-1]
    assert Cn == 64 and state.dtype == torch.float32 and state.is_contiguous() and state.shape == (Hv, Dv, Dk)
    out = torch.empty((Hv, nc, Cn, Dv), dtype=torch.float32, device=U0.device)
    a = GdnCarryArgs()
    a.U0, a.W, a.Qd, a.Kd, a.P, a.gamma, a.state, a.out = _p(U0), _p(W), _p(Qd), _p(Kd), _p(P), _p(gamma), _p(state), _p(out)
    a.Hv, a.nc, a.Dk, a.Dv = Hv, nc, Dk, Dv
    native.check(_lib().tsb_gdn_chunk_carry(C.byref(a), _stream()), "gdn_chunk_carry")
    _count(1)
    return out


def mamba2_recurrent(xbc, dt, dt_bias, A, D, state, cu_q, seq_slots, *, H, P, G, N):
    T = xbc.shape[0]
    check_index("mamba2_recurrent", "state slot", seq_slots, state.shape[0])
    check_index("mamba2_recurrent", "row offset", cu_q, T + 1)
    y = torch.empty((T, H * P), dtype=torch.float32, device=xbc.device)
    a = MambaArgs()
    a.xbc, a.xbc_s = _p(xbc), xbc.stride(0)
    a.dt, a.dt_s, a.dt_f32 = _p(dt), dt.stride(0), int(dt.dtype == torch.float32)
    a.dt_bias, a.A, a.D, a.state = _p(dt_bias), _p(A), _p(D), _p(state)
    a.cu_q, a.seq_slots, a.y, a.y_s = _p(cu_q), _p(seq_slots), _p(y), H * P
    a.H, a.P, a.G, a.N, a.B = H, P, G, N, cu_q.numel() - 1
    native.check(_lib().tsb_mamba2_recurrent(C.byref(a), _stream()), "mamba2_recurrent")
    _count(1)
    return y
