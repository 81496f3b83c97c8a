"""The op set the model graphs are written against.

Every function has exactly two implementations: the sm_100a kernels (tensors on a CUDA
device) and the fp32 PyTorch restatement in :mod:`reference` (tensors on the CPU), which
is both the CPU backend and the numerical oracle.  On a CUDA device there is no fallback:
a missing kernel library raises.

Data conventions
  * the residual stream ``h`` is float32 ``[T, D]`` (T = packed tokens of all sequences)
  * :class:`Act` carries a normalised activation as bf16 and / or as int8 groups of 32
    with ``(scale, sum)`` pairs, which is what the quantised GEMV consumes
  * the KV cache is paged: ``k_cache / v_cache`` are ``[n_slots, Hkv, Dh]``
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

from ..quant.qweight import QuantWeight
from . import reference as ref

GEMV_MAX_M = 16   # "small batch": token count up to which the models take their decode-style paths (int8 activations, mailbox exchanges)
# Dense projections of 9 to 16 rows go to the tensor-core GEMM on the bf16 weight copy all the same: measured on the
# Qwen3-4B shape at batch 16, 10.95 ms per step with the weight-streaming GEMVs against 8.15 ms (TSB_GEMV_MAX_M moves it)
DENSE_GEMV_MAX_M = min(GEMV_MAX_M, int(os.environ.get("TSB_GEMV_MAX_M", "8")))


@dataclass
class Act:
    """A (normalised) activation in the forms the linear kernels consume."""
    b: Optional[torch.Tensor] = None      # [T, K] bf16 (CUDA) or f32 (CPU)
    q: Optional[torch.Tensor] = None      # [T, K] int8
    ds: Optional[torch.Tensor] = None     # [T, K/32, 2] f32 (scale, sum)

    @property
    def T(self) -> int:
        return (self.b if self.b is not None else self.q).shape[0]


@dataclass
class RopeSpec:
    rot_dim: int
    theta_base: float
    mode: int = 0                 # 0 NeoX, 1 adjacent pairs
    freq_scale: float = 1.0
    ext_factor: float = 0.0
    attn_factor: float = 1.0
    corr_lo: float = 0.0
    corr_hi: float = 0.0
    freq_factors: Optional[torch.Tensor] = None


@dataclass
class Batch:
    """Packed batch metadata (all int tensors live on the compute device)."""
    tokens: torch.Tensor          # [T] int32
    positions: torch.Tensor       # [T] int32
    slots: torch.Tensor           # [T] int64 flat KV slot per token
    cu_q: torch.Tensor            # [B+1] int32
    kv_lens: torch.Tensor         # [B] int32 (cache length after this step)
    block_table: torch.Tensor     # [B, P] int32
    last_idx: torch.Tensor        # [B] int64 index of each sequence's last token in the packed dim
    seq_slots: torch.Tensor       # [B] int64 recurrent-state slot per sequence
    max_q_len: int
    max_kv_len: int
    is_decode: bool               # every sequence contributes exactly one query
    page_size: int
    # host copies for the CPU path and for planning
    h_cu_q: Tuple[int, ...] = ()
    h_kv_lens: Tuple[int, ...] = ()
    cache: dict = field(default_factory=dict)   # per-forward memo (RoPE tables); cleared by the step runner
    # Sliding-window layers that keep a ring of pages (runtime/paged_kv.py): their own slot per token and their own block
    # table (logical page -> physical page of the ring).  None when the pool keeps every page of every layer.
    slots_w: Optional[torch.Tensor] = None
    block_table_w: Optional[torch.Tensor] = None

    def windowed(self) -> "Batch":
        """The view of this batch that a sliding-window layer uses: the same tokens and lengths with the ring's slots
        and block table in place of the full ones (the batch itself when the pool has no ring)."""
        if self.block_table_w is None:
            return self
        w = self.cache.get("_windowed")
        if w is None or w.slots is not self.slots_w:
            import dataclasses
            w = dataclasses.replace(self, slots=self.slots_w, block_table=self.block_table_w, slots_w=None, block_table_w=None,
                                    cache=self.cache)
            self.cache["_windowed"] = w
        return w

    @property
    def B(self) -> int:
        return self.kv_lens.shape[0]

    @property
    def T(self) -> int:
        return self.tokens.shape[0]


def _k():
    from . import kernels
    return kernels


# --------------------------------------------------------------------------------------------
def embed(w: QuantWeight, ids: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Token embedding lookup with on-the-fly dequantisation -> f32 [T, D]."""
    if w.device.type == "cuda":
        return _k().gather_rows(w, ids.to(torch.int32), scale, torch.float32)
    return w.dequantize()[ids.long()] * scale


def norm(h: torch.Tensor, w: Optional[torch.Tensor], eps: float, *, delta: Optional[torch.Tensor] = None,
         want_q8: bool = False, want_bf16: bool = True, l2: bool = False) -> Act:
    """(h += delta, in place) then RMSNorm (or L2 norm) with optional weight."""
    if h.is_cuda:
        if delta is not None and delta.dtype != torch.bfloat16:
            h.add_(delta)
            delta = None
        yb, _, yq, yds = _k().rmsnorm(h, w, eps, delta=delta, want_bf16=want_bf16, want_q8=want_q8, l2=l2)
        return Act(yb, yq, yds)
    if delta is not None:
        h.add_(delta.float())
    return Act(ref.l2norm(h, eps) if l2 else ref.rmsnorm(h, w, eps))


def norm_add(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, h: torch.Tensor) -> torch.Tensor:
    """Sandwich post-norm: returns h + RMSNorm(x) * w as a new f32 tensor."""
    if x.is_cuda:
        _, yf, _, _ = _k().rmsnorm(x.contiguous(), w, eps, want_bf16=False, add=h)
        return yf
    return h + ref.rmsnorm(x, w, eps)


def as_act(x, w: Optional[QuantWeight] = None) -> Act:
    """Wrap a plain activation tensor (an ``Act`` passes through)."""
    if isinstance(x, Act):
        return x
    if not x.is_cuda:
        return Act(x.float())
    a = Act(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16))
    return a


as_act_of = as_act


def _ensure_q8(a: Act) -> Act:
    if a.q is None:
        a.q, a.ds = _k().quantize_q8(a.b.contiguous())
    return a


FUSED_MAX_M = 4       # rows handled by the GEMV with the in-kernel norm / quantise prologue


def can_fuse(x: torch.Tensor, w: QuantWeight) -> bool:
    """Whether ``linear_fused`` should use the single-kernel path for this input (CUDA, at most
    FUSED_MAX_M rows, row length within the shared-memory staging limit).  Off unless
    TSB_FUSED_GEMV=1: on B200 the in-CTA prologue measured slower than the separate norm /
    quantise launches (Qwen3-4B decode 3.8 ms per step against 2.6 ms), because redoing the
    prologue per CTA costs more L2 traffic and occupancy than the two launches it removes."""
    return (os.environ.get("TSB_FUSED_GEMV", "0") == "1" and x.is_cuda and x.numel() // x.shape[-1] <= FUSED_MAX_M
            and w.K % 32 == 0 and w.K <= 10240 and w.experts == 1)


def linear_fused(x: torch.Tensor, w: QuantWeight, *, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                 do_norm: bool = False, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 out_dtype=torch.float32, act: Optional[str] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(RMSNorm(x) * norm_w @ w^T + bias) + residual`` (the norm only with ``do_norm``) with
    ``x`` the f32 residual stream or a bf16 activation.  One kernel for small batches on CUDA
    (K-1 of the kernel list fused with K-5); the separate norm / linear ops otherwise."""
    if can_fuse(x, w):
        x = x.contiguous()
        kw = {"x_f32": x} if x.dtype == torch.float32 else {"x_bf16": x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)}
        return _k().fused_gemv(w, norm_w=norm_w, eps=eps, do_norm=do_norm, out_dtype=out_dtype, bias=bias,
                               residual=residual, act=act, out=out, **kw)
    T = x.numel() // x.shape[-1]
    a = norm(x, norm_w, eps, want_q8=T <= GEMV_MAX_M) if do_norm else as_act(x)
    y = linear(a, w, bias=bias, residual=residual, out_dtype=out_dtype, act=act)
    if out is not None:
        out.copy_(y)
        return out
    return y


_scratch = {}
_bf16_used = {}          # device index -> bytes of bf16 weight copies held
_bf16_auto = {}          # device index -> default budget


def _bf16_budget(device) -> int:
    """Bytes of spare HBM the prefill path may spend on bf16 copies of quantised weights.
    ``TSB_BF16_WEIGHT_CACHE_GB`` sets it (0 turns the copies off); the default is 35 % of the device's
    memory, at most 64 GB: a B200 holds a 4-bit 20 B-parameter model and its bf16 copy several times over."""
    env = os.environ.get("TSB_BF16_WEIGHT_CACHE_GB")
    if env is not None:
        return int(float(env) * (1 << 30))
    key = torch.device(device).index or 0
    if key not in _bf16_auto:
        _bf16_auto[key] = int(min(64 << 30, 0.35 * torch.cuda.get_device_properties(device).total_memory))
    return _bf16_auto[key]


def _release_bf16(dev_index: int, nbytes: int) -> None:
    _bf16_used[dev_index] = _bf16_used.get(dev_index, 0) - nbytes


def _dequant_scratch(w: QuantWeight, holder: Optional[QuantWeight] = None, slot: int = 0) -> torch.Tensor:
    """bf16 form of ``w`` for the tensor-core GEMM; bf16 weights are used in place.

    A quantised weight is decoded once and the copy is kept with the weight object (with ``holder`` and
    ``slot``: with the expert stack that ``w`` is a view of, so the copy outlives the temporary view) for
    as long as the budget of ``_bf16_budget`` lasts: prefill then reads weights the way a bf16 model would,
    while decode keeps streaming the GGUF blocks.  Past the budget the weight is decoded into a per-device
    scratch that every layer reuses (it stays L2-resident between the decode and the GEMM that follows)."""
    from ..gguf.constants import GGMLType
    if w.ggml_type == GGMLType.BF16:
        return w.planes[0].view(torch.bfloat16).view(w.rows, w.K)
    owner = holder if holder is not None else w
    cache = owner.__dict__.setdefault("_bf16_copies", {})
    hit = cache.get(slot)
    if hit is not None:
        return hit
    need = w.rows * w.K
    dev = w.device.index or 0
    if _bf16_used.get(dev, 0) + 2 * need <= _bf16_budget(w.device):
        import weakref
        out = torch.empty((w.rows, w.K), dtype=torch.bfloat16, device=w.device)
        _k().gather_rows(w, None, 1.0, out=out)
        cache[slot] = out
        _bf16_used[dev] = _bf16_used.get(dev, 0) + 2 * need
        weakref.finalize(out, _release_bf16, dev, 2 * need)
        return out
    key = (w.device.index, )
    buf = _scratch.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(max(need, 32 << 20), dtype=torch.bfloat16, device=w.device)
        _scratch[key] = buf
    out = buf[:need].view(w.rows, w.K)
    _k().gather_rows(w, None, 1.0, out=out)
    return out


def linear(a: Act, w: QuantWeight, *, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
           out_dtype=torch.float32, act: Optional[str] = None) -> torch.Tensor:
    """y = a @ w^T (+ bias) (+ residual), optional GLU over the row halves of ``w``
    (rows [0, N/2) gate, [N/2, N) up).  ``residual`` is added in the output dtype."""
    T = a.T
    if w.device.type != "cuda":
        y = a.b.float() @ w.dequantize().t()
        if bias is not None:
            y = y + bias.float()
        if act is not None:
            half = w.N // 2
            y = ref.glu(act, y[:, :half], y[:, half:]) if act not in ("relu2", "silu") else ref.glu(act, y, None)
        if residual is not None:
            y = y + residual.float()
        return y.to(out_dtype) if out_dtype != torch.float32 else y
    k = _k()
    if T <= DENSE_GEMV_MAX_M or (T <= GEMV_MAX_M and (a.b is None or w.experts != 1 or w.K % 8)):
        if w.uses_q8_activations:
            _ensure_q8(a)
            return k.gemv(w, xq=a.q, xds=a.ds, M=T, out_dtype=out_dtype, bias=bias, residual=residual, act=act)
        return k.gemv(w, xb=a.b.contiguous(), M=T, out_dtype=out_dtype, bias=bias, residual=residual, act=act)
    wb = _dequant_scratch(w)
    if act is None:
        return k.gemm_bf16(wb, a.b, out_dtype=out_dtype, bias=bias, residual=residual)
    y = k.gemm_bf16(wb, a.b, out_dtype=torch.bfloat16, bias=bias)
    half = w.N // 2
    if act in ("relu2", "silu"):
        out, _, _ = k.glu(y, None, act, w.N, w.N, 0, T)
    else:
        out, _, _ = k.glu(y, y[:, half:], act, half, w.N, w.N, T)
    if residual is not None:
        out = out.to(out_dtype) + residual
    return out if out.dtype == out_dtype else out.to(out_dtype)


def linear_multi(a: Act, ws, *, out_dtype=torch.float32):
    """``[a @ w^T for w in ws]`` for matrices that share the input.  Decode-sized CUDA batches run them
    as one launch (the separate Q / K / V projections of files whose tensors differ in quantisation
    type); anything else is the plain sequence of ``linear`` calls."""
    ws = list(ws)
    T = a.T
    if (ws[0].device.type == "cuda" and T <= DENSE_GEMV_MAX_M and 2 <= len(ws) <= 3 and all(w.experts == 1 and w.K == ws[0].K for w in ws)
            and len({w.uses_q8_activations for w in ws}) == 1):
        if ws[0].uses_q8_activations:
            _ensure_q8(a)
            y = _k().gemv_multi(ws, xq=a.q, xds=a.ds, M=T, out_dtype=out_dtype)
        else:
            y = _k().gemv_multi(ws, xb=a.b.contiguous(), M=T, out_dtype=out_dtype)
        outs, o = [], 0
        for w in ws:
            outs.append(y[:, o:o + w.N])
            o += w.N
        return outs
    return [linear(a, w, out_dtype=out_dtype) for w in ws]


def glu(act: str, gate: torch.Tensor, up: Optional[torch.Tensor]) -> torch.Tensor:
    """Standalone gated activation on two [T, F] tensors (row-strided views allowed)."""
    if not gate.is_cuda:
        return ref.glu(act, gate, up)
    T, F = gate.shape
    if up is not None and up.dtype != gate.dtype:      # the kernel reads both operands with one element type
        up = up.to(gate.dtype)
    out, _, _ = _k().glu(gate, up, act, F, gate.stride(0), up.stride(0) if up is not None else 0, T)
    return out


def qkv_rope_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, Hq: int, Hkv: int, Dh: int,
                   batch: Batch, k_cache: torch.Tensor, v_cache: torch.Tensor, rope: Optional[RopeSpec],
                   qn: Optional[torch.Tensor] = None, kn: Optional[torch.Tensor] = None, v_norm: bool = False,
                   eps: float = 1e-6, q_scale: float = 1.0, write_kv: bool = True) -> torch.Tensor:
    """Per-head norm on Q / K (and optionally V), RoPE on Q / K, write K / V into the paged
    cache at ``batch.slots``; returns the rotated queries ``[T, Hq, Dh]``.
    ``q``, ``k``, ``v`` are ``[T, H*, Dh]`` views (any token / head stride, last dim dense)."""
    T = batch.T
    if q.is_cuda:
        kk = _k()
        rp = kk.RopeParams()
        if rope is not None:
            rp.theta_base, rp.freq_scale, rp.ext_factor = rope.theta_base, rope.freq_scale, rope.ext_factor
            rp.attn_factor, rp.corr_lo, rp.corr_hi = rope.attn_factor, rope.corr_lo, rope.corr_hi
            rp.rot_dim, rp.mode = rope.rot_dim, rope.mode
        else:
            rp.rot_dim, rp.mode, rp.theta_base, rp.freq_scale, rp.attn_factor = 0, 0, 10000.0, 1.0, 1.0
        table = None
        if rope is not None and rope.rot_dim > 0:
            key = ("rope", id(rope))
            table = batch.cache.get(key)
            if table is None:
                table = kk.rope_table(batch.positions, rp, rope.freq_factors)
                batch.cache[key] = table
        q_out = torch.empty((T, Hq, Dh), dtype=torch.bfloat16, device=q.device)
        assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and q.dtype == k.dtype == v.dtype
        slots, kc, vc = batch.slots, k_cache, v_cache
        fp8 = write_kv and is_fp8(k_cache)
        if fp8:
            # 8-bit pages: the kernel leaves the finished K / V rows in dense bf16 staging rows, which one more
            # kernel converts and scatters to their slots
            slots = batch.cache.get("arange_T")
            if slots is None:
                slots = batch.cache["arange_T"] = torch.arange(T, dtype=torch.int64, device=q.device)
            kc = torch.empty((T, Hkv, Dh), dtype=torch.bfloat16, device=q.device)
            vc = torch.empty_like(kc)
        kk.qkv_rope(q=q, k=k, v=v, q_strides=(q.stride(0), q.stride(1)), k_strides=(k.stride(0), k.stride(1)),
                    v_strides=(v.stride(0), v.stride(1)), Hq=Hq, Hkv=Hkv if write_kv else 0, Dh=Dh,
                    pos=batch.positions, slot=slots,
                    q_out=q_out, k_cache=kc, v_cache=vc, qn=qn, kn=kn, v_norm=v_norm, eps=eps, rope=rp,
                    freq_factors=rope.freq_factors if rope is not None else None, q_scale=q_scale,
                    cs_table=table)
        if fp8:
            kk.kv_store_fp8(kc, vc, k_cache, v_cache, batch.slots)
        return q_out
    qf, kf, vf = q.float(), k.float(), v.float()
    if qn is not None:
        qf = ref.rmsnorm(qf, qn, eps)
    if kn is not None:
        kf = ref.rmsnorm(kf, kn, eps)
    if v_norm:
        vf = ref.rmsnorm(vf, None, eps)
    if rope is not None and rope.rot_dim > 0:
        cos, sin = ref.rope_cos_sin(batch.positions, rope.rot_dim, rope.theta_base, rope.freq_scale,
                                    rope.ext_factor, rope.attn_factor, rope.corr_lo, rope.corr_hi,
                                    rope.freq_factors)
        qf = ref.apply_rope(qf, cos, sin, rope.rot_dim, rope.mode)
        kf = ref.apply_rope(kf, cos, sin, rope.rot_dim, rope.mode)
    if write_kv:
        kv_scatter(k_cache, batch.slots, kf)
        kv_scatter(v_cache, batch.slots, vf)
    return qf * q_scale


FP8 = torch.float8_e4m3fn


def is_fp8(cache: torch.Tensor) -> bool:
    return cache.dtype == FP8


def kv_scatter(cache: torch.Tensor, slots: torch.Tensor, rows: torch.Tensor) -> None:
    """``cache[slots] = rows`` in the cache's element type (8-bit caches are indexed through their bytes)."""
    if is_fp8(cache):
        cache.view(torch.uint8)[slots] = rows.to(FP8).view(torch.uint8)
    else:
        cache[slots] = rows.to(cache.dtype)


def kv_gather(cache: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``cache[idx]``; rows of an 8-bit cache come back as float32."""
    if is_fp8(cache):
        return cache.view(torch.uint8)[idx].view(FP8).float()
    return cache[idx]


def fp8_prefill_view(k_cache: torch.Tensor, v_cache: torch.Tensor, batch: Batch):
    """The cache rows of the batch's sequences as dense bf16 tensors, laid out as one page per sequence, with the
    block table that goes with them: (K, V, table, page size).  Converting a prompt's keys once per layer costs their
    bytes three times over; the flash kernel then reads them once per query tile as it does bf16 pages."""
    ps, B = batch.page_size, batch.B
    L = (batch.max_kv_len + 63) // 64 * 64
    key = ("fp8_idx", id(batch.block_table))
    cached = batch.cache.get(key)
    if cached is None:
        j = torch.arange(L, device=k_cache.device)
        width = batch.block_table.shape[1]
        pages = batch.block_table.long()[:, (j // ps).clamp_max(width - 1)]           # [B, L]; rows past a sequence's end are never read
        idx = (pages * ps + (j % ps)[None, :]).reshape(-1).contiguous()
        table = torch.arange(B, dtype=torch.int32, device=k_cache.device).view(B, 1)
        cached = batch.cache[key] = (idx, table)
    idx, table = cached
    kd, vd = _k().kv_load_fp8(k_cache, v_cache, idx)
    return kd, vd, table, L


def decode_split_len(batch: Batch, splits: int, window: int) -> int:
    """Positions per split fixed on the host from the reserved maximum length (0 with a sliding window, whose
    start depends on the actual length): the kernel then knows its range before it has read the length."""
    if window:
        return 0
    return ((batch.max_kv_len + splits - 1) // splits + 31) & ~31


def decode_splits(batch: Batch, Hkv: int, window: int) -> int:
    """Split-KV factor for decode attention: enough CTAs to cover the GPU's 148 SMs."""
    span = batch.max_kv_len if not window else min(batch.max_kv_len, window)
    # one sequence: about two CTAs per SM; batches: up to eight (a CTA is 128 threads and latency-bound, and with 16
    # sequences two splits per (sequence, KV head) left the kernel at a fifth of the memory rate)
    want = max(1, (148 * (2 if batch.B == 1 else 8)) // max(1, batch.B * Hkv))
    per = int(os.environ.get("TSB_ATTN_SPLIT_LEN", "128"))
    n = int(max(1, min(want, (span + per - 1) // per, 64)))
    # TSB_ATTN_CLUSTER=1: 8 or 16 splits are merged inside the attention kernel by a thread-block cluster (no combine
    # launch), so take those counts when the natural one is close (measured slower than the combine launch: off by default)
    if os.environ.get("TSB_ATTN_CLUSTER", "0") not in ("", "0"):
        if want >= 16 and 13 <= n <= 20:
            return 16
        if want >= 8 and 7 <= n <= 10:
            return 8
    return n


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: Batch, *, scale: float,
              Hq: int, Hkv: int, Dh: int, window: int = 0, sinks: Optional[torch.Tensor] = None,
              softcap: float = 0.0, as_act: bool = False):
    """Causal attention of the packed queries against the paged cache -> [T, Hq * Dh].  ``as_act`` returns an
    ``Act``; on the CUDA decode path it already carries the int8 form written by the combine kernel, so
    the quantised projection that follows needs no quantise launch."""
    T = q.shape[0]
    if as_act:
        if q.is_cuda and batch.is_decode and Dh % 32 == 0:
            sp = decode_splits(batch, Hkv, window)
            out, oq, ods = _k().attn_decode(q, k_cache, v_cache, batch.block_table, batch.kv_lens, scale=scale, Hq=Hq, Hkv=Hkv,
                                            Dh=Dh, page_size=batch.page_size, splits=sp, split_len=decode_split_len(batch, sp, window),
                                            sinks=sinks, softcap=softcap, window=window, want_q8=True)
            return Act(out.view(T, Hq * Dh), oq, ods)
        return as_act_of(attention(q, k_cache, v_cache, batch, scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh, window=window, sinks=sinks,
                                   softcap=softcap))
    if q.is_cuda:
        kk = _k()
        if batch.is_decode:
            sp = decode_splits(batch, Hkv, window)
            out = kk.attn_decode(q, k_cache, v_cache, batch.block_table, batch.kv_lens, scale=scale, Hq=Hq, Hkv=Hkv,
                                 Dh=Dh, page_size=batch.page_size, splits=sp, split_len=decode_split_len(batch, sp, window),
                                 sinks=sinks, softcap=softcap, window=window)
        else:
            table, ps = batch.block_table, batch.page_size
            if is_fp8(k_cache):
                k_cache, v_cache, table, ps = fp8_prefill_view(k_cache, v_cache, batch)
            out = kk.attn_prefill(q, k_cache, v_cache, table, batch.kv_lens, batch.cu_q, batch.max_q_len,
                                  scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=ps, sinks=sinks,
                                  softcap=softcap, window=window)
        return out.view(T, Hq * Dh)
    outs = []
    ps = batch.page_size
    for b in range(batch.B):
        q0, q1 = batch.h_cu_q[b], batch.h_cu_q[b + 1]
        L = batch.h_kv_lens[b]
        pages = batch.block_table[b, :(L + ps - 1) // ps].long()
        idx = (pages.unsqueeze(1) * ps + torch.arange(ps)).reshape(-1)[:L]
        kb, vb = kv_gather(k_cache, idx), kv_gather(v_cache, idx)
        outs.append(ref.attention(q[q0:q1], kb, vb, batch.positions[q0:q1], scale=scale, window=window, sinks=sinks,
                                  softcap=softcap))
    return torch.cat(outs, 0).reshape(T, Hq * Dh)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    if logits.is_cuda:
        return _k().argmax(logits.float().contiguous())
    return logits.argmax(-1).to(torch.int32)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return torch.tanh(x / cap) * cap if cap and cap > 0 else x


# --------------------------------------------------------------------------------------------
# Mixture of experts
# --------------------------------------------------------------------------------------------
MOE_TILE_MAX_PAIRS = int(os.environ.get("TSB_MOE_TILE_MAX_PAIRS", "1024"))


def route_topk_softmax(logits: torch.Tensor, k: int):
    """Top-k on the router logits, then softmax over the selected k (GPT-OSS, Qwen3.5 decode;
    GptOssModel.cs:814-865).  Equivalent to softmax over all -> top-k -> renormalise."""
    if logits.is_cuda and logits.dtype == torch.float32 and logits.shape[-1] <= 1024 and k <= 16:
        return _k().moe_route(logits.contiguous(), k, mode=0)
    vals, ids = torch.topk(logits.float(), k, dim=-1)
    return ids.to(torch.int32), torch.softmax(vals, -1)


def route_sigmoid(logits: torch.Tensor, k: int, bias: Optional[torch.Tensor], normalize: bool, scale: float):
    """Nemotron-H router: selection on sigmoid(logits) + bias, weights are the unbiased
    sigmoid values, optionally normalised (floor 6.1e-5) and scaled (NemotronModel.cs:822-856)."""
    if logits.is_cuda and logits.dtype == torch.float32 and logits.shape[-1] <= 1024 and k <= 16:
        return _k().moe_route(logits.contiguous(), k, mode=1, sel_bias=bias.float().contiguous() if bias is not None else None,
                              normalize=normalize, scale=scale)
    p = torch.sigmoid(logits.float())
    sel = p + bias.float() if bias is not None else p
    _, ids = torch.topk(sel, k, dim=-1)
    w = p.gather(-1, ids)
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(6.103515625e-5)
    return ids.to(torch.int32), w * scale


def moe_experts(a: Act, ids: torch.Tensor, weights: torch.Tensor, gate_up: QuantWeight, down: QuantWeight, *,
                act: str, gate_up_bias: Optional[torch.Tensor] = None, down_bias: Optional[torch.Tensor] = None,
                expert_offset: int = 0, down_scale: Optional[torch.Tensor] = None, push=None) -> Optional[torch.Tensor]:
    """sum_k weights[t, k] * down_e(act(gate_up_e(x_t)))  with e = ids[t, k]  -> f32 [T, D].

    ``gate_up`` / ``down`` are expert stacks; when they hold only experts
    ``[expert_offset, expert_offset + E_local)`` (expert parallelism) the other selections are
    skipped and the caller sums the partial results over ranks.  For non-gated activations
    (relu2) ``gate_up`` is the plain up projection.  ``push`` (a ``TpExchange``; small CUDA batches
    only) makes the down projection store its weighted slot rows straight into every rank's
    mailbox - the expert-parallel combine happens in the consumer of the exchange, which adds
    ``k`` parts per source (``reduce_norm(parts=k)``), and nothing is returned."""
    T, k = ids.shape
    D = down.N
    E_local = gate_up.experts
    glu_act = act not in ("relu2", "silu")
    F_out = gate_up.N // 2 if glu_act else gate_up.N
    dev = ids.device
    local = ids - expert_offset
    if expert_offset != 0 or E_local != int(1e9):
        local = torch.where((local >= 0) & (local < E_local), local, torch.full_like(local, -1))
    if dev.type == "cuda" and T * k <= 4 * GEMV_MAX_M:
        kk = _k()
        flat = local.reshape(-1).contiguous()
        if gate_up.uses_q8_activations:
            _ensure_q8(a)
            gu = torch.zeros((T * k, F_out), dtype=torch.bfloat16, device=dev)
            kk.gemv(gate_up, xq=a.q, xds=a.ds, M=1, ids=flat, x_div=k, act=act if glu_act or act == "relu2" else None,
                    bias=gate_up_bias, out=gu)
        else:
            gu = torch.zeros((T * k, F_out), dtype=torch.bfloat16, device=dev)
            kk.gemv(gate_up, xb=a.b.contiguous(), M=1, ids=flat, x_div=k,
                    act=act if glu_act or act == "relu2" else None, bias=gate_up_bias, out=gu)
        if act == "silu":
            gu, _, _ = kk.glu(gu, None, "silu", F_out, F_out, 0, T * k)
        w = weights.reshape(-1).float().contiguous()
        if down_scale is not None:
            w = w * down_scale[ids.reshape(-1).long()]
        pk = dict(push=push.struct.data_ptr()) if push is not None else dict(out=torch.zeros((T * k, D), dtype=torch.float32, device=dev))
        if down.uses_q8_activations:
            gq, gds = kk.quantize_q8(gu)
            y = kk.gemv(down, xq=gq, xds=gds, M=1, ids=flat, x_div=1, bias=down_bias, row_scale=w, **pk)
        else:
            y = kk.gemv(down, xb=gu, M=1, ids=flat, x_div=1, bias=down_bias, row_scale=w, **pk)
        return y.view(T, k, D).sum(1) if push is None else None
    if push is not None:
        raise ValueError("moe_experts(push=...) needs a CUDA batch of at most 4 * GEMV_MAX_M slots")
    if dev.type == "cuda" and T * k <= MOE_TILE_MAX_PAIRS:
        # medium batches (batched decode): routing stays on the device, each expert's rows are streamed
        # once per tile of 8 pairs; the launch sequence is fixed, so the step can be graph-captured
        kk = _k()
        wts = weights.reshape(-1).float()
        if down_scale is not None:
            wts = wts * down_scale[ids.reshape(-1).long()]
        if gate_up.uses_q8_activations:
            _ensure_q8(a)
            return kk.moe_grouped(xq=a.q, xds=a.ds, ids=ids, weights=wts, gate_up=gate_up, down=down, act=act,
                                  gate_up_bias=gate_up_bias, down_bias=down_bias, expert_offset=expert_offset)
        return kk.moe_grouped(xb=a.b.contiguous(), ids=ids, weights=wts, gate_up=gate_up, down=down, act=act,
                              gate_up_bias=gate_up_bias, down_bias=down_bias, expert_offset=expert_offset)
    if dev.type == "cuda" and os.environ.get("TSB_MOE_GROUPED_GEMM", "1") != "0" and gate_up.K % 8 == 0 and down.K % 8 == 0:
        return _moe_grouped_gemm(a, ids, local, weights, gate_up, down, act, gate_up_bias, down_bias, down_scale)
    # per-expert path (CPU oracle, and CUDA with TSB_MOE_GROUPED_GEMM=0): sort the (token, slot) pairs by expert on the
    # host and run each expert on its rows
    out = torch.zeros((T, D), dtype=torch.float32, device=dev)
    flat = local.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount((flat[order] + 1).long(), minlength=E_local + 1).tolist()
    x = a.b
    off = counts[0]                      # skipped (non-local) selections sort first (-1)
    wflat = weights.reshape(-1).float()
    if down_scale is not None:
        wflat = wflat * down_scale[ids.reshape(-1).long()]
    for e in range(E_local):
        n = counts[e + 1]
        if n == 0:
            continue
        rows = order[off:off + n]
        off += n
        tok = torch.div(rows, k, rounding_mode="floor")
        xe = Act(x[tok].contiguous())
        gb = gate_up_bias[e] if gate_up_bias is not None else None
        y1 = linear(xe, gate_up.expert(e), bias=gb, act=act, out_dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
        db = down_bias[e] if down_bias is not None else None
        y2 = linear(as_act(y1), down.expert(e), bias=db, out_dtype=torch.float32)
        out.index_add_(0, tok, y2 * wflat[rows].unsqueeze(1))
    return out


def moe_tile_list(flat: torch.Tensor, n_groups: int, bn: int):
    """Device-side work list of a grouped GEMM.  ``flat`` [P]: group of every row, -1 = skipped.  Returns ``(order,
    tiles)``: ``order`` sorts the rows by group (skipped rows first), ``tiles`` int32 [ceil(P / bn) + n_groups, 3] holds
    (group or -1, first sorted row, end sorted row) per tile of at most ``bn`` rows.  Nothing is read back to the host:
    the list has a fixed upper-bound length and unused entries are marked -1."""
    P = flat.numel()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount((flat + 1).long(), minlength=n_groups + 1)
    starts = torch.cumsum(counts, 0) - counts
    cnt, st = counts[1:], starts[1:]
    per = (cnt + bn - 1) // bn
    cum = torch.cumsum(per, 0)
    n_tiles = (P + bn - 1) // bn + n_groups
    t = torch.arange(n_tiles, device=flat.device)
    e = torch.searchsorted(cum, t, right=True)
    valid = e < n_groups
    ec = e.clamp(max=n_groups - 1)
    first = st[ec] + (t - (cum[ec] - per[ec])) * bn
    tiles = torch.stack([torch.where(valid, e, torch.full_like(e, -1)), first, st[ec] + cnt[ec]], 1).to(torch.int32)
    return order, tiles.contiguous()


def _moe_grouped_gemm(a: Act, ids, local, weights, gate_up: QuantWeight, down: QuantWeight, act, gate_up_bias, down_bias,
                      down_scale) -> torch.Tensor:
    """Large batches (prefill): the (token, slot) pairs are sorted by expert on the device, both projections run as one
    grouped tensor-core GEMM each over a device-built tile list (no host read-back, two GEMM launches whatever the
    number of experts), and the weighted rows are added back to their tokens."""
    kk = _k()
    T, k = ids.shape
    D, E = down.N, gate_up.experts
    P = T * k
    avg = max(1, P // max(1, E))
    bn = 32 if avg <= 32 else 64 if avg <= 64 else 128 if avg <= 128 else 256
    flat = local.reshape(-1)
    order, tiles = moe_tile_list(flat, E, bn)
    tok = torch.div(order, k, rounding_mode="floor")
    x = a.b if a.b.dtype == torch.bfloat16 else a.b.to(torch.bfloat16)
    xs = x[tok].contiguous()                                         # rows in expert order
    glu_act = act not in ("relu2", "silu")
    y1 = kk.gemm_bf16_grouped(_dequant_scratch(gate_up), E, xs, tiles, bn, out_dtype=torch.bfloat16,
                              bias=gate_up_bias.float().contiguous() if gate_up_bias is not None else None)
    if glu_act:
        half = gate_up.N // 2
        h, _, _ = kk.glu(y1, y1[:, half:], act, half, gate_up.N, gate_up.N, P)
    else:
        h, _, _ = kk.glu(y1, None, act, gate_up.N, gate_up.N, 0, P)
    y2 = kk.gemm_bf16_grouped(_dequant_scratch(down), E, h, tiles, bn, out_dtype=torch.float32,
                              bias=down_bias.float().contiguous() if down_bias is not None else None)
    w = weights.reshape(-1).float()
    if down_scale is not None:
        w = w * down_scale[ids.reshape(-1).long()]
    if D % 4 == 0:
        # every token gathers its own k rows (fixed summation order, no atomics): pos = where each pair went
        pos = torch.empty(P, dtype=torch.int32, device=ids.device)
        pos[order] = torch.arange(P, dtype=torch.int32, device=ids.device)
        pos = torch.where(flat >= 0, pos, torch.full_like(pos, -1))          # skipped pairs contribute nothing
        return kk.moe_combine_weighted(y2, pos, w, T, k)
    w = torch.where(flat >= 0, w, torch.zeros_like(w))[order]
    out = torch.zeros((T, D), dtype=torch.float32, device=ids.device)
    out.index_add_(0, tok, y2 * w.unsqueeze(1))
    return out


# --------------------------------------------------------------------------------------------
# Recurrent layers (state tensors are indexed by ``batch.seq_slots``)
# --------------------------------------------------------------------------------------------
def causal_conv1d(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, batch: Batch,
                  act_silu: bool = True) -> torch.Tensor:
    """Depth-wise causal conv over the packed tokens; ``state`` [slots, K-1, C] carries each
    sequence's last K-1 inputs between calls.  Returns f32 [T, C]."""
    if x.is_cuda:
        return _k().causal_conv1d(x, w, bias, state, batch.cu_q, batch.seq_slots, batch.max_q_len, act_silu)
    outs = []
    slots = batch.seq_slots.tolist()
    for b in range(batch.B):
        q0, q1 = batch.h_cu_q[b], batch.h_cu_q[b + 1]
        o, tail = ref.causal_conv1d(x[q0:q1], w, bias, state[slots[b]], act_silu)
        state[slots[b]] = tail
        outs.append(o)
    return torch.cat(outs, 0)


def _gdn_chunk_min() -> int:
    """Prompts of at least this many tokens take the chunked form of the recurrence (the reference's
    GDN_CHUNK_PREFILL_MIN_SEQ_LEN, default 64; GDN_DISABLE_CHUNKED_PREFILL=1 keeps the token-by-token scan)."""
    if os.environ.get("GDN_DISABLE_CHUNKED_PREFILL", "0") not in ("", "0"):
        return 1 << 62
    return max(2, int(os.environ.get("GDN_CHUNK_PREFILL_MIN_SEQ_LEN", "64") or 64))


CUDA_CHUNKED_MIN_TOKENS = 1024


def _use_chunked_scan(batch: Batch, on_cuda: bool, switch: str) -> bool:
    """Whether a recurrent layer runs its chunked form for this batch.  CPU: prompts of ``_gdn_chunk_min()`` tokens or
    more.  CUDA: prompts of ``CUDA_CHUNKED_MIN_TOKENS`` or more (one B200, 2048 tokens: GatedDeltaNet 5.9 ms as a scan,
    3.6 ms chunked; Mamba2 3.3 against 2.9 ms; at 8192 tokens 23.8 / 12.9 and 18.8 / 8.1 ms; at 512 the scan wins);
    ``<switch>=1`` lowers the bar to the CPU's, ``=0`` keeps the scan kernel."""
    if not on_cuda:
        return batch.max_q_len >= _gdn_chunk_min()
    mode = os.environ.get(switch, "")
    if mode == "0":
        return False
    return batch.max_q_len >= (_gdn_chunk_min() if mode == "1" else max(CUDA_CHUNKED_MIN_TOKENS, _gdn_chunk_min()))


def gdn(qkv: torch.Tensor, z: torch.Tensor, beta: torch.Tensor, alpha: torch.Tensor, dt_bias, a_log, norm_w,
        state: torch.Tensor, batch: Batch, *, Hk: int, Hv: int, Dk: int, Dv: int, eps: float) -> torch.Tensor:
    """GatedDeltaNet recurrence over the packed tokens -> gated output [T, Hv*Dv].  Decode steps and short prompts
    run the token-by-token scan (one kernel on CUDA); longer prompts run the chunked form (matrix products over heads x
    chunks; thresholds in :func:`_use_chunked_scan`)."""
    chunked = _use_chunked_scan(batch, qkv.is_cuda, "TSB_GDN_CHUNKED")
    if qkv.is_cuda and not chunked:
        return _k().gdn_recurrent(qkv, z, beta, alpha, dt_bias, a_log, norm_w, state, batch.cu_q, batch.seq_slots,
                                  Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=eps)
    slots = batch.seq_slots.tolist()
    if chunked and qkv.is_cuda and os.environ.get("TSB_GDN_CHUNK_KERNELS", "1") != "0" and _k().gdn_chunked_supported(Dk, Dv) \
            and qkv.dtype == torch.float32 and beta.dtype == alpha.dtype and beta.stride(0) == alpha.stride(0):
        return _k().gdn_chunked(qkv, z, beta, alpha, dt_bias, a_log, norm_w, state, batch.cu_q, list(batch.h_cu_q), slots,
                                Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=eps)
    if chunked:                                 # every sequence of a batch that took this route, short ones included
        carry = None
        if qkv.is_cuda and os.environ.get("TSB_GDN_CARRY_KERNEL", "1") != "0" and _k().gdn_chunk_carry_supported(Dk, Dv, 64):
            carry = _k().gdn_chunk_carry
        out = ref.gdn_chunked_batch(qkv, z, beta, alpha, dt_bias, a_log, norm_w, [state[sl] for sl in slots], list(batch.h_cu_q),
                                    Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=eps, carry=carry)
        return out.to(torch.bfloat16 if qkv.is_cuda else torch.float32)
    outs = []
    for b in range(batch.B):
        q0, q1 = batch.h_cu_q[b], batch.h_cu_q[b + 1]
        outs.append(ref.gdn_recurrent(qkv[q0:q1], z[q0:q1], beta[q0:q1], alpha[q0:q1], dt_bias, a_log, norm_w, state[slots[b]],
                                      Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, eps=eps))
    return torch.cat(outs, 0).to(torch.bfloat16 if qkv.is_cuda else torch.float32)     # the kernel's output types


def mamba2(xbc: torch.Tensor, dt: torch.Tensor, dt_bias, A, D, state: torch.Tensor, batch: Batch, *, H: int, P: int,
           G: int, N: int) -> torch.Tensor:
    """Mamba2 selective scan over the packed tokens -> y f32 [T, H*P] (before gating).  Long prompts take
    the chunked form (thresholds in :func:`_use_chunked_scan`)."""
    chunked = _use_chunked_scan(batch, xbc.is_cuda, "TSB_MAMBA_CHUNKED")
    if xbc.is_cuda and not chunked:
        return _k().mamba2_recurrent(xbc, dt, dt_bias, A, D, state, batch.cu_q, batch.seq_slots, H=H, P=P, G=G, N=N)
    outs = []
    slots = batch.seq_slots.tolist()
    if (chunked and xbc.is_cuda and os.environ.get("TSB_MAMBA_CHUNK_KERNELS", "1") != "0"
            and os.environ.get("TSB_MAMBA_CARRY_KERNEL", "1") != "0" and _k().mamba2_chunked_supported(N, P)
            and _k().gdn_chunk_carry_supported(N, P, 64) and state.dtype == torch.float32 and xbc.dtype == torch.float32
            and batch.B * H <= 65535):
        # the whole batch in two kernels: the chunk-parallel algebra, then the chunk-carry kernel of the delta rule
        return _k().mamba2_chunked(xbc, dt, dt_bias, A, D, state, batch.cu_q, batch.h_cu_q, slots, H=H, P=P, G=G, N=N)
    scan = ref.mamba2_chunked if chunked else ref.mamba2_recurrent
    kw = {}
    if chunked and xbc.is_cuda and os.environ.get("TSB_MAMBA_CARRY_KERNEL", "1") != "0" and _k().gdn_chunk_carry_supported(N, P, 64) \
            and state.dtype == torch.float32:
        kw["carry"] = _k().gdn_chunk_carry          # the state update has the delta rule's shape with nothing to correct
    for b in range(batch.B):
        q0, q1 = batch.h_cu_q[b], batch.h_cu_q[b + 1]
        outs.append(scan(xbc[q0:q1], dt[q0:q1], dt_bias, A, D, state[slots[b]], H=H, P=P, G=G, N=N, **kw))
    return torch.cat(outs, 0)
