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

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

from ..quant.qweight import QuantWeight
from . import reference as ref

GEMV_MAX_M = 16   # token count up to which the weight-streaming GEMV beats dequant + tensor-core GEMM


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


def as_act(x: torch.Tensor, w: Optional[QuantWeight] = None) -> Act:
    """Wrap a plain activation tensor; quantises to q8 on CUDA when the weight needs it."""
    if not x.is_cuda:
        return Act(x.float())
    a = Act(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16))
    return a


def _ensure_q8(a: Act) -> Act:
    if a.q is None:
        a.q, a.ds = _k().quantize_q8(a.b.contiguous())
    return a


_scratch = {}


def _dequant_scratch(w: QuantWeight) -> torch.Tensor:
    """bf16 copy of ``w`` for the tensor-core GEMM.  Quantised weights are decoded into a
    per-device scratch that is reused by every layer (it stays L2-resident between the
    decode and the GEMM that follows); bf16 weights are used in place."""
    from ..gguf.constants import GGMLType
    if w.ggml_type == GGMLType.BF16:
        return w.planes[0].view(torch.bfloat16).view(w.rows, w.K)
    key = (w.device.index, )
    need = w.rows * w.K
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
    if T <= GEMV_MAX_M:
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


def glu(act: str, gate: torch.Tensor, up: Optional[torch.Tensor]) -> torch.Tensor:
    """Standalone gated activation on two [T, F] tensors (row-strided views allowed)."""
    if not gate.is_cuda:
        return ref.glu(act, gate, up)
    T, F = gate.shape
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
        kk.qkv_rope(q=q, k=k, v=v, q_strides=(q.stride(0), q.stride(1)), k_strides=(k.stride(0), k.stride(1)),
                    v_strides=(v.stride(0), v.stride(1)), Hq=Hq, Hkv=Hkv if write_kv else 0, Dh=Dh,
                    pos=batch.positions, slot=batch.slots,
                    q_out=q_out, k_cache=k_cache, v_cache=v_cache, qn=qn, kn=kn, v_norm=v_norm, eps=eps, rope=rp,
                    freq_factors=rope.freq_factors if rope is not None else None, q_scale=q_scale,
                    cs_table=table)
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
        k_cache[batch.slots] = kf.to(k_cache.dtype)
        v_cache[batch.slots] = vf.to(v_cache.dtype)
    return qf * q_scale


def decode_splits(batch: Batch, Hkv: int, window: int) -> int:
    """Split-KV factor for decode attention: enough CTAs to cover the GPU's 148 SMs."""
    span = batch.max_kv_len if not window else min(batch.max_kv_len, window)
    want = max(1, (148 * 2) // max(1, batch.B * Hkv))
    return int(max(1, min(want, (span + 127) // 128, 64)))


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: Batch, *, scale: float,
              Hq: int, Hkv: int, Dh: int, window: int = 0, sinks: Optional[torch.Tensor] = None,
              softcap: float = 0.0) -> torch.Tensor:
    """Causal attention of the packed queries against the paged cache -> [T, Hq * Dh]."""
    T = q.shape[0]
    if q.is_cuda:
        kk = _k()
        G = Hq // Hkv
        if batch.is_decode and G in (1, 2, 4, 8):
            out = kk.attn_decode(q, k_cache, v_cache, batch.block_table, batch.kv_lens, scale=scale, Hq=Hq, Hkv=Hkv,
                                 Dh=Dh, page_size=batch.page_size, splits=decode_splits(batch, Hkv, window),
                                 sinks=sinks, softcap=softcap, window=window)
        else:
            out = kk.attn_prefill(q, k_cache, v_cache, batch.block_table, batch.kv_lens, batch.cu_q, batch.max_q_len,
                                  scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh, page_size=batch.page_size, sinks=sinks,
                                  softcap=softcap, window=window)
        return out.view(T, Hq * Dh)
    outs = []
    ps = batch.page_size
    for b in range(batch.B):
        q0, q1 = batch.h_cu_q[b], batch.h_cu_q[b + 1]
        L = batch.h_kv_lens[b]
        pages = batch.block_table[b, :(L + ps - 1) // ps].long()
        idx = (pages.unsqueeze(1) * ps + torch.arange(ps)).reshape(-1)[:L]
        kb, vb = k_cache[idx], v_cache[idx]
        outs.append(ref.attention(q[q0:q1], kb, vb, batch.positions[q0:q1], scale=scale, window=window, sinks=sinks,
                                  softcap=softcap))
    return torch.cat(outs, 0).reshape(T, Hq * Dh)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    if logits.is_cuda:
        return _k().argmax(logits.float().contiguous())
    return logits.argmax(-1).to(torch.int32)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return torch.tanh(x / cap) * cap if cap and cap > 0 else x
