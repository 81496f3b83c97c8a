"""Block codecs for GGUF tensor types, written as vectorised torch ops.

These are the layout oracle: every device kernel that consumes GGUF blocks is tested
against :func:`dequantize`.  They run on any torch device, so the same code quantises a
4-billion-parameter synthetic model on a GPU in seconds and checks a handful of
hand-packed blocks on the CPU.

Parity: TensorSharp.Models/ManagedQuantizedOps.cs:411 (Q8_0), :447-479 + :685 (Q4_K and
its 6-bit scale/min unpacking), :520 (Q6_K), :579-598 + :678 (MXFP4 and its E8M0
half-scale); ExternalProjects/ggml/src/ggml-quants.c for the remaining layouts.
The quantisers are simple min/max fitters (not ggml's iterative search); they emit
valid blocks, which is all a random-weight benchmark needs.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..gguf.constants import GGMLType, block_size, type_size

_MXFP4_VALUES = (0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12)
_IQ4NL_VALUES = (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)


def _as_blocks(raw: torch.Tensor, t: GGMLType) -> torch.Tensor:
    raw = raw.reshape(-1)
    if raw.dtype != torch.uint8:
        raw = raw.view(torch.uint8)
    ts = type_size(t)
    if raw.numel() % ts:
        raise ValueError(f"{raw.numel()} bytes is not a whole number of {t.name} blocks ({ts} B)")
    return raw.view(-1, ts)


def _f16(b: torch.Tensor) -> torch.Tensor:
    """[nb, 2] uint8 -> [nb, 1] float32 (little-endian IEEE half)."""
    return b.contiguous().view(torch.float16).to(torch.float32)


def _scale_min_k4(sc: torch.Tensor):
    """Unpack the 12-byte Q4_K / Q5_K scale field into 8 scales and 8 mins (6 bit each)."""
    sc = sc.to(torch.int32)
    lo_s = sc[:, 0:4] & 63
    lo_m = sc[:, 4:8] & 63
    hi_s = (sc[:, 8:12] & 0xF) | ((sc[:, 0:4] >> 6) << 4)
    hi_m = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
    return torch.cat([lo_s, hi_s], 1).float(), torch.cat([lo_m, hi_m], 1).float()


def e8m0_to_fp32_half(e: torch.Tensor) -> torch.Tensor:
    """ggml's MXFP4 block scale: 2**(e-127) / 2, including the two denormal encodings."""
    e = e.to(torch.int32)
    bits = torch.where(e < 2, torch.tensor(0x00200000, dtype=torch.int32, device=e.device) << e,
                       (e - 1) << 23)
    return bits.view(torch.float32)


def dequantize(raw: torch.Tensor, t: GGMLType, shape: Sequence[int] = None) -> torch.Tensor:
    """Decode raw GGUF blocks to float32.  ``shape`` (row-major) reshapes the result."""
    t = GGMLType(t)
    dev = raw.device
    if t == GGMLType.F32:
        out = raw.reshape(-1).view(torch.uint8).view(torch.float32).clone()
    elif t == GGMLType.F16:
        out = raw.reshape(-1).view(torch.uint8).view(torch.float16).float()
    elif t == GGMLType.BF16:
        out = raw.reshape(-1).view(torch.uint8).view(torch.bfloat16).float()
    elif t in (GGMLType.I8, GGMLType.I16, GGMLType.I32):
        dt = {GGMLType.I8: torch.int8, GGMLType.I16: torch.int16, GGMLType.I32: torch.int32}[t]
        out = raw.reshape(-1).view(torch.uint8).view(dt).float()
    else:
        b = _as_blocks(raw, t)
        if t == GGMLType.Q8_0:
            out = _f16(b[:, 0:2]) * b[:, 2:34].view(torch.int8).float()
        elif t == GGMLType.Q4_0:
            q = b[:, 2:18].to(torch.int32)
            out = _f16(b[:, 0:2]) * (torch.cat([q & 0xF, q >> 4], 1) - 8).float()
        elif t == GGMLType.Q4_1:
            q = b[:, 4:20].to(torch.int32)
            out = _f16(b[:, 0:2]) * torch.cat([q & 0xF, q >> 4], 1).float() + _f16(b[:, 2:4])
        elif t == GGMLType.IQ4_NL:
            q = b[:, 2:18].to(torch.int64)
            tab = torch.tensor(_IQ4NL_VALUES, dtype=torch.float32, device=dev)
            out = _f16(b[:, 0:2]) * tab[torch.cat([q & 0xF, q >> 4], 1)]
        elif t in (GGMLType.Q5_0, GGMLType.Q5_1):
            o = 2 if t == GGMLType.Q5_0 else 4
            qh = b[:, o:o + 4].contiguous().view(torch.int32)          # [nb, 1]
            q = b[:, o + 4:o + 20].to(torch.int32)
            j = torch.arange(16, device=dev, dtype=torch.int32)
            x0 = (q & 0xF) | (((qh >> j) & 1) << 4)
            x1 = (q >> 4) | (((qh >> (j + 16)) & 1) << 4)
            x = torch.cat([x0, x1], 1).float()
            if t == GGMLType.Q5_0:
                out = _f16(b[:, 0:2]) * (x - 16.0)
            else:
                out = _f16(b[:, 0:2]) * x + _f16(b[:, 2:4])
        elif t == GGMLType.MXFP4:
            d = e8m0_to_fp32_half(b[:, 0:1])
            q = b[:, 1:17].to(torch.int64)
            tab = torch.tensor(_MXFP4_VALUES, dtype=torch.float32, device=dev)
            out = d * tab[torch.cat([q & 0xF, q >> 4], 1)]
        elif t == GGMLType.Q4_K:
            d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
            sc, mn = _scale_min_k4(b[:, 4:16])
            q = b[:, 16:144].to(torch.int32).view(-1, 4, 32)
            vals = torch.stack([q & 0xF, q >> 4], 2).reshape(-1, 8, 32).float()
            out = (d * sc).unsqueeze(2) * vals - (dmin * mn).unsqueeze(2)
        elif t == GGMLType.Q5_K:
            d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
            sc, mn = _scale_min_k4(b[:, 4:16])
            qh = b[:, 16:48].to(torch.int32)                            # [nb, 32]
            q = b[:, 48:176].to(torch.int32).view(-1, 4, 32)
            c = torch.arange(4, device=dev, dtype=torch.int32).view(1, 4, 1)
            hb_lo = (qh.unsqueeze(1) >> (2 * c)) & 1
            hb_hi = (qh.unsqueeze(1) >> (2 * c + 1)) & 1
            lo = (q & 0xF) + (hb_lo << 4)
            hi = (q >> 4) + (hb_hi << 4)
            vals = torch.stack([lo, hi], 2).reshape(-1, 8, 32).float()
            out = (d * sc).unsqueeze(2) * vals - (dmin * mn).unsqueeze(2)
        elif t == GGMLType.Q6_K:
            ql = b[:, 0:128].to(torch.int32).view(-1, 2, 64)
            qh = b[:, 128:192].to(torch.int32).view(-1, 2, 32)
            sc = b[:, 192:208].view(torch.int8).float().view(-1, 2, 8)
            d = _f16(b[:, 208:210])
            q1 = (ql[:, :, 0:32] & 0xF) | (((qh >> 0) & 3) << 4)
            q2 = (ql[:, :, 32:64] & 0xF) | (((qh >> 2) & 3) << 4)
            q3 = (ql[:, :, 0:32] >> 4) | (((qh >> 4) & 3) << 4)
            q4 = (ql[:, :, 32:64] >> 4) | (((qh >> 6) & 3) << 4)
            qs = torch.stack([q1, q2, q3, q4], 2).float() - 32.0          # [nb, 2, 4, 32]
            # value l of quarter k uses scale index (l // 16) + 2k
            s = sc.view(-1, 2, 4, 2).repeat_interleave(16, dim=3)        # [nb, 2, 4, 32]
            out = d.view(-1, 1, 1, 1) * s * qs
        elif t == GGMLType.Q2_K:
            scb = b[:, 0:16].to(torch.int32)
            qs = b[:, 16:80].to(torch.int32).view(-1, 2, 1, 32)
            d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
            sh = (2 * torch.arange(4, device=dev, dtype=torch.int32)).view(1, 1, 4, 1)
            q = ((qs >> sh) & 3).float().reshape(-1, 16, 16)             # 16 sub-blocks of 16
            dl = d * (scb & 0xF).float()
            ml = dmin * (scb >> 4).float()
            out = dl.unsqueeze(2) * q - ml.unsqueeze(2)
        else:
            raise NotImplementedError(f"dequantize: unsupported GGML type {t.name}")
    out = out.reshape(-1)
    return out.reshape(tuple(shape)) if shape is not None else out


# ---------------------------------------------------------------------------- quantisers
def _to_f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8).view(x.shape[0], -1)


def _pack_scale_min_k4(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`_scale_min_k4`: 8 + 8 six-bit integers -> 12 bytes."""
    sc, mn = sc.to(torch.int32), mn.to(torch.int32)
    out = torch.empty(sc.shape[0], 12, dtype=torch.int32, device=sc.device)
    out[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    return out.to(torch.uint8)


def quantize(x: torch.Tensor, t: GGMLType) -> torch.Tensor:
    """Encode a float tensor (last dim a multiple of the block size) into raw GGUF
    blocks; returns a flat ``uint8`` tensor on ``x``'s device."""
    t = GGMLType(t)
    if t == GGMLType.F32:
        return x.float().contiguous().view(-1).view(torch.uint8)
    if t == GGMLType.F16:
        return x.to(torch.float16).contiguous().view(-1).view(torch.uint8)
    if t == GGMLType.BF16:
        return x.to(torch.bfloat16).contiguous().view(-1).view(torch.uint8)
    bs = block_size(t)
    if x.shape[-1] % bs:
        raise ValueError(f"last dim {x.shape[-1]} is not a multiple of the {t.name} block size {bs}")
    xb = x.float().reshape(-1, bs)
    nb = xb.shape[0]
    dev = xb.device
    if t == GGMLType.Q8_0:
        d = xb.abs().amax(1, keepdim=True) / 127.0
        d16 = d.to(torch.float16)
        inv = torch.where(d16 > 0, 1.0 / d16.float(), torch.zeros_like(d))
        q = torch.round(xb * inv).clamp(-127, 127).to(torch.int8)
        out = torch.cat([_to_f16_bytes(d16), q.view(torch.uint8)], 1)
    elif t == GGMLType.Q4_0:
        idx = xb.abs().argmax(1, keepdim=True)
        mx = xb.gather(1, idx)
        d = mx / -8.0
        d16 = d.to(torch.float16)
        inv = torch.where(d16 != 0, 1.0 / d16.float(), torch.zeros_like(d))
        q = torch.clamp(torch.floor(xb * inv + 8.5), 0, 15).to(torch.int32)
        out = torch.cat([_to_f16_bytes(d16), (q[:, :16] | (q[:, 16:] << 4)).to(torch.uint8)], 1)
    elif t == GGMLType.MXFP4:
        amax = xb.abs().amax(1, keepdim=True).clamp_min(1e-30)
        e = (torch.floor(torch.log2(amax)) - 2 + 127).clamp(1, 254).to(torch.int32)
        scale = torch.exp2((e - 127).float())                           # value = scale * e2m1
        y = xb / scale
        grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device=dev)
        code = (y.abs().unsqueeze(2) - grid).abs().argmin(2).to(torch.int32)
        code = code | ((y < 0).to(torch.int32) << 3)
        out = torch.cat([e.to(torch.uint8), (code[:, :16] | (code[:, 16:] << 4)).to(torch.uint8)], 1)
    elif t in (GGMLType.Q4_K, GGMLType.Q5_K):
        nmax = 15.0 if t == GGMLType.Q4_K else 31.0
        sb = xb.view(nb, 8, 32)
        mn = torch.clamp(sb.amin(2), max=0.0)
        mx = sb.amax(2)
        scale_f = (mx - mn) / nmax
        min_f = -mn
        d = (scale_f.amax(1, keepdim=True) / 63.0).to(torch.float16)
        dm = (min_f.amax(1, keepdim=True) / 63.0).to(torch.float16)
        invd = torch.where(d > 0, 1.0 / d.float(), torch.zeros_like(d, dtype=torch.float32))
        invm = torch.where(dm > 0, 1.0 / dm.float(), torch.zeros_like(dm, dtype=torch.float32))
        sc = torch.round(scale_f * invd).clamp(0, 63)
        mq = torch.round(min_f * invm).clamp(0, 63)
        eff = d.float() * sc
        inv_eff = torch.where(eff > 0, 1.0 / eff, torch.zeros_like(eff))
        q = torch.round((sb + (dm.float() * mq).unsqueeze(2)) * inv_eff.unsqueeze(2)).clamp(0, nmax)
        q = q.to(torch.int32).view(nb, 4, 2, 32)
        qs = ((q[:, :, 0] & 0xF) | ((q[:, :, 1] & 0xF) << 4)).to(torch.uint8).view(nb, 128)
        parts = [_to_f16_bytes(d), _to_f16_bytes(dm), _pack_scale_min_k4(sc, mq)]
        if t == GGMLType.Q5_K:
            c = torch.arange(4, device=dev, dtype=torch.int32).view(1, 4, 1)
            qh = (((q[:, :, 0] >> 4) & 1) << (2 * c)) | (((q[:, :, 1] >> 4) & 1) << (2 * c + 1))
            parts.append(qh.sum(1).to(torch.uint8))
        parts.append(qs)
        out = torch.cat(parts, 1)
    elif t == GGMLType.Q6_K:
        sb = xb.view(nb, 16, 16)
        idx = sb.abs().argmax(2, keepdim=True)
        mxv = sb.gather(2, idx).squeeze(2)
        scale_f = mxv / -32.0
        d = (scale_f.abs().amax(1, keepdim=True) / 127.0).to(torch.float16)
        invd = torch.where(d > 0, 1.0 / d.float(), torch.zeros_like(d, dtype=torch.float32))
        sc = torch.round(scale_f * invd).clamp(-128, 127)
        eff = d.float() * sc
        inv_eff = torch.where(eff != 0, 1.0 / eff, torch.zeros_like(eff))
        q = (torch.round(sb * inv_eff.unsqueeze(2)).clamp(-32, 31) + 32).to(torch.int32)
        # sub-block s = 8*half + 2*quarter + (l // 16); value index l within a quarter of 32
        q = q.view(nb, 2, 4, 32)
        ql0 = (q[:, :, 0] & 0xF) | ((q[:, :, 2] & 0xF) << 4)
        ql1 = (q[:, :, 1] & 0xF) | ((q[:, :, 3] & 0xF) << 4)
        ql = torch.cat([ql0, ql1], 2).reshape(nb, 128)
        qh = ((q[:, :, 0] >> 4) | ((q[:, :, 1] >> 4) << 2) | ((q[:, :, 2] >> 4) << 4)
              | ((q[:, :, 3] >> 4) << 6)).reshape(nb, 64)
        sc_b = sc.view(nb, 2, 4, 2).reshape(nb, 16).to(torch.int8).view(torch.uint8)
        out = torch.cat([ql.to(torch.uint8), qh.to(torch.uint8), sc_b, _to_f16_bytes(d)], 1)
    else:
        raise NotImplementedError(f"quantize: unsupported GGML type {t.name}")
    assert out.shape[1] == type_size(t), (out.shape, t)
    return out.contiguous().view(-1)
