"""Block codecs for GGUF tensor types, written as vectorised torch ops.

These are the layout oracle: every device kernel that consumes GGUF blocks is tested
against :func:`dequantize`.  They run on any torch device, so the same code quantises a
4-billion-parameter synthetic model on a GPU in seconds and checks a handful of
hand-packed blocks on the CPU.

Parity: TensorSharp.Models/ManagedQuantizedOps.cs:411 (Q8_0), :447-479 + :685 (Q4_K and
its 6-bit scale/min unpacking), :520 (Q6_K), :579-598 + :678 (MXFP4 and its E8M0
half-scale); ExternalProjects/ggml/src/ggml-quants.c for the remaining layouts (Q2_K, Q3_K, Q5_*, Q8_K, IQ4_NL / IQ4_XS,
the codebook formats IQ2_* / IQ3_* / IQ1_*, the ternary TQ1_0 / TQ2_0).
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


def _dequantize_codebook(b: torch.Tensor, t: GGMLType) -> torch.Tensor:
    """The IQ formats: 256-value blocks of codebook indices (vectors of 8 or 4 magnitudes, ``iq_grids.py``), sign
    fields, and 3- or 4-bit scales per 32 (or 16) values (ggml-quants.c: dequantize_row_iq2_xxs ... dequantize_row_iq1_m)."""
    from . import iq_grids
    dev = b.device
    nb = b.shape[0]
    i32 = lambda x: x.to(torch.int32)
    u16 = lambda x: x.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    u32 = lambda x: x.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    bit8 = torch.arange(8, device=dev, dtype=torch.int32)
    sign_of = lambda byte: 1.0 - 2.0 * ((byte.unsqueeze(-1) >> bit8) & 1).float()          # [..., 8] from a sign byte
    if t == GGMLType.IQ2_XXS:
        d = _f16(b[:, 0:2])
        w = u32(b[:, 2:66]).view(nb, 8, 2)                                # per 32 values: 4 index bytes, then signs + scale
        idx = (w[:, :, 0:1] >> (8 * torch.arange(4, device=dev))) & 0xFF                       # [nb, 8, 4]
        sg = (w[:, :, 1:2] >> (7 * torch.arange(4, device=dev))) & 127
        db = d * (0.5 + (w[:, :, 1] >> 28).float()) * 0.25                                     # [nb, 8]
        vals = iq_grids.grid("iq2xxs").to(dev)[idx] * iq_grids.signs7().to(dev)[sg]            # [nb, 8, 4, 8]
        return db.view(nb, 8, 1, 1) * vals
    if t == GGMLType.IQ2_XS:
        d = _f16(b[:, 0:2])
        q = u16(b[:, 2:66]).to(torch.int64).view(nb, 8, 4)
        sc = i32(b[:, 66:74])
        db = d.unsqueeze(2) * (0.5 + torch.stack([sc & 0xF, sc >> 4], 2).float()) * 0.25       # [nb, 8, 2]
        vals = iq_grids.grid("iq2xs").to(dev)[q & 511] * iq_grids.signs7().to(dev)[q >> 9]
        return db.repeat_interleave(2, dim=2).unsqueeze(3) * vals
    if t == GGMLType.IQ2_S:
        d = _f16(b[:, 0:2])
        lo = i32(b[:, 2:34]).view(nb, 8, 4)
        sg = i32(b[:, 34:66]).view(nb, 8, 4)
        qh = i32(b[:, 66:74]).view(nb, 8, 1)
        sc = i32(b[:, 74:82])
        l = torch.arange(4, device=dev, dtype=torch.int32)
        idx = (lo | ((qh << (8 - 2 * l)) & 0x300)).to(torch.int64)
        db = d.unsqueeze(2) * (0.5 + torch.stack([sc & 0xF, sc >> 4], 2).float()) * 0.25
        vals = iq_grids.grid("iq2s").to(dev)[idx] * sign_of(sg)
        return db.repeat_interleave(2, dim=2).unsqueeze(3) * vals
    if t == GGMLType.IQ3_XXS:
        d = _f16(b[:, 0:2])
        idx = b[:, 2:66].to(torch.int64).view(nb, 8, 4, 2)                 # two 4-value vectors per 8 values
        w = u32(b[:, 66:98]).view(nb, 8, 1)
        sg = (w >> (7 * torch.arange(4, device=dev))) & 127                                    # [nb, 8, 4]
        db = d * (0.5 + (w[:, :, 0] >> 28).float()) * 0.5
        vals = iq_grids.grid("iq3xxs").to(dev)[idx].reshape(nb, 8, 4, 8) * iq_grids.signs7().to(dev)[sg]
        return db.view(nb, 8, 1, 1) * vals
    if t == GGMLType.IQ3_S:
        d = _f16(b[:, 0:2])
        lo = i32(b[:, 2:66]).view(nb, 8, 8)                                # per 32 values: 8 index bytes
        qh = i32(b[:, 66:74]).view(nb, 8, 1)
        sg = i32(b[:, 74:106]).view(nb, 8, 4)
        sc = i32(b[:, 106:110])
        idx = (lo | (((qh >> torch.arange(8, device=dev, dtype=torch.int32)) & 1) << 8)).to(torch.int64)
        db = d.unsqueeze(2) * (1 + 2 * torch.stack([sc & 0xF, sc >> 4], 2)).float()            # [nb, 4, 2] -> per 32
        vals = iq_grids.grid("iq3s").to(dev)[idx].reshape(nb, 8, 4, 8) * sign_of(sg)
        return db.reshape(nb, 8, 1, 1) * vals
    grid1 = iq_grids.grid("iq1s").to(dev)
    if t == GGMLType.IQ1_S:
        d = _f16(b[:, 0:2])
        lo = i32(b[:, 2:34]).view(nb, 8, 4)
        qh = u16(b[:, 34:50]).view(nb, 8, 1)
        idx = (lo | (((qh >> (3 * torch.arange(4, device=dev, dtype=torch.int32))) & 7) << 8)).to(torch.int64)
        dl = d * (2 * ((qh[:, :, 0] >> 12) & 7) + 1).float()
        delta = torch.where((qh & 0x8000) != 0, -0.125, 0.125)                                 # [nb, 8, 1]
        return dl.view(nb, 8, 1, 1) * (grid1[idx] + delta.unsqueeze(3))
    # IQ1_M: the block's half-precision scale is spread over the top nibbles of the four 16-bit scale words
    lo = i32(b[:, 0:32]).view(nb, 8, 4)
    qh = i32(b[:, 32:48]).view(nb, 8, 2).repeat_interleave(2, dim=2)       # byte l // 2 serves vectors l = 0..3
    sc = u16(b[:, 48:56])                                                  # [nb, 4]
    dbits = (sc[:, 0] >> 12) | ((sc[:, 1] >> 8) & 0x00F0) | ((sc[:, 2] >> 4) & 0x0F00) | (sc[:, 3] & 0xF000)
    d = dbits.to(torch.int16).view(torch.float16).float().view(nb, 1, 1)
    odd = (torch.arange(4, device=dev, dtype=torch.int32) % 2).view(1, 1, 4)
    idx = (lo | ((qh << (8 - 4 * odd)) & 0x700)).to(torch.int64)
    delta = torch.where((qh & (0x08 << (4 * odd))) != 0, -0.125, 0.125)
    ib = torch.arange(8, device=dev)
    half = torch.arange(2, device=dev, dtype=torch.int32).view(1, 1, 2)
    s3 = (sc[:, ib // 2].unsqueeze(2) >> (6 * (ib % 2).view(1, 8, 1).to(torch.int32) + 3 * half)) & 7      # [nb, 8, 2]
    dl = d * (2 * s3 + 1).float()
    return dl.repeat_interleave(2, dim=2).unsqueeze(3) * (grid1[idx] + delta.unsqueeze(3))


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
        elif t == GGMLType.Q3_K:
            hm = b[:, 0:32].to(torch.int32)
            qs = b[:, 32:96].to(torch.int32).view(-1, 2, 1, 32)
            scb = b[:, 96:108].to(torch.int32)
            d = _f16(b[:, 108:110])
            j = torch.arange(16, device=dev)
            low = torch.where(j < 8, scb[:, j % 8] & 0xF, scb[:, j % 8] >> 4)
            high = (scb[:, 8 + j % 4] >> (2 * (j // 4))) & 3
            sc = ((low | (high << 4)) - 32).float()                       # 16 six-bit scales, each for 16 values
            sh = (2 * torch.arange(4, device=dev, dtype=torch.int32)).view(1, 1, 4, 1)
            bit = torch.arange(8, device=dev, dtype=torch.int32).view(1, 8, 1)
            q = ((qs >> sh) & 3).reshape(-1, 8, 32)                       # group g = half * 4 + shift index
            hi = (hm.unsqueeze(1) >> bit) & 1                             # bit g of hmask[l]: set = no offset
            vals = (q - 4 * (1 - hi)).float().reshape(-1, 16, 16)
            out = (d * sc).unsqueeze(2) * vals
        elif t == GGMLType.Q8_K:
            d = b[:, 0:4].contiguous().view(torch.float32)
            out = d * b[:, 4:260].view(torch.int8).float()
        elif t == GGMLType.IQ4_XS:
            d = _f16(b[:, 0:2])
            sh = b[:, 2:4].contiguous().view(torch.int16).to(torch.int32) & 0xFFFF          # [nb, 1]
            sl = b[:, 4:8].to(torch.int32)
            ib = torch.arange(8, device=dev)
            ls = ((sl[:, ib // 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)
            q = b[:, 8:136].to(torch.int64).view(-1, 8, 16)
            tab = torch.tensor(_IQ4NL_VALUES, dtype=torch.float32, device=dev)
            out = (d * (ls - 32).float()).unsqueeze(2) * tab[torch.cat([q & 0xF, q >> 4], 2)]
        elif t == GGMLType.TQ2_0:
            qs = b[:, 0:64].to(torch.int32).view(-1, 2, 1, 32)
            sh = (2 * torch.arange(4, device=dev, dtype=torch.int32)).view(1, 1, 4, 1)
            out = _f16(b[:, 64:66]) * (((qs >> sh) & 3) - 1).float().reshape(-1, 256)
        elif t == GGMLType.TQ1_0:
            # five ternary digits per byte (four in the last four bytes), most significant first: digit n of byte q is
            # ((q * 3^n mod 256) * 3) >> 8
            def trits(x, n):
                p3 = torch.tensor([1, 3, 9, 27, 81][:n], device=dev, dtype=torch.int32).view(1, n, 1)
                return ((((x.to(torch.int32).unsqueeze(1) * p3) & 0xFF) * 3) >> 8) - 1
            vals = torch.cat([trits(b[:, 0:32], 5).reshape(-1, 160), trits(b[:, 32:48], 5).reshape(-1, 80),
                              trits(b[:, 48:52], 4).reshape(-1, 16)], 1)
            out = _f16(b[:, 52:54]) * vals.float()
        elif t in (GGMLType.IQ2_XXS, GGMLType.IQ2_XS, GGMLType.IQ2_S, GGMLType.IQ3_XXS, GGMLType.IQ3_S, GGMLType.IQ1_S,
                   GGMLType.IQ1_M):
            out = _dequantize_codebook(b, t)
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
