"""Gemma 4 audio front end: file decoding, log-mel spectrogram and the conformer encoder.

Parity: Gemma4AudioPreprocessor.cs (16 kHz mono, 20 ms frames / 10 ms hop, periodic Hann window
sampled at half-integer points, FFT length 1024, 128 triangular mel filters on the HTK scale from
0 to 8 kHz applied to the magnitude spectrum, floor 1e-3, natural log; frames =
(samples - 321) // 160 :212-238) and Gemma4AudioEncoder.cs (two stride-2 3x3 convolutions with
channel LayerNorm + ReLU, input projection, conformer blocks = half-step FFW, chunked local
attention with relative position logits and a tanh soft cap, light depthwise convolution module,
second half-step FFW, block norm; output projection, unweighted RMSNorm, projection to the text
width).  WAV is decoded here; other containers need an external decoder and raise a clear error.
On a GPU the encoder's projections run on this package's tcgen05 GEMM (bf16 operands, bias in the epilogue);
``TSB_AUDIO_KERNELS=0`` keeps them on library calls.
"""
from __future__ import annotations

import math
import os
import struct
from typing import Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as TF

from ..gguf.reader import GGUFFile
from ..quant import codecs
from .vision import rms_norm

SAMPLE_RATE = 16000
MEL_BINS = 128
FRAME_LENGTH = 320
HOP_LENGTH = 160
FFT_LENGTH = 1024
MEL_FLOOR = 1e-3


# ---------------------------------------------------------------------------- decoding
def resample_linear(x: np.ndarray, src: int, dst: int) -> np.ndarray:
    if src == dst or x.size == 0:
        return x.astype(np.float32)
    n = int(x.size * dst / src)
    pos = np.arange(n, dtype=np.float64) * (src / dst)
    i0 = np.minimum(pos.astype(np.int64), x.size - 1)
    i1 = np.minimum(i0 + 1, x.size - 1)
    f = (pos - i0).astype(np.float32)
    return (x[i0] * (1 - f) + x[i1] * f).astype(np.float32)


def decode_wav(data: bytes) -> np.ndarray:
    """PCM 8/16/24/32-bit or IEEE float WAV -> mono float32 at 16 kHz."""
    if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
        raise ValueError("not a RIFF/WAVE file")
    pos, fmt, pcm = 12, None, None
    while pos + 8 <= len(data):
        cid, size = data[pos:pos + 4], struct.unpack_from("<I", data, pos + 4)[0]
        body = data[pos + 8:pos + 8 + size]
        if cid == b"fmt ":
            fmt = struct.unpack_from("<HHIIHH", body, 0)
        elif cid == b"data":
            pcm = body
        pos += 8 + size + (size & 1)
    if fmt is None or pcm is None:
        raise ValueError("WAV file has no fmt / data chunk")
    tag, channels, rate, _, _, bits = fmt
    if tag == 0xFFFE and len(data) >= 44:          # WAVE_FORMAT_EXTENSIBLE: PCM or float by bit depth
        tag = 3 if bits == 32 and b"\x03\x00\x00\x00" in data[20:64] else 1
    if tag == 3 and bits == 32:
        x = np.frombuffer(pcm, dtype="<f4").astype(np.float32)
    elif tag == 1 and bits == 16:
        x = np.frombuffer(pcm[:len(pcm) // 2 * 2], dtype="<i2").astype(np.float32) / 32768.0
    elif tag == 1 and bits == 8:
        x = (np.frombuffer(pcm, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    elif tag == 1 and bits == 24:
        b = np.frombuffer(pcm[:len(pcm) // 3 * 3], dtype=np.uint8).reshape(-1, 3).astype(np.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = np.where(v >= 1 << 23, v - (1 << 24), v).astype(np.float32) / float(1 << 23)
    elif tag == 1 and bits == 32:
        x = np.frombuffer(pcm[:len(pcm) // 4 * 4], dtype="<i4").astype(np.float32) / float(1 << 31)
    else:
        raise ValueError(f"unsupported WAV encoding: format tag {tag}, {bits} bits")
    if channels > 1:
        x = x[:x.size // channels * channels].reshape(-1, channels).mean(axis=1)
    return resample_linear(x, rate, SAMPLE_RATE)


def decode_audio_file(path: str) -> np.ndarray:
    with open(path, "rb") as f:
        data = f.read()
    if data[:4] == b"RIFF":
        return decode_wav(data)
    raise ValueError(f"{path}: only WAV audio is decoded in this build (MP3 / OGG need an external decoder)")


# ---------------------------------------------------------------------------- mel spectrogram
def hann_window() -> torch.Tensor:
    i = torch.arange(FRAME_LENGTH, dtype=torch.float64)
    return 0.5 - 0.5 * torch.cos(2.0 * math.pi / FRAME_LENGTH * (i + 0.5))


def mel_filter_bank(n_freq: int = FFT_LENGTH // 2 + 1, n_mels: int = MEL_BINS, f_min: float = 0.0, f_max: float = 8000.0,
                    sr: int = SAMPLE_RATE) -> torch.Tensor:
    """``[n_freq, n_mels]`` triangular filters with HTK mel spacing, unnormalised."""
    hz2mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)   # noqa: E731
    pts = torch.linspace(hz2mel(f_min), hz2mel(f_max), n_mels + 2, dtype=torch.float64)
    edges = 700.0 * (10.0 ** (pts / 2595.0) - 1.0)
    fft = torch.arange(n_freq, dtype=torch.float64) * sr / (2.0 * (n_freq - 1))
    left, centre, right = edges[:-2], edges[1:-1], edges[2:]
    f = fft[:, None]
    up = (f - left) / (centre - left)
    down = (right - f) / (right - centre)
    w = torch.where((f >= left) & (f <= centre), up, torch.where((f > centre) & (f <= right), down, torch.zeros_like(up)))
    return w.clamp_min(0).float()


def mel_spectrogram(samples: np.ndarray) -> Tuple[Optional[torch.Tensor], int]:
    """float32 ``[frames, 128]`` log-mel features (or ``(None, 0)`` for a clip shorter than a frame)."""
    n = (len(samples) - (FRAME_LENGTH + 1)) // HOP_LENGTH
    if n <= 0:
        return None, 0
    x = torch.from_numpy(np.asarray(samples, dtype=np.float32)).double()
    idx = torch.arange(n)[:, None] * HOP_LENGTH + torch.arange(FRAME_LENGTH)[None, :]
    frames = x[idx] * hann_window()
    spec = torch.fft.rfft(frames, n=FFT_LENGTH).abs()
    mel = (spec @ mel_filter_bank().double()).clamp_min(MEL_FLOOR).log()
    return mel.float(), n


def audio_token_count(n_samples: int) -> int:
    if n_samples % 128:
        n_samples += 128 - n_samples % 128
    n = (n_samples - (FRAME_LENGTH + 1)) // HOP_LENGTH
    if n <= 0:
        return 0
    t0 = (n + 2 - 3) // 2 + 1
    return (t0 + 2 - 3) // 2 + 1


# ---------------------------------------------------------------------------- conformer encoder
class Gemma4AudioEncoder:
    CHUNK, MAX_PAST, MAX_FUTURE = 12, 12, 0
    LOGIT_CAP, RESIDUAL_WEIGHT, GRAD_CLIP = 50.0, 0.5, 1e10

    def __init__(self, path: str, device="cpu"):
        self.device = torch.device(device)
        self.native = self.device.type == "cuda" and os.environ.get("TSB_AUDIO_KERNELS", "1") != "0"
        self.w: Dict[str, torch.Tensor] = {}
        self._wk: Dict[str, torch.Tensor] = {}
        with GGUFFile(path) as g:
            def key(name, default, getter=g.get_int):
                v = getter("clip.audio." + name, None)
                return v if v is not None else getter("gemma4.audio." + name, default)
            self.hidden = key("embedding_length", 1024)
            self.heads = key("attention.head_count", 8)
            self.layers = key("block_count", 12)
            self.mel_bins = g.get_int("clip.audio.num_mel_bins", 128)
            self.eps = key("attention.layer_norm_epsilon", 1e-6, g.get_float)
            self.projection_dim = g.get_int("clip.audio.projection_dim", 2560)
            for name, ti in g.tensors.items():
                if name.startswith(("a.", "mm.a.")):
                    raw = torch.from_numpy(np.array(g.tensor_bytes_view(name)))
                    self.w[name] = codecs.dequantize(raw, ti.ggml_type, ti.shape).float().to(self.device).contiguous()
        self.head_dim = self.hidden // self.heads
        self.context = self.CHUNK + self.MAX_PAST + self.MAX_FUTURE
        self.ollama_names = "a.blk.0.ln1.weight" in self.w
        self.clamps: Dict[str, Tuple[float, float, float, float]] = {}
        for name, t in self.w.items():
            for suffix, idx in (("input_min", 0), ("input_max", 1), ("output_min", 2), ("output_max", 3)):
                if name.endswith("." + suffix):
                    k = name[:name.rfind(".")]
                    cur = list(self.clamps.get(k, (-math.inf, math.inf, -math.inf, math.inf)))
                    cur[idx] = float(t.flatten()[0])
                    self.clamps[k] = tuple(cur)
        r = torch.arange(self.CHUNK)[:, None]
        c = torch.arange(self.context)[None, :]
        self.causal_valid = ((r <= c) & (c <= r + self.MAX_PAST + self.MAX_FUTURE)).to(self.device)
        self._pos_cache: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ helpers
    def name(self, prefix: str, short: str) -> str:
        if self.ollama_names:
            return {"attn_pre_norm": f"{prefix}.ln1", "block_norm": f"{prefix}.layer_pre_norm",
                    "attn_post_norm": f"{prefix}.ln2", "attn_k_rel": f"{prefix}.linear_pos"}.get(short, f"{prefix}.{short}")
        return f"{prefix}.ln2" if short == "block_norm" else f"{prefix}.{short}"

    def linear(self, x: torch.Tensor, prefix: str) -> torch.Tensor:
        c = self.clamps.get(prefix)
        if c is not None:
            x = x.clamp(c[0], c[1])
        W = self.w[prefix + ".weight"]
        b = self.w.get(prefix + ".bias")
        if self.native and x.is_cuda and W.dim() == 2 and W.numel() >= 4096:
            y = self.gemm(x, prefix, W, b)
        else:
            y = x @ W.t()
            if b is not None:
                y = y + b
        return y.clamp(c[2], c[3]) if c is not None else y

    def gemm(self, x: torch.Tensor, prefix: str, W: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
        """The projection on the tcgen05 GEMM: a bf16 copy of the weight (input dimension padded to whole 64-column
        k-blocks), rows of ``x`` flattened, bias in the epilogue, float32 out."""
        from ..ops import kernels
        K = W.shape[1]
        Kp = (K + 63) // 64 * 64
        Wp = self._wk.get(prefix)
        if Wp is None:
            Wp = self._wk[prefix] = TF.pad(W.to(torch.bfloat16), (0, Kp - K)).contiguous()
        xb = TF.pad(x.reshape(-1, K).to(torch.bfloat16), (0, Kp - K)).contiguous()
        y = kernels.gemm_bf16(Wp, xb, out_dtype=torch.float32, bias=b.float().contiguous() if b is not None else None)
        return y.view(*x.shape[:-1], W.shape[0])

    def norm(self, x: torch.Tensor, weight_name: str) -> torch.Tensor:
        w = self.w.get(weight_name)
        return rms_norm(x, w, self.eps) if w is not None else x

    def conv_block(self, x: torch.Tensor, prefix: str) -> torch.Tensor:
        """``x`` ``[C, T, F]`` -> stride-2 3x3 convolution, LayerNorm over channels, ReLU."""
        y = TF.conv2d(x[None], self.w[prefix + ".weight"], None, stride=2, padding=1)[0]
        nw = self.w.get(prefix + ".norm.weight")
        if nw is not None:
            y = TF.layer_norm(y.permute(1, 2, 0), (y.shape[0],), nw, self.w.get(prefix + ".norm.bias"), self.eps).permute(2, 0, 1)
        return y.relu()

    # ------------------------------------------------------------------ blocks
    def ffw(self, x, p, norm, up, down, post):
        h = self.norm(x.clamp(-self.GRAD_CLIP, self.GRAD_CLIP), f"{p}.{norm}.weight")
        h = self.linear(TF.silu(self.linear(h, f"{p}.{up}")), f"{p}.{down}").clamp(-self.GRAD_CLIP, self.GRAD_CLIP)
        return x + self.norm(h, f"{p}.{post}.weight") * self.RESIDUAL_WEIGHT

    def position_embeddings(self, p: str) -> torch.Tensor:
        """Relative-position key vectors ``[span, heads, head_dim]`` for distances max_past .. -max_future."""
        if p in self._pos_cache:
            return self._pos_cache[p]
        span = self.MAX_PAST + self.MAX_FUTURE + 1
        half = self.hidden // 2
        inc = math.log(10000.0) / max(half - 1, 1)
        rel = (self.MAX_PAST - torch.arange(span, dtype=torch.float64))[:, None]
        ang = rel * torch.exp(-torch.arange(half, dtype=torch.float64) * inc)[None, :]
        emb = torch.cat([ang.sin(), ang.cos()], dim=1).float().to(self.device)
        W = self.w.get(self.name(p, "attn_k_rel") + ".weight")
        if W is not None:
            emb = emb[:, :W.shape[1]] @ W.t()
        out = emb.view(span, self.heads, self.head_dim)
        self._pos_cache[p] = out
        return out

    def attention(self, x: torch.Tensor, p: str) -> torch.Tensor:
        T, H, D, cs, ctx = x.shape[0], self.heads, self.head_dim, self.CHUNK, self.context
        h = self.norm(x.clamp(-self.GRAD_CLIP, self.GRAD_CLIP), self.name(p, "attn_pre_norm") + ".weight")
        q = self.linear(h, p + ".attn_q") * (D ** -0.5 / math.log(2))
        k = self.linear(h, p + ".attn_k") * (math.log(1 + math.e) / math.log(2))
        v = self.linear(h, p + ".attn_v")
        pds = self.w.get(p + ".per_dim_scale.weight")
        q = q.view(T, H, D)
        if pds is not None:
            q = q * pds
        n_chunks = (T + cs - 1) // cs
        padded = n_chunks * cs
        pad_right = self.MAX_FUTURE + cs - 1
        qp = TF.pad(q, (0, 0, 0, 0, 0, padded - T)).view(n_chunks, cs, H, D)
        kp = TF.pad(k.view(T, H, D), (0, 0, 0, 0, self.MAX_PAST, padded - T + pad_right))
        vp = TF.pad(v.view(T, H, D), (0, 0, 0, 0, self.MAX_PAST, padded - T + pad_right))
        win = torch.arange(n_chunks, device=x.device)[:, None] * cs + torch.arange(ctx, device=x.device)[None, :]
        kc, vc = kp[win], vp[win]                                          # [chunks, ctx, H, D]
        logits = torch.einsum("uqhd,uchd->uhqc", qp, kc)
        pos = self.position_embeddings(p)                                  # [span, H, D]
        span = pos.shape[0]
        rel = torch.arange(ctx, device=x.device)[None, :] - torch.arange(cs, device=x.device)[:, None]   # context - query
        ok = (rel >= 0) & (rel < span)
        qpos = torch.einsum("uqhd,shd->uhqs", qp, pos)                     # [chunks, H, cs, span]
        gathered = qpos.gather(3, rel.clamp(0, span - 1)[None, None].expand(n_chunks, H, cs, ctx))
        logits = logits + torch.where(ok[None, None], gathered, torch.zeros_like(gathered))
        logits = torch.tanh(logits / self.LOGIT_CAP) * self.LOGIT_CAP
        time = win - self.MAX_PAST                                          # actual frame of every context slot
        valid = (time >= 0) & (time < T)
        mask = self.causal_valid[None, None] & valid[:, None, None, :]
        logits = logits.masked_fill(~mask, -1e9)
        o = torch.einsum("uhqc,uchd->uqhd", logits.softmax(-1), vc).reshape(padded, H * D)[:T]
        o = self.linear(o, p + ".attn_out").clamp(-self.GRAD_CLIP, self.GRAD_CLIP)
        return x + self.norm(o, self.name(p, "attn_post_norm") + ".weight")

    def light_conv(self, x: torch.Tensor, p: str) -> torch.Tensor:
        h = self.linear(self.norm(x, p + ".conv_norm.weight"), p + ".conv_pw1")
        half = h.shape[1] // 2
        g = h[:, :half] * torch.sigmoid(h[:, half:])
        dw = self.w.get(p + ".conv_dw.weight")
        if dw is not None:                                                  # causal depthwise convolution, [channels, taps]
            k = dw.shape[1]
            g = TF.conv1d(TF.pad(g.t()[None], (k - 1, 0)), dw[:, None, :], groups=half)[0].t()
        g = TF.silu(self.norm(g.clamp(-self.GRAD_CLIP, self.GRAD_CLIP), p + ".norm_conv.weight"))
        return x + self.linear(g, p + ".conv_pw2")

    def block(self, x: torch.Tensor, i: int) -> torch.Tensor:
        p = f"a.blk.{i}"
        x = self.ffw(x, p, "ffn_norm", "ffn_up", "ffn_down", "ffn_post_norm")
        x = self.attention(x, p)
        x = self.light_conv(x, p)
        x = self.ffw(x, p, "ffn_norm_1", "ffn_up_1", "ffn_down_1", "ffn_post_norm_1")
        return self.norm(x.clamp(-self.GRAD_CLIP, self.GRAD_CLIP), self.name(p, "block_norm") + ".weight")

    # ------------------------------------------------------------------ encode
    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        """``mel`` ``[frames, mel_bins]`` -> ``[tokens, projection_dim]`` (a quarter of the frames)."""
        x = mel.to(self.device, torch.float32)[None]                        # [1, T, F]
        x = self.conv_block(self.conv_block(x, "a.conv1d.0"), "a.conv1d.1")  # [C, T/4, F/4]
        C, T, Fq = x.shape
        h = x.permute(1, 2, 0).reshape(T, Fq * C)                            # feature index = c + f * C
        for nm in ("a.input_projection", "a.pre_encode.out"):
            if nm + ".weight" in self.w:
                h = self.linear(h, nm)
                break
        for i in range(self.layers):
            h = self.block(h, i)
        if "a.output_proj.weight" in self.w:
            h = self.linear(h, "a.output_proj")
        if "mm.a.fc.weight" in self.w:
            h = self.linear(h, "mm.a.fc")
        h = rms_norm(h, None, self.eps)
        if "mm.a.input_projection.weight" in self.w:
            h = self.linear(h, "mm.a.input_projection")
        return h
