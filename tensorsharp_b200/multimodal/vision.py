"""Vision encoders of the multimodal model families, loaded from an ``mmproj`` GGUF.

Parity (tensor names, metadata keys and arithmetic):
  * Gemma 3  - SigLIP-style ViT: conv patch embed + learned positions, LayerNorm blocks with biased
    q/k/v/out and a tanh-GELU MLP whose first layer is stored as ``ffn_down``, post LayerNorm,
    4 x 4 average pool to 256 tokens, RMSNorm, projection (Gemma3VisionEncoder.cs).
  * Gemma 4  - RMSNorm sandwich blocks, per-head q/k RMSNorm, unweighted v norm, 2-D RoPE (theta
    100, x on the first half of a head, y on the second), attention scale 1, QuickGELU-gated MLP,
    optional per-linear input / output clamps, average pool by ``projector_scale_factor``,
    * sqrt(hidden), standardisation, projection, unweighted RMSNorm (Gemma4VisionEncoder.cs).
  * Qwen 3.5 - dynamic resolution: two summed temporal patch kernels, bilinearly interpolated
    learned positions, patches re-ordered into merge x merge blocks, fused qkv, 2-D RoPE with
    interleaved (y, x) bands, post LayerNorm, 2 x 2 merge, two-layer GELU projector
    (Qwen35VisionEncoder.cs).
  * Mistral 3 - Pixtral: conv patch embed, RMSNorm, 2-D RoPE with alternating height / width
    frequencies, SwiGLU blocks, patch merger + two-layer GELU projector (Mistral3VisionEncoder.cs).
    The reference fills its cos / sin table frequency-major but indexes it patch-major; here the
    table is built patch-major, which is what the layout it copies from intends.

All encoders return float32 ``[tokens, projection_dim]`` on the compute device.

On a GPU the two heavy parts of every block run on this package's own kernels (the reference's counterparts are
the fused ``TSGgml_FusedVisionMLP`` / ``TSGgml_FusedVisionAttention`` graphs, Native/ggml_ops_fused.cpp:1490, :1519):
the projections on the tcgen05 GEMM with the bias added in its epilogue, and the bidirectional attention on the flash
prefill kernel, which sees the whole patch sequence as one cache page and is told, through its position override, that
every query stands behind the last key.  Head sizes the kernel has no instance for (72 in the SigLIP towers) are padded
with zero columns, which change neither the scores nor the kept output columns.  ``TSB_VISION_KERNELS=0`` keeps the
encoder on library calls.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as TF

from ..gguf.reader import GGUFFile
from ..quant import codecs


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608 * (x + 0.044715 * x * x * x)))


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y * w if w is not None else y


class VisionEncoderBase:
    PREFIXES: Tuple[str, ...] = ("v.", "mm.")

    def __init__(self, path: str, device="cpu"):
        self.device = torch.device(device)
        self.mat_dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.native = self.device.type == "cuda" and os.environ.get("TSB_VISION_KERNELS", "1") != "0"
        self.w: Dict[str, torch.Tensor] = {}
        self._wk: Dict[str, torch.Tensor] = {}      # weights with the input dimension padded to whole 64-column k-blocks
        with GGUFFile(path) as g:
            self.read_config(g)
            for name, ti in g.tensors.items():
                if not name.startswith(self.PREFIXES):
                    continue
                raw = torch.from_numpy(np.array(g.tensor_bytes_view(name)))
                t = codecs.dequantize(raw, ti.ggml_type, ti.shape).float()
                big = t.dim() >= 2 and t.numel() >= 4096 and not name.endswith(("position_embd.weight",))
                self.w[name] = t.to(self.device, self.mat_dtype if big else torch.float32).contiguous()
        self.clamps: Dict[str, Tuple[float, float, float, float]] = {}
        for name, t in self.w.items():
            for suffix, idx in (("input_min", 0), ("input_max", 1), ("output_min", 2), ("output_max", 3)):
                if name.endswith("." + suffix):
                    key = name[:name.rfind(".")]
                    cur = list(self.clamps.get(key, (-math.inf, math.inf, -math.inf, math.inf)))
                    cur[idx] = float(t.flatten()[0])
                    self.clamps[key] = tuple(cur)

    # ------------------------------------------------------------------ helpers
    def read_config(self, g: GGUFFile) -> None:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        return name in self.w

    def linear(self, x: torch.Tensor, prefix: str, bias: bool = True) -> torch.Tensor:
        """``x @ W^T (+ b)`` with ``W`` stored ``[out, in]``; optional Gemma-4 style clamps."""
        c = self.clamps.get(prefix)
        if c is not None:
            x = x.clamp(c[0], c[1])
        W = self.w[prefix + ".weight"]
        b = self.w.get(prefix + ".bias") if bias else None
        if self.native and x.is_cuda and x.dim() == 2 and W.dtype == torch.bfloat16:
            y = self.gemm(x, prefix + ".weight", W, b)
        else:
            y = (x.to(W.dtype) @ W.t()).float()
            if b is not None:
                y = y + b
        if c is not None:
            y = y.clamp(c[2], c[3])
        return y

    def gemm(self, x: torch.Tensor, name: str, W: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
        """``x [T, K] @ W [N, K]^T + b`` in float32 on the tcgen05 GEMM (bf16 operands, bias in the epilogue)."""
        from ..ops import kernels
        K = W.shape[1]
        Kp = (K + 63) // 64 * 64
        Wp = self._wk.get(name)
        if Wp is None:
            Wp = self._wk[name] = W.contiguous() if Kp == K else TF.pad(W, (0, Kp - K)).contiguous()
        xb = x.to(torch.bfloat16)
        xb = xb.contiguous() if Kp == K else TF.pad(xb, (0, Kp - K))
        if b is not None:
            b = b.float().contiguous()
        return kernels.gemm_bf16(Wp, xb, out_dtype=torch.float32, bias=b)

    def project_x_w(self, x: torch.Tensor, name: str) -> torch.Tensor:
        """``x @ W`` for projector weights stored ``[in, out]`` (``mm.input_projection``)."""
        W = self.w[name]
        if self.native and x.is_cuda and x.dim() == 2 and W.dtype == torch.bfloat16:
            Wt = self._wk.get(name + "^T")
            if Wt is None:
                Wt = self._wk[name + "^T"] = W.t().contiguous()
            return self.gemm(x, name + "^T.k", Wt, None)
        return (x.to(W.dtype) @ W).float()

    def layer_norm(self, x: torch.Tensor, prefix: str, eps: float) -> torch.Tensor:
        return TF.layer_norm(x, (x.shape[-1],), self.w[prefix + ".weight"], self.w.get(prefix + ".bias"), eps)

    def patch_embed(self, pixels: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], P: int) -> torch.Tensor:
        """``pixels`` ``[3, H, W]`` -> ``[gh * gw, hidden]`` in raster order."""
        x = TF.conv2d(pixels.to(self.device, weight.dtype)[None], weight, None, stride=P).float()
        x = x[0].flatten(1).t().contiguous()
        return x + bias if bias is not None else x

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        """``[n, heads, d]`` each -> ``[n, heads * d]``; full bidirectional attention."""
        if self.native and q.is_cuda and q.shape[-1] <= 512:
            return self.flash_attention(q, k, v, scale)
        o = TF.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                            scale=scale)
        return o[0].transpose(0, 1).reshape(q.shape[0], -1)

    @staticmethod
    def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        """The flash prefill kernel as a bidirectional attention: K and V are one cache page of ``n`` slots, and the
        first query's cache position is set to ``n``, so the causal bound of every query lies behind the last key."""
        from ..ops import kernels
        n, H, d = q.shape
        dp = next(s for s in (64, 128, 256, 512) if s >= d)

        def prep(t):
            t = t.to(torch.bfloat16)
            return (TF.pad(t, (0, dp - d)) if dp != d else t).contiguous()
        dev = q.device
        meta = torch.tensor([0, n, n, n, 0], dtype=torch.int32, device=dev)     # cu_q | cache length | first position | page
        o = kernels.attn_prefill(prep(q), prep(k), prep(v), meta[4:5].view(1, 1), meta[2:3], meta[0:2], n, scale=float(scale),
                                 Hq=H, Hkv=H, Dh=dp, page_size=n, q_pos0=meta[3:4])
        return o[..., :d].float().reshape(n, H * d)

    @staticmethod
    def avg_pool_grid(x: torch.Tensor, gh: int, gw: int, k: int) -> torch.Tensor:
        """Average non-overlapping ``k x k`` windows of the ``[gh * gw, d]`` raster grid."""
        d = x.shape[1]
        g = x.view(gh, gw, d)[:gh // k * k, :gw // k * k]
        return g.view(gh // k, k, gw // k, k, d).mean(dim=(1, 3)).reshape(-1, d)


# ---------------------------------------------------------------------------------------------
class Gemma3VisionEncoder(VisionEncoderBase):
    def read_config(self, g):
        self.image_size = g.get_int("clip.vision.image_size", 896)
        self.patch_size = g.get_int("clip.vision.patch_size", 14)
        self.hidden = g.get_int("clip.vision.embedding_length", 1152)
        self.heads = g.get_int("clip.vision.attention.head_count", 16)
        self.blocks = g.get_int("clip.vision.block_count", 27)
        self.eps = g.get_float("clip.vision.attention.layer_norm_epsilon", 1e-6)
        self.projection_dim = g.get_int("clip.vision.projection_dim", 2560)
        self.tokens_per_image = 256

    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        side = self.image_size // self.patch_size
        n, dh = side * side, self.hidden // self.heads
        x = self.patch_embed(pixels, self.w["v.patch_embd.weight"], self.w.get("v.patch_embd.bias"), self.patch_size)
        x = x + self.w["v.position_embd.weight"][:n].float()
        for i in range(self.blocks):
            p = f"v.blk.{i}"
            a = self.layer_norm(x, p + ".ln1", self.eps)
            q = self.linear(a, p + ".attn_q").view(n, self.heads, dh)
            k = self.linear(a, p + ".attn_k").view(n, self.heads, dh)
            v = self.linear(a, p + ".attn_v").view(n, self.heads, dh)
            x = x + self.linear(self.attention(q, k, v, dh ** -0.5), p + ".attn_out")
            m = self.layer_norm(x, p + ".ln2", self.eps)
            x = x + self.linear(gelu_tanh(self.linear(m, p + ".ffn_down")), p + ".ffn_up")   # fc1 is stored as ffn_down
        x = self.layer_norm(x, "v.post_ln", self.eps)
        k = side // int(math.sqrt(self.tokens_per_image))
        pooled = self.avg_pool_grid(x, side, side, k)
        return self.project_x_w(rms_norm(pooled, self.w["mm.soft_emb_norm.weight"], self.eps), "mm.input_projection.weight")


# ---------------------------------------------------------------------------------------------
class Gemma4VisionEncoder(VisionEncoderBase):
    def read_config(self, g):
        self.hidden = g.get_int("clip.vision.embedding_length", 768)
        self.heads = g.get_int("clip.vision.attention.head_count", 12)
        self.blocks = g.get_int("clip.vision.block_count", 16)
        self.eps = g.get_float("clip.vision.attention.layer_norm_epsilon", 1e-6)
        self.projection_dim = g.get_int("clip.vision.projection_dim", 2560)
        self.patch_size = g.get_int("clip.vision.patch_size", 16)
        self.n_merge = g.get_int("clip.vision.projector_scale_factor", 0) or 3
        self.rope_theta = 100.0

    def rope_tables(self, gw: int, gh: int, dh: int):
        quarter = dh // 4
        inv = 1.0 / (self.rope_theta ** (2.0 * torch.arange(quarter, dtype=torch.float64) / (dh // 2)))
        p = torch.arange(gw * gh)
        px, py = (p % gw), (p // gw)
        ax, ay = px.double()[:, None] * inv, py.double()[:, None] * inv
        f = lambda t: t.float().to(self.device)   # noqa: E731
        return px.to(self.device), py.to(self.device), f(ax.cos()), f(ax.sin()), f(ay.cos()), f(ay.sin())

    @staticmethod
    def rope_2d(x: torch.Tensor, cx, sx, cy, sy) -> torch.Tensor:
        """``x`` ``[n, heads, d]``: the first half of a head rotates with the x position, the second
        half with the y position, each as (j, j + quarter) pairs."""
        n, H, d = x.shape
        q = d // 4
        xa, xb, ya, yb = x[..., :q], x[..., q:2 * q], x[..., 2 * q:3 * q], x[..., 3 * q:]
        cx, sx, cy, sy = (t[:, None, :] for t in (cx, sx, cy, sy))
        return torch.cat([xa * cx - xb * sx, xa * sx + xb * cx, ya * cy - yb * sy, ya * sy + yb * cy], dim=-1)

    def encode(self, pixels: torch.Tensor, width: int, height: int) -> torch.Tensor:
        P = self.patch_size
        gw, gh = width // P, height // P
        n, dh = gw * gh, self.hidden // self.heads
        px, py, cx, sx, cy, sy = self.rope_tables(gw, gh, dh)
        x = self.patch_embed(pixels, self.w["v.patch_embd.weight"], self.w.get("v.patch_embd.bias"), P)
        pos = self.w["v.position_embd.weight"].float()                  # [2, max_pos, hidden]: x table, y table
        x = x + pos[0][px] + pos[1][py]
        for i in range(self.blocks):
            p = f"v.blk.{i}"
            a = rms_norm(x, self.w[p + ".ln1.weight"], self.eps)
            q = self.linear(a, p + ".attn_q", bias=False).view(n, self.heads, dh)
            k = self.linear(a, p + ".attn_k", bias=False).view(n, self.heads, dh)
            v = self.linear(a, p + ".attn_v", bias=False).view(n, self.heads, dh)
            q = rms_norm(q, self.w[p + ".attn_q_norm.weight"], self.eps)
            k = rms_norm(k, self.w[p + ".attn_k_norm.weight"], self.eps)
            v = rms_norm(v, None, self.eps)
            q, k = self.rope_2d(q, cx, sx, cy, sy), self.rope_2d(k, cx, sx, cy, sy)
            o = self.linear(self.attention(q, k, v, 1.0), p + ".attn_out", bias=False)
            x1 = rms_norm(o, self.w[p + ".attn_post_norm.weight"], self.eps) + x
            m = rms_norm(x1, self.w[p + ".ln2.weight"], self.eps)
            gate, up = self.linear(m, p + ".ffn_gate", bias=False), self.linear(m, p + ".ffn_up", bias=False)
            d = self.linear(gate * torch.sigmoid(1.702 * gate) * up, p + ".ffn_down", bias=False)
            x = x1 + rms_norm(d, self.w[p + ".ffn_post_norm.weight"], self.eps)
            sc = self.w.get(p + ".out_scale.weight")
            if sc is not None:
                x = x * sc
        pooled = self.avg_pool_grid(x, gh, gw, self.n_merge) * math.sqrt(self.hidden)
        if self.has("v.std_bias") and self.has("v.std_scale"):
            pooled = (pooled - self.w["v.std_bias"]) * self.w["v.std_scale"]
        return rms_norm(self.project_x_w(pooled, "mm.input_projection.weight"), None, self.eps)


# ---------------------------------------------------------------------------------------------
class Qwen35VisionEncoder(VisionEncoderBase):
    def read_config(self, g):
        self.image_size = g.get_int("clip.vision.image_size", 768)
        self.patch_size = g.get_int("clip.vision.patch_size", 16)
        self.hidden = g.get_int("clip.vision.embedding_length", 1152)
        self.heads = g.get_int("clip.vision.attention.head_count", 16)
        self.blocks = g.get_int("clip.vision.block_count", 27)
        self.eps = g.get_float("clip.vision.attention.layer_norm_epsilon", 1e-6)
        self.projection_dim = g.get_int("clip.vision.projection_dim", 4096)
        self.spatial_merge_size = g.get_int("clip.vision.spatial_merge_size", 2)
        self.rope_theta = g.get_float("clip.vision.rope.freq_base", 10000.0)
        self.grid_per_side = self.image_size // self.patch_size

    def position_embedding(self, gh: int, gw: int) -> torch.Tensor:
        """Bilinear interpolation of the learned ``[side * side, hidden]`` table onto a ``gh x gw`` grid."""
        S = self.grid_per_side
        table = self.w["v.position_embd.weight"].float()
        ys = torch.arange(gh, dtype=torch.float32) * ((S - 1) / (gh - 1) if gh > 1 else 0.0)
        xs = torch.arange(gw, dtype=torch.float32) * ((S - 1) / (gw - 1) if gw > 1 else 0.0)
        fy, fx = ys.trunc().long(), xs.trunc().long()
        cy, cx = (fy + 1).clamp_max(S - 1), (fx + 1).clamp_max(S - 1)
        dy, dx = (ys - fy)[:, None, None].to(self.device), (xs - fx)[None, :, None].to(self.device)
        idx = lambda a, b: (a[:, None] * S + b[None, :]).to(self.device)   # noqa: E731
        out = (table[idx(fy, fx)] * (1 - dy) * (1 - dx) + table[idx(fy, cx)] * (1 - dy) * dx +
               table[idx(cy, fx)] * dy * (1 - dx) + table[idx(cy, cx)] * dy * dx)
        return out.view(gh * gw, -1)

    def block_order(self, gh: int, gw: int) -> torch.Tensor:
        """Raster index of every patch in merge-block order (the merge x merge patches that become one
        output token are consecutive)."""
        m = self.spatial_merge_size
        idx = torch.arange(gh * gw).view(gh // m, m, gw // m, m).permute(0, 2, 1, 3)
        return idx.reshape(-1)

    def rope_tables(self, order: torch.Tensor, gw: int, half: int):
        bands = half // 2
        inv = 1.0 / (self.rope_theta ** (2.0 * torch.arange(bands, dtype=torch.float32) / half))
        y, x = (order // gw).float(), (order % gw).float()
        ang = torch.stack([y[:, None] * inv, x[:, None] * inv], dim=-1).view(order.numel(), half)   # (y, x) interleaved
        return ang.cos().to(self.device), ang.sin().to(self.device)

    def encode(self, pixels: torch.Tensor, height: int, width: int) -> torch.Tensor:
        P, m = self.patch_size, self.spatial_merge_size
        gh, gw = height // P, width // P
        n, dh = gh * gw, self.hidden // self.heads
        half = dh // 2
        W = self.w["v.patch_embd.weight"]
        if self.has("v.patch_embd.weight.1"):
            W = W + self.w["v.patch_embd.weight.1"]                     # the two temporal slices see the same still frame
        x = self.patch_embed(pixels, W, self.w.get("v.patch_embd.bias"), P)
        x = x + self.position_embedding(gh, gw)
        order = self.block_order(gh, gw)
        x = x[order.to(self.device)]
        cos, sin = self.rope_tables(order, gw, half)
        cos, sin = cos[:, None, :], sin[:, None, :]

        def rope(t):
            a, b = t[..., :half], t[..., half:]
            return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
        for i in range(self.blocks):
            p = f"v.blk.{i}"
            a = self.layer_norm(x, p + ".ln1", self.eps)
            qkv = self.linear(a, p + ".attn_qkv").view(n, 3, self.heads, dh)
            q, k, v = rope(qkv[:, 0]), rope(qkv[:, 1]), qkv[:, 2]
            x = x + self.linear(self.attention(q, k, v, dh ** -0.5), p + ".attn_out")
            f = self.layer_norm(x, p + ".ln2", self.eps)
            x = x + self.linear(gelu_tanh(self.linear(f, p + ".ffn_up")), p + ".ffn_down")
        x = self.layer_norm(x, "v.post_ln", self.eps)
        merged = x.reshape(n // (m * m), self.hidden * m * m)
        return self.linear(gelu_tanh(self.linear(merged, "mm.0")), "mm.2")


# ---------------------------------------------------------------------------------------------
class Mistral3VisionEncoder(VisionEncoderBase):
    def read_config(self, g):
        def key(name, default, getter=g.get_int):
            v = getter("vision." + name, None)
            return v if v is not None else getter("clip.vision." + name, default)
        self.image_size = key("image_size", 1540)
        self.patch_size = key("patch_size", 14)
        self.hidden = key("embedding_length", 1024)
        self.heads = key("attention.head_count", 16)
        self.head_dim = g.get_int("vision.attention.key_length", None) or self.hidden // self.heads
        self.blocks = key("block_count", 24)
        self.eps = key("attention.layer_norm_epsilon", 1e-5, g.get_float)
        self.rope_base = g.get_float("vision.rope.freq_base", 10000.0)
        self.spatial_merge_size = g.get_int("spatial_merge_size", 2)

    def rope_tables(self, gw: int, gh: int):
        d = self.head_dim
        freqs = d // 2
        i = torch.arange(freqs, dtype=torch.float64)
        inv = 1.0 / (self.rope_base ** (i * 2 / d))
        h = torch.arange(gh, dtype=torch.float64).repeat_interleave(gw)
        w = torch.arange(gw, dtype=torch.float64).repeat(gh)
        ang = torch.cat([h[:, None] * inv[0::2], w[:, None] * inv[1::2]], dim=1)     # even frequencies: rows, odd: columns
        ang = torch.cat([ang, ang], dim=1).float().to(self.device)
        return ang.cos()[:, None, :], ang.sin()[:, None, :]

    def encode(self, pixels: torch.Tensor, width: int, height: int) -> torch.Tensor:
        P, m = self.patch_size, self.spatial_merge_size
        gw, gh = width // P, height // P
        n, dh, half = gw * gh, self.head_dim, self.head_dim // 2
        x = self.patch_embed(pixels, self.w["v.patch_conv.weight"], self.w.get("v.patch_conv.bias"), P)
        x = rms_norm(x, self.w["v.encoder_norm.weight"], self.eps)
        cos, sin = self.rope_tables(gw, gh)

        def rope(t):
            a, b = t[..., :half], t[..., half:]
            return torch.cat([a * cos[..., :half] - b * sin[..., :half], b * cos[..., :half] + a * sin[..., :half]], dim=-1)
        for i in range(self.blocks):
            p = f"v.blk.{i}"
            a = rms_norm(x, self.w[p + ".attn_norm.weight"], self.eps)
            q = rope(self.linear(a, p + ".attn_q", bias=False).view(n, self.heads, dh))
            k = rope(self.linear(a, p + ".attn_k", bias=False).view(n, self.heads, dh))
            v = self.linear(a, p + ".attn_v", bias=False).view(n, self.heads, dh)
            x = x + self.linear(self.attention(q, k, v, dh ** -0.5), p + ".attn_output", bias=False)
            f = rms_norm(x, self.w[p + ".ffn_norm.weight"], self.eps)
            g = self.linear(f, p + ".ffn_gate", bias=False)
            x = x + self.linear(TF.silu(g) * self.linear(f, p + ".ffn_up", bias=False), p + ".ffn_down", bias=False)
        x = rms_norm(x, self.w["mm.norm.weight"], self.eps)
        mh, mw = gh // m, gw // m
        grid = x.view(gh, gw, self.hidden)[:mh * m, :mw * m].view(mh, m, mw, m, self.hidden)
        merged = grid.permute(0, 2, 1, 3, 4).reshape(mh * mw, m * m * self.hidden)     # (sy, sx) order inside a block
        y = self.linear(merged, "mm.patch_merger.merging_layer", bias=False)
        return self.linear(gelu_tanh(self.linear(y, "mm.linear_1", bias=False)), "mm.linear_2", bias=False)


def create_vision_encoder(arch: str, path: str, device="cpu") -> VisionEncoderBase:
    cls = {"gemma3": Gemma3VisionEncoder, "gemma4": Gemma4VisionEncoder, "qwen35": Qwen35VisionEncoder,
           "qwen35moe": Qwen35VisionEncoder, "qwen3next": Qwen35VisionEncoder, "mistral3": Mistral3VisionEncoder}.get(arch)
    if cls is None:
        raise ValueError(f"architecture {arch!r} has no vision encoder")
    return cls(path, device)
