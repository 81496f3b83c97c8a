"""Mistral 3: GQA decoder with YaRN-scaled, adjacent-pair (GPT-J style) RoPE, a
position-dependent query scale and SwiGLU FFN.

Parity: TensorSharp.Models/Models/Mistral3/Mistral3Model.cs - YaRN keys :61-75, RoPE through
RoPEEx mode 0 (adjacent pairs) with ext_factor / beta_fast / beta_slow and attn_factor
1 / (0.1 ln(scale) + 1) when both mscale keys are set (:545-567), query scale
1 + beta * ln(1 + floor(pos / original_context)) (:573-599).
"""
from __future__ import annotations

import math

import torch

from ..ops.functional import Batch, RopeSpec
from ..ops.kernels import yarn_corr_dims
from .base import register_architecture
from .qwen3 import Qwen3Model


@register_architecture("mistral3", "mistral")
class Mistral3Model(Qwen3Model):
    def parse_config(self) -> None:
        g, a, c = self.gguf, self.arch, self.cfg
        self.rope_dim = g.get_int(f"{a}.rope.dimension_count", c.head_dim) or c.head_dim
        self.rope_type = g.get_str(f"{a}.rope.scaling.type", "") or ""
        self.q_beta = g.get_float(f"{a}.attention.temperature_scale", g.get_float(f"{a}.rope.scaling_beta", 0.1))
        self.orig_ctx = g.get_int(f"{a}.rope.scaling.original_context_length", 0)
        self.ext_factor = g.get_float(f"{a}.rope.scaling.extrapolation_factor", 1.0)
        self.beta_fast = g.get_float(f"{a}.rope.scaling.yarn_beta_fast", g.get_float(f"{a}.rope.scaling.beta_fast", 32.0))
        self.beta_slow = g.get_float(f"{a}.rope.scaling.yarn_beta_slow", g.get_float(f"{a}.rope.scaling.beta_slow", 1.0))
        self.mscale = g.get_float(f"{a}.rope.scaling.mscale", 0.0)
        self.mscale_all = g.get_float(f"{a}.rope.scaling.mscale_all_dim", 0.0)

    def load_weights(self) -> None:
        super().load_weights()
        c = self.cfg
        yarn = self.rope_type == "yarn" and self.orig_ctx > 0
        attn_factor = 1.0 / (0.1 * math.log(c.rope_scale) + 1.0) if (self.mscale and self.mscale_all) else 1.0
        lo, hi = yarn_corr_dims(self.rope_dim, self.orig_ctx, c.rope_base, self.beta_fast, self.beta_slow) if yarn else (0.0, 0.0)
        self.rope = RopeSpec(rot_dim=self.rope_dim, theta_base=c.rope_base, mode=1, freq_scale=1.0 / c.rope_scale,
                             ext_factor=self.ext_factor if yarn else 0.0, attn_factor=attn_factor, corr_lo=lo, corr_hi=hi)

    def q_post_scale(self, qr: torch.Tensor, batch: Batch) -> torch.Tensor:
        """q *= 1 + beta * ln(1 + floor(pos / original_context)); identity below the original context."""
        if self.orig_ctx <= 0 or batch.max_kv_len <= self.orig_ctx:
            return qr
        s = 1.0 + self.q_beta * torch.log1p(torch.floor(batch.positions.float() / self.orig_ctx))
        return (qr.float() * s.view(-1, 1, 1)).to(qr.dtype)
