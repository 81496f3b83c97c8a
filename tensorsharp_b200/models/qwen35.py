"""Qwen3.5 / Qwen3-Next: hybrid of GatedDeltaNet linear-attention layers and gated full
attention layers, dense SwiGLU or mixture-of-experts FFN with a sigmoid-gated shared expert.

Parity: TensorSharp.Models/Models/Qwen35/Qwen35Model.cs - layer i is recurrent when
(i+1) % full_attention_interval != 0 (:264-266); metadata keys :232-262; full attention
(:1042-1317): attn_q emits [Q | gate] per head (:1357 DeinterleaveQGate), QK-norm, partial
NeoX RoPE over rope.dimension_count dims, scale 1/sqrt(d), output * sigmoid(gate); MoE
(:1931-2402): softmax -> top-k -> renormalise (== top-k then softmax over the selected),
shared expert scaled by sigmoid(x . ffn_gate_inp_shexp); no KV truncation (:807).
Qwen35Model.GatedDeltaNet.cs - packed input projection [qkv | z | beta | alpha] (:851-858),
causal conv1d + SiLU over the qkv channels (:1500), per-head delta rule (:1449-1490).
With text-only input every M-RoPE section carries the same position, so the multi-section
rotation reduces to plain partial NeoX RoPE, which is what runs here.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import functional as F
from ..ops.functional import Batch, RopeSpec
from ..parallel.dist import even_split, head_split
from ..quant.qweight import QuantWeight
from .base import ModelBase, register_architecture


@register_architecture("qwen35", "qwen35moe", "qwen3next")
class Qwen35Model(ModelBase):
    supports_kv_truncation = False
    supports_pipeline = True

    def parse_config(self) -> None:
        g, a, c = self.gguf, self.arch, self.cfg
        self.d_inner = g.get_int(f"{a}.ssm.inner_size")
        self.d_state = g.get_int(f"{a}.ssm.state_size")
        self.n_group = g.get_int(f"{a}.ssm.group_count")
        self.dt_rank = g.get_int(f"{a}.ssm.time_step_rank")
        self.conv_k = g.get_int(f"{a}.ssm.conv_kernel", 4)
        self.Hv, self.Hk = self.dt_rank, self.n_group
        self.Dv, self.Dk = self.d_inner // max(1, self.Hv), self.d_state
        self.interval = g.get_int(f"{a}.full_attention_interval", 4)
        self.rope_dims = g.get_int(f"{a}.rope.dimension_count", 0) or c.head_dim
        self.n_experts = g.get_int(f"{a}.expert_count", 0)
        self.top_k = g.get_int(f"{a}.expert_used_count", 0)
        self.is_recurrent = [(i + 1) % self.interval != 0 for i in range(c.n_layers)]

    def kv_layer_shapes(self):
        c = self.cfg
        l0, l1 = self.layer_range
        (_, _), (k0, k1) = head_split(c.n_heads, c.n_kv_heads, self.tp_size, self.tp_rank)
        return [None if (self.is_recurrent[l] or not l0 <= l < l1) else (k1 - k0, c.head_dim) for l in range(c.n_layers)]

    def load_weights(self) -> None:
        c = self.cfg
        ep, er = (self.ep_size, self.ep_rank) if self.ep_size > 1 else (self.tp_size, self.tp_rank)
        self.e0, self.e1 = even_split(self.n_experts, ep, er) if self.n_experts else (0, 0)
        self.tok_emb, self.out_norm, self.lm_head = self.stage_tensors()
        self.l0, l1 = self.layer_range
        (self.q0, self.q1), (self.k0, self.k1) = head_split(c.n_heads, c.n_kv_heads, self.tp_size, self.tp_rank)
        self.layers = []
        qkv_dim = 2 * self.Hk * self.Dk + self.Hv * self.Dv
        dev = self.device
        S = max(self.max_seqs, 1)
        for l in range(self.l0, l1):
            p = f"blk.{l}."
            L = {"attn_norm": self.f32(p + "attn_norm.weight"),
                 "post_norm": self.f32(p + "post_attention_norm.weight")}
            if self.is_recurrent[l]:
                parts = [self.qw(p + n) for n in ("attn_qkv.weight", "attn_gate.weight", "ssm_beta.weight",
                                                   "ssm_alpha.weight")]
                if len({w.ggml_type for w in parts}) == 1:
                    L["in_proj"] = QuantWeight.concat_rows(parts, p + "ssm_in_proj")
                else:
                    L["in_parts"] = parts
                L["conv_w"] = self.f32(p + "ssm_conv1d.weight").contiguous()          # [qkvDim, K]
                L["dt_bias"] = self.f32(p + "ssm_dt.bias")
                L["a"] = self.f32(p + "ssm_a")
                L["ssm_norm"] = self.f32(p + "ssm_norm.weight")
                L["ssm_out"] = self.qw(p + "ssm_out.weight")
                L["conv_state"] = torch.zeros((S, self.conv_k - 1, qkv_dim), dtype=torch.float32, device=dev)
                L["delta_state"] = torch.zeros((S, self.Hv, self.Dv, self.Dk), dtype=torch.float32, device=dev)
            else:
                L["wq"], L["wk"], L["wv"] = (self.qw(p + f"attn_{n}.weight") for n in "qkv")
                L["q_norm"] = self.f32(p + "attn_q_norm.weight", optional=True)
                L["k_norm"] = self.f32(p + "attn_k_norm.weight", optional=True)
                L["wo"] = self.qw(p + "attn_output.weight")
                if self.tp_size > 1:
                    # attention heads are dealt to the ranks (a query row holds the head's query and its gate); with fewer
                    # KV heads than ranks a KV head is held by several ranks
                    Dh = c.head_dim
                    L["wq"] = L["wq"].row_slice(self.q0 * 2 * Dh, self.q1 * 2 * Dh)
                    L["wk"], L["wv"] = L["wk"].row_slice(self.k0 * Dh, self.k1 * Dh), L["wv"].row_slice(self.k0 * Dh, self.k1 * Dh)
                    L["wo"] = L["wo"].col_slice(self.q0 * Dh, self.q1 * Dh)
            if self.has(p + "ffn_gate_inp.weight"):
                L["router"] = self.qw(p + "ffn_gate_inp.weight")
                ge, ue, de = (self.qw(p + f"ffn_{n}_exps.weight") for n in ("gate", "up", "down"))
                if self.e1 - self.e0 != self.n_experts:
                    ge, ue, de = (w.expert_range(self.e0, self.e1) for w in (ge, ue, de))
                L["gate_up_exps"] = QuantWeight.concat_rows_per_expert([ge, ue], p + "ffn_gate_up_exps")
                L["down_exps"] = de
                if self.has(p + "ffn_up_shexp.weight"):
                    g, u = self.qw(p + "ffn_gate_shexp.weight"), self.qw(p + "ffn_up_shexp.weight")
                    L["sh_gate_up"] = QuantWeight.concat_rows([g, u]) if g.ggml_type == u.ggml_type else None
                    L["sh_gate"], L["sh_up"] = g, u
                    L["sh_down"] = self.qw(p + "ffn_down_shexp.weight")
                    L["sh_inp"] = self.qw(p + "ffn_gate_inp_shexp.weight", optional=True)
            else:
                g, u = self.qw(p + "ffn_gate.weight"), self.qw(p + "ffn_up.weight")
                L["gate_up"] = QuantWeight.concat_rows([g, u]) if g.ggml_type == u.ggml_type else None
                L["gate"], L["up"] = g, u
                L["down"] = self.qw(p + "ffn_down.weight")
            self.layers.append(L)
        self.rope = RopeSpec(rot_dim=self.rope_dims, theta_base=c.rope_base, mode=0, freq_scale=1.0 / c.rope_scale)

    def recurrent_state_tensors(self) -> list:
        return [L[k] for L in self.layers if "conv_state" in L for k in ("conv_state", "delta_state")]

    def reset_recurrent_state(self, slot: int) -> None:
        for L in self.layers:
            if "conv_state" in L:
                L["conv_state"][slot].zero_()
                L["delta_state"][slot].zero_()

    # ------------------------------------------------------------------ blocks
    def _swiglu(self, a, fused, gate, up, down, mid):
        if fused is not None:
            gu = F.linear(a, fused, act="swiglu", out_dtype=torch.bfloat16)
        else:
            gu = F.glu("swiglu", F.linear(a, gate, out_dtype=mid), F.linear(a, up, out_dtype=mid))
        return F.linear(F.as_act(gu), down, out_dtype=torch.float32)

    def _ffn(self, L, a, mid) -> torch.Tensor:
        if "router" not in L:
            return self._swiglu(a, L["gate_up"], L["gate"], L["up"], L["down"], mid)
        logits = F.linear(a, L["router"], out_dtype=torch.float32)
        ids, w = F.route_topk_softmax(logits, self.top_k)
        y = F.moe_experts(a, ids, w, L["gate_up_exps"], L["down_exps"], act="swiglu", expert_offset=self.e0)
        if self.e1 - self.e0 != self.n_experts and self.comm is not None:
            self.tp_all_reduce(y)
        if "sh_down" in L:
            s = self._swiglu(a, L["sh_gate_up"], L["sh_gate"], L["sh_up"], L["sh_down"], mid)
            if L.get("sh_inp") is not None:
                s = s * torch.sigmoid(F.linear(a, L["sh_inp"], out_dtype=torch.float32))
            y = y + s
        return y

    def _gdn_layer(self, L, a, batch: Batch, mid) -> torch.Tensor:
        T = batch.T
        qkv_dim = 2 * self.Hk * self.Dk + self.Hv * self.Dv
        vdim = self.Hv * self.Dv
        if "in_proj" in L:
            packed = F.linear(a, L["in_proj"], out_dtype=torch.float32)
        else:
            packed = torch.cat([F.linear(a, w, out_dtype=torch.float32) for w in L["in_parts"]], 1)
        qkv = packed[:, :qkv_dim]
        z = packed[:, qkv_dim:qkv_dim + vdim]
        beta = packed[:, qkv_dim + vdim:qkv_dim + vdim + self.Hv]
        alpha = packed[:, qkv_dim + vdim + self.Hv:]
        conv = F.causal_conv1d(qkv, L["conv_w"], None, L["conv_state"], batch, act_silu=True)
        y = F.gdn(conv, z, beta, alpha, L["dt_bias"], L["a"], L["ssm_norm"], L["delta_state"], batch,
                  Hk=self.Hk, Hv=self.Hv, Dk=self.Dk, Dv=self.Dv, eps=self.cfg.eps)
        return F.linear(F.as_act(y), L["ssm_out"], out_dtype=torch.float32)

    def _attn_layer(self, l, L, a, batch: Batch, mid) -> torch.Tensor:
        c = self.cfg
        Hq, Hkv, Dh = self.q1 - self.q0, self.k1 - self.k0, c.head_dim
        T = batch.T
        qg = F.linear(a, L["wq"], out_dtype=mid).view(T, Hq, 2 * Dh)
        k = F.linear(a, L["wk"], out_dtype=mid).view(T, Hkv, Dh)
        v = F.linear(a, L["wv"], out_dtype=mid).view(T, Hkv, Dh)
        q, gate = qg[:, :, :Dh], qg[:, :, Dh:]
        qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[l],
                              v_cache=self.kv.v[l], rope=self.rope, qn=L["q_norm"], kn=L["k_norm"], eps=c.eps)
        o = F.attention(qr, self.kv.k[l], self.kv.v[l], batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh)
        o = F.glu("sigmoid_mul", gate.reshape(T, Hq * Dh).contiguous(), o)
        y = F.linear(F.as_act(o), L["wo"], out_dtype=torch.float32)
        if self.tp_size > 1:
            self.tp_all_reduce(y)
        return y

    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        c = self.cfg
        small = batch.T <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        h = self.stage_input(batch, lambda: self.inject_pending_embeddings(F.embed(self.tok_emb, batch.tokens)))
        for i, L in enumerate(self.layers):
            l = self.l0 + i
            a = F.norm(h, L["attn_norm"], c.eps, want_q8=small)
            y = self._gdn_layer(L, a, batch, mid) if self.is_recurrent[l] else self._attn_layer(l, L, a, batch, mid)
            h = h + y
            a = F.norm(h, L["post_norm"], c.eps, want_q8=small)
            h = h + self._ffn(L, a, mid)
        if self.stage_handoff(h) or not want_logits:
            return None
        last = h[batch.last_idx].contiguous()
        a = F.norm(last, self.out_norm, c.eps, want_q8=True)
        return F.linear(a, self.lm_head, out_dtype=torch.float32)
