"""Nemotron-H: every layer is exactly one of Mamba2, attention (no RoPE) or FFN (ReLU^2 dense
or a sigmoid-routed mixture of experts with latent projections and shared experts).

Parity: TensorSharp.Models/Models/Nemotron/NemotronModel.cs - layer type from the per-layer
attention.head_count_kv[] and feed_forward_length[] arrays (:141-178); Mamba2 (:1103-1331):
ssm_in -> [z | xBC | dt], causal conv1d (+bias) + SiLU over xBC, dt = softplus(dt + bias),
dA = exp(dt A), state = state dA + B (x) x dt, y = state C + D x, y *= silu(z), per-group
RMSNorm, ssm_out; attention (:624-740) without positional encoding, scale attention.scale or
1/sqrt(d); dense FFN up -> ReLU^2 -> down (:759-767); MoE (:769-1030): sigmoid router,
selection on sigmoid + exp_probs_b, weights = unbiased sigmoid values (optionally normalised
with floor 6.1e-5) times expert_weights_scale, experts up -> ReLU^2 -> down in the latent
space of ffn_latent_in / ffn_latent_out, plus shared experts on the layer input.
The reference runs Mamba2 on the host token by token; here conv and scan are device kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import functional as F
from ..ops.functional import Batch
from .base import ModelBase, register_architecture


@register_architecture("nemotron_h", "nemotron_h_moe", "nemotronh")
class NemotronHModel(ModelBase):
    supports_kv_truncation = False
    supports_pipeline = True

    def parse_config(self) -> None:
        g, a, c = self.gguf, self.arch, self.cfg
        self.d_conv = g.get_int(f"{a}.ssm.conv_kernel", 4)
        self.d_inner = g.get_int(f"{a}.ssm.inner_size")
        self.d_state = g.get_int(f"{a}.ssm.state_size")
        self.n_head = g.get_int(f"{a}.ssm.time_step_rank")
        self.n_group = g.get_int(f"{a}.ssm.group_count", 1)
        self.head_p = self.d_inner // max(1, self.n_head)
        self.attn_scale = g.get_float(f"{a}.attention.scale", 0.0)
        self.n_experts = g.get_int(f"{a}.expert_count", 0)
        self.top_k = g.get_int(f"{a}.expert_used_count", 0)
        self.w_norm = g.get_bool(f"{a}.expert_weights_norm", False)
        self.w_scale = g.get_float(f"{a}.expert_weights_scale", 1.0)
        kv = g.get_array(f"{a}.attention.head_count_kv") or []
        ff = g.get_array(f"{a}.feed_forward_length") or []
        hc = g.get_array(f"{a}.attention.head_count") or []
        self.layer_type, self.layer_heads, self.layer_kv = [], [], []
        for i in range(c.n_layers):
            k = int(kv[i]) if i < len(kv) else 1
            f = int(ff[i]) if i < len(ff) else 0
            self.layer_type.append("mamba" if (k == 0 and f == 0) else ("attn" if f == 0 else "ffn"))
            self.layer_kv.append(k)
            self.layer_heads.append(int(hc[i]) if i < len(hc) else c.n_heads)
        for i in range(c.n_layers):
            if self.layer_type[i] == "attn":
                c.n_heads, c.n_kv_heads = self.layer_heads[i], self.layer_kv[i]
                break
        if c.n_heads and not self.gguf.get_int(f"{a}.attention.key_length", 0):
            c.head_dim = c.hidden // c.n_heads

    def kv_layer_shapes(self):
        c = self.cfg
        l0, l1 = self.layer_range
        return [(self.layer_kv[l], c.head_dim) if (self.layer_type[l] == "attn" and l0 <= l < l1) else None for l in range(c.n_layers)]

    def load_weights(self) -> None:
        c = self.cfg
        self.tok_emb, self.out_norm, self.lm_head = self.stage_tensors()
        self.l0, l1 = self.layer_range
        # expert parallelism: each rank of the group keeps a contiguous range of the routed experts (everything else is
        # replicated); the experts' contributions are summed over the group
        from ..parallel.dist import even_split
        ep, er = (self.ep_size, self.ep_rank) if self.ep_size > 1 else (self.tp_size, self.tp_rank)
        self.e0, self.e1 = even_split(self.n_experts, ep, er) if self.n_experts else (0, 0)
        self.layers = []
        S = max(self.max_seqs, 1)
        xbc = self.d_inner + 2 * self.n_group * self.d_state
        for l in range(self.l0, l1):
            p = f"blk.{l}."
            L = {"norm": self.f32(p + "attn_norm.weight"), "type": self.layer_type[l]}
            if L["type"] == "mamba":
                L["ssm_in"] = self.qw(p + "ssm_in.weight")
                L["conv_w"] = self.f32(p + "ssm_conv1d.weight").contiguous()
                L["conv_b"] = self.f32(p + "ssm_conv1d.bias", optional=True)
                L["dt_bias"] = self.f32(p + "ssm_dt.bias")
                L["A"] = self.f32(p + "ssm_a").reshape(-1).contiguous()
                d = self.f32(p + "ssm_d", optional=True)
                L["D"] = d.reshape(-1).contiguous() if d is not None else None
                L["ssm_norm"] = self.f32(p + "ssm_norm.weight", optional=True)
                L["ssm_out"] = self.qw(p + "ssm_out.weight")
                L["conv_state"] = torch.zeros((S, self.d_conv - 1, xbc), dtype=torch.float32, device=self.device)
                L["ssm_state"] = torch.zeros((S, self.n_head, self.head_p, self.d_state), dtype=torch.float32,
                                             device=self.device)
            elif L["type"] == "attn":
                L["wq"], L["wk"], L["wv"] = (self.qw(p + f"attn_{n}.weight") for n in "qkv")
                L["wo"] = self.qw(p + "attn_output.weight")
            elif self.n_experts and self.has(p + "ffn_gate_inp.weight"):
                L["router"] = self.qw(p + "ffn_gate_inp.weight")
                b = self.f32(p + "exp_probs_b.bias", optional=True)
                L["router_bias"] = b if b is not None else self.f32(p + "exp_probs_b", optional=True)
                L["up_exps"], L["down_exps"] = self.qw(p + "ffn_up_exps.weight"), self.qw(p + "ffn_down_exps.weight")
                if self.e1 - self.e0 != self.n_experts:
                    L["up_exps"], L["down_exps"] = (w.expert_range(self.e0, self.e1) for w in (L["up_exps"], L["down_exps"]))
                L["latent_in"] = self.qw(p + "ffn_latent_in.weight", optional=True)
                L["latent_out"] = self.qw(p + "ffn_latent_out.weight", optional=True)
                L["sh_up"] = self.qw(p + "ffn_up_shexp.weight", optional=True)
                L["sh_down"] = self.qw(p + "ffn_down_shexp.weight", optional=True)
            else:
                L["up"], L["down"] = self.qw(p + "ffn_up.weight"), self.qw(p + "ffn_down.weight")
            self.layers.append(L)

    def recurrent_state_tensors(self) -> list:
        return [L[k] for L in self.layers if "conv_state" in L for k in ("conv_state", "ssm_state")]

    def reset_recurrent_state(self, slot: int) -> None:
        for L in self.layers:
            if "conv_state" in L:
                L["conv_state"][slot].zero_()
                L["ssm_state"][slot].zero_()

    def _mamba(self, L, a, batch: Batch) -> torch.Tensor:
        di, G, N, H, P = self.d_inner, self.n_group, self.d_state, self.n_head, self.head_p
        proj = F.linear(a, L["ssm_in"], out_dtype=torch.float32)
        z = proj[:, :di]
        xbc = proj[:, di:2 * di + 2 * G * N]
        dt = proj[:, 2 * di + 2 * G * N:]
        conv = F.causal_conv1d(xbc, L["conv_w"], L["conv_b"], L["conv_state"], batch, act_silu=True)
        y = F.mamba2(conv, dt, L["dt_bias"], L["A"], L["D"], L["ssm_state"], batch, H=H, P=P, G=G, N=N)
        y = y * torch.nn.functional.silu(z.float())
        if L["ssm_norm"] is not None:
            yg = y.view(-1, G, di // G)
            yg = yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + self.cfg.eps)
            y = yg.reshape(-1, di) * L["ssm_norm"].reshape(-1)
        return F.linear(F.as_act(y), L["ssm_out"], out_dtype=torch.float32)

    def _attn(self, l, L, a, batch: Batch, mid) -> torch.Tensor:
        c = self.cfg
        Hq, Hkv, Dh = self.layer_heads[l], self.layer_kv[l], c.head_dim
        T = batch.T
        q = F.linear(a, L["wq"], out_dtype=mid).view(T, Hq, Dh)
        k = F.linear(a, L["wk"], out_dtype=mid).view(T, Hkv, Dh)
        v = F.linear(a, L["wv"], out_dtype=mid).view(T, Hkv, Dh)
        qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[l],
                              v_cache=self.kv.v[l], rope=None, eps=c.eps)
        scale = self.attn_scale if self.attn_scale > 0 else Dh ** -0.5
        o = F.attention(qr, self.kv.k[l], self.kv.v[l], batch, scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh)
        return F.linear(F.as_act(o), L["wo"], out_dtype=torch.float32)

    def _ffn(self, L, a, mid) -> torch.Tensor:
        if "router" not in L:
            up = F.linear(a, L["up"], act="relu2", out_dtype=torch.bfloat16 if a.b.is_cuda else torch.float32)
            return F.linear(F.as_act(up), L["down"], out_dtype=torch.float32)
        logits = F.linear(a, L["router"], out_dtype=torch.float32)
        ids, w = F.route_sigmoid(logits, self.top_k, L["router_bias"], self.w_norm, self.w_scale)
        x = a
        if L["latent_in"] is not None:
            x = F.as_act(F.linear(a, L["latent_in"], out_dtype=torch.float32))
        y = F.moe_experts(x, ids, w, L["up_exps"], L["down_exps"], act="relu2", expert_offset=self.e0)
        if self.e1 - self.e0 != self.n_experts and self.comm is not None:
            self.tp_all_reduce(y)
        if L["latent_out"] is not None:
            y = F.linear(F.as_act(y), L["latent_out"], out_dtype=torch.float32)
        if L["sh_up"] is not None:
            s = F.linear(a, L["sh_up"], act="relu2", out_dtype=torch.bfloat16 if a.b.is_cuda else torch.float32)
            y = y + F.linear(F.as_act(s), L["sh_down"], out_dtype=torch.float32)
        return y

    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        c = self.cfg
        small = batch.T <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        h = self.stage_input(batch, lambda: F.embed(self.tok_emb, batch.tokens))
        for i, L in enumerate(self.layers):
            a = F.norm(h, L["norm"], c.eps, want_q8=small)
            if L["type"] == "mamba":
                y = self._mamba(L, a, batch)
            elif L["type"] == "attn":
                y = self._attn(self.l0 + i, L, a, batch, mid)
            else:
                y = self._ffn(L, a, mid)
            h = h + y
        if self.stage_handoff(h) or not want_logits:
            return None
        last = h[batch.last_idx].contiguous()
        a = F.norm(last, self.out_norm, c.eps, want_q8=True)
        return F.linear(a, self.lm_head, out_dtype=torch.float32)
