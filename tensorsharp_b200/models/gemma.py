"""Gemma 3 and Gemma 4 decoders.

Gemma 3 (TensorSharp.Models/Models/Gemma3/Gemma3Model.cs): layer l is global when
(l+1) % 6 == 0 (:94), other layers use a sliding window (default 1024); two RoPE bases (local
for sliding layers, global / rope scale for global layers; the scale is forced to 8 for the
34-layer model, :67); QK RMSNorm; query scale 1/sqrt(key_length); sandwich norms
(attn_norm, post_attention_norm, ffn_norm, post_ffw_norm, :280-311); GeGLU; embeddings
times sqrt(hidden); final logit soft-cap.

Gemma 4 (Models/Gemma4/Gemma4Model.cs): per-layer pattern from
attention.sliding_window_pattern (:136), different head dims for sliding (key_length_swa) and
global (key_length) layers (:141-142), per-type KV head counts (:152-170), attention scale 1.0
(:1941), V heads RMS-normalised without weights, NeoX RoPE with the local base on sliding
layers and base / rope_freqs.weight over the partial rotary dims on global layers (:329-353),
the last shared_kv_layers layers reuse the cache of the nearest earlier layer of the same type
(:242-263), optional MoE branch added to the dense MLP with its own norms (:1398-1426) and
router = unweighted RMSNorm * 1/sqrt(hidden) * ffn_gate_inp.scale -> linear -> softmax ->
top-k -> renormalise, per-expert output scale (:1574-1649), per-layer embeddings (:1255-1352,
injected :1446-1461), per-layer output scalar, logit soft-cap (:755).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..ops import functional as F
from ..ops import reference as ref
from ..ops.functional import Batch, RopeSpec
from ..parallel.dist import block_split, head_split
from ..gguf.constants import block_size
from ..quant.qweight import QuantWeight
from .base import ModelBase, register_architecture


class _GemmaBase(ModelBase):
    glu_act = "geglu"
    supports_context_parallel = True

    # per-layer geometry, filled by parse_config
    def kv_window_layers(self):
        return {l: self.window for l in range(self.cfg.n_layers) if self.is_local(l)}

    def is_local(self, l: int) -> bool:
        raise NotImplementedError

    def head_dim_of(self, l: int) -> int:
        return self.cfg.head_dim

    def kv_heads_of(self, l: int) -> int:
        return self.cfg.n_kv_heads

    def kv_layer_shapes(self):
        l0, l1 = self.layer_range
        return [(self.kv_heads_of(l) // self.tp_size, self.head_dim_of(l)) if l0 <= l < l1 else None
                for l in range(self.cfg.n_layers)]

    def _load_common_layer(self, l: int) -> Dict:
        c = self.cfg
        tp, r = self.tp_size, self.tp_rank
        p = f"blk.{l}."
        Dh, Hkv_full = self.head_dim_of(l), self.kv_heads_of(l)
        (q0, q1), (k0, k1) = head_split(c.n_heads, Hkv_full, tp, r)
        L = {"Hq": q1 - q0, "Hkv": k1 - k0, "Dh": Dh,
             "attn_norm": self.f32(p + "attn_norm.weight"),
             "post_attn_norm": self.f32(p + "post_attention_norm.weight"),
             "ffn_norm": self.f32(p + "ffn_norm.weight"),
             "post_ffn_norm": self.f32(p + ("post_ffw_norm.weight" if self.has(p + "post_ffw_norm.weight")
                                            else "ffn_post_norm.weight")),
             "q_norm": self.f32(p + "attn_q_norm.weight", optional=True),
             "k_norm": self.f32(p + "attn_k_norm.weight", optional=True)}
        q = self.qw(p + "attn_q.weight")
        wo = self.qw(p + "attn_output.weight")
        if tp > 1:
            q, wo = q.row_slice(q0 * Dh, q1 * Dh), wo.col_slice(q0 * Dh, q1 * Dh)
        L["wq"], L["wo"] = q, wo
        if self.has(p + "attn_k.weight"):
            k, v = self.qw(p + "attn_k.weight"), self.qw(p + "attn_v.weight", optional=True)
            if tp > 1:
                k = k.row_slice(k0 * Dh, k1 * Dh)
                v = v.row_slice(k0 * Dh, k1 * Dh) if v is not None else None
            L["wk"], L["wv"] = k, v
            if v is not None and q.ggml_type == k.ggml_type == v.ggml_type:
                L["wqkv"] = QuantWeight.concat_rows([q, k, v], p + "attn_qkv")
        g, u, d = self.qw(p + "ffn_gate.weight"), self.qw(p + "ffn_up.weight"), self.qw(p + "ffn_down.weight")
        if tp > 1:
            f0, f1 = block_split(g.N, block_size(d.ggml_type), tp, r)
            g, u, d = g.row_slice(f0, f1), u.row_slice(f0, f1), d.col_slice(f0, f1)
        L["gate_up"] = QuantWeight.concat_rows([g, u]) if g.ggml_type == u.ggml_type else None
        L["gate"], L["up"], L["down"] = g, u, d
        return L

    def _mlp(self, L, a, mid) -> torch.Tensor:
        if L["gate_up"] is not None:
            gu = F.linear(a, L["gate_up"], act=self.glu_act, out_dtype=torch.bfloat16)
        else:
            gu = F.glu(self.glu_act, F.linear(a, L["gate"], out_dtype=mid), F.linear(a, L["up"], out_dtype=mid))
        y = F.linear(F.as_act(gu), L["down"], out_dtype=torch.float32)
        if self.tp_size > 1:
            self.tp_all_reduce(y)
        return y

    def _attention(self, l, L, a, batch: Batch, mid, rope: RopeSpec, scale: float, window: int, v_norm: bool,
                   kv_layer: int, write_kv: bool) -> torch.Tensor:
        c = self.cfg
        Hq, Hkv, Dh = L["Hq"], L["Hkv"], L["Dh"]
        T = batch.T
        if write_kv and "wqkv" in L:
            qkv = F.linear(a, L["wqkv"], out_dtype=mid)
            q = qkv[:, :Hq * Dh].view(T, Hq, Dh)
            k = qkv[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh)
            v = qkv[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)
        else:
            q = F.linear(a, L["wq"], out_dtype=mid).view(T, Hq, Dh)
            if write_kv:
                k = F.linear(a, L["wk"], out_dtype=mid).view(T, Hkv, Dh)
                v = F.linear(a, L["wv"], out_dtype=mid).view(T, Hkv, Dh) if L.get("wv") is not None else k
            else:
                k = v = q            # unused: this layer reads a donor layer's cache
        kc, vc = self.kv.k[kv_layer], self.kv.v[kv_layer]
        if self.kv.is_window_layer(kv_layer):
            batch = batch.windowed()                    # the ring's slots and block table
        qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=kc, v_cache=vc, rope=rope,
                              qn=L["q_norm"], kn=L["k_norm"], v_norm=v_norm, eps=c.eps, q_scale=1.0,
                              write_kv=write_kv)
        if write_kv:
            self.cp_sync_kv(kv_layer)
        o = F.attention(qr, kc, vc, batch, scale=scale, Hq=Hq, Hkv=Hkv, Dh=Dh, window=window)
        y = F.linear(F.as_act(o), L["wo"], out_dtype=torch.float32)
        if self.tp_size > 1:
            self.tp_all_reduce(y)
        return y

    def _logits(self, h, batch: Batch) -> torch.Tensor:
        last = h[batch.last_idx].contiguous()
        a = F.norm(last, self.out_norm, self.cfg.eps, want_q8=True)
        logits = F.linear(a, self.lm_head, out_dtype=torch.float32)
        return F.softcap(logits, self.softcap)


@register_architecture("gemma3", "gemma2")
class Gemma3Model(_GemmaBase):
    supports_pipeline = True

    def parse_config(self) -> None:
        g, a, c = self.gguf, self.arch, self.cfg
        c.head_dim = g.get_int(f"{a}.attention.key_length", 0) or 256
        self.window = g.get_int(f"{a}.attention.sliding_window", 1024)
        self.rope_local = g.get_float(f"{a}.rope.local.freq_base", 10000.0)
        self.rope_scale = 8.0 if c.n_layers == 34 else c.rope_scale
        self.softcap = g.get_float(f"{a}.final_logit_softcapping", 0.0)

    def is_local(self, l: int) -> bool:
        return (l + 1) % 6 != 0

    def load_weights(self) -> None:
        c = self.cfg
        self.tok_emb, self.out_norm, self.lm_head = self.stage_tensors()
        self.l0, l1 = self.layer_range
        self.layers = [self._load_common_layer(l) for l in range(self.l0, l1)]
        Dh = c.head_dim
        self.rope_l = RopeSpec(rot_dim=Dh, theta_base=self.rope_local, mode=0)
        self.rope_g = RopeSpec(rot_dim=Dh, theta_base=c.rope_base, mode=0, freq_scale=1.0 / self.rope_scale)

    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        c = self.cfg
        small = batch.T <= F.GEMV_MAX_M
        if self.cp_wanted(batch) and self.__dict__.get("_cp_ctx") is None:
            return self.cp_run(batch, want_logits, lambda sub: self.forward_batch(sub, want_logits))
        mid = torch.float32 if small else torch.bfloat16
        h = self.stage_input(batch, lambda: self.inject_pending_embeddings(
            F.embed(self.tok_emb, batch.tokens, scale=math.sqrt(c.hidden))))
        for i, L in enumerate(self.layers):
            l = self.l0 + i
            local = self.is_local(l)
            a = F.norm(h, L["attn_norm"], c.eps, want_q8=small)
            y = self._attention(l, L, a, batch, mid, self.rope_l if local else self.rope_g, L["Dh"] ** -0.5,
                                self.window if local else 0, False, l, True)
            h = F.norm_add(y, L["post_attn_norm"], c.eps, h)
            a = F.norm(h, L["ffn_norm"], c.eps, want_q8=small)
            h = F.norm_add(self._mlp(L, a, mid), L["post_ffn_norm"], c.eps, h)
        if self.stage_handoff(h):
            return None
        return self._logits(h, batch) if want_logits else None


@register_architecture("gemma4", "gemma3n")
class Gemma4Model(_GemmaBase):
    supports_pipeline = True

    def parse_config(self) -> None:
        g, a, c = self.gguf, self.arch, self.cfg
        pat = g.get_array(f"{a}.attention.sliding_window_pattern")
        self.pattern = [bool(x) for x in pat] if pat else [((l + 1) % 6 != 0) for l in range(c.n_layers)]
        self.window = g.get_int(f"{a}.attention.sliding_window", 512)
        self.dh_global = g.get_int(f"{a}.attention.key_length", 512)
        self.dh_local = g.get_int(f"{a}.attention.key_length_swa", 256)
        self.rot_global = g.get_int(f"{a}.rope.dimension_count", 0) or int(
            self.dh_global * g.get_float(f"{a}.rope.partial_rotary_factor", 1.0))
        kv_arr = g.get_array(f"{a}.attention.head_count_kv")
        self.kv_global = g.get_int(f"{a}.attention.global_head_count_kv", 0)
        if kv_arr:
            c.n_kv_heads = int(kv_arr[0])
            if self.kv_global == 0:
                for i, loc in enumerate(self.pattern[:len(kv_arr)]):
                    if not loc:
                        self.kv_global = int(kv_arr[i])
                        break
        self.kv_global = self.kv_global or c.n_kv_heads
        self.rope_local = g.get_float(f"{a}.rope.freq_base_swa", 0.0) or g.get_float(f"{a}.rope.local.freq_base", 10000.0)
        self.softcap = g.get_float(f"{a}.final_logit_softcapping", 0.0)
        self.ple_dim = g.get_int(f"{a}.embedding_length_per_layer_input", 0)
        self.shared_kv = g.get_int(f"{a}.attention.shared_kv_layers", 0)
        self.n_experts = g.get_int(f"{a}.expert_count", 0)
        self.top_k = g.get_int(f"{a}.expert_used_count", 0)
        self.donors: Dict[int, int] = {}
        first = c.n_layers - self.shared_kv
        if self.shared_kv > 0:
            for i in range(first, c.n_layers):
                for j in range(first - 1, -1, -1):
                    if self.is_local(j) == self.is_local(i):
                        self.donors[i] = j
                        break

    def is_local(self, l: int) -> bool:
        return l < len(self.pattern) and self.pattern[l]

    def head_dim_of(self, l: int) -> int:
        return self.dh_local if self.is_local(l) else self.dh_global

    def kv_heads_of(self, l: int) -> int:
        return self.cfg.n_kv_heads if self.is_local(l) else self.kv_global

    def kv_donors(self) -> Dict[int, int]:
        l0, l1 = self.layer_range
        return {l: d for l, d in self.donors.items() if l0 <= l < l1}

    def load_weights(self) -> None:
        c = self.cfg
        self.l0, l1 = self.layer_range
        for l, d in self.donors.items():
            if self.l0 <= l < l1 and not self.l0 <= d < l1:
                raise ValueError(f"pipeline stage {self.pp_rank} holds layers {self.l0}..{l1 - 1}, but layer {l} reads the KV cache of "
                                 f"layer {d}: choose a number of stages that keeps shared-KV layers with their donors")
        self.tok_emb, self.out_norm, self.lm_head = self.stage_tensors()
        if self.tok_emb is None and self.ple_dim:
            self.tok_emb = self.qw("token_embd.weight")        # every stage derives its per-layer inputs from the embedded tokens
        self.layers = []
        for l in range(self.l0, l1):
            L = self._load_common_layer(l)
            p = f"blk.{l}."
            sc = self.f32(p + "layer_output_scale.weight", optional=True)
            L["out_scale"] = float(sc.reshape(-1)[0]) if sc is not None else 1.0
            if self.has(p + "inp_gate.weight"):
                L["ple_gate"], L["ple_proj"] = self.qw(p + "inp_gate.weight"), self.qw(p + "proj.weight")
                L["ple_norm"] = self.f32(p + "post_norm.weight")
            if self.n_experts and self.has(p + "ffn_gate_inp.weight"):
                L["router"] = self.qw(p + "ffn_gate_inp.weight")
                L["router_scale"] = self.f32(p + "ffn_gate_inp.scale", optional=True)
                ge, ue, de = (self.qw(p + f"ffn_{n}_exps.weight") for n in ("gate", "up", "down"))
                L["gate_up_exps"] = QuantWeight.concat_rows_per_expert([ge, ue])
                L["down_exps"] = de
                ds = self.f32(p + "ffn_down_exps.scale", optional=True)
                L["down_scale"] = ds if ds is not None else self.f32(p + "ffn_gate_inp.per_expert_scale", optional=True)
                nm = lambda a_, b_: self.f32(p + (a_ if self.has(p + a_) else b_))
                L["pre_norm_2"] = nm("pre_ffw_norm_2.weight", "ffn_pre_norm_2.weight")
                L["post_norm_1"] = nm("post_ffw_norm_1.weight", "ffn_post_norm_1.weight")
                L["post_norm_2"] = nm("post_ffw_norm_2.weight", "ffn_post_norm_2.weight")
            self.layers.append(L)
        if self.ple_dim:
            self.ple_emb = self.qw("per_layer_token_embd.weight", optional=True)
            self.ple_model_proj = self.qw("per_layer_model_proj.weight", optional=True)
            self.ple_proj_norm = self.f32("per_layer_proj_norm.weight", optional=True)
        ff = self.f32("rope_freqs.weight", optional=True)
        self.rope_l = RopeSpec(rot_dim=self.dh_local, theta_base=self.rope_local, mode=0)
        self.rope_g = RopeSpec(rot_dim=self.rot_global, theta_base=c.rope_base, mode=0,
                               freq_factors=ff[:self.rot_global // 2].contiguous() if ff is not None else None)

    def _ple(self, batch: Batch, h: torch.Tensor) -> Optional[torch.Tensor]:
        """Per-layer inputs [T, n_layers, ple_dim] (Gemma4Model.cs:1255-1352)."""
        if not self.ple_dim:
            return None
        c = self.cfg
        tok = proj = None
        if self.ple_emb is not None:
            tok = F.embed(self.ple_emb, batch.tokens, scale=math.sqrt(self.ple_dim))
        if self.ple_model_proj is not None:
            proj = F.linear(F.as_act(h), self.ple_model_proj, out_dtype=torch.float32) * (c.hidden ** -0.5)
            proj = ref.rmsnorm(proj.view(-1, self.ple_dim), self.ple_proj_norm, c.eps).view(batch.T, -1)
        if tok is not None and proj is not None:
            out = (proj + tok) * (2.0 ** -0.5)
        else:
            out = proj if proj is not None else tok
        return out.view(batch.T, c.n_layers, self.ple_dim) if out is not None else None

    def _moe(self, L, h_mid, small) -> torch.Tensor:
        c = self.cfg
        x = ref.rmsnorm(h_mid, None, c.eps) * (c.hidden ** -0.5)
        if L["router_scale"] is not None:
            x = x * L["router_scale"]
        logits = F.linear(F.as_act(x.to(torch.bfloat16) if x.is_cuda else x), L["router"], out_dtype=torch.float32)
        ids, w = F.route_topk_softmax(logits, self.top_k)
        a = F.norm(h_mid, L["pre_norm_2"], c.eps, want_q8=small)
        return F.moe_experts(a, ids, w, L["gate_up_exps"], L["down_exps"], act=self.glu_act,
                             down_scale=L["down_scale"])

    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        c = self.cfg
        small = batch.T <= F.GEMV_MAX_M
        if self.cp_wanted(batch) and self.__dict__.get("_cp_ctx") is None:
            return self.cp_run(batch, want_logits, lambda sub: self.forward_batch(sub, want_logits))
        mid = torch.float32 if small else torch.bfloat16
        h0 = None
        if self.is_first_stage or self.ple_dim:
            h0 = self.inject_pending_embeddings(F.embed(self.tok_emb, batch.tokens, scale=math.sqrt(c.hidden)))
        ple = self._ple(batch, h0) if h0 is not None else None
        h = self.stage_input(batch, lambda: h0)
        for i, L in enumerate(self.layers):
            l = self.l0 + i
            local = self.is_local(l)
            a = F.norm(h, L["attn_norm"], c.eps, want_q8=small)
            donor = self.donors.get(l)
            y = self._attention(l, L, a, batch, mid, self.rope_l if local else self.rope_g, 1.0,
                                self.window if local else 0, True, donor if donor is not None else l, donor is None)
            h = F.norm_add(y, L["post_attn_norm"], c.eps, h)
            a = F.norm(h, L["ffn_norm"], c.eps, want_q8=small)
            mlp = self._mlp(L, a, mid)
            if "router" in L:
                mlp = ref.rmsnorm(mlp, L["post_norm_1"], c.eps) + ref.rmsnorm(self._moe(L, h, small),
                                                                              L["post_norm_2"], c.eps)
            h = F.norm_add(mlp, L["post_ffn_norm"], c.eps, h)
            if ple is not None and "ple_gate" in L:
                g = F.linear(F.as_act(h), L["ple_gate"], out_dtype=torch.float32)
                g = F.glu(self.glu_act, g, ple[:, l].contiguous().to(g.dtype))
                pr = F.linear(F.as_act(g), L["ple_proj"], out_dtype=torch.float32)
                h = F.norm_add(pr, L["ple_norm"], c.eps, h)
            if L["out_scale"] != 1.0:
                h = h * L["out_scale"]
        if self.stage_handoff(h):
            return None
        return self._logits(h, batch) if want_logits else None

    def prefill_chunk(self, requested: int) -> int:
        """Gemma 4 prefills in chunks of min(2048, max(2 * window, 1024)) tokens, or ``TS_PREFILL_CHUNK`` when set
        (Gemma4Model.cs:593-637); a caller may ask for smaller chunks, not larger ones."""
        import os
        env = os.environ.get("TS_PREFILL_CHUNK")
        own = int(env) if env and env.isdigit() and int(env) > 0 else min(2048, max(2 * self.window, 1024))
        return max(1, min(requested, own))

    def forward_refill(self, tokens, chunk: int = 2048):
        return super().forward_refill(tokens, self.prefill_chunk(chunk))
