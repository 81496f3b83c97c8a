"""GPT-OSS: alternating sliding-window / full attention with learned sinks, YaRN RoPE,
mixture of experts (top-k on router logits, softmax over the selected), SwiGLU with clamp,
MXFP4 expert weights, biases on every projection.

Parity: TensorSharp.Models/Models/GptOss/GptOssModel.cs - metadata keys :60-75, expert bias
split :95, gate/up fusion by concatenation :126, fused QKV + bias :182, even layers are
sliding-window :473, RoPE NeoX + YaRN (ext_factor 1, beta_fast 32, beta_slow 1,
freq_scale 1/scale) :683-687, sinks in the softmax :591-623, decode window :625-671,
router :814-865, clamp activation :901-934, last layer's MoE only on the last prompt token
:429-454.  Tensor names: attn_{q,k,v,output}.{weight,bias}, attn_sinks.weight,
post_attention_norm.weight, ffn_gate_inp.{weight,bias}, ffn_{gate,up,down}_exps.{weight,bias}.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..ops import functional as F
from ..ops.functional import Act, Batch, RopeSpec
from ..ops.kernels import yarn_corr_dims
from ..parallel.dist import even_split, head_split
from ..quant.qweight import QuantWeight
from .base import ModelBase, register_architecture


@register_architecture("gpt-oss", "gptoss")
class GptOssModel(ModelBase):
    supports_pipeline = True
    supports_context_parallel = True

    def parse_config(self) -> None:
        g, a, c = self.gguf, self.arch, self.cfg
        self.n_experts = g.get_int(f"{a}.expert_count", 0)
        self.top_k = g.get_int(f"{a}.expert_used_count", 0)
        self.window = g.get_int(f"{a}.attention.sliding_window", 128)
        self.expert_ffn = g.get_int(f"{a}.expert_feed_forward_length", 0)
        self.orig_ctx = g.get_int(f"{a}.rope.scaling.original_context_length", 4096)

    def load_weights(self) -> None:
        c = self.cfg
        tp, r = self.tp_size, self.tp_rank
        Dh = c.head_dim
        (q0, q1), (k0, k1) = head_split(c.n_heads, c.n_kv_heads, tp, r)
        self.Hq, self.Hkv = q1 - q0, k1 - k0
        # expert parallelism: contiguous expert ranges per rank (ep defaults to the tp group)
        ep, er = (self.ep_size, self.ep_rank) if self.ep_size > 1 else (tp, r)
        self.e0, self.e1 = even_split(self.n_experts, ep, er)
        # pipeline stages hold a contiguous range of layers; the embedding lives on the first stage (and on the last
        # one when the lm_head is tied to it), the output norm and lm_head on the last
        l0, l1 = self.layer_range
        self.l0 = l0
        tied = not self.has("output.weight")
        self.tok_emb = self.qw("token_embd.weight") if (self.is_first_stage or (self.is_last_stage and tied)) else None
        self.out_norm = self.f32("output_norm.weight") if self.is_last_stage else None
        self.lm_head = (self.qw("output.weight", optional=True) or self.tok_emb) if self.is_last_stage else None
        self.layers = []
        for l in range(l0, l1):
            p = f"blk.{l}."
            q, k, v = self.qw(p + "attn_q.weight"), self.qw(p + "attn_k.weight"), self.qw(p + "attn_v.weight")
            bq, bk, bv = (self.f32(p + f"attn_{n}.bias", optional=True) for n in "qkv")
            wo = self.qw(p + "attn_output.weight")
            sinks = self.f32(p + "attn_sinks.weight", optional=True)
            if tp > 1:
                q, k, v = q.row_slice(q0 * Dh, q1 * Dh), k.row_slice(k0 * Dh, k1 * Dh), v.row_slice(k0 * Dh, k1 * Dh)
                wo = wo.col_slice(q0 * Dh, q1 * Dh)
                if bq is not None:
                    bq, bk, bv = bq[q0 * Dh:q1 * Dh], bk[k0 * Dh:k1 * Dh], bv[k0 * Dh:k1 * Dh]
                if sinks is not None:
                    sinks = sinks[q0:q1].contiguous()
            L = {
                "attn_norm": self.f32(p + "attn_norm.weight"),
                "wo": wo,
                "bo": self.f32(p + "attn_output.bias", optional=True),
                "sinks": sinks,
                "ffn_norm": self.f32(p + ("post_attention_norm.weight" if self.has(p + "post_attention_norm.weight")
                                          else "ffn_norm.weight")),
                "router": self.qw(p + "ffn_gate_inp.weight"),
                "router_bias": self.f32(p + "ffn_gate_inp.bias", optional=True),
            }
            if q.ggml_type == k.ggml_type == v.ggml_type:
                L["wqkv"] = QuantWeight.concat_rows([q, k, v], p + "attn_qkv")
                L["bqkv"] = torch.cat([bq, bk, bv]).contiguous() if bq is not None else None
            else:
                L["wq"], L["wk"], L["wv"], L["bq"], L["bk"], L["bv"] = q, k, v, bq, bk, bv
            ge, ue, de = (self.qw(p + f"ffn_{n}_exps.weight") for n in ("gate", "up", "down"))
            gb, ub, db = (self.f32(p + f"ffn_{n}_exps.bias", optional=True) for n in ("gate", "up", "down"))
            if self.e1 - self.e0 != self.n_experts:
                ge, ue, de = (w.expert_range(self.e0, self.e1) for w in (ge, ue, de))
                gb, ub, db = (b[self.e0:self.e1] if b is not None else None for b in (gb, ub, db))
            if ge.ggml_type == ue.ggml_type:
                L["gate_up_exps"] = QuantWeight.concat_rows_per_expert([ge, ue], p + "ffn_gate_up_exps")
                L["gate_up_bias"] = torch.cat([gb, ub], 1).contiguous() if gb is not None else None
            else:
                raise ValueError(f"{p}ffn_gate_exps / ffn_up_exps have different types; cannot fuse")
            L["down_exps"], L["down_bias"] = de, (db.contiguous() if db is not None else None)
            self.layers.append(L)
        scale = c.rope_scale
        lo, hi = yarn_corr_dims(Dh, self.orig_ctx, c.rope_base, 32.0, 1.0)
        self.rope = RopeSpec(rot_dim=Dh, theta_base=c.rope_base, mode=0, freq_scale=1.0 / scale,
                             ext_factor=1.0 if scale != 1.0 else 0.0, attn_factor=1.0, corr_lo=lo, corr_hi=hi)

    @property
    def exchange_parts(self) -> int:
        return max(1, self.top_k)

    def kv_window_layers(self):
        return {l: self.window for l in range(self.cfg.n_layers) if l % 2 == 0}

    def attention_block(self, a, L, l: int, batch: Batch, mid, proj) -> torch.Tensor:
        """QKV projection (``proj(weight, bias)``), RoPE + cache write, attention -> ``[T, Hq * Dh]``."""
        c = self.cfg
        Hq, Hkv, Dh, T = self.Hq, self.Hkv, c.head_dim, batch.T
        if "wqkv" in L:
            qkv = proj(L["wqkv"], L["bqkv"])
            q = qkv[:, :Hq * Dh].view(T, Hq, Dh)
            k = qkv[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh)
            v = qkv[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)
        else:
            q, k, v = (proj(L["wq"], L["bq"]).view(T, Hq, Dh), proj(L["wk"], L["bk"]).view(T, Hkv, Dh),
                       proj(L["wv"], L["bv"]).view(T, Hkv, Dh))
        if self.kv.is_window_layer(l):
            batch = batch.windowed()                    # the ring's slots and block table
        qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[l], v_cache=self.kv.v[l],
                              rope=self.rope, eps=c.eps)
        self.cp_sync_kv(l)
        return F.attention(qr, self.kv.k[l], self.kv.v[l], batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh,
                           window=self.window if l % 2 == 0 else 0, sinks=L["sinks"])

    def forward_exchange_small(self, h: torch.Tensor, batch: Batch, want_logits: bool, tpx) -> Optional[torch.Tensor]:
        """Tensor + expert parallel small batches with the collectives inside the kernels: o_proj stores
        its partial sums into every rank's mailbox, and so does the experts' down projection (one
        weighted row per top-k slot: the expert-parallel combine), each followed by one kernel that adds
        the parts to the residual stream and normalises for the next projection."""
        c = self.cfg
        n_layers = len(self.layers)
        a = F.norm(h, self.layers[0]["attn_norm"], c.eps, want_q8=True)
        for l, L in enumerate(self.layers):
            o = self.attention_block(a, L, l, batch, torch.float32,
                                     lambda w, b: F.linear(a, w, bias=b, out_dtype=torch.float32))
            tpx.linear_push(F.as_act(o), L["wo"], bias=L["bo"])
            a = tpx.reduce_norm(h, L["ffn_norm"], c.eps)
            logits = F.linear(a, L["router"], bias=L["router_bias"], out_dtype=torch.float32)
            ids, w = F.route_topk_softmax(logits, self.top_k)
            F.moe_experts(a, ids, w, L["gate_up_exps"], L["down_exps"], act="swiglu_oai", gate_up_bias=L["gate_up_bias"],
                          down_bias=L["down_bias"], expert_offset=self.e0, push=tpx)
            nxt = self.layers[l + 1]["attn_norm"] if l + 1 < n_layers else None
            a = tpx.reduce_norm(h, nxt, c.eps, norm=nxt is not None, parts=self.top_k)
        if not want_logits:
            return None
        last = h[batch.last_idx].contiguous()
        return F.linear(F.norm(last, self.out_norm, c.eps, want_q8=True), self.lm_head, out_dtype=torch.float32)

    def forward_seq_parallel(self, h_all: torch.Tensor, batch: Batch, want_logits: bool, sp) -> Optional[torch.Tensor]:
        """Tensor + expert parallel prefill on sequence shards: o_proj reduces into the token owners from
        its GEMM epilogue.  Expert dispatch / combine: the owner normalises and routes its own rows, a kernel stores
        each row into the gathered buffer of the ranks that hold one of its chosen experts (and the routing records into
        every rank's), each rank runs its experts on the rows it received, and only those ranks store a partial sum back
        into the owner's accumulators, which the owner's next norm kernel adds.  With ``TSB_EP_ROUTED=0`` (or experts
        that do not divide evenly) every row goes to every rank and every rank sends a partial sum back."""
        c = self.cfg
        T = batch.T
        r0 = self.tp_rank * sp.shard
        mine = max(0, min(T, r0 + sp.shard) - r0)
        h = torch.zeros((sp.shard, c.hidden), dtype=torch.float32, device=h_all.device)
        if mine:
            h[:mine].copy_(h_all[r0:r0 + mine])
        sp.norm_gather(h, self.layers[0]["attn_norm"], c.eps, False)
        n_layers = len(self.layers)
        # TSB_EP_ROUTED=0: every row to every rank (all-gather) and a partial sum back from every rank (reduce-scatter)
        epr = self.n_experts // self.tp_size
        routed = (os.environ.get("TSB_EP_ROUTED", "1") != "0" and self.n_experts % self.tp_size == 0
                  and (self.e0, self.e1) == (self.tp_rank * epr, (self.tp_rank + 1) * epr) and self.top_k <= sp.route_kmax)
        for l, L in enumerate(self.layers):
            o = self.attention_block(None, L, l, batch, torch.bfloat16, lambda w, b: sp.gemm_ag(w, T, bias=b))
            sp.gemm_rs(o.view(T, -1), L["wo"], bias=L["bo"])
            nxt = self.layers[l + 1]["attn_norm"] if l + 1 < n_layers else self.out_norm
            if routed:
                # dispatch / combine by destination: the owner routes its own rows and sends each one only to the ranks
                # that hold one of its experts; only those ranks send a partial sum back
                sp.norm_gather(h, L["ffn_norm"], c.eps, True, local_only=True)
                mine_rows = Act(sp.xfull[sp.rows])
                logits = F.linear(mine_rows, L["router"], bias=L["router_bias"], out_dtype=torch.float32)
                ids, w = F.route_topk_softmax(logits, self.top_k)
                sp.dispatch(ids, w, T, epr)
                sp.wait_all()
                ids, w = sp.routes(T, self.top_k)
                a = Act(sp.xfull[:T])
                y = F.moe_experts(a, ids, w, L["gate_up_exps"], L["down_exps"], act="swiglu_oai", gate_up_bias=L["gate_up_bias"],
                                  down_bias=L["down_bias"], expert_offset=self.e0)
                sp.push_rows(y.contiguous(), T, k_routed=self.top_k, e0=self.e0, e1=self.e1)
                sp.norm_gather(h, nxt, c.eps, True, acc_k=self.top_k, experts_per_rank=epr)
                continue
            sp.norm_gather(h, L["ffn_norm"], c.eps, True)
            sp.wait_all()                                            # the router and the experts read the gathered rows
            a = Act(sp.xfull[:T])
            logits = F.linear(a, L["router"], bias=L["router_bias"], out_dtype=torch.float32)
            ids, w = F.route_topk_softmax(logits, self.top_k)
            y = F.moe_experts(a, ids, w, L["gate_up_exps"], L["down_exps"], act="swiglu_oai", gate_up_bias=L["gate_up_bias"],
                              down_bias=L["down_bias"], expert_offset=self.e0)
            sp.push_rows(y.contiguous(), T)
            sp.norm_gather(h, nxt, c.eps, True)
        if not want_logits:
            return None
        sp.wait_all()
        last = sp.xfull[batch.last_idx].contiguous()               # already normalised with the output norm
        return F.linear(Act(last), self.lm_head, out_dtype=torch.float32)

    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        c = self.cfg
        Hq, Hkv, Dh = self.Hq, self.Hkv, c.head_dim
        T = batch.T
        small = T <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        if self.pp_size > 1 and not self.is_first_stage:
            from ..parallel.pipeline import recv_hidden
            return self.run_layers(recv_hidden(self.pp_comm, self.pp_rank - 1, (T, c.hidden), self.device), batch, want_logits)
        if self.cp_wanted(batch):
            return self.cp_run(batch, want_logits, lambda sub: self.run_layers(F.embed(self.tok_emb, sub.tokens), sub, want_logits))
        h = F.embed(self.tok_emb, batch.tokens)
        if self.pp_size > 1:
            return self.run_layers(h, batch, want_logits)
        n_layers = len(self.layers)
        sharded = self.tp_size > 1 and (self.e1 - self.e0) != self.n_experts and self.ep_size <= 1
        if sharded and h.is_cuda:
            if small and T * self.top_k <= 4 * F.GEMV_MAX_M:
                tpx = self.tp_exchange()
                if tpx is not None:
                    return self.forward_exchange_small(h, batch, want_logits, tpx)
            elif not small and not batch.is_decode:      # sequence shards pay off for prompts, not for decode batches
                sp = self.tp_seq(T)
                if sp is not None:
                    return self.forward_seq_parallel(h, batch, want_logits, sp)
        return self.run_layers(h, batch, want_logits)

    def run_layers(self, h: torch.Tensor, batch: Batch, want_logits: bool) -> Optional[torch.Tensor]:
        """This process's layers on the residual stream ``h``; on the last (or only) pipeline stage the logits."""
        c = self.cfg
        T = batch.T
        small = T <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            a = F.norm(h, L["attn_norm"], c.eps, want_q8=small)
            o = self.attention_block(a, L, self.l0 + l, batch, mid, lambda w, b: F.linear(a, w, bias=b, out_dtype=mid))
            h = self.reduce_add(F.linear(F.as_act(o), L["wo"], bias=L["bo"] if self.tp_rank == 0 else None), h)
            # mixture of experts; on the last layer of a prefill only the last token of each
            # sequence feeds the logits, so only those rows are run
            last_only = self.is_last_stage and (l == n_layers - 1) and not batch.is_decode
            hm = h[batch.last_idx].contiguous() if last_only else h
            a = F.norm(hm, L["ffn_norm"], c.eps, want_q8=hm.shape[0] <= F.GEMV_MAX_M)
            logits = F.linear(a, L["router"], bias=L["router_bias"], out_dtype=torch.float32)
            ids, w = F.route_topk_softmax(logits, self.top_k)
            y = F.moe_experts(a, ids, w, L["gate_up_exps"], L["down_exps"], act="swiglu_oai",
                              gate_up_bias=L["gate_up_bias"], down_bias=L["down_bias"], expert_offset=self.e0)
            if self.e1 - self.e0 != self.n_experts and self.comm is not None:
                self.comm.all_reduce(y)
            if last_only:
                h = hm + y
            else:
                h = h + y
        if not self.is_last_stage:
            from ..parallel.pipeline import send_hidden
            send_hidden(self.pp_comm, self.pp_rank + 1, h)
            return None
        if not want_logits:
            return None
        last = h if (not batch.is_decode and n_layers > 0) else h[batch.last_idx].contiguous()
        a = F.norm(last.contiguous(), self.out_norm, c.eps, want_q8=True)
        return F.linear(a, self.lm_head, out_dtype=torch.float32)

    def reduce_add(self, y: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            self.comm.all_reduce(y)
        return h + y
