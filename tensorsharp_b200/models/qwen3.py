"""Qwen3 dense decoder: GQA attention with per-head QK RMSNorm, NeoX RoPE, SwiGLU FFN.

Parity: TensorSharp.Models/Models/Qwen3/Qwen3Model.cs:32-55 (construction, fused QKV and
gate/up), :175-236 (Forward: embedding, blocks, output_norm, last-row logits, tied
embeddings), :317-421 (attention: QK-norm, RoPE mode NeoX, cache write, causal softmax).
Tensor names: blk.{l}.{attn_norm, attn_q, attn_k, attn_v, attn_q_norm, attn_k_norm,
attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down}.weight, output_norm.weight,
output.weight (optional), token_embd.weight.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..gguf.constants import block_size
from ..ops import functional as F
from ..ops.functional import Batch, RopeSpec
from ..parallel.dist import block_split, even_split, head_split
from ..quant.qweight import QuantWeight
from .base import ModelBase, register_architecture


@register_architecture("qwen3", "qwen2", "llama")
class Qwen3Model(ModelBase):
    supports_pipeline = True
    supports_context_parallel = True

    def load_weights(self) -> None:
        c = self.cfg
        tp, r = self.tp_size, self.tp_rank
        Dh = c.head_dim
        # tensor parallelism: heads are dealt to ranks (column-parallel QKV, row-parallel o_proj),
        # the FFN width is dealt in units of ffn_down's quant block (column-parallel gate / up,
        # row-parallel down), the vocabulary is dealt evenly for the lm_head
        (q0, q1), (k0, k1) = head_split(c.n_heads, c.n_kv_heads, tp, r)
        self.Hq, self.Hkv = q1 - q0, k1 - k0
        # pipeline stages: the embedding lives on the first stage (and on the last one when the lm_head is tied
        # to it), the output norm and lm_head on the last
        l0, l1 = self.layer_range
        self.l0 = l0
        tied = not self.has("output.weight")
        self.tok_emb = self.qw("token_embd.weight") if (self.is_first_stage or (self.is_last_stage and tied)) else None
        self.out_norm = self.f32("output_norm.weight") if self.is_last_stage else None
        self.lm_head = (self.qw("output.weight", optional=True) or self.tok_emb) if self.is_last_stage else None
        self.vocab_sharded = tp > 1 and c.vocab % tp == 0 and self.lm_head is not None
        if self.vocab_sharded:
            v0, v1 = even_split(c.vocab, tp, r)
            self.lm_head = self.lm_head.row_slice(v0, v1)
        self.layers = []
        for l in range(l0, l1):
            p = f"blk.{l}."
            q, k, v = self.qw(p + "attn_q.weight"), self.qw(p + "attn_k.weight"), self.qw(p + "attn_v.weight")
            wo, down = self.qw(p + "attn_output.weight"), self.qw(p + "ffn_down.weight")
            f0, f1 = block_split(c.ffn, block_size(down.ggml_type), tp, r)
            if tp > 1:
                q, k, v = q.row_slice(q0 * Dh, q1 * Dh), k.row_slice(k0 * Dh, k1 * Dh), v.row_slice(k0 * Dh, k1 * Dh)
                wo, down = wo.col_slice(q0 * Dh, q1 * Dh), down.col_slice(f0, f1)
            L = {
                "attn_norm": self.f32(p + "attn_norm.weight"),
                "q_norm": self.f32(p + "attn_q_norm.weight", optional=True),
                "k_norm": self.f32(p + "attn_k_norm.weight", optional=True),
                "wo": wo,
                "ffn_norm": self.f32(p + "ffn_norm.weight"),
                "down": down,
            }
            # fused QKV needs one ggml type for the three matrices (Qwen3Model.cs:67-78)
            if q.ggml_type == k.ggml_type == v.ggml_type:
                L["wqkv"] = QuantWeight.concat_rows([q, k, v], p + "attn_qkv")
            else:
                L["wq"], L["wk"], L["wv"] = q, k, v
            g, u = self.qw(p + "ffn_gate.weight"), self.qw(p + "ffn_up.weight")
            if tp > 1:
                g, u = g.row_slice(f0, f1), u.row_slice(f0, f1)
            if g.ggml_type == u.ggml_type:
                L["gate_up"] = QuantWeight.concat_rows([g, u], p + "ffn_gate_up")
            else:
                L["gate"], L["up"] = g, u
            for b, (s0, s1) in (("attn_q.bias", (q0 * Dh, q1 * Dh)), ("attn_k.bias", (k0 * Dh, k1 * Dh)),
                                ("attn_v.bias", (k0 * Dh, k1 * Dh))):
                if self.has(p + b):
                    L.setdefault("qkv_bias", [])
                    L["qkv_bias"].append(self.f32(p + b)[s0:s1] if tp > 1 else self.f32(p + b))
            if "qkv_bias" in L:
                L["qkv_bias"] = torch.cat(L["qkv_bias"])
            self.layers.append(L)
        self.rope = RopeSpec(rot_dim=self.gguf.get_int(f"{self.arch}.rope.dimension_count", c.head_dim) or c.head_dim,
                             theta_base=c.rope_base, mode=0 if self.arch != "llama" else 1,
                             freq_scale=1.0 / c.rope_scale)

    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        c = self.cfg
        Hq, Hkv, Dh = self.Hq, self.Hkv, c.head_dim
        T = batch.T
        tp = self.tp_size > 1
        small = T <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        if self.pp_size > 1:
            return self.forward_stage(batch, want_logits)
        in_cp = self.__dict__.get("_cp_ctx") is not None
        if T == 1 and batch.is_decode and batch.B == 1 and not in_cp and not self._pending_embeddings:
            mega = self.mega_decoder()
            if mega is not None:
                # one sequence, one token: the whole step is one persistent kernel (ops/mega.py)
                logits = mega.step(batch)
                if not want_logits:
                    return None
                if self.vocab_sharded:
                    return self.comm.all_gather_cat(logits, dim=1)
                return logits if torch.cuda.is_current_stream_capturing() else logits.clone()
        if self.cp_wanted(batch) and not in_cp:
            # new sequence, equal slices, GPUs: attention pulls the earlier slices from peer memory; otherwise the general
            # route (two balanced pieces per rank, caches completed layer by layer)
            fused = (self.device.type == "cuda" and os.environ.get("TSB_CP_FUSED", "1") != "0"
                     and batch.h_kv_lens[0] == batch.T and batch.T % self.cp_comm.size == 0)
            if fused:
                return self.forward_context_parallel(batch, want_logits)
            return self.cp_run(batch, want_logits, lambda sub: self.forward_batch(sub, want_logits))
        h = self.inject_pending_embeddings(F.embed(self.tok_emb, batch.tokens))
        if h.is_cuda and not in_cp and T <= F.FUSED_MAX_M and F.can_fuse(h, self.layers[0].get("wqkv", self.layers[0].get("wq"))):
            return self.forward_fused_small(h, batch, want_logits)
        if tp and not small and not batch.is_decode and h.is_cuda:     # prompts only: decode batches stay on the GEMV / GEMM + all-reduce path
            sp = self.tp_seq(T)
            if sp is not None:
                return self.forward_seq_parallel(h, batch, want_logits, sp)
        # Tensor-parallel small batches exchange partial sums through peer memory inside the
        # projection and norm kernels (parallel/fused.py); everything else reduces with NCCL.
        tpx = self.tp_exchange() if (tp and small and h.is_cuda) else None
        a = F.norm(h, self.layers[0]["attn_norm"], c.eps, want_q8=small)
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            q, k, v = self.qkv_proj(a, L, T, mid)
            qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[self.l0 + l],
                                  v_cache=self.kv.v[self.l0 + l], rope=self.rope, qn=L["q_norm"], kn=L["k_norm"], eps=c.eps)
            qr = self.q_post_scale(qr, batch)
            self.cp_sync_kv(self.l0 + l)
            o = F.attention(qr, self.kv.k[self.l0 + l], self.kv.v[self.l0 + l], batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh,
                            as_act=small and L["wo"].uses_q8_activations)
            if tpx is not None:
                tpx.linear_push(F.as_act(o), L["wo"])
                a = tpx.reduce_norm(h, L["ffn_norm"], c.eps)
            else:
                h = self.row_parallel(F.as_act(o), L["wo"], h)
                a = F.norm(h, L["ffn_norm"], c.eps, want_q8=small)
            if "gate_up" in L:
                gu = F.linear(a, L["gate_up"], act="swiglu", out_dtype=torch.bfloat16)
            else:
                gu = F.glu("swiglu", F.linear(a, L["gate"], out_dtype=mid), F.linear(a, L["up"], out_dtype=mid))
            nxt = self.layers[l + 1]["attn_norm"] if l + 1 < n_layers else None
            if tpx is not None:
                tpx.linear_push(F.as_act(gu), L["down"])
                a = tpx.reduce_norm(h, nxt, c.eps, norm=nxt is not None)
            else:
                h = self.row_parallel(F.as_act(gu), L["down"], h)
                a = F.norm(h, nxt, c.eps, want_q8=small) if nxt is not None else None
        if not want_logits:
            return None
        last = h[batch.last_idx].contiguous()
        a = F.norm(last, self.out_norm, c.eps, want_q8=True)
        return self.lm_head_logits(a)

    def forward_stage(self, batch: Batch, want_logits: bool) -> Optional[torch.Tensor]:
        """One pipeline stage: the residual stream comes from the previous stage (or from the embedding on
        the first), runs through this stage's layers and goes to the next stage; the last stage returns the
        logits, the others ``None``.  Every stage is called with the same batch."""
        from ..parallel.pipeline import recv_hidden, send_hidden
        c = self.cfg
        Hq, Hkv, Dh, T = self.Hq, self.Hkv, c.head_dim, batch.T
        small = T <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        if self.is_first_stage:
            h = self.inject_pending_embeddings(F.embed(self.tok_emb, batch.tokens))
        else:
            h = recv_hidden(self.pp_comm, self.pp_rank - 1, (T, c.hidden), self.device)
        for l, L in enumerate(self.layers):
            a = F.norm(h, L["attn_norm"], c.eps, want_q8=small)
            q, k, v = self.qkv_proj(a, L, T, mid)
            qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[self.l0 + l],
                                  v_cache=self.kv.v[self.l0 + l], rope=self.rope, qn=L["q_norm"], kn=L["k_norm"], eps=c.eps)
            qr = self.q_post_scale(qr, batch)
            o = F.attention(qr, self.kv.k[self.l0 + l], self.kv.v[self.l0 + l], batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh)
            h = self.row_parallel(F.as_act(o), L["wo"], h)
            a = F.norm(h, L["ffn_norm"], c.eps, want_q8=small)
            if "gate_up" in L:
                gu = F.linear(a, L["gate_up"], act="swiglu", out_dtype=torch.bfloat16)
            else:
                gu = F.glu("swiglu", F.linear(a, L["gate"], out_dtype=mid), F.linear(a, L["up"], out_dtype=mid))
            h = self.row_parallel(F.as_act(gu), L["down"], h)
        if not self.is_last_stage:
            send_hidden(self.pp_comm, self.pp_rank + 1, h)
            return None
        if not want_logits:
            return None
        last = h[batch.last_idx].contiguous()
        return self.lm_head_logits(F.norm(last, self.out_norm, c.eps, want_q8=True))

    def forward_context_parallel(self, batch: Batch, want_logits: bool) -> Optional[torch.Tensor]:
        """A long prompt over a context-parallel group: this rank runs every layer on its slice of the tokens.
        Attention needs the keys and values of the earlier slices: on GPUs, when the sequence is new and the
        slices are equal, they are pulled from the peers' memory inside the attention kernels
        (parallel/context.py); otherwise they are taken from this rank's cache after the exchange.  The exchange
        runs in every layer either way, so that all ranks end with the whole cache and decode alike."""
        from ..parallel.context import exchange_kv_shards, shard_batch, shard_bounds
        c, cp = self.cfg, self.cp_comm
        Hq, Hkv, Dh = self.Hq, self.Hkv, c.head_dim
        bounds = [shard_bounds(batch.T, cp.size, s) for s in range(cp.size)]
        t0, t1 = bounds[cp.rank]
        sub = shard_batch(batch, t0, t1)
        n = sub.T
        small = n <= F.GEMV_MAX_M
        mid = torch.float32 if small else torch.bfloat16
        fresh = batch.h_kv_lens[0] == batch.T and all(b - a == n for a, b in bounds)
        cpa = self.cp_attention(n, Hkv, Dh) if fresh else None
        h = F.embed(self.tok_emb, sub.tokens)
        for l, L in enumerate(self.layers):
            kc, vc = self.kv.k[self.l0 + l], self.kv.v[self.l0 + l]
            a = F.norm(h, L["attn_norm"], c.eps, want_q8=small)
            q, k, v = self.qkv_proj(a, L, n, mid)
            qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=sub, k_cache=kc, v_cache=vc, rope=self.rope,
                                  qn=L["q_norm"], kn=L["k_norm"], eps=c.eps)
            qr = self.q_post_scale(qr, sub)
            if cpa is not None:
                o = cpa.attention(qr, kc.index_select(0, sub.slots), vc.index_select(0, sub.slots), Dh ** -0.5).view(n, Hq * Dh)
                exchange_kv_shards(cp, batch, bounds, kc, vc)
            else:
                exchange_kv_shards(cp, batch, bounds, kc, vc)
                o = F.attention(qr, kc, vc, sub, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh)
            h = F.linear(F.as_act(o), L["wo"], residual=h)
            a = F.norm(h, L["ffn_norm"], c.eps, want_q8=small)
            if "gate_up" in L:
                gu = F.linear(a, L["gate_up"], act="swiglu", out_dtype=torch.bfloat16)
            else:
                gu = F.glu("swiglu", F.linear(a, L["gate"], out_dtype=mid), F.linear(a, L["up"], out_dtype=mid))
            h = F.linear(F.as_act(gu), L["down"], residual=h)
        if not want_logits:
            return None
        # the prompt's last token sits on the last rank; the others compute a row of the same shape and take its
        last = h[sub.last_idx].contiguous()
        logits = F.linear(F.norm(last, self.out_norm, c.eps, want_q8=True), self.lm_head, out_dtype=torch.float32)
        return cp.all_gather_list(logits)[cp.size - 1]

    def qkv_proj(self, a, L, T: int, mid):
        Hq, Hkv, Dh = self.Hq, self.Hkv, self.cfg.head_dim
        if "wqkv" in L:
            qkv = F.linear(a, L["wqkv"], bias=L.get("qkv_bias"), out_dtype=mid)
            return (qkv[:, :Hq * Dh].view(T, Hq, Dh), qkv[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh),
                    qkv[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh))
        q, k, v = F.linear_multi(a, (L["wq"], L["wk"], L["wv"]), out_dtype=mid)
        return q.view(T, Hq, Dh), k.view(T, Hkv, Dh), v.view(T, Hkv, Dh)

    def forward_fused_small(self, h: torch.Tensor, batch: Batch, want_logits: bool) -> Optional[torch.Tensor]:
        """Decode-sized batches (at most ``F.FUSED_MAX_M`` rows) on CUDA: every projection does its
        own RMSNorm / cast and activation quantisation in-kernel, so a layer is QKV, RoPE + cache
        write, attention, o_proj, gate_up and down: no norm or quantise launches.  With tensor
        parallelism the row-parallel projections store their partial sums into the peer mailboxes
        and one kernel per exchange adds them to the residual stream."""
        c = self.cfg
        Hq, Hkv, Dh = self.Hq, self.Hkv, c.head_dim
        T = batch.T
        tpx = self.tp_exchange() if self.tp_size > 1 else None
        nccl = self.tp_size > 1 and tpx is None
        a = None                                     # normalised input left behind by an exchange
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            def proj(w, bias=None):
                if a is not None:
                    return F.linear(a, w, bias=bias, out_dtype=torch.float32)
                return F.linear_fused(h, w, norm_w=L["attn_norm"], eps=c.eps, do_norm=True, bias=bias)
            if "wqkv" in L:
                qkv = proj(L["wqkv"], L.get("qkv_bias"))
                q = qkv[:, :Hq * Dh].view(T, Hq, Dh)
                k = qkv[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh)
                v = qkv[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)
            else:
                q, k, v = proj(L["wq"]).view(T, Hq, Dh), proj(L["wk"]).view(T, Hkv, Dh), proj(L["wv"]).view(T, Hkv, Dh)
            qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[self.l0 + l],
                                  v_cache=self.kv.v[self.l0 + l], rope=self.rope, qn=L["q_norm"], kn=L["k_norm"], eps=c.eps)
            qr = self.q_post_scale(qr, batch)
            o = F.attention(qr, self.kv.k[self.l0 + l], self.kv.v[self.l0 + l], batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh).view(T, Hq * Dh)
            if tpx is not None:
                tpx.linear_push_fused(o, L["wo"])
                a = tpx.reduce_norm(h, L["ffn_norm"], c.eps)
                gu = F.linear(a, L["gate_up"], act="swiglu", out_dtype=torch.bfloat16) if "gate_up" in L else None
            else:
                if nccl:
                    y = F.linear_fused(o, L["wo"])
                    self.comm.all_reduce(y)
                    h.add_(y)
                else:
                    F.linear_fused(o, L["wo"], residual=h, out=h)
                gu = (F.linear_fused(h, L["gate_up"], norm_w=L["ffn_norm"], eps=c.eps, do_norm=True, act="swiglu",
                                     out_dtype=torch.bfloat16) if "gate_up" in L else None)
            if gu is None:
                an = a if tpx is not None else F.norm(h, L["ffn_norm"], c.eps, want_q8=True)
                gu = F.glu("swiglu", F.linear(an, L["gate"]), F.linear(an, L["up"]))
            if tpx is not None:
                nxt = self.layers[l + 1]["attn_norm"] if l + 1 < n_layers else None
                tpx.linear_push_fused(gu, L["down"])
                a = tpx.reduce_norm(h, nxt, c.eps, norm=nxt is not None)
            elif nccl:
                y = F.linear_fused(gu, L["down"])
                self.comm.all_reduce(y)
                h.add_(y)
            else:
                F.linear_fused(gu, L["down"], residual=h, out=h)
        if not want_logits:
            return None
        last = h if batch.last_idx.numel() == T else h[batch.last_idx].contiguous()
        logits = F.linear_fused(last, self.lm_head, norm_w=self.out_norm, eps=c.eps, do_norm=True)
        if self.vocab_sharded:
            logits = self.comm.all_gather_cat(logits, dim=1)
        return logits

    def forward_seq_parallel(self, h_all: torch.Tensor, batch: Batch, want_logits: bool, sp) -> Optional[torch.Tensor]:
        """Tensor-parallel prefill with the collectives inside the kernels: every rank keeps only its
        shard of the residual stream; o_proj and down reduce straight into the token owners'
        accumulators from the GEMM epilogue, the owner's norm kernel scatters the normalised rows to
        all ranks, and the QKV / gate_up GEMMs start each token tile when its shard has landed."""
        c = self.cfg
        Hq, Hkv, Dh = self.Hq, self.Hkv, c.head_dim
        T = batch.T
        r0 = self.tp_rank * sp.shard
        mine = max(0, min(T, r0 + sp.shard) - r0)
        h = torch.zeros((sp.shard, c.hidden), dtype=torch.float32, device=h_all.device)
        if mine:
            h[:mine].copy_(h_all[r0:r0 + mine])
        sp.norm_gather(h, self.layers[0]["attn_norm"], c.eps, False)
        n_layers = len(self.layers)
        for l, L in enumerate(self.layers):
            if "wqkv" in L:
                qkv = sp.gemm_ag(L["wqkv"], T, bias=L.get("qkv_bias"))
                q = qkv[:, :Hq * Dh].view(T, Hq, Dh)
                k = qkv[:, Hq * Dh:(Hq + Hkv) * Dh].view(T, Hkv, Dh)
                v = qkv[:, (Hq + Hkv) * Dh:].view(T, Hkv, Dh)
            else:
                q = sp.gemm_ag(L["wq"], T).view(T, Hq, Dh)
                k = sp.gemm_ag(L["wk"], T).view(T, Hkv, Dh)
                v = sp.gemm_ag(L["wv"], T).view(T, Hkv, Dh)
            qr = F.qkv_rope_cache(q, k, v, Hq=Hq, Hkv=Hkv, Dh=Dh, batch=batch, k_cache=self.kv.k[self.l0 + l],
                                  v_cache=self.kv.v[self.l0 + l], rope=self.rope, qn=L["q_norm"], kn=L["k_norm"], eps=c.eps)
            qr = self.q_post_scale(qr, batch)
            o = F.attention(qr, self.kv.k[self.l0 + l], self.kv.v[self.l0 + l], batch, scale=Dh ** -0.5, Hq=Hq, Hkv=Hkv, Dh=Dh)
            sp.gemm_rs(o.view(T, Hq * Dh), L["wo"])
            sp.norm_gather(h, L["ffn_norm"], c.eps, True)
            if "gate_up" in L:
                y = sp.gemm_ag(L["gate_up"], T)
                half = L["gate_up"].N // 2
                gu = F.glu("swiglu", y[:, :half], y[:, half:])
            else:
                gu = F.glu("swiglu", sp.gemm_ag(L["gate"], T), sp.gemm_ag(L["up"], T))
            sp.gemm_rs(gu, L["down"])
            sp.norm_gather(h, self.layers[l + 1]["attn_norm"] if l + 1 < n_layers else self.out_norm, c.eps, True)
        if not want_logits:
            return None
        sp.wait_all()
        last = sp.xfull[batch.last_idx].contiguous()       # already normalised with the output norm
        return self.lm_head_logits(F.Act(last))

    def q_post_scale(self, qr: torch.Tensor, batch: Batch) -> torch.Tensor:
        return qr

    def mega_decoder(self):
        """The one-kernel decode step for this model, or ``None`` when it does not apply (CPU, pipeline stages, a
        graph or weight types the kernel does not cover).  Built on first use.  ``TSB_MEGA``: ``1`` always, ``0``
        never; by default it runs with tensor parallelism, where it is what makes decode scale (its exchanges cost no
        launch and no collective), while one GPU keeps the per-op step, which measured faster there (2.0 ms against
        2.2 ms per token on the Qwen3-4B shape)."""
        m = self.__dict__.get("_mega")
        if m is None:
            m = False
            want = os.environ.get("TSB_MEGA", "auto")
            ok = (self.device.type == "cuda" and self.pp_size == 1 and want != "0"
                  and (want == "1" or self.tp_size > 1)
                  and type(self).q_post_scale is Qwen3Model.q_post_scale and self.kv_dtype == torch.bfloat16
                  and (self.tp_size == 1 or os.environ.get("TSB_TP_FUSED", "1") != "0"))
            if ok:
                from ..ops.mega import MegaDecoder
                m = MegaDecoder.try_create(self) or False
            self.__dict__["_mega"] = m
        return m or None

    def row_parallel(self, a, w: QuantWeight, h: torch.Tensor) -> torch.Tensor:
        """h + a @ w^T where ``w`` holds this rank's slice of the input features: the partial
        products are summed over the tensor-parallel group before the residual add."""
        if self.tp_size == 1:
            return F.linear(a, w, residual=h)
        y = F.linear(a, w)
        self.comm.all_reduce(y)
        return h.add_(y) if h.is_cuda else h + y

    def lm_head_logits(self, a) -> torch.Tensor:
        logits = F.linear(a, self.lm_head, out_dtype=torch.float32)
        if self.vocab_sharded:
            logits = self.comm.all_gather_cat(logits, dim=1)
        return logits
