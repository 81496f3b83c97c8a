"""The fused decode step: one persistent kernel per token (csrc/decode_mega.cu).

``MegaDecoder`` binds a dense decoder (Qwen3 / Qwen2 / Llama graph: RMSNorm, fused or separate Q / K / V, optional
per-head QK norm, RoPE, gated FFN, Q4_K / Q6_K matrices) to the kernel: it builds the device table of per-layer
weight pointers once, plans the launch (grid, shared-memory ring) and owns the exchange buffer that carries the
tagged words between CTAs and, with tensor parallelism, between ranks (a symmetric buffer mapped into every rank).
``step(batch)`` runs one token of one sequence and returns the logits of this rank's vocabulary rows.

The reference's counterpart is TSGgml_TransformerModelDecode (TensorSharp.GGML.Native/ggml_ops_transformer.cpp
:1012-1298), a ggml graph rebuilt on the host for every token.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import List, Optional

import torch

from ..gguf.constants import GGMLType
from ..quant.qweight import QuantWeight
from . import native

MAX_RANKS = 8
ACT = {"swiglu": 1, "geglu_tanh": 2, "geglu_erf": 3}


class QW(C.Structure):
    _fields_ = [("p0", C.c_void_p), ("p1", C.c_void_p), ("p2", C.c_void_p), ("p3", C.c_void_p),
                ("type", C.c_int), ("N", C.c_int), ("K", C.c_int)]


class MegaLayer(C.Structure):
    _fields_ = [("qkv", QW * 3), ("wo", QW), ("gate_up", QW), ("down", QW),
                ("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("qkv_bias", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p)]


class MegaArgs(C.Structure):
    _fields_ = [("layers", C.c_void_p), ("n_layers", C.c_int), ("embed", QW), ("lm_head", QW), ("out_norm", C.c_void_p),
                ("embed_scale", C.c_float), ("hidden", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("Dh", C.c_int),
                ("ffn", C.c_int), ("eps", C.c_float), ("attn_scale", C.c_float), ("rope_freq", C.c_void_p),
                ("rope_mscale", C.c_float), ("rot_dim", C.c_int), ("rope_mode", C.c_int), ("act", C.c_int),
                ("tokens", C.c_void_p), ("positions", C.c_void_p), ("kv_lens", C.c_void_p), ("slots", C.c_void_p),
                ("block_table", C.c_void_p), ("max_pages", C.c_int), ("page_size", C.c_int), ("logits", C.c_void_p),
                ("xbuf", C.c_void_p * MAX_RANKS), ("rank", C.c_int), ("size", C.c_int),
                ("off_qkv", C.c_long), ("off_part", C.c_long), ("off_attn", C.c_long), ("off_opr", C.c_long),
                ("off_act", C.c_long), ("off_dwn", C.c_long), ("step", C.c_void_p), ("status", C.c_void_p), ("prof", C.c_void_p),
                ("debug", C.c_int), ("splits", C.c_int), ("grid", C.c_int), ("stage_bytes", C.c_int), ("n_stages", C.c_int),
                ("off_h", C.c_int), ("off_xq", C.c_int), ("off_xds", C.c_int), ("off_bsum_words", C.c_int), ("off_qs", C.c_int), ("off_red", C.c_int),
                ("off_ring", C.c_int), ("smem_bytes", C.c_int)]


def rope_angles(rope, device) -> torch.Tensor:
    """Angle per position and rotated pair, with frequency factors, linear scaling and the YaRN ramp folded in
    (the arithmetic of rope_cs in csrc/elementwise.cu, which depends on the pair only)."""
    half = rope.rot_dim // 2
    pair = torch.arange(half, dtype=torch.float64)
    theta = torch.pow(torch.tensor(float(rope.theta_base), dtype=torch.float64), -2.0 * pair / float(rope.rot_dim))
    if rope.freq_factors is not None:
        theta = theta / rope.freq_factors.detach().double().cpu()[:half]
    th = rope.freq_scale * theta
    if rope.ext_factor != 0.0:
        y = (pair - rope.corr_lo) / max(0.001, rope.corr_hi - rope.corr_lo)
        ramp = (1.0 - y.clamp(0.0, 1.0)) * rope.ext_factor
        th = th * (1.0 - ramp) + theta * ramp
    return th.to(torch.float32).to(device)


def rope_mscale(rope) -> float:
    ms = float(rope.attn_factor)
    if rope.ext_factor != 0.0:
        ms *= 1.0 + 0.1 * math.log(1.0 / rope.freq_scale)
    return ms


def _supported(w: Optional[QuantWeight]) -> bool:
    return (w is not None and w.experts == 1 and w.ggml_type in (GGMLType.Q4_K, GGMLType.Q6_K) and w.K % 256 == 0
            and w.K <= 16384)


class MegaDecoder:
    """One-kernel decode steps for ``model`` (see the module docstring).  ``MegaDecoder.try_create`` returns ``None``
    when the model's graph or weight types are outside what the kernel covers; the per-op path runs then."""

    @staticmethod
    def try_create(model, act: str = "swiglu") -> Optional["MegaDecoder"]:
        try:
            return MegaDecoder(model, act)
        except (ValueError, native.NativeLibraryError):
            return None

    def __init__(self, model, act: str = "swiglu"):
        c = model.cfg
        dev = model.device
        if dev.type != "cuda":
            raise ValueError("the fused decode step needs a CUDA device")
        if model.pp_size > 1:
            raise ValueError("the fused decode step does not span pipeline stages")
        lib = native.lib()
        for f in ("tsb_mega_plan", "tsb_mega_decode", "tsb_mega_args_bytes", "tsb_mega_layer_bytes"):
            getattr(lib, f).restype = C.c_int
        lib.tsb_mega_xbuf_words.restype = C.c_long
        if lib.tsb_mega_args_bytes() != C.sizeof(MegaArgs) or lib.tsb_mega_layer_bytes() != C.sizeof(MegaLayer):
            raise native.NativeLibraryError("MegaArgs / MegaLayer layouts differ between the library and its binding")
        self.model, self.lib = model, lib
        self._keep: List[torch.Tensor] = []
        comm = model.comm if model.tp_size > 1 else None
        layers = (MegaLayer * len(model.layers))()
        for l, L in enumerate(model.layers):
            ml = layers[l]
            mats = [L["wqkv"]] if "wqkv" in L else [L["wq"], L["wk"], L["wv"]]
            if "gate_up" not in L:
                raise ValueError("gate and up have different block types")
            for w in mats + [L["wo"], L["gate_up"], L["down"]]:
                if not _supported(w):
                    raise ValueError(f"{w.name}: {w.ggml_type.name} with K={w.K} is outside the fused decode step")
            for i, w in enumerate(mats):
                self._fill(ml.qkv[i], w)
            self._fill(ml.wo, L["wo"])
            self._fill(ml.gate_up, L["gate_up"])
            self._fill(ml.down, L["down"])
            ml.attn_norm, ml.ffn_norm = L["attn_norm"].data_ptr(), L["ffn_norm"].data_ptr()
            ml.q_norm = L["q_norm"].data_ptr() if L.get("q_norm") is not None else None
            ml.k_norm = L["k_norm"].data_ptr() if L.get("k_norm") is not None else None
            ml.qkv_bias = L["qkv_bias"].data_ptr() if L.get("qkv_bias") is not None else None
            ml.k_cache = model.kv.k[model.l0 + l].data_ptr()
            ml.v_cache = model.kv.v[model.l0 + l].data_ptr()
        self.host_layers = layers
        raw = torch.frombuffer(bytearray(bytes(layers)), dtype=torch.uint8)
        self.dev_layers = raw.to(dev)
        a = MegaArgs()
        a.layers, a.n_layers = self.dev_layers.data_ptr(), len(model.layers)
        if not _supported(model.lm_head):
            raise ValueError("lm_head type is outside the fused decode step")
        self._fill(a.embed, model.tok_emb, pad=False)
        self._fill(a.lm_head, model.lm_head)
        a.out_norm = model.out_norm.data_ptr()
        a.embed_scale = float(getattr(model, "embed_scale", 1.0))
        a.hidden, a.Hq, a.Hkv, a.Dh = c.hidden, model.Hq, model.Hkv, c.head_dim
        a.ffn = model.layers[0]["gate_up"].N // 2
        a.eps, a.attn_scale = float(c.eps), float(c.head_dim) ** -0.5
        rope = model.rope
        self.rope_freq = rope_angles(rope, dev)
        a.rope_freq, a.rope_mscale = self.rope_freq.data_ptr(), rope_mscale(rope)
        a.rot_dim, a.rope_mode, a.act = int(rope.rot_dim), int(rope.mode), ACT[act]
        a.rank, a.size = (comm.rank, comm.size) if comm is not None else (0, 1)
        a.debug = int(os.environ.get("TSB_MEGA_DEBUG", "0"))
        words = lib.tsb_mega_xbuf_words(C.byref(a))
        if comm is not None:
            from ..parallel.symm import SymmetricBuffer
            self.xbuf = SymmetricBuffer(comm, words * 8)
            ptrs = self.xbuf.ptrs
        else:
            self.xbuf = torch.zeros(words * 2, dtype=torch.float32, device=dev)
            ptrs = [self.xbuf.data_ptr()]
        for r, p in enumerate(ptrs):
            a.xbuf[r] = p
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)        # [0] steps completed, [1] status
        a.step, a.status = self.state.data_ptr(), self.state.data_ptr() + 4
        self.status_word = self.state[1:2]
        self.logits = torch.zeros((1, model.lm_head.N), dtype=torch.float32, device=dev)
        a.logits = self.logits.data_ptr()
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        rc = lib.tsb_mega_plan(C.byref(a), layers, C.c_int(sms))
        if rc != 0:
            raise ValueError(lib.tsb_last_error().decode())
        self.args = a
        if comm is not None:
            comm.barrier()

    def _fill(self, q: QW, w: QuantWeight, pad: bool = True) -> None:
        ps = list(w.planes) + [None] * (4 - len(w.planes))
        if pad and w.ggml_type == GGMLType.Q6_K:
            # the kernel copies the 2-byte super-scales in 16-byte pieces: give the plane room behind its last row
            d = torch.cat([ps[3], torch.zeros(32, dtype=torch.uint8, device=ps[3].device)])
            self._keep.append(d)
            ps[3] = d
        q.p0, q.p1, q.p2, q.p3 = (p.data_ptr() if p is not None else None for p in ps)
        q.type, q.N, q.K = int(w.ggml_type), w.N, w.K

    PROFILE_SLOTS = ("of the rows: hoisting", "wait down + norm", "qkv rows", "attention", "merge", "wait attention", "o_proj rows",
                     "of the rows: dot products",
                     "wait o_proj + norm", "gate/up rows", "wait activations", "down rows", "final wait + norm", "lm_head rows",
                     "of the rows: waiting for stages", "tasks (count)", "attention: wait for q", "attention: norm + rope",
                     "attention: keys and values", "attention: merge of the warps")

    def enable_profile(self) -> torch.Tensor:
        """Diagnostics: from now on every step overwrites a ``[grid, 16]`` table of nanoseconds that thread 0 of each
        CTA spent per phase (summed over the layers; slot names in ``PROFILE_SLOTS``).  Costs a timer read per phase."""
        self.prof = torch.zeros((self.args.grid, 24), dtype=torch.int64, device=self.model.device)
        self.args.prof = self.prof.data_ptr()
        return self.prof

    def supports(self, batch) -> bool:
        return batch.is_decode and batch.T == 1 and batch.B == 1

    def step(self, batch) -> torch.Tensor:
        """One token of one sequence: ``batch`` carries the token id, its position, the cache length after the step,
        the KV slot and the block-table row (device tensors).  Returns f32 logits ``[1, rows of this rank's lm_head]``."""
        from . import kernels as k
        a = self.args
        a.tokens, a.positions, a.kv_lens = batch.tokens.data_ptr(), batch.positions.data_ptr(), batch.kv_lens.data_ptr()
        a.slots, a.block_table = batch.slots.data_ptr(), batch.block_table.data_ptr()
        a.max_pages, a.page_size = int(batch.block_table.shape[1]), int(batch.page_size)
        native.check(self.lib.tsb_mega_decode(C.byref(a), k._stream()), "mega_decode")
        k._count(1)
        return self.logits

    def status(self) -> int:
        torch.cuda.synchronize(self.model.device)
        return int(self.state[1].item())

    def close(self) -> None:
        if hasattr(self.xbuf, "close"):
            self.xbuf.close()


def phase_table(model, context: int = 2048, steps: int = 5) -> str:
    """Per-phase time table of the fused decode step on ``model`` (one GPU): prefill ``context`` random tokens, run
    ``steps`` decode steps with the in-kernel timers on and report, per slot of ``PROFILE_SLOTS``, the min / median /
    max over the CTAs of the microseconds that thread 0 of the CTA spent there in the last step."""
    md = model.mega_decoder()
    if md is None:
        raise RuntimeError("the fused decode step does not accept this model (set TSB_MEGA=1 on one GPU)")
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, model.cfg.vocab, (context,), generator=g).tolist()
    t = int(model.forward(prompt).argmax())
    prof = md.enable_profile()
    for _ in range(steps):
        t = int(model.forward([t]).argmax())
    torch.cuda.synchronize()
    us = prof.cpu().double() / 1e3
    a = md.args
    lines = [f"grid {a.grid}  stages {a.n_stages} x {a.stage_bytes} B  shared memory {a.smem_bytes} B  attention splits {a.splits}"]
    tot = us[:, [1, 2, 3, 4, 5, 6, 8, 9, 10, 11, 12, 13]].sum(1)
    lines.append("phases per CTA, us: min %.1f  median %.1f  max %.1f" % (tot.min(), tot.median(), tot.max()))
    for i, name in enumerate(md.PROFILE_SLOTS):
        c = us[:, i] * (1e3 if "count" in name else 1.0)
        lines.append("%-34s min %8.1f  median %8.1f  max %8.1f" % (name, c.min(), c.median(), c.max()))
    return "\n".join(lines)


if __name__ == "__main__":
    import argparse
    import os
    ap = argparse.ArgumentParser(description="phase table of the fused decode step for a GGUF model on cuda:0")
    ap.add_argument("model")
    ap.add_argument("--context", type=int, default=2048)
    cli = ap.parse_args()
    os.environ["TSB_MEGA"] = "1"
    os.environ["TSB_GRAPH_FORWARD"] = "0"
    from ..models.base import ModelBase
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:      # under torch.distributed.run: one tensor-parallel shard per rank
        from ..parallel.dist import init_from_env
        comm = init_from_env()
        model = ModelBase.create(cli.model, comm.device, max_context=cli.context + 256, max_seqs=2, tp_rank=comm.rank,
                                 tp_size=comm.size, comm=comm)
        table = phase_table(model, cli.context)
        if comm.rank == 0:
            print(f"rank 0 of {comm.size}\n{table}")
        comm.barrier()
        torch.cuda.synchronize()
        os._exit(0)                                     # (skip the NCCL teardown)
    print(phase_table(ModelBase.create(cli.model, "cuda", max_context=cli.context + 256), cli.context))
