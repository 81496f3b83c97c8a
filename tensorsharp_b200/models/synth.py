"""Random-initialised models written to GGUF (the benchmark and test fixtures).

No checkpoint can be downloaded where this runs, so every benchmark model is generated:
N(0, 0.02) weights from a seed, quantised with the block codecs, and serialised with the
same tensor names, shapes and metadata keys a real GGUF of that architecture carries.
The engine then loads the file exactly as it would load a released model.

The Q4_K_M recipe follows llama.cpp's mixture: Q4_K everywhere except ``attn_v`` and
``ffn_down`` in the first eighth, last eighth and every third layer in between (Q6_K),
and the output / tied embedding matrix (Q6_K).  Norms and biases are F32.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..gguf.constants import GGMLType, GGUFValueType
from ..gguf.writer import GGUFWriter
from ..quant import codecs


def _use_more_bits(i: int, n: int) -> bool:
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def file_type(name: str, layer: int, n_layers: int, scheme: str) -> GGMLType:
    """GGML type of a 2-D / 3-D weight under quantisation scheme ``scheme``."""
    scheme = scheme.upper()
    if scheme in ("F16", "BF16", "F32", "Q8_0", "Q4_0", "Q4_K", "Q5_K", "Q6_K", "MXFP4"):
        return GGMLType[scheme]
    if scheme == "Q4_K_UNIFORM":     # one type per matrix class (what the reference's fused decode needs)
        return GGMLType.Q6_K if name in ("output.weight", "token_embd.weight") else GGMLType.Q4_K
    if scheme == "Q4_K_M":
        if name in ("output.weight", "token_embd.weight"):
            return GGMLType.Q6_K
        if (name.endswith("attn_v.weight") or name.endswith("ffn_down.weight")
                or name.endswith("ffn_down_exps.weight")) and _use_more_bits(layer, n_layers):
            return GGMLType.Q6_K
        return GGMLType.Q4_K
    raise ValueError(f"unknown quantisation scheme {scheme}")


class SynthBuilder:
    """Accumulates metadata and lazily generated tensors, then writes the file."""

    def __init__(self, path: str, arch: str, seed: int = 0, device: Optional[str] = None, std: float = 0.02):
        self.w = GGUFWriter(path)
        self.arch = arch
        self.std = std
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.w.add("general.architecture", arch)
        self.w.add("general.name", f"synthetic-{arch}")

    def meta(self, key: str, value, vtype=None, elem_type=None):
        self.w.add(key if key.startswith(("general.", "tokenizer.")) else f"{self.arch}.{key}", value, vtype, elem_type)

    def _randn(self, shape, std=None):
        n = 1
        for s in shape:
            n *= s
        # generate in row chunks so a 150k x 2560 embedding never needs more than ~1 GB at once
        return torch.randn(tuple(shape), generator=self.gen, device=self.device, dtype=torch.float32) * (std or self.std)

    def weight(self, name: str, shape, t: GGMLType, std=None, fill: Optional[float] = None, random_codes=False):
        """Register a tensor; its data is generated when the file is written."""
        shape = tuple(int(s) for s in shape)

        def make():
            if random_codes and t == GGMLType.MXFP4:
                nb = math.prod(shape) // 32
                codes = torch.randint(0, 256, (nb, 16), generator=self.gen, device=self.device, dtype=torch.uint8)
                # scales near 2^-7 .. 2^-5 so that values stay O(0.02)
                e = torch.randint(119, 122, (nb, 1), generator=self.gen, device=self.device, dtype=torch.uint8)
                return torch.cat([e, codes], 1).reshape(-1).cpu().numpy()
            if fill is not None:
                x = torch.full(shape, float(fill), device=self.device)
            else:
                x = self._randn(shape, std)
            return codecs.quantize(x, t).cpu().numpy()
        self.w.add_tensor(name, shape, t, make)

    def tokenizer_stub(self, vocab: int, bos: int = 1, eos: int = 2, template: Optional[str] = None):
        """A byte-level BPE vocabulary with no merges: enough for the engine to load,
        encode ASCII text and decode ids."""
        toks = [f"<|tok{i}|>" for i in range(vocab)]
        types = [1] * vocab
        base = 3
        from ..runtime.tokenizer_bpe import byte_to_unicode
        b2u = byte_to_unicode()
        for b in range(256):
            if base + b < vocab:
                toks[base + b] = b2u[b]
        for i, name in ((0, "<unk>"), (bos, "<|bos|>"), (eos, "<|eos|>")):
            if i < vocab:
                toks[i] = name
                types[i] = 3
        self.w.add("tokenizer.ggml.model", "gpt2")
        self.w.add("tokenizer.ggml.pre", "default")
        self.w.add("tokenizer.ggml.tokens", toks, GGUFValueType.ARRAY, GGUFValueType.STRING)
        self.w.add("tokenizer.ggml.token_type", types, GGUFValueType.ARRAY, GGUFValueType.INT32)
        self.w.add("tokenizer.ggml.merges", [], GGUFValueType.ARRAY, GGUFValueType.STRING)
        self.w.add("tokenizer.ggml.bos_token_id", bos)
        self.w.add("tokenizer.ggml.eos_token_id", eos)
        self.w.add("tokenizer.ggml.add_bos_token", False)
        if template:
            self.w.add("tokenizer.chat_template", template)

    def write(self) -> int:
        return self.w.write()


CHATML_TEMPLATE = (
    "{%- for message in messages %}{{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>\\n' }}"
    "{%- endfor %}{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- endif %}")


def write_qwen3(path: str, *, n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=768, vocab=4096,
                scheme="Q8_0", eps=1e-6, rope_base=1e6, tied=True, context=40960, seed=0, device=None) -> int:
    """Qwen3-architecture decoder.  The defaults are the tiny CPU test config; the 4B
    benchmark shape is (36, 2560, 32, 8, 128, 9728, 151936, 'Q4_K_M')."""
    b = SynthBuilder(path, "qwen3", seed, device)
    b.meta("block_count", n_layers)
    b.meta("embedding_length", hidden)
    b.meta("attention.head_count", n_heads)
    b.meta("attention.head_count_kv", n_kv_heads)
    b.meta("attention.key_length", head_dim)
    b.meta("attention.value_length", head_dim)
    b.meta("attention.layer_norm_rms_epsilon", float(eps))
    b.meta("rope.freq_base", float(rope_base))
    b.meta("feed_forward_length", ffn)
    b.meta("context_length", context)
    b.tokenizer_stub(vocab, template=CHATML_TEMPLATE)
    ft = lambda n, l=0: file_type(n, l, n_layers, scheme)
    b.weight("token_embd.weight", (vocab, hidden), ft("token_embd.weight"))
    if not tied:
        b.weight("output.weight", (vocab, hidden), ft("output.weight"))
    b.weight("output_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
    for l in range(n_layers):
        p = f"blk.{l}."
        b.weight(p + "attn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        b.weight(p + "attn_q.weight", (n_heads * head_dim, hidden), ft(p + "attn_q.weight", l))
        b.weight(p + "attn_k.weight", (n_kv_heads * head_dim, hidden), ft(p + "attn_k.weight", l))
        b.weight(p + "attn_v.weight", (n_kv_heads * head_dim, hidden), ft(p + "attn_v.weight", l))
        b.weight(p + "attn_q_norm.weight", (head_dim,), GGMLType.F32, fill=1.0)
        b.weight(p + "attn_k_norm.weight", (head_dim,), GGMLType.F32, fill=1.0)
        b.weight(p + "attn_output.weight", (hidden, n_heads * head_dim), ft(p + "attn_output.weight", l))
        b.weight(p + "ffn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        b.weight(p + "ffn_gate.weight", (ffn, hidden), ft(p + "ffn_gate.weight", l))
        b.weight(p + "ffn_up.weight", (ffn, hidden), ft(p + "ffn_up.weight", l))
        b.weight(p + "ffn_down.weight", (hidden, ffn), ft(p + "ffn_down.weight", l))
    return b.write()


QWEN3_4B = dict(n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, ffn=9728, vocab=151936,
                scheme="Q4_K_M", rope_base=1e6, tied=True)
QWEN3_TINY = dict(n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=768, vocab=4096, scheme="Q8_0",
                  rope_base=1e6, tied=True)


def write_gptoss(path: str, *, n_layers=2, hidden=256, n_heads=8, n_kv_heads=2, head_dim=64, n_experts=8, top_k=2,
                 expert_ffn=256, vocab=4096, window=16, attn_scheme="BF16", expert_scheme="MXFP4", rope_base=150000.0,
                 rope_scale=32.0, orig_ctx=4096, eps=1e-5, context=131072, seed=0, device=None,
                 random_codes=True) -> int:
    """gpt-oss-architecture MoE.  The 20b benchmark shape is (24, 2880, 64, 8, 64, 32 experts
    top-4, expert_ffn 2880, vocab 201088, window 128), bf16 attention and MXFP4 experts with
    uniform-random fp4 codes and E8M0 scales."""
    b = SynthBuilder(path, "gpt-oss", seed, device)
    b.meta("block_count", n_layers)
    b.meta("embedding_length", hidden)
    b.meta("attention.head_count", n_heads)
    b.meta("attention.head_count_kv", n_kv_heads)
    b.meta("attention.key_length", head_dim)
    b.meta("attention.value_length", head_dim)
    b.meta("attention.layer_norm_rms_epsilon", float(eps))
    b.meta("attention.sliding_window", window)
    b.meta("rope.freq_base", float(rope_base))
    b.meta("rope.scaling.factor", float(rope_scale))
    b.meta("rope.scaling.original_context_length", orig_ctx)
    b.meta("expert_count", n_experts)
    b.meta("expert_used_count", top_k)
    b.meta("expert_feed_forward_length", expert_ffn)
    b.meta("feed_forward_length", expert_ffn)
    b.meta("context_length", context)
    b.tokenizer_stub(vocab)
    at, et = GGMLType[attn_scheme], GGMLType[expert_scheme]
    b.weight("token_embd.weight", (vocab, hidden), at)
    b.weight("output.weight", (vocab, hidden), at)
    b.weight("output_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
    for l in range(n_layers):
        p = f"blk.{l}."
        b.weight(p + "attn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        for n, rows in (("q", n_heads * head_dim), ("k", n_kv_heads * head_dim), ("v", n_kv_heads * head_dim)):
            b.weight(p + f"attn_{n}.weight", (rows, hidden), at)
            b.weight(p + f"attn_{n}.bias", (rows,), GGMLType.F32, std=0.02)
        b.weight(p + "attn_output.weight", (hidden, n_heads * head_dim), at)
        b.weight(p + "attn_output.bias", (hidden,), GGMLType.F32, std=0.02)
        b.weight(p + "attn_sinks.weight", (n_heads,), GGMLType.F32, std=1.0)
        b.weight(p + "post_attention_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        b.weight(p + "ffn_gate_inp.weight", (n_experts, hidden), GGMLType.F32, std=0.5)
        b.weight(p + "ffn_gate_inp.bias", (n_experts,), GGMLType.F32, std=0.1)
        rc = random_codes and et == GGMLType.MXFP4
        b.weight(p + "ffn_gate_exps.weight", (n_experts, expert_ffn, hidden), et, random_codes=rc)
        b.weight(p + "ffn_up_exps.weight", (n_experts, expert_ffn, hidden), et, random_codes=rc)
        b.weight(p + "ffn_down_exps.weight", (n_experts, hidden, expert_ffn), et, random_codes=rc)
        b.weight(p + "ffn_gate_exps.bias", (n_experts, expert_ffn), GGMLType.F32, std=0.02)
        b.weight(p + "ffn_up_exps.bias", (n_experts, expert_ffn), GGMLType.F32, std=0.02)
        b.weight(p + "ffn_down_exps.bias", (n_experts, hidden), GGMLType.F32, std=0.02)
    return b.write()


GPTOSS_20B = dict(n_layers=24, hidden=2880, n_heads=64, n_kv_heads=8, head_dim=64, n_experts=32, top_k=4,
                  expert_ffn=2880, vocab=201088, window=128)


def write_qwen35(path: str, *, n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, rope_dims=32,
                 interval=4, hk=2, hv=4, dk=64, dv=64, conv_k=4, n_experts=8, top_k=2, expert_ffn=128,
                 shared_ffn=128, ffn=512, vocab=4096, scheme="Q8_0", eps=1e-6, rope_base=1e7, context=262144,
                 seed=0, device=None) -> int:
    """Qwen3.5-architecture hybrid (GatedDeltaNet + gated attention).  ``n_experts=0`` gives the
    dense variant.  The 35B-A3B benchmark shape is 40 layers, hidden 2048, interval 4, GDN
    16 QK / 32 V heads of 128, attention 16 q / 2 kv heads of 256, 256 experts top-8 + shared,
    expert_ffn 512, vocab 151936, Q4_K_M."""
    arch = "qwen35moe" if n_experts else "qwen35"
    b = SynthBuilder(path, arch, seed, device)
    b.meta("block_count", n_layers)
    b.meta("embedding_length", hidden)
    b.meta("attention.head_count", n_heads)
    b.meta("attention.head_count_kv", n_kv_heads)
    b.meta("attention.key_length", head_dim)
    b.meta("attention.value_length", head_dim)
    b.meta("attention.layer_norm_rms_epsilon", float(eps))
    b.meta("rope.freq_base", float(rope_base))
    b.meta("rope.dimension_count", rope_dims)
    b.meta("rope.dimension_sections", [rope_dims // 4, rope_dims // 4, 0, 0])
    b.meta("full_attention_interval", interval)
    b.meta("ssm.inner_size", hv * dv)
    b.meta("ssm.state_size", dk)
    b.meta("ssm.group_count", hk)
    b.meta("ssm.time_step_rank", hv)
    b.meta("ssm.conv_kernel", conv_k)
    b.meta("feed_forward_length", ffn)
    b.meta("context_length", context)
    if n_experts:
        b.meta("expert_count", n_experts)
        b.meta("expert_used_count", top_k)
        b.meta("expert_feed_forward_length", expert_ffn)
        b.meta("expert_shared_feed_forward_length", shared_ffn)
    b.tokenizer_stub(vocab, template=CHATML_TEMPLATE)
    ft = lambda n, l=0: file_type(n, l, n_layers, scheme)
    b.weight("token_embd.weight", (vocab, hidden), ft("token_embd.weight"))
    b.weight("output.weight", (vocab, hidden), ft("output.weight"))
    b.weight("output_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
    qkv_dim = 2 * hk * dk + hv * dv
    for l in range(n_layers):
        p = f"blk.{l}."
        b.weight(p + "attn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        b.weight(p + "post_attention_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        if (l + 1) % interval != 0:
            b.weight(p + "attn_qkv.weight", (qkv_dim, hidden), ft(p + "attn_qkv.weight", l), std=0.05)
            b.weight(p + "attn_gate.weight", (hv * dv, hidden), ft(p + "attn_gate.weight", l), std=0.05)
            b.weight(p + "ssm_beta.weight", (hv, hidden), GGMLType.F32, std=0.05)
            b.weight(p + "ssm_alpha.weight", (hv, hidden), GGMLType.F32, std=0.05)
            b.weight(p + "ssm_conv1d.weight", (qkv_dim, conv_k), GGMLType.F32, std=0.3)
            b.weight(p + "ssm_dt.bias", (hv,), GGMLType.F32, std=0.5)
            b.weight(p + "ssm_a", (hv,), GGMLType.F32, fill=-1.0)
            b.weight(p + "ssm_norm.weight", (dv,), GGMLType.F32, fill=1.0)
            b.weight(p + "ssm_out.weight", (hidden, hv * dv), ft(p + "ssm_out.weight", l))
        else:
            b.weight(p + "attn_q.weight", (2 * n_heads * head_dim, hidden), ft(p + "attn_q.weight", l))
            b.weight(p + "attn_k.weight", (n_kv_heads * head_dim, hidden), ft(p + "attn_k.weight", l))
            b.weight(p + "attn_v.weight", (n_kv_heads * head_dim, hidden), ft(p + "attn_v.weight", l))
            b.weight(p + "attn_q_norm.weight", (head_dim,), GGMLType.F32, fill=1.0)
            b.weight(p + "attn_k_norm.weight", (head_dim,), GGMLType.F32, fill=1.0)
            b.weight(p + "attn_output.weight", (hidden, n_heads * head_dim), ft(p + "attn_output.weight", l))
        if n_experts:
            b.weight(p + "ffn_gate_inp.weight", (n_experts, hidden), GGMLType.F32, std=0.5)
            b.weight(p + "ffn_gate_exps.weight", (n_experts, expert_ffn, hidden), ft(p + "ffn_gate_exps.weight", l))
            b.weight(p + "ffn_up_exps.weight", (n_experts, expert_ffn, hidden), ft(p + "ffn_up_exps.weight", l))
            b.weight(p + "ffn_down_exps.weight", (n_experts, hidden, expert_ffn), ft(p + "ffn_down_exps.weight", l))
            b.weight(p + "ffn_gate_shexp.weight", (shared_ffn, hidden), ft(p + "ffn_gate_shexp.weight", l))
            b.weight(p + "ffn_up_shexp.weight", (shared_ffn, hidden), ft(p + "ffn_up_shexp.weight", l))
            b.weight(p + "ffn_down_shexp.weight", (hidden, shared_ffn), ft(p + "ffn_down_shexp.weight", l))
            b.weight(p + "ffn_gate_inp_shexp.weight", (1, hidden), GGMLType.F32, std=0.1)
        else:
            b.weight(p + "ffn_gate.weight", (ffn, hidden), ft(p + "ffn_gate.weight", l))
            b.weight(p + "ffn_up.weight", (ffn, hidden), ft(p + "ffn_up.weight", l))
            b.weight(p + "ffn_down.weight", (hidden, ffn), ft(p + "ffn_down.weight", l))
    return b.write()


def write_gemma(path: str, *, arch="gemma3", n_layers=6, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512,
                vocab=4096, window=16, scheme="Q8_0", softcap=30.0, rope_base=1e6, rope_local=1e4, eps=1e-6,
                pattern=None, head_dim_global=None, kv_heads_global=None, rot_global=None, shared_kv=0, ple_dim=0,
                n_experts=0, top_k=0, expert_ffn=128, context=131072, seed=0, device=None) -> int:
    """Gemma 3 / Gemma 4 decoder.  The Gemma-4-31B-class benchmark shape is 60 layers, hidden 5376,
    32 q / 16 kv heads of 128, GeGLU 21504, window 1024, 5 sliding : 1 global, vocab 262144, Q8_0."""
    b = SynthBuilder(path, arch, seed, device)
    g4 = arch.startswith("gemma4")
    dh_g = head_dim_global or head_dim
    kv_g = kv_heads_global or n_kv_heads
    pattern = pattern if pattern is not None else [((l + 1) % 6 != 0) for l in range(n_layers)]
    b.meta("block_count", n_layers)
    b.meta("embedding_length", hidden)
    b.meta("attention.head_count", n_heads)
    b.meta("attention.layer_norm_rms_epsilon", float(eps))
    b.meta("attention.sliding_window", window)
    b.meta("rope.freq_base", float(rope_base))
    b.meta("feed_forward_length", ffn)
    b.meta("final_logit_softcapping", float(softcap))
    b.meta("context_length", context)
    if g4:
        b.meta("attention.head_count_kv", [n_kv_heads if loc else kv_g for loc in pattern])
        b.meta("attention.sliding_window_pattern", [bool(x) for x in pattern], GGUFValueType.ARRAY, GGUFValueType.BOOL)
        b.meta("attention.key_length", dh_g)
        b.meta("attention.key_length_swa", head_dim)
        b.meta("rope.freq_base_swa", float(rope_local))
        b.meta("rope.dimension_count", rot_global or dh_g)
        b.meta("attention.shared_kv_layers", shared_kv)
        if ple_dim:
            b.meta("embedding_length_per_layer_input", ple_dim)
        if n_experts:
            b.meta("expert_count", n_experts)
            b.meta("expert_used_count", top_k)
    else:
        b.meta("attention.head_count_kv", n_kv_heads)
        b.meta("attention.key_length", head_dim)
        b.meta("attention.value_length", head_dim)
        b.meta("rope.local.freq_base", float(rope_local))
    b.tokenizer_stub(vocab)
    ft = lambda n, l=0: file_type(n, l, n_layers, scheme)
    b.weight("token_embd.weight", (vocab, hidden), ft("token_embd.weight"))
    b.weight("output_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
    if g4 and ple_dim:
        b.weight("per_layer_token_embd.weight", (vocab, ple_dim * n_layers), ft("per_layer_token_embd.weight"))
        b.weight("per_layer_model_proj.weight", (ple_dim * n_layers, hidden), ft("per_layer_model_proj.weight"))
        b.weight("per_layer_proj_norm.weight", (ple_dim,), GGMLType.F32, fill=1.0)
    if g4 and (rot_global or dh_g):
        b.weight("rope_freqs.weight", ((rot_global or dh_g) // 2,), GGMLType.F32, fill=1.0)
    first_shared = n_layers - shared_kv
    for l in range(n_layers):
        p = f"blk.{l}."
        loc = pattern[l] if g4 else ((l + 1) % 6 != 0)
        dh = head_dim if (loc or not g4) else dh_g
        hkv = n_kv_heads if (loc or not g4) else kv_g
        for nm in ("attn_norm", "post_attention_norm", "ffn_norm", "post_ffw_norm"):
            b.weight(p + nm + ".weight", (hidden,), GGMLType.F32, fill=1.0)
        # Gemma 4 attends with scale 1.0 on RMS-normalised q / k; released checkpoints learn small
        # norm gains, so the synthetic ones are small too (unit gains give +-head_dim logits)
        b.weight(p + "attn_q_norm.weight", (dh,), GGMLType.F32, fill=0.35 if g4 else 1.0)
        b.weight(p + "attn_k_norm.weight", (dh,), GGMLType.F32, fill=0.35 if g4 else 1.0)
        b.weight(p + "attn_q.weight", (n_heads * dh, hidden), ft(p + "attn_q.weight", l))
        if not (g4 and shared_kv and l >= first_shared):
            b.weight(p + "attn_k.weight", (hkv * dh, hidden), ft(p + "attn_k.weight", l))
            b.weight(p + "attn_v.weight", (hkv * dh, hidden), ft(p + "attn_v.weight", l))
        b.weight(p + "attn_output.weight", (hidden, n_heads * dh), ft(p + "attn_output.weight", l))
        b.weight(p + "ffn_gate.weight", (ffn, hidden), ft(p + "ffn_gate.weight", l))
        b.weight(p + "ffn_up.weight", (ffn, hidden), ft(p + "ffn_up.weight", l))
        b.weight(p + "ffn_down.weight", (hidden, ffn), ft(p + "ffn_down.weight", l))
        if g4:
            b.weight(p + "layer_output_scale.weight", (1,), GGMLType.F32, fill=0.9 + 0.02 * l)
            if ple_dim:
                b.weight(p + "inp_gate.weight", (ple_dim, hidden), ft(p + "inp_gate.weight", l))
                b.weight(p + "proj.weight", (hidden, ple_dim), ft(p + "proj.weight", l))
                b.weight(p + "post_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
            if n_experts:
                b.weight(p + "ffn_gate_inp.weight", (n_experts, hidden), GGMLType.F32, std=1.0)
                b.weight(p + "ffn_gate_inp.scale", (hidden,), GGMLType.F32, fill=1.0)
                b.weight(p + "ffn_gate_exps.weight", (n_experts, expert_ffn, hidden), ft(p + "x", l))
                b.weight(p + "ffn_up_exps.weight", (n_experts, expert_ffn, hidden), ft(p + "x", l))
                b.weight(p + "ffn_down_exps.weight", (n_experts, hidden, expert_ffn), ft(p + "x", l))
                b.weight(p + "ffn_down_exps.scale", (n_experts,), GGMLType.F32, fill=1.0)
                for nm in ("pre_ffw_norm_2", "post_ffw_norm_1", "post_ffw_norm_2"):
                    b.weight(p + nm + ".weight", (hidden,), GGMLType.F32, fill=1.0)
    return b.write()


def write_mistral3(path: str, *, n_layers=3, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=4096,
                   scheme="Q8_0", rope_base=1e6, rope_scale=4.0, orig_ctx=64, eps=1e-5, seed=0, device=None) -> int:
    """Mistral-3-architecture decoder with YaRN metadata (a small original context so that
    tests exercise the blended frequencies and the position-dependent query scale)."""
    b = SynthBuilder(path, "mistral3", seed, device)
    b.meta("block_count", n_layers)
    b.meta("embedding_length", hidden)
    b.meta("attention.head_count", n_heads)
    b.meta("attention.head_count_kv", n_kv_heads)
    b.meta("attention.key_length", head_dim)
    b.meta("attention.value_length", head_dim)
    b.meta("attention.layer_norm_rms_epsilon", float(eps))
    b.meta("rope.freq_base", float(rope_base))
    b.meta("rope.dimension_count", head_dim)
    b.meta("rope.scaling.type", "yarn")
    b.meta("rope.scaling.factor", float(rope_scale))
    b.meta("rope.scaling.original_context_length", orig_ctx)
    b.meta("rope.scaling.yarn_beta_fast", 32.0)
    b.meta("rope.scaling.yarn_beta_slow", 1.0)
    b.meta("rope.scaling.mscale", 1.0)
    b.meta("rope.scaling.mscale_all_dim", 1.0)
    b.meta("attention.temperature_scale", 0.1)
    b.meta("feed_forward_length", ffn)
    b.meta("context_length", 32768)
    b.tokenizer_stub(vocab)
    ft = lambda n, l=0: file_type(n, l, n_layers, scheme)
    b.weight("token_embd.weight", (vocab, hidden), ft("token_embd.weight"))
    b.weight("output.weight", (vocab, hidden), ft("output.weight"))
    b.weight("output_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
    for l in range(n_layers):
        p = f"blk.{l}."
        b.weight(p + "attn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        b.weight(p + "attn_q.weight", (n_heads * head_dim, hidden), ft(p + "attn_q.weight", l))
        b.weight(p + "attn_k.weight", (n_kv_heads * head_dim, hidden), ft(p + "attn_k.weight", l))
        b.weight(p + "attn_v.weight", (n_kv_heads * head_dim, hidden), ft(p + "attn_v.weight", l))
        b.weight(p + "attn_output.weight", (hidden, n_heads * head_dim), ft(p + "attn_output.weight", l))
        b.weight(p + "ffn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        b.weight(p + "ffn_gate.weight", (ffn, hidden), ft(p + "ffn_gate.weight", l))
        b.weight(p + "ffn_up.weight", (ffn, hidden), ft(p + "ffn_up.weight", l))
        b.weight(p + "ffn_down.weight", (hidden, ffn), ft(p + "ffn_down.weight", l))
    return b.write()


def write_nemotron_h(path: str, *, pattern="MAFMEM", hidden=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=4096,
                     d_inner=256, d_state=64, ssm_heads=4, n_group=2, d_conv=4, n_experts=4, top_k=2, expert_ffn=128,
                     latent=128, scheme="Q8_0", eps=1e-5, seed=0, device=None) -> int:
    """Nemotron-H-architecture hybrid.  ``pattern``: one letter per layer - M Mamba2, A attention,
    F dense ReLU^2 FFN, E mixture of experts (latent projections + shared expert)."""
    has_moe = "E" in pattern
    b = SynthBuilder(path, "nemotron_h_moe" if has_moe else "nemotron_h", seed, device)
    n_layers = len(pattern)
    b.meta("block_count", n_layers)
    b.meta("embedding_length", hidden)
    b.meta("attention.head_count", [n_heads if ch == "A" else 0 for ch in pattern])
    b.meta("attention.head_count_kv", [n_kv_heads if ch == "A" else 0 for ch in pattern])
    b.meta("feed_forward_length", [ffn if ch in "FE" else 0 for ch in pattern])
    b.meta("attention.layer_norm_rms_epsilon", float(eps))
    b.meta("ssm.conv_kernel", d_conv)
    b.meta("ssm.inner_size", d_inner)
    b.meta("ssm.state_size", d_state)
    b.meta("ssm.time_step_rank", ssm_heads)
    b.meta("ssm.group_count", n_group)
    b.meta("context_length", 32768)
    if has_moe:
        b.meta("expert_count", n_experts)
        b.meta("expert_used_count", top_k)
        b.meta("expert_weights_norm", True)
        b.meta("expert_weights_scale", 2.5)
    b.tokenizer_stub(vocab)
    ft = lambda n, l=0: file_type(n, l, n_layers, scheme)
    hd = hidden // n_heads
    b.weight("token_embd.weight", (vocab, hidden), ft("token_embd.weight"))
    b.weight("output.weight", (vocab, hidden), ft("output.weight"))
    b.weight("output_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
    xbc = d_inner + 2 * n_group * d_state
    for l, ch in enumerate(pattern):
        p = f"blk.{l}."
        b.weight(p + "attn_norm.weight", (hidden,), GGMLType.F32, fill=1.0)
        if ch == "M":
            b.weight(p + "ssm_in.weight", (2 * d_inner + 2 * n_group * d_state + ssm_heads, hidden), GGMLType.F32, std=0.05)
            b.weight(p + "ssm_conv1d.weight", (xbc, d_conv), GGMLType.F32, std=0.3)
            b.weight(p + "ssm_conv1d.bias", (xbc,), GGMLType.F32, std=0.1)
            b.weight(p + "ssm_dt.bias", (ssm_heads,), GGMLType.F32, std=0.5)
            b.weight(p + "ssm_a", (ssm_heads,), GGMLType.F32, fill=-0.5)
            b.weight(p + "ssm_d", (ssm_heads,), GGMLType.F32, fill=1.0)
            b.weight(p + "ssm_norm.weight", (d_inner,), GGMLType.F32, fill=1.0)
            b.weight(p + "ssm_out.weight", (hidden, d_inner), ft(p + "ssm_out.weight", l))
        elif ch == "A":
            b.weight(p + "attn_q.weight", (n_heads * hd, hidden), ft(p + "attn_q.weight", l))
            b.weight(p + "attn_k.weight", (n_kv_heads * hd, hidden), ft(p + "attn_k.weight", l))
            b.weight(p + "attn_v.weight", (n_kv_heads * hd, hidden), ft(p + "attn_v.weight", l))
            b.weight(p + "attn_output.weight", (hidden, n_heads * hd), ft(p + "attn_output.weight", l))
        elif ch == "E":
            b.weight(p + "ffn_gate_inp.weight", (n_experts, hidden), GGMLType.F32, std=0.5)
            b.weight(p + "exp_probs_b.bias", (n_experts,), GGMLType.F32, std=0.05)
            b.weight(p + "ffn_latent_in.weight", (latent, hidden), ft(p + "ffn_latent_in.weight", l))
            b.weight(p + "ffn_latent_out.weight", (hidden, latent), ft(p + "ffn_latent_out.weight", l))
            b.weight(p + "ffn_up_exps.weight", (n_experts, expert_ffn, latent), ft(p + "x", l))
            b.weight(p + "ffn_down_exps.weight", (n_experts, latent, expert_ffn), ft(p + "x", l))
            b.weight(p + "ffn_up_shexp.weight", (ffn, hidden), ft(p + "x", l))
            b.weight(p + "ffn_down_shexp.weight", (hidden, ffn), ft(p + "x", l))
        else:
            b.weight(p + "ffn_up.weight", (ffn, hidden), ft(p + "ffn_up.weight", l))
            b.weight(p + "ffn_down.weight", (hidden, ffn), ft(p + "ffn_down.weight", l))
    return b.write()
