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
from typing import Dict, List, Optional

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
