"""Build the tokenizer a GGUF file describes.

Parity: TensorSharp.Models/ModelBase.cs:456-492 (ParseTokenizer): ``tokenizer.ggml.model`` in
{llama, t5, gemma4} selects the SentencePiece tokenizer (and adds ``eot_token_id``, default 106,
to the end-of-sequence set), anything else the byte-level BPE tokenizer with
``tokenizer.ggml.pre`` choosing the pre-tokeniser pattern.
"""
from __future__ import annotations

from ..gguf.reader import GGUFFile
from .tokenizer_bpe import BpeTokenizer
from .tokenizer_spm import SentencePieceTokenizer


def tokenizer_from_gguf(g: GGUFFile):
    vocab = g.get_array("tokenizer.ggml.tokens") or []
    types = g.get_array("tokenizer.ggml.token_type")
    bos = g.get_int("tokenizer.ggml.bos_token_id", -1)
    eos = g.get_int("tokenizer.ggml.eos_token_id", -1)
    add_bos = g.get_bool("tokenizer.ggml.add_bos_token", False)
    add_eos = g.get_bool("tokenizer.ggml.add_eos_token", False)
    eos_ids = [eos] if eos >= 0 else []
    for e in (g.get_array("tokenizer.ggml.eos_token_ids") or []):
        if int(e) not in eos_ids:
            eos_ids.append(int(e))
    model = g.get_str("tokenizer.ggml.model", "gpt2")
    if model in ("llama", "t5", "gemma4"):
        scores = g.get_array("tokenizer.ggml.scores") or []
        eot = g.get_int("tokenizer.ggml.eot_token_id", 106)
        if eot not in eos_ids:
            eos_ids.append(eot)
        return SentencePieceTokenizer(vocab, types, scores, bos, eos_ids, add_bos, add_eos)
    merges = g.get_array("tokenizer.ggml.merges") or []
    return BpeTokenizer(vocab, merges, types, bos, eos_ids, add_bos, add_eos, g.get_str("tokenizer.ggml.pre", "default") or "default")
