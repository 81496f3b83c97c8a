"""Byte-level BPE tokenizer driven by GGUF metadata.

Behaviour matched to TensorSharp.Runtime/BpeTokenizer.cs: pre-tokeniser patterns for
``gpt-4o`` / ``tekken`` / default (:67-79); control (type 3) and user-defined (type 4)
tokens are cut out of the text first and mapped to their ids directly (:84-138); the
rest goes through GPT-2's byte→unicode table (:176-191) and a rank-priority merge loop
(:193-281); decoding inverts the byte table and tolerates partial UTF-8 (:289-311).
"""
from __future__ import annotations

from functools import lru_cache
from typing import Dict, Iterable, List, Optional, Sequence

import regex

_PATTERNS = {
    "gpt-4o": (r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?|"
               r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?|"
               r"\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+"),
    "tekken": (r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+|"
               r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*|"
               r"\p{N}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+"),
    "default": (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                r"\s*[\r\n]+|\s+(?!\S)|\s+"),
}

TOKEN_TYPE_CONTROL = 3
TOKEN_TYPE_USER_DEFINED = 4


@lru_cache(maxsize=1)
def byte_to_unicode() -> Dict[int, str]:
    """GPT-2's reversible byte → printable-unicode map."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


@lru_cache(maxsize=1)
def unicode_to_byte() -> Dict[str, int]:
    return {v: k for k, v in byte_to_unicode().items()}


class BpeTokenizer:
    def __init__(self, vocab: Sequence[str], merges: Sequence[str], token_types: Optional[Sequence[int]] = None,
                 bos_id: int = -1, eos_ids: Iterable[int] = (), add_bos: bool = False, add_eos: bool = False,
                 pre: str = "default"):
        self.vocab = list(vocab)
        self.token_to_id = {t: i for i, t in enumerate(self.vocab)}
        self.ranks = {m: i for i, m in enumerate(merges)}
        self.token_types = list(token_types) if token_types is not None else None
        self.bos_id = bos_id
        self.eos_ids = [int(e) for e in eos_ids]
        self.add_bos, self.add_eos = add_bos, add_eos
        key = pre if pre in _PATTERNS else ("gpt-4o" if pre in ("gpt-4o", "o200k") else "default")
        self._pre = regex.compile(_PATTERNS[key])
        specials = []
        if self.token_types is not None:
            for i, t in enumerate(self.token_types[:len(self.vocab)]):
                if t in (TOKEN_TYPE_CONTROL, TOKEN_TYPE_USER_DEFINED) and self.vocab[i]:
                    specials.append(self.vocab[i])
        self.special_tokens = specials
        # longest first so that a special token that prefixes another never wins by accident
        self._special_re = (regex.compile("|".join(regex.escape(s) for s in sorted(specials, key=len, reverse=True)))
                            if specials else None)
        self._cache: Dict[str, List[int]] = {}

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    @property
    def eos_id(self) -> int:
        return self.eos_ids[0] if self.eos_ids else -1

    def lookup_token(self, s: str) -> int:
        """Id of the vocabulary entry spelled ``s`` (special tokens included), or -1."""
        return self.token_to_id.get(s, -1) if hasattr(self, "token_to_id") else -1

    def is_eos(self, tid: int) -> bool:
        return tid in self.eos_ids

    # ------------------------------------------------------------------ encode
    def _bpe(self, piece: str) -> List[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        b2u = byte_to_unicode()
        syms = [b2u[b] for b in piece.encode("utf-8")]
        while len(syms) > 1:
            best, best_i = None, -1
            for i in range(len(syms) - 1):
                r = self.ranks.get(syms[i] + " " + syms[i + 1])
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            a, b = syms[best_i], syms[best_i + 1]
            out, i = [], 0
            while i < len(syms):
                if i < len(syms) - 1 and syms[i] == a and syms[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(syms[i])
                    i += 1
            syms = out
        ids = []
        for s in syms:
            tid = self.token_to_id.get(s)
            if tid is not None:
                ids.append(tid)
            else:  # unknown symbol: fall back to its single-byte tokens
                for ch in s:
                    t = self.token_to_id.get(ch)
                    if t is not None:
                        ids.append(t)
        if len(self._cache) < 65536:
            self._cache[piece] = ids
        return ids

    def _encode_plain(self, text: str, out: List[int]) -> None:
        for m in self._pre.finditer(text):
            out.extend(self._bpe(m.group(0)))

    def encode(self, text: str, add_special: bool = True) -> List[int]:
        ids: List[int] = []
        if add_special and self.add_bos and self.bos_id >= 0:
            ids.append(self.bos_id)
        if self._special_re is None:
            self._encode_plain(text, ids)
        else:
            pos = 0
            for m in self._special_re.finditer(text):
                if m.start() > pos:
                    self._encode_plain(text[pos:m.start()], ids)
                ids.append(self.token_to_id[m.group(0)])
                pos = m.end()
            if pos < len(text):
                self._encode_plain(text[pos:], ids)
        if add_special and self.add_eos and self.eos_ids:
            ids.append(self.eos_ids[0])
        return ids

    # ------------------------------------------------------------------ decode
    def token_bytes(self, tid: int) -> bytes:
        if tid < 0 or tid >= len(self.vocab):
            return b""
        tok = self.vocab[tid]
        u2b = unicode_to_byte()
        out = bytearray()
        for ch in tok:
            b = u2b.get(ch)
            if b is None:
                out.extend(ch.encode("utf-8"))
            else:
                out.append(b)
        return bytes(out)

    def decode(self, ids: Iterable[int]) -> str:
        return b"".join(self.token_bytes(int(i)) for i in ids).decode("utf-8", errors="replace")
