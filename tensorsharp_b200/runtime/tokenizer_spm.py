"""SentencePiece-style tokenizer driven by GGUF metadata (vocabulary + scores).

Behaviour matched to TensorSharp.Runtime/SentencePieceTokenizer.cs: control / user-defined
tokens are cut out first; the remaining text has spaces replaced by U+2581; a fragment that is
itself a vocabulary entry maps directly; otherwise adjacent pieces are merged greedily by the
highest vocabulary score of the merged piece, ties resolved towards the left-most pair
(:144-231), with ``<0xNN>`` byte fallback for pieces outside the vocabulary.  Decoding joins
byte-fallback tokens into UTF-8 and turns U+2581 back into spaces.
"""
from __future__ import annotations

import heapq
from typing import Dict, Iterable, List, Optional, Sequence

SPACE = "▁"


class SentencePieceTokenizer:
    def __init__(self, vocab: Sequence[str], token_types: Optional[Sequence[int]], scores: Optional[Sequence[float]],
                 bos_id: int = -1, eos_ids: Iterable[int] = (), add_bos: bool = False, add_eos: bool = False):
        self.vocab = list(vocab)
        self.token_to_id: Dict[str, int] = {}
        for i, t in enumerate(self.vocab):
            self.token_to_id[t] = i
        self.scores = list(scores) if scores is not None else []
        self.bos_id = bos_id
        self.eos_ids = [int(e) for e in eos_ids]
        self.add_bos, self.add_eos = add_bos, add_eos
        self.special_tokens = []
        if token_types is not None:
            for i, tt in enumerate(token_types[:len(self.vocab)]):
                if tt in (3, 4) and self.vocab[i]:
                    self.special_tokens.append(self.vocab[i])

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    @property
    def eos_id(self) -> int:
        return self.eos_ids[0] if self.eos_ids else -1

    def is_eos(self, tid: int) -> bool:
        return tid in self.eos_ids

    def lookup_token(self, s: str) -> int:
        return self.token_to_id.get(s, -1)

    # ------------------------------------------------------------------ encode
    def _byte_fallback(self, piece: str) -> List[int]:
        out = []
        for b in piece.encode("utf-8"):
            tid = self.token_to_id.get(f"<0x{b:02X}>")
            if tid is not None:
                out.append(tid)
        return out

    def _score(self, tid: int) -> float:
        return self.scores[tid] if tid < len(self.scores) else 0.0

    def _tokenize_piece(self, text: str) -> List[int]:
        syms = list(text)
        n = len(syms)
        if n == 0:
            return []
        if n == 1:
            tid = self.token_to_id.get(syms[0])
            return [tid] if tid is not None else self._byte_fallback(syms[0])
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        active = [True] * n
        heap: List = []

        def push(a: int, b: int) -> None:
            tid = self.token_to_id.get(syms[a] + syms[b])
            if tid is not None:
                # max score first; ties: smaller a, then smaller b
                heapq.heappush(heap, (-self._score(tid), a, b, len(syms[a]), len(syms[b])))

        for i in range(n - 1):
            push(i, i + 1)
        while heap:
            _, a, b, la, lb = heapq.heappop(heap)
            if not active[a] or not active[b] or len(syms[a]) != la or len(syms[b]) != lb or nxt[a] != b:
                continue
            syms[a] += syms[b]
            active[b] = False
            nxt[a] = nxt[b]
            if nxt[a] < n:
                prev[nxt[a]] = a
            if prev[a] >= 0 and active[prev[a]]:
                push(prev[a], a)
            if nxt[a] < n and active[nxt[a]]:
                push(a, nxt[a])
        out: List[int] = []
        for i in range(n):
            if not active[i] or not syms[i]:
                continue
            tid = self.token_to_id.get(syms[i])
            if tid is not None:
                out.append(tid)
            else:
                out.extend(self._byte_fallback(syms[i]))
        return out

    def encode(self, text: str, add_special: bool = True) -> List[int]:
        frags = [(text, None)]
        for sp in self.special_tokens:
            sid = self.token_to_id.get(sp)
            if sid is None:
                continue
            new = []
            for ftext, fid in frags:
                if fid is not None:
                    new.append((ftext, fid))
                    continue
                start = 0
                while True:
                    i = ftext.find(sp, start)
                    if i < 0:
                        if start < len(ftext):
                            new.append((ftext[start:], None))
                        break
                    if i > start:
                        new.append((ftext[start:i], None))
                    new.append((sp, sid))
                    start = i + len(sp)
            frags = new
        ids: List[int] = []
        for ftext, fid in frags:
            if fid is not None:
                ids.append(fid)
                continue
            sp_text = ftext.replace(" ", SPACE)
            direct = self.token_to_id.get(sp_text)
            if direct is not None:
                ids.append(direct)
            else:
                ids.extend(self._tokenize_piece(sp_text))
        if add_special:
            if self.add_bos and self.bos_id >= 0:
                ids.insert(0, self.bos_id)
            if self.add_eos and self.eos_ids:
                ids.append(self.eos_ids[0])
        return ids

    # ------------------------------------------------------------------ decode
    def token_bytes(self, tid: int) -> bytes:
        if tid < 0 or tid >= len(self.vocab):
            return b""
        tok = self.vocab[tid]
        if len(tok) == 6 and tok.startswith("<0x") and tok.endswith(">"):
            try:
                return bytes([int(tok[3:5], 16)])
            except ValueError:
                pass
        return tok.replace(SPACE, " ").encode("utf-8")

    def decode(self, ids: Iterable[int]) -> str:
        return b"".join(self.token_bytes(int(i)) for i in ids).decode("utf-8", errors="replace")
