"""Turns image / audio attachments of a conversation into embedding spans of the prompt.

Parity: TensorSharp.Models/ModelMultimodalInjector.cs — per-architecture placeholder expansion
(Gemma 4 ``<|image>`` / ``<|audio>`` single tokens -> start, n soft tokens, end; Gemma 3
``<start_of_image>`` -> ``\\n\\n``, start, 256 pads, end, ``\\n\\n``; Qwen 3.5 one ``<|image_pad|>``
per image -> n pads; Mistral 3 ``[IMG]`` -> rows of ``[IMG]`` closed by ``[IMG_BREAK]`` /
``[IMG_END]``), an embedding cache keyed by absolute path + size + mtime, and the span arithmetic
the KV-reuse planner needs (``clamp_reusable_prefix``, ``clamp_trim_start``, ``trim_prepared_prompt``,
``queue_prompt_embeddings``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from ..runtime.chat import ChatMessage
from . import audio as A
from . import image as I
from .vision import create_vision_encoder


@dataclass
class CachedEmbedding:
    path: str
    size: int
    mtime_ns: int
    embeddings: torch.Tensor
    extra0: int = 0
    extra1: int = 0

    @property
    def token_count(self) -> int:
        return int(self.embeddings.shape[0])


@dataclass
class PreparedSpan:
    entry: CachedEmbedding
    insert_position: int
    prompt_start: int
    prompt_end: int            # exclusive

    @property
    def end_position(self) -> int:
        return self.insert_position + self.entry.token_count


def find_token(tokens: List[int], tid: int, start: int) -> int:
    for i in range(max(start, 0), len(tokens)):
        if tokens[i] == tid:
            return i
    return -1


def expand_single_token_placeholder(tokens: List[int], pos: int, start_id: int, n: int, end_id: int) -> List[int]:
    """``tokens[pos]`` (the placeholder) becomes ``start, n x start_id-soft-token, end``: the soft
    tokens carry the placeholder id; their embeddings are overwritten by the encoder output."""
    return tokens[:pos] + [start_id] + [start_id] * n + [end_id] + tokens[pos + 1:]


def expand_image_tokens(tokens: List[int], pad_id: int, counts: List[int]) -> List[int]:
    """The i-th occurrence of ``pad_id`` is repeated ``counts[i]`` times (ChatTemplate.ExpandImageTokens)."""
    out, k = [], 0
    for t in tokens:
        if t == pad_id and k < len(counts):
            out.extend([pad_id] * counts[k])
            k += 1
        else:
            out.append(t)
    return out


def expand_gemma3_image_tokens(tokens: List[int], start_id: int, end_id: int, newline_id: int, pad_id: int, n: int) -> List[int]:
    """Every ``<start_of_image>`` becomes ``\\n\\n <start_of_image> pad x n <end_of_image> \\n\\n``."""
    out = []
    for t in tokens:
        if t == start_id:
            out += [newline_id, start_id] + [pad_id] * n + [end_id, newline_id]
        else:
            out.append(t)
    return out


class MultimodalInjector:
    def __init__(self, model):
        self.model = model
        self.vision = None
        self.audio = None
        self._vision_cache: Dict[str, CachedEmbedding] = {}
        self._audio_cache: Dict[str, CachedEmbedding] = {}
        self.vision_spans: List[PreparedSpan] = []
        self.audio_spans: List[PreparedSpan] = []

    # ------------------------------------------------------------------ projectors
    @property
    def has_vision_encoder(self) -> bool:
        return self.vision is not None

    def load_projectors(self, path: str) -> None:
        if not path or not path.strip():
            return
        self.vision = create_vision_encoder(self.model.arch, path, self.model.device)
        self._vision_cache.clear()
        if self.model.arch == "gemma4":
            from ..gguf.reader import GGUFFile
            with GGUFFile(path) as g:
                has_audio = any(n.startswith("a.") for n in g.tensors)
            self.audio = A.Gemma4AudioEncoder(path, self.model.device) if has_audio else None
            self._audio_cache.clear()

    def unload(self) -> None:
        self.vision = self.audio = None
        self._vision_cache.clear()
        self._audio_cache.clear()
        self.clear_prepared()

    # ------------------------------------------------------------------ cache
    @staticmethod
    def _version(path: str):
        try:
            st = os.stat(path)
            return st.st_size, st.st_mtime_ns
        except OSError:
            return -1, 0

    def _cached(self, cache: Dict[str, CachedEmbedding], path: str, make: Callable[[str], CachedEmbedding]) -> CachedEmbedding:
        full = os.path.abspath(path) if path and path.strip() else (path or "")
        size, mtime = self._version(full)
        hit = cache.get(full.lower())
        if hit is not None and hit.size == size and hit.mtime_ns == mtime:
            return hit
        fresh = make(full)
        fresh.size, fresh.mtime_ns = self._version(full)
        cache[full.lower()] = fresh
        return fresh

    # ------------------------------------------------------------------ prompt processing
    def clear_prepared(self) -> None:
        self.vision_spans, self.audio_spans = [], []

    def process_prompt_tokens(self, history: Optional[List[ChatMessage]], tokens: List[int]) -> List[int]:
        self.clear_prepared()
        if not history or not tokens:
            return tokens
        fn = {"gemma4": self._gemma4, "gemma3": self._gemma3, "mistral3": self._mistral3}.get(self.model.arch)
        if fn is None and self.model.arch in ("qwen35", "qwen35moe", "qwen3next"):
            fn = self._qwen35
        return fn(history, list(tokens)) if fn is not None else tokens

    @staticmethod
    def image_paths(history: List[ChatMessage]) -> List[str]:
        return [p for m in history if m.image_paths for p in m.image_paths if p]

    def _lookup(self, text: str, default: int) -> int:
        tok = self.model.tokenizer
        tid = tok.lookup_token(text) if hasattr(tok, "lookup_token") else -1
        return tid if tid is not None and tid >= 0 else default

    def _gemma4(self, history, tokens):
        img_start, img_end = self._lookup("<|image>", 255999), self._lookup("<image|>", 256000)
        aud_start, aud_end = self._lookup("<|audio>", -1), self._lookup("<audio|>", -1)
        proc = I.Gemma4ImageProcessor() if self.vision is not None else None
        search = 0
        for m in history:
            if m.image_paths and self.vision is not None:
                for path in m.image_paths:
                    def make(full, proc=proc):
                        px, w, h = proc.process(full)
                        return CachedEmbedding(full, 0, 0, self.vision.encode(px, w, h))
                    e = self._cached(self._vision_cache, path, make)
                    pos = find_token(tokens, img_start, search)
                    if pos >= 0:
                        tokens = expand_single_token_placeholder(tokens, pos, img_start, e.token_count, img_end)
                        self.vision_spans.append(PreparedSpan(e, pos + 1, pos, pos + e.token_count + 2))
                        search = pos + e.token_count + 2
            if m.audio_paths and self.audio is not None and aud_start >= 0 and aud_end >= 0:
                for path in m.audio_paths:
                    e = self._cached(self._audio_cache, path, self._encode_audio)
                    pos = find_token(tokens, aud_start, search)
                    if pos >= 0:
                        tokens = expand_single_token_placeholder(tokens, pos, aud_start, e.token_count, aud_end)
                        self.audio_spans.append(PreparedSpan(e, pos + 1, pos, pos + e.token_count + 2))
                        search = pos + e.token_count + 2
        return tokens

    def _encode_audio(self, full: str) -> CachedEmbedding:
        import numpy as np
        samples = A.decode_audio_file(full)
        if samples.size % 128:
            samples = np.concatenate([samples, np.zeros(128 - samples.size % 128, dtype=np.float32)])
        mel, frames = A.mel_spectrogram(samples)
        if mel is None or frames == 0:
            raise ValueError(f"Audio file '{full}' did not produce a valid mel spectrogram.")
        return CachedEmbedding(full, 0, 0, self.audio.encode(mel))

    def _gemma3(self, history, tokens):
        if self.vision is None:
            return tokens
        paths = self.image_paths(history)
        if not paths:
            return tokens
        proc = I.Gemma3ImageProcessor()
        start = self._lookup("<start_of_image>", proc.START_OF_IMAGE)
        tokens = expand_gemma3_image_tokens(tokens, start, proc.END_OF_IMAGE, proc.NEWLINE_NEWLINE, proc.PAD, proc.tokens_per_image)
        search = 0
        for path in paths:
            e = self._cached(self._vision_cache, path,
                             lambda full: CachedEmbedding(full, 0, 0, self.vision.encode(proc.process(full))))
            s = find_token(tokens, start, search)
            if s >= 0 and s + 1 < len(tokens) and tokens[s + 1] == proc.PAD:
                ins = s + 1
                self.vision_spans.append(PreparedSpan(e, ins, ins - 2, ins + e.token_count + 2))
                search = ins + proc.tokens_per_image + 2
        return tokens

    def _qwen35(self, history, tokens):
        if self.vision is None:
            return tokens
        paths = self.image_paths(history)
        pad = self._lookup("<|image_pad|>", -1)
        if not paths or pad < 0:
            return tokens
        proc = I.Qwen35ImageProcessor(self.vision.patch_size, self.vision.spatial_merge_size)

        def make(full):
            px, h, w = proc.process(full)
            return CachedEmbedding(full, 0, 0, self.vision.encode(px, h, w))
        entries = [self._cached(self._vision_cache, p, make) for p in paths]
        counts = [e.token_count for e in entries]
        tokens = expand_image_tokens(tokens, pad, counts)
        search = 0
        for e, n in zip(entries, counts):
            s = find_token(tokens, pad, search)
            if s >= 0:
                self.vision_spans.append(PreparedSpan(e, s, s, s + n))
                search = s + n
        return tokens

    def _mistral3(self, history, tokens):
        if self.vision is None:
            return tokens
        paths = self.image_paths(history)
        if not paths:
            return tokens
        proc = I.Mistral3ImageProcessor(self.vision.image_size, self.vision.patch_size)
        merge = self.vision.spatial_merge_size
        search = 0
        for path in paths:
            def make(full):
                px, w, h = proc.process(full)
                return CachedEmbedding(full, 0, 0, self.vision.encode(px, w, h), h // self.vision.patch_size // merge,
                                       w // self.vision.patch_size // merge)
            e = self._cached(self._vision_cache, path, make)
            rows, cols = e.extra0, e.extra1
            pos = find_token(tokens, proc.IMG, search)
            if pos < 0:
                continue
            block: List[int] = []
            for r in range(rows):
                block += [proc.IMG] * cols + [proc.IMG_END if r == rows - 1 else proc.IMG_BREAK]
            tokens = tokens[:pos] + block + tokens[pos + 1:]
            self.vision_spans.append(PreparedSpan(e, pos, pos, pos + rows * cols + rows))
            search = pos + rows * cols + rows
        return tokens

    # ------------------------------------------------------------------ span arithmetic
    def clamp_reusable_prefix(self, prefix: int) -> int:
        """A reused prefix must not end inside an embedding span: pull it back to the span's start."""
        for spans in (self.vision_spans, self.audio_spans):
            for s in spans:
                if s.insert_position < prefix < s.end_position:
                    prefix = min(prefix, s.insert_position)
        return prefix

    def clamp_trim_start(self, trim: int) -> int:
        """Context trimming must not cut through a span: push the cut past the span's end."""
        if trim <= 0:
            return trim
        for spans in (self.vision_spans, self.audio_spans):
            for s in spans:
                if s.prompt_start < trim < s.prompt_end:
                    trim = max(trim, s.prompt_end)
        return trim

    def trim_prepared_prompt(self, trim: int) -> None:
        if trim <= 0:
            return
        for spans in (self.vision_spans, self.audio_spans):
            kept = []
            for s in spans:
                if s.prompt_end <= trim:
                    continue
                s.insert_position -= trim
                s.prompt_start -= trim
                s.prompt_end -= trim
                kept.append(s)
            spans[:] = kept

    def queue_prompt_embeddings(self, reusable_prefix: int) -> bool:
        """Hand every span that is not wholly inside the reused prefix to the model; positions are
        relative to the first token that will be forwarded.  Mistral 3's spans interleave break
        tokens with image tokens, so its embeddings are scattered row by row."""
        queued = False
        for spans, setter in ((self.vision_spans, self.model.set_vision_embeddings),
                              (self.audio_spans, self.model.set_audio_embeddings)):
            for s in spans:
                if s.end_position <= reusable_prefix and not (self.model.arch == "mistral3" and s.prompt_end > reusable_prefix):
                    continue
                if self.model.arch == "mistral3" and s.entry.extra1 > 0:
                    rows, cols = s.entry.extra0, s.entry.extra1
                    for r in range(rows):
                        setter(s.entry.embeddings[r * cols:(r + 1) * cols], s.insert_position + r * (cols + 1) - reusable_prefix)
                else:
                    setter(s.entry.embeddings.clone(), s.insert_position - reusable_prefix)
                queued = True
        return queued


class SlotInjector(MultimodalInjector):
    """The injector of one request slot when several requests share a loaded model: its own prepared spans and its
    own queue (``model`` is the slot, whose ``set_vision_embeddings`` travels with the slot's next forward call), the
    encoders and the embedding caches of the shared model's injector."""

    def __init__(self, slot, shared: MultimodalInjector):
        super().__init__(slot)
        self.__dict__["_shared"] = shared
        self._vision_cache, self._audio_cache = shared._vision_cache, shared._audio_cache

    @property
    def vision(self):
        return self._shared.vision

    @vision.setter
    def vision(self, value):               # the base constructor's ``self.vision = None``: the encoders live on the shared injector
        pass

    @property
    def audio(self):
        return self._shared.audio

    @audio.setter
    def audio(self, value):
        pass

    def load_projectors(self, path: str) -> None:
        self._shared.load_projectors(path)

    def unload(self) -> None:
        self.clear_prepared()

