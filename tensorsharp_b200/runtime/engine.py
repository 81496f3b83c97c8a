"""Generation loops: eager token loop, CUDA-graph decode, and the throughput benchmark.

The reference's hot loop is the host token loop of ModelService / Program.RunBenchmark
(TensorSharp.Cli/Program.cs:1515-1607): one native call per token, logits downloaded,
arg-max on the host.  Here a decode step is one CUDA-graph replay that ends with the
sampled ids on the device and the batch bookkeeping (positions, cache lengths, KV slots)
advanced by a kernel, so consecutive steps need no host work at all; the host only reads
ids when a caller wants them.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import torch

from ..ops import functional as F
from ..ops.functional import Batch
from .paged_kv import SeqState
from .sampling import SamplingConfig, TokenSampler


class DecodeGraph:
    """Greedy batched decode of ``seqs`` captured as one CUDA graph."""

    def __init__(self, model, seqs: Sequence[SeqState], max_new_tokens: int, use_graph: bool = True):
        self.model = model
        self.seqs = list(seqs)
        kv = model.kv
        for s in self.seqs:
            kv.reserve(s, s.length + max_new_tokens + 1)
        B = len(self.seqs)
        dev = model.device
        ps = kv.page_size
        width = max(len(s.pages) for s in self.seqs)
        table = torch.zeros((B, width), dtype=torch.int32)
        for i, s in enumerate(self.seqs):
            table[i, :len(s.pages)] = torch.tensor(s.pages, dtype=torch.int32)
        max_len = max(s.length for s in self.seqs) + max_new_tokens + 1
        self.batch = Batch(
            tokens=torch.zeros(B, dtype=torch.int32, device=dev),
            positions=torch.zeros(B, dtype=torch.int32, device=dev),
            slots=torch.zeros(B, dtype=torch.int64, device=dev),
            cu_q=torch.arange(B + 1, dtype=torch.int32, device=dev),
            kv_lens=torch.zeros(B, dtype=torch.int32, device=dev),
            block_table=table.to(dev),
            last_idx=torch.arange(B, dtype=torch.int64, device=dev),
            seq_slots=torch.tensor([s.slot for s in self.seqs], dtype=torch.int64, device=dev),
            max_q_len=1, max_kv_len=max_len, is_decode=True, page_size=ps,
            h_cu_q=tuple(range(B + 1)), h_kv_lens=tuple(s.length + 1 for s in self.seqs))
        self.sampled = torch.zeros(B, dtype=torch.int32, device=dev)
        self.h_tokens = torch.zeros(B, dtype=torch.int32).pin_memory() if dev.type == "cuda" else torch.zeros(B, dtype=torch.int32)
        self.h_sampled = torch.zeros(B, dtype=torch.int32).pin_memory() if dev.type == "cuda" else torch.zeros(B, dtype=torch.int32)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.use_graph = use_graph and dev.type == "cuda"
        self.launches_per_step = 0

    # ------------------------------------------------------------------ state
    def set_tokens(self, tokens: Sequence[int]) -> None:
        """Load the next input token of every sequence and the matching positions / slots."""
        ps = self.batch.page_size
        pos = [s.length for s in self.seqs]
        slots = [s.pages[p // ps] * ps + p % ps for s, p in zip(self.seqs, pos)]
        dev = self.model.device
        self.h_tokens.copy_(torch.tensor(list(tokens), dtype=torch.int32))
        self.batch.tokens.copy_(self.h_tokens, non_blocking=True)
        self.batch.positions.copy_(torch.tensor(pos, dtype=torch.int32), non_blocking=False)
        self.batch.kv_lens.copy_(torch.tensor([p + 1 for p in pos], dtype=torch.int32))
        self.batch.slots.copy_(torch.tensor(slots, dtype=torch.int64))

    def _step_body(self) -> None:
        self.batch.cache.clear()
        logits = self.model.forward_batch(self.batch, True)
        self.sampled.copy_(F.argmax(logits))
        if self.model.device.type == "cuda":
            from ..ops import kernels
            kernels.decode_advance(self.sampled, self.batch)
        else:
            self._advance_host()

    def _advance_host(self) -> None:
        b, ps = self.batch, self.batch.page_size
        b.tokens.copy_(self.sampled)
        b.positions.add_(1)
        b.kv_lens.copy_(b.positions + 1)
        page = (b.positions // ps).long()
        b.slots.copy_(b.block_table.gather(1, page.unsqueeze(1)).squeeze(1).long() * ps + (b.positions % ps).long())
        b.h_kv_lens = tuple(int(x) for x in b.kv_lens.tolist())

    def capture(self) -> None:
        """Warm up once (eagerly, without advancing) and capture the step."""
        if not self.use_graph:
            return
        from ..ops import kernels
        snap = [t.clone() for t in (self.batch.tokens, self.batch.positions, self.batch.kv_lens, self.batch.slots)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            n0 = kernels.LAUNCHES
            self._step_body()
            self.launches_per_step = kernels.LAUNCHES - n0
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for dst, src in zip((self.batch.tokens, self.batch.positions, self.batch.kv_lens, self.batch.slots), snap):
            dst.copy_(src)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step_body()

    # ------------------------------------------------------------------ stepping
    def step(self) -> torch.Tensor:
        """One decode step for every sequence; returns the sampled ids (device int32 [B])."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step_body()
        for s in self.seqs:
            s.length += 1
        return self.sampled

    def step_host(self, tokens: Sequence[int]) -> List[int]:
        """End-to-end step: token ids in from pinned host memory, sampled ids back out."""
        self.h_tokens.copy_(torch.tensor(list(tokens), dtype=torch.int32))
        self.batch.tokens.copy_(self.h_tokens, non_blocking=True)
        out = self.step()
        self.h_sampled.copy_(out, non_blocking=True)
        if self.model.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return self.h_sampled.tolist()


def generate(model, prompt: Sequence[int], max_tokens: int, sampler: Optional[TokenSampler] = None,
             eos_ids: Iterable[int] = (), on_token: Optional[Callable[[int], bool]] = None,
             prefill_chunk: int = 2048) -> List[int]:
    """Single-sequence generation on the model's default sequence (prefix already cached is
    the caller's business: pass only the suffix that still has to be prefilled)."""
    sampler = sampler or TokenSampler(SamplingConfig.greedy())
    eos = set(int(e) for e in eos_ids)
    logits = model.forward_refill(list(prompt), prefill_chunk)
    out: List[int] = []
    for _ in range(max_tokens):
        t = sampler.sample(logits, out)
        if t in eos:
            break
        out.append(t)
        if on_token is not None and on_token(t) is False:
            break
        logits = model.forward([t])
    return out


@dataclass
class BenchResult:
    prefill_tokens: int
    decode_tokens: int
    prefill_ms: float
    decode_ms: float

    @property
    def prefill_tps(self) -> float:
        return self.prefill_tokens / (self.prefill_ms / 1e3) if self.prefill_ms > 0 else 0.0

    @property
    def decode_tps(self) -> float:
        return self.decode_tokens / (self.decode_ms / 1e3) if self.decode_ms > 0 else 0.0

    @property
    def ms_per_token(self) -> float:
        return self.decode_ms / max(1, self.decode_tokens)


def synthetic_prompt(n: int, vocab: int) -> List[int]:
    """The reference benchmark's prompt ids: min(100, vocab-1) + (i % 17) (Program.cs:1515-1607)."""
    base = min(100, vocab - 1)
    return [min(vocab - 1, base + (i % 17)) for i in range(n)]


def run_benchmark(model, prefill: int = 32, decode: int = 64, runs: int = 1, chunked: bool = False,
                  use_graph: bool = True) -> List[BenchResult]:
    """``--benchmark``: per run reset the cache, time one prefill, then ``decode`` greedy
    steps.  Timed with CUDA events on a CUDA device (host clock on the CPU)."""
    cuda = model.device.type == "cuda"
    ids = synthetic_prompt(prefill, model.cfg.vocab)
    results = []
    for _ in range(runs):
        model.reset_kv_cache()
        if cuda:
            torch.cuda.synchronize()
            e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
            e0.record()
        t0 = time.perf_counter()
        logits = model.forward_refill(ids) if chunked else model.forward(ids)
        nxt = int(F.argmax(logits.view(1, -1))[0])
        if cuda:
            e1.record()
        t1 = time.perf_counter()
        seq = model._seq()
        if cuda and use_graph and decode > 0:
            dg = DecodeGraph(model, [seq], decode + 1)
            dg.set_tokens([nxt])
            dg.capture()
            torch.cuda.synchronize()
            e3.record()
            for _ in range(decode):
                dg.step()
            e2.record()
            torch.cuda.synchronize()
            pre_ms = e0.elapsed_time(e1)
            dec_ms = e3.elapsed_time(e2)
        else:
            for _ in range(decode):
                logits = model.forward([nxt])
                nxt = int(F.argmax(logits.view(1, -1))[0])
            if cuda:
                e2.record()
                torch.cuda.synchronize()
                pre_ms, dec_ms = e0.elapsed_time(e1), e1.elapsed_time(e2)
            else:
                t2 = time.perf_counter()
                pre_ms, dec_ms = 1e3 * (t1 - t0), 1e3 * (t2 - t1)
        results.append(BenchResult(prefill, decode, pre_ms, dec_ms))
    return results
