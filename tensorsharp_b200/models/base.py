"""Model base class: GGUF loading, configuration, weights, KV pool and the public
single-sequence API (``forward`` / ``reset_kv_cache`` / ``truncate_kv_cache``).

Parity: TensorSharp.Models/ModelBase.cs:285-300 (ParseBaseConfig), :302-408 (context
length: env MAX_CONTEXT, then metadata, fallback 4096), :499-511 (which tensors stay
quantised), :532-658 (LoadWeights), :660-706 (one-time device upload), :1991-2007
(factory by ``general.architecture``); TensorSharp.Runtime/Contracts.cs
(IModelArchitecture: Forward, ResetKVCache, SupportsKVCacheTruncation, TruncateKVCache).
Unlike the reference, ``forward_batch`` runs any number of sequences in one packed batch.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..gguf.reader import GGUFFile
from ..ops import functional as F
from ..ops.functional import Batch
from ..quant import codecs
from ..quant.qweight import QuantWeight
from ..runtime.paged_kv import PagedKV, SeqState


@dataclass
class ModelConfig:
    """Fields read from ``{arch}.*`` GGUF metadata (ModelPrimitives.cs ModelConfig)."""
    arch: str = ""
    n_layers: int = 0
    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    ffn: int = 0
    vocab: int = 0
    eps: float = 1e-6
    rope_base: float = 10000.0
    rope_scale: float = 1.0
    context_length: int = 4096
    chat_template: Optional[str] = None
    extra: Dict[str, object] = field(default_factory=dict)


_REGISTRY: Dict[str, Callable] = {}


def register_architecture(*names: str):
    def deco(cls):
        for n in names:
            _REGISTRY[n] = cls
        return cls
    return deco


def supported_architectures() -> List[str]:
    return sorted(_REGISTRY)


class ModelBase:
    supports_kv_truncation = True
    supports_pipeline = False
    supports_context_parallel = False

    def __init__(self, path: str, device="cuda", *, max_context: Optional[int] = None, max_seqs: int = 1,
                 page_size: int = 64, kv_dtype: Optional[torch.dtype] = None, tp_rank: int = 0, tp_size: int = 1,
                 ep_rank: int = 0, ep_size: int = 1, comm=None, pp_rank: int = 0, pp_size: int = 1, pp_comm=None,
                 cp_comm=None):
        self.path = path
        self.device = torch.device(device)
        self.gguf = GGUFFile(path)
        self.tp_rank, self.tp_size, self.ep_rank, self.ep_size, self.comm = tp_rank, tp_size, ep_rank, ep_size, comm
        # pipeline parallelism: this process holds a contiguous range of layers (and only their KV cache);
        # the first stage owns the embedding, the last one the output norm and lm_head
        self.pp_rank, self.pp_size, self.pp_comm = pp_rank, pp_size, pp_comm
        if pp_size > 1 and not self.supports_pipeline:
            raise ValueError(f"{type(self).__name__} has no pipeline-parallel path")
        # context parallelism: every rank of ``cp_comm`` holds all the weights; a long prompt is dealt to the ranks
        # in order, each runs the layers on its slice and the K / V rows are exchanged layer by layer
        self.cp_comm = cp_comm if (cp_comm is not None and cp_comm.size > 1) else None
        if self.cp_comm is not None and not self.supports_context_parallel:
            raise ValueError(f"{type(self).__name__} has no context-parallel prefill")
        if self.cp_comm is not None and (tp_size > 1 or pp_size > 1):
            raise ValueError("context parallelism is not combined with tensor or pipeline parallelism")
        if pp_size > 1 and tp_size > 1:
            raise ValueError("pipeline stages are not combined with tensor parallelism")
        g = self.gguf
        self.arch = g.get_str("general.architecture", "")
        self.cfg = self.parse_base_config()
        self.parse_config()
        ctx_env = os.environ.get("MAX_CONTEXT")
        self.max_context = int(max_context or (int(ctx_env) if ctx_env else 0) or self.cfg.context_length or 4096)
        self.page_size = page_size
        self.max_seqs = max_seqs
        # TSB_KV_DTYPE=fp8: e4m3 pages, half the bytes of the bf16 cache (ops/functional.py: is_fp8)
        if kv_dtype is None and os.environ.get("TSB_KV_DTYPE", "").lower() in ("fp8", "e4m3", "float8_e4m3fn"):
            kv_dtype = torch.float8_e4m3fn
        self.kv_dtype = kv_dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        if self.kv_dtype == torch.float8_e4m3fn and self.cp_comm is not None:
            raise ValueError("the 8-bit KV cache is not combined with context parallelism (the shard exchange moves bf16 rows)")
        self.weights: Dict[str, object] = {}
        self.load_weights()
        self.kv = self.make_kv_pool()
        self._default_seq: Optional[SeqState] = None
        self.timing: Dict[str, float] = {}
        self._pending_embeddings: List[Tuple[torch.Tensor, int]] = []
        self._multimodal = None

    # ------------------------------------------------------------------ configuration
    def parse_base_config(self) -> ModelConfig:
        g, a = self.gguf, self.arch
        c = ModelConfig(arch=a)
        c.n_layers = g.get_int(f"{a}.block_count")
        c.hidden = g.get_int(f"{a}.embedding_length")
        c.n_heads = g.get_int(f"{a}.attention.head_count")
        c.n_kv_heads = g.get_int(f"{a}.attention.head_count_kv", c.n_heads)
        c.eps = g.get_float(f"{a}.attention.layer_norm_rms_epsilon", 1e-6)
        c.rope_base = g.get_float(f"{a}.rope.freq_base", 10000.0)
        c.rope_scale = g.get_float(f"{a}.rope.scaling.factor", 1.0) or 1.0
        c.chat_template = g.get_str("tokenizer.chat_template")
        kl = g.get_int(f"{a}.attention.key_length", 0)
        vl = g.get_int(f"{a}.attention.value_length", 0)
        c.head_dim = kl or vl or (c.hidden // max(1, c.n_heads))
        c.ffn = g.get_int(f"{a}.feed_forward_length", 0)
        c.context_length = g.get_int(f"{a}.context_length", 4096)
        if "token_embd.weight" in g.tensors:
            c.vocab = g.tensors["token_embd.weight"].shape[0]
        else:
            toks = g.get_array("tokenizer.ggml.tokens")
            c.vocab = len(toks) if toks else 0
        return c

    def parse_config(self) -> None:
        """Architecture-specific metadata; subclasses override."""

    @property
    def tokenizer(self):
        """The tokenizer described by the file's ``tokenizer.*`` metadata (built on first use)."""
        if getattr(self, "_tokenizer", None) is None:
            from ..runtime.tokenizer import tokenizer_from_gguf
            self._tokenizer = tokenizer_from_gguf(self.gguf)
        return self._tokenizer

    # ------------------------------------------------------------------ multimodal
    @property
    def multimodal(self):
        """The injector that turns image / audio attachments into embedding spans of the prompt
        (ModelBase.MultimodalInjector in the reference); ``None`` for text-only architectures."""
        if self._multimodal is None and self.arch in ("gemma3", "gemma4", "qwen35", "qwen35moe", "qwen3next", "mistral3"):
            from ..multimodal.injector import MultimodalInjector
            self._multimodal = MultimodalInjector(self)
        return self._multimodal

    def set_vision_embeddings(self, embeddings: torch.Tensor, insert_position: int) -> None:
        """Queue ``embeddings`` ``[n, hidden]`` to replace the token embeddings of rows
        ``[insert_position, insert_position + n)`` of the next forward call (SetVisionEmbeddings /
        SetAudioEmbeddings of the reference's multimodal models).  Only the pipeline stage that embeds tokens keeps them."""
        if self.pp_size > 1 and not self.is_first_stage and not getattr(self, "ple_dim", 0):
            return                                   # (stages that derive per-layer inputs from the embedded tokens keep them too)
        self._pending_embeddings.append((embeddings, int(insert_position)))

    set_audio_embeddings = set_vision_embeddings

    def inject_pending_embeddings(self, h: torch.Tensor) -> torch.Tensor:
        """Overwrite the queued spans in the (already scaled) embedding rows ``h``; spans that
        start before the chunk (a reused prefix) are clipped."""
        if not self._pending_embeddings:
            return h
        T = h.shape[0]
        for emb, pos in self._pending_embeddings:
            n = emb.shape[0]
            s, e = max(pos, 0), min(pos + n, T)
            if e > s:
                h[s:e] = emb[s - pos:e - pos].to(device=h.device, dtype=h.dtype)
        self._pending_embeddings = []
        return h

    # ------------------------------------------------------------------ tensor-parallel exchanges
    exchange_parts = 1     # partial rows a rank sends per token in the small-batch exchange (top-k for MoE models)

    def tp_exchange(self):
        """The peer-memory exchange of this tensor-parallel group for small batches (created on first
        use; TSB_TP_FUSED=0 keeps the NCCL all-reduce path, the baseline it is measured against)."""
        if getattr(self, "_tpx", None) is None:
            if os.environ.get("TSB_TP_FUSED", "1") == "0" or self.comm is None or self.device.type != "cuda":
                self._tpx = False
            else:
                from ..parallel.fused import TpExchange
                self._tpx = TpExchange(self.comm, F.GEMV_MAX_M * max(1, self.exchange_parts), self.cfg.hidden)
        return self._tpx or None

    def tp_all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        """Sum a row-parallel projection's output over the tensor-parallel group in place: through the peer-memory
        mailboxes for small batches (decode, short prompts), through NCCL otherwise (long prompts, CPU, TSB_TP_FUSED=0)."""
        if self.comm is None or self.comm.size <= 1:
            return y
        x = self.tp_exchange() if y.is_cuda else None
        if x is not None and x.fits(y):
            return x.all_reduce(y)
        return self.comm.all_reduce(y)

    def tp_seq(self, T: int):
        """The sequence-parallel prefill exchange, sized for at least ``T`` tokens (TSB_TP_FUSED=0
        keeps the GEMM + NCCL all-reduce path)."""
        if os.environ.get("TSB_TP_FUSED", "1") == "0" or self.comm is None or self.device.type != "cuda":
            return None
        sp = getattr(self, "_tpseq", None)
        if sp is None or sp.shard * self.tp_size < T:
            if sp is not None:
                sp.close()
            from ..parallel.fused import TpSeqParallel
            self._tpseq = sp = TpSeqParallel(self.comm, max(T, 4096), self.cfg.hidden)
        return sp

    def stage_tensors(self):
        """(embedding, output norm, lm_head) as this pipeline stage needs them: the embedding on the first stage (and on
        the last one when the lm_head is tied to it), norm and head on the last; everything without stages."""
        tied = not self.has("output.weight")
        emb = self.qw("token_embd.weight") if (self.is_first_stage or (self.is_last_stage and tied)) else None
        norm = self.f32("output_norm.weight") if self.is_last_stage else None
        head = (self.qw("output.weight", optional=True) or emb) if self.is_last_stage else None
        return emb, norm, head

    def stage_input(self, batch, embed):
        """The residual stream entering this process's layers: ``embed()`` on the first (or only) stage, else the
        previous stage's output (float32 ``[T, hidden]``)."""
        if self.pp_size > 1 and not self.is_first_stage:
            from ..parallel.pipeline import recv_hidden
            return recv_hidden(self.pp_comm, self.pp_rank - 1, (batch.T, self.cfg.hidden), self.device)
        return embed()

    def stage_handoff(self, h) -> bool:
        """On every stage but the last: send the residual stream on and return True (the caller returns ``None``)."""
        if self.pp_size > 1 and not self.is_last_stage:
            from ..parallel.pipeline import send_hidden
            send_hidden(self.pp_comm, self.pp_rank + 1, h.float())
            return True
        return False

    def cp_wanted(self, batch) -> bool:
        """A prompt goes through the context-parallel path when the model was given a group for it, the batch is
        one sequence's prompt and it has at least ``TSB_CP_MIN_TOKENS`` tokens (default 2048) and one per rank."""
        if self.cp_comm is None or batch.B != 1 or batch.is_decode or self._pending_embeddings:
            return False
        return batch.T >= max(self.cp_comm.size, int(os.environ.get("TSB_CP_MIN_TOKENS", "2048")))

    def cp_sync_kv(self, layer: int) -> None:
        """Called by attention blocks between the cache write and the attention.  During a context-parallel prefill it
        completes this rank's cache of ``layer`` with the other ranks' slices; otherwise it does nothing."""
        ctx = self.__dict__.get("_cp_ctx")
        if ctx is not None:
            from ..parallel.context import exchange_kv_shards
            exchange_kv_shards(self.cp_comm, ctx[0], ctx[1], self.kv.k[layer], self.kv.v[layer])

    def cp_run(self, batch, want_logits: bool, run):
        """Context-parallel prefill for any model whose attention blocks call :meth:`cp_sync_kv`: ``run(sub)`` is the
        model's ordinary forward on this rank's slice of the prompt (a batch of its own that sees the cache up to its
        last position); the logits are those of the rank that holds the prompt's last token."""
        from ..parallel.context import balanced_ranges, shard_batch
        cp = self.cp_comm
        bounds = [balanced_ranges(batch.T, cp.size, s) for s in range(cp.size)]      # two pieces per rank: equal causal work
        sub = shard_batch(batch, bounds[cp.rank])
        self.__dict__["_cp_ctx"] = (batch, bounds)
        try:
            logits = run(sub)
        finally:
            self.__dict__["_cp_ctx"] = None
        if not want_logits:
            return None
        # the prompt's last token is the end of one rank's last piece: that rank's last row is the answer
        owner = next(s for s in range(cp.size) if bounds[s][-1][1] == batch.T)
        return cp.all_gather_list(logits[-1:].contiguous())[owner]

    def cp_attention(self, n: int, Hkv: int, Dh: int):
        """The peer-memory attention of the context-parallel group for shards of ``n`` tokens (CUDA only,
        created on first use and regrown on demand; TSB_CP_FUSED=0 keeps the all-gather + local attention path)."""
        if self.device.type != "cuda" or os.environ.get("TSB_CP_FUSED", "1") == "0":
            return None
        cpa = self.__dict__.get("_cpa")
        if cpa is None or cpa.max_shard < n or (cpa.Hkv, cpa.Dh) != (Hkv, Dh):
            if cpa is not None:
                cpa.close()
            from ..parallel.context import ContextParallelAttention
            cpa = self.__dict__["_cpa"] = ContextParallelAttention(self.cp_comm, max(n, 4096), Hkv, Dh)
        return cpa

    # ------------------------------------------------------------------ weights
    def has(self, name: str) -> bool:
        return name in self.gguf.tensors

    def qw(self, name: str, optional: bool = False) -> Optional[QuantWeight]:
        """A matrix kept in its GGUF block form (2-D weights and 3-D expert stacks)."""
        if name not in self.gguf.tensors:
            if optional:
                return None
            raise KeyError(f"{self.path}: tensor {name!r} not found")
        ti = self.gguf.tensors[name]
        raw = self.gguf.tensor_bytes_view(name)
        return QuantWeight.from_raw(raw, ti.ggml_type, ti.shape, self.device, name)

    def f32(self, name: str, optional: bool = False) -> Optional[torch.Tensor]:
        """A small tensor (norm weight, bias, scalar table) decoded to float32 on the device."""
        if name not in self.gguf.tensors:
            if optional:
                return None
            raise KeyError(f"{self.path}: tensor {name!r} not found")
        ti = self.gguf.tensors[name]
        raw = torch.from_numpy(np.array(self.gguf.tensor_bytes_view(name)))
        return codecs.dequantize(raw, ti.ggml_type, ti.shape).to(self.device).contiguous()

    def load_weights(self) -> None:
        raise NotImplementedError

    # ------------------------------------------------------------------ KV pool
    @property
    def layer_range(self) -> Tuple[int, int]:
        """[first, last + 1) of the layers this pipeline stage runs (all of them without pipelining)."""
        from ..parallel.dist import even_split
        return even_split(self.cfg.n_layers, self.pp_size, self.pp_rank)

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    def kv_layer_shapes(self) -> List[Optional[Tuple[int, int]]]:
        c = self.cfg
        l0, l1 = self.layer_range
        return [(c.n_kv_heads // self.tp_size, c.head_dim) if l0 <= l < l1 else None for l in range(c.n_layers)]

    def kv_donors(self) -> Dict[int, int]:
        return {}

    def kv_window_layers(self) -> Dict[int, int]:
        """Layer -> sliding window, for the layers whose attention never looks further back (families with such layers
        override this); with TSB_KV_WINDOW_RING=1 those layers keep a ring of pages instead of the whole context."""
        return {}

    def make_kv_pool(self) -> PagedKV:
        pages_per_seq = (self.max_context + self.page_size - 1) // self.page_size
        ring_chunk = 0
        if (os.environ.get("TSB_KV_WINDOW_RING", "0") not in ("", "0") and self.cp_comm is None and self.pp_size == 1
                and self.kv_dtype != torch.float8_e4m3fn):
            ring_chunk = max(self.page_size, int(os.environ.get("TSB_KV_RING_CHUNK", "2048")))
        return PagedKV(self.kv_layer_shapes(), pages_per_seq * self.max_seqs, self.page_size, self.device,
                       self.kv_dtype, self.kv_donors(), max_seqs=max(self.max_seqs, 1),
                       window_layers=self.kv_window_layers() if ring_chunk else None, ring_chunk=ring_chunk)

    # ------------------------------------------------------------------ execution
    def forward_batch(self, batch: Batch, want_logits: bool = True) -> Optional[torch.Tensor]:
        """Run the packed batch; returns float32 logits ``[B, vocab]`` for the last token of
        every sequence (or ``None`` when ``want_logits`` is false: prefill chunks)."""
        raise NotImplementedError

    def recurrent_state_tensors(self) -> list:
        """The per-slot recurrent state tensors (first dimension = sequence slot) of models with linear-attention / SSM
        layers; empty for attention-only models.  A CUDA-graph capture snapshots them around its warm-up step."""
        return []

    def reset_recurrent_state(self, slot: int) -> None:
        """Zero per-sequence recurrent state (models with linear-attention / SSM layers)."""

    # ------------------------------------------------------------------ single-sequence API
    def _seq(self) -> SeqState:
        if self._default_seq is None:
            self._default_seq = self.kv.new_seq()
            self.reset_recurrent_state(self._default_seq.slot)
        return self._default_seq

    def new_sequence(self) -> SeqState:
        """A fresh sequence in the KV pool (recurrent state zeroed); raises OutOfPagesError when
        every one of the pool's ``max_seqs`` slots is in use."""
        s = self.kv.new_seq()
        self.reset_recurrent_state(s.slot)
        return s

    def free_sequence(self, seq: SeqState) -> None:
        self.__dict__.get("_steppers", {}).pop(seq.seq_id, None)
        if self._default_seq is seq:
            self._default_seq = None
        self.kv.free_seq(seq)

    def bind_sequence(self, seq: Optional[SeqState]) -> None:
        """Make ``seq`` the one the single-sequence API (forward / reset / truncate) acts on, so a
        host that keeps several chats resident switches between them without forwarding."""
        self._default_seq = seq

    @property
    def cache_length(self) -> int:
        return self._default_seq.length if self._default_seq is not None else 0

    def forward(self, tokens: Sequence[int], want_logits: bool = True) -> Optional[torch.Tensor]:
        """Append ``tokens`` to the default sequence and return the next-token logits
        (float32 ``[vocab]`` on the compute device).  IModelArchitecture.Forward."""
        self.poll_status()
        if len(tokens) == 1 and self._graph_forward_ok():
            with self.timer.phase("decode"):
                out = self._graph_stepper().step(tokens[0])
            if out is not None:
                return out if want_logits else None
        chunk = self.kv.ring_chunk
        if chunk and len(tokens) > chunk:               # window layers keep a ring of pages: prompts go in by chunks
            tokens = list(tokens)
            for i in range(0, len(tokens) - chunk, chunk):
                self.forward(tokens[i:i + chunk], want_logits=False)
            tokens = tokens[(len(tokens) - 1) // chunk * chunk:]
        batch = self.kv.build_batch([self._seq()], [list(tokens)])
        with self.timer.phase("decode" if len(tokens) == 1 else "prefill"):
            out = self.forward_batch(batch, want_logits)
        return out[0] if out is not None else None

    def _graph_forward_ok(self) -> bool:
        """Single-token ``forward`` replays a captured graph on one GPU (TSB_GRAPH_FORWARD=0 keeps it eager):
        not with tensor / pipeline parallel shards (their hosts drive the steps themselves), not for models
        with recurrent state, and not while multimodal embeddings wait to be injected."""
        if self.device.type != "cuda" or self.tp_size > 1 or self.pp_size > 1 or self._pending_embeddings:
            return False
        if not self.supports_kv_truncation:             # recurrent state: the capture's warm-up step would advance it
            return False
        if self.kv.ring:                                # the steppers rewrite block-table rows themselves (full table only)
            return False
        return os.environ.get("TSB_GRAPH_FORWARD", "1") != "0"

    def _graph_stepper(self):
        from ..runtime.engine import GraphStepper
        seq = self._seq()
        steppers = self.__dict__.setdefault("_steppers", {})
        st = steppers.get(seq.seq_id)
        if st is None or st.seq is not seq:
            if len(steppers) > 8:                       # sequences come and go (sessions): keep the table small
                steppers.clear()
            st = steppers[seq.seq_id] = GraphStepper(self, seq)
        return st

    @property
    def timer(self):
        """Per-phase device timer (enabled by ``TSB_PROFILE=1``; NVTX ranges by ``TSB_NVTX=1``)."""
        t = self.__dict__.get("_timer")
        if t is None:
            from ..runtime.profiling import PhaseTimer
            t = self.__dict__["_timer"] = PhaseTimer(self.device)
        return t

    def print_timing_stats(self, out=None) -> None:
        """Table of accumulated phase times (ModelBase.PrintTimingStats in the reference)."""
        import sys
        print(self.timer.table(), file=out or sys.stderr)

    def check_exchanges(self) -> None:
        """Raise a typed error if any in-kernel exchange of this model gave up waiting for a peer."""
        for name in ("_tpx", "_tpseq"):
            x = self.__dict__.get(name)
            for e in (x.values() if isinstance(x, dict) else [x]):
                if e is not None and hasattr(e, "check"):
                    e.check()

    # Status words of the bounded device-side waits.  A wait that ran out makes its kernel carry on with zeros and
    # leaves a code in a device word; nothing on the device stops.  The token loops therefore look at those words
    # themselves: every ``STATUS_POLL_EVERY`` calls of ``forward`` the words are copied to pinned host memory behind
    # the step (no synchronisation), and the copy made by an earlier call, long complete by then because the host
    # has read that call's logits since, is examined.  A non-zero word ends the request with ExchangeTimeoutError
    # (HTTP 500 on the front end; a follower process leaves its loop and exits).
    STATUS_POLL_EVERY = 16

    def status_sources(self):
        """``(name, int32 device tensor of one element)`` for every status word this model's kernels may set."""
        out = []
        if self.device.type != "cuda":
            return out
        from ..ops import kernels
        out.append(("tcgen05 GEMM pipeline", kernels.gemm_status(self.device)))
        x = self.__dict__.get("_tpx")
        if x:
            out.append(("tensor-parallel mailbox exchange", x.counters[4:5]))
        x = self.__dict__.get("_tpseq")
        if x:
            out.append(("sequence-parallel prefill exchange", x.local[8:9]))
        x = self.__dict__.get("_cpa")
        if x is not None:
            out.append(("context-parallel attention", x.local[4:5]))
        x = self.__dict__.get("_mega")
        if x:
            out.append(("fused decode step", x.status_word))
        return out

    def recover_exchanges(self) -> int:
        """Recovery after a bounded device wait gave up (``ExchangeTimeoutError``): fail the request, then call this on
        every rank at the same point.  It drops every in-kernel exchange of this model (mailboxes, sequence-parallel
        regions, the context-parallel ring, the fused decode step) together with their symmetric buffers, so that the
        next call that needs one sets it up afresh across the ranks; forgets the captured graphs, which point into the
        old buffers; clears the status words; and empties the KV pool's sequences (a step that gave up left rows of
        unknown content).  The weights stay where they are.  Returns the number of exchange objects closed."""
        closed = 0
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        # no rank unmaps or frees a buffer while another rank's kernels may still store into it: every rank has drained
        # its own device above, and nobody goes on before all of them have
        for comm in (self.comm, self.cp_comm):
            if comm is not None and getattr(comm, "size", 1) > 1:
                comm.barrier()
        for name in ("_tpx", "_tpseq", "_cpa", "_mega"):
            x = self.__dict__.pop(name, None)
            for e in (list(x.values()) if isinstance(x, dict) else [x]):
                if e is not None and e is not False and hasattr(e, "close"):
                    try:
                        e.close()
                    finally:
                        closed += 1
        self.__dict__.pop("_steppers", None)
        self.__dict__.pop("_status_poll", None)
        self.__dict__["_cp_ctx"] = None
        for _, word in self.status_sources():           # what is left: the GEMM pipeline's word
            word.zero_()
        if self._default_seq is not None:
            self.reset_kv_cache()
        return closed

    def raise_on_status(self, names, values) -> None:
        from ..parallel.errors import ExchangeTimeoutError
        for name, v in zip(names, values):
            if int(v):
                raise ExchangeTimeoutError(name, int(v))

    def poll_status(self, force: bool = False) -> None:
        """See the note above ``STATUS_POLL_EVERY``.  ``force`` synchronises and checks the words as they are now."""
        st = self.__dict__.setdefault("_status_poll", {"n": 0, "pending": None})
        if force or self.device.type != "cuda":
            src = self.status_sources()                 # host tensors (a test's stand-in) are read as they are
            if src:
                if self.device.type == "cuda":
                    torch.cuda.synchronize(self.device)
                self.raise_on_status([n for n, _ in src], [int(t.item()) for _, t in src])
            return
        pend = st["pending"]
        if pend is not None and pend[2].query():
            st["pending"] = None
            self.raise_on_status(pend[0], pend[1].tolist())
        st["n"] += 1
        if st["pending"] is None and st["n"] % self.STATUS_POLL_EVERY == 1:
            src = self.status_sources()
            if src:
                host = torch.empty(len(src), dtype=torch.int32).pin_memory()
                host.copy_(torch.cat([t.reshape(1) for _, t in src]), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                st["pending"] = ([n for n, _ in src], host, ev)

    def forward_refill(self, tokens: Sequence[int], chunk: int = 2048) -> torch.Tensor:
        """Chunked prefill: all chunks but the last skip the logits (Qwen3Model.cs:238
        ForwardRefill; chunk size policy TensorSharp.Server/ModelService.cs:791-801)."""
        tokens = list(tokens)
        out = None
        for i in range(0, len(tokens), chunk):
            last = i + chunk >= len(tokens)
            out = self.forward(tokens[i:i + chunk], want_logits=last)
        return out

    def reset_kv_cache(self) -> None:
        if self._default_seq is not None:
            self.kv.truncate(self._default_seq, 0)
            self.reset_recurrent_state(self._default_seq.slot)

    def truncate_kv_cache(self, n_tokens: int) -> None:
        """Keep the first ``n_tokens`` of the default sequence.  Keeping everything is always allowed (the second
        turn of a chat re-uses the whole cache: ModelBase.TruncateKVCache is a no-op there); a model with recurrent
        state refuses only a real shrink, which its state cannot follow."""
        seq = self._default_seq
        if seq is None or n_tokens >= seq.length:
            return
        if not self.supports_kv_truncation:
            raise RuntimeError(f"{type(self).__name__} cannot truncate its cache (recurrent state)")
        if not self.kv.can_truncate(seq, n_tokens):     # the window layers' ring has overwritten what the cut needs: start over
            self.reset_kv_cache()
            return
        self.kv.truncate(seq, n_tokens)

    def warm_up_kernels(self) -> None:
        """Run one short prefill and one decode step so lazy initialisation (cuBLAS handles,
        tensor maps, scratch buffers) is paid before the first request, then clear the cache
        (ModelBase.WarmUpKernels in the reference)."""
        n = max(1, min(8, self.max_context - 2))
        tok = min(self.cfg.vocab - 1, 100)
        self.forward([tok] * n)
        self.forward([tok])
        self.reset_kv_cache()
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def close(self) -> None:
        self.gguf.close()

    # ------------------------------------------------------------------ factory
    @staticmethod
    def create(path: str, device="cuda", **kw) -> "ModelBase":
        """Open ``path`` and instantiate the graph for its ``general.architecture``."""
        from . import _load_all  # noqa: F401  (registers every architecture)
        with GGUFFile(path) as g:
            arch = g.get_str("general.architecture", "")
        if arch not in _REGISTRY:
            raise ValueError(f"unsupported architecture {arch!r}; supported: {supported_architectures()}")
        return _REGISTRY[arch](path, device, **kw)
