"""Flag parsing for the command-line tool.

Parity: TensorSharp.Cli/Program.cs:60-150 — the same flags with the same defaults
(``--max-tokens`` 100, greedy sampling unless sampling flags are given, benchmark 32 prefill /
64 decode / 1 run, chunked-prefill correctness 1500 / 8, KV-cache bench 4 turns) and
Logging/CliLoggingSetup (``--log-level --log-dir --log-file off --log-console off``).  The
default backend is ``b200`` (falls back to ``cpu`` without a CUDA device); the reference's
backend names are accepted as aliases.  ``--tp N`` is this build's tensor-parallel switch and
``--batch-size N`` decodes up to N requests of ``--input-jsonl`` together.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from ..runtime.sampling import SamplingConfig

USAGE = ("Usage: python -m tensorsharp_b200.cli --model <path.gguf> [--input <input.txt>] "
         "[--input-jsonl <requests.jsonl>] [--multi-turn-jsonl <turns.jsonl>] [--image <image.png>] [--audio <a.wav>] "
         "[--video <v.mp4>] [--mmproj <path.gguf>] [--output <output.txt>] [--max-tokens N] [--test] "
         "[--backend b200|cpu] [--interactive] [--system <text>] [--system-file <path>] "
         "[--temperature F] [--top-k N] [--top-p F] [--min-p F] [--repeat-penalty F] [--presence-penalty F] "
         "[--frequency-penalty F] [--seed N] [--stop <text>] [--think] [--tools <tools.json>] [--dump-prompt] "
         "[--benchmark [--bench-prefill N] [--bench-decode N] [--bench-runs N] [--bench-chunked]] "
         "[--test-chunked-prefill [--correct-prefill N] [--correct-decode N]] [--bench-kvcache [--bench-kv-turns N]] "
         "[--test-templates <dir>] [--log-level info|debug|trace] [--log-dir <path>] [--log-file off] [--log-console off] "
         "[--batch-size N] [--max-context N] [--kv-dtype bf16|fp8] [--tp N | --pp N | --cp N  (one process per GPU: python -m torch.distributed.run "
         "--nproc-per-node N -m tensorsharp_b200.cli ...)]")


@dataclass
class CliOptions:
    model: Optional[str] = None
    input_file: Optional[str] = None
    input_jsonl: Optional[str] = None
    output_file: Optional[str] = None
    image: Optional[str] = None
    audio: Optional[str] = None
    video: Optional[str] = None
    mmproj: Optional[str] = None
    max_tokens: int = 100
    run_test: bool = False
    backend: str = "b200"
    test_templates_dir: Optional[str] = None
    multi_turn_jsonl: Optional[str] = None
    think: bool = False
    tools_file: Optional[str] = None
    dump_prompt: bool = False
    benchmark: bool = False
    bench_prefill: int = 32
    bench_decode: int = 64
    bench_runs: int = 1
    bench_chunked: bool = False
    test_chunked_prefill: bool = False
    correct_prefill: int = 1500
    correct_decode: int = 8
    bench_kvcache: bool = False
    bench_kv_turns: int = 4
    interactive: bool = False
    system: Optional[str] = None
    sampling: SamplingConfig = field(default_factory=SamplingConfig.greedy)
    log_level: Optional[str] = None
    log_dir: Optional[str] = None
    log_file: bool = True
    log_console: bool = True
    tp: int = 1
    pp: int = 1                       # pipeline stages (one process per stage)
    cp: int = 1                       # context-parallel ranks: long prompts are dealt to them slice by slice
    batch_size: int = 1               # JSONL mode: requests decoded together (continuous batching)
    max_context: Optional[int] = None
    kv_dtype: Optional[str] = None          # "bf16" or "fp8" (exported as TSB_KV_DTYPE before the model loads)
    unknown: List[str] = field(default_factory=list)


_STR = {"--model": "model", "--input": "input_file", "--input-jsonl": "input_jsonl", "--output": "output_file",
        "--image": "image", "--audio": "audio", "--video": "video", "--mmproj": "mmproj",
        "--test-templates": "test_templates_dir", "--tools": "tools_file", "--multi-turn-jsonl": "multi_turn_jsonl",
        "--system": "system", "--log-level": "log_level", "--log-dir": "log_dir"}
_INT = {"--max-tokens": "max_tokens", "--bench-prefill": "bench_prefill", "--bench-decode": "bench_decode",
        "--bench-runs": "bench_runs", "--correct-prefill": "correct_prefill", "--correct-decode": "correct_decode",
        "--bench-kv-turns": "bench_kv_turns", "--tp": "tp", "--max-context": "max_context",
        "--batch-size": "batch_size", "--pp": "pp", "--cp": "cp"}
_BOOL = {"--test": "run_test", "--think": "think", "--dump-prompt": "dump_prompt", "--benchmark": "benchmark",
         "--bench-chunked": "bench_chunked", "--test-chunked-prefill": "test_chunked_prefill",
         "--bench-kvcache": "bench_kvcache", "--interactive": "interactive", "--chat": "interactive"}
_SAMPLING = {"--temperature": ("temperature", float), "--top-k": ("top_k", int), "--top-p": ("top_p", float),
             "--min-p": ("min_p", float), "--repeat-penalty": ("repetition_penalty", float),
             "--presence-penalty": ("presence_penalty", float), "--frequency-penalty": ("frequency_penalty", float),
             "--seed": ("seed", int)}


def kv_dtype_name(v: str) -> str:
    """``--kv-dtype``: ``bf16`` (default pages) or ``fp8`` (e4m3 bytes, half the cache)."""
    n = {"bf16": "bf16", "bfloat16": "bf16", "fp8": "fp8", "e4m3": "fp8", "float8_e4m3fn": "fp8"}.get(v.strip().lower())
    if n is None:
        raise ValueError(f"Invalid value for --kv-dtype: '{v}' (bf16 or fp8).")
    return n


def parse_cli_args(args: Sequence[str]) -> CliOptions:
    o = CliOptions()
    i = 0

    def value(flag: str) -> str:
        nonlocal i
        if i + 1 >= len(args):
            raise ValueError(f"Missing value for option '{flag}'.")
        i += 1
        return args[i]

    while i < len(args):
        a = args[i]
        if a in _STR:
            setattr(o, _STR[a], value(a))
        elif a in _INT:
            v = value(a)
            try:
                setattr(o, _INT[a], int(v))
            except ValueError:
                raise ValueError(f"Invalid value for {a}: '{v}'.") from None
        elif a in _BOOL:
            setattr(o, _BOOL[a], True)
        elif a in _SAMPLING:
            name, conv = _SAMPLING[a]
            v = value(a)
            try:
                setattr(o.sampling, name, conv(v))
            except ValueError:
                raise ValueError(f"Invalid value for {a}: '{v}'.") from None
        elif a == "--stop":
            o.sampling.stop_sequences = (o.sampling.stop_sequences or []) + [value(a)]
        elif a == "--backend":
            o.backend = value(a).lower()
        elif a == "--kv-dtype":
            o.kv_dtype = kv_dtype_name(value(a))
        elif a == "--system-file":
            with open(value(a), "r", encoding="utf-8") as f:
                o.system = f.read()
        elif a == "--log-file":
            o.log_file = value(a).lower() not in ("off", "0", "false", "no")
        elif a == "--log-console":
            o.log_console = value(a).lower() not in ("off", "0", "false", "no")
        else:
            o.unknown.append(a)
        i += 1
    return o
