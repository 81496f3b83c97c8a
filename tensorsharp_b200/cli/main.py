"""Command-line modes.

Parity: TensorSharp.Cli/Program.cs — MainCore :60 (mode dispatch order: --test-templates,
--test, --benchmark, --test-chunked-prefill, --bench-kvcache, --multi-turn-jsonl, --input-jsonl,
--interactive, else one-shot with --input / --image / --audio / --video / --dump-prompt),
RunMultiTurnTest :468, RunJsonlBatch :660 (result fields ``id output tokens_generated prefill_ms
total_ms tokens_per_second``), RunInference :892, FormatParsedResult :1426, RunBenchmark :1515,
RunChunkedPrefillCorrectness :1635, RunKvCacheBenchmark :1706, TestChatTemplates :2001.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Dict, List, Optional, Sequence

from ..runtime import media
from ..runtime.chat import ChatMessage, ToolFunction, ToolParameter, dotnet_json
from ..runtime.chat_template import build_jinja_context, render_hardcoded
from ..runtime.engine import run_benchmark, synthetic_prompt
from ..runtime.jinja import Jinja2Template
from ..runtime.kv_cache import KVCache, ReusePlan, ReusePlanKind
from ..runtime.logging import Ev, NULL_LOGGER, setup_file_logging
from ..runtime.output_parser import ParsedOutput, create_output_parser
from ..runtime.prompt_renderer import GgufPromptRenderer, KVCachePromptRenderer
from ..runtime.sampling import SamplingConfig, TokenSampler
from .args import USAGE, CliOptions, parse_cli_args

PROMPT_RENDERER = GgufPromptRenderer()

AUTO_MMPROJ = {"gemma3": "mmproj-gemma3-4b-f16.gguf", "mistral3": "mistral3-mmproj.gguf",
               "gemma4": "gemma-4-mmproj-F16.gguf", "qwen35": "Qwen3.5-mmproj-F16.gguf",
               "qwen35moe": "Qwen3.5-mmproj-F16.gguf", "qwen3next": "Qwen3.5-mmproj-F16.gguf"}

KV_BENCH_TURNS = (
    "Give me a short overview of how a transformer language model produces the next token.",
    "Now explain what the key/value cache stores and why it makes decoding cheaper.",
    "How does that change when the conversation has several turns?",
    "Summarise the three answers above in two sentences.",
    "Which of those points matters most for latency, and why?",
    "Rewrite the summary for a reader who has never seen a neural network.",
)


class Console:
    """Where user-facing text goes (tests capture it)."""

    def __init__(self, out=None, err=None):
        self.out, self.err = out or sys.stdout, err or sys.stderr

    def print(self, text: str = "", end: str = "\n") -> None:
        self.out.write(text + end)
        self.out.flush()

    def error(self, text: str) -> None:
        self.err.write(text + "\n")
        self.err.flush()


def resolve_device(backend: str) -> str:
    from ..server.options import canonicalize_backend
    b = canonicalize_backend(backend)
    if b not in ("b200", "cpu"):
        raise ValueError(f"Unknown backend '{backend}'. Use: b200, cpu (aliases: cuda, ggml_cuda, ggml_cpu)")
    if b == "b200":
        import torch
        if not torch.cuda.is_available():
            return "cpu"
        return "cuda"
    return "cpu"


def load_tools(path: str) -> List[ToolFunction]:
    """Tool definitions: a list of ``{name, description, parameters: {arg: {type, description,
    enum}}, required}`` objects (keys case-insensitive), or the OpenAI ``{"type": "function",
    "function": {...}}`` shape."""
    with open(path, "r", encoding="utf-8") as f:
        data = json.load(f)
    out = []
    for item in data:
        low = {k.lower(): v for k, v in item.items()}
        if isinstance(low.get("function"), dict):
            from ..server.parsers import _parse_function
            out.append(_parse_function(low["function"]))
            continue
        tf = ToolFunction(name=low.get("name", ""), description=low.get("description"))
        params = low.get("parameters")
        if isinstance(params, dict):
            tf.parameters = {}
            for name, p in params.items():
                pl = {k.lower(): v for k, v in (p or {}).items()}
                tf.parameters[name] = ToolParameter(pl.get("type"), pl.get("description"), pl.get("enum"))
        tf.required = low.get("required")
        out.append(tf)
    return out


def format_parsed_result(parsed: ParsedOutput, show_thinking: bool) -> str:
    out = []
    if show_thinking and parsed.thinking:
        out += ["\n--- Thinking ---\n", parsed.thinking.strip(), "\n--- End Thinking ---\n\n"]
    if parsed.content:
        out.append(parsed.content)
    if parsed.tool_calls:
        out.append("\n--- Tool Calls ---\n")
        for tc in parsed.tool_calls:
            out.append(f"  Function: {tc.name}\n  Arguments: {dotnet_json(tc.arguments, indented=True)}\n\n")
        out.append("--- End Tool Calls ---\n")
    return "".join(out)


def describe_plan(plan: ReusePlan, total: int) -> str:
    if plan.kind == ReusePlanKind.EXACT_MATCH:
        return f"Exact match: reusing all {total} cached tokens (saved 100%)"
    if plan.kind == ReusePlanKind.PARTIAL_REUSE:
        return (f"Partial reuse: keeping {plan.reused_prefix_length}/{total} tokens, forwarding {plan.tokens_to_forward} "
                f"new (saved {100.0 * plan.reused_prefix_length / total:.0f}%)")
    return f"Full reset: forwarding {plan.tokens_to_forward} tokens"


def apply_reuse_plan(model, kv: KVCache, plan: ReusePlan, tokens: List[int]):
    if plan.kind == ReusePlanKind.EXACT_MATCH:
        return plan.cached_logits
    if plan.kind == ReusePlanKind.PARTIAL_REUSE:
        n = plan.reused_prefix_length
        model.truncate_kv_cache(n)
        kv.truncate_to(n)
        suffix = list(tokens[n:n + plan.tokens_to_forward])
        logits = model.forward_refill(suffix)
        kv.record_append(suffix, logits)
        return logits
    model.reset_kv_cache()
    kv.reset()
    logits = model.forward(list(tokens))
    kv.record_append(list(tokens), logits)
    return logits


def _sync(model) -> None:
    if getattr(model.device, "type", str(model.device)) == "cuda":
        import torch
        torch.cuda.synchronize()


def sample_loop(model, logits, max_tokens: int, cfg: SamplingConfig, kv: Optional[KVCache] = None, on_piece=None):
    """Token loop shared by the batch modes; returns ``(token ids, text, stopped_on_stop_sequence)``."""
    tok = model.tokenizer
    sampler = TokenSampler(cfg)
    ids: List[int] = []
    text = ""
    for _ in range(max_tokens):
        nxt = sampler.sample(logits, ids)
        if tok.is_eos(nxt):
            break
        ids.append(nxt)
        new_text = tok.decode(ids)
        if on_piece is not None and len(new_text) > len(text) and not new_text.endswith("�"):
            on_piece(new_text[len(text):])
        text = new_text
        if cfg.stop_sequences:
            trimmed, stop = sampler.check_stop_sequences(text)
            if stop:
                return ids, trimmed, True
        logits = model.forward([nxt])
        if kv is not None:
            kv.record_append(nxt, logits)
    return ids, text, False


# ---------------------------------------------------------------------------- modes
def run_inference(model, text: str, image_paths, max_tokens: int, audio_paths=None, is_video=False,
                  sampling: Optional[SamplingConfig] = None, think=False, tools=None, log=NULL_LOGGER) -> str:
    arch = model.arch
    messages = [ChatMessage(role="user", content=text, image_paths=image_paths, audio_paths=audio_paths, is_video=is_video)]
    rendered = PROMPT_RENDERER.render(model.cfg.chat_template, messages, True, arch, tools, think)
    tokens = model.tokenizer.encode(rendered, add_special=True)
    mm = getattr(model, "multimodal", None)
    if mm is not None:
        tokens = mm.process_prompt_tokens(messages, tokens)
        mm.queue_prompt_embeddings(0)
    model.reset_kv_cache()
    t0 = time.perf_counter()
    logits = model.forward(tokens)
    _sync(model)
    prefill_ms = (time.perf_counter() - t0) * 1e3
    t1 = time.perf_counter()
    ids, raw, _ = sample_loop(model, logits, max_tokens, sampling or SamplingConfig.greedy())
    decode_ms = (time.perf_counter() - t1) * 1e3
    log.info(Ev.ChatCompleted, "cli.inference promptTokens={PromptTokens} prefillMs={PrefillMs:.1f} tokens={Tokens} "
             "decodeMs={DecodeMs:.1f} tokPerSec={TokensPerSec:.2f}", PromptTokens=len(tokens), PrefillMs=prefill_ms,
             Tokens=len(ids), DecodeMs=decode_ms, TokensPerSec=len(ids) / (decode_ms / 1e3) if decode_ms > 0 else 0.0)
    parser = create_output_parser(arch)
    parser.init(think, tools)
    return format_parsed_result(parser.add(raw, True), think)


def run_benchmark_mode(model, o: CliOptions, con: Console, log) -> Dict[str, Any]:
    log.info(Ev.CliBenchmark, "inference benchmark starting: prefillTokens={PrefillTokens} decodeTokens={DecodeTokens} "
             "runs={Runs} chunked={Chunked}", PrefillTokens=o.bench_prefill, DecodeTokens=o.bench_decode, Runs=o.bench_runs,
             Chunked=o.bench_chunked)
    results = run_benchmark(model, o.bench_prefill, o.bench_decode, o.bench_runs, o.bench_chunked)
    for i, r in enumerate(results):
        line = (f"benchmark run {i + 1}/{len(results)}: prefillMs={r.prefill_ms:.0f} prefillTps={r.prefill_tps:.1f} "
                f"decodeMs={r.decode_ms:.0f} decodeTps={r.decode_tps:.1f} msPerTok={r.ms_per_token:.1f}")
        con.print(line)
        log.info(Ev.CliBenchmark, line)
    bp = min(results, key=lambda r: r.prefill_ms)
    bd = min(results, key=lambda r: r.decode_ms)
    summary = {"bestPrefillMs": bp.prefill_ms, "bestPrefillTps": bp.prefill_tps, "bestDecodeMs": bd.decode_ms,
               "bestDecodeTps": bd.decode_tps, "bestDecodeMsPerTok": bd.ms_per_token,
               "avgPrefillTps": sum(r.prefill_tps for r in results) / len(results),
               "avgDecodeTps": sum(r.decode_tps for r in results) / len(results)}
    line = ("benchmark summary: bestPrefillMs={bestPrefillMs:.0f} bestPrefillTps={bestPrefillTps:.1f} bestDecodeMs="
            "{bestDecodeMs:.0f} bestDecodeTps={bestDecodeTps:.1f} bestDecodeMsPerTok={bestDecodeMsPerTok:.2f} "
            "avgPrefillTps={avgPrefillTps:.1f} avgDecodeTps={avgDecodeTps:.1f}").format(**summary)
    con.print(line)
    log.info(Ev.CliBenchmark, line)
    return summary


def run_chunked_prefill_correctness(model, prefill_tokens: int, decode_tokens: int, con: Console, log) -> bool:
    """Greedy-decode after a one-shot prefill and after a chunked one; the ids must agree."""
    ids = synthetic_prompt(prefill_tokens, model.cfg.vocab)

    def decode_with(prefill):
        model.reset_kv_cache()
        logits = prefill(ids)
        out = []
        nxt = int(logits.argmax())
        for _ in range(decode_tokens):
            out.append(nxt)
            nxt = int(model.forward([nxt]).argmax())
        return out
    a = decode_with(lambda t: model.forward(t))
    b = decode_with(lambda t: model.forward_refill(t, max(64, min(2048, (prefill_tokens + 3) // 4))))
    matches = 0
    for x, y in zip(a, b):
        if x != y:
            break
        matches += 1
    ok = matches == decode_tokens
    line = (f"chunked prefill correctness: matched {matches}/{decode_tokens} decode tokens -> {'PASS' if ok else 'FAIL'} "
            f"forward=[{','.join(map(str, a))}] refill=[{','.join(map(str, b))}]")
    con.print(line)
    log.info(Ev.CliBenchmark, line)
    return ok


def _bench_pass(model, turns: Sequence[str], max_tokens: int, cfg: SamplingConfig, think: bool, use_cache: bool, log):
    arch = model.arch
    model.reset_kv_cache()
    kv = KVCache()
    renderer = KVCachePromptRenderer(PROMPT_RENDERER)
    history: List[ChatMessage] = []
    prefill_ms, prompt_tokens = [], []
    for turn, user in enumerate(turns):
        history.append(ChatMessage(role="user", content=user))
        tokens = renderer.render_to_tokens(model.tokenizer, model.cfg.chat_template, history, arch, True, None, think)
        prompt_tokens.append(len(tokens))
        if not use_cache:
            model.reset_kv_cache()
            kv.reset()
        _sync(model)
        t0 = time.perf_counter()
        plan = kv.plan_reuse(tokens, model.supports_kv_truncation)
        logits = apply_reuse_plan(model, kv, plan, tokens)
        _sync(model)
        prefill_ms.append((time.perf_counter() - t0) * 1e3)
        ids, raw, _ = sample_loop(model, logits, max_tokens, cfg, kv)
        log.info(Ev.CliBenchmark, "kv bench turn {Turn}: promptTokens={PromptTokens} prefillMs={PrefillMs:.1f} generated="
                 "{Generated} plan={Plan}", Turn=turn + 1, PromptTokens=len(tokens), PrefillMs=prefill_ms[-1],
                 Generated=len(ids), Plan=plan.kind.value)
        parser = create_output_parser(arch)
        parser.init(think, None)
        parsed = parser.add(raw, True)
        history.append(ChatMessage(role="assistant", content=parsed.content or "", thinking=parsed.thinking or "",
                                   raw_output_tokens=ids))
    return prefill_ms, prompt_tokens


def run_kv_cache_benchmark(model, turns: int, max_tokens: int, cfg: SamplingConfig, think: bool, con: Console, log):
    """Same multi-turn conversation with and without KV reuse; reports per-turn prefill time."""
    n = min(max(2, turns), len(KV_BENCH_TURNS))
    cached, ptoks = _bench_pass(model, KV_BENCH_TURNS[:n], max_tokens, cfg, think, True, log)
    plain, _ = _bench_pass(model, KV_BENCH_TURNS[:n], max_tokens, cfg, think, False, log)
    rows = []
    for i in range(n):
        speed = plain[i] / cached[i] if cached[i] > 0 else 0.0
        rows.append({"turn": i + 1, "promptTokens": ptoks[i], "cachedMs": cached[i], "noCacheMs": plain[i], "speedup": speed})
        line = (f"kv bench turn {i + 1}: promptTokens={ptoks[i]} cachedPrefillMs={cached[i]:.1f} "
                f"noCachePrefillMs={plain[i]:.1f} speedup={speed:.2f}x")
        con.print(line)
        log.info(Ev.CliBenchmark, line)
    ac, an = sum(cached[1:]) / (n - 1), sum(plain[1:]) / (n - 1)
    line = (f"kv bench summary over turns 2..{n}: avgCachedPrefillMs={ac:.1f} avgNoCachePrefillMs={an:.1f} "
            f"avgSpeedup={an / ac if ac > 0 else 0.0:.2f}x")
    con.print(line)
    log.info(Ev.CliBenchmark, line)
    return rows


def run_multi_turn_test(model, path: str, max_tokens: int, cfg: SamplingConfig, think: bool, con: Console, log) -> int:
    """Each JSONL line is a user turn: ``{"content": ..., "max_tokens": N, "force_reset": bool}`` or
    plain text.  Reports the KV reuse plan of every turn."""
    if not os.path.isfile(path):
        log.error(Ev.CliFailed, "Multi-turn jsonl not found: {File}", File=path)
        con.error(f"Multi-turn jsonl not found: {path}")
        return 1
    with open(path, "r", encoding="utf-8") as f:
        lines = [l.strip() for l in f.read().splitlines()]
    history: List[ChatMessage] = []
    kv = KVCache()
    renderer = KVCachePromptRenderer(PROMPT_RENDERER)
    arch = model.arch
    for turn, line in enumerate(lines):
        if not line:
            continue
        user, turn_max, force_reset = line, max_tokens, False
        try:
            d = json.loads(line)
            if isinstance(d, dict):
                user = d.get("content", line)
                turn_max = int(d.get("max_tokens", max_tokens))
                force_reset = bool(d.get("force_reset", False))
        except ValueError:
            pass
        history.append(ChatMessage(role="user", content=user))
        if force_reset:
            kv.reset()
            model.reset_kv_cache()
        tokens = renderer.render_to_tokens(model.tokenizer, model.cfg.chat_template, history, arch, True, None, think)
        t0 = time.perf_counter()
        plan = kv.plan_reuse(tokens, model.supports_kv_truncation)
        logits = apply_reuse_plan(model, kv, plan, tokens)
        _sync(model)
        prefill_ms = (time.perf_counter() - t0) * 1e3
        t1 = time.perf_counter()
        ids, raw, _ = sample_loop(model, logits, turn_max, cfg, kv)
        decode_ms = (time.perf_counter() - t1) * 1e3
        parser = create_output_parser(arch)
        parser.init(think, None)
        parsed = parser.add(raw, True)
        con.print(f"[turn {turn + 1}] promptTokens={len(tokens)} plan={plan.kind.value} prefillMs={prefill_ms:.1f} "
                  f"{describe_plan(plan, len(tokens))}")
        con.print(f"[turn {turn + 1}] tokens={len(ids)} decodeMs={decode_ms:.0f} content={parsed.content or ''!r}")
        log.info(Ev.KvCacheReusePlan, "kv plan={Plan} prefillMs={PrefillMs:.1f} description={Description}",
                 Plan=plan.kind.value, PrefillMs=prefill_ms, Description=describe_plan(plan, len(tokens)))
        if "<unused" in raw:
            log.error(Ev.ChatFailed, "multi-turn output contains <unused> tokens; first 500 chars: {RawPreview}", RawPreview=raw[:500])
            return 1
        history.append(ChatMessage(role="assistant", content=parsed.content or "", thinking=parsed.thinking or "",
                                   raw_output_tokens=ids))
    log.info(Ev.CliCompleted, "multi-turn test completed: {Turns} turns", Turns=len(history) // 2)
    return 0


def parse_batch_messages(root: Dict[str, Any]) -> List[ChatMessage]:
    out: List[ChatMessage] = []
    if isinstance(root.get("messages"), list):
        for m in root["messages"]:
            cm = ChatMessage(role=m.get("role", "user"), content=m.get("content", ""))
            if isinstance(m.get("images"), list):
                cm.image_paths = list(m["images"])
            if isinstance(m.get("audios"), list):
                cm.audio_paths = list(m["audios"])
            if "is_video" in m:
                cm.is_video = bool(m["is_video"])
            out.append(cm)
    elif "prompt" in root:
        out.append(ChatMessage(role="user", content=root["prompt"]))
    return out


def parse_batch_sampling(root: Dict[str, Any], fallback: SamplingConfig) -> SamplingConfig:
    cfg = fallback.clone()
    any_set = False
    for key, attr, conv in (("temperature", "temperature", float), ("top_k", "top_k", int), ("top_p", "top_p", float),
                            ("min_p", "min_p", float), ("repetition_penalty", "repetition_penalty", float),
                            ("presence_penalty", "presence_penalty", float),
                            ("frequency_penalty", "frequency_penalty", float), ("seed", "seed", int)):
        if key in root:
            setattr(cfg, attr, conv(root[key]))
            any_set = True
    if isinstance(root.get("stop"), list):
        cfg.stop_sequences = [s for s in root["stop"] if isinstance(s, str)]
        any_set = True
    return cfg if any_set else fallback


def run_jsonl_batch_concurrent(model, lines: List[str], default_max_tokens: int, default_sampling: SamplingConfig,
                               think: bool, batch_size: int, log) -> List[str]:
    """``--batch-size N``: the requests of the file share decode steps, up to N at a time (text-only
    requests; one with attachments falls back to a turn of its own).  Result lines keep the file's order
    and the sequential mode's fields."""
    from ..runtime.batching import ContinuousBatcher, GenRequest
    slots: List[Any] = []                       # per input line: a result string, or a GenRequest
    for idx, line in enumerate(lines):
        line = line.strip()
        if not line:
            continue
        try:
            root = json.loads(line)
            if not isinstance(root, dict):
                raise ValueError("request must be a JSON object")
        except ValueError as e:
            slots.append(dotnet_json({"line": idx + 1, "error": f"Invalid JSON: {e}"}))
            continue
        rid = root.get("id") or f"request_{idx + 1}"
        try:
            messages = parse_batch_messages(root)
            if any(m.image_paths or m.audio_paths for m in messages):
                raise ValueError("attachments are not supported with --batch-size > 1")
            cfg = parse_batch_sampling(root, default_sampling)
            req_think = think or root.get("enable_thinking") is True
            rendered = PROMPT_RENDERER.render(model.cfg.chat_template, messages, True, model.arch, None, req_think)
            tokens = model.tokenizer.encode(rendered, add_special=True)
            slots.append(GenRequest(tokens, int(root.get("max_tokens", default_max_tokens)), cfg, tag=rid))
        except Exception as e:
            log.error(Ev.CliFailed, "batch request {Index} id={Id} failed: {Error}", exc=e, Index=idx + 1, Id=rid, Error=str(e))
            slots.append(dotnet_json({"id": rid, "error": str(e)}))
    eng = ContinuousBatcher(model, batch_size)
    model.reset_kv_cache()
    eng.run([s for s in slots if isinstance(s, GenRequest)])
    log.info(Ev.CliBatchProgress, "continuous batching: {Steps} decode steps, mean batch {Mean:.2f}", Steps=eng.steps,
             Mean=eng.step_rows / max(1, eng.steps))
    out: List[str] = []
    for s in slots:
        if not isinstance(s, GenRequest):
            out.append(s)
        elif s.error is not None:
            out.append(dotnet_json({"id": s.tag, "error": s.error}))
        else:
            out.append(dotnet_json({"id": s.tag, "output": s.text, "tokens_generated": len(s.ids),
                                    "prefill_ms": round(s.prefill_ms, 2), "total_ms": round(s.total_ms, 2),
                                    "tokens_per_second": round(len(s.ids) / (s.total_ms / 1e3), 2) if s.total_ms > 0 else 0.0}))
    return out


def run_jsonl_batch(model, path: str, output_file: Optional[str], default_max_tokens: int, default_sampling: SamplingConfig,
                    think: bool, con: Console, log, batch_size: int = 1) -> int:
    if not os.path.isfile(path):
        log.error(Ev.CliFailed, "Input JSONL not found: {File}", File=path)
        con.error(f"Input JSONL not found: {path}")
        return 1
    with open(path, "r", encoding="utf-8") as f:
        lines = f.read().splitlines()
    if batch_size > 1:
        t_all = time.perf_counter()
        results = run_jsonl_batch_concurrent(model, lines, default_max_tokens, default_sampling, think, batch_size, log)
        log.info(Ev.CliCompleted, "batch completed: {Completed}/{Total} in {Seconds:.1f}s",
                 Completed=sum('"error"' not in r for r in results), Total=len(lines), Seconds=time.perf_counter() - t_all)
        return _emit_jsonl_results(results, output_file, con)
    results: List[str] = []
    done = 0
    t_all = time.perf_counter()
    for idx, line in enumerate(lines):
        line = line.strip()
        if not line:
            continue
        try:
            root = json.loads(line)
            if not isinstance(root, dict):
                raise ValueError("request must be a JSON object")
        except ValueError as e:
            results.append(dotnet_json({"line": idx + 1, "error": f"Invalid JSON: {e}"}))
            continue
        rid = root.get("id") or f"request_{idx + 1}"
        log.info(Ev.CliBatchProgress, "batch request {Index}/{Total} id={Id}", Index=idx + 1, Total=len(lines), Id=rid)
        try:
            messages = parse_batch_messages(root)
            max_tokens = int(root.get("max_tokens", default_max_tokens))
            cfg = parse_batch_sampling(root, default_sampling)
            req_think = think or root.get("enable_thinking") is True
            model.reset_kv_cache()
            rendered = PROMPT_RENDERER.render(model.cfg.chat_template, messages, True, model.arch, None, req_think)
            tokens = model.tokenizer.encode(rendered, add_special=True)
            mm = getattr(model, "multimodal", None)
            if mm is not None:
                tokens = mm.process_prompt_tokens(messages, tokens)
                mm.queue_prompt_embeddings(0)
            t0 = time.perf_counter()
            logits = model.forward(tokens)
            _sync(model)
            prefill_ms = (time.perf_counter() - t0) * 1e3
            ids, text, _ = sample_loop(model, logits, max_tokens, cfg)
            total_ms = (time.perf_counter() - t0) * 1e3
            results.append(dotnet_json({"id": rid, "output": text, "tokens_generated": len(ids),
                                        "prefill_ms": round(prefill_ms, 2), "total_ms": round(total_ms, 2),
                                        "tokens_per_second": round(len(ids) / (total_ms / 1e3), 2) if total_ms > 0 else 0.0}))
            done += 1
        except Exception as e:                                  # one bad request must not end the batch
            log.error(Ev.CliFailed, "batch request {Index} id={Id} failed: {Error}", exc=e, Index=idx + 1, Id=rid, Error=str(e))
            results.append(dotnet_json({"id": rid, "error": str(e)}))
            recover_if_exchange_failed(model, e, log)
    log.info(Ev.CliCompleted, "batch completed: {Completed}/{Total} in {Seconds:.1f}s", Completed=done, Total=len(lines),
             Seconds=time.perf_counter() - t_all)
    return _emit_jsonl_results(results, output_file, con)


def recover_if_exchange_failed(model, error, log) -> bool:
    """A bounded device-side wait that gave up ends a request with ``ExchangeTimeoutError``; the requests that follow
    need the exchanges rebuilt and the cache emptied (ModelBase.recover_exchanges; the weights stay loaded)."""
    from ..parallel.errors import ExchangeTimeoutError
    if not isinstance(error, ExchangeTimeoutError) or not hasattr(model, "recover_exchanges"):
        return False
    closed = model.recover_exchanges()
    log.warning(Ev.CliFailed, "exchange failure: {Closed} exchange objects dropped, they are rebuilt on next use", Closed=closed)
    return True


def _emit_jsonl_results(results: List[str], output_file: Optional[str], con: Console) -> int:
    if output_file:
        with open(output_file, "w", encoding="utf-8") as f:
            f.write("\n".join(results) + "\n")
        con.print(f"Results written to {output_file}")
    else:
        con.print("\n=== Results (JSONL) ===")
        for r in results:
            con.print(r)
    return 0


def test_chat_templates(model_dir: str, con: Console, log) -> Dict[str, int]:
    """For every GGUF in the directory, render three conversations with the file's Jinja template
    and with the built-in renderer of its architecture, and compare."""
    from ..gguf.reader import GGUFFile
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".gguf") and "mmproj" not in f.lower()) \
        if os.path.isdir(model_dir) else []
    counts = {"passed": 0, "failed": 0, "skipped": 0, "total": len(files)}
    scenarios = (
        ("single-turn", [ChatMessage(role="user", content="What is 1+1?")]),
        ("multi-turn", [ChatMessage(role="user", content="Hello!"),
                        ChatMessage(role="assistant", content="Hi there! How can I help?"),
                        ChatMessage(role="user", content="What is the capital of France?")]),
        ("with-system", [ChatMessage(role="system", content="You are a helpful assistant."),
                         ChatMessage(role="user", content="Tell me a joke.")]))
    for name in files:
        try:
            with GGUFFile(os.path.join(model_dir, name)) as g:
                arch = g.get_str("general.architecture", "")
                template = g.get_str("tokenizer.chat_template")
            if template is None:
                con.print(f"{name}: SKIP (no chat template in GGUF metadata)")
                counts["skipped"] += 1
                continue
            ok = True
            for sname, msgs in scenarios:
                try:
                    j2 = Jinja2Template(template).render(build_jinja_context(msgs, True, arch)).strip()
                except Exception as e:
                    con.print(f"{name} [{sname}] FAIL Jinja2 error: {e}")
                    ok = False
                    continue
                hc = (render_hardcoded(msgs, True, arch) or "").strip()
                if j2 == hc:
                    con.print(f"{name} [{sname}] PASS chars={len(j2)}")
                else:
                    con.print(f"{name} [{sname}] MISMATCH jinja2Chars={len(j2)} hardcodedChars={len(hc)} "
                              f"jinja2Sample={j2[:120]!r} hardcodedSample={hc[:120]!r}")
                    ok = False
            counts["passed" if ok else "failed"] += 1
        except Exception as e:
            con.print(f"{name} ERROR: {e}")
            counts["failed"] += 1
    line = "chat template scan results: passed={passed} failed={failed} skipped={skipped} total={total}".format(**counts)
    con.print(line)
    log.info(Ev.CliBenchmark, line)
    return counts


def run_self_tests(model, max_tokens: int, con: Console, log) -> int:
    """``--test``: tokenizer round trip, template render, and a short greedy generation."""
    tok = model.tokenizer
    bad = 0
    for s in ("Hello, world!", "What is 1+1?", "The quick brown fox jumps over the lazy dog.", "こんにちは世界", "  spaces  "):
        ids = tok.encode(s, add_special=False)
        back = tok.decode(ids)
        ok = back.strip() == s.strip()
        bad += 0 if ok else 1
        con.print(f"tokenizer {'OK ' if ok else 'BAD'} {s!r} -> {len(ids)} tokens -> {back!r}")
    rendered = PROMPT_RENDERER.render(model.cfg.chat_template, [ChatMessage(role="user", content="What is 1+1?")], True, model.arch)
    con.print(f"template rendered {len(rendered)} chars")
    out = run_inference(model, "What is 1+1?", None, max_tokens, log=log)
    con.print("=== Generated Output ===")
    con.print(out)
    return 1 if bad else 0


# ---------------------------------------------------------------------------- entry point
def load_model(o: CliOptions, log):
    from ..models.base import ModelBase
    device = resolve_device(o.backend)
    kw: Dict[str, Any] = {}
    if o.max_context:
        kw["max_context"] = o.max_context
    if o.kv_dtype:
        os.environ["TSB_KV_DTYPE"] = o.kv_dtype       # read by ModelBase (every rank parses the same command line)
    if o.batch_size > 1:
        kw["max_seqs"] = o.batch_size + 1          # one KV sequence per request in flight, plus the default one
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if o.pp > 1:
        # layer ranges on successive processes: python -m torch.distributed.run --nproc-per-node N -m tensorsharp_b200.cli --pp N
        if world != o.pp or o.tp > 1:
            raise ValueError(f"--pp {o.pp} needs {o.pp} processes and no --tp (WORLD_SIZE is {world}); start the CLI with "
                             f"python -m torch.distributed.run --nproc-per-node {o.pp} --master-addr 127.0.0.1 "
                             f"-m tensorsharp_b200.cli --pp {o.pp} ...")
        from ..parallel.dist import init_from_env
        from ..parallel.pipeline import PipelinedModel
        comm = init_from_env("gloo" if device == "cpu" else None)
        device = str(comm.device) if device != "cpu" else "cpu"
        stage = ModelBase.create(o.model, device, pp_rank=comm.rank, pp_size=comm.size, pp_comm=comm, **kw)
        model = PipelinedModel(stage)
        model.warm_up_kernels()
        return model
    if o.cp > 1:
        # every process holds the whole model; prompts of TSB_CP_MIN_TOKENS tokens or more are dealt to the processes
        if world != o.cp or o.tp > 1:
            raise ValueError(f"--cp {o.cp} needs {o.cp} processes and no --tp (WORLD_SIZE is {world}); start the CLI with "
                             f"python -m torch.distributed.run --nproc-per-node {o.cp} --master-addr 127.0.0.1 "
                             f"-m tensorsharp_b200.cli --cp {o.cp} ...")
        from ..parallel.dist import init_from_env
        comm = init_from_env("gloo" if device == "cpu" else None)
        device = str(comm.device) if device != "cpu" else "cpu"
        kw.update(cp_comm=comm)
    elif o.tp > 1 or world > 1:
        # one process per GPU, started by ``python -m torch.distributed.run --nproc-per-node N -m tensorsharp_b200.cli --tp N``
        if world != max(o.tp, 1):
            raise ValueError(f"--tp {o.tp} needs {o.tp} processes (WORLD_SIZE is {world}); start the CLI with "
                             f"python -m torch.distributed.run --nproc-per-node {max(o.tp, 2)} --master-addr 127.0.0.1 "
                             f"-m tensorsharp_b200.cli --tp {max(o.tp, 2)} ...")
        from ..parallel.dist import init_from_env
        comm = init_from_env("gloo" if device == "cpu" else None)
        device = str(comm.device) if device != "cpu" else "cpu"
        kw.update(tp_rank=comm.rank, tp_size=comm.size, comm=comm)
    log.info(Ev.ModelLoadStarted, "Loading model {ModelFile} on backend {Backend} (path={ModelPath})",
             ModelFile=os.path.basename(o.model), Backend=o.backend, ModelPath=o.model)
    t0 = time.perf_counter()
    model = ModelBase.create(o.model, device, **kw)
    log.info(Ev.ModelLoadCompleted, "Loaded model {ModelFile} architecture={Architecture} contextLength={ContextLength} "
             "elapsedMs={ElapsedMs:.1f}", ModelFile=os.path.basename(o.model), Architecture=model.arch or "(unknown)",
             ContextLength=model.max_context, ElapsedMs=(time.perf_counter() - t0) * 1e3)
    warm = getattr(model, "warm_up_kernels", None)
    if warm is not None:
        warm()
    return model


def attach_projector(model, o: CliOptions, log) -> None:
    mm = getattr(model, "multimodal", None)
    path = o.mmproj
    if path is None and (o.image or o.audio or o.video):
        auto = AUTO_MMPROJ.get(model.arch)
        cand = os.path.join(os.path.dirname(os.path.abspath(o.model)), auto) if auto else None
        if cand and os.path.isfile(cand):
            path = cand
            log.info(Ev.HostConfiguration, "Auto-loading multimodal encoder: {MmProj}", MmProj=cand)
    if path is None:
        return
    if mm is None:
        raise RuntimeError(f"architecture {model.arch!r} has no multimodal encoder in this build")
    mm.load_projectors(path)


def main(argv: Optional[Sequence[str]] = None, console: Optional[Console] = None) -> int:
    con = console or Console()
    try:
        o = parse_cli_args(list(sys.argv[1:] if argv is None else argv))
    except (ValueError, OSError) as e:
        con.error(f"error: {e}")
        con.error(USAGE)
        return 2
    provider = setup_file_logging(o.log_dir, o.log_level, prefix="tensorsharp-cli", enabled=o.log_file)
    log = provider.get_logger("TensorSharp.Cli") if provider is not None else NULL_LOGGER
    try:
        return _run(o, con, log)
    except Exception as e:
        log.error(Ev.CliFailed, "CLI failed: {Error}", exc=e, Error=str(e))
        con.error(f"error: {e}")
        return 1
    finally:
        if provider is not None:
            provider.close()


def _run(o: CliOptions, con: Console, log) -> int:
    tools = None
    if o.tools_file is not None:
        if not os.path.isfile(o.tools_file):
            con.error(f"Tools file not found: {o.tools_file}")
            return 1
        tools = load_tools(o.tools_file)
        log.info(Ev.HostConfiguration, "Loaded {ToolCount} tool definition(s) from {ToolsFile}", ToolCount=len(tools),
                 ToolsFile=o.tools_file)
    if o.test_templates_dir is not None:
        return 1 if test_chat_templates(o.test_templates_dir, con, log)["failed"] else 0
    if o.model is None or not os.path.isfile(o.model):
        log.error(Ev.CliFailed, "Model file not found: {ModelPath}", ModelPath=o.model or "(none)")
        con.error(f"Model file not found: {o.model or '(none)'}")
        con.error(USAGE)
        return 1
    model = load_model(o, log)
    cp_comm = getattr(model, "cp_comm", None)
    if getattr(model, "tp_rank", 0) != 0 or getattr(model, "pp_rank", 0) != 0 or (cp_comm is not None and cp_comm.rank != 0):
        con = Console(open(os.devnull, "w"), con.err)          # every rank runs the same steps; rank 0 does the talking
    try:
        attach_projector(model, o, log)
        if o.run_test:
            return run_self_tests(model, o.max_tokens, con, log)
        if o.benchmark:
            run_benchmark_mode(model, o, con, log)
            return 0
        if o.test_chunked_prefill:
            return 0 if run_chunked_prefill_correctness(model, o.correct_prefill, o.correct_decode, con, log) else 1
        if o.bench_kvcache:
            run_kv_cache_benchmark(model, o.bench_kv_turns, o.max_tokens, o.sampling, o.think, con, log)
            return 0
        if o.multi_turn_jsonl is not None:
            return run_multi_turn_test(model, o.multi_turn_jsonl, o.max_tokens, o.sampling, o.think, con, log)
        if o.input_jsonl is not None:
            return run_jsonl_batch(model, o.input_jsonl, o.output_file, o.max_tokens, o.sampling, o.think, con, log,
                                   batch_size=o.batch_size)
        if o.interactive:
            from .interactive import InteractiveSession
            s = InteractiveSession(model, o.model, o.backend, o.mmproj, o.sampling, tools, o.think,
                                   o.max_tokens if o.max_tokens > 0 else 512, log, con)
            if o.system:
                s.set_initial_system_prompt(o.system)
            s.run()
            return 0
        return _one_shot(model, o, tools, con, log)
    finally:
        model.close()


def _one_shot(model, o: CliOptions, tools, con: Console, log) -> int:
    if o.input_file is not None and os.path.isfile(o.input_file):
        with open(o.input_file, "r", encoding="utf-8") as f:
            text = f.read().rstrip()
    else:
        text = "What is 1+1?"
    image_paths = audio_paths = None
    if o.video is not None:
        if not os.path.isfile(o.video):
            con.error(f"Video file not found: {o.video}")
            return 1
        image_paths = media.extract_video_frames(o.video)
        text = "What is happening in this video? Please describe it."
    elif o.image is not None:
        if not os.path.isfile(o.image):
            con.error(f"Image file not found: {o.image}")
            return 1
        image_paths = [o.image]
        text = "What is in this image? Please describe it."
    if o.audio is not None:
        if not os.path.isfile(o.audio):
            con.error(f"Audio file not found: {o.audio}")
            return 1
        audio_paths = [o.audio]
        text = "Listen to this audio and describe what you hear."
    if o.dump_prompt:
        rendered = PROMPT_RENDERER.render(model.cfg.chat_template, [ChatMessage(role="user", content=text)], True,
                                          model.arch, tools, o.think)
        con.print("=== Rendered Prompt ===")
        con.print(rendered)
        tail = f"0x{ord(rendered[-1]):02X}" if rendered else "empty"
        con.print(f"=== End ({len(rendered)} chars, ends with: {tail}) ===")
        toks = model.tokenizer.encode(rendered, add_special=True)
        con.print(f"Token count: {len(toks)}")
        con.print(f"First 20 tokens: [{', '.join(map(str, toks[:20]))}]")
        con.print(f"Last 10 tokens: [{', '.join(map(str, toks[-10:]))}]")
        return 0
    log.info(Ev.ChatStarted, "cli.inference.start tokensRequested={MaxTokens} thinking={Thinking} tools={ToolCount}",
             MaxTokens=o.max_tokens, Thinking=o.think, ToolCount=len(tools or []))
    result = run_inference(model, text, image_paths, o.max_tokens, audio_paths, o.video is not None, o.sampling, o.think,
                           tools, log)
    if o.output_file is not None:
        with open(o.output_file, "w", encoding="utf-8") as f:
            f.write(result)
        con.print(f"Output written to {o.output_file}")
    else:
        con.print("\n=== Generated Output ===")
        con.print(result)
    return 0
