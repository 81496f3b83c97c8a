"""Command-line tool on CPU with the tiny synthetic model: flag parsing, every batch mode, the
interactive session's commands and multi-turn KV reuse."""
import io
import json
import os

import pytest
import torch

from tensorsharp_b200.cli.args import parse_cli_args
from tensorsharp_b200.cli.interactive import InteractiveSession
from tensorsharp_b200.cli.main import Console, describe_plan, format_parsed_result, load_tools, main
from tensorsharp_b200.runtime.chat import ToolCall
from tensorsharp_b200.runtime.kv_cache import ReusePlan
from tensorsharp_b200.runtime.output_parser import ParsedOutput
from tensorsharp_b200.runtime.sampling import SamplingConfig


def run_cli(args):
    out, err = io.StringIO(), io.StringIO()
    rc = main(list(args) + ["--log-file", "off"], Console(out, err))
    return rc, out.getvalue(), err.getvalue()


def test_parse_cli_args_defaults_and_flags(tmp_path):
    o = parse_cli_args([])
    assert (o.max_tokens, o.backend, o.bench_prefill, o.bench_decode, o.bench_runs) == (100, "b200", 32, 64, 1)
    assert (o.correct_prefill, o.correct_decode, o.bench_kv_turns) == (1500, 8, 4)
    assert o.sampling.is_greedy and o.sampling.repetition_penalty == 1.0
    sysf = tmp_path / "sys.txt"
    sysf.write_text("be brief")
    o = parse_cli_args(["--model", "m.gguf", "--backend", "CUDA", "--chat", "--temperature", "0.7", "--top-k", "5", "--stop", "a",
                        "--stop", "b", "--think", "--bench-chunked", "--system-file", str(sysf), "--log-console", "off",
                        "--max-tokens", "7", "--wat"])
    assert (o.model, o.backend, o.interactive, o.think, o.bench_chunked, o.system) == ("m.gguf", "cuda", True, True, True, "be brief")
    assert (o.sampling.temperature, o.sampling.top_k, o.sampling.stop_sequences, o.max_tokens) == (0.7, 5, ["a", "b"], 7)
    assert not o.log_console and o.unknown == ["--wat"]
    with pytest.raises(ValueError):
        parse_cli_args(["--max-tokens", "x"])
    with pytest.raises(ValueError):
        parse_cli_args(["--model"])


def test_formatting_helpers(tmp_path):
    p = ParsedOutput(content="Answer", thinking=" why ", tool_calls=[ToolCall("f", {"a": 1})])
    s = format_parsed_result(p, True)
    assert "--- Thinking ---\nwhy\n--- End Thinking ---" in s and "Answer" in s and "Function: f" in s and '"a": 1' in s
    assert "Thinking" not in format_parsed_result(p, False)
    assert describe_plan(ReusePlan.reuse(30, 10), 40) == "Partial reuse: keeping 30/40 tokens, forwarding 10 new (saved 75%)"
    assert describe_plan(ReusePlan.reset(9), 9) == "Full reset: forwarding 9 tokens"
    assert describe_plan(ReusePlan.exact_match([1.0]), 5).startswith("Exact match: reusing all 5")
    tf = tmp_path / "tools.json"
    tf.write_text(json.dumps([{"Name": "get", "Description": "d", "Parameters": {"x": {"Type": "string", "Enum": ["a"]}},
                               "Required": ["x"]},
                              {"type": "function", "function": {"name": "g", "parameters": {"properties": {"y": {"type": "integer"}}}}}]))
    tools = load_tools(str(tf))
    assert tools[0].name == "get" and tools[0].parameters["x"].enum == ["a"] and tools[0].required == ["x"]
    assert tools[1].name == "g" and tools[1].parameters["y"].type == "integer"


def test_missing_model_prints_usage():
    rc, out, err = run_cli(["--model", "/nonexistent.gguf"])
    assert rc == 1 and "Model file not found" in err and "Usage:" in err


def test_one_shot_dump_prompt_and_output_file(tiny_qwen3_path, tmp_path):
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--dump-prompt"])
    assert rc == 0 and "<|im_start|>user\nWhat is 1+1?<|im_end|>\n<|im_start|>assistant\n===" in out
    assert "ends with: 0x74" in out              # the Jinja result is right-trimmed, as in the reference and "Token count:" in out and "First 20 tokens: [" in out
    inp, outp = tmp_path / "in.txt", tmp_path / "out.txt"
    inp.write_text("Say hi\n\n")
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--input", str(inp), "--output", str(outp), "--max-tokens", "5"])
    assert rc == 0 and f"Output written to {outp}" in out and outp.exists()
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--max-tokens", "4"])
    assert rc == 0 and "=== Generated Output ===" in out


def test_benchmark_modes(tiny_qwen3_path):
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--benchmark", "--bench-prefill", "16", "--bench-decode", "4",
                          "--bench-runs", "2"])
    assert rc == 0 and "benchmark run 2/2:" in out and "benchmark summary: bestPrefillMs=" in out and "avgDecodeTps=" in out
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--test-chunked-prefill", "--correct-prefill", "200",
                          "--correct-decode", "4"])
    assert rc == 0 and "matched 4/4 decode tokens -> PASS" in out
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--bench-kvcache", "--bench-kv-turns", "3", "--max-tokens", "4"])
    assert rc == 0 and "kv bench turn 3:" in out and "kv bench summary over turns 2..3" in out


def test_jsonl_batch_and_multi_turn(tiny_qwen3_path, tmp_path):
    req = tmp_path / "req.jsonl"
    req.write_text("\n".join([
        json.dumps({"id": "a", "prompt": "Hello", "max_tokens": 3}),
        "{broken",
        json.dumps({"messages": [{"role": "system", "content": "s"}, {"role": "user", "content": "u"}], "temperature": 0.5, "seed": 1,
                    "stop": ["zz"]}),
        "", json.dumps([1, 2])]))
    res = tmp_path / "res.jsonl"
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--input-jsonl", str(req), "--output", str(res), "--max-tokens", "4"])
    assert rc == 0
    rows = [json.loads(l) for l in res.read_text().splitlines()]
    assert list(rows[0]) == ["id", "output", "tokens_generated", "prefill_ms", "total_ms", "tokens_per_second"]
    assert rows[0]["id"] == "a" and rows[0]["tokens_generated"] <= 3
    assert rows[1]["line"] == 2 and rows[1]["error"].startswith("Invalid JSON")
    assert rows[2]["id"] == "request_3" and rows[2]["tokens_generated"] <= 4 and "error" in rows[3]
    mt = tmp_path / "turns.jsonl"
    mt.write_text("\n".join([json.dumps({"content": "first question", "max_tokens": 3}), "plain second line",
                             json.dumps({"content": "third", "force_reset": True})]))
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--multi-turn-jsonl", str(mt), "--max-tokens", "3"])
    assert rc == 0
    assert "[turn 1] promptTokens=" in out and "plan=Reset" in out.split("[turn 1]")[1].split("\n")[0]
    assert "plan=PartialReuse" in out.split("[turn 2]")[1].split("\n")[0]
    assert "plan=Reset" in out.split("[turn 3]")[1].split("\n")[0]


def test_self_test_and_template_scan(tiny_qwen3_path, tmp_path):
    rc, out, _ = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--test", "--max-tokens", "3"])
    assert "tokenizer OK  'Hello, world!'" in out and "template rendered" in out
    rc, out, _ = run_cli(["--test-templates", os.path.dirname(tiny_qwen3_path)])
    assert "[single-turn] PASS" in out and "[multi-turn] PASS" in out and "[with-system] PASS" in out
    assert "passed=1 failed=0" in out and rc == 0


class Script:
    def __init__(self, lines):
        self.lines = list(lines)

    def __call__(self, prompt):
        return self.lines.pop(0) if self.lines else None


def test_interactive_session_commands_and_kv_reuse(tiny_qwen3_path, tmp_path):
    from tensorsharp_b200.models.base import ModelBase
    model = ModelBase.create(tiny_qwen3_path, "cpu")
    note = tmp_path / "note.txt"
    note.write_text("remember 42")
    saved = tmp_path / "chat.txt"
    out = io.StringIO()
    s = InteractiveSession(model, tiny_qwen3_path, "cpu", None, SamplingConfig.greedy(), None, False, 4, console=Console(out, out),
                           read_line=Script(["/help", "/bogus", "/temp 0.5", "/temp x", "/topk 3", "/seed 7", "/stop END", "/clearstop",
                                             "/temp 0", "/topk 0", "/max 3", "/max -1", "/think on", "/think", "/system Be brief.",
                                             f"/text {note}", "/image /nope.png", "/info", "hello there", "and again", "/history",
                                             f"/save {saved}", "/multiline on", "line one", "line two", ".", "/multiline off",
                                             "/reset", "/info", "/exit"]))
    s.run()
    text = out.getvalue()
    assert "Conversation:" in text and "Unknown command: /bogus" in text and "temperature updated." in text
    assert "Could not parse 'x' as float for temperature." in text and "Seed set to 7 (deterministic)." in text
    assert 'Added stop sequence "END". Now 1 configured.' in text and "Cleared all stop sequences." in text
    assert "Max tokens per reply set to 3." in text and "Could not parse '-1' as a positive integer." in text
    assert "Thinking is now on." in text and "Thinking is now off." in text
    assert "System prompt set (9 chars). Conversation reset." in text and "Text file attached:" in text
    assert "Image file not found: /nope.png" in text and "Architecture: qwen3" in text and "1 text file(s)." in text
    assert "(Reset, prefill" in text and "(PartialReuse, prefill" in text            # second turn re-used the first
    assert "--- system ---\nBe brief." in text and "[Attached file: note.txt]\nremember 42\n[End of file]" in text
    body = saved.read_text()
    assert body.startswith("=== System ===\nBe brief.\n=== user ===") and body.count("=== assistant ===") == 2
    assert "Multi-line input on" in text and "Conversation history and KV cache cleared." in text and text.rstrip().endswith("Bye.")
    assert [m.role for m in s.history] == [] and s.kv.is_empty
    model.close()


def test_tp_flag_needs_matching_process_count(tiny_qwen3_path, monkeypatch):
    """``--tp 2`` in a single process explains how to start the job instead of silently running unsharded."""
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    rc, out, err = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--tp", "2", "--benchmark"])
    assert rc == 1 and "torch.distributed.run" in err


def test_jsonl_batch_size_gives_the_sequential_outputs(tiny_qwen3_path, tmp_path):
    """--batch-size N decodes the requests together; every request's text and token count equal the
    one-at-a-time run (greedy), bad lines stay where they were, and the file's order is kept."""
    prompts = ["Hello", "Tell me about the sea", "One two three four five six", "x", "What is 2+2?", "Goodbye now"]
    lines = [json.dumps({"id": f"r{i}", "prompt": p, "max_tokens": 3 + 2 * (i % 3)}) for i, p in enumerate(prompts)]
    lines.insert(2, "{broken")
    lines.append(json.dumps({"id": "stop", "prompt": "Hello", "max_tokens": 6, "stop": ["<|tok"]}))
    req = tmp_path / "req.jsonl"
    req.write_text("\n".join(lines))
    outs = {}
    for bs in (1, 3):
        res = tmp_path / f"res{bs}.jsonl"
        rc, _, err = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--input-jsonl", str(req), "--output", str(res),
                              "--max-tokens", "4", "--batch-size", str(bs)])
        assert rc == 0, err
        outs[bs] = [json.loads(l) for l in res.read_text().splitlines()]
    assert len(outs[1]) == len(outs[3]) == len(lines)
    for a, b in zip(outs[1], outs[3]):
        assert list(a) == list(b)
        for k in ("id", "line", "output", "tokens_generated"):
            assert a.get(k) == b.get(k), (a, b)
    assert outs[3][2]["error"].startswith("Invalid JSON")


@pytest.mark.parametrize("graph_steps", ["0", "1"])
def test_continuous_batcher_refills_the_batch(tiny_qwen3_path, monkeypatch, graph_steps):
    """``graph_steps`` = 1: the decode steps go through the static batch of the graph stepper (eager on CPU)."""
    monkeypatch.setenv("TSB_GATHER_GRAPH", graph_steps)
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.batching import ContinuousBatcher, GenRequest
    from tensorsharp_b200.runtime.engine import generate
    m = ModelBase.create(tiny_qwen3_path, "cpu", max_context=128, max_seqs=4)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(5, 4000, (n,), generator=g).tolist() for n in (7, 19, 3, 11, 26)]
    lens = [5, 2, 9, 1, 6]
    pieces = []
    reqs = [GenRequest(p, n, on_piece=(pieces.append if i == 0 else None), tag=i) for i, (p, n) in enumerate(zip(prompts, lens))]
    eng = ContinuousBatcher(m, max_batch=3, prefill_chunk=8)
    free0 = m.kv.free_pages
    eng.run(reqs)
    assert m.kv.free_pages == free0                         # every sequence gave its pages back
    assert eng.steps < sum(lens) and eng.step_rows / eng.steps > 1.5
    assert (eng.graph_steps == eng.steps) if graph_steps == "1" else eng.graph_steps == 0
    eos = [t for t in range(m.cfg.vocab) if m.tokenizer.is_eos(t)]
    for r, p, n in zip(reqs, prompts, lens):
        m.reset_kv_cache()
        assert r.error is None and r.ids == generate(m, p, n, eos_ids=eos)
    assert "".join(pieces) == reqs[0].text


TESTDATA = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tensorsharp_b200", "cli", "testdata")


def test_shipped_fixtures_run_through_the_cli(tiny_qwen3_path, tmp_path):
    """The fixtures that ship with the CLI (tool definitions in both accepted shapes, a JSONL batch, a
    multi-turn script, prompt files) load and run."""
    units = load_tools(os.path.join(TESTDATA, "tools_units.json"))
    cal = load_tools(os.path.join(TESTDATA, "tools_calendar.json"))
    assert [t.name for t in units] == ["convert_length", "list_units"] and units[0].required == ["value", "from_unit", "to_unit"]
    assert units[0].parameters["from_unit"].enum == ["m", "km", "ft", "mi"]
    assert cal[0].name == "days_between" and set(cal[0].parameters) == {"start", "end"}
    res = tmp_path / "res.jsonl"
    rc, _, err = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--input-jsonl", os.path.join(TESTDATA, "batch_requests.jsonl"),
                          "--output", str(res), "--max-tokens", "4", "--batch-size", "2"])
    assert rc == 0, err
    rows = [json.loads(l) for l in res.read_text().splitlines()]
    assert [r["id"] for r in rows] == ["sum", "chat", "stop", "think"] and not any("error" in r for r in rows)
    rc, out, err = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--multi-turn-jsonl", os.path.join(TESTDATA, "multi_turn.jsonl"),
                            "--max-tokens", "3"])
    assert rc == 0 and "[turn 4]" in out and "plan=Reset" in out.split("[turn 4]")[1].split("\n")[0], err
    rc, out, err = run_cli(["--model", tiny_qwen3_path, "--backend", "cpu", "--input", os.path.join(TESTDATA, "input_tool_convert.txt"),
                            "--tools", os.path.join(TESTDATA, "tools_units.json"), "--dump-prompt", "--max-tokens", "2"])
    assert rc == 0 and "3.2 kilometres" in out, err          # (the synthetic model's template has no tool section)
