"""Runtime services on CPU: KV reuse planner, raw-token-splicing prompt renderer, chat templates and
the Jinja interpreter, streaming output parsers, structured outputs, samplers, tokenizers, the
JSONL logger and media helpers.  Cases and golden strings follow the reference's InferenceWeb.Tests
(KVCacheTests, KVCachePromptRendererTests, StructuredOutputTests, SamplingConfigCloneTests,
FileLoggerProviderTests, MediaHelperTests)."""
import datetime as dt
import json
import os

import pytest
import torch

from tensorsharp_b200.runtime import media
from tensorsharp_b200.runtime.chat import ChatMessage, ToolCall, ToolFunction, ToolParameter, dotnet_json
from tensorsharp_b200.runtime.chat_template import render_from_gguf_template, render_hardcoded
from tensorsharp_b200.runtime.jinja import Jinja2Template
from tensorsharp_b200.runtime.kv_cache import KVCache, ReusePlanKind
from tensorsharp_b200.runtime.logging import Ev, FileLoggerOptions, FileLoggerProvider, log_scope
from tensorsharp_b200.runtime.output_parser import create_output_parser, is_always_required
from tensorsharp_b200.runtime.prompt_renderer import KVCachePromptRenderer, assistant_generation_suffix
from tensorsharp_b200.runtime.sampling import SamplingConfig, TokenSampler
from tensorsharp_b200.runtime.structured import (StructuredOutputFormat, StructuredOutputKind, apply_to_messages,
                                                 normalize_output, validate_schema)


# ---------------------------------------------------------------------------- KVCache
def test_kv_cache_bookkeeping():
    c = KVCache()
    assert c.is_empty and c.count == 0 and list(c.tokens) == [] and c.next_logits is None
    lg = [0.1, 0.2]
    c.record_append(42, lg)
    assert c.count == 1 and list(c.tokens) == [42] and c.next_logits is lg
    c.record_append([1, 2, 3, 4], [0.7])
    assert list(c.tokens) == [42, 1, 2, 3, 4] and c.next_logits == [0.7]
    c.record_append(None, [9.0])
    assert c.count == 5 and c.next_logits == [0.7]
    c.record_append([5], None)
    assert c.count == 6 and c.next_logits is None
    c.reset()
    assert c.is_empty and c.next_logits is None
    c.record_append([1, 2, 3, 4, 5], lg)
    c.truncate_to(5)
    assert c.next_logits is lg
    c.truncate_to(3)
    assert list(c.tokens) == [1, 2, 3] and c.next_logits is None
    for bad in (-1, 4):
        with pytest.raises(ValueError):
            c.truncate_to(bad)
    c.truncate_to(0)
    assert c.is_empty


def test_kv_cache_prefix_queries():
    c = KVCache()
    c.record_append([1, 2, 3], [0.5])
    assert c.common_prefix_length([4, 5, 6]) == 0 and c.common_prefix_length([1, 2, 3, 99, 100]) == 3
    assert c.common_prefix_length([1, 2, 3, 4, 5]) == 3 and c.common_prefix_length([1, 2]) == 2
    assert c.common_prefix_length(None) == 0 and c.common_prefix_length([]) == 0
    assert c.is_prefix_of([1, 2, 3]) and c.is_prefix_of([1, 2, 3, 4])
    assert not c.is_prefix_of([1, 99, 3]) and not c.is_prefix_of([1, 2])
    assert c.try_get_exact_match_logits([1, 2, 3]) == [0.5]
    assert c.try_get_exact_match_logits([1, 2]) is None and c.try_get_exact_match_logits([1, 2, 3, 4]) is None
    c.record_append([4], None)
    assert c.try_get_exact_match_logits([1, 2, 3, 4]) is None


def plan_of(cached, logits, new, trunc=True):
    c = KVCache()
    if cached:
        c.record_append(cached, logits)
    p = c.plan_reuse(new, trunc)
    return p.kind, p.reused_prefix_length, p.tokens_to_forward, p.cached_logits


def test_kv_cache_plan_reuse():
    R, P, E = ReusePlanKind.RESET, ReusePlanKind.PARTIAL_REUSE, ReusePlanKind.EXACT_MATCH
    assert plan_of([], None, [1, 2, 3, 4]) == (R, 0, 4, None)
    assert plan_of([1, 2], [0.5], [])[0:3] == (R, 0, 0) and plan_of([1, 2], [0.5], None)[0:3] == (R, 0, 0)
    assert plan_of([1, 2, 3], [0.9], [1, 2, 3]) == (E, 0, 0, [0.9])
    assert plan_of([1, 2, 3], None, [1, 2, 3])[0:3] == (P, 2, 1)              # no logits cached: re-forward the last token
    assert plan_of([1, 2, 3, 4, 5], [0.5], [1, 2, 3, 99, 100])[0:3] == (P, 3, 2)
    assert plan_of([1, 2, 3], [0.5], [1, 2, 3, 4, 5])[0:3] == (P, 3, 2)
    assert plan_of([1, 2, 3, 4, 5], [0.5], [1, 2, 3, 99, 100], trunc=False)[0:3] == (R, 0, 5)
    assert plan_of([1, 2, 3], [0.5], [1, 2, 3, 4, 5, 6], trunc=False)[0:3] == (P, 3, 3)   # pure extension needs no rewind
    assert plan_of([1, 2, 3], [0.5], [99, 100])[0:3] == (R, 0, 2)
    assert plan_of([1, 2, 3, 4], [0.5], [99, 2, 3, 4])[0:3] == (R, 0, 4)
    assert plan_of([1, 2, 3, 4, 5], [0.5], [1, 2, 3])[0:3] == (P, 2, 1)


# ---------------------------------------------------------------------------- KVCachePromptRenderer
class FakeRenderer:
    def __init__(self, trim=False):
        self.trim = trim

    def render(self, template, messages, add_generation_prompt=True, architecture=None, tools=None, enable_thinking=False):
        s = "<|bos|>" + "".join(f"<{m.role}>{m.content or ''}</{m.role}>\n" for m in messages)
        if add_generation_prompt:
            s += "<assistant>"
        return s.rstrip() if self.trim else s


class GrowingCharTokenizer:
    def __init__(self):
        self.ids, self.vocab = {}, ["<bos>", "<eos>"]

    def encode(self, text, add_special=True):
        out = [0] if add_special else []
        for ch in text or "":
            if ch not in self.ids:
                self.ids[ch] = len(self.vocab)
                self.vocab.append(ch)
            out.append(self.ids[ch])
        return out

    def decode(self, ids):
        return "".join(self.vocab[i] for i in ids if i > 1 and i < len(self.vocab))


def find_sub(hay, needle):
    return next((i for i in range(len(hay) - len(needle) + 1) if hay[i:i + len(needle)] == needle), -1)


def test_prompt_renderer_splices_raw_tokens():
    r, tok = KVCachePromptRenderer(FakeRenderer()), GrowingCharTokenizer()
    plain = [ChatMessage(role="user", content="Hi")]
    assert r.render_to_tokens(tok, None, plain, "fake", True) == tok.encode(FakeRenderer().render(None, plain))
    msgs = [ChatMessage(role="user", content="Hi"),
            ChatMessage(role="assistant", content="DOES_NOT_MATTER", raw_output_tokens=[1001, 1002, 1003]),
            ChatMessage(role="user", content="again"),
            ChatMessage(role="assistant", content="x", raw_output_tokens=[2001, 2002]),
            ChatMessage(role="user", content="third")]
    out = r.render_to_tokens(tok, None, msgs, "fake", True)
    assert "DOES_NOT_MATTER" not in tok.decode(out)
    a, b = find_sub(out, [1001, 1002, 1003]), find_sub(out, [2001, 2002])
    assert 0 < a < b
    # structure around the splice is what the inner renderer produced
    assert tok.decode(out[:a]).endswith("<assistant>") and tok.decode(out[a + 3:]).startswith("</assistant>\n<user>again")
    # empty raw list: content is rendered normally
    e = [ChatMessage(role="user", content="Hi"), ChatMessage(role="assistant", content="Hello", raw_output_tokens=[])]
    assert "Hello" in tok.decode(r.render_to_tokens(tok, None, e, "fake", True))
    with pytest.raises(ValueError):
        r.render_to_tokens(tok, None, None, "fake", True)
    with pytest.raises(ValueError):
        r.render_to_tokens(None, None, plain, "fake", True)
    with pytest.raises(ValueError):
        KVCachePromptRenderer(None)


@pytest.mark.parametrize("trim", [False, True])
def test_prompt_renderer_prefix_is_stable_across_turns(trim):
    """Turn N+1's tokens start with turn N's prompt + the tokens sampled in turn N."""
    r, tok = KVCachePromptRenderer(FakeRenderer(trim)), GrowingCharTokenizer()
    t1 = [ChatMessage(role="user", content="Hello")]
    p1 = r.render_to_tokens(tok, None, t1, "fake", True)
    raw1 = [5001, 5002, 5003, 5004]                       # e.g. <think>..</think>answer: differs from the parsed text
    t2 = t1 + [ChatMessage(role="assistant", content="answer", raw_output_tokens=raw1), ChatMessage(role="user", content="More")]
    p2 = r.render_to_tokens(tok, None, t2, "fake", True)
    assert p2[:len(p1) + len(raw1)] == p1 + raw1
    raw2 = [6001]
    t3 = t2 + [ChatMessage(role="assistant", content="b", raw_output_tokens=raw2), ChatMessage(role="user", content="Z")]
    p3 = r.render_to_tokens(tok, None, t3, "fake", True)
    assert p3[:len(p2) + 1] == p2 + raw2


def test_assistant_generation_suffix():
    assert assistant_generation_suffix("gemma4", False) == "<|channel>thought\n<channel|>"
    assert assistant_generation_suffix("gemma4", True) == ""
    for a in ("qwen35", "qwen35moe", "qwen3next"):
        assert assistant_generation_suffix(a, True) == "<think>\n" and assistant_generation_suffix(a, False) == ""
    for a in ("qwen3", "gemma3", "gptoss", "mistral3", None, ""):
        assert assistant_generation_suffix(a, True) == "" and assistant_generation_suffix(a, False) == ""


# ---------------------------------------------------------------------------- templates / Jinja
def test_qwen35_no_thinking_keeps_prior_answer_as_prefix():
    t1 = [ChatMessage(role="user", content="What is the tallest mountain in the world?")]
    r1 = render_from_gguf_template("{{ 'from-jinja' }}", t1, True, "qwen35", None, False)
    t2 = t1 + [ChatMessage(role="assistant", content="Mount Everest"), ChatMessage(role="user", content="How tall is it in meters?")]
    r2 = render_from_gguf_template("{{ 'from-jinja' }}", t2, True, "qwen35", None, False)
    assert "from-jinja" not in r1 and r2.startswith(r1 + "Mount Everest")


def test_hardcoded_templates_shapes():
    m = [ChatMessage(role="system", content="S"), ChatMessage(role="user", content="U")]
    q = render_hardcoded(m, True, "qwen3")
    assert q == "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nU<|im_end|>\n<|im_start|>assistant\n"
    g = render_hardcoded([ChatMessage(role="user", content="U")], True, "gemma3")
    assert g.startswith("<start_of_turn>user\nU<end_of_turn>\n<start_of_turn>model\n")
    h = render_hardcoded(m, True, "gptoss")
    assert "<|start|>user<|message|>U<|end|>" in h and h.endswith("<|start|>assistant")
    mi = render_hardcoded([ChatMessage(role="user", content="U")], True, "mistral3")
    assert "[INST]U[/INST]" in mi
    tools = [ToolFunction("f", "d", {"a": ToolParameter("string", "x")}, ["a"])]
    qt = render_hardcoded(m, True, "qwen3", tools)
    assert "access to the following functions" in qt and '"Name":"f"' in qt and '"Required":["a"]' in qt


def test_jinja_interpreter_features():
    t = Jinja2Template(
        "{%- set ns = namespace(n=0) -%}{%- for m in messages if m.role != 'system' -%}"
        "{%- set ns.n = ns.n + 1 -%}{{ loop.index }}:{{ m.role|upper }}={{ m.content|trim }}{% if not loop.last %};{% endif %}"
        "{%- endfor %} n={{ ns.n }} {{ 'yes' if add_generation_prompt else 'no' }} {{ messages[0]['content'][:3] }}"
        "{% if tools is defined and tools %}T{% else %}-{% endif %}{{ x|default('dflt') }} {{ [1,2,3]|length }} {{ 'a,b'.split(',')|join('+') }}")
    out = t.render({"messages": [{"role": "system", "content": "sysmsg"}, {"role": "user", "content": " hi "},
                                 {"role": "assistant", "content": "yo"}], "add_generation_prompt": True})
    assert out == "1:USER=hi;2:ASSISTANT=yo n=2 yes sys-dflt 3 a+b"
    macro = Jinja2Template("{% macro wrap(x, tag='b') %}<{{ tag }}>{{ x }}</{{ tag }}>{% endmacro %}{{ wrap('q') }}{{ wrap('r', tag='i') }}")
    assert macro.render({}) == "<b>q</b><i>r</i>"
    assert Jinja2Template("{{ d|tojson }}").render({"d": {"a": [1, "x", None, True]}}) in ('{"a": [1, "x", null, true]}', '{"a":[1,"x",null,true]}')
    assert Jinja2Template("{% if a is string %}s{% elif a is mapping %}m{% else %}o{% endif %}").render({"a": {}}) == "m"
    with pytest.raises(Exception):
        Jinja2Template("{{ raise_exception('boom') }}").render({})


def test_dotnet_json_escaping():
    assert dotnet_json({"a": "x<y>&'\"+é\n", "b": [1, 2.5, True, None]}) == \
        '{"a":"x\\u003Cy\\u003E\\u0026\\u0027\\u0022\\u002B\\u00E9\\n","b":[1,2.5,true,null]}'
    assert dotnet_json("😀") == '"\\uD83D\\uDE00"'
    assert dotnet_json({"a": {"b": 1}}, indented=True) == '{\n  "a": {\n    "b": 1\n  }\n}'


# ---------------------------------------------------------------------------- output parsers
def stream(parser, text, step=3):
    content, thinking, calls = "", "", None
    for i in range(0, len(text), step):
        p = parser.add(text[i:i + step], False)
        content += p.content or ""
        thinking += p.thinking or ""
        calls = p.tool_calls if p.tool_calls is not None else calls
    p = parser.add("", True)
    content += p.content or ""
    thinking += p.thinking or ""
    calls = p.tool_calls if p.tool_calls is not None else calls
    return content, thinking, calls


TOOLS = [ToolFunction("get_weather", "w", {"city": ToolParameter("string")}, ["city"])]


@pytest.mark.parametrize("step", [1, 3, 1000])
def test_qwen3_parser_streams_thinking_content_and_tools(step):
    p = create_output_parser("qwen3")
    p.init(True, TOOLS)
    c, t, calls = stream(p, 'reason here</think>\n\nThe answer.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>', step)
    assert t.strip() == "reason here" and c.strip() == "The answer."
    assert len(calls) == 1 and calls[0].name == "get_weather" and calls[0].arguments == {"city": "Paris"}
    p = create_output_parser("qwen3")
    p.init(False, None)
    c, t, calls = stream(p, "plain <b>text</b>", step)                 # thinking off: everything is content
    assert c == "plain <b>text</b>" and t == "" and calls is None


@pytest.mark.parametrize("step", [1, 4, 1000])
def test_harmony_and_gemma4_parsers(step):
    assert is_always_required("gptoss") and is_always_required("gemma4") and not is_always_required("qwen3")
    p = create_output_parser("gptoss")
    p.init(True, None)
    c, t, _ = stream(p, "<|channel|>analysis<|message|>thinking it over<|end|><|start|>assistant<|channel|>final<|message|>Done.", step)
    assert t == "thinking it over" and c == "Done."
    p = create_output_parser("gemma4")
    p.init(True, TOOLS)
    c, t, calls = stream(p, '<|channel>thought\nhmm<channel|>Answer<|tool_call>call:get_weather{city:<|"|>Paris<|"|>}<tool_call|>', step)
    assert t.strip() == "hmm" and c.strip() == "Answer" and calls[0].name == "get_weather" and calls[0].arguments == {"city": "Paris"}
    p = create_output_parser("llama")
    p.init(False, None)
    assert stream(p, "as <is>", step)[0] == "as <is>"


# ---------------------------------------------------------------------------- structured outputs
def test_structured_schema_validation():
    bad = StructuredOutputFormat.json_schema("bad_schema", json.dumps({"anyOf": [{
        "type": "object", "properties": {"answer": {"type": "string"}}, "required": [], "additionalProperties": False}]}), True)
    v = validate_schema(bad)
    assert not v.is_valid and any("root schema" in e.lower() for e in v.errors) and any("required" in e.lower() for e in v.errors)
    loose = StructuredOutputFormat.json_schema("weather", json.dumps({
        "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}), False)
    v = validate_schema(loose)
    assert not v.is_valid and any("strict" in e.lower() for e in v.errors) and any("additionalproperties" in e.lower() for e in v.errors)
    ok = StructuredOutputFormat.json_schema("w", json.dumps({
        "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"], "additionalProperties": False}), True)
    assert validate_schema(ok).is_valid and validate_schema(StructuredOutputFormat.json_object()).is_valid


def test_structured_normalisation_golden_vectors():
    n = normalize_output('Here you go:\n```json\n{\n  "answer": 5\n}\n```\n', StructuredOutputFormat.json_object())
    assert n.is_valid and n.normalized_content == '{"answer":5}'
    fmt = StructuredOutputFormat.json_schema("result", json.dumps({
        "type": "object", "properties": {"answer": {"type": "string"}, "optional_note": {"type": ["string", "null"]},
                                         "done": {"type": "boolean"}},
        "required": ["answer", "optional_note", "done"], "additionalProperties": False}), True)
    n = normalize_output('{"done": true, "extra": "remove me", "answer": "ok"}', fmt)
    assert n.is_valid and n.normalized_content == '{"answer":"ok","optional_note":null,"done":true}'
    fmt = StructuredOutputFormat.json_schema("container", json.dumps({
        "type": "object",
        "properties": {"item": {"anyOf": [{"$ref": "#/$defs/person"}, {
            "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"], "additionalProperties": False}]}},
        "$defs": {"person": {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}},
                             "required": ["name", "age"], "additionalProperties": False}},
        "required": ["item"], "additionalProperties": False}), True)
    n = normalize_output('{"item": {"age": 30, "name": "Ada", "ignored": true}}', fmt)
    assert n.is_valid and n.normalized_content == '{"item":{"name":"Ada","age":30}}'
    assert not normalize_output("no json at all", StructuredOutputFormat.json_object()).is_valid
    assert not normalize_output('{"answer": 3, "optional_note": null, "done": true}', StructuredOutputFormat.json_schema(
        "result", fmt.schema_json.replace("container", "x"), True)).is_valid


def test_structured_prompt_injection():
    msgs = [ChatMessage(role="system", content="Be nice."), ChatMessage(role="user", content="q")]
    assert apply_to_messages(msgs, None) is msgs or apply_to_messages(msgs, None) == msgs
    out = apply_to_messages(msgs, StructuredOutputFormat.json_object())
    assert out is not msgs and msgs[0].content == "Be nice." and "valid JSON" in "".join(m.content for m in out)
    assert StructuredOutputFormat.json_object().kind == StructuredOutputKind.JSON_OBJECT


# ---------------------------------------------------------------------------- sampling
def test_sampling_config_clone_and_presets():
    c = SamplingConfig(temperature=0.3, stop_sequences=["a"])
    d = c.clone()
    d.stop_sequences.append("b")
    d.temperature = 1.0
    assert c.stop_sequences == ["a"] and c.temperature == 0.3
    assert SamplingConfig().clone().stop_sequences is None
    assert SamplingConfig.greedy().is_greedy and not SamplingConfig.default().is_greedy
    assert (SamplingConfig.default().temperature, SamplingConfig.default().top_k, SamplingConfig.default().top_p,
            SamplingConfig.default().repetition_penalty) == (0.8, 40, 0.9, 1.1)


def test_token_sampler_behaviour():
    logits = torch.tensor([0.1, 3.0, 2.9, -1.0])
    assert TokenSampler(SamplingConfig.greedy()).sample(logits) == 1
    rep = SamplingConfig.greedy()
    rep.repetition_penalty = 2.0
    assert TokenSampler(rep).sample(logits, [1]) == 2                       # 3.0/2 < 2.9
    pres = SamplingConfig.greedy()
    pres.presence_penalty = 0.5
    assert TokenSampler(pres).sample(logits, [1]) == 2
    s1 = [TokenSampler(SamplingConfig(seed=7)).sample(logits) for _ in range(3)]
    assert s1[0] == s1[1] == s1[2]
    topk1 = SamplingConfig(temperature=1.0, top_k=1, top_p=1.0, repetition_penalty=1.0, seed=3)
    assert all(TokenSampler(topk1).sample(logits) == 1 for _ in range(5))
    minp = SamplingConfig(temperature=1.0, top_k=0, top_p=1.0, min_p=0.95, repetition_penalty=1.0, seed=1)
    assert all(TokenSampler(minp).sample(logits) == 1 for _ in range(5))
    draws = {TokenSampler(SamplingConfig(temperature=5.0, top_k=0, top_p=1.0, repetition_penalty=1.0, seed=s)).sample(logits) for s in range(40)}
    assert len(draws) >= 3
    st = SamplingConfig(stop_sequences=["END", "zz"])
    assert TokenSampler(st).check_stop_sequences("abc END tail") == ("abc ", True)
    assert TokenSampler(st).check_stop_sequences("abc") == ("abc", False)


# ---------------------------------------------------------------------------- tokenizers
def test_bpe_and_spm_tokenizers_from_gguf(tiny_qwen3_path):
    from tensorsharp_b200.models.base import ModelBase
    m = ModelBase.create(tiny_qwen3_path, "cpu")
    tok = m.tokenizer
    for s in ("Hello, world!", "tabs\tand\nnewlines", "naïve café ✓", "😀 emoji"):
        ids = tok.encode(s, add_special=False)
        assert tok.decode(ids) == s and b"".join(tok.token_bytes(i) for i in ids).decode() == s
    assert tok.is_eos(2) and not tok.is_eos(5)
    m.close()
    from tensorsharp_b200.runtime.tokenizer_spm import SentencePieceTokenizer
    extra = {"▁": -3.5, "he": -2.7, "ll": -2.5, "llo": -2.1, "▁he": -2.0, "▁hello": -1.0, "▁w": -2.8, "or": -2.6, "▁wor": -1.5,
             "ld": -2.2, "h": -4.0, "e": -4.0, "l": -4.0, "o": -4.0, "w": -4.0, "r": -4.0, "d": -4.0}
    vocab = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + list(extra)
    types = [2, 3, 3] + [6] * 256 + [1] * len(extra)
    scores = [0.0] * 259 + list(extra.values())
    spm = SentencePieceTokenizer(vocab, types, scores, bos_id=1, eos_ids=[2], add_bos=True)
    ids = spm.encode(" hello world")
    assert ids[0] == 1 and [vocab[i] for i in ids[1:]] == ["▁hello", "▁wor", "ld"]      # merges by best score
    assert spm.decode(ids[1:]) == " hello world"
    assert [vocab[i] for i in spm.encode("a</s>he", add_special=False)] == ["<0x61>", "</s>", "he"]   # control token cut out first
    z = spm.encode("hé", add_special=False)                  # é is not in the vocabulary: UTF-8 byte fallback
    assert [vocab[i] for i in z] == ["h", "<0xC3>", "<0xA9>"] and spm.decode(z) == "hé"


# ---------------------------------------------------------------------------- logging
def read_entries(provider):
    return [json.loads(l) for l in open(provider.current_file, encoding="utf-8")]


def test_file_logger_json_lines(tmp_path):
    p = FileLoggerProvider(FileLoggerOptions(directory=str(tmp_path), file_prefix="t", minimum_level="Information"))
    log = p.get_logger("Cat.Sub")
    with log_scope(RequestId="r1", Operation="op"):
        with log_scope(SessionId="s9"):
            log.info(Ev.ChatStarted, "Sent {Count} bytes to {Name}", Count=3, Name="bob")
    log.debug(Ev.ChatStarted, "dropped {X}", X=1)
    try:
        raise ValueError("boom")
    except ValueError as e:
        log.error(Ev.ChatFailed, "failed {What}", exc=e, What="it")
    p.close()
    assert os.path.basename(p.current_file).startswith("t-") and p.current_file.endswith(".jsonl")
    a, b = read_entries(p)
    assert list(a) == ["ts", "level", "category", "event", "message", "template", "props", "scope"]
    assert a["level"] == "Information" and a["category"] == "Cat.Sub" and a["event"] == {"id": 1500, "name": "ChatStarted"}
    assert a["message"] == "Sent 3 bytes to bob" and a["template"] == "Sent {Count} bytes to {Name}" and a["props"] == {"Count": 3, "Name": "bob"}
    assert list(a["scope"].items()) == [("RequestId", "r1"), ("Operation", "op"), ("SessionId", "s9")] and a["ts"].endswith("Z")
    assert b["level"] == "Error" and "ValueError: boom" in b["exception"] and "scope" not in b


def test_file_logger_rotation_overflow_and_text_format(tmp_path):
    p = FileLoggerProvider(FileLoggerOptions(directory=str(tmp_path / "rot"), file_prefix="r", max_file_size_bytes=400))
    log = p.get_logger("C")
    for i in range(12):
        log.info(None, "entry {I} " + "x" * 60, I=i)
        p.flush()
    p.close()
    files = sorted(os.listdir(tmp_path / "rot"))
    assert len(files) >= 3 and any(f.endswith("-0001.jsonl") for f in files) and any(f.count("-") == 1 for f in files)
    clock = [dt.datetime(2026, 1, 1, 23, 59, 59, tzinfo=dt.timezone.utc)]
    p = FileLoggerProvider(FileLoggerOptions(directory=str(tmp_path / "day"), file_prefix="d", flush_interval_s=30), clock=lambda: clock[0])
    log = p.get_logger("C")
    log.info(None, "before midnight")
    p.flush()
    clock[0] = dt.datetime(2026, 1, 2, 0, 0, 1, tzinfo=dt.timezone.utc)
    log.info(None, "after midnight")
    p.close()
    assert sorted(os.listdir(tmp_path / "day")) == ["d-20260101.jsonl", "d-20260102.jsonl"]
    p = FileLoggerProvider(FileLoggerOptions(directory=str(tmp_path / "of"), max_queued_entries=5, flush_interval_s=30))
    p._drain = lambda: None           # hold the writer off so the queue fills
    log = p.get_logger("C")
    for i in range(50):
        log.info(None, "n {I}", I=i)
    assert p.dropped == 45 and len(p._q) == 5 and json.loads(p._q[-1])["props"]["I"] == 49      # oldest entries were dropped
    del p._drain
    p.close()
    p = FileLoggerProvider(FileLoggerOptions(directory=str(tmp_path / "txt"), use_json_format=False))
    with log_scope(RequestId="r"):
        p.get_logger("Plain").info(Ev.ChatStarted, "Hello {Name}", Name="world")
    p.close()
    line = open(p.current_file).read().strip()
    assert " INF [1500:ChatStarted] Plain: Hello world => RequestId=r" in line and '"level":' not in line


# ---------------------------------------------------------------------------- media
def test_media_helpers(monkeypatch, tmp_path):
    assert media.select_evenly_spaced_indices(3, 8) == [0, 1, 2]
    assert media.select_evenly_spaced_indices(10, 4) == [0, 3, 6, 9]
    assert media.select_evenly_spaced_indices(9, 1) == [4]
    assert media.select_evenly_spaced_indices(0, 4) == [] and media.select_evenly_spaced_indices(5, 0) == []
    monkeypatch.delenv("VIDEO_MAX_FRAMES", raising=False)
    assert media.get_configured_max_video_frames() == 4 and media.get_configured_max_video_frames(0) == 4
    monkeypatch.setenv("VIDEO_MAX_FRAMES", "9")
    assert media.get_configured_max_video_frames() == 9
    monkeypatch.setenv("VIDEO_MAX_FRAMES", "-2")
    assert media.get_configured_max_video_frames(6) == 6
    from PIL import Image
    img = Image.new("RGBA", (4, 2), (255, 0, 0, 0))
    path = tmp_path / "a.png"
    img.save(path)
    t = media.load_image_rgb(str(path))
    assert t.shape == (2, 4, 3) and t.dtype == torch.uint8 and int(t.min()) == 255       # transparent -> white


def test_banner_colour_rules_and_layout():
    import io

    from tensorsharp_b200.runtime.banner import color_allowed, render_banner, wordmark_rows

    class Tty(io.StringIO):
        def isatty(self):
            return True
    assert color_allowed(Tty(), env={}) is True
    assert color_allowed(Tty(), env={"NO_COLOR": ""}) is False           # presence counts, whatever the value
    assert color_allowed(Tty(), env={"TERM": "dumb"}) is False
    assert color_allowed(io.StringIO(), env={}) is False                  # redirected output
    rows = wordmark_rows()
    assert len(rows) == 5 and len({len(r) for r in rows}) <= 2
    plain = render_banner(["model: x.gguf"], color=False)
    assert "\x1b[" not in plain and "model: x.gguf" in plain
    colored = render_banner(["model: x.gguf"], color=True)
    assert "\x1b[38;2;" in colored and colored.count("\x1b[0m") >= 6
    strip = __import__("re").sub(r"\x1b\[[0-9;]*m", "", colored)
    assert strip == plain
