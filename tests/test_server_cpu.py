"""Serving layer on CPU: queue, sessions, options, parsers, ModelService KV reuse with a recording
fake model, every HTTP route through in-memory exchanges, and a loopback run on a real tiny model.

Cases follow the reference's InferenceWeb.Tests (KVCacheMultiTurnIntegrationTests,
ModelServiceKVCacheTests, ModelServiceSessionTests, ServerOptionsBuilderTests,
SamplingConfigParserTests, SessionManagerTests, TextUploadHelperTests, WebUiChatPolicyTests,
RequestLoggingMiddlewareTests, StructuredOutputTests).
"""
import http.client
import json
import os
import threading
import time
from types import SimpleNamespace

import pytest
import torch

from tensorsharp_b200.runtime.chat import ChatMessage
from tensorsharp_b200.runtime.logging import FileLoggerOptions, FileLoggerProvider
from tensorsharp_b200.runtime.sampling import SamplingConfig
from tensorsharp_b200.server import parsers as P
from tensorsharp_b200.server.app import (Exchange, ServerApp, classify_client, classify_extension, prepare_text_content,
                                         serve, validate_webui_chat_request)
from tensorsharp_b200.server.inference_queue import CancellationToken, InferenceQueue
from tensorsharp_b200.server.model_service import (ModelService, PromptTooLongError, augment_with_cached_raw_tokens,
                                                   find_valid_utf8_length, resolve_prefill_chunk_size)
from tensorsharp_b200.server.options import (ServerHostingOptions, build_options, canonicalize_backend,
                                             matches_hosted_file_request, resolve_default_backend, supported_backends,
                                             try_resolve_hosted_model_request, try_validate_hosted_mmproj_request)
from tensorsharp_b200.server.sessions import DEFAULT_SESSION_ID, ChatSession, SessionManager

TEMPLATE = ("{%- for message in messages %}{{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>\\n' }}"
            "{%- endfor %}{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- endif %}")


# ---------------------------------------------------------------------------- fakes
class CharTokenizer:
    """One token per UTF-8 byte (+3), 0 = unk, 1 = bos, 2 = eos."""
    vocab_size = 300

    def encode(self, text, add_special=True):
        return [b + 3 for b in text.encode("utf-8")]

    def token_bytes(self, tid):
        return bytes([tid - 3]) if 3 <= tid < 259 else b""

    def decode(self, ids):
        return b"".join(self.token_bytes(i) for i in ids).decode("utf-8", errors="replace")

    def is_eos(self, tid):
        return tid == 2


class RecordingModel:
    """Records what the service asks of the model; emits a scripted reply then EOS."""

    def __init__(self, path="fake.gguf", device="cpu", arch="llama", supports_truncation=True, max_context=4096, **kw):
        self.path, self.arch, self.device = path, arch, device
        self.kw = kw
        self.cfg = SimpleNamespace(chat_template=TEMPLATE)
        self.tokenizer = CharTokenizer()
        self.supports_kv_truncation = supports_truncation
        self.max_context = max_context
        self.ops = []
        self.cache_len = 0
        self.script = []          # token ids still to emit
        self.closed = False

    def say(self, text):
        self.script = self.tokenizer.encode(text) + [2]

    def _logits(self):
        v = torch.full((300,), -10.0)
        v[self.script.pop(0) if self.script else 2] = 10.0
        return v

    def forward(self, tokens, want_logits=True):
        self.ops.append(("forward", len(tokens)))
        self.cache_len += len(tokens)
        return self._logits() if want_logits else None

    def forward_refill(self, tokens, chunk=2048):
        out = None
        for i in range(0, len(tokens), chunk):
            self.ops.append(("prefill", len(tokens[i:i + chunk])))
            self.cache_len += len(tokens[i:i + chunk])
        return self._logits()

    def reset_kv_cache(self):
        self.ops.append(("reset", 0))
        self.cache_len = 0

    def truncate_kv_cache(self, n):
        if not self.supports_kv_truncation and n != self.cache_len:
            raise RuntimeError("recurrent model can only truncate to its current length")
        self.ops.append(("truncate", n))
        self.cache_len = n

    def close(self):
        self.closed = True


GREEDY = SamplingConfig.greedy()


def make_service(**model_kw):
    holder = {}

    def factory(path, device, **kw):
        holder["model"] = RecordingModel(path, device, **{**model_kw, **kw})
        return holder["model"]
    svc = ModelService(model_factory=factory)
    svc.load_model("/models/fake.gguf", None, "cpu")
    return svc, holder["model"]


def run_chat(svc, history, reply, max_tokens=64, **kw):
    svc.model.say(reply)
    svc.model.ops.clear()
    items = list(svc.chat_stream_with_metrics(history, max_tokens, sampling=GREEDY, **kw))
    text = "".join(i.piece for i in items if not i.done)
    return text, items[-1]


# ---------------------------------------------------------------------------- queue
def test_queue_fifo_positions_and_release():
    q = InferenceQueue()
    t1 = q.enqueue(request_id="a")
    assert t1.is_ready and t1.position == 0 and q.is_busy
    t2, t3 = q.enqueue(request_id="b"), q.enqueue(request_id="c")
    assert (t2.position, t3.position, q.pending_count) == (1, 2, 2)
    assert not t2.is_ready
    st = q.get_status()
    assert (st.busy, st.pending_requests, st.total_processed, st.current_request_id) == (True, 2, 0, "a")
    t1.dispose()
    assert t2.is_ready and t2.position == 0 and t3.position == 1 and q.total_processed == 1
    t2.dispose()
    t3.dispose()
    assert not q.is_busy and q.total_processed == 3 and q.get_status().current_request_id is None


def test_queue_cancel_while_waiting_and_skip_on_activation():
    q = InferenceQueue()
    t1 = q.enqueue()
    ct = CancellationToken()
    t2 = q.enqueue(ct)
    t3 = q.enqueue()
    ct.cancel()
    assert q.pending_count == 1 and t3.position == 1 and t2.is_cancelled
    t0 = time.time()
    t2.wait(5.0)                       # returns at once: cancelled tickets are woken
    assert time.time() - t0 < 1.0
    t2.dispose()
    t1.dispose()
    assert t3.is_ready
    t3.dispose()
    assert q.total_processed == 2      # the cancelled one never ran


def test_queue_wakes_waiter_from_other_thread():
    q = InferenceQueue()
    t1 = q.enqueue()
    t2 = q.enqueue()
    threading.Timer(0.05, t1.dispose).start()
    t2.wait_until_ready()
    assert t2.is_ready
    t2.dispose()


# ---------------------------------------------------------------------------- sessions
def test_session_manager_contract():
    m = SessionManager()
    assert m.session_count == 1 and m.session_ids == [DEFAULT_SESSION_ID]
    a, b = m.create_session(), m.create_session()
    assert a.id != b.id and len(a.id) == 32 and m.get_session(a.id) is a
    assert m.get_session("") is m.default_session and m.get_session(None) is m.default_session
    assert m.get_session("nope") is None
    assert m.try_remove(DEFAULT_SESSION_ID) is None and m.session_count == 3
    a.kv_cache.record_append([1, 2, 3], [0.5])
    assert b.kv_cache.is_empty
    got = m.try_remove(a.id)
    assert got is a and not got.is_disposed and m.get_session(a.id) is None
    assert m.try_remove("nope") is None


def test_chat_session_dispose():
    s = ChatSession()
    assert s.last_used_at == s.created_at and s.kv_cache.is_empty and s.tracked_history == []
    s.kv_cache.record_append([1, 2], [0.1])
    s.tracked_history.append(ChatMessage(role="user", content="x"))
    s.dispose()
    s.dispose()
    assert s.is_disposed and s.kv_cache.is_empty and s.tracked_history == []
    with pytest.raises(ValueError):
        ChatSession("  ")


# ---------------------------------------------------------------------------- options / guard
def test_build_options_flags_env_and_errors(tmp_path):
    base = str(tmp_path)
    o = build_options([], base, env={})
    d = SamplingConfig()
    assert (o.default_sampling_config.temperature, o.default_sampling_config.top_k) == (d.temperature, d.top_k)
    assert o.default_web_max_tokens == 20000 and o.max_text_file_chars == 8000 and os.path.isdir(o.upload_directory)
    args = ["--temperature", "0.42", "--top-k", "12", "--top-p=0.55", "--min-p", "0.07", "--repeat-penalty", "1.4",
            "--presence-penalty", "0.2", "--frequency-penalty", "0.3", "--seed", "1234", "--stop", "</s>", "--STOP", "<|eot|>"]
    s = build_options(args, base, env={}).default_sampling_config
    assert (s.temperature, s.top_k, s.top_p, s.min_p, s.repetition_penalty, s.presence_penalty, s.frequency_penalty,
            s.seed, s.stop_sequences) == (0.42, 12, 0.55, 0.07, 1.4, 0.2, 0.3, 1234, ["</s>", "<|eot|>"])
    s = build_options(["--temperature", "0.9"], base,
                      env={"TENSORSHARP_TEMPERATURE": "0.6", "TENSORSHARP_TOP_K": "15"}).default_sampling_config
    assert (s.temperature, s.top_k, s.top_p) == (0.9, 15, d.top_p)
    for bad in (["--temperature", "not-a-number"], ["--top-k", "abc"], ["--max-tokens", "0"], ["--model"]):
        with pytest.raises(ValueError) as e:
            build_options(bad, base, env={})
        assert bad[0] in str(e.value)
    with pytest.raises(ValueError):
        build_options(["--mmproj", "p.gguf"], base, env={})
    o = build_options(["--model", "m/x.gguf", "--mmproj", "proj.gguf", "--max-tokens", "77"], base,
                      env={"MAX_TOKENS": "5", "MAX_TEXT_FILE_CHARS": "123", "TENSORSHARP_LOG_FILE": "0"})
    assert o.startup_model_path == os.path.abspath("m/x.gguf")
    assert o.startup_mmproj_path == os.path.join(os.path.dirname(os.path.abspath("m/x.gguf")), "proj.gguf")
    assert o.default_web_max_tokens == 77 and o.max_text_file_chars == 123 and not o.file_logging_enabled
    assert build_options([], base, env={"MAX_TOKENS": "5"}).default_web_max_tokens == 5
    # listener: --host / --port, then TENSORSHARP_HOST / PORT, then the first http:// entry of ASPNETCORE_URLS
    o = build_options([], base, env={"ASPNETCORE_URLS": "https://+:5001;http://*:8088"})
    assert (o.host, o.port) == ("0.0.0.0", 8088)
    o = build_options(["--port", "7000"], base, env={"ASPNETCORE_URLS": "http://localhost:8088", "PORT": "9"})
    assert (o.host, o.port) == ("localhost", 7000)
    o = build_options([], base, env={"ASPNETCORE_URLS": "http://localhost:8088", "PORT": "9", "TENSORSHARP_HOST": "10.0.0.1"})
    assert (o.host, o.port) == ("10.0.0.1", 9)
    o = build_options([], base, env={})
    assert (o.host, o.port) == ("127.0.0.1", 5000)


def test_backend_catalog():
    assert [b["value"] for b in supported_backends(lambda n: False)] == ["cpu"]
    both = supported_backends(lambda n: True)
    assert [b["value"] for b in both] == ["b200", "cpu"]
    assert resolve_default_backend("CUDA", both) == "b200" and resolve_default_backend("ggml_cuda", both) == "b200"
    assert resolve_default_backend("ggml_metal", both) == "b200"          # unsupported -> first supported
    assert resolve_default_backend("b200", supported_backends(lambda n: False)) == "cpu"
    assert canonicalize_backend("  GGML_CPU ") == "cpu" and canonicalize_backend("") is None


def test_hosted_model_guard():
    hosted = "/models/Qwen3-4B-Q8_0.gguf"
    for ok in ("Qwen3-4B-Q8_0.gguf", "qwen3-4b-q8_0", " Qwen3-4B-Q8_0 ", hosted):
        assert matches_hosted_file_request(ok, hosted, True)
    assert not matches_hosted_file_request("Qwen3-4B-Q8_0", hosted, False)
    assert not matches_hosted_file_request("other.gguf", hosted, True)
    assert try_resolve_hosted_model_request("x", None)[1].startswith("No model is hosted")
    assert try_resolve_hosted_model_request(" ", hosted)[1] == "model is required"
    assert "is not hosted by this server" in try_resolve_hosted_model_request("other", hosted)[1]
    assert try_resolve_hosted_model_request("qwen3-4b-q8_0", hosted) == (hosted, None)
    assert try_validate_hosted_mmproj_request(None, None) is None
    assert try_validate_hosted_mmproj_request("none", None) is None
    assert "without --mmproj" in try_validate_hosted_mmproj_request("p.gguf", None)
    assert "was started with mmproj 'p.gguf'" in try_validate_hosted_mmproj_request("", "/m/p.gguf")
    assert try_validate_hosted_mmproj_request("p.gguf", "/m/p.gguf") is None
    assert "is not hosted" in try_validate_hosted_mmproj_request("q.gguf", "/m/p.gguf")


# ---------------------------------------------------------------------------- parsers
def test_sampling_parsers():
    d = SamplingConfig(temperature=0.3, top_k=7, stop_sequences=["A"])
    c = P.parse_sampling_webui({}, d)
    assert c is not d and c.temperature == 0.3 and c.top_k == 7 and c.stop_sequences == ["A"]
    c.stop_sequences.append("B")
    assert d.stop_sequences == ["A"]
    c = P.parse_sampling_webui({"temperature": 1.5, "topK": 3, "top_p": 0.5, "minP": 0.1, "repetitionPenalty": 1.3,
                                "presence_penalty": 0.4, "frequencyPenalty": 0.6, "seed": 9, "stop": ["x", 3, "y"]}, d)
    assert (c.temperature, c.top_k, c.top_p, c.min_p, c.repetition_penalty, c.presence_penalty, c.frequency_penalty,
            c.seed, c.stop_sequences) == (1.5, 3, 0.5, 0.1, 1.3, 0.4, 0.6, 9, ["x", "y"])
    c = P.parse_sampling_ollama({"options": {"temperature": 0.1, "top_k": 5, "repeat_penalty": 1.2, "stop": ["\n"]},
                                 "temperature": 9}, None)
    assert (c.temperature, c.top_k, c.repetition_penalty, c.stop_sequences) == (0.1, 5, 1.2, ["\n"])
    assert P.parse_sampling_ollama({}, d).temperature == 0.3
    assert P.parse_sampling_openai({"stop": "END", "top_p": 0.2, "top_k": 99}, None).stop_sequences == ["END"]
    assert P.parse_sampling_openai({"stop": ["a", "b"]}, None).stop_sequences == ["a", "b"]
    assert P.parse_sampling_openai({"top_k": 99}, None).top_k == SamplingConfig().top_k


def test_tool_message_and_response_format_parsers(tmp_path):
    fn = {"name": "get_weather", "description": "d", "parameters": {"type": "object", "properties": {
        "city": {"type": "string", "description": "c"}, "unit": {"enum": ["c", "f"]}}, "required": ["city"]}}
    t = P.parse_tools_openai({"tools": [{"type": "function", "function": fn}, {"type": "retrieval"}]})
    assert len(t) == 1 and t[0].name == "get_weather" and t[0].required == ["city"]
    assert t[0].parameters["unit"].type == "string" and t[0].parameters["unit"].enum == ["c", "f"]
    assert P.parse_tools_ollama({"tools": [{"function": fn}, {"nofn": 1}]})[0].parameters["city"].description == "c"
    assert P.parse_tools_ollama({"tools": []}) is None and P.parse_tools_openai({}) is None
    png = "iVBORw0KGgo="
    up = str(tmp_path / "up")
    m = P.parse_messages_openai([{"role": "user", "content": [
        {"type": "text", "text": "a"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64," + png}},
        {"type": "text", "text": "b"}, {"type": "image_url", "image_url": {"url": "http://x/y.png"}}]},
        {"content": "plain"}], up)
    assert m[0].content == "a\nb" and len(m[0].image_paths) == 1 and open(m[0].image_paths[0], "rb").read()[:4] == b"\x89PNG"
    assert m[1].role == "user" and m[1].content == "plain" and m[1].image_paths is None
    o = P.parse_messages_ollama([{"role": "user", "content": "hi", "images": [png, ""]}], up)
    assert len(o[0].image_paths) == 1
    w = P.parse_messages_webui([{"role": "user", "content": "v", "imagePaths": ["a", "b"], "isVideo": True, "audioPaths": []}])
    assert w[0].image_paths == ["a", "b"] and w[0].is_video and w[0].audio_paths is None
    assert P.parse_response_format({}) == (None, None)
    assert P.parse_response_format({"response_format": {"type": "text"}}) == (None, None)
    assert P.parse_response_format({"response_format": 3})[1] == "response_format must be an object."
    assert P.parse_response_format({"response_format": {}})[1] == "response_format.type is required."
    assert P.parse_response_format({"response_format": {"type": "xml"}})[1] == "Unsupported response_format.type 'xml'."
    f, e = P.parse_response_format({"response_format": {"type": "json_schema", "json_schema": {
        "name": "n", "strict": True, "description": "d", "schema": {"type": "object"}}}})
    assert e is None and f.name == "n" and f.strict and f.description == "d" and json.loads(f.schema_json) == {"type": "object"}
    assert P.parse_response_format({"response_format": {"type": "json_schema", "name": "flat", "schema": {}}})[0].name == "flat"
    assert P.parse_response_format({"response_format": {"type": "json_schema", "json_schema": {"schema": {}}}})[1] == \
        "response_format.json_schema.name is required."
    assert P.parse_response_format({"response_format": {"type": "json_schema", "json_schema": {"name": "n"}}})[1] == \
        "response_format.json_schema.schema must be an object."


# ---------------------------------------------------------------------------- small helpers
def test_small_policies():
    assert resolve_prefill_chunk_size("b200", 20000) == 5120 and resolve_prefill_chunk_size("cuda", 100) == 100
    assert resolve_prefill_chunk_size("cpu", 20000) == 2048 and resolve_prefill_chunk_size("cpu", 0) == 0
    assert resolve_prefill_chunk_size("cpu", -4) == 0
    e = "é".encode()
    assert find_valid_utf8_length(b"ab" + e[:1]) == 2 and find_valid_utf8_length(b"ab" + e) == 4
    smile = "😀".encode()
    assert [find_valid_utf8_length(b"x" + smile[:k]) for k in range(5)] == [1, 1, 1, 1, 5]
    assert validate_webui_chat_request(None, " ") is None
    assert validate_webui_chat_request("m", None).startswith("Use /api/models/load")
    assert classify_extension(".PNG") == "image" and classify_extension(".mkv") == "video"
    assert classify_extension(".flac") == "audio" and classify_extension(".rs") == "text" and classify_extension(".bin") == "unknown"
    assert classify_client("/v1/models") == "openai" and classify_client("/api/chat/ollama") == "ollama"
    assert classify_client("/api/chat") == "webui" and classify_client("/api/tags") == "ollama" and classify_client("/") is None


def test_prepare_text_content():
    tok = CharTokenizer()
    r = prepare_text_content("abcdefghij", tok, 8, 1000)
    assert r == {"textContent": "abcd", "truncated": True, "truncateLimit": 4, "truncateUnit": "tokens",
                 "modelContextLimit": 8, "originalTokenCount": 10, "returnedTokenCount": 4}
    r = prepare_text_content("abcdefghij", None, 0, 5)
    assert (r["textContent"], r["truncated"], r["truncateUnit"], r["modelContextLimit"]) == ("abcde", True, "characters", None)
    assert prepare_text_content(None, None, 0, 5)["textContent"] == ""


# ---------------------------------------------------------------------------- augment
def test_augment_with_cached_raw_tokens():
    inc = [ChatMessage(role="user", content="hi")]
    assert augment_with_cached_raw_tokens(inc, []) == inc and augment_with_cached_raw_tokens(None, []) is None
    tracked = [ChatMessage(role="user", content="hi"),
               ChatMessage(role="assistant", content="<think>x</think>hello", raw_output_tokens=[7, 8, 9]),
               ChatMessage(role="user", content="more"),
               ChatMessage(role="assistant", content="again", raw_output_tokens=[5, 6])]
    inc = [ChatMessage(role="user", content="hi"), ChatMessage(role="assistant", content="hello"),   # parsed: differs
           ChatMessage(role="user", content="more"), ChatMessage(role="assistant", content="again"),
           ChatMessage(role="user", content="third")]
    out = augment_with_cached_raw_tokens(inc, tracked)
    assert out[1].raw_output_tokens == [7, 8, 9] and out[1].content == "hello" and out[3].raw_output_tokens == [5, 6]
    assert out[0] is inc[0] and out[4] is inc[4] and inc[1].raw_output_tokens is None
    inc[1].raw_output_tokens = [1]
    assert augment_with_cached_raw_tokens(inc, tracked)[1].raw_output_tokens == [1]       # caller's ids win
    inc[1].raw_output_tokens = None
    inc[2] = ChatMessage(role="user", content="EDITED")
    out = augment_with_cached_raw_tokens(inc, tracked)
    assert out[1].raw_output_tokens == [7, 8, 9] and out[3].raw_output_tokens is None     # stops at the edit


# ---------------------------------------------------------------------------- ModelService
def test_multi_turn_forwards_only_the_delta():
    svc, model = make_service()
    h = [ChatMessage(role="user", content="hello")]
    text, fin = run_chat(svc, h, "hi there")
    assert text == "hi there" and fin.done and fin.kv_reused_tokens == 0 and fin.eval_tokens == 8
    assert model.ops[0] == ("reset", 0) and [o for o in model.ops if o[0] == "prefill"] == [("prefill", fin.prompt_tokens)]
    assert fin.total_ns >= fin.prompt_ns > 0 and fin.eval_ns > 0
    first_prompt = fin.prompt_tokens
    # the client sends back the parsed text; the service splices the sampled ids back in
    h += [ChatMessage(role="assistant", content="hi there"), ChatMessage(role="user", content="and?")]
    text, fin = run_chat(svc, h, "ok")
    assert text == "ok"
    assert fin.kv_reused_tokens == first_prompt + 8          # whole first turn, prompt + reply
    kinds = [o for o in model.ops if o[0] in ("reset", "prefill", "truncate")]
    assert kinds[0] == ("truncate", first_prompt + 8) and kinds[1] == ("prefill", fin.prompt_tokens - fin.kv_reused_tokens)
    assert ("reset", 0) not in model.ops
    assert [m.role for m in svc.tracked_history] == ["user", "assistant", "user", "assistant"]
    assert svc.tracked_history[-1].raw_output_tokens == svc.model.tokenizer.encode("ok")


def test_edit_truncates_and_recurrent_model_resets():
    svc, model = make_service()
    h = [ChatMessage(role="user", content="hello")]
    run_chat(svc, h, "aaaa")
    h2 = [ChatMessage(role="user", content="hellO")]
    _, fin = run_chat(svc, h2, "bbbb")
    assert 0 < fin.kv_reused_tokens < fin.prompt_tokens and model.ops[0] == ("truncate", fin.kv_reused_tokens)
    svc, model = make_service(supports_truncation=False)
    h = [ChatMessage(role="user", content="hello")]
    _, f1 = run_chat(svc, h, "aaaa")
    _, fin = run_chat(svc, [ChatMessage(role="user", content="hellO")], "bbbb")
    assert fin.kv_reused_tokens == 0 and model.ops[0] == ("reset", 0)
    # pure extension needs no rewind, so it is reused even without truncation support
    h = [ChatMessage(role="user", content="hellO"), ChatMessage(role="assistant", content="bbbb"),
         ChatMessage(role="user", content="x")]
    _, fin = run_chat(svc, h, "c")
    assert fin.kv_reused_tokens > 0 and ("reset", 0) not in model.ops


def test_exact_match_reuses_cached_logits():
    svc, model = make_service()
    h = [ChatMessage(role="user", content="hello")]
    model.say("zz")
    it = svc.chat_stream_with_metrics(h, 0, sampling=GREEDY)         # max_tokens 0: prefill only
    fin = list(it)[-1]
    assert fin.eval_tokens == 0
    model.ops.clear()
    model.script = []
    _, fin = run_chat(svc, h, "", max_tokens=0)
    assert fin.kv_reused_tokens == fin.prompt_tokens and not [o for o in model.ops if o[0] in ("prefill", "forward")]


def test_stop_sequences_utf8_pieces_and_cancel():
    svc, model = make_service()
    cfg = SamplingConfig.greedy()
    cfg.stop_sequences = ["STOP"]
    model.say("ab😀cd STOP tail")
    items = list(svc.chat_stream_with_metrics([ChatMessage(role="user", content="q")], 64, sampling=cfg))
    pieces = [i.piece for i in items if not i.done]
    assert "😀" in pieces and all("�" not in p for p in pieces)
    assert "".join(pieces) == "ab😀cd STOP"            # chat emits the piece that completed the stop text
    model.say("one STOP two")
    g = [i.piece for i in svc.generate_stream("q", None, 64, sampling=cfg) if not i.done]
    assert "".join(g) == "one STO"                     # generate stops before emitting it
    ct = CancellationToken()
    model.say("abcdefgh")
    out = []
    for it in svc.chat_stream_with_metrics([ChatMessage(role="user", content="q2")], 64, ct, GREEDY):
        if not it.done:
            out.append(it.piece)
            if len(out) == 3:
                ct.cancel()
    assert "".join(out) == "abc" and it.done and it.eval_tokens == 3


def test_prompt_truncated_to_context_and_chunked_prefill():
    svc, model = make_service(max_context=64)
    long = "x" * 100
    _, fin = run_chat(svc, [ChatMessage(role="user", content=long)], "y", max_tokens=16)
    assert fin.prompt_tokens == 48 and ("prefill", 48) in model.ops
    with pytest.raises(PromptTooLongError):
        list(svc.chat_stream_with_metrics([ChatMessage(role="user", content=long)], 64, sampling=GREEDY))
    svc, model = make_service(max_context=100000)
    _, fin = run_chat(svc, [ChatMessage(role="user", content="x" * 5000)], "y", max_tokens=4)
    pre = [o for o in model.ops if o[0] == "prefill"]
    assert [n for _, n in pre][:2] == [2048, 2048] and sum(n for _, n in pre) == fin.prompt_tokens


def test_sessions_switching_reset_and_dispose():
    svc, model = make_service()
    a, b = ChatSession(), ChatSession()
    assert svc.active_session is None
    run_chat(svc, [ChatMessage(role="user", content="one")], "r1", session=a)
    assert svc.active_session is a and not a.kv_cache.is_empty
    run_chat(svc, [ChatMessage(role="user", content="two")], "r2", session=b)
    assert svc.active_session is b and a.kv_cache.is_empty and model.ops[0] == ("reset", 0)
    svc.reset_session(a)
    assert not b.kv_cache.is_empty
    svc.reset_session(None)
    svc.dispose_session(b)
    svc.dispose_session(b)
    svc.dispose_session(None)
    assert b.is_disposed and svc.active_session is None and model.ops[-1] == ("reset", 0)
    with pytest.raises(RuntimeError):
        list(svc.chat_stream_with_metrics([ChatMessage(role="user", content="x")], 4, session=b))
    ModelService().invalidate_kv_cache()          # no model loaded: must not raise


def test_load_model_replaces_previous_and_resets_state():
    svc, m1 = make_service()
    run_chat(svc, [ChatMessage(role="user", content="one")], "r1")
    svc.load_model("/models/other.gguf", None, "cuda")
    assert m1.closed and svc.loaded_model_name == "other.gguf" and svc.loaded_backend == "b200"
    assert svc.model.device == "cuda" and svc.kv_cache.is_empty and svc.tracked_history == []
    assert svc.is_model_already_loaded("OTHER.gguf")


# ---------------------------------------------------------------------------- HTTP (in-memory exchanges)
def make_app(tmp_path, log=False, **model_kw):
    model_path = tmp_path / "Fake-1B.gguf"
    model_path.write_bytes(b"GGUF")
    holder = {}

    def factory(path, device, **kw):
        holder["model"] = RecordingModel(path, device, **{**model_kw, **kw})
        return holder["model"]
    opts = ServerHostingOptions(startup_model_path=str(model_path), default_backend="cpu",
                                supported_backends=supported_backends(lambda n: False),
                                upload_directory=str(tmp_path / "uploads"), log_directory=str(tmp_path / "logs"),
                                default_sampling_config=SamplingConfig.greedy(), default_web_max_tokens=64)
    provider = FileLoggerProvider(FileLoggerOptions(directory=str(tmp_path / "logs"), minimum_level="Debug")) if log else None
    app = ServerApp(opts, svc=ModelService(model_factory=factory), log_provider=provider, queue_poll_s=0.02)
    return app, holder, provider


def call(app, method, path, body=None, headers=None, raw=None):
    data = raw if raw is not None else (json.dumps(body).encode() if body is not None else b"")
    ex = Exchange(method, path, headers or {}, data)
    app.handle(ex)
    return ex


def lines(ex):
    return [json.loads(l) for l in ex.text.splitlines() if l.strip()]


def sse(ex):
    return [l[6:] for l in ex.text.split("\n\n") if l.startswith("data: ")]


def test_plain_routes(tmp_path):
    app, holder, _ = make_app(tmp_path)
    ex = call(app, "GET", "/")
    assert ex.status == 200 and ex.text == '"TensorSharp.Server is running"' and len(ex.response_headers["X-TensorSharp-Request-Id"]) == 12
    assert call(app, "GET", "/", headers={"X-TensorSharp-Request-Id": "abc"}).response_headers["X-TensorSharp-Request-Id"] == "abc"
    assert call(app, "GET", "/api/version").text == '{"version":"0.1.0"}'
    tags = json.loads(call(app, "GET", "/api/tags").text)["models"][0]
    assert list(tags) == ["name", "model", "size", "modified_at"] and tags["name"] == "Fake-1B" and tags["size"] == 4
    assert json.loads(call(app, "GET", "/v1/models").text) == {"object": "list", "data": [
        {"id": "Fake-1B", "object": "model", "owned_by": "local"}]}
    assert call(app, "GET", "/api/queue/status").text == '{"busy":false,"pending_requests":0,"total_processed":0}'
    show = call(app, "POST", "/api/show", {"model": "fake-1b"})
    assert json.loads(show.text)["model_info"] == {"file": "Fake-1B.gguf", "size": 4}
    assert call(app, "POST", "/api/show", {}).status == 400 and call(app, "POST", "/api/show", {"model": "zzz"}).status == 404
    m = json.loads(call(app, "GET", "/api/models").text)
    assert m["models"] == ["Fake-1B.gguf"] and m["loaded"] is None and m["defaultBackend"] == "cpu" and m["defaultMaxTokens"] == 64
    assert list(m) == ["models", "mmProjModels", "loaded", "loadedMmProj", "loadedBackend", "defaultBackend",
                       "supportedBackends", "architecture", "hostedModelPath", "hostedMmProjPath", "defaultMaxTokens"]
    page = call(app, "GET", "/some/ui/route")
    assert page.status == 200 and page.content_type == "text/html" and b"<html" in page.chunks[0]
    assert call(app, "POST", "/api/show", raw=b"{not json").status == 400


def test_sessions_routes_and_model_load(tmp_path):
    app, holder, _ = make_app(tmp_path)
    s = json.loads(call(app, "POST", "/api/sessions").text)
    assert list(s) == ["sessionId", "createdAt"] and s["createdAt"].endswith("Z") and len(s["createdAt"]) == 28
    assert call(app, "DELETE", "/api/sessions/" + DEFAULT_SESSION_ID).status == 400
    assert call(app, "DELETE", "/api/sessions/nope").status == 404
    assert json.loads(call(app, "DELETE", "/api/sessions/" + s["sessionId"]).text) == {"ok": True, "sessionId": s["sessionId"]}
    assert app.queue.total_processed == 1
    assert call(app, "POST", "/api/chat", {"messages": []}).text == '{"error":"No model loaded"}'
    bad = call(app, "POST", "/api/models/load", {"model": "Fake-1B.gguf", "backend": "cuda"})
    assert bad.status == 400 and "not supported on this machine" in bad.text
    assert call(app, "POST", "/api/models/load", {"model": "other.gguf"}).status == 400
    assert call(app, "POST", "/api/models/load", {"model": "Fake-1B.gguf", "mmproj": "p.gguf"}).status == 400
    ok = json.loads(call(app, "POST", "/api/models/load", {"model": "Fake-1B.gguf"}).text)
    assert ok == {"ok": True, "model": "Fake-1B.gguf", "loadedMmProj": None, "architecture": "llama"}


def test_ollama_generate_and_chat(tmp_path):
    app, holder, _ = make_app(tmp_path)
    assert call(app, "POST", "/api/generate", {"prompt": "x"}).status == 400
    assert call(app, "POST", "/api/generate", {"model": "nope", "stream": False}).status == 404
    err = lines(call(app, "POST", "/api/generate", {"model": "nope"}))
    assert err[-1]["done_reason"] == "error" and "not hosted" in err[-1]["error"]
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    holder["model"].say("héllo")
    ex = call(app, "POST", "/api/generate", {"model": "Fake-1B", "prompt": "p", "stream": False, "options": {"num_predict": 32}})
    r = json.loads(ex.text)
    assert list(r) == ["model", "created_at", "response", "done", "done_reason", "total_duration", "prompt_eval_count",
                       "prompt_eval_duration", "eval_count", "eval_duration", "prompt_cache_hit_tokens", "prompt_cache_hit_ratio"]
    assert r["response"] == "héllo" and r["model"] == "Fake-1B.gguf" and r["eval_count"] == 6 and "h\\u00E9llo" in ex.text
    holder["model"].say("ab")
    ex = call(app, "POST", "/api/generate", {"model": "Fake-1B", "prompt": "p"})
    assert ex.content_type == "application/x-ndjson" and ex.response_headers["Cache-Control"] == "no-cache"
    ls = lines(ex)
    assert [l["response"] for l in ls] == ["a", "b", ""] and ls[-1]["done"] and ls[-1]["done_reason"] == "stop"
    assert call(app, "POST", "/api/chat/ollama", {"model": "Fake-1B"}).status == 400
    holder["model"].say("yo")
    ls = lines(call(app, "POST", "/api/chat/ollama", {"model": "Fake-1B", "messages": [{"role": "user", "content": "q"}]}))
    assert [l["message"]["content"] for l in ls] == ["y", "o", ""] and "thinking" not in ls[0]["message"]
    assert ls[-1]["done_reason"] == "stop" and ls[-1]["prompt_eval_count"] > 0
    holder["model"].say("yo")
    r = json.loads(call(app, "POST", "/api/chat/ollama", {"model": "Fake-1B", "stream": False,
                                                          "messages": [{"role": "user", "content": "q"}]}).text)
    assert r["message"] == {"role": "assistant", "content": "yo"} and r["done_reason"] == "stop"
    assert r["prompt_cache_hit_tokens"] > 0          # the same conversation prefix was cached


def test_ollama_chat_with_thinking_and_tools(tmp_path):
    app, holder, _ = make_app(tmp_path, arch="qwen3")
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"properties": {"a": {"type": "integer"}}}}}]
    reply = 'hm</think>Sure.<tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>'
    holder["model"].say(reply)
    ls = lines(call(app, "POST", "/api/chat/ollama", {"model": "Fake-1B", "think": True, "tools": tools,
                                                      "messages": [{"role": "user", "content": "q"}]}))
    assert "".join(l["message"].get("thinking", "") for l in ls) == "hm"
    assert "".join(l["message"]["content"] for l in ls).strip() == "Sure."
    assert ls[-1]["done_reason"] == "tool_calls"
    assert ls[-1]["message"]["tool_calls"] == [{"function": {"name": "f", "arguments": {"a": 1}}}]
    holder["model"].say(reply)
    r = json.loads(call(app, "POST", "/api/chat/ollama", {"model": "Fake-1B", "think": True, "tools": tools, "stream": False,
                                                          "messages": [{"role": "user", "content": "q2"}]}).text)
    assert r["message"]["thinking"] == "hm" and r["message"]["content"].strip() == "Sure." and r["done_reason"] == "tool_calls"


def test_openai_chat_completions(tmp_path):
    app, holder, _ = make_app(tmp_path)
    e = json.loads(call(app, "POST", "/v1/chat/completions", {"messages": []}).text)
    assert e == {"error": {"message": "model is required", "type": "invalid_request_error"}}
    assert call(app, "POST", "/v1/chat/completions", {"model": "m"}).status == 400
    assert call(app, "POST", "/v1/chat/completions", {"model": "zz", "messages": []}).status == 404
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    msgs = [{"role": "user", "content": "q"}]
    holder["model"].say("hi!")
    ex = call(app, "POST", "/v1/chat/completions", {"model": "Fake-1B", "messages": msgs, "max_tokens": 16})
    r = json.loads(ex.text)
    assert list(r) == ["id", "object", "created", "model", "choices", "usage"] and r["object"] == "chat.completion"
    assert r["id"].startswith("chatcmpl-") and len(r["id"]) == 30
    assert r["choices"] == [{"index": 0, "message": {"role": "assistant", "content": "hi!"}, "finish_reason": "stop"}]
    u = r["usage"]
    assert u["total_tokens"] == u["prompt_tokens"] + 3 and u["prompt_tokens_details"] == {"cached_tokens": 0}
    holder["model"].say("ab")
    ex = call(app, "POST", "/v1/chat/completions", {"model": "Fake-1B", "messages": msgs, "stream": True})
    ev = sse(ex)
    assert ex.content_type == "text/event-stream" and ev[-1] == "[DONE]"
    chunks = [json.loads(x) for x in ev[:-1]]
    assert [c["choices"][0]["delta"]["content"] for c in chunks] == ["a", "b", None]
    assert chunks[0]["choices"][0]["delta"]["role"] is None and chunks[-1]["choices"][0]["finish_reason"] == "stop"
    assert chunks[-1]["usage"]["prompt_tokens_details"]["cached_tokens"] > 0
    # tool call through the OpenAI surface
    app2, holder2, _ = make_app(tmp_path, arch="qwen3")
    app2.svc.load_model(app2.options.startup_model_path, None, "cpu")
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"properties": {"a": {"type": "integer"}}}}}]
    holder2["model"].say('<tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>')
    r = json.loads(call(app2, "POST", "/v1/chat/completions", {"model": "Fake-1B", "messages": msgs, "tools": tools}).text)
    tc = r["choices"][0]["message"]["tool_calls"][0]
    assert r["choices"][0]["finish_reason"] == "tool_calls" and tc["type"] == "function" and tc["id"].startswith("call_")
    assert len(tc["id"]) == 24 and tc["function"] == {"name": "f", "arguments": '{"a":1}'}
    assert "thinking" not in r["choices"][0]["message"]


def test_openai_structured_outputs(tmp_path):
    app, holder, _ = make_app(tmp_path)
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    msgs = [{"role": "user", "content": "q"}]
    base = {"model": "Fake-1B", "messages": msgs}
    schema = {"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": ["string", "null"]}},
              "required": ["a", "b"], "additionalProperties": False}
    rf = {"type": "json_schema", "json_schema": {"name": "n", "strict": True, "schema": schema}}
    assert "think=true" in call(app, "POST", "/v1/chat/completions", {**base, "response_format": rf, "think": True}).text
    t = [{"type": "function", "function": {"name": "f"}}]
    assert "combined with tools" in call(app, "POST", "/v1/chat/completions", {**base, "response_format": rf, "tools": t}).text
    bad = {"type": "json_schema", "json_schema": {"name": "n", "strict": True, "schema": {"anyOf": []}}}
    e = call(app, "POST", "/v1/chat/completions", {**base, "response_format": bad})
    assert e.status == 400 and "details" in json.loads(e.text)["error"]
    holder["model"].say('```json\n{"b": "x", "a": 3, "extra": 1}\n```')
    r = json.loads(call(app, "POST", "/v1/chat/completions", {**base, "response_format": rf}).text)
    assert r["choices"][0]["message"]["content"] == '{"a":3,"b":"x"}'
    # the instruction reached the prompt
    assert "JSON" in app.svc.tracked_history[0].content or "JSON" in app.svc.tracked_history[-2].content
    holder["model"].say("no json here")
    e = call(app, "POST", "/v1/chat/completions", {**base, "response_format": rf})
    assert e.status == 422 and json.loads(e.text)["error"]["type"] == "invalid_response_error"
    holder["model"].say('{"a": 1, "b": null}')
    ex = call(app, "POST", "/v1/chat/completions", {**base, "response_format": {"type": "json_object"}, "stream": True})
    ev = sse(ex)
    first = json.loads(ev[0])
    assert first["choices"][0]["delta"] == {"role": "assistant", "content": '{"a":1,"b":null}'} and ev[-1] == "[DONE]"
    holder["model"].say("nope")
    assert call(app, "POST", "/v1/chat/completions", {**base, "response_format": rf, "stream": True}).status == 422


def test_webui_chat_sse_sessions_and_kv_reuse(tmp_path):
    app, holder, _ = make_app(tmp_path)
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    assert call(app, "POST", "/api/chat", {"model": "x", "messages": []}).status == 400
    assert call(app, "POST", "/api/chat", {"sessionId": "nope", "messages": []}).status == 404
    holder["model"].say("hey")
    ex = call(app, "POST", "/api/chat", {"messages": [{"role": "user", "content": "q"}], "maxTokens": 8})
    ev = [json.loads(x) for x in sse(ex)]
    assert ex.response_headers["Connection"] == "keep-alive" and [e["token"] for e in ev[:-1]] == ["h", "e", "y"]
    d = ev[-1]
    assert list(d) == ["done", "tokenCount", "elapsed", "tokPerSec", "aborted", "error", "sessionId", "promptTokens",
                       "kvReusedTokens", "kvReusePercent"]
    assert d["tokenCount"] == 3 and d["sessionId"] == DEFAULT_SESSION_ID and d["kvReusedTokens"] == 0 and d["error"] is None
    holder["model"].say("k")
    ev = [json.loads(x) for x in sse(call(app, "POST", "/api/chat", {"messages": [
        {"role": "user", "content": "q"}, {"role": "assistant", "content": "hey"}, {"role": "user", "content": "w"}]}))]
    assert ev[-1]["kvReusedTokens"] == d["promptTokens"] + 3 and ev[-1]["kvReusePercent"] > 40
    sid = json.loads(call(app, "POST", "/api/sessions").text)["sessionId"]
    holder["model"].say("n")
    ev = [json.loads(x) for x in sse(call(app, "POST", "/api/chat", {"sessionId": sid, "messages": [{"role": "user", "content": "q"}]}))]
    assert ev[-1]["sessionId"] == sid and ev[-1]["kvReusedTokens"] == 0
    holder["model"].say("n")
    ev = [json.loads(x) for x in sse(call(app, "POST", "/api/chat", {"sessionId": sid, "newChat": True,
                                                                    "messages": [{"role": "user", "content": "q"}]}))]
    assert ev[-1]["kvReusedTokens"] == 0          # newChat dropped the session's cache

    class Boom(RecordingModel):
        def forward(self, tokens, want_logits=True):
            raise RuntimeError("device lost")
    app.svc._model.__class__ = Boom
    holder["model"].say("abc")
    ev = [json.loads(x) for x in sse(call(app, "POST", "/api/chat", {"messages": [{"role": "user", "content": "zz"}]}))]
    assert ev[-1]["done"] and ev[-1]["error"] == "device lost"


def test_queue_progress_is_streamed_while_waiting(tmp_path):
    app, holder, _ = make_app(tmp_path)
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    holder["model"].say("z")
    blocker = app.queue.enqueue(request_id="blocker")
    threading.Timer(0.15, blocker.dispose).start()
    ls = lines(call(app, "POST", "/api/chat/ollama", {"model": "Fake-1B", "messages": [{"role": "user", "content": "q"}]}))
    waiting = [l for l in ls if "queue_position" in l]
    assert len(waiting) >= 2 and waiting[0]["queue_position"] == 1 and waiting[0]["queue_pending"] == 1
    assert ls[-1]["done"] and "".join(l["message"]["content"] for l in ls) == "z"


def test_upload_route(tmp_path):
    app, holder, _ = make_app(tmp_path)
    assert call(app, "POST", "/api/upload", raw=b"x", headers={"Content-Type": "text/plain"}).status == 400
    bnd = "XbOuNd"

    def form(name, data):
        return (f"--{bnd}\r\nContent-Disposition: form-data; name=\"file\"; filename=\"{name}\"\r\n"
                "Content-Type: application/octet-stream\r\n\r\n").encode() + data + f"\r\n--{bnd}--\r\n".encode()
    h = {"Content-Type": f"multipart/form-data; boundary={bnd}"}
    r = json.loads(call(app, "POST", "/api/upload", raw=form("notes.TXT", b"a" * 9000), headers=h).text)
    assert r["ok"] and r["mediaType"] == "text" and r["truncated"] and r["truncateUnit"] == "characters"
    assert len(r["textContent"]) == 8000 and r["fileName"] == "notes.TXT" and r["path"].endswith(".txt")
    r = json.loads(call(app, "POST", "/api/upload", raw=form("p.png", b"\x89PNG\r\n\x00\xff"), headers=h).text)
    assert r == {"ok": True, "path": r["path"], "mediaType": "image", "fileName": "p.png"}
    assert open(r["path"], "rb").read() == b"\x89PNG\r\n\x00\xff"
    none = call(app, "POST", "/api/upload", raw=f"--{bnd}\r\nContent-Disposition: form-data; name=\"x\"\r\n\r\nv\r\n--{bnd}--\r\n".encode(), headers=h)
    assert none.status == 400 and "No file uploaded" in none.text


def test_request_logging(tmp_path):
    app, holder, provider = make_app(tmp_path, log=True)
    call(app, "GET", "/api/version", headers={"X-TensorSharp-Request-Id": "rid-1"})
    call(app, "POST", "/api/show", {})
    call(app, "GET", "/api/queue/status")
    app._routes.append(("GET", "/boom", lambda ex: (_ for _ in ()).throw(RuntimeError("kaput"))))
    assert call(app, "GET", "/boom").status == 500
    provider.close()
    entries = [json.loads(l) for l in open(provider.current_file, encoding="utf-8")]
    http = [e for e in entries if e["category"].endswith("RequestLoggingMiddleware")]
    v = [e for e in http if e["scope"]["RequestId"] == "rid-1"]
    assert [e["event"]["name"] for e in v] == ["HttpRequestStarted", "HttpRequestCompleted"]
    assert v[0]["scope"] == {"RequestId": "rid-1", "Operation": "GET /api/version", "Client": "ollama"}
    rejected = [e for e in http if e["event"]["name"] == "HttpRequestRejected"]
    assert rejected[0]["level"] == "Warning" and rejected[0]["props"]["StatusCode"] == 400
    assert all(e["level"] == "Debug" for e in http if e["scope"]["Operation"] == "GET /api/queue/status")
    failed = [e for e in http if e["event"]["name"] == "HttpRequestFailed"]
    assert failed[0]["level"] == "Error" and "kaput" in failed[0]["exception"]


# ---------------------------------------------------------------------------- loopback on a real tiny model
def test_http_loopback_with_tiny_qwen3(tmp_path, tiny_qwen3_path):
    opts = build_options(["--model", tiny_qwen3_path, "--backend", "cpu", "--port", "0", "--temperature", "0", "--top-k", "0",
                          "--top-p", "1", "--repeat-penalty", "1"], str(tmp_path), env={"TENSORSHARP_LOG_FILE": "0"})
    app = ServerApp(opts)
    httpd = serve(app, "127.0.0.1", 0)
    port = httpd.server_address[1]
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    try:
        name = os.path.basename(tiny_qwen3_path)

        def post(path, body):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
            c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
            r = c.getresponse()
            data = r.read().decode()
            c.close()
            return r, data
        r, data = post("/api/generate", {"model": name, "prompt": "Hello", "stream": False, "options": {"num_predict": 6}})
        g = json.loads(data)
        assert r.status == 200 and g["done"] and g["eval_count"] <= 6 and g["prompt_eval_count"] > 5
        r, data = post("/api/chat", {"messages": [{"role": "user", "content": "Hello"}], "maxTokens": 5})
        assert r.getheader("Transfer-Encoding") == "chunked" and r.getheader("Content-Type") == "text/event-stream"
        ev = [json.loads(l[6:]) for l in data.split("\n\n") if l.startswith("data: ")]
        assert ev[-1]["done"] and ev[-1]["error"] is None and ev[-1]["promptTokens"] > 5
        reply = "".join(e.get("token", "") for e in ev)
        r, data = post("/api/chat", {"messages": [{"role": "user", "content": "Hello"}, {"role": "assistant", "content": reply},
                                                  {"role": "user", "content": "again"}], "maxTokens": 3})
        ev2 = [json.loads(l[6:]) for l in data.split("\n\n") if l.startswith("data: ")]
        assert ev2[-1]["kvReusedTokens"] >= ev[-1]["promptTokens"]        # second turn re-used the first
        r, data = post("/v1/chat/completions", {"model": name, "messages": [{"role": "user", "content": "Hi"}], "max_tokens": 4})
        assert r.status == 200 and json.loads(data)["usage"]["completion_tokens"] <= 4
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/api/queue/status")
        q = json.loads(c.getresponse().read())
        assert q["busy"] is False and q["total_processed"] == 4
    finally:
        httpd.shutdown()
        httpd.server_close()
        app.svc.close()


def test_queue_capacity_and_preferred_slots():
    """With capacity N the queue runs N tickets at once, hands a ticket its preferred running slot when that
    slot is free, and makes the next one wait with position 1 until a slot is released."""
    q = InferenceQueue(capacity=3)
    a, b, c = q.enqueue(prefer_slot=2), q.enqueue(prefer_slot=2), q.enqueue()
    assert (a.is_ready, b.is_ready, c.is_ready) == (True, True, True)
    assert a.slot == 2 and sorted([b.slot, c.slot]) == [0, 1]
    d = q.enqueue(prefer_slot=2)
    assert not d.is_ready and d.position == 1 and q.pending_count == 1
    assert q.slot_for_thread() in (0, 1, 2)
    a.dispose()
    assert d.is_ready and d.slot == 2 and q.pending_count == 0
    for t in (b, c, d):
        t.dispose()
    st = q.get_status()
    assert st.busy is False and st.total_processed == 4


def test_metrics_endpoint_counts_generations(tmp_path):
    from tensorsharp_b200.server.metrics import METRICS
    app, holder, _ = make_app(tmp_path)
    app.svc.load_model(app.options.startup_model_path, None, "cpu")
    METRICS.reset()
    r = call(app, "POST", "/api/generate", {"model": app.svc.loaded_model_name, "prompt": "hi", "stream": False, "options": {"num_predict": 3}})
    assert r.status == 200
    assert call(app, "POST", "/api/generate", {"prompt": "x"}).status == 400
    m = call(app, "GET", "/metrics")
    assert m.status == 200 and m.content_type.startswith("text/plain")
    vals = {l.split(" ")[0]: l.split(" ")[1] for l in m.text.splitlines() if l and not l.startswith("#")}
    assert vals["tensorsharp_generations_total"] == "1" and int(vals["tensorsharp_generated_tokens_total"]) == json.loads(r.text)["eval_count"]
    assert int(vals["tensorsharp_prompt_tokens_total"]) >= 1 and vals["tensorsharp_queue_busy"] == "0"
    assert vals['tensorsharp_http_responses_total{client="ollama",status="2xx"}'] == "1"
    assert vals['tensorsharp_http_responses_total{client="ollama",status="4xx"}'] == "1"
    assert "# TYPE tensorsharp_generated_tokens_total counter" in m.text


@pytest.mark.parametrize("family", ["qwen35", "nemotron_h"])
def test_second_turn_on_models_that_cannot_truncate(tmp_path, family):
    """A model with recurrent state refuses to shrink its cache, but the second turn of a chat only extends it: the
    re-use plan keeps the whole cache and the turn must go through (server path and CLI path, real synthetic models)."""
    from tensorsharp_b200.cli.main import apply_reuse_plan
    from tensorsharp_b200.models import synth
    from tensorsharp_b200.models.base import ModelBase
    from tensorsharp_b200.runtime.kv_cache import KVCache, ReusePlanKind
    path = str(tmp_path / f"{family}.gguf")
    getattr(synth, "write_" + family)(path, device="cpu")
    opts = build_options(["--model", path, "--backend", "cpu", "--port", "0", "--temperature", "0", "--top-k", "0",
                          "--top-p", "1", "--repeat-penalty", "1"], str(tmp_path), env={"TENSORSHARP_LOG_FILE": "0"})
    app = ServerApp(opts)
    httpd = serve(app, "127.0.0.1", 0)
    port = httpd.server_address[1]
    th = threading.Thread(target=httpd.serve_forever, daemon=True)
    th.start()
    try:
        def chat(messages, n):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
            c.request("POST", "/api/chat", json.dumps({"messages": messages, "maxTokens": n}), {"Content-Type": "application/json"})
            data = c.getresponse().read().decode()
            c.close()
            return [json.loads(l[6:]) for l in data.split("\n\n") if l.startswith("data: ")]
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)       # the first request that names the model loads it
        c.request("POST", "/api/generate", json.dumps({"model": os.path.basename(path), "prompt": "Hi", "stream": False,
                                                       "options": {"num_predict": 2}}), {"Content-Type": "application/json"})
        assert c.getresponse().status == 200
        c.close()
        ev = chat([{"role": "user", "content": "Hello"}], 4)
        assert ev[-1]["done"] and ev[-1]["error"] is None
        reply = "".join(e.get("token", "") for e in ev)
        ev2 = chat([{"role": "user", "content": "Hello"}, {"role": "assistant", "content": reply},
                    {"role": "user", "content": "again"}], 3)
        assert ev2[-1]["done"] and ev2[-1]["error"] is None
        assert ev2[-1]["kvReusedTokens"] >= ev[-1]["promptTokens"]
    finally:
        httpd.shutdown()
        httpd.server_close()
        app.svc.close()
    # the CLI's re-use path on the same kind of model
    model = ModelBase.create(path, device="cpu")
    assert not model.supports_kv_truncation
    kv = KVCache()
    first = [5, 6, 7, 8, 9]
    logits = model.forward(first)
    kv.record_append(first, logits)
    second = first + [10, 11]
    plan = kv.plan_reuse(second, model.supports_kv_truncation)
    assert plan.kind == ReusePlanKind.PARTIAL_REUSE and plan.reused_prefix_length == len(first)
    out = apply_reuse_plan(model, kv, plan, second)
    assert out is not None and kv.count == len(second)
    with pytest.raises(RuntimeError):
        model.truncate_kv_cache(2)                  # a real shrink is still refused
    model.close()
