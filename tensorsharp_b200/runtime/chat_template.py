"""Chat prompt rendering: the GGUF file's Jinja template when it renders, otherwise the
hardcoded per-architecture renderers.

Output text is matched to TensorSharp.Runtime/ChatTemplate.cs: RenderQwen3 :66, RenderQwen35
:112, RenderGemma3 :309, RenderFromGgufTemplate :337-373 (Qwen3.5 without thinking and
Mistral 3 always use the hardcoded renderer; Jinja output is right-trimmed; Gemma 4 without
thinking gets an empty thought block appended; any Jinja failure falls back), Jinja context
:412-501, multimodal token injection :507, RenderMistral3 :568, RenderHarmony :605,
RenderGemma4 :665 with tool declarations :742.
"""
from __future__ import annotations

import datetime as _dt
import sys
from typing import Any, Dict, List, Optional

from .chat import ChatMessage, ToolCall, ToolFunction, dotnet_json
from .jinja import Jinja2Template

QWEN35_FAMILY = ("qwen35", "qwen35moe", "qwen3next", "qwen3vl", "qwen3vlmoe")


def _tool_call_json(tc: ToolCall) -> str:
    return dotnet_json({"name": tc.name, "arguments": tc.arguments})


def render_qwen3(messages: List[ChatMessage], add_generation_prompt: bool = True,
                 tools: Optional[List[ToolFunction]] = None, enable_thinking: bool = False) -> str:
    out = []
    if tools:
        out.append("<|im_start|>system\nYou are a helpful assistant with access to the following functions. "
                   "Use them if required -\n")
        out.append(dotnet_json(list(tools)))
        out.append("<|im_end|>\n")
    for m in messages:
        out.append(f"<|im_start|>{m.role}\n")
        for tc in (m.tool_calls or []):
            out.append(f"\n<tool_call>\n{_tool_call_json(tc)}\n</tool_call>")
        out.append(f"{m.content if m.content is not None else ''}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
        if enable_thinking:
            out.append("<think>\n")
    return "".join(out)


def _tool_params_dict(tool: ToolFunction, required_default_all: bool = False) -> Dict[str, Any]:
    props: Dict[str, Any] = {}
    for k, p in (tool.parameters or {}).items():
        d: Dict[str, Any] = {"type": p.type or "string"}
        if p.description:
            d["description"] = p.description
        if p.enum:
            d["enum"] = list(p.enum)
        props[k] = d
    out: Dict[str, Any] = {"type": "object", "properties": props}
    if tool.required:
        out["required"] = list(tool.required)
    elif required_default_all and tool.parameters:
        out["required"] = list(tool.parameters.keys())
    return out


def _split_qwen35_assistant(m: ChatMessage):
    content = m.content or ""
    reasoning = m.thinking or ""
    if reasoning:
        return reasoning.strip(), content
    close = content.find("</think>")
    if close < 0:
        return "", content
    open_ = content.rfind("<think>", 0, close + 1)
    if open_ < 0:
        return "", content
    reasoning = content[open_ + len("<think>"):close].strip()
    return reasoning, content[close + len("</think>"):].lstrip("\r\n")


def _fmt_qwen35_arg(v) -> str:
    if isinstance(v, str):
        return v
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (dict, list)):
        return dotnet_json(v)
    return "null" if v is None else str(v)


def render_qwen35(messages: List[ChatMessage], add_generation_prompt: bool = True, enable_thinking: bool = False,
                  tools: Optional[List[ToolFunction]] = None) -> str:
    out: List[str] = []
    has_system = bool(messages) and messages[0].role == "system"
    start = 0
    if tools:
        out.append("<|im_start|>system\n# Tools\n\nYou have access to the following functions:\n\n<tools>")
        for t in tools:
            out.append("\n")
            out.append(dotnet_json({"type": "function", "function": {
                "name": t.name, "description": t.description or "", "parameters": _tool_params_dict(t)}},
                indented=True))
        out.append("\n</tools>\n\n")
        out.append("If you choose to call a function ONLY reply in the following format with NO suffix:\n\n")
        out.append("<tool_call>\n<function=example_function_name>\n<parameter=example_parameter_1>\nvalue_1\n</parameter>\n")
        out.append("<parameter=example_parameter_2>\nThis is the value for the second parameter\nthat can span\n"
                   "multiple lines\n</parameter>\n</function>\n</tool_call>\n\n")
        out.append("<IMPORTANT>\nReminder:\n- Function calls MUST follow the specified format: an inner "
                   "<function=...></function> block must be nested within <tool_call></tool_call> XML tags\n")
        out.append("- Required parameters MUST be specified\n")
        out.append("- You may provide optional reasoning for your function call in natural language BEFORE the "
                   "function call, but NOT after\n")
        out.append("- If there is no function call available, answer the question like normal with your current "
                   "knowledge and do not tell the user about function calls\n</IMPORTANT>")
        if has_system:
            sys_c = (messages[0].content or "").strip()
            if sys_c:
                out.append("\n\n" + sys_c)
            start = 1
        out.append("<|im_end|>\n")
    elif has_system:
        out.append(f"<|im_start|>system\n{(messages[0].content or '').strip()}<|im_end|>\n")
        start = 1
    n = len(messages)
    for i in range(start, n):
        m = messages[i]
        last = i == n - 1
        prefill = last and m.role == "assistant"
        if m.role == "assistant":
            out.append("<|im_start|>assistant\n")
            reasoning, content = _split_qwen35_assistant(m)
            if not enable_thinking or reasoning:
                out.append("<think>\n")
                if reasoning:
                    out.append(reasoning)
                out.append("\n</think>\n\n")
            if m.tool_calls:
                if content:
                    out.append(content)
                for j, tc in enumerate(m.tool_calls):
                    if j == 0 and content.strip():
                        out.append("\n\n")
                    elif j > 0:
                        out.append("\n")
                    out.append(f"<tool_call>\n<function={tc.name}>\n")
                    for k, v in (tc.arguments or {}).items():
                        out.append(f"<parameter={k}>\n{_fmt_qwen35_arg(v)}\n</parameter>\n")
                    out.append("</function>\n</tool_call>")
            else:
                out.append(content)
            if not prefill:
                out.append("<|im_end|>\n")
        elif m.role == "tool":
            first_tool = i == start or messages[i - 1].role != "tool"
            last_tool = i == n - 1 or messages[i + 1].role != "tool"
            if first_tool:
                out.append("<|im_start|>user")
            out.append(f"\n<tool_response>\n{(m.content or '').strip()}\n</tool_response>")
            if last_tool:
                out.append("<|im_end|>\n")
        else:
            out.append(f"<|im_start|>{m.role}\n")
            for _ in (m.image_paths or []):
                out.append("<|vision_start|><|image_pad|><|vision_end|>")
            out.append(f"{(m.content or '').strip()}<|im_end|>\n")
        if last and not prefill:
            out.append("<|im_start|>assistant\n")
            out.append("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n")
    return "".join(out)


def render_gemma3(messages: List[ChatMessage], add_generation_prompt: bool = True) -> str:
    out = []
    for m in messages:
        role = "model" if m.role == "assistant" else m.role
        out.append(f"<start_of_turn>{role}\n")
        for _ in (m.image_paths or []):
            out.append("<start_of_image>")
        out.append(f"{m.content if m.content is not None else ''}<end_of_turn>\n")
    if add_generation_prompt:
        out.append("<start_of_turn>model\n")
    return "".join(out)


def render_mistral3(messages: List[ChatMessage], add_generation_prompt: bool = True) -> str:
    out = []
    start = 0
    if messages and messages[0].role == "system":
        out.append(f"[SYSTEM_PROMPT]{messages[0].content or ''}[/SYSTEM_PROMPT]")
        start = 1
    for m in messages[start:]:
        if m.role == "user":
            out.append(f"[INST]{m.content or ''}[/INST]")
        elif m.role == "assistant":
            out.append(m.content or "")
    return "".join(out)


def render_harmony(messages: List[ChatMessage], add_generation_prompt: bool = True,
                   today: Optional[str] = None) -> str:
    out = []
    start = 0
    developer = None
    if messages and messages[0].role in ("system", "developer"):
        developer = messages[0].content
        start = 1
    out.append("<|start|>system<|message|>You are ChatGPT, a large language model trained by OpenAI.\n")
    out.append("Knowledge cutoff: 2024-06\n")
    out.append(f"Current date: {today or _dt.datetime.now().strftime('%Y-%m-%d')}\n\n")
    out.append("Reasoning: medium\n\n")
    out.append("# Valid channels: analysis, commentary, final. Channel must be included for every message.<|end|>")
    if developer:
        out.append(f"<|start|>developer<|message|># Instructions\n\n{developer}<|end|>")
    for m in messages[start:]:
        if m.role == "assistant":
            out.append(f"<|start|>assistant<|channel|>final<|message|>{m.content or ''}<|end|>")
        else:
            out.append(f"<|start|>{m.role}<|message|>{m.content or ''}<|end|>")
    if add_generation_prompt:
        out.append("<|start|>assistant")
    return "".join(out)


_Q = '<|"|>'


def _gemma4_tool_declaration(tool: ToolFunction) -> str:
    out = [f"<|tool>declaration:{tool.name}{{", f"description:{_Q}{tool.description or ''}{_Q}", ",parameters:{"]
    comma = False
    if tool.parameters:
        out.append("properties:{")
        first = True
        for key in sorted(tool.parameters):
            p = tool.parameters[key]
            if not first:
                out.append(",")
            first = False
            out.append(f"{key}:{{")
            has = False
            if p.description:
                out.append(f"description:{_Q}{p.description}{_Q}")
                has = True
            if p.enum and (p.type or "string").lower() == "string":
                if has:
                    out.append(",")
                out.append("enum:[" + ",".join(f"{_Q}{e}{_Q}" for e in p.enum) + "]")
                has = True
            if has:
                out.append(",")
            out.append(f"type:{_Q}{(p.type or 'string').upper()}{_Q}}}")
        out.append("}")
        comma = True
    if tool.required:
        if comma:
            out.append(",")
        out.append("required:[" + ",".join(f"{_Q}{r}{_Q}" for r in tool.required) + "]")
        comma = True
    if comma:
        out.append(",")
    out.append(f"type:{_Q}OBJECT{_Q}}}")
    out.append("}<tool|>")
    return "".join(out)


def _gemma4_arg(v) -> str:
    if isinstance(v, str):
        return f"{_Q}{v}{_Q}"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if isinstance(v, float):
        return str(int(v)) if v == int(v) else repr(v)
    if isinstance(v, dict):
        return "{" + ",".join(f"{k}:{_gemma4_arg(v[k])}" for k in sorted(v)) + "}"
    if isinstance(v, list):
        return "[" + ",".join(_gemma4_arg(x) for x in v) + "]"
    return "null" if v is None else str(v)


def _gemma4_tool_call(tc: ToolCall) -> str:
    args = tc.arguments or {}
    return f"<|tool_call>call:{tc.name}{{" + ",".join(f"{k}:{_gemma4_arg(args[k])}" for k in sorted(args)) + "}<tool_call|>"


def strip_gemma4_thinking(text: str) -> str:
    out = []
    while True:
        s = text.find("<|channel>")
        if s < 0:
            out.append(text)
            break
        out.append(text[:s])
        e = text.find("<channel|>", s)
        if e < 0:
            break
        text = text[e + 10:]
    return "".join(out).strip()


def render_gemma4(messages: List[ChatMessage], add_generation_prompt: bool = True,
                  tools: Optional[List[ToolFunction]] = None, enable_thinking: bool = False) -> str:
    out = ["<bos>"]
    has_system = bool(messages) and messages[0].role in ("system", "developer")
    start = 0
    if has_system or tools or enable_thinking:
        out.append("<|turn>system\n")
        if enable_thinking:
            out.append("<|think|>\n")
        if has_system:
            out.append((messages[0].content or "").strip())
            start = 1
        for t in (tools or []):
            out.append(_gemma4_tool_declaration(t))
        out.append("<turn|>\n")
    for m in messages[start:]:
        role = "model" if m.role == "assistant" else m.role
        out.append(f"<|turn>{role}\n")
        if m.role == "assistant" and m.tool_calls is not None:
            for tc in m.tool_calls:
                out.append(_gemma4_tool_call(tc))
            if m.content:
                out.append(strip_gemma4_thinking(m.content))
        elif m.role == "tool":
            out.append((m.content or "").strip())
        elif m.role == "assistant":
            out.append(strip_gemma4_thinking(m.content or "").strip())
        else:
            if m.image_paths is not None:
                if m.is_video:
                    out.append("<|video>")
                out.extend("<|image>" for _ in m.image_paths)
            out.extend("<|audio>" for _ in (m.audio_paths or []))
            out.append((m.content or "").strip())
        out.append("<turn|>\n")
    if add_generation_prompt:
        out.append("<|turn>model\n")
        if not enable_thinking:
            out.append("<|channel>thought\n<channel|>")
    return "".join(out)


def render_hardcoded(messages, add_generation_prompt=True, architecture=None, tools=None, enable_thinking=False) -> str:
    a = architecture or ""
    if a == "gemma3":
        return render_gemma3(messages, add_generation_prompt)
    if a == "gemma4":
        return render_gemma4(messages, add_generation_prompt, tools, enable_thinking)
    if a in ("gptoss", "gpt-oss"):
        return render_harmony(messages, add_generation_prompt)
    if a in QWEN35_FAMILY:
        return render_qwen35(messages, add_generation_prompt, enable_thinking, tools)
    if a == "mistral3":
        return render_mistral3(messages, add_generation_prompt)
    return render_qwen3(messages, add_generation_prompt, tools, enable_thinking)


def inject_multimodal_tokens(messages: List[ChatMessage], architecture: Optional[str]) -> List[ChatMessage]:
    out = []
    for m in messages:
        if not (m.image_paths or m.audio_paths):
            out.append(m)
            continue
        pre = []
        if architecture == "gemma4":
            if m.is_video and m.image_paths is not None:
                pre.append("<|video>")
            pre.extend("<|image>" for _ in (m.image_paths or []))
            pre.extend("<|audio>" for _ in (m.audio_paths or []))
        elif architecture == "gemma3":
            pre.extend("<start_of_image>" for _ in (m.image_paths or []))
        elif architecture in QWEN35_FAMILY:
            pre.extend("<|vision_start|><|image_pad|><|vision_end|>" for _ in (m.image_paths or []))
        elif architecture == "mistral3":
            pre.extend("[IMG]" for _ in (m.image_paths or []))
        out.append(ChatMessage(role=m.role, content="".join(pre) + (m.content or ""), image_paths=m.image_paths,
                               audio_paths=m.audio_paths, is_video=m.is_video))
    return out


def build_jinja_context(messages, add_generation_prompt, architecture, tools=None, enable_thinking=False) -> Dict[str, Any]:
    msgs = []
    for m in messages:
        d: Dict[str, Any] = {"role": m.role, "content": m.content or ""}
        if m.tool_calls:
            d["tool_calls"] = [{"function": {"name": tc.name, "arguments": tc.arguments or {}}} for tc in m.tool_calls]
        msgs.append(d)
    ctx: Dict[str, Any] = {"messages": msgs, "add_generation_prompt": add_generation_prompt,
                           "bos_token": "<bos>" if architecture == "gemma4" else "", "eos_token": ""}
    if enable_thinking:
        ctx["enable_thinking"] = True
    if tools:
        ctx["tools"] = [{"type": "function", "function": {"name": t.name, "description": t.description or "",
                                                           "parameters": _tool_params_dict(t, True)}} for t in tools]
    return ctx


def render_from_gguf_template(template: Optional[str], messages: List[ChatMessage], add_generation_prompt: bool = True,
                              architecture: Optional[str] = None, tools: Optional[List[ToolFunction]] = None,
                              enable_thinking: bool = False, log=None) -> str:
    if architecture in QWEN35_FAMILY and not enable_thinking:
        return render_hardcoded(messages, add_generation_prompt, architecture, tools, enable_thinking)
    if architecture == "mistral3":
        return render_hardcoded(messages, add_generation_prompt, architecture, tools, enable_thinking)
    if template and template.strip():
        try:
            pre = inject_multimodal_tokens(messages, architecture)
            ctx = build_jinja_context(pre, add_generation_prompt, architecture, tools, enable_thinking)
            result = Jinja2Template(template).render(ctx).rstrip()
            if result:
                if architecture == "gemma4" and add_generation_prompt and not enable_thinking:
                    block = "<|channel>thought\n<channel|>"
                    if not result.endswith(block):
                        if not result.endswith("\n"):
                            result += "\n"
                        result += block
                return result
        except Exception as exc:  # noqa: BLE001 - any template failure falls back to the hardcoded renderer
            (log or (lambda s: print(s, file=sys.stderr)))(
                f"[ChatTemplate] Jinja2 rendering failed for architecture '{architecture}': {exc}; "
                "falling back to the hardcoded template.")
    return render_hardcoded(messages, add_generation_prompt, architecture, tools, enable_thinking)
