"""Structured outputs: ``response_format`` = ``json_object`` / ``json_schema``.

Rules follow TensorSharp.Runtime/StructuredOutputs.cs: the instruction is merged into (or
prepended as) the system message (:54-118); a strict schema must be a JSON object schema
with ``additionalProperties: false`` and every property listed in ``required``, only local
``$ref``s, no ``allOf / not / if / pattern / min* / max* ...`` keywords, at most depth 10,
5000 properties, 1000 enum values, 120000 name / enum / const characters (:157-238,
:350-553); the model's answer is located (whole text, fenced block, or the first balanced
``{...}`` that parses, :914-1010), coerced to the schema (property order follows the schema,
missing nullable properties become ``null``, integral doubles become integers, unknown
properties are dropped, ``enum`` / ``const`` checked, :555-790) and re-serialised compactly.
"""
from __future__ import annotations

import enum
import json
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .chat import ChatMessage, dotnet_json


class StructuredOutputKind(enum.Enum):
    TEXT = "text"
    JSON_OBJECT = "json_object"
    JSON_SCHEMA = "json_schema"


@dataclass
class StructuredOutputFormat:
    kind: StructuredOutputKind
    name: Optional[str] = None
    schema_json: Optional[str] = None
    strict: bool = False
    description: Optional[str] = None

    @staticmethod
    def json_object() -> "StructuredOutputFormat":
        return StructuredOutputFormat(StructuredOutputKind.JSON_OBJECT)

    @staticmethod
    def json_schema(name, schema_json, strict=False, description=None) -> "StructuredOutputFormat":
        return StructuredOutputFormat(StructuredOutputKind.JSON_SCHEMA, name, schema_json, strict, description)


@dataclass
class ValidationResult:
    is_valid: bool = False
    errors: List[str] = field(default_factory=list)
    normalized_content: Optional[str] = None

    @property
    def error_message(self) -> str:
        return " ".join(self.errors)


_NO_FENCES = ("Do not include Markdown code fences, explanations, or extra text before or after the JSON.")


def build_instruction(fmt: Optional[StructuredOutputFormat]) -> str:
    if fmt is None:
        return ""
    if fmt.kind == StructuredOutputKind.JSON_OBJECT:
        return "You must answer with valid JSON. Return exactly one JSON object and nothing else. " + _NO_FENCES
    out = ["You must answer with valid JSON that matches the provided JSON Schema exactly. ",
           "Return exactly one JSON object and nothing else. ", _NO_FENCES,
           "\n\nStructured output schema name: ", fmt.name or ""]
    if fmt.description and fmt.description.strip():
        out += ["\nSchema description: ", fmt.description.strip()]
    out += ["\nRules:", "\n- Include every required property.",
            "\n- Do not add properties that are not defined in the schema.",
            "\n- Use `null` only when the schema allows it.", "\n- Keep property order aligned with the schema.",
            "\n\nJSON Schema:", "\n", fmt.schema_json or ""]
    return "".join(out)


def _clone(m: ChatMessage) -> ChatMessage:
    return ChatMessage(role=m.role, content=m.content, image_paths=list(m.image_paths) if m.image_paths else m.image_paths,
                       audio_paths=list(m.audio_paths) if m.audio_paths else m.audio_paths, is_video=m.is_video,
                       tool_calls=list(m.tool_calls) if m.tool_calls else m.tool_calls, thinking=m.thinking)


def apply_to_messages(messages: Optional[List[ChatMessage]], fmt: Optional[StructuredOutputFormat]) -> List[ChatMessage]:
    if fmt is None:
        return messages
    instr = build_instruction(fmt)
    if messages and messages[0].role in ("system", "developer"):
        first = _clone(messages[0])
        first.content = instr if not (first.content or "").strip() else first.content.rstrip() + "\n\n" + instr
        return [first] + [_clone(m) for m in messages[1:]]
    return [ChatMessage(role="system", content=instr)] + [_clone(m) for m in (messages or [])]


# ------------------------------------------------------------------------------------------ schema validation
_TYPES = {"string", "number", "integer", "boolean", "object", "array", "null"}
_UNSUPPORTED = {"allOf", "not", "dependentRequired", "dependentSchemas", "if", "then", "else", "minLength", "maxLength",
                "pattern", "format", "minimum", "maximum", "multipleOf", "patternProperties", "minItems", "maxItems"}


def _resolve_ref(root, ref) -> Tuple[Optional[Any], Optional[str]]:
    if not ref or not str(ref).strip():
        return None, "Encountered an empty `$ref`."
    if ref == "#":
        return root, None
    if not ref.startswith("#/"):
        return None, f"Only local refs are supported, but received `{ref}`."
    cur = root
    for seg in ref[2:].split("/"):
        seg = seg.replace("~1", "/").replace("~0", "~")
        if not isinstance(cur, dict) or seg not in cur:
            return None, f"Could not resolve `$ref` path `{ref}`."
        cur = cur[seg]
    return cur, None


def _type_list(schema, path, errors) -> set:
    types = set()
    if "type" not in schema:
        return types
    t = schema["type"]
    if isinstance(t, str):
        if t in _TYPES:
            types.add(t)
        else:
            errors.append(f"{path}: unsupported type `{t}`.")
    elif isinstance(t, list):
        for item in t:
            if not isinstance(item, str):
                errors.append(f"{path}: `type` arrays may only contain strings.")
            elif item in _TYPES:
                types.add(item)
            else:
                errors.append(f"{path}: unsupported type `{item}`.")
    else:
        errors.append(f"{path}: `type` must be a string or array of strings.")
    return types


def _has_type(schema, name) -> bool:
    t = schema.get("type") if isinstance(schema, dict) else None
    return t == name or (isinstance(t, list) and name in t)


def _object_like(schema, root) -> bool:
    if not isinstance(schema, dict):
        return False
    if "$ref" in schema:
        tgt, _ = _resolve_ref(root, schema["$ref"])
        if tgt is not None:
            return _object_like(tgt, root)
    return "properties" in schema or "additionalProperties" in schema or _has_type(schema, "object")


def _allows_object(schema, root) -> bool:
    if "$ref" in schema:
        tgt, _ = _resolve_ref(root, schema["$ref"])
        return tgt is not None and _allows_object(tgt, root)
    if "type" in schema and _has_type(schema, "object"):
        return True
    if "type" in schema and isinstance(schema["type"], str):
        return False
    return "properties" in schema or "additionalProperties" in schema


def _allows_null(schema, root) -> bool:
    if not isinstance(schema, dict):
        return False
    if "$ref" in schema:
        tgt, _ = _resolve_ref(root, schema["$ref"])
        return tgt is not None and _allows_null(tgt, root)
    if "type" in schema:
        t = schema["type"]
        if isinstance(t, str):
            return t == "null"
        if isinstance(t, list):
            return "null" in t
    return any(_allows_null(v, root) for v in schema.get("anyOf", []) if isinstance(schema.get("anyOf"), list))


class _Ctx:
    def __init__(self, root, errors):
        self.root, self.errors = root, errors
        self.active_refs: set = set()
        self.props = self.enums = self.chars = 0


def _validate_node(schema, path, depth, is_root, ctx: _Ctx) -> None:
    if len(ctx.errors) >= 16:
        return
    if depth > 10:
        ctx.errors.append(f"Schema nesting exceeds the supported depth of 10 at {path}.")
        return
    if not isinstance(schema, dict):
        return
    for k in schema:
        if k in _UNSUPPORTED:
            ctx.errors.append(f"{path}: `{k}` is not supported by structured outputs.")
    if "enum" in schema:
        if not isinstance(schema["enum"], list):
            ctx.errors.append(f"{path}: `enum` must be an array.")
        else:
            for item in schema["enum"]:
                ctx.enums += 1
                if isinstance(item, str):
                    ctx.chars += len(item)
            if isinstance(schema.get("const"), str):
                ctx.chars += len(schema["const"])
    elif isinstance(schema.get("const"), str):
        ctx.chars += len(schema["const"])
    if "$ref" in schema:
        ref = schema["$ref"]
        tgt, err = _resolve_ref(ctx.root, ref)
        if tgt is None:
            ctx.errors.append(f"{path}: {err}")
            return
        if ref in ctx.active_refs:
            return
        ctx.active_refs.add(ref)
        _validate_node(tgt, f"{path}->$ref({ref})", depth + 1, False, ctx)
        ctx.active_refs.discard(ref)
        return
    if "anyOf" in schema:
        if is_root:
            ctx.errors.append("Structured outputs do not allow `anyOf` at the root schema.")
        any_of = schema["anyOf"]
        if not isinstance(any_of, list) or not any_of:
            ctx.errors.append(f"{path}: `anyOf` must be a non-empty array.")
            return
        for i, v in enumerate(any_of):
            _validate_node(v, f"{path}.anyOf[{i}]", depth + 1, False, ctx)
    types = _type_list(schema, path, ctx.errors)
    if _object_like(schema, ctx.root):
        if schema.get("additionalProperties", None) is not False:
            ctx.errors.append(f"{path}: `additionalProperties: false` is required for every object schema.")
        names = []
        if "properties" in schema:
            if not isinstance(schema["properties"], dict):
                ctx.errors.append(f"{path}: `properties` must be an object.")
            else:
                for n, sub in schema["properties"].items():
                    names.append(n)
                    ctx.props += 1
                    ctx.chars += len(n)
                    _validate_node(sub, f"{path}.properties.{n}", depth + 1, False, ctx)
        if not isinstance(schema.get("required"), list):
            ctx.errors.append(f"{path}: `required` must be an array listing every property.")
        else:
            req = [r for r in schema["required"] if isinstance(r, str)]
            for n in names:
                if n not in req:
                    ctx.errors.append(f"{path}: property `{n}` must be listed in `required`.")
            for r in dict.fromkeys(req):
                if r not in names:
                    ctx.errors.append(f"{path}: `required` contains unknown property `{r}`.")
    if "items" in schema or "array" in types:
        if "items" not in schema:
            ctx.errors.append(f"{path}: array schemas must define `items`.")
        else:
            _validate_node(schema["items"], f"{path}.items", depth + 1, False, ctx)
    if "$defs" in schema:
        if not isinstance(schema["$defs"], dict):
            ctx.errors.append(f"{path}: `$defs` must be an object.")
        else:
            for n, sub in schema["$defs"].items():
                ctx.chars += len(n)
                _validate_node(sub, f"{path}.$defs.{n}", depth + 1, False, ctx)


def validate_schema(fmt: Optional[StructuredOutputFormat]) -> ValidationResult:
    if fmt is None or fmt.kind != StructuredOutputKind.JSON_SCHEMA:
        return ValidationResult(True)
    errors: List[str] = []
    missing = False
    if not (fmt.name or "").strip():
        errors.append("response_format.json_schema.name is required.")
        missing = True
    if not (fmt.schema_json or "").strip():
        errors.append("response_format.json_schema.schema is required.")
        missing = True
    if not fmt.strict:
        errors.append("response_format.json_schema.strict must be true.")
    if missing:
        return ValidationResult(False, errors)
    try:
        root = json.loads(fmt.schema_json)
    except ValueError as exc:
        errors.append("response_format.json_schema.schema is not valid JSON: " + str(exc))
        return ValidationResult(False, errors)
    if not isinstance(root, dict):
        errors.append("Structured outputs require the schema root to be a JSON object.")
        return ValidationResult(False, errors)
    if "anyOf" in root:
        errors.append("Structured outputs do not allow `anyOf` at the root schema.")
    if not _allows_object(root, root):
        errors.append("Structured outputs require the schema root to describe a JSON object.")
    ctx = _Ctx(root, errors)
    _validate_node(root, "$", 1, True, ctx)
    if ctx.props > 5000:
        errors.append("Structured outputs allow at most 5000 object properties across the schema.")
    if ctx.enums > 1000:
        errors.append("Structured outputs allow at most 1000 enum values across the schema.")
    if ctx.chars > 120000:
        errors.append("Structured outputs allow at most 120000 total characters across names, enum values, and const values.")
    return ValidationResult(not errors, errors)


# ------------------------------------------------------------------------------------------ output normalisation
_FENCE = re.compile(r"```(?:json)?\s*(.*?)\s*```", re.I | re.S)


def _parse_object(candidate: str) -> Optional[dict]:
    if not candidate or not candidate.strip():
        return None
    try:
        v = json.loads(candidate)
    except ValueError:
        return None
    return v if isinstance(v, dict) else None


def _balanced_object(text: str, start: int) -> Optional[str]:
    in_str = esc = False
    depth = 0
    for i in range(start, len(text)):
        ch = text[i]
        if esc:
            esc = False
            continue
        if ch == "\\" and in_str:
            esc = True
            continue
        if ch == '"':
            in_str = not in_str
            continue
        if in_str:
            continue
        if ch == "{":
            depth += 1
        elif ch == "}":
            depth -= 1
        if depth == 0:
            return text[start:i + 1]
    return None


def extract_json_object(raw: str) -> Tuple[Optional[dict], Optional[str]]:
    t = raw.strip()
    v = _parse_object(t)
    if v is not None:
        return v, None
    for m in _FENCE.finditer(t):
        v = _parse_object(m.group(1).strip())
        if v is not None:
            return v, None
    for i, ch in enumerate(t):
        if ch == "{":
            cand = _balanced_object(t, i)
            v = _parse_object(cand) if cand else None
            if v is not None:
                return v, None
    return None, "The model response did not contain a valid JSON object."


_FAIL = object()


def _json_equal(a, b) -> bool:
    if isinstance(a, bool) != isinstance(b, bool):
        return False
    if isinstance(a, (int, float)) and isinstance(b, (int, float)):
        return float(a) == float(b)
    if type(a) != type(b):
        return False
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_json_equal(a[k], b[k]) for k in a)
    if isinstance(a, list):
        return len(a) == len(b) and all(_json_equal(x, y) for x, y in zip(a, b))
    return a == b


def _check_enum_const(schema, value, errors, path) -> bool:
    if value is None:
        return True
    if "const" in schema and not _json_equal(value, schema["const"]):
        errors.append(f"{path}: value does not match the schema const.")
        return False
    if "enum" in schema and not any(_json_equal(value, e) for e in schema["enum"]):
        errors.append(f"{path}: value is not in the schema enum.")
        return False
    return True


def _normalize(value, schema, root, path, depth, errors):
    if depth > 128:
        errors.append(f"{path}: response exceeded the supported normalization depth.")
        return _FAIL
    if not isinstance(schema, dict):
        return value
    if "$ref" in schema:
        tgt, err = _resolve_ref(root, schema["$ref"])
        if tgt is None:
            errors.append(f"{path}: {err}")
            return _FAIL
        return _normalize(value, tgt, root, path, depth + 1, errors)
    if "anyOf" in schema:
        for variant in schema["anyOf"]:
            out = _normalize(value, variant, root, path, depth + 1, [])
            if out is not _FAIL:
                return out
        errors.append(f"{path}: value did not match any schema in `anyOf`.")
        return _FAIL
    type_errors: List[str] = []
    types = _type_list(schema, path, type_errors)
    if "null" in types and value is None:
        return None
    if _object_like(schema, root):
        if not isinstance(value, dict):
            errors.append(f"{path}: expected an object.")
            return _FAIL
        props = schema.get("properties")
        out: Dict[str, Any] = {}
        if isinstance(props, dict):
            for name, sub in props.items():
                if name in value:
                    child = _normalize(value[name], sub, root, f"{path}.{name}", depth + 1, errors)
                    if child is _FAIL:
                        return _FAIL
                    out[name] = child
                elif _allows_null(sub, root):
                    out[name] = None
                else:
                    errors.append(f"{path}: missing required property `{name}`.")
                    return _FAIL
        return out if _check_enum_const(schema, out, errors, path) else _FAIL
    if "items" in schema or _has_type(schema, "array"):
        if not isinstance(value, list):
            errors.append(f"{path}: expected an array.")
            return _FAIL
        if "items" not in schema:
            return value
        arr = []
        for i, item in enumerate(value):
            child = _normalize(item, schema["items"], root, f"{path}[{i}]", depth + 1, errors)
            if child is _FAIL:
                return _FAIL
            arr.append(child)
        return arr if _check_enum_const(schema, arr, errors, path) else _FAIL
    # primitives
    out = _FAIL
    is_num = isinstance(value, (int, float)) and not isinstance(value, bool)
    if not types:
        out = value
    elif "string" in types and isinstance(value, str):
        out = value
    elif "boolean" in types and isinstance(value, bool):
        out = value
    elif "integer" in types and is_num:
        if isinstance(value, int):
            out = value
        elif abs(value - round(value)) < 1e-9:
            out = int(round(value))
        else:
            errors.append(f"{path}: expected an integer.")
            return _FAIL
    elif "number" in types and is_num:
        out = value
    elif "null" in types and value is None:
        return None
    else:
        errors.append(f"{path}: value does not match the schema type.")
        errors.extend(type_errors)
        return _FAIL
    return out if _check_enum_const(schema, out, errors, path) else _FAIL


def normalize_output(raw: Optional[str], fmt: Optional[StructuredOutputFormat]) -> ValidationResult:
    if fmt is None:
        return ValidationResult(True, [], raw or "")
    if not raw or not raw.strip():
        return ValidationResult(False, ["The model returned an empty response."])
    if fmt.kind == StructuredOutputKind.JSON_OBJECT:
        obj, err = extract_json_object(raw)
        if obj is None:
            return ValidationResult(False, [err])
        return ValidationResult(True, [], dotnet_json(obj))
    sv = validate_schema(fmt)
    if not sv.is_valid:
        return ValidationResult(False, list(sv.errors))
    obj, err = extract_json_object(raw)
    if obj is None:
        return ValidationResult(False, [err])
    schema = json.loads(fmt.schema_json)
    errors: List[str] = []
    out = _normalize(obj, schema, schema, "$", 1, errors)
    if out is _FAIL:
        return ValidationResult(False, errors)
    if not isinstance(out, dict):
        return ValidationResult(False, ["Structured outputs require a JSON object response."])
    return ValidationResult(True, [], dotnet_json(out))
