"""A self-contained Jinja2-subset interpreter for GGUF chat templates.

Covers what chat templates shipped in GGUF files use (the same subset as
TensorSharp.Runtime/Jinja2Template.cs:88-162 lexer with ``{%- -%}`` trimming, :473-485 loop
variables, :581-1300 expressions, tests, filters and methods): ``for`` (tuple unpacking,
inline ``if`` filter, ``else``, ``loop.*``), ``if / elif / else``, ``set`` (including
``namespace`` attribute assignment and block ``set``), ``macro`` / ``call``-free use,
comments; expressions with ternaries, ``and / or / not``, comparisons, ``in / not in``,
``is [not] <test>``, ``~ + - * / // %``, unary minus, list / dict literals, indexing,
slices, attribute access, method calls, filters, ``namespace()``, ``range()``,
``raise_exception()``, ``strftime_now()``.  ``selectattr / rejectattr / select / reject /
map`` are implemented rather than stubbed.  ``tojson`` writes ``", "`` / ``": "``
separators with .NET-style string escaping and ignores ``indent``, as the reference does.
"""
from __future__ import annotations

import datetime as _dt
import re
from typing import Any, Callable, Dict, List, Optional, Tuple

from .chat import _esc_str


class TemplateError(Exception):
    pass


class _Undefined:
    __slots__ = ()

    def __bool__(self):
        return False

    def __str__(self):
        return ""

    def __iter__(self):
        return iter(())

    def __len__(self):
        return 0

    def __eq__(self, other):
        return isinstance(other, _Undefined) or other is None

    def __hash__(self):
        return 0

    def __repr__(self):
        return "Undefined"


UNDEFINED = _Undefined()


class Namespace:
    def __init__(self, **kw):
        self.__dict__.update(kw)


class _LoopCtx:
    def __init__(self, items: List[Any]):
        self.items = items
        self.index0 = 0

    @property
    def index(self):
        return self.index0 + 1

    @property
    def first(self):
        return self.index0 == 0

    @property
    def last(self):
        return self.index0 == len(self.items) - 1

    @property
    def length(self):
        return len(self.items)

    @property
    def revindex(self):
        return len(self.items) - self.index0

    @property
    def revindex0(self):
        return len(self.items) - self.index0 - 1

    @property
    def previtem(self):
        return self.items[self.index0 - 1] if self.index0 > 0 else UNDEFINED

    @property
    def nextitem(self):
        return self.items[self.index0 + 1] if self.index0 + 1 < len(self.items) else UNDEFINED


# ------------------------------------------------------------------------------------------ lexer
_TOKEN_RE = re.compile(r"""
    (?P<ws>\s+)
  | (?P<num>\d+\.\d+|\d+)
  | (?P<str>"(?:\\.|[^"\\])*"|'(?:\\.|[^'\\])*')
  | (?P<name>[A-Za-z_][A-Za-z0-9_]*)
  | (?P<op>==|!=|<=|>=|//|\*\*|[-+*/%~<>=().,\[\]{}:|])
""", re.X | re.S)


def _tokenize_expr(src: str) -> List[Tuple[str, str]]:
    out, pos = [], 0
    while pos < len(src):
        m = _TOKEN_RE.match(src, pos)
        if not m:
            raise TemplateError(f"unexpected character {src[pos]!r} in expression {src!r}")
        pos = m.end()
        kind = m.lastgroup
        if kind == "ws":
            continue
        out.append((kind, m.group(kind)))
    out.append(("eof", ""))
    return out


def _unescape(s: str) -> str:
    body = s[1:-1]
    return re.sub(r"\\(.)", lambda m: {"n": "\n", "t": "\t", "r": "\r", "\\": "\\", "'": "'", '"': '"'}.get(
        m.group(1), "\\" + m.group(1)), body)


def _split_template(src: str) -> List[Tuple[str, str]]:
    """-> [(kind, text)] with kind in {text, var, stmt}; applies ``-`` whitespace control."""
    out: List[Tuple[str, str]] = []
    pos = 0
    pat = re.compile(r"\{\{-?|\{%-?|\{#-?")
    trim_next = False
    while True:
        m = pat.search(src, pos)
        if not m:
            text = src[pos:]
            if trim_next:
                text = text.lstrip()
            if text:
                out.append(("text", text))
            break
        text = src[pos:m.start()]
        if trim_next:
            text = text.lstrip()
        opener = m.group(0)
        if opener.endswith("-"):
            text = text.rstrip()
        if text:
            out.append(("text", text))
        kind = {"{{": "var", "{%": "stmt", "{#": "comment"}[opener[:2]]
        closer = {"var": "}}", "stmt": "%}", "comment": "#}"}[kind]
        end = _find_closer(src, m.end(), closer)
        if end < 0:
            raise TemplateError(f"unclosed {opener!r} tag")
        body = src[m.end():end]
        trim_next = body.endswith("-")
        if trim_next:
            body = body[:-1]
        if kind != "comment":
            out.append((kind, body.strip()))
        pos = end + 2
    return out


def _find_closer(src: str, pos: int, closer: str) -> int:
    """Index of ``closer`` outside string literals."""
    quote = None
    i = pos
    while i < len(src) - 1:
        ch = src[i]
        if quote:
            if ch == "\\":
                i += 2
                continue
            if ch == quote:
                quote = None
        elif ch in "'\"" and closer != "#}":
            quote = ch
        elif src.startswith(closer, i):
            return i
        i += 1
    return -1


# ------------------------------------------------------------------------------------------ parser
class _ExprParser:
    def __init__(self, toks: List[Tuple[str, str]]):
        self.toks = toks
        self.i = 0

    def peek(self):
        return self.toks[self.i]

    def next(self):
        t = self.toks[self.i]
        self.i += 1
        return t

    def accept(self, kind, val=None):
        t = self.toks[self.i]
        if t[0] == kind and (val is None or t[1] == val):
            self.i += 1
            return True
        return False

    def expect(self, kind, val=None):
        if not self.accept(kind, val):
            raise TemplateError(f"expected {val or kind}, got {self.peek()[1]!r}")

    def at_name(self, val):
        t = self.peek()
        return t[0] == "name" and t[1] == val

    # precedence climbing
    def parse(self):
        return self.ternary()

    def ternary(self):
        e = self.or_()
        if self.at_name("if"):
            self.next()
            cond = self.or_()
            other = ("const", UNDEFINED)
            if self.at_name("else"):
                self.next()
                other = self.ternary()
            return ("cond", cond, e, other)
        return e

    def or_(self):
        e = self.and_()
        while self.at_name("or"):
            self.next()
            e = ("or", e, self.and_())
        return e

    def and_(self):
        e = self.not_()
        while self.at_name("and"):
            self.next()
            e = ("and", e, self.not_())
        return e

    def not_(self):
        if self.at_name("not"):
            self.next()
            return ("not", self.not_())
        return self.compare()

    def compare(self):
        e = self.concat()
        while True:
            t = self.peek()
            if t[0] == "op" and t[1] in ("==", "!=", "<", ">", "<=", ">="):
                self.next()
                e = ("cmp", t[1], e, self.concat())
            elif self.at_name("in"):
                self.next()
                e = ("in", e, self.concat())
            elif self.at_name("not") and self.toks[self.i + 1] == ("name", "in"):
                self.i += 2
                e = ("not", ("in", e, self.concat()))
            elif self.at_name("is"):
                self.next()
                neg = False
                if self.at_name("not"):
                    self.next()
                    neg = True
                name = self.next()[1]
                args = []
                if self.peek() == ("op", "("):
                    args = self.call_args()[0]
                elif self.peek()[0] in ("num", "str") or (self.peek()[0] == "name" and self.peek()[1] not in (
                        "and", "or", "else", "if", "not", "in", "is")):
                    args = [self.unary()]
                e = ("test", name, e, args)
                if neg:
                    e = ("not", e)
            else:
                return e

    def concat(self):
        e = self.additive()
        while self.peek() == ("op", "~"):
            self.next()
            e = ("concat", e, self.additive())
        return e

    def additive(self):
        e = self.term()
        while self.peek()[0] == "op" and self.peek()[1] in ("+", "-"):
            op = self.next()[1]
            e = ("bin", op, e, self.term())
        return e

    def term(self):
        e = self.unary()
        while self.peek()[0] == "op" and self.peek()[1] in ("*", "/", "//", "%"):
            op = self.next()[1]
            e = ("bin", op, e, self.unary())
        return e

    def unary(self):
        if self.peek() == ("op", "-"):
            self.next()
            return ("neg", self.unary())
        if self.peek() == ("op", "+"):
            self.next()
            return self.unary()
        return self.postfix()

    def call_args(self):
        self.expect("op", "(")
        args, kwargs = [], {}
        while not self.accept("op", ")"):
            if self.peek()[0] == "name" and self.toks[self.i + 1] == ("op", "="):
                k = self.next()[1]
                self.next()
                kwargs[k] = self.parse()
            else:
                args.append(self.parse())
            self.accept("op", ",")
        return args, kwargs

    def postfix(self):
        e = self.primary()
        while True:
            t = self.peek()
            if t == ("op", "."):
                self.next()
                name = self.next()[1]
                if self.peek() == ("op", "("):
                    a, k = self.call_args()
                    e = ("method", e, name, a, k)
                else:
                    e = ("attr", e, name)
            elif t == ("op", "["):
                self.next()
                start = stop = step = None
                is_slice = False
                if self.peek() != ("op", ":"):
                    start = self.parse()
                if self.accept("op", ":"):
                    is_slice = True
                    if self.peek() not in (("op", "]"), ("op", ":")):
                        stop = self.parse()
                    if self.accept("op", ":"):
                        if self.peek() != ("op", "]"):
                            step = self.parse()
                self.expect("op", "]")
                e = ("slice", e, start, stop, step) if is_slice else ("index", e, start)
            elif t == ("op", "("):
                a, k = self.call_args()
                e = ("call", e, a, k)
            elif t == ("op", "|"):
                self.next()
                name = self.next()[1]
                a, k = ([], {})
                if self.peek() == ("op", "("):
                    a, k = self.call_args()
                e = ("filter", name, e, a, k)
            else:
                return e

    def primary(self):
        kind, val = self.next()
        if kind == "num":
            return ("const", float(val) if "." in val else int(val))
        if kind == "str":
            return ("const", _unescape(val))
        if kind == "name":
            if val in ("true", "True"):
                return ("const", True)
            if val in ("false", "False"):
                return ("const", False)
            if val in ("none", "None"):
                return ("const", None)
            return ("name", val)
        if (kind, val) == ("op", "("):
            items = []
            is_tuple = False
            while not self.accept("op", ")"):
                items.append(self.parse())
                if self.accept("op", ","):
                    is_tuple = True
            return ("list", items) if is_tuple or not items else items[0]
        if (kind, val) == ("op", "["):
            items = []
            while not self.accept("op", "]"):
                items.append(self.parse())
                self.accept("op", ",")
            return ("list", items)
        if (kind, val) == ("op", "{"):
            pairs = []
            while not self.accept("op", "}"):
                k = self.parse()
                self.expect("op", ":")
                pairs.append((k, self.parse()))
                self.accept("op", ",")
            return ("dict", pairs)
        raise TemplateError(f"unexpected token {val!r}")


def _parse_expr(src: str):
    p = _ExprParser(_tokenize_expr(src))
    e = p.parse()
    if p.peek()[0] != "eof":
        raise TemplateError(f"trailing tokens in expression {src!r}")
    return e


def _parse_targets(src: str) -> List[str]:
    return [s.strip() for s in src.strip().strip("()").split(",") if s.strip()]


class _Parser:
    def __init__(self, parts):
        self.parts = parts
        self.i = 0

    def parse(self, stop: Tuple[str, ...] = ()):
        body = []
        while self.i < len(self.parts):
            kind, text = self.parts[self.i]
            if kind == "text":
                body.append(("text", text))
                self.i += 1
            elif kind == "var":
                body.append(("out", _parse_expr(text)))
                self.i += 1
            else:
                word = text.split(None, 1)[0] if text else ""
                if word in stop:
                    return body
                self.i += 1
                rest = text[len(word):].strip()
                if word == "if":
                    branches = [(_parse_expr(rest), self.parse(("elif", "else", "endif")))]
                    else_body = []
                    while True:
                        k2, t2 = self.parts[self.i]
                        w2 = t2.split(None, 1)[0]
                        self.i += 1
                        if w2 == "elif":
                            branches.append((_parse_expr(t2[4:].strip()), self.parse(("elif", "else", "endif"))))
                        elif w2 == "else":
                            else_body = self.parse(("endif",))
                        else:
                            break
                    body.append(("if", branches, else_body))
                elif word == "for":
                    m = re.match(r"(.+?)\s+in\s+(.+)$", rest, re.S)
                    if not m:
                        raise TemplateError(f"malformed for tag: {text!r}")
                    targets = _parse_targets(m.group(1))
                    it_src = m.group(2)
                    cond = None
                    toks = _tokenize_expr(it_src)
                    depth = 0
                    # split off an inline " if <cond>" at bracket depth 0 that is not a ternary
                    p = _ExprParser(toks)
                    it_expr = p.or_()
                    if p.at_name("if"):
                        p.next()
                        cond = p.parse()
                    recursive = False
                    if p.at_name("recursive"):
                        p.next()
                        recursive = True
                    loop_body = self.parse(("else", "endfor"))
                    else_body = []
                    if self.parts[self.i][1].split(None, 1)[0] == "else":
                        self.i += 1
                        else_body = self.parse(("endfor",))
                    self.i += 1
                    body.append(("for", targets, it_expr, cond, loop_body, else_body))
                elif word == "set":
                    if "=" in rest and not re.match(r"^[\w.,\s()]+$", rest):
                        lhs, rhs = rest.split("=", 1)
                        body.append(("set", lhs.strip(), _parse_expr(rhs)))
                    elif "=" in rest:
                        lhs, rhs = rest.split("=", 1)
                        body.append(("set", lhs.strip(), _parse_expr(rhs)))
                    else:
                        blk = self.parse(("endset",))
                        self.i += 1
                        body.append(("setblock", rest.strip(), blk))
                elif word == "macro":
                    m = re.match(r"(\w+)\s*\((.*)\)\s*$", rest, re.S)
                    if not m:
                        raise TemplateError(f"malformed macro tag: {text!r}")
                    params = []
                    if m.group(2).strip():
                        p = _ExprParser(_tokenize_expr(m.group(2)))
                        while p.peek()[0] != "eof":
                            name = p.next()[1]
                            default = None
                            if p.accept("op", "="):
                                default = p.parse()
                            params.append((name, default))
                            p.accept("op", ",")
                    mbody = self.parse(("endmacro",))
                    self.i += 1
                    body.append(("macro", m.group(1), params, mbody))
                elif word in ("generation", "endgeneration", "filter", "endfilter"):
                    continue       # HF-specific markers: transparent
                else:
                    raise TemplateError(f"unsupported tag {word!r}")
        return body


# ------------------------------------------------------------------------------------------ evaluation
def _truthy(v) -> bool:
    if v is None or isinstance(v, _Undefined):
        return False
    if isinstance(v, (bool, int, float, str, list, dict, tuple)):
        return bool(v)
    return True


def _to_str(v) -> str:
    if v is None:
        return "None"
    if isinstance(v, bool):
        return "True" if v else "False"
    if isinstance(v, float) and v == int(v):
        return str(v)
    return str(v)


def to_json(v) -> str:
    if v is None or isinstance(v, _Undefined):
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return repr(v) if isinstance(v, float) and v != int(v) else str(int(v)) if isinstance(v, float) else str(v)
    if isinstance(v, str):
        return _esc_str(v)
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(to_json(x) for x in v) + "]"
    if isinstance(v, dict):
        return "{" + ", ".join(f"{_esc_str(str(k))}: {to_json(x)}" for k, x in v.items()) + "}"
    if isinstance(v, Namespace):
        return to_json(v.__dict__)
    return _esc_str(str(v))


_TESTS: Dict[str, Callable[..., bool]] = {
    "defined": lambda v: not isinstance(v, _Undefined),
    "undefined": lambda v: isinstance(v, _Undefined),
    "none": lambda v: v is None,
    "mapping": lambda v: isinstance(v, dict),
    "string": lambda v: isinstance(v, str),
    "boolean": lambda v: isinstance(v, bool),
    "sequence": lambda v: isinstance(v, (list, tuple, str)),
    "iterable": lambda v: isinstance(v, (list, tuple, str, dict)),
    "number": lambda v: isinstance(v, (int, float)) and not isinstance(v, bool),
    "integer": lambda v: isinstance(v, int) and not isinstance(v, bool),
    "float": lambda v: isinstance(v, float),
    "true": lambda v: v is True,
    "false": lambda v: v is False,
    "odd": lambda v: v % 2 == 1,
    "even": lambda v: v % 2 == 0,
    "equalto": lambda v, o: v == o,
    "eq": lambda v, o: v == o,
    "ne": lambda v, o: v != o,
    "in": lambda v, o: v in o,
}


class Jinja2Template:
    def __init__(self, source: str):
        self.source = source
        self.ast = _Parser(_split_template(source)).parse()

    # -------------------------------------------------------------- public
    def render(self, context: Optional[Dict[str, Any]] = None, **kw) -> str:
        scope: Dict[str, Any] = {
            "namespace": lambda **k: Namespace(**k),
            "range": lambda *a: list(range(*[int(x) for x in a])),
            "raise_exception": self._raise,
            "strftime_now": lambda fmt: _dt.datetime.now().strftime(fmt),
            "dict": lambda **k: dict(k),
            "len": len,
        }
        scope.update(context or {})
        scope.update(kw)
        out: List[str] = []
        self._exec(self.ast, [scope], out)
        return "".join(out)

    @staticmethod
    def _raise(msg=""):
        raise TemplateError(str(msg))

    # -------------------------------------------------------------- statements
    def _lookup(self, scopes, name):
        for s in reversed(scopes):
            if name in s:
                return s[name]
        return UNDEFINED

    def _exec(self, body, scopes, out):
        for node in body:
            k = node[0]
            if k == "text":
                out.append(node[1])
            elif k == "out":
                v = self._eval(node[1], scopes)
                if v is not None and not isinstance(v, _Undefined):
                    out.append(_to_str(v))
                elif v is None:
                    out.append("None")
            elif k == "if":
                done = False
                for cond, blk in node[1]:
                    if _truthy(self._eval(cond, scopes)):
                        self._exec(blk, scopes, out)
                        done = True
                        break
                if not done:
                    self._exec(node[2], scopes, out)
            elif k == "for":
                _, targets, it_expr, cond, blk, else_blk = node
                seq = self._eval(it_expr, scopes)
                if isinstance(seq, dict):
                    seq = list(seq.keys())
                elif isinstance(seq, str):
                    seq = list(seq)
                elif seq is None or isinstance(seq, _Undefined):
                    seq = []
                else:
                    seq = list(seq)
                if cond is not None:
                    kept = []
                    for item in seq:
                        loc = {}
                        self._bind(targets, item, loc)
                        if _truthy(self._eval(cond, scopes + [loc])):
                            kept.append(item)
                    seq = kept
                if not seq:
                    self._exec(else_blk, scopes, out)
                    continue
                loop = _LoopCtx(seq)
                for i, item in enumerate(seq):
                    loop.index0 = i
                    loc = {"loop": loop}
                    self._bind(targets, item, loc)
                    self._exec(blk, scopes + [loc], out)
            elif k == "set":
                val = self._eval(node[2], scopes)
                lhs = node[1]
                if "." in lhs:
                    obj_name, attr = lhs.split(".", 1)
                    obj = self._lookup(scopes, obj_name.strip())
                    if isinstance(obj, Namespace):
                        setattr(obj, attr.strip(), val)
                    elif isinstance(obj, dict):
                        obj[attr.strip()] = val
                    else:
                        raise TemplateError(f"cannot assign attribute on {obj_name!r}")
                else:
                    targets = _parse_targets(lhs)
                    self._bind(targets, val, scopes[-1])
            elif k == "setblock":
                buf: List[str] = []
                self._exec(node[2], scopes, buf)
                scopes[-1][node[1]] = "".join(buf)
            elif k == "macro":
                _, name, params, mbody = node
                scopes[-1][name] = self._make_macro(params, mbody, scopes)

    def _make_macro(self, params, mbody, def_scopes):
        def macro(*args, **kwargs):
            loc = {}
            for i, (pname, default) in enumerate(params):
                if i < len(args):
                    loc[pname] = args[i]
                elif pname in kwargs:
                    loc[pname] = kwargs[pname]
                elif default is not None:
                    loc[pname] = self._eval(default, def_scopes)
                else:
                    loc[pname] = UNDEFINED
            buf: List[str] = []
            self._exec(mbody, def_scopes + [loc], buf)
            return "".join(buf)
        return macro

    @staticmethod
    def _bind(targets, value, scope):
        if len(targets) == 1:
            scope[targets[0]] = value
            return
        vals = list(value) if not isinstance(value, dict) else list(value.items())
        if len(vals) != len(targets):
            raise TemplateError(f"cannot unpack {len(vals)} values into {len(targets)} names")
        for t, v in zip(targets, vals):
            scope[t] = v

    # -------------------------------------------------------------- expressions
    def _eval(self, e, scopes):
        k = e[0]
        if k == "const":
            return e[1]
        if k == "name":
            return self._lookup(scopes, e[1])
        if k == "cond":
            return self._eval(e[2], scopes) if _truthy(self._eval(e[1], scopes)) else self._eval(e[3], scopes)
        if k == "or":
            l = self._eval(e[1], scopes)
            return l if _truthy(l) else self._eval(e[2], scopes)
        if k == "and":
            l = self._eval(e[1], scopes)
            return self._eval(e[2], scopes) if _truthy(l) else l
        if k == "not":
            return not _truthy(self._eval(e[1], scopes))
        if k == "cmp":
            l, r = self._eval(e[2], scopes), self._eval(e[3], scopes)
            op = e[1]
            if op == "==":
                return l == r
            if op == "!=":
                return l != r
            try:
                return {"<": l < r, ">": l > r, "<=": l <= r, ">=": l >= r}[op]
            except TypeError:
                return False
        if k == "in":
            l, r = self._eval(e[1], scopes), self._eval(e[2], scopes)
            try:
                return l in r
            except TypeError:
                return False
        if k == "test":
            fn = _TESTS.get(e[1])
            if fn is None:
                raise TemplateError(f"unknown test {e[1]!r}")
            return bool(fn(self._eval(e[2], scopes), *[self._eval(a, scopes) for a in e[3]]))
        if k == "concat":
            return _to_str(self._eval(e[1], scopes)) + _to_str(self._eval(e[2], scopes))
        if k == "bin":
            l, r = self._eval(e[2], scopes), self._eval(e[3], scopes)
            op = e[1]
            if op == "+":
                if isinstance(l, str) or isinstance(r, str):
                    return _to_str(l) + _to_str(r)
                if isinstance(l, _Undefined):
                    return r
                if isinstance(r, _Undefined):
                    return l
                return l + r
            if isinstance(l, _Undefined) or isinstance(r, _Undefined):
                return UNDEFINED
            if op == "-":
                return l - r
            if op == "*":
                return l * r
            if op == "/":
                return l / r
            if op == "//":
                return l // r
            if op == "%":
                return l % r
        if k == "neg":
            return -self._eval(e[1], scopes)
        if k == "list":
            return [self._eval(x, scopes) for x in e[1]]
        if k == "dict":
            return {self._eval(a, scopes): self._eval(b, scopes) for a, b in e[1]}
        if k == "attr":
            return self._getattr(self._eval(e[1], scopes), e[2])
        if k == "index":
            obj, idx = self._eval(e[1], scopes), self._eval(e[2], scopes)
            try:
                if isinstance(obj, dict):
                    return obj.get(idx, UNDEFINED)
                if isinstance(obj, Namespace):
                    return getattr(obj, idx, UNDEFINED)
                return obj[idx]
            except (IndexError, KeyError, TypeError):
                return UNDEFINED
        if k == "slice":
            obj = self._eval(e[1], scopes)
            s = [None if x is None else self._eval(x, scopes) for x in e[2:5]]
            try:
                return obj[slice(*s)]
            except TypeError:
                return UNDEFINED
        if k == "call":
            fn = self._eval(e[1], scopes)
            if not callable(fn):
                raise TemplateError("attempt to call a non-callable value")
            return fn(*[self._eval(a, scopes) for a in e[2]], **{n: self._eval(v, scopes) for n, v in e[3].items()})
        if k == "method":
            obj = self._eval(e[1], scopes)
            args = [self._eval(a, scopes) for a in e[3]]
            kwargs = {n: self._eval(v, scopes) for n, v in e[4].items()}
            return self._method(obj, e[2], args, kwargs)
        if k == "filter":
            val = self._eval(e[2], scopes)
            args = [self._eval(a, scopes) for a in e[3]]
            kwargs = {n: self._eval(v, scopes) for n, v in e[4].items()}
            return self._filter(e[1], val, args, kwargs)
        raise TemplateError(f"cannot evaluate node {k!r}")

    @staticmethod
    def _getattr(obj, name):
        if isinstance(obj, dict):
            if name in obj:
                return obj[name]
            return UNDEFINED
        if isinstance(obj, (Namespace, _LoopCtx)):
            return getattr(obj, name, UNDEFINED)
        if isinstance(obj, tuple) and name in ("key", "value") and len(obj) == 2:
            return obj[0] if name == "key" else obj[1]
        if obj is None or isinstance(obj, _Undefined):
            return UNDEFINED
        return getattr(obj, name, UNDEFINED)

    @staticmethod
    def _method(obj, name, args, kwargs):
        if isinstance(obj, dict):
            if name == "get":
                v = obj.get(args[0], args[1] if len(args) > 1 else None)
                return v
            if name == "items":
                return list(obj.items())
            if name == "keys":
                return list(obj.keys())
            if name == "values":
                return list(obj.values())
            if name == "update":
                obj.update(*args, **kwargs)
                return None
            if name in obj and callable(obj[name]):
                return obj[name](*args, **kwargs)
        if isinstance(obj, str):
            if name in ("strip", "lstrip", "rstrip", "upper", "lower", "title", "capitalize", "startswith",
                        "endswith", "split", "replace", "find", "count", "splitlines", "join", "rsplit", "isdigit"):
                return getattr(obj, name)(*args)
        if isinstance(obj, list):
            if name == "append":
                obj.append(args[0])
                return None
            if name in ("pop", "insert", "extend", "index", "count"):
                return getattr(obj, name)(*args)
        if isinstance(obj, _Undefined) or obj is None:
            if name == "get":
                return args[1] if len(args) > 1 else None
            return UNDEFINED
        fn = getattr(obj, name, None)
        if callable(fn):
            return fn(*args, **kwargs)
        raise TemplateError(f"unknown method {name!r} on {type(obj).__name__}")

    def _filter(self, name, val, args, kwargs):
        if name == "trim":
            return _to_str(val).strip() if not isinstance(val, _Undefined) else ""
        if name in ("length", "count"):
            try:
                return len(val)
            except TypeError:
                return 0
        if name == "upper":
            return _to_str(val).upper()
        if name == "lower":
            return _to_str(val).lower()
        if name == "title":
            return _to_str(val).title()
        if name == "capitalize":
            return _to_str(val).capitalize()
        if name == "first":
            try:
                return val[0] if len(val) else UNDEFINED
            except TypeError:
                return UNDEFINED
        if name == "last":
            try:
                return val[-1] if len(val) else UNDEFINED
            except TypeError:
                return UNDEFINED
        if name in ("default", "d"):
            dflt = args[0] if args else kwargs.get("default_value", "")
            boolean = (args[1] if len(args) > 1 else kwargs.get("boolean", False))
            if isinstance(val, _Undefined) or (boolean and not _truthy(val)):
                return dflt
            return val
        if name == "list":
            if isinstance(val, dict):
                return list(val.keys())
            return list(val) if not isinstance(val, _Undefined) and val is not None else []
        if name == "int":
            try:
                return int(float(val)) if not isinstance(val, bool) else int(val)
            except (TypeError, ValueError):
                return args[0] if args else 0
        if name == "float":
            try:
                return float(val)
            except (TypeError, ValueError):
                return 0.0
        if name == "string":
            return _to_str(val)
        if name == "join":
            sep = args[0] if args else kwargs.get("d", "")
            attr = kwargs.get("attribute")
            seq = [self._getattr(x, attr) if attr else x for x in (val or [])]
            return sep.join(_to_str(x) for x in seq)
        if name == "tojson":
            return to_json(val)
        if name == "dictsort":
            return sorted(val.items(), key=lambda kv: kv[0]) if isinstance(val, dict) else val
        if name in ("safe", "e", "escape"):
            return val
        if name == "replace":
            return _to_str(val).replace(_to_str(args[0]), _to_str(args[1]))
        if name == "items":
            return list(val.items()) if isinstance(val, dict) else []
        if name == "reverse":
            return val[::-1]
        if name == "sort":
            attr = kwargs.get("attribute")
            return sorted(val, key=(lambda x: self._getattr(x, attr)) if attr else None, reverse=kwargs.get("reverse", False))
        if name == "unique":
            seen, out = set(), []
            for x in val:
                key = repr(x)
                if key not in seen:
                    seen.add(key)
                    out.append(x)
            return out
        if name == "map":
            attr = kwargs.get("attribute")
            if attr is not None:
                return [self._getattr(x, attr) for x in val]
            if args:
                return [self._filter(args[0], x, list(args[1:]), {}) for x in val]
            return list(val)
        if name in ("selectattr", "rejectattr"):
            attr = args[0]
            test = args[1] if len(args) > 1 else None
            targs = args[2:]
            out = []
            for x in val or []:
                v = self._getattr(x, attr)
                ok = _truthy(v) if test is None else bool(_TESTS[test](v, *targs))
                if ok == (name == "selectattr"):
                    out.append(x)
            return out
        if name in ("select", "reject"):
            test = args[0] if args else None
            out = []
            for x in val or []:
                ok = _truthy(x) if test is None else bool(_TESTS[test](x, *args[1:]))
                if ok == (name == "select"):
                    out.append(x)
            return out
        if name == "abs":
            return abs(val)
        if name == "round":
            return round(val, int(args[0]) if args else 0)
        if name == "indent":
            width = int(args[0]) if args else 4
            pad = " " * width
            lines = _to_str(val).split("\n")
            return ("\n" + pad).join(lines)
        if name in ("min", "max", "sum"):
            return {"min": min, "max": max, "sum": sum}[name](val)
        raise TemplateError(f"unknown filter {name!r}")
