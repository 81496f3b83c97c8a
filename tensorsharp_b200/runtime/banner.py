"""Start-up banner for the CLI and the server.

The reference prints a half-block picture of its mascot and a gradient logo with 24-bit ANSI colours,
falling back to plain text when the output is redirected or ``NO_COLOR`` is set
(TensorSharp.Runtime/ConsoleBanner.cs:114).  This build has its own wordmark (block letters drawn here,
coloured with a horizontal gradient) and the same rules for when colour is allowed.
"""
from __future__ import annotations

import os
import sys
from typing import Iterable, List, Optional, Sequence, Tuple

# 5-row block letters for the wordmark
_GLYPHS = {
    "T": ["█████", "  █  ", "  █  ", "  █  ", "  █  "],
    "E": ["████", "█   ", "███ ", "█   ", "████"],
    "N": ["█   █", "██  █", "█ █ █", "█  ██", "█   █"],
    "S": [" ████", "█    ", " ███ ", "    █", "████ "],
    "O": [" ███ ", "█   █", "█   █", "█   █", " ███ "],
    "R": ["████ ", "█   █", "████ ", "█  █ ", "█   █"],
    "H": ["█   █", "█   █", "█████", "█   █", "█   █"],
    "A": [" ███ ", "█   █", "█████", "█   █", "█   █"],
    "P": ["████ ", "█   █", "████ ", "█    ", "█    "],
    "B": ["████ ", "█   █", "████ ", "█   █", "████ "],
    "2": ["████ ", "    █", " ███ ", "█    ", "█████"],
    "0": [" ███ ", "█  ██", "█ █ █", "██  █", " ███ "],
    " ": ["  ", "  ", "  ", "  ", "  "],
}
WORDMARK = "TENSORSHARP B200"
_START, _END = (118, 185, 0), (0, 174, 239)        # gradient end points (green to blue)


def wordmark_rows(text: str = WORDMARK) -> List[str]:
    rows = ["", "", "", "", ""]
    for ch in text:
        g = _GLYPHS.get(ch.upper(), _GLYPHS[" "])
        for i in range(5):
            rows[i] += g[i] + " "
    return [r.rstrip() for r in rows]


def color_allowed(stream=None, env: Optional[dict] = None) -> bool:
    """Colour only on a terminal, and never when NO_COLOR is set (any value) or TERM is ``dumb``."""
    env = os.environ if env is None else env
    if env.get("NO_COLOR") is not None or env.get("TERM", "") == "dumb":
        return False
    stream = stream or sys.stdout
    isatty = getattr(stream, "isatty", None)
    return bool(isatty and isatty())


def _lerp(a: Tuple[int, int, int], b: Tuple[int, int, int], t: float) -> Tuple[int, int, int]:
    return tuple(int(round(x + (y - x) * t)) for x, y in zip(a, b))


def gradient(line: str, width: int) -> str:
    out = []
    for i, ch in enumerate(line):
        if ch == " ":
            out.append(ch)
            continue
        r, g, b = _lerp(_START, _END, i / max(1, width - 1))
        out.append(f"\x1b[38;2;{r};{g};{b}m{ch}")
    return "".join(out) + "\x1b[0m"


def render_banner(subtitle: Sequence[str] = (), color: Optional[bool] = None, stream=None) -> str:
    """The banner as one string: wordmark, a rule, then the subtitle lines (version, model, address ...)."""
    color = color_allowed(stream) if color is None else color
    rows = wordmark_rows()
    width = max(len(r) for r in rows)
    body = [gradient(r, width) for r in rows] if color else list(rows)
    rule = "─" * width
    lines = [""] + body + [gradient(rule, width) if color else rule] + [f"  {s}" for s in subtitle] + [""]
    return "\n".join(lines)


def print_banner(subtitle: Iterable[str] = (), stream=None) -> None:
    stream = stream or sys.stdout
    stream.write(render_banner(list(subtitle), stream=stream) + "\n")
    stream.flush()
