"""Command-line overrides of the form ``a.b.c=value`` (reference ``steptronoss/utils/arguments.py:5-28``)."""
from __future__ import annotations

import ast
import sys
from typing import Any


def parse_value(text: str) -> Any:
    """Literal-evaluate a value; anything that is not a Python literal stays a string."""
    try:
        return ast.literal_eval(text)
    except (ValueError, SyntaxError):
        low = text.lower()
        if low in ("true", "false"):
            return low == "true"
        if low in ("none", "null"):
            return None
        return text


def parse_args(argv: list[str] | None = None) -> dict[str, Any]:
    """Collect every ``key=value`` token of ``argv`` (default ``sys.argv[1:]``) into a dict.

    Tokens without ``=`` and tokens that start with ``-`` are ignored so that launchers may
    pass their own flags through.
    """
    argv = sys.argv[1:] if argv is None else argv
    out: dict[str, Any] = {}
    for tok in argv:
        if tok.startswith("-") or "=" not in tok:
            continue
        key, _, val = tok.partition("=")
        key = key.strip()
        if not key:
            continue
        out[key] = parse_value(val.strip())
    return out
