"""Math-answer utilities for verifiable rewards and evaluation: repetition score, extraction of the boxed /
final answer, normalisation and equality (string level, then symbolic with a deadline).

Behavioural reference: ``steptronoss/text_processing/oone_math_utils.py:17-448``.
"""
from __future__ import annotations

import re

import numpy as np

from .utils import get_runner


# ----------------------------------------------------------------------------------------- repetition
def _suffix_array(codes: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Prefix doubling with numpy sorts: ``rank[i]`` of suffix ``i`` and ``sa[r]`` = start of the r-th suffix."""
    n = codes.size
    rank = np.unique(codes, return_inverse=True)[1].astype(np.int64)
    k = 1
    while k < n:
        nxt = np.full(n, -1, dtype=np.int64)
        nxt[: n - k] = rank[k:]
        key = rank * (n + 1) + (nxt + 1)
        rank = np.unique(key, return_inverse=True)[1].astype(np.int64)
        if rank.max() == n - 1:
            break
        k <<= 1
    sa = np.empty(n, dtype=np.int64)
    sa[rank] = np.arange(n)
    return rank, sa


def repeatness_score(s: str) -> float:
    """``2 * sum(LCP of lexicographically adjacent suffixes) / (n (n + 1))``: 0 for text without repeated
    substrings, towards 1 for text that is one pattern repeated."""
    n = len(s)
    if n <= 1:
        return 0
    codes = np.frombuffer(s.encode("utf-32-le"), dtype=np.uint32).astype(np.int64)
    rank, sa = _suffix_array(codes)
    total, k = 0, 0
    for i in range(n):  # Kasai
        r = rank[i]
        if r == n - 1:
            k = 0
            continue
        j = sa[r + 1]
        while i + k < n and j + k < n and codes[i + k] == codes[j + k]:
            k += 1
        total += k
        if k:
            k -= 1
    return total * 2 / (n * (n + 1))


def repeatness(s: str) -> bool:
    return repeatness_score(s) > 0.2


# ----------------------------------------------------------------------------------------- extraction
def last_boxed_only_string(string: str) -> str | None:
    """The last ``\\boxed{...}`` (or ``\\fbox{...}``) with balanced braces, or None."""
    idx = string.rfind("\\boxed")
    if idx < 0:
        idx = string.rfind("\\fbox")
        if idx < 0:
            return None
    depth = 0
    for i in range(idx, len(string)):
        ch = string[i]
        if ch == "{":
            depth += 1
        elif ch == "}":
            depth -= 1
            if depth == 0:
                return string[idx: i + 1]
    return None


def remove_boxed(s: str | None) -> str | None:
    left = "\\boxed{"
    if s is None or not s.startswith(left) or not s.endswith("}"):
        return None
    return s[len(left): -1]


def get_answer_str(s: str) -> str:
    inner = remove_boxed(last_boxed_only_string(s))
    return inner if inner is not None else s


def solution2answer(solution: str, math_mode: str = "eval_peeking") -> str:
    if math_mode != "eval_peeking":
        raise ValueError(f"Invalid math_mode: {math_mode}")
    return get_answer_str(solution)


def get_final_answer(output: str) -> str:
    output = output.replace("is:", "is").replace("answer:", "answer is").strip()
    if output.endswith("."):
        output = output[:-1]
    output = output.replace(".$", "$")
    for pat in (r"answer is (-?\d+\.?\d*)$", r"answer is (.+?)$"):
        m = re.findall(pat, output, re.S)
        if m:
            return get_answer_str(m[0])
    return get_answer_str(output)


# ----------------------------------------------------------------------------------------- normalisation
_SUBSTITUTIONS = [("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), (r"\ ", ""), (" ", ""), ("mbox", "text"),
                  (",\\text{and}", ","), ("\\text{and}", ","), ("\\text{m}", "\\text{}")]
_REMOVED = ["square", "ways", "integers", "dollars", "mph", "inches", "ft", "hours", "km", "units", "\\ldots", "sue",
            "points", "feet", "minutes", "digits", "cents", "degrees", "cm", "gm", "pounds", "meters", "meals", "edges",
            "students", "childrentickets", "multiples", "\\text{s}", "\\text{.}", "\\text{\ns}", "\\text{}^2",
            "\\text{}^3", "\\text{\n}", "\\text{}", r"\mathrm{th}", r"^\circ", r"^{\circ}", r"\;", r",\!", "{,}", '"',
            "\\dots"]


def normalize_final_answer(ans: str) -> str:
    """The answer normalisation of Lewkowycz et al. 2022 (appendix D): drop units and prose, unwrap
    ``$...$`` / ``\\text`` / ``\\boxed``, brace shorthand fractions and roots, drop thousands separators."""
    for a, b in _SUBSTITUTIONS:
        ans = ans.replace(a, b)
    for e in _REMOVED:
        ans = ans.replace(e, "")
    ans = re.sub(r"(.*?)(\$)(.*?)(\$)(.*)", "$\\3$", ans)
    for tag in ("text", "textbf", "overline"):
        ans = re.sub(r"(\\%s\{)(.*?)(\})" % tag, "\\2", ans)
    ans = re.sub(r"(\\boxed\{)(.*)(\})", "\\2", ans)
    ans = re.sub(r"(frac)([^{])(.)", "frac{\\2}{\\3}", ans)
    ans = re.sub(r"(sqrt)([^{])", "sqrt{\\2}", ans)
    ans = ans.replace("$", "")
    if ans.replace(",", "").isdigit():
        ans = ans.replace(",", "")
    return ans


def _fix_fracs(s: str) -> str:
    parts = s.split("\\frac")
    out = parts[0]
    for p in parts[1:]:
        out += "\\frac"
        if p[:1] == "{" or len(p) < 2:
            out += p
            continue
        a, b, rest = p[0], p[1], p[2:]
        out += "{" + a + "}" + (b if b == "{" else "{" + b + "}") + rest
    return out


def _fix_a_slash_b(s: str) -> str:
    m = re.fullmatch(r"(-?\d+)/(-?\d+)", s)
    return f"\\frac{{{int(m.group(1))}}}{{{int(m.group(2))}}}" if m else s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt([^{])", r"\\sqrt{\1}", s)


def _strip_string(s: str) -> str:
    s = s.replace("\n", "").replace("\\!", "").replace("\\\\", "\\")
    s = s.replace("tfrac", "frac").replace("dfrac", "frac").replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "")
    if "\\text{ " in s:  # trailing units
        s = s.split("\\text{ ")[0]
    s = s.replace("\\%", "").replace("%", "")
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if not s:
        return s
    if s[0] == ".":
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:  # "x = 3" -> "3"
        s = s.split("=")[1]
    s = _fix_sqrt(s).replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    return _fix_a_slash_b(s)


def is_equiv(a, b, verbose: bool = False) -> bool:
    if a is None and b is None:
        return True
    if a is None or b is None:
        return False
    try:
        sa, sb = _strip_string(a), _strip_string(b)
        if verbose:
            print(sa, sb)
        try:
            return float(sa) == float(sb)
        except ValueError:
            return sa == sb
    except Exception:
        return a == b


def latex_eval(latex: str):
    from sympy.parsing.latex import parse_latex

    sym = parse_latex(latex)
    return sym, sym.evalf()


def _is_latex_equal(a: str, b: str) -> bool:
    def same(x, y):
        sx, vx = latex_eval(x)
        sy, vy = latex_eval(y)
        return sx == sy or vx == vy

    try:
        if same(a, b):
            return True
    except Exception:
        pass
    na, nb = normalize_final_answer(a), normalize_final_answer(b)
    try:
        return bool(same(na, nb))
    except Exception:
        return na == nb


def is_latex_equal(a: str, b: str, math_mode: str = "legacy") -> bool:
    if math_mode == "legacy":
        if (len(a) > 128 and repeatness(a)) or (len(b) > 128 and repeatness(b)):
            return False
        try:
            return bool(get_runner()(_is_latex_equal, a, b, timeout=2))
        except TimeoutError:
            return False
    if math_mode == "math_verify":
        from math_verify import parse, verify

        try:
            return bool(get_runner()(verify, parse(a), parse(b), timeout=2))
        except TimeoutError:
            return False
    raise NotImplementedError(f"Math mode {math_mode} is not implemented")


def is_equal(a: str, b: str, math_mode: str = "legacy") -> bool:
    return True if is_equiv(a, b) else is_latex_equal(a, b, math_mode)
