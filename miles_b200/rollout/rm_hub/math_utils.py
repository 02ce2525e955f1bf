"""Answer extraction and equivalence checks for math-style rewards (``deepscaler`` / ``math`` / ``dapo``).

String normalisation (units, ``\\text{}``, ``\\dfrac``, spacing, percent, trailing zeros), numeric
comparison, and symbolic equality through sympy when it is installed.  Behavioural counterpart of the
reference's miles/rollout/rm_hub/math_utils.py and math_dapo_utils.py.
"""
from __future__ import annotations

import re
from typing import Optional


def extract_boxed(text: str) -> Optional[str]:
    """Content of the last ``\\boxed{...}`` (or ``\\fbox{...}``) with balanced braces."""
    if not text:
        return None
    idx = max(text.rfind("\\boxed"), text.rfind("\\fbox"))
    if idx < 0:
        return None
    i = text.find("{", idx)
    if i < 0:
        m = re.match(r"\\boxed\s+([^\s$]+)", text[idx:])
        return m.group(1) if m else None
    depth, j = 0, i
    while j < len(text):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i + 1:j]
        j += 1
    return None


_UNITS = ["degrees", "degree", "cm", "centimeters", "meters", "meter", "mph", "inches", "inch", "feet", "foot", "units",
          "unit", "square", "dollars", "dollar", "cents", "cent", "hours", "hour", "minutes", "minute", "seconds", "second"]


def _fix_fracs(s: str) -> str:
    # \frac12 -> \frac{1}{2}
    return re.sub(r"\\frac\s*([0-9a-zA-Z])\s*([0-9a-zA-Z])", r"\\frac{\1}{\2}", s)


def normalize_answer(ans: str) -> str:
    s = str(ans).strip()
    s = s.replace("\n", "").replace("\\!", "").replace("\\,", "").replace("\\;", "").replace("\\ ", "")
    s = s.replace("tfrac", "frac").replace("dfrac", "frac").replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "").replace("$", "")
    s = re.sub(r"\\text\{\s*([^}]*)\}", r"\1", s)
    s = re.sub(r"\\mbox\{\s*([^}]*)\}", r"\1", s)
    for u in _UNITS:
        s = re.sub(rf"(?<=[0-9}}\s]){u}\b", "", s)
    s = s.replace("\\%", "").replace("%", "")
    if s.startswith("x=") or s.startswith("y=") or re.match(r"^[a-zA-Z]\s*=", s):
        s = s.split("=", 1)[1]
    s = s.replace(" ", "")
    s = _fix_fracs(s)
    if s.endswith("."):
        s = s[:-1]
    if re.fullmatch(r"-?\d+\.\d*0+", s):
        s = s.rstrip("0").rstrip(".")
    if s.startswith("."):
        s = "0" + s
    s = s.replace(",\\!", "")
    if re.fullmatch(r"-?\d{1,3}(,\d{3})+(\.\d+)?", s):
        s = s.replace(",", "")
    if s == "0.5":
        s = "\\frac{1}{2}"
    return s


def _to_float(s: str) -> Optional[float]:
    s = s.replace(",", "")
    m = re.fullmatch(r"\\frac\{(-?[\d.]+)\}\{(-?[\d.]+)\}", s)
    try:
        if m:
            return float(m.group(1)) / float(m.group(2))
        m = re.fullmatch(r"(-?[\d.]+)/(-?[\d.]+)", s)
        if m:
            return float(m.group(1)) / float(m.group(2))
        return float(s)
    except (ValueError, ZeroDivisionError):
        return None


def _sympy_equal(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing.latex import parse_latex  # needs antlr; fall back to sympify below
    except Exception:
        parse_latex = None
        try:
            import sympy
        except Exception:
            return False
    try:
        def parse(x):
            if parse_latex is not None and "\\" in x:
                return parse_latex(x)
            return sympy.sympify(x.replace("^", "**"))

        return bool(sympy.simplify(parse(a) - parse(b)) == 0)
    except Exception:
        return False


def grade_math_answer(response: str, label: str) -> bool:
    """True when the final answer of ``response`` matches ``label``."""
    if response is None or label is None:
        return False
    pred = extract_boxed(response)
    if pred is None:
        m = re.findall(r"(?:answer is|Answer:)\s*([^\n]+)", response)
        pred = m[-1] if m else response.strip().split("\n")[-1]
    gold = extract_boxed(label) or label
    p, g = normalize_answer(pred), normalize_answer(gold)
    if not p:
        return False
    if p == g:
        return True
    fp, fg = _to_float(p), _to_float(g)
    if fp is not None and fg is not None:
        return abs(fp - fg) <= 1e-6 * max(1.0, abs(fg))
    if len(p) < 64 and len(g) < 64:
        return _sympy_equal(p, g)
    return False
