"""Answer extraction and equivalence for math word problems (no external verifier):
last ``\\boxed{...}``, ``#### x`` or the last number; comparison of normalised
strings, fractions, percentages and decimals within a tolerance."""

from __future__ import annotations

import re
from fractions import Fraction

_NUM = re.compile(r"-?\d[\d,]*(?:\.\d+)?(?:/\d+)?|-?\.\d+")


def _last_boxed(text: str) -> str | None:
    idx = text.rfind("\\boxed")
    if idx < 0:
        return None
    i = text.find("{", idx)
    if i < 0:
        return None
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


def extract_answer(text: str) -> str | None:
    if text is None:
        return None
    b = _last_boxed(text)
    if b is not None:
        return b.strip()
    if "####" in text:
        return text.split("####")[-1].strip().split("\n")[0].strip()
    m = re.search(r"(?:answer is|answer:)\s*([^\n]+)", text, flags=re.I)
    if m:
        nums = _NUM.findall(m.group(1))
        if nums:
            return nums[-1]
        return m.group(1).strip().rstrip(".")
    nums = _NUM.findall(text)
    return nums[-1] if nums else None


def _normalise(s: str) -> str:
    s = s.strip().strip("$").replace("\\!", "").replace("\\,", "").replace("\\ ", "").replace(" ", "")
    s = re.sub(r"\\text\{([^}]*)\}", r"\1", s)
    s = re.sub(r"\\d?frac\{([^{}]+)\}\{([^{}]+)\}", r"(\1)/(\2)", s)
    s = s.replace("\\left", "").replace("\\right", "").replace("dollars", "").replace("\\%", "%")
    s = s.rstrip(".")
    if s.startswith("(") and s.endswith(")") and s.count("(") == 1 and "/" not in s:
        s = s[1:-1]
    return s


def _to_number(s: str) -> Fraction | None:
    s = s.replace(",", "")
    pct = s.endswith("%")
    if pct:
        s = s[:-1]
    s = s.replace("(", "").replace(")", "")
    try:
        if "/" in s:
            a, b = s.split("/", 1)
            v = Fraction(a) / Fraction(b)
        else:
            v = Fraction(s)
    except (ValueError, ZeroDivisionError):
        return None
    return v / 100 if pct else v


def math_equal(pred: str | None, ref: str | None, rel_tol: float = 1e-4) -> bool:
    if pred is None or ref is None:
        return False
    p, r = _normalise(str(pred)), _normalise(str(ref))
    if p == r:
        return True
    pn, rn = _to_number(p), _to_number(r)
    if pn is not None and rn is not None:
        if pn == rn:
            return True
        scale = max(abs(float(rn)), 1e-12)
        return abs(float(pn) - float(rn)) / scale <= rel_tol
    return p.lower() == r.lower()
