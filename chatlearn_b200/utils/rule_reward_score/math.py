"""MATH-style answer checking: extract the last ``\\boxed{...}`` from a response
and compare it with the ground truth after normalisation.

Parity: chatlearn/utils/rule_reward_score/math.py:2-220 (same decision: reward 1.0
when the normalised boxed answer equals the normalised ground truth, else 0.0).
The normaliser here is a small rewrite-rule list rather than a chain of helper
functions.
"""
import re
from typing import Optional


def last_boxed_only_string(text: str) -> Optional[str]:
    idx = text.rfind("\\boxed")
    if idx < 0:
        idx = text.rfind("\\fbox")
        if idx < 0:
            return None
    i, depth, start = idx, 0, None
    while i < len(text):
        ch = text[i]
        if ch == "{":
            depth += 1
            if start is None:
                start = i
        elif ch == "}":
            depth -= 1
            if depth == 0 and start is not None:
                return text[idx:i + 1]
        i += 1
    return None


def remove_boxed(s: str) -> str:
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    m = re.match(r"\\(?:boxed|fbox)\{(.*)\}$", s, re.S)
    return m.group(1) if m else s


_UNITS = re.compile(r"\\text\{\s*[a-zA-Z ]+\}$")


def _fix_fracs(s: str) -> str:
    # \frac12 -> \frac{1}{2}, \frac1{2} -> \frac{1}{2}
    s = re.sub(r"\\frac(\d)(\d)", r"\\frac{\1}{\2}", s)
    s = re.sub(r"\\frac(\d)\{", r"\\frac{\1}{", s)
    s = re.sub(r"\\frac\{([^{}]+)\}(\d)", r"\\frac{\1}{\2}", s)
    return s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def _simple_slash_to_frac(s: str) -> str:
    m = re.fullmatch(r"(-?\d+)/(\d+)", s)
    return f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}" if m else s


def strip_string(s: str) -> str:
    s = str(s).replace("\n", "").replace("\\!", "")
    s = s.replace("\\\\", "\\").replace("tfrac", "frac").replace("dfrac", "frac")
    s = s.replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "")
    s = s.replace("\\$", "").replace("$", "")
    s = _UNITS.sub("", s)
    s = s.replace("\\%", "").replace("%", "")
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if s.startswith("."):
        s = "0" + s
    if "=" in s and len(s.split("=")[0]) <= 2:
        s = s.split("=", 1)[1]
    s = _fix_sqrt(s)
    s = s.replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    s = _simple_slash_to_frac(s)
    return s


def is_equiv(a: Optional[str], b: Optional[str]) -> bool:
    if a is None or b is None:
        return a is None and b is None
    try:
        return strip_string(a) == strip_string(b)
    except Exception:  # malformed latex: fall back to the raw comparison
        return a == b


def compute_score(solution_str: str, ground_truth: str) -> float:
    boxed = last_boxed_only_string(solution_str)
    if boxed is None:
        return 0.0
    return 1.0 if is_equiv(remove_boxed(boxed), ground_truth) else 0.0
