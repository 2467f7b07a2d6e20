"""String normalisation of MATH-style answers (the rules of the MATH benchmark's
``math_equivalence`` as used by the reference, math_utils/math_normalize.py:8-161): strip
``\\text{}``, ``\\left/\\right``, units, degrees, dollar and percent signs, canonicalise
``\\frac`` / ``\\sqrt`` arguments, ``a/b`` -> ``\\frac{a}{b}``, ``0.5`` -> ``\\frac{1}{2}``."""
from __future__ import annotations

import re
from typing import Optional


def normalize_answer(answer: Optional[str]) -> Optional[str]:
    if answer is None:
        return None
    answer = answer.strip()
    try:
        m = re.search(r"^\\text\{(?P<text>.+?)\}$", answer)
        if m is not None:
            answer = m.group("text").strip()
        return _strip_string(answer)
    except Exception:  # malformed LaTeX: compare the raw string
        return answer


def _fix_fracs(string: str) -> str:
    """``\\frac12`` -> ``\\frac{1}{2}``, ``\\frac1{72}`` -> ``\\frac{1}{72}``; braces are added
    only to single-character arguments, anything already braced is left alone."""
    head, *rest = string.split("\\frac")
    out = head
    for part in rest:
        out += "\\frac"
        if part.startswith("{"):
            out += part
            continue
        if len(part) < 2:
            return string
        a, b, tail = part[0], part[1], part[2:]
        out += "{" + a + "}" + (b if b == "{" else "{" + b + "}") + tail
    return out


def _fix_a_slash_b(string: str) -> str:
    parts = string.split("/")
    if len(parts) != 2:
        return string
    try:
        a, b = int(parts[0]), int(parts[1])
    except ValueError:
        return string
    if string != f"{a}/{b}":
        return string
    return "\\frac{" + str(a) + "}{" + str(b) + "}"


def _remove_right_units(string: str) -> str:
    # "\text{ " (with the space) introduces a unit in this data
    if "\\text{ " in string:
        pieces = string.split("\\text{ ")
        assert len(pieces) == 2
        return pieces[0]
    return string


def _fix_sqrt(string: str) -> str:
    if "\\sqrt" not in string:
        return string
    head, *rest = string.split("\\sqrt")
    out = head
    for part in rest:
        out += "\\sqrt" + (part if part.startswith("{") else "{" + part[0] + "}" + part[1:])
    return out




def _strip_string(string: str) -> str:
    string = string.replace("\n", "").replace("\\!", "").replace("\\\\", "\\")
    string = string.replace("tfrac", "frac").replace("dfrac", "frac")
    for tok in ("\\left", "\\right", "^{\\circ}", "^\\circ", "\\$"):
        string = string.replace(tok, "")
    string = _remove_right_units(string)
    string = string.replace("\\%", "").replace(r"\%", "")
    string = string.replace(" .", " 0.").replace("{.", "{0.")
    if not string:
        return string
    if string[0] == ".":
        string = "0" + string
    sides = string.split("=")
    if len(sides) == 2 and len(sides[0]) <= 2:   # "k = 5" -> "5"
        string = sides[1]
    string = _fix_sqrt(string).replace(" ", "")
    string = _fix_fracs(string)
    if string == "0.5":
        string = "\\frac{1}{2}"
    return _fix_a_slash_b(string)
