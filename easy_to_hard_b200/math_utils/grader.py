"""Answer grading for MATH-style problems (behaviour of the reference's
math_utils/grader.py:235-289, itself the PRM800K grader).

``grade_answer(given, truth)`` is True when the two normalise to the same string under the
MATH rules, or under the second, more aggressive normalisation below (units, "million",
LaTeX -> text, mixed numbers, thousands separators), element-wise for tuples / intervals with
identical brackets. As in the reference, symbolic (sympy) equality is NOT used for the verdict
(its call is commented out upstream, grader.py:284-285): unreduced fractions and non-identical
integers are wrong. ``are_equal_under_sympy`` is kept as a utility.

LaTeX -> text uses pylatexenc when it is installed and a small built-in converter otherwise.
"""
from __future__ import annotations

import re
from typing import List, Optional

from . import math_normalize

BAD_SUBSTRINGS = ["^{", "^("]
BAD_REGEXES = [r"\^[0-9]+\^", r"\^[0-9][0-9]+"]
TUPLE_CHARS = "()[]"
_UNITS = ["degree", "cm", "centimeter", "meter", "mile", "second", "minute", "hour", "day",
          "week", "month", "year", "foot", "feet", "inch", "yard"]


def _sympy_parse(expr: str):
    from sympy.parsing import sympy_parser
    return sympy_parser.parse_expr(
        expr.replace("^", "**"),
        transformations=(sympy_parser.standard_transformations
                         + (sympy_parser.implicit_multiplication_application,)))


def _latex_to_text_builtin(expr: str) -> str:
    """Minimal LaTeX -> text: fractions, roots, common symbols, braces."""
    frac = re.compile(r"\\frac\s*\{([^{}]*)\}\s*\{([^{}]*)\}")
    prev = None
    while prev != expr:
        prev = expr
        expr = frac.sub(r"\1/\2", expr)
    expr = re.sub(r"\\sqrt\s*\{([^{}]*)\}", r"√(\1)", expr)
    for src, dst in (("\\pi", "π"), ("\\infty", "∞"), ("\\cup", "∪"), ("\\cdot", "·"),
                     ("\\times", "×"), ("\\le", "≤"), ("\\ge", "≥"), ("\\ ", " "), ("\\,", " ")):
        expr = expr.replace(src, dst)
    expr = re.sub(r"\\(text|mathrm|mathbf|textbf)\s*\{([^{}]*)\}", r"\2", expr)
    expr = re.sub(r"\\[a-zA-Z]+", "", expr)
    return expr.replace("{", "").replace("}", "")


def _parse_latex(expr: str) -> str:
    expr = expr.replace("\\tfrac", "\\frac").replace("\\dfrac", "\\frac")
    expr = expr.replace("\\frac", " \\frac")  # keeps mixed numbers apart
    try:
        from pylatexenc import latex2text
        expr = latex2text.LatexNodes2Text().latex_to_text(expr)
    except ImportError:
        expr = _latex_to_text_builtin(expr)
    for src, dst in (("√", "sqrt"), ("π", "pi"), ("∞", "inf"), ("∪", "U"), ("·", "*"),
                     ("×", "*")):
        expr = expr.replace(src, dst)
    return expr.strip()


def _is_float(num: str) -> bool:
    try:
        float(num)
        return True
    except ValueError:
        return False


def _is_int(x: float) -> bool:
    try:
        return abs(x - int(round(x))) <= 1e-7
    except Exception:
        return False


def _is_frac(expr: str) -> bool:
    return bool(re.search(r"^-?[0-9]+.?/0*[1-9][0-9]*.?$", expr))


def _strip_properly_formatted_commas(expr: str) -> str:
    """1,234,567 -> 1234567 without touching tuple commas."""
    pat = re.compile(r"(\d)(,)(\d\d\d)($|\D)")
    while True:
        nxt = pat.sub(r"\1\3\4", expr)
        if nxt == expr:
            return nxt
        expr = nxt


def _str_is_int(x: str) -> bool:
    try:
        v = float(_strip_properly_formatted_commas(x))
        return abs(v - int(round(v))) <= 1e-7
    except Exception:
        return False


def _str_to_int(x: str) -> int:
    return int(float(x.replace(",", "")))


def _inject_implicit_mixed_number(step: str) -> str:
    """"7 3/4" -> "7+3/4"."""
    return re.sub(r"([0-9]) +([0-9])", r"\1+\2", step)


def _normalize(expr: Optional[str]) -> Optional[str]:
    if expr is None:
        return None
    m = re.search(r"^\\text\{(?P<text>.+?)\}$", expr)
    if m is not None:
        expr = m.group("text")
    expr = expr.replace("\\%", "%").replace("\\$", "$").replace("$", "").replace("%", "")
    expr = expr.replace(" or ", " , ").replace(" and ", " , ")
    expr = (expr.replace("million", "*10^6").replace("billion", "*10^9")
            .replace("trillion", "*10^12"))
    for unit in _UNITS:
        expr = re.sub(rf"{unit}(es)?(s)? *(\^[0-9]+)?", "", expr)
    expr = re.sub(r"\^ *\\circ", "", expr)
    if expr and expr[0] == "{" and expr[-1] == "}":
        expr = expr[1:-1]
    expr = re.sub(r",\\! *", "", expr)
    if _is_float(expr) and _is_int(float(expr)):
        expr = str(int(round(float(expr))))
    if "\\" in expr:
        try:
            expr = _parse_latex(expr)
        except Exception:
            pass
    expr = re.sub("- *", "-", expr)
    expr = _inject_implicit_mixed_number(expr).replace(" ", "")
    expr = expr.replace("{", "").replace("}", "").lower()
    if _str_is_int(expr):
        expr = str(_str_to_int(expr))
    return expr


def count_unknown_letters_in_expr(expr: str) -> int:
    expr = expr.replace("sqrt", "").replace("frac", "")
    return len({c for c in expr if c.isalpha()})


def should_allow_eval(expr: str) -> bool:
    """Keep sympy away from free text and from towers of exponents (it may hang)."""
    if count_unknown_letters_in_expr(expr) > 2:
        return False
    if any(s in expr for s in BAD_SUBSTRINGS):
        return False
    return not any(re.search(r, expr) for r in BAD_REGEXES)


def are_equal_under_sympy(ground_truth_normalized: str, given_normalized: str) -> bool:
    try:
        import sympy
        diff = f"({ground_truth_normalized})-({given_normalized})"
        if should_allow_eval(diff):
            return sympy.simplify(_sympy_parse(diff)) == 0
    except Exception:
        pass
    return False


def split_tuple(expr: str) -> List[str]:
    """Elements of a tuple / interval; a plain value is a 1-element list."""
    expr = _strip_properly_formatted_commas(expr)
    if not expr:
        return []
    if (len(expr) > 2 and expr[0] in TUPLE_CHARS and expr[-1] in TUPLE_CHARS
            and all(ch not in expr[1:-1] for ch in TUPLE_CHARS)):
        return [e.strip() for e in expr[1:-1].split(",")]
    return [expr]


def grade_answer(given_answer: Optional[str], ground_truth: str) -> bool:
    if given_answer is None:
        return False
    if math_normalize.normalize_answer(ground_truth) == \
            math_normalize.normalize_answer(given_answer):
        return True
    truth, given = _normalize(ground_truth), _normalize(given_answer)
    if truth is None:
        return False
    if truth == given:
        return True
    if not given:
        return False
    t_elems, g_elems = split_tuple(truth), split_tuple(given)
    if len(t_elems) > 1 and (truth[0] != given[0] or truth[-1] != given[-1]):
        return False
    if len(t_elems) != len(g_elems):
        return False
    for t, g in zip(t_elems, g_elems):
        if _is_frac(t) and _is_frac(g):
            ok = t == g            # unreduced fractions are not accepted
        else:
            ok = False             # integers must match exactly; no symbolic fallback
        if not ok:
            return False
    return True
