"""Are two final answers of a maths problem the same answer?

Used only by the certainty test of the early-exit controller: consecutive probe answers such
as ``0.5``, ``\\frac{1}{2}`` and ``50\\%`` must count as agreement. Layers, cheapest first
(the reference's ``math_equal`` has the same layers: arctic_inference/dynasor/
evaluator.py:554-742):

1. normalised strings (case, spaces, ``\\left`` / ``\\right``, ``\\text{}``, units, ``$``);
2. multiple-choice letters (``(B)`` vs ``B``);
3. numbers, allowing thousands separators and the percentage variants x, x/100, 100x,
   relative tolerance 1e-4;
4. tuples / intervals / matrices element by element, equations as lhs - rhs;
5. symbolic difference with sympy after a small LaTeX-to-text translation.
"""

from __future__ import annotations

import math
import re
from typing import Optional

REL_TOL = 1e-4
_CHOICE = re.compile(r"^\(?([A-Ea-e])\)?[.:]?$")
_UNIT_WORDS = re.compile(r"\\?(text|mathrm|mbox)\{[^}]*\}")


def normalize(s) -> str:
    s = str(s).strip()
    s = s.replace("\\!", "").replace("\\,", "").replace("\\;", "").replace("\\ ", "")
    s = s.replace("\\left", "").replace("\\right", "").replace("$", "")
    s = s.replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac")
    s = re.sub(r"^\\boxed\{(.*)\}$", r"\1", s)
    s = _UNIT_WORDS.sub(lambda m: m.group(0)[m.group(0).index("{") + 1:-1]
                        if re.fullmatch(r"[\d.\-+/ ]*", m.group(0)[m.group(0).index("{") + 1:-1]) else "", s)
    s = s.replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    s = s.rstrip(".").strip()
    if s.startswith("{") and s.endswith("}") and _balanced(s[1:-1]):
        s = s[1:-1]
    return re.sub(r"\s+", "", s)


def _balanced(s: str) -> bool:
    d = 0
    for c in s:
        d += c in "{([" 
        d -= c in "})]"
        if d < 0:
            return False
    return d == 0


def parse_number(s: str) -> Optional[float]:
    t = s.replace(",", "").replace("\\%", "%")
    pct = t.endswith("%")
    if pct:
        t = t[:-1]
    m = re.fullmatch(r"\\frac\{(-?[\d.]+)\}\{(-?[\d.]+)\}", t)
    try:
        if m:
            v = float(m.group(1)) / float(m.group(2))
        elif re.fullmatch(r"-?\d+/\d+", t):
            a, b = t.split("/")
            v = float(a) / float(b)
        else:
            v = float(t)
    except (ValueError, ZeroDivisionError):
        return None
    return v / 100.0 if pct else v


def numeric_equal(a: float, b: float, include_percentage: bool = True) -> bool:
    cands = [b, b / 100.0, b * 100.0] if include_percentage else [b]
    return any(math.isclose(a, c, rel_tol=REL_TOL, abs_tol=1e-12) for c in cands)


def _split_top(s: str, sep: str = ",") -> list:
    out, d, cur = [], 0, ""
    for c in s:
        if c in "{([":
            d += 1
        elif c in "})]":
            d -= 1
        if c == sep and d == 0:
            out.append(cur)
            cur = ""
        else:
            cur += c
    out.append(cur)
    return out


def latex_to_text(s: str) -> str:
    """Enough LaTeX for final answers: fractions, roots, powers, products, pi."""
    for _ in range(8):
        t = re.sub(r"\\frac\{([^{}]*)\}\{([^{}]*)\}", r"((\1)/(\2))", s)
        t = re.sub(r"\\sqrt\[([^\]]*)\]\{([^{}]*)\}", r"((\2)**(1/(\1)))", t)
        t = re.sub(r"\\sqrt\{([^{}]*)\}", r"sqrt(\1)", t)
        t = re.sub(r"\^\{([^{}]*)\}", r"**(\1)", t)
        if t == s:
            break
        s = t
    s = s.replace("^", "**").replace("\\cdot", "*").replace("\\times", "*").replace("\\div", "/")
    s = s.replace("\\pi", "pi").replace("\\infty", "oo").replace("\\%", "/100")
    s = re.sub(r"\\(sin|cos|tan|log|ln|exp)", r"\1", s).replace("ln(", "log(")
    s = s.replace("{", "(").replace("}", ")")
    s = re.sub(r"(\d)([a-zA-Z(])", r"\1*\2", s)       # 2x -> 2*x, 3(…) -> 3*(…)
    s = re.sub(r"\)([\w(])", r")*\1", s)
    return s


def symbolic_equal(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr
        ea, eb = parse_expr(latex_to_text(a)), parse_expr(latex_to_text(b))
        if ea == eb:
            return True
        diff = sympy.simplify(ea - eb)
        if diff == 0:
            return True
        return bool(abs(complex(sympy.N(diff))) < 1e-9) if not diff.free_symbols else False
    except Exception:  # noqa: BLE001 - unparsable answers are simply not equal here
        return False


def math_equal(pred, ref, include_percentage: bool = True) -> bool:
    if pred is None or ref is None:
        return False
    a, b = normalize(pred), normalize(ref)
    if a == "" or b == "":
        return False
    if a.lower() == b.lower():
        return True
    ca, cb = _CHOICE.match(a), _CHOICE.match(b)
    if ca and cb:
        return ca.group(1).upper() == cb.group(1).upper()
    na, nb = parse_number(a), parse_number(b)
    if na is not None and nb is not None:
        return numeric_equal(na, nb, include_percentage)
    # matrices: rows separated by \\, entries by &
    if "\\begin{" in a and "\\begin{" in b:
        strip = lambda s: re.sub(r"\\(begin|end)\{[a-z]*matrix\}", "", s)
        ra, rb = strip(a).split("\\\\"), strip(b).split("\\\\")
        if len(ra) != len(rb):
            return False
        return all(len(x.split("&")) == len(y.split("&")) and
                   all(math_equal(p, q, include_percentage) for p, q in zip(x.split("&"), y.split("&")))
                   for x, y in zip(ra, rb))
    # tuples / intervals / sets
    if a[:1] in "([{" and b[:1] in "([{" and a[-1:] in ")]}" and b[-1:] in ")]}":
        if (a[0], a[-1]) != (b[0], b[-1]):
            return False
        pa, pb = _split_top(a[1:-1]), _split_top(b[1:-1])
        return len(pa) == len(pb) and all(math_equal(p, q, include_percentage) for p, q in zip(pa, pb))
    # equations: compare lhs - rhs (up to sign); "x = 5" also matches the bare "5"
    if a.count("=") == 1 and b.count("=") == 1:
        la, ra_ = a.split("=")
        lb, rb_ = b.split("=")
        if symbolic_equal("(%s)-(%s)" % (la, ra_), "(%s)-(%s)" % (lb, rb_)) or \
                symbolic_equal("(%s)-(%s)" % (la, ra_), "(%s)-(%s)" % (rb_, lb)):
            return True
        return math_equal(la, lb) and math_equal(ra_, rb_)
    if a.count("=") == 1 and len(a.split("=")[0]) <= 2 and "=" not in b:
        return math_equal(a.split("=")[1], b, include_percentage)
    if b.count("=") == 1 and len(b.split("=")[0]) <= 2 and "=" not in a:
        return math_equal(a, b.split("=")[1], include_percentage)
    return symbolic_equal(a, b)
