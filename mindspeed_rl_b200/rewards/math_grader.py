"""Answer extraction and mathematical equivalence grading for the rule verifiers.

Capabilities (reference: ``mindspeed_rl/utils/math_eval_toolkit/{parser,grader}.py``,
``mindspeed_rl/models/math_dapo.py``): pull the final answer out of a response (``\\boxed{}``,
"the answer is", last number), normalise LaTeX-ish strings, compare numerically (with percent
forms and relative tolerance), element-wise for tuples / intervals / matrices, and symbolically
through sympy when available -- always under a wall-clock limit.
"""
from __future__ import annotations

import math
import multiprocessing as mp
import re
import threading
from typing import Any, Callable, List, Optional, Sequence

# ----------------------------------------------------------------------------------------------
# bounded execution
# ----------------------------------------------------------------------------------------------
_warm = False


def warm_up() -> None:
    """Load the symbolic-algebra package once, outside any time limit: its first import takes seconds, which
    would otherwise make the first graded answer of a process time out (and score as wrong)."""
    global _warm
    if _warm:
        return
    _warm = True
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr

        sympy.simplify(parse_expr("x + 1") - parse_expr("1 + x"))
    except Exception:
        pass
    _latex_parser()


_parse_latex: Any = False            # False: not looked up yet; None: unavailable


def _latex_parser():
    """sympy's LaTeX front end when its grammar runtime is installed (looked up once: the failed import alone
    takes a second)."""
    global _parse_latex
    if _parse_latex is False:
        try:
            from sympy.parsing.latex import parse_latex

            parse_latex("x")
            _parse_latex = parse_latex
        except Exception:
            _parse_latex = None
    return _parse_latex


def call_with_timeout(fn: Callable, *args, timeout: float = 1.0, default: Any = None, **kw) -> Any:
    """Run ``fn`` in a daemon thread and give up after ``timeout`` seconds (returns ``default``).
    Exceptions inside ``fn`` also yield ``default``."""
    warm_up()
    box: List[Any] = [default]

    def run():
        try:
            box[0] = fn(*args, **kw)
        except Exception:
            box[0] = default

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(timeout)
    return box[0] if not t.is_alive() else default


def bounded_map(fn: Callable, items: Sequence[Sequence[Any]], timeout: float = 1.0, default: Any = None,
                total_timeout: Optional[float] = None) -> List[Any]:
    """``[fn(*item) for item in items]``, every call under ``timeout`` seconds.  With more than one grading
    process configured (``bounded_pool.set_parallel``) the calls run in worker processes, which are killed
    and replaced when a call passes its limit; otherwise they run here, bounded by a thread join (a call
    that never returns then leaves a sleeping daemon thread behind)."""
    from . import bounded_pool

    if bounded_pool.parallel() > 1 and len(items) > 0:
        return bounded_pool.shared_pool().map(fn, items, timeout=timeout, default=default,
                                              total_timeout=total_timeout)
    return [call_with_timeout(fn, *item, timeout=timeout, default=default) for item in items]


# ----------------------------------------------------------------------------------------------
# extraction
# ----------------------------------------------------------------------------------------------
def last_boxed_span(text: str) -> Optional[str]:
    """Return the last ``\\boxed{...}`` (or ``\\fbox{...}``) including the command, brace-matched."""
    idx = max(text.rfind("\\boxed"), text.rfind("\\fbox"))
    if idx < 0:
        return None
    i = text.find("{", idx)
    if i < 0:
        return None
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[idx:j + 1]
    return None


def extract_boxed_content(text: str) -> Optional[str]:
    span = last_boxed_span(text)
    if span is None:
        return None
    return span[span.find("{") + 1:-1]


_NUM_RE = re.compile(r"-?\d[\d,]*\.?\d*(?:[eE][-+]?\d+)?%?|-?\.\d+")


def extract_answer(pred: str, data_name: str = "math") -> str:
    pred = pred.strip()
    boxed = extract_boxed_content(pred)
    if boxed is not None:
        ans = boxed
    elif "he answer is" in pred:
        ans = pred.split("he answer is")[-1].strip()
    elif "final answer is" in pred:
        ans = pred.split("final answer is")[-1].strip()
    else:
        nums = _NUM_RE.findall(pred.replace(",", ""))
        ans = nums[-1] if nums else ""
    ans = re.sub(r"\n\s*", "", ans).strip()
    ans = ans.rstrip(".").rstrip("/")
    return strip_string(ans)


# ----------------------------------------------------------------------------------------------
# normalisation
# ----------------------------------------------------------------------------------------------
def _fix_fracs(s: str) -> str:
    parts = s.split("\\frac")
    out = parts[0]
    for p in parts[1:]:
        out += "\\frac"
        if p and p[0] != "{":
            if len(p) >= 2:
                a, b, rest = p[0], p[1], p[2:]
                out += "{" + a + "}" + (b if b == "{" else "{" + b + "}") + rest if b != "{" \
                    else "{" + a + "}" + p[1:]
            else:
                out += p
        else:
            out += p
    return out


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def _fix_a_slash_b(s: str) -> str:
    m = re.fullmatch(r"(-?\d+)/(\d+)", s)
    return f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}" if m else s


def strip_string(s: str) -> str:
    s = str(s).strip().replace("\n", "").rstrip(".")
    s = s.replace("\\!", "").replace("\\ ", " ")
    s = s.replace("tfrac", "frac").replace("dfrac", "frac")
    s = s.replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "").replace("$", "")
    s = re.sub(r"\\text\{\s*([^}]*)\}", r"\1", s)
    s = re.sub(r"\\mbox\{[^}]*\}", "", s)
    s = s.replace("\\%", "%")
    for unit in ("degrees", "degree", "cm", "units", "unit", "meters", "inches", "square"):
        s = re.sub(rf"\s+{unit}\b", "", s)
    if s.startswith("."):
        s = "0" + s
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = _fix_sqrt(s)
    s = s.replace(" ", "")
    s = _fix_fracs(s)
    s = _fix_a_slash_b(s)
    return s


# ----------------------------------------------------------------------------------------------
# comparison
# ----------------------------------------------------------------------------------------------
def _to_number(s: str) -> Optional[float]:
    s = s.replace(",", "").strip()
    pct = s.endswith("%")
    if pct:
        s = s[:-1]
    m = re.fullmatch(r"\\frac\{(-?[\d.]+)\}\{(-?[\d.]+)\}", s)
    try:
        v = float(m.group(1)) / float(m.group(2)) if m else float(s)
    except (ValueError, ZeroDivisionError):
        return None
    return v / 100 if pct else v


def numeric_equal(a: float, b: float, rel_tol: float = 1e-4) -> bool:
    return math.isclose(a, b, rel_tol=rel_tol, abs_tol=1e-9)


def symbolic_equal(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr
    except Exception:
        return False

    latex = _latex_parser()

    def parse(s):
        for f in ((latex,) if latex is not None else ()) + (lambda x: parse_expr(x.replace("^", "**")),):
            try:
                return f(s)
            except Exception:
                continue
        return None

    ea, eb = parse(a), parse(b)
    if ea is None or eb is None:
        return False
    try:
        if ea == eb or sympy.simplify(ea - eb) == 0:
            return True
    except Exception:
        pass
    try:
        return numeric_equal(float(sympy.N(ea)), float(sympy.N(eb)))
    except Exception:
        return False


def _split_elements(s: str) -> Optional[List[str]]:
    if len(s) >= 2 and s[0] in "([" and s[-1] in ")]":
        inner, parts, depth, cur = s[1:-1], [], 0, ""
        for ch in inner:
            if ch in "([{":
                depth += 1
            elif ch in ")]}":
                depth -= 1
            if ch == "," and depth == 0:
                parts.append(cur)
                cur = ""
            else:
                cur += ch
        parts.append(cur)
        return parts
    return None


def math_equal(prediction: Any, reference: Any, include_percentage: bool = True,
               is_close: bool = True) -> bool:
    """Equivalence of two answers: exact string, numeric (also x/100 and x*100 readings),
    element-wise for bracketed lists, equations side by side, then symbolic."""
    if prediction is None or reference is None:
        return False
    p, r = strip_string(str(prediction)), strip_string(str(reference))
    if p.lower() == r.lower():
        return True
    pn, rn = _to_number(p), _to_number(r)
    if pn is not None and rn is not None:
        cands = [rn, rn / 100, rn * 100] if include_percentage else [rn]
        return any(numeric_equal(pn, c) if is_close else pn == c for c in cands)
    pe, re_ = _split_elements(p), _split_elements(r)
    if pe is not None and re_ is not None:
        if len(pe) != len(re_) or (p[0], p[-1]) != (r[0], r[-1]):
            return False
        return all(math_equal(x, y, include_percentage, is_close) for x, y in zip(pe, re_))
    if p.count("=") == 1 and r.count("=") == 1:
        pl, pr = p.split("=")
        rl, rr = r.split("=")
        return symbolic_equal(f"({pl})-({pr})", f"({rl})-({rr})") or \
            symbolic_equal(f"({pl})-({pr})", f"({rr})-({rl})")
    if p.count("=") == 1 and len(p.split("=")[0]) <= 2 and "=" not in r:
        return math_equal(p.split("=")[1], r, include_percentage, is_close)
    return bool(call_with_timeout(symbolic_equal, p, r, timeout=1.0, default=False))


def grade_answer(given: Optional[str], truth: str) -> bool:
    if given is None:
        return False
    return bool(call_with_timeout(math_equal, given, truth, timeout=2.0, default=False))


def math_verify_score(solution: str, truth: str) -> float:
    """Score with the ``math_verify`` package when importable, else the built-in grader."""
    try:
        from math_verify import parse, verify  # type: ignore

        gold = parse(f"\\boxed{{{truth}}}")
        return 1.0 if verify(gold, parse(solution)) else 0.0
    except Exception:
        boxed = extract_boxed_content(solution)
        return 1.0 if grade_answer(boxed, truth) else 0.0


# ----------------------------------------------------------------------------------------------
# DAPO "Answer:" protocol (Minerva-style normalisation)
# ----------------------------------------------------------------------------------------------
_SUBS = [("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), (r"\ ", ""), (" ", ""), ("mbox", "text"),
         (",\\text{and}", ","), ("\\text{and}", ","), ("\\text{m}", "\\text{}")]
_REMOVED = ["square", "ways", "integers", "dollars", "mph", "inches", "hours", "km", "units", "\\ldots",
            "sue", "points", "feet", "minutes", "digits", "cents", "degrees", "cm", "gm", "pounds",
            "meters", "meals", "edges", "students", "childrentickets", "multiples", "\\text{s}",
            "\\text{.}", "\\text{\ns}", "\\text{}^2", "\\text{}^3", "\\text{\n}", "\\text{}",
            r"\mathrm{th}", r"^\circ", r"^{\circ}", r"\;", r",\!", "{,}", '"', "\\dots"]


def normalize_final_answer(ans: str) -> str:
    ans = ans.split("=")[-1]
    for a, b in _SUBS:
        ans = ans.replace(a, b)
    for w in _REMOVED:
        ans = ans.replace(w, "")
    ans = re.sub(r"(.*?)(\$)(.*?)(\$)(.*)", r"$\3$", ans)
    for cmd in ("text", "textbf", "overline", "boxed"):
        ans = re.sub(rf"(\\{cmd}\{{)(.*?)(\}})", r"\2", ans)
    ans = re.sub(r"(frac)([^{])(.)", r"frac{\2}{\3}", ans)
    ans = re.sub(r"(sqrt)([^{])", r"sqrt{\2}", ans)
    ans = ans.replace("$", "")
    if ans.replace(",", "").isdigit():
        ans = ans.replace(",", "")
    return ans.strip()


def dapo_is_correct(solution_tail: str, truth: str) -> bool:
    m = re.findall(r"(?i)Answer\s*:\s*([^\n]+)", solution_tail)
    if not m:
        return False
    return normalize_final_answer(m[-1]) == normalize_final_answer(str(truth))


def dapo_is_correct_boxed(solution_tail: str, truth: str) -> bool:
    boxed = extract_boxed_content(solution_tail)
    if boxed is None:
        return False
    return normalize_final_answer(boxed) == normalize_final_answer(str(truth)) or boxed.strip() == str(truth).strip()
