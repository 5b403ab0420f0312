"""Reward functions for agent tasks (reference: skyrl-agent/skyrl_agent/tasks/verifiers/{qa,py_functional,naive_dapo}.py).

* ``qa_scores(prediction, golds)``        exact match, substring match and token-level F1 after the usual normalisation
                                          (lower case, no punctuation, no articles), best over the gold answers;
* ``qa_reward(prediction, golds, metric)``;
* ``math_reward(response, gold, ...)``    the last boxed / ``Answer:`` expression against the gold one under the Minerva
                                          normalisation (``gym/envs/aime.py``), with a numeric fallback: two answers that
                                          both parse as numbers are equal when their values are;
* ``code_reward(response, tests, ...)``   the response's last code block against stdin / call-based tests in the guarded
                                          grader (``gym/envs/lcb.py``), all-or-nothing or the fraction of tests passed.
"""

from __future__ import annotations

from collections import Counter
from fractions import Fraction

from ..gym.envs import aime as _aime
from ..gym.envs import lcb as _lcb
from ..gym.envs.search import normalize_answer


def _f1(pred: str, gold: str) -> float:
    p, g = normalize_answer(pred).split(), normalize_answer(gold).split()
    if not p or not g:
        return float(p == g)
    same = sum((Counter(p) & Counter(g)).values())
    if same == 0:
        return 0.0
    prec, rec = same / len(p), same / len(g)
    return 2 * prec * rec / (prec + rec)


def qa_scores(prediction: str, golds) -> dict:
    golds = [golds] if isinstance(golds, (str, int, float)) else list(golds)
    p = normalize_answer(str(prediction))
    gs = [normalize_answer(str(g)) for g in golds]
    return {"em": float(any(g == p for g in gs)), "sub_em": float(any(g and g in p for g in gs)),
            "f1": max((_f1(str(prediction), str(g)) for g in golds), default=0.0)}


def qa_reward(prediction: str, golds, metric: str = "em") -> float:
    return qa_scores(prediction, golds)[metric]


def _as_number(text: str):
    t = text.replace(",", "").replace("$", "").strip()
    try:
        if t.startswith("\\frac{") and "}{" in t and t.endswith("}"):
            a, b = t[len("\\frac{"):-1].split("}{", 1)
            return Fraction(a) / Fraction(b)
        return Fraction(t)
    except (ValueError, ZeroDivisionError):
        return None


def math_reward(response: str, gold, mode: str = "auto", wrong_reward: float = 0.0) -> float:
    info = _aime.score_info(response, gold, mode)
    if info["acc"]:
        return 1.0
    if info["pred"] is not None and mode != "strict_box":
        a, b = _as_number(info["pred"]), _as_number(_aime.normalize(str(gold)))
        if a is not None and a == b:
            return 1.0
    return wrong_reward


def code_reward(response: str, tests, timeout_s: int = 6, partial: bool = False) -> float:
    code = _lcb.extract_code(response)
    if code is None:
        return 0.0
    tests = _lcb.normalize_tests(tests)
    if not tests:
        return 0.0
    if not partial:
        return _lcb.compute_score(response, tests, timeout_s)[1]
    passed = 0
    for t in tests:                                          # the grader stops at the first failure: one run per test
        res, _ = _lcb.grade(code, [t], timeout_s)
        passed += bool(res and res[0] is True)
    return passed / len(tests)
