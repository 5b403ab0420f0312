"""AIME / MATH-style environment: one turn, the final answer of the response is compared with the ground truth after
normalisation (reference: skyrl-gym/skyrl_gym/envs/aime/{env,utils}.py, the Minerva / DAPO math scoring).

``env_config.mode`` selects how the answer is found:

* ``"auto"`` (default): the last ``\\boxed{...}`` of the response, else the last ``Answer: ...`` line;
* ``"minerva"``: only an ``Answer: ...`` line within the last 300 characters (the reference's default);
* ``"strict_box"``: the last ``\\boxed{...}`` within the last 100 characters, compared as a string without normalisation.

Normalisation (``normalize``) follows the Minerva recipe: what stands left of the last ``=`` is dropped, ``$`` and spaces
go, unit words and typographic commands go, ``\\text{..}`` / ``\\textbf{..}`` / ``\\overline{..}`` / ``\\boxed{..}`` are
unwrapped, ``\\fracab`` and ``\\sqrta`` get their braces, digit groups lose their commas; on top of that integers lose
leading zeros and a trailing ``.0``.

Reward: 1 for a correct answer, ``env_config.wrong_reward`` otherwise (default -1, the reference's value; 0 is common
too). The ground truth is ``reward_spec.ground_truth`` (``reward_model.ground_truth`` is read as well)."""

from __future__ import annotations

import re

from ..core import BaseTextEnv, register

# words and commands that say nothing about the value (units, counting nouns, spacing)
_UNITS = ("square", "ways", "integers", "dollars", "mph", "inches", "hours", "km", "units", "points", "feet", "minutes", "digits",
          "cents", "degrees", "cm", "gm", "pounds", "meters", "meals", "edges", "students", "childrentickets", "multiples", "sue")
_DROP = ("\\ldots", "\\dots", "\\text{s}", "\\text{.}", "\\text{\ns}", "\\text{}^2", "\\text{}^3", "\\text{\n}", "\\text{}",
         "\\mathrm{th}", "^\\circ", "^{\\circ}", "\\;", ",\\!", "{,}", '"', "\\!", "\\,")
_SWAP = (("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), ("\\ ", ""), (" ", ""), ("mbox", "text"), (",\\text{and}", ","),
         ("\\text{and}", ","), ("\\text{m}", "\\text{}"))


def last_boxed(text: str) -> str | None:
    """Content of the last ``\\boxed{...}`` (braces balanced), or None."""
    i = text.rfind("\\boxed")
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0:
        return None
    depth = 0
    for k in range(j, len(text)):
        if text[k] == "{":
            depth += 1
        elif text[k] == "}":
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
    return None


def normalize(ans: str) -> str:
    a = str(ans).split("=")[-1]
    for old, new in _SWAP:
        a = a.replace(old, new)
    for w in _UNITS + _DROP:
        a = a.replace(w, "")
    a = re.sub(r"(.*?)(\$)(.*?)(\$)(.*)", r"$\3$", a)                  # keep the first inline formula when there is one
    for cmd in ("text", "textbf", "overline"):
        a = re.sub(r"\\" + cmd + r"\{(.*?)\}", r"\1", a)
    a = re.sub(r"\\boxed\{(.*)\}", r"\1", a)
    a = re.sub(r"frac([^{])(.)", r"frac{\1}{\2}", a)
    a = re.sub(r"sqrt([^{])", r"sqrt{\1}", a)
    a = a.replace("$", "").replace("\\%", "").replace("%", "").strip().rstrip(".")
    if a.replace(",", "").isdigit():
        a = a.replace(",", "")
    if re.fullmatch(r"-?\d+\.0+", a):
        a = a.split(".")[0]
    if re.fullmatch(r"-?\d+", a):
        sign, digits = ("-", a[1:]) if a.startswith("-") else ("", a)
        a = sign + (digits.lstrip("0") or "0")
    return a


def find_answer(text: str, mode: str = "auto") -> str | None:
    if mode == "strict_box":
        return last_boxed(text[-100:])
    if mode == "minerva":
        m = re.findall(r"(?i)answer\s*:\s*([^\n<]+)", text[-300:])
        return m[-1] if m else None
    ans = last_boxed(text)
    if ans is None:
        m = re.findall(r"(?i)answer\s*[:=]\s*([^\n<]+)", text)
        ans = m[-1] if m else None
    return ans


def score_info(text: str, ground_truth, mode: str = "auto") -> dict:
    """{"acc": bool, "pred": the normalised prediction or None}."""
    ans = find_answer(text, mode)
    if ans is None:
        return {"acc": False, "pred": None}
    if mode == "strict_box":
        return {"acc": ans == str(ground_truth), "pred": ans}
    pred = normalize(ans)
    return {"acc": pred == normalize(str(ground_truth)), "pred": pred}


def compute_score(text: str, ground_truth, mode: str = "auto", wrong_reward: float = 0.0) -> float:
    return 1.0 if score_info(text, ground_truth, mode)["acc"] else wrong_reward


class AIMEEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or self.extras.get("reward_model") or {}
        if "ground_truth" not in spec:
            raise ValueError("aime needs extras['reward_spec']['ground_truth']")
        self.ground_truth = spec["ground_truth"]
        self.mode = self.env_config.get("mode", "auto")
        if self.mode not in ("auto", "minerva", "strict_box"):
            raise ValueError(f"aime mode {self.mode!r} must be auto, minerva or strict_box")
        self.wrong_reward = float(self.env_config.get("wrong_reward", -1.0))
        self.acc = 0.0

    def step(self, action: str):
        info = score_info(action, self.ground_truth, self.mode)
        self.acc = float(info["acc"])
        return {"observations": [], "reward": 1.0 if info["acc"] else self.wrong_reward, "done": True, "metadata": info}

    def get_metrics(self) -> dict:
        return {"acc": self.acc}


register("aime", lambda c, e: AIMEEnv(c, e))
