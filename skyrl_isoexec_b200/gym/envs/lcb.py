"""LiveCodeBench-style code generation: the model's last fenced code block is run against the task's tests and the
episode's reward is 1 only if every test passes (reference: skyrl-gym/skyrl_gym/envs/lcb/env.py and livecodebench.py).

Tests come as ``reward_spec.ground_truth``: a list (or its JSON text) of ``{"input", "output", "testtype", "metadata"}``.

* ``testtype == "functional"``: ``metadata.func_name`` names a method of ``class Solution`` (or a top-level function);
  ``input`` holds one JSON value per line, the arguments; ``output`` is the expected return value as JSON. A returned
  tuple counts as the list of its items.
* otherwise (``"stdin"``): the program reads ``input`` on standard input; what it prints is compared with ``output`` line
  by line after stripping, and where the text differs, number by number (so ``1.0`` equals ``1`` and ``0.50`` equals ``0.5``).
* the older ``{"assert": "<statements>"}`` form appends the statements to the program.

Grading happens in ONE child interpreter per submission (``python -I``, fed a JSON job on its standard input), which

* caps its address space and forbids core dumps, child processes and the usual destructive calls (``os.system``,
  ``os.remove``, ``shutil.rmtree``, ``subprocess.Popen`` ...) before it touches the submission,
* gives every test its own alarm (``timeout_s``) and stops at the first failing test,
* reports one verdict per test: ``true``, or ``-2`` wrong answer, ``-3`` time limit, ``-4`` runtime / compile error,

and the parent kills the child if it overruns ``(timeout_s + 1) * tests + 5`` seconds in total (every test then counts as
failed, ``-1``).
"""

from __future__ import annotations

import json
import re
import subprocess
import sys

from ..core import BaseTextEnv, register

_HARNESS = r'''
import faulthandler, io, json, os, signal, sys, time
from decimal import Decimal, InvalidOperation

job = json.loads(sys.stdin.read())
real_stdout = sys.stdout

def guard(mem_bytes):
    import builtins, resource, shutil, subprocess
    if mem_bytes:
        for lim in (resource.RLIMIT_AS, resource.RLIMIT_DATA):
            try:
                resource.setrlimit(lim, (mem_bytes, mem_bytes))
            except (ValueError, OSError):
                pass
    resource.setrlimit(resource.RLIMIT_CORE, (0, 0))
    faulthandler.disable()
    builtins.exit = builtins.quit = None
    os.environ["OMP_NUM_THREADS"] = "1"
    for name in ("kill", "system", "putenv", "remove", "removedirs", "rmdir", "fchdir", "setuid", "fork", "forkpty", "killpg",
                 "rename", "renames", "truncate", "replace", "unlink", "fchmod", "fchown", "chmod", "chown", "chroot", "lchown",
                 "chdir", "execv", "execve", "execl", "execlp", "execvp", "popen", "spawnl", "spawnv"):
        if hasattr(os, name):
            setattr(os, name, None)
    shutil.rmtree = shutil.move = shutil.chown = None
    subprocess.Popen = None

class Timeout(Exception):
    pass

def on_alarm(signum, frame):
    raise Timeout()

def short(x, n=300):
    s = x if isinstance(x, str) else repr(x)
    return s if len(s) <= n else s[:n // 2] + "...(truncated)..." + s[-n // 2:]

PRELUDE = ("import sys, os, math, re, json, heapq, bisect, itertools, functools, collections, string, random, operator, copy, typing\n"
           "from typing import *\nfrom collections import *\nfrom itertools import *\nfrom functools import *\nfrom heapq import *\n"
           "from bisect import *\nfrom math import *\nsys.setrecursionlimit(50000)\n")

def lines_of(s):
    return [ln.strip() for ln in s.strip().split("\n")]

def same_output(got, want):
    a, b = lines_of(got), lines_of(want)
    if len(a) != len(b):
        return False
    for x, y in zip(a, b):
        if x == y:
            continue
        try:
            if [Decimal(t) for t in x.split()] != [Decimal(t) for t in y.split()]:
                return False
        except InvalidOperation:
            return False
    return True

def run():
    code, tests, limit = job["code"], job["tests"], job["timeout"]
    signal.signal(signal.SIGALRM, on_alarm)
    guard(job.get("memory_bytes"))
    results = []
    def fail(code_, msg, **kw):
        results.append(code_)
        return results, dict(kw, error_code=code_, error_message=msg)
    fn_name = next((t.get("metadata", {}).get("func_name") for t in tests if t.get("testtype") == "functional"), None)
    fn = None
    if fn_name is not None:
        ns = {"__name__": "__submission__"}
        signal.alarm(limit)
        try:
            exec(compile(PRELUDE + code, "<submission>", "exec"), ns)
            owner = ns.get("Solution")
            fn = getattr(owner(), fn_name) if owner is not None and hasattr(owner, fn_name) else ns.get(fn_name)
        except BaseException as e:
            return fail(-4, "Compilation Error" if isinstance(e, SyntaxError) else "Runtime Error", error=repr(e))
        finally:
            signal.alarm(0)
        if fn is None:
            return fail(-4, "Runtime Error", error="no function " + fn_name)
    spent = 0.0
    for t in tests:
        kind = "assert" if "assert" in t else ("functional" if t.get("testtype") == "functional" else "stdin")
        signal.alarm(limit)
        t0 = time.time()
        try:
            if kind == "functional":
                args = [json.loads(ln) for ln in t["input"].split("\n") if ln.strip() != ""]
                want = json.loads(t["output"])
                got = fn(*args)
                if isinstance(got, tuple):
                    got = list(got)
                ok, shown = got == want, got
            else:
                src = code + ("\n" + t["assert"] if kind == "assert" else "")
                sys.stdin, sys.stdout = io.StringIO(t.get("input", "")), io.StringIO()
                try:
                    exec(compile(PRELUDE + src, "<submission>", "exec"), {"__name__": "__main__"})
                except SystemExit:
                    pass
                finally:
                    got, sys.stdout, sys.stdin = sys.stdout.getvalue(), real_stdout, sys.__stdin__
                ok, shown = (True if kind == "assert" else same_output(got, str(t.get("output", "")))), got
            signal.alarm(0)
            spent += time.time() - t0
            if not ok:
                return fail(-2, "Wrong Answer", output=short(shown), inputs=short(t.get("input", "")), expected=short(t.get("output", "")))
            results.append(True)
        except Timeout:
            sys.stdout = real_stdout
            return fail(-3, "Time Limit Exceeded", inputs=short(t.get("input", "")))
        except BaseException as e:
            signal.alarm(0)
            sys.stdout = real_stdout
            return fail(-4, "Compilation Error" if isinstance(e, SyntaxError) else "Runtime Error", error=short(repr(e)), inputs=short(t.get("input", "")))
        finally:
            signal.alarm(0)
    return results, {"execution_time": spent}

res, meta = run()
real_stdout.write("\n@@verdict@@" + json.dumps({"results": res, "metadata": meta}) + "\n")
real_stdout.flush()
'''


def extract_code(text: str) -> str | None:
    """The LAST fenced block of a response (any language tag), or None."""
    m = re.findall(r"```(?:\w+)?\n(.*?)```", text, flags=re.S)
    return m[-1].strip() if m else None


def normalize_tests(tests) -> list[dict]:
    if isinstance(tests, str):
        tests = json.loads(tests)
    if isinstance(tests, dict) and "inputs" in tests:           # the packed form: {"inputs": [...], "outputs": [...], "fn_name"?}
        fn = tests.get("fn_name")
        tests = [{"input": i, "output": o, "testtype": "functional" if fn else "stdin", "metadata": {"func_name": fn} if fn else {}}
                 for i, o in zip(tests["inputs"], tests["outputs"])]
    tests = list(tests or [])
    for t in tests:
        if t.get("testtype") == "functional" and not (t.get("metadata") or {}).get("func_name"):
            raise ValueError("a functional test needs metadata.func_name (is the dataset preprocessed?)")
    return tests


def grade(code: str, tests: list[dict], timeout_s: int = 6, memory_bytes: int | None = 4 << 30) -> tuple[list, dict]:
    """(one verdict per test reached, metadata of the first failure or the execution time)."""
    tests = normalize_tests(tests)
    if not tests:
        return [], {"error_message": "no tests"}
    job = json.dumps({"code": code, "tests": tests, "timeout": int(max(1, timeout_s)), "memory_bytes": memory_bytes})
    try:
        p = subprocess.run([sys.executable, "-I", "-c", _HARNESS], input=job, capture_output=True, text=True,
                           timeout=(timeout_s + 1) * len(tests) + 5)
    except subprocess.TimeoutExpired:
        return [-1] * len(tests), {"error_code": -1, "error_message": "global timeout"}
    mark = p.stdout.rfind("@@verdict@@")
    if mark < 0:                                                 # the child died (memory cap, hard exit) before its verdict
        return [-1] * len(tests), {"error_code": -1, "error_message": "grader exited without a verdict", "stderr": p.stderr[-500:]}
    out = json.loads(p.stdout[mark + len("@@verdict@@"):])
    return out["results"], out["metadata"]


def compute_score(response: str, tests, timeout_s: int = 6) -> tuple[str | None, float, dict]:
    """(extracted code, reward, metadata)."""
    code = extract_code(response)
    if code is None:
        return None, 0.0, {"error_message": "no code block"}
    tests = normalize_tests(tests)
    results, meta = grade(code, tests, timeout_s)
    ok = len(results) == len(tests) and len(tests) > 0 and all(r is True for r in results)
    return code, 1.0 if ok else 0.0, meta


class LCBEnv(BaseTextEnv):
    """Single turn. ``env_config``: ``timeout_s`` per test (default 6)."""

    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        spec = self.extras.get("reward_spec") or {}
        if "ground_truth" not in spec and "tests" not in spec:
            raise KeyError("the lcb environment needs reward_spec.ground_truth (the tests)")
        self.tests = normalize_tests(spec.get("ground_truth") or spec.get("tests"))
        self.timeout_s = int(self.env_config.get("timeout_s", 6))
        self.last: dict = {}

    def step(self, action: str):
        self.turns += 1
        code, reward, meta = compute_score(action, self.tests, self.timeout_s)
        self.last = {"has_code": code is not None, "error_code": meta.get("error_code", 0)}
        return {"observations": [], "reward": reward, "done": True, "metadata": dict(meta, has_code=code is not None)}

    def get_metrics(self) -> dict:
        return {"has_code": float(self.last.get("has_code", False)), "timed_out": float(self.last.get("error_code") == -3),
                "runtime_error": float(self.last.get("error_code") == -4)}


register("lcb", lambda c, e: LCBEnv(c, e))
