"""A persistent in-process Python REPL for environments whose code blocks must call back into the rollout (reference:
skyrl-gym/skyrl_gym/envs/rlm/repl.py ``PersistentREPL``): variables live across ``execute`` calls, output is captured,
every call has a time limit, and the helper names the environment provides (``FINAL_VAR``, ``SHOW_VARS``, the language-model
query functions, task tools) are put back after every call, so that a block cannot redefine them for the next one.

Unlike ``gym/tools.py::PythonToolGroup`` (a fresh ``python -I`` per call) this runs in the trainer's process: it is for
code that needs callables of the host (a language-model callback, a child agent), and it narrows what the code can reach
instead of isolating it: builtins without ``open`` / ``exec`` / ``eval`` / ``compile`` / ``input`` / ``exit``, and an
``import`` that only lets a list of standard-library modules through.

Language-model helpers (present when ``lm_callback`` is given; ``lm_callback(list of prompts) -> list of answers``):

* ``llm_query(prompt)`` / ``llm_query_batched(prompts)``: one plain completion per prompt;
* ``rlm_query(prompt, context=None)`` / ``rlm_query_batched(prompts, context_list=None)``: a CHILD agent with a REPL of its
  own works on the sub-task (``subcall_fn(prompt, context=...) -> str``; without one they fall back to the plain queries);
  an answer that reads as a Python literal comes back as that object. Batched children run two at a time.

A failure of a helper is returned as an ``"Error: ..."`` string, not raised, so that the model sees it in its output.
"""

from __future__ import annotations

import ast
import builtins
import io
import signal
import threading
import traceback
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

ALLOWED_IMPORTS = ("math", "re", "json", "collections", "itertools", "functools", "heapq", "bisect", "statistics", "string",
                   "datetime", "random", "fractions", "decimal", "textwrap", "difflib", "operator", "copy", "typing", "dataclasses",
                   "enum", "unicodedata", "csv", "io")
_BLOCKED = ("open", "exec", "eval", "compile", "input", "exit", "quit", "breakpoint", "help", "__import__", "globals", "locals", "vars",
            "memoryview")


def _safe_import(name, globals=None, locals=None, fromlist=(), level=0):
    if level or name.split(".")[0] not in ALLOWED_IMPORTS:
        raise ImportError(f"import of {name!r} is not allowed in this REPL (allowed: {', '.join(ALLOWED_IMPORTS)})")
    return builtins.__import__(name, globals, locals, fromlist, level)


def safe_builtins() -> dict:
    out = {k: getattr(builtins, k) for k in dir(builtins) if k not in _BLOCKED}
    out["__import__"] = _safe_import
    return out


@dataclass
class REPLResult:
    stdout: str
    stderr: str
    ok: bool
    timed_out: bool = False


class _Timeout(Exception):
    pass


class PersistentREPL:
    def __init__(self, timeout_s: float = 15.0, tools: dict | None = None, lm_callback=None, subcall_fn=None):
        self.timeout_s, self.lm_callback, self.subcall_fn = timeout_s, lm_callback, subcall_fn
        self.tools = dict(tools or {})
        for name in self.tools:
            if not name.isidentifier() or name in ("FINAL_VAR", "SHOW_VARS", "context", "llm_query", "llm_query_batched", "rlm_query", "rlm_query_batched"):
                raise ValueError(f"tool name {name!r} is not an identifier or shadows a built-in helper")
        self.ns: dict = {}
        self.lm_calls = self.child_calls = 0
        self._scaffold: dict = {}
        self._install()

    def _install(self) -> None:
        s = {"__builtins__": safe_builtins(), "__name__": "__main__", "FINAL_VAR": self.final_var, "SHOW_VARS": self.show_vars}
        if self.lm_callback is not None:
            s.update(llm_query=self.llm_query, llm_query_batched=self.llm_query_batched, rlm_query=self.rlm_query,
                     rlm_query_batched=self.rlm_query_batched)
        s.update({k: v for k, v in self.tools.items() if callable(v)})
        self._scaffold = s
        self.ns.update(s)
        self.ns.update({k: v for k, v in self.tools.items() if not callable(v) and k not in self.ns})

    def set_context(self, payload, index: int = 0) -> None:
        self.ns["context" if index == 0 else f"context_{index}"] = payload

    # ------------------------------------------------------------------ helpers visible to the code
    def user_vars(self) -> dict:
        return {k: v for k, v in self.ns.items() if not k.startswith("_") and k not in self._scaffold and k not in self.tools}

    def show_vars(self) -> str:
        v = {k: type(x).__name__ for k, x in self.user_vars().items()}
        return f"Available variables: {v}" if v else "No variables created yet. Use ```repl``` blocks to create variables."

    def final_var(self, name) -> str:
        """The value of a variable as the final answer's text (an error text when there is no such variable)."""
        name = str(name).strip().strip("\"'")
        if name not in self.ns or name in self._scaffold:
            return f"Error: variable {name!r} not found. {self.show_vars()}"
        return str(self.ns[name])

    def llm_query(self, prompt: str, model: str | None = None) -> str:
        try:
            self.lm_calls += 1
            return self.lm_callback([prompt])[0]
        except Exception as e:  # noqa: BLE001 - shown to the model
            return f"Error: LM query failed - {e}"

    def llm_query_batched(self, prompts: list, model: str | None = None) -> list:
        try:
            self.lm_calls += len(prompts)
            return list(self.lm_callback(list(prompts)))
        except Exception as e:  # noqa: BLE001
            return [f"Error: LM query failed - {e}"] * len(prompts)

    @staticmethod
    def _literal(text):
        try:
            return ast.literal_eval(text)
        except (ValueError, SyntaxError):
            return text

    def rlm_query(self, prompt: str, model: str | None = None, context=None):
        if self.subcall_fn is None:
            return self.llm_query(prompt, model)
        try:
            self.child_calls += 1
            return self._literal(self.subcall_fn(prompt, context=context))
        except Exception as e:  # noqa: BLE001
            return f"Error: RLM query failed - {e}"

    def rlm_query_batched(self, prompts: list, model: str | None = None, context_list: list | None = None) -> list:
        if self.subcall_fn is None:
            return self.llm_query_batched(prompts, model)
        ctxs = list(context_list) if context_list is not None else [None] * len(prompts)
        if len(ctxs) != len(prompts):
            return [f"Error: RLM query failed - {len(ctxs)} contexts for {len(prompts)} prompts"] * len(prompts)
        with ThreadPoolExecutor(max_workers=max(1, min(2, len(prompts)))) as pool:
            return list(pool.map(lambda pc: self.rlm_query(pc[0], model, pc[1]), zip(prompts, ctxs)))

    # ------------------------------------------------------------------ execution
    def execute(self, code: str) -> REPLResult:
        out, err = io.StringIO(), io.StringIO()
        timed_out = False
        # output goes through a print of the block's own (the process-wide stdout is never redirected: a block that is
        # abandoned at its time limit must not keep it)
        self.ns["__builtins__"] = dict(self._scaffold["__builtins__"], print=lambda *a, **kw: builtins.print(*a, **dict(kw, file=out)))

        def body():
            try:
                exec(builtins.compile(code, "<repl>", "exec"), self.ns)       # noqa: S102 - the point of a REPL
            except _Timeout:
                raise
            except BaseException:  # noqa: BLE001 - the traceback is the model's feedback
                import sys

                et, ev, tb = sys.exc_info()
                frames = [f for f in traceback.extract_tb(tb) if f.filename == "<repl>"]       # the block's own frames only
                err.write("Traceback (most recent call last):\n" + "".join(traceback.format_list(frames))
                          + "".join(traceback.format_exception_only(et, ev)).rstrip())

        if threading.current_thread() is threading.main_thread() and hasattr(signal, "SIGALRM"):
            def on_alarm(*_):
                raise _Timeout()

            old = signal.signal(signal.SIGALRM, on_alarm)
            signal.setitimer(signal.ITIMER_REAL, self.timeout_s)
            try:
                body()
            except _Timeout:
                timed_out = True
            finally:
                signal.setitimer(signal.ITIMER_REAL, 0)
                signal.signal(signal.SIGALRM, old)
        else:
            # off the main thread no signal can interrupt the code: it runs in a helper thread that is abandoned at the limit
            t = threading.Thread(target=body, daemon=True)
            t.start()
            t.join(self.timeout_s)
            timed_out = t.is_alive()
        if timed_out:
            err.write(f"TimeoutError: the block ran longer than {self.timeout_s:g} s and was stopped")
        self.ns.update(self._scaffold)                    # a block cannot keep a helper redefined
        return REPLResult(out.getvalue(), err.getvalue(), ok=not err.getvalue(), timed_out=timed_out)
