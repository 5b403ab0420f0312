"""Tool groups for multi-turn text environments (reference: skyrl-gym/skyrl_gym/tools/{core,sql,search,python}.py).

A tool group is an object with a ``name``, a ``tools()`` list and one method per tool; environments parse the
model's action for a tool call (``<tool>...</tool>`` style tags), run it through ``BaseTextEnv._execute_tool`` and
return the result as the next observation. Everything here runs offline: SQLite in memory, a local corpus for
search, a subprocess with a time limit for Python.
"""

from __future__ import annotations

import math
import re
import sqlite3
import subprocess
import sys
from collections import Counter


class SQLToolGroup:
    name = "sql"

    def __init__(self, schema_sql: str = "", db_path: str = ":memory:", max_rows: int = 50):
        self.conn = sqlite3.connect(db_path)
        self.max_rows = max_rows
        if schema_sql:
            self.conn.executescript(schema_sql)

    def tools(self):
        return ["sql"]

    def sql(self, query: str):
        try:
            cur = self.conn.execute(query)
            rows = cur.fetchmany(self.max_rows)
            return {"ok": True, "rows": rows, "columns": [d[0] for d in cur.description] if cur.description else []}
        except sqlite3.Error as e:
            return {"ok": False, "error": str(e)}


_WORD = re.compile(r"[a-z0-9]+")


class SearchToolGroup:
    """BM25 over a local list of documents (the reference calls a retrieval server)."""

    name = "search"

    def __init__(self, corpus: list[str], k1: float = 1.5, b: float = 0.75):
        self.docs = list(corpus)
        self.tok = [_WORD.findall(d.lower()) for d in self.docs]
        self.df = Counter(w for t in self.tok for w in set(t))
        self.avg = sum(len(t) for t in self.tok) / max(1, len(self.tok))
        self.k1, self.b = k1, b

    def tools(self):
        return ["search"]

    def search(self, query: str, topk: int = 3):
        q = _WORD.findall(query.lower())
        N = len(self.docs)
        scores = []
        for i, t in enumerate(self.tok):
            tf = Counter(t)
            s = 0.0
            for w in q:
                if w not in tf:
                    continue
                idf = math.log(1 + (N - self.df[w] + 0.5) / (self.df[w] + 0.5))
                s += idf * tf[w] * (self.k1 + 1) / (tf[w] + self.k1 * (1 - self.b + self.b * len(t) / max(1e-9, self.avg)))
            scores.append((s, -i))
        top = sorted(scores, reverse=True)[:topk]
        return [{"doc_id": -j, "score": s, "text": self.docs[-j]} for s, j in top if s > 0]


class PythonToolGroup:
    """Runs a snippet in a fresh interpreter with a time limit; returns stdout/stderr."""

    name = "python"

    def __init__(self, timeout_s: float = 5.0):
        self.timeout_s = timeout_s

    def tools(self):
        return ["python"]

    def python(self, code: str, stdin: str = ""):
        try:
            p = subprocess.run([sys.executable, "-I", "-c", code], input=stdin, capture_output=True, text=True, timeout=self.timeout_s)
            return {"ok": p.returncode == 0, "stdout": p.stdout[-4000:], "stderr": p.stderr[-2000:]}
        except subprocess.TimeoutExpired:
            return {"ok": False, "stdout": "", "stderr": f"timeout after {self.timeout_s}s"}
