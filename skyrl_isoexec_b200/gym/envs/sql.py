"""Multi-turn text-to-SQL (reference: skyrl-gym/skyrl_gym/envs/sql/{env,utils}.py and tools/sql.py).

A turn of the model is reasoning in ``<think>...</think>`` followed by either a probe ``<sql>...</sql>``, which is run
against the task's SQLite database and answered with ``<observation>`` (the rows as a table, cut to 50 rows when the text
is long, plus a reminder of the turns left), or the commit ``<solution>...</solution>``. The episode ends on the commit or
when the turns are used up, and is scored ON THE WHOLE TRANSCRIPT:

* ``-1``  the transcript does not follow the format: exactly one ``<solution>`` block with no tool tags inside, at least
          one ``<think>`` block, and a ``<think>`` right after every observation;
* ``1``   the committed query returns the same SET of rows as the reference query (order and duplicates do not count);
* ``0``   otherwise (wrong rows, an error, a timeout).

Queries run in a worker thread inside a transaction that is always rolled back, so a probe cannot change the database for
the next one; a query that overruns its time limit is interrupted through ``sqlite3.Connection.interrupt``.

The database is ``{env_config.db_path}/{layout of extras.data}/{db_id}/{db_id}.sqlite`` with the layouts of the SynSQL,
Spider and BIRD releases, or, for self-contained data and tests, an in-memory database built from ``extras.schema_sql``.
"""

from __future__ import annotations

import os
import re
import sqlite3
import tempfile
import threading

from ..core import BaseTextEnv, register

LAYOUTS = {"synsql": "SynSQL-2.5M/databases", "spider": "spider/database", "bird": "bird/train/train_databases"}
INVALID_ACTION = "Your previous action is invalid. Follow the format of outputting thinking process and sql tool, and try again."


def run_query(db_file: str, sql: str, timeout_s: float = 5.0):
    """(status, payload): ("ok", frozenset of row tuples) | ("error", message) | ("timeout", the query)."""
    box: dict = {}
    done = threading.Event()

    def worker():
        conn = None
        try:
            conn = sqlite3.connect(db_file, check_same_thread=False)
            box["conn"] = conn
            conn.execute("BEGIN")
            box["out"] = ("ok", frozenset(conn.execute(sql).fetchall()))
        except Exception as e:  # noqa: BLE001 - whatever the query raises is the model's feedback
            box["out"] = ("error", f"Error executing SQL: {e}")
        finally:
            if conn is not None:
                for undo in (conn.rollback, conn.close):
                    try:
                        undo()
                    except sqlite3.Error:
                        pass
            done.set()

    threading.Thread(target=worker, daemon=True).start()
    if not done.wait(timeout_s):
        conn = box.get("conn")
        if conn is not None:
            try:
                conn.interrupt()
            except sqlite3.Error:
                pass
        done.wait(timeout_s)
        return "timeout", sql
    return box["out"]


def table_text(rows: frozenset, limit_chars: int = 9000, head: int = 50) -> str:
    rows = sorted(rows, key=repr)
    if not rows:
        return "Empty result"

    def render(rs):
        cols = list(zip(*[[str(c) for c in r] for r in rs]))
        widths = [max(len(c) for c in col) for col in cols]
        return "\n".join(" ".join(str(c).rjust(w) for c, w in zip(r, widths)) for r in rs)

    text = render(rows)
    if len(text) > limit_chars:
        text = f"Truncated to {head} lines since returned response too long: " + render(rows[:head])
    return text


def check_format(transcript: str) -> tuple[bool, str | None]:
    """(follows the protocol, the committed query)."""
    if transcript.count("<solution>") != 1:
        return False, None
    before, tail = transcript.split("<solution>", 1)
    if tail.count("</solution>") != 1:
        return False, None
    solution = tail.split("</solution>", 1)[0]
    if re.search(r"</?(think|sql|observation)\b", solution, re.I):
        return False, None
    if not re.search(r"<think>.*?</think>", transcript, re.S):
        return False, None
    for m in re.finditer(r"</observation>", before, re.I):
        if not before[m.end():].lstrip().lower().startswith("<think>"):
            return False, None
    return True, solution.strip()


def score_transcript(transcript: str, gold_sql: str, db_file: str, timeout_s: float = 30.0) -> float:
    ok, pred = check_format(transcript)
    if not ok:
        return -1.0
    a, b = run_query(db_file, pred, timeout_s), run_query(db_file, gold_sql, timeout_s)
    return 1.0 if a[0] == "ok" and b[0] == "ok" and a[1] == b[1] else 0.0


class SQLEnv(BaseTextEnv):
    def __init__(self, env_config=None, extras=None):
        super().__init__(env_config, extras)
        ex = self.extras
        if "reward_spec" not in ex or "ground_truth" not in ex["reward_spec"]:
            raise KeyError("the sql environment needs reward_spec.ground_truth (the reference query)")
        self.gold_sql = ex["reward_spec"]["ground_truth"]
        self.max_turns = int(ex.get("max_turns", 5))
        self.query_timeout_s = float(self.env_config.get("query_timeout_s", 5))
        self.score_timeout_s = float(self.env_config.get("score_timeout_s", 30))
        self._tmp = None
        if ex.get("schema_sql"):
            # self-contained task: the schema (and rows) travel with the sample; a private file, so that worker threads
            # can open it and a rolled-back probe leaves it as it was
            fd, self._tmp = tempfile.mkstemp(suffix=".sqlite")
            os.close(fd)
            conn = sqlite3.connect(self._tmp)
            conn.executescript(ex["schema_sql"])
            conn.commit()
            conn.close()
            self.db_file = self._tmp
        else:
            for need in ("db_id", "data"):
                if need not in ex:
                    raise KeyError(f"the sql environment needs extras.{need} (or extras.schema_sql)")
            if ex["data"] not in LAYOUTS:
                raise NotImplementedError(f"unknown text-to-SQL data set {ex['data']!r}; known: {sorted(LAYOUTS)}")
            root = os.path.join(self.env_config.get("db_path", "."), LAYOUTS[ex["data"]])
            self.db_file = os.path.join(root, ex["db_id"], ex["db_id"] + ".sqlite")
            if not os.path.exists(self.db_file):
                raise FileNotFoundError(f"database file not found at: {self.db_file}")
        self.chat_history: list[dict] = []
        self.queries = self.errors = 0

    def _observe(self, sql: str | None) -> str:
        left = self.max_turns - self.turns
        if sql is None:
            body = INVALID_ACTION
        else:
            self.queries += 1
            status, payload = run_query(self.db_file, sql, self.query_timeout_s)
            if status == "ok":
                body = table_text(payload)
            else:
                self.errors += 1
                body = f"SQL Timeout:\n{payload}" if status == "timeout" else payload
        return f"\n\n<observation>{body}\n<reminder>You have {left} turns left to complete the task.</reminder></observation>\n\n"

    def step(self, action: str):
        self.turns += 1
        self.chat_history.append({"role": "assistant", "content": action})
        done = self.turns >= self.max_turns or ("<solution>" in action and "</solution>" in action)
        if done:
            transcript = "".join(m["content"] for m in self.chat_history)
            reward = score_transcript(transcript, self.gold_sql, self.db_file, self.score_timeout_s)
            return {"observations": [], "reward": reward, "done": True, "metadata": {"format_ok": reward >= 0}}
        m = re.search(r"<sql>(.*?)</sql>", action, re.S)
        obs = {"role": "user", "content": self._observe(m.group(1) if m else None)}
        self.chat_history.append(obs)
        return {"observations": [obs], "reward": 0.0, "done": False,
                "metadata": {"tool_group": "sql", "tool_name": "sql", "tool_input": m.group(1) if m else None}}

    def close(self) -> None:
        if self._tmp and os.path.exists(self._tmp):
            os.remove(self._tmp)
            self._tmp = None

    def get_metrics(self) -> dict:
        return {"turns": self.turns, "queries": self.queries, "query_errors": self.errors}


register("sql", lambda c, e: SQLEnv(c, e))
