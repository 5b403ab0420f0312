"""Executable ordering asserts for the weight-sync lifecycle of a colocated run (reference:
ISO/lifecycle/ordering.py:60-151). Each check is fail-soft: it returns a list of problem strings
(and logs them) rather than raising, because a mis-ordered lifecycle is a deployment fault to be
reported by the ledger, not a numerics fault."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class LifecycleLog:
    """Events appended by the trainer/engine as they happen: (name, detail)."""

    events: list[tuple[str, dict]] = field(default_factory=list)

    def add(self, name: str, **detail) -> None:
        self.events.append((name, detail))

    def names(self) -> list[str]:
        return [n for n, _ in self.events]


def _index(names, what, start=0):
    try:
        return names.index(what, start)
    except ValueError:
        return -1


def check_wake_before_sync(log: LifecycleLog) -> list[str]:
    """The engine's weights must be resident (woken with the ``weights`` tag or never slept) before a sync writes them."""
    out, asleep = [], False
    for n, d in log.events:
        if n == "engine_sleep":
            asleep = True
        elif n == "engine_wake" and "weights" in d.get("tags", ["weights", "kv_cache"]):
            asleep = False
        elif n == "weight_sync" and asleep:
            out.append("weight_sync while the engine's weights were asleep")
    return out


def check_sleep_tag_scoping(log: LifecycleLog) -> list[str]:
    """A sleep that drops weights must be followed by a sync before the next generate."""
    out, need_sync = [], False
    for n, d in log.events:
        if n == "engine_sleep" and d.get("level", 1) >= 2:
            need_sync = True
        elif n == "weight_sync":
            need_sync = False
        elif n == "generate" and need_sync:
            out.append("generate after a weight-dropping sleep without a weight sync in between")
    return out


def check_transfers_drained(log: LifecycleLog) -> list[str]:
    """Every ``sync_begin`` has its ``sync_end`` before the next generate (no transfer left in flight)."""
    out, open_ = [], 0
    for n, _ in log.events:
        if n == "sync_begin":
            open_ += 1
        elif n == "sync_end":
            open_ -= 1
        elif n == "generate" and open_ > 0:
            out.append("generate started while a weight transfer was still in flight")
    return out


def check_state_invalidated_after_sync(log: LifecycleLog) -> list[str]:
    """After every weight sync the engine's caches (prefix cache, recurrent state) are flushed before it generates."""
    out, dirty = [], False
    for n, _ in log.events:
        if n == "weight_sync":
            dirty = True
        elif n == "state_invalidated":
            dirty = False
        elif n == "generate" and dirty:
            out.append("generate with engine state that predates the last weight sync")
    return out


def check_handshake_before_first_sync(log: LifecycleLog) -> list[str]:
    names = log.names()
    s = _index(names, "weight_sync")
    h = _index(names, "handshake_ok")
    return ["first weight sync happened before the contract handshake"] if s >= 0 and (h < 0 or h > s) else []


ALL_CHECKS = (check_wake_before_sync, check_sleep_tag_scoping, check_transfers_drained, check_state_invalidated_after_sync,
              check_handshake_before_first_sync)


def run_all(log: LifecycleLog) -> list[str]:
    problems = []
    for chk in ALL_CHECKS:
        problems += chk(log)
    return problems
