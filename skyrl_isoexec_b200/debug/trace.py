"""Debug-mode capture: per-region output digests written as JSONL, one file per process
(reference: ISO/debug/trace.py:100-357, install.py:271-349).

Enabled by ``SKYRL_ISOEXEC_DEBUG_TRACE=<directory>`` (which also demotes contract refusals to
warnings, core/ledger.py). The model calls ``record(region, tensor)`` at its region boundaries
(the "doors"); when no tracer is active the call is a single attribute test. Each record carries
the row keys of the forward ((sequence uid, position) per row) so the offline comparator can line
up the trainer's packed rows with the engine's batched rows.
"""

from __future__ import annotations

import json
import os
import time

from . import thash

ENV = "SKYRL_ISOEXEC_DEBUG_TRACE"
FORMAT = "isoexec-trace-1"
_active: "Tracer | None" = None


class Tracer:
    def __init__(self, directory: str, side: str, rank: int = 0, max_rows: int = 4096):
        os.makedirs(directory, exist_ok=True)
        self.path = os.path.join(directory, f"trace.{side}.r{rank}.jsonl")
        self.f = open(self.path, "w")
        self.side, self.rank, self.max_rows = side, rank, max_rows
        self.seq = 0
        self.row_keys: list | None = None
        self.site = "unknown"
        self.step = 0
        self._write({"format": FORMAT, "side": side, "rank": rank, "ladder": list(thash.LADDER), "t": time.time()})

    def _write(self, obj):
        self.f.write(json.dumps(obj, separators=(",", ":")) + "\n")
        self.f.flush()

    def begin_forward(self, site: str, row_keys: list | None, step: int = 0):
        self.site, self.row_keys, self.step = site, row_keys, step

    def record(self, region: str, x, rows_are_tokens: bool = True):
        import torch

        with torch.no_grad():
            x2 = x.reshape(x.shape[0], -1) if x.dim() > 1 else x.reshape(-1, 1)
            rec = {"i": self.seq, "region": region, "site": self.site, "step": self.step, "shape": list(x.shape),
                   "dtype": str(x.dtype).replace("torch.", ""), "digest": thash.ladder(x2)}
            if rows_are_tokens and self.row_keys is not None and len(self.row_keys) == x2.shape[0] and x2.shape[0] <= self.max_rows:
                rec["row_keys"] = [list(k) for k in self.row_keys]
                rec["rows"] = thash.row_ladder(x2)
            self.seq += 1
            self._write(rec)

    def close(self):
        self.f.close()


def install(side: str, rank: int = 0, directory: str | None = None) -> Tracer | None:
    """Activate tracing for this process if the environment (or ``directory``) asks for it."""
    global _active
    d = directory or os.environ.get(ENV)
    if not d:
        return None
    _active = Tracer(d, side, rank)
    return _active


def uninstall():
    global _active
    if _active is not None:
        _active.close()
    _active = None


def active() -> Tracer | None:
    return _active


def record(region: str, x) -> None:
    if _active is not None:
        _active.record(region, x)
