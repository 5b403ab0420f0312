"""Profiling helpers (reference: B/utils/profiler.py:8-99): a ``torch.profiler`` wrapper driven by a
small config (enable / ranks / step window / output dir), a CUDA-event timer, NVTX ranges and the
memory-snapshot hook used after forward_backward / optim_step."""

from __future__ import annotations

import contextlib
import os
from dataclasses import dataclass, field

import torch


@dataclass
class ProfilerConfig:
    enable: bool = False
    ranks: list = field(default_factory=lambda: [0])
    save_path: str = "profiles_out"
    start_step: int = 2
    end_step: int = 3
    with_stack: bool = False


class Profiler:
    def __init__(self, cfg: ProfilerConfig, rank: int = 0):
        self.cfg, self.rank, self.prof, self.step_no = cfg, rank, None, 0
        self.active = cfg.enable and rank in cfg.ranks

    def step(self) -> None:
        """Call once per training step; opens / closes the torch profiler at the configured window."""
        if not self.active:
            return
        if self.step_no == self.cfg.start_step and self.prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.prof = torch.profiler.profile(activities=acts, with_stack=self.cfg.with_stack)
            self.prof.__enter__()
        elif self.step_no == self.cfg.end_step and self.prof is not None:
            self.prof.__exit__(None, None, None)
            os.makedirs(self.cfg.save_path, exist_ok=True)
            self.prof.export_chrome_trace(os.path.join(self.cfg.save_path, f"trace_rank{self.rank}.json"))
            self.prof = None
        self.step_no += 1


class CudaTimer:
    """``with CudaTimer() as t: ...`` then ``t.ms`` (device time between two events on the current stream)."""

    def __enter__(self):
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.e0.record()
        return self

    def __exit__(self, *exc):
        self.e1.record()
        self.e1.synchronize()
        self.ms = self.e0.elapsed_time(self.e1)
        return False


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()


def start_memory_history(max_entries: int = 100000) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=max_entries)


def save_memory_snapshot(directory: str, tag: str, rank: int = 0) -> str | None:
    """Dump the allocator history (``torch.cuda.memory._dump_snapshot``) as ``{dir}/mem_{tag}_r{rank}.pickle``."""
    if not torch.cuda.is_available():
        return None
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, f"mem_{tag}_r{rank}.pickle")
    torch.cuda.memory._dump_snapshot(path)
    return path
