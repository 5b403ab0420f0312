"""Worker dispatch: one object through which a controller drives the policy / critic / reference workers of its
process (reference: B/workers/worker_dispatch.py:138-186,199,286,351,394,427,562 ``WorkerDispatch``; there the verbs
fan out to Ray actors, here the workers are local and ranks run the same program).

Verbs: ``forward``, ``forward_backward``, ``optim_step``, ``stage_data`` + ``forward_backward_from_staged`` (hand a
batch over once, then train on row ranges of it), ``get_lcm_dp_size`` (what a batch must be padded to so that every
model's data-parallel group gets whole rows), ``save_checkpoint`` / ``load_checkpoint``, ``save_weights_for_sampler``,
and the residency state machine of a colocated job: at most ONE model's optimizer state is on the GPU at a time;
``ensure_resident(name)`` brings that model's state back and parks the others in pinned host memory.
"""

from __future__ import annotations

import math
import uuid

from .batch import TrainingInputBatch, pad_training_input_batch


class WorkerDispatch:
    def __init__(self, workers: dict, colocate_all: bool = True, sync_fn=None):
        """``workers``: name -> worker (``policy`` / ``critic`` / ``ref``); workers without an optimizer (ref) are
        never offloaded. ``sync_fn``: what publishes the policy weights to the sampler."""
        self.workers = {k: v for k, v in workers.items() if v is not None}
        self.colocate_all = colocate_all
        self.sync_fn = sync_fn
        self.staged: dict[str, TrainingInputBatch] = {}
        self.residency = {k: "gpu" for k in self.workers}
        self.transitions: list[tuple[str, str]] = []

    # ---- sizes
    def dp_size(self, name: str) -> int:
        return int(getattr(self.workers[name].ps, "dp", 1))

    def get_lcm_dp_size(self) -> int:
        out = 1
        for name in self.workers:
            out = math.lcm(out, self.dp_size(name))
        return out

    def pad_batch(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        return pad_training_input_batch(batch, self.get_lcm_dp_size())

    # ---- residency (colocated jobs)
    def _has_optimizer(self, name: str) -> bool:
        return getattr(self.workers[name], "opt", None) is not None

    def offload(self, name: str) -> None:
        if self.residency[name] == "gpu" and self._has_optimizer(name):
            self.workers[name].opt.offload()
            self.residency[name] = "cpu"
            self.transitions.append((name, "cpu"))

    def backload(self, name: str) -> None:
        if self.residency[name] == "cpu":
            w = self.workers[name]
            w.opt.backload(w.device)
            self.residency[name] = "gpu"
            self.transitions.append((name, "gpu"))

    def ensure_resident(self, name: str) -> None:
        """Before a training verb of ``name``: its optimizer state on the GPU, everybody else's parked (colocated)."""
        if self.colocate_all:
            for other in self.workers:
                if other != name:
                    self.offload(other)
        self.backload(name)

    def offload_all(self) -> None:
        """Before rollout in a colocated job: every optimizer state leaves the GPU."""
        for name in self.workers:
            self.offload(name)

    # ---- compute verbs
    def forward(self, name: str, batch: TrainingInputBatch):
        return self.workers[name].forward(batch)

    def forward_backward(self, name: str, batch: TrainingInputBatch) -> dict:
        self.ensure_resident(name)
        return self.workers[name].forward_backward(batch)

    def optim_step(self, name: str) -> float:
        self.ensure_resident(name)
        return self.workers[name].optim_step()

    def stage_data(self, batch: TrainingInputBatch) -> str:
        key = "staged-" + uuid.uuid4().hex[:8]
        self.staged[key] = batch
        return key

    def forward_backward_from_staged(self, name: str, key: str, lo: int, hi: int) -> dict:
        if key not in self.staged:
            raise KeyError(f"no staged batch {key!r}")
        return self.forward_backward(name, self.staged[key].slice(lo, hi))

    def drop_staged(self, key: str) -> None:
        self.staged.pop(key, None)

    # ---- state verbs
    def save_checkpoint(self, ckpt_path: str, step: int, data_state: dict, trainer_state: dict, max_to_keep: int = -1) -> str:
        from . import checkpoint as ckpt

        w = self.workers["policy"]
        return ckpt.save_checkpoint(ckpt_path, step, w, data_state, trainer_state, w.ps, max_to_keep=max_to_keep)

    def load_checkpoint(self, path: str):
        from . import checkpoint as ckpt

        w = self.workers["policy"]
        self.backload("policy")
        return ckpt.load_checkpoint(path, w, w.ps)

    def save_weights_for_sampler(self) -> None:
        if self.sync_fn is None:
            raise RuntimeError("no weight-sync function was given to the dispatch")
        self.sync_fn()
