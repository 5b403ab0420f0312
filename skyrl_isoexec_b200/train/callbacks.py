"""Trainer callbacks (reference: R/train/utils/callbacks.py:35-162, ``CallbackInput`` / ``TrainingControl`` /
``TrainingCallback`` / ``CallbackHandler``).

A callback overrides the events it cares about; every event gets the trainer, a snapshot of where the run is
(``CallbackInput``; fields that do not apply to the event are None) and the shared ``TrainingControl``. The trainer reads
the control flags once per step, right after ``on_step_end``, acts on them (an extra checkpoint, an extra evaluation) and
clears them, so a flag set from a later event of the same step is honoured one step later."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

EVENTS = ("on_train_start", "on_train_end", "on_epoch_start", "on_epoch_end", "on_step_start", "on_step_end",
          "on_eval_start", "on_eval_end", "on_save", "on_log")


@dataclass
class CallbackInput:
    global_step: int
    epoch: int
    total_steps: int
    steps_per_epoch: int
    batch: Any = None                   # step events: the prompt rows of the step
    metrics: dict | None = None         # on_step_end / on_eval_end
    logs: dict | None = None            # on_log: the dict about to be committed; callbacks may add fields in place
    ckpt_path: str | None = None        # on_save


@dataclass
class TrainingControl:
    should_save: bool = False
    should_evaluate: bool = False
    should_stop: bool = False           # ends the run after the current step (an early-stopping hook)

    def reset(self) -> None:
        self.should_save = self.should_evaluate = False


class TrainingCallback:
    """Base class: every event is a no-op."""


def _noop(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
    return None


for _e in EVENTS:
    setattr(TrainingCallback, _e, _noop)


class CallbackHandler(TrainingCallback):
    """Calls a list of callbacks in order; itself a callback, so handlers nest."""

    def __init__(self, callbacks=None):
        self.callbacks: list[TrainingCallback] = list(callbacks or [])

    def add(self, callback: TrainingCallback) -> None:
        self.callbacks.append(callback)

    def __bool__(self) -> bool:
        return bool(self.callbacks)


def _fan_out(name):
    def dispatch(self, trainer, callback_input: CallbackInput, control: TrainingControl) -> None:
        for cb in self.callbacks:
            getattr(cb, name)(trainer, callback_input, control)
    dispatch.__name__ = name
    return dispatch


for _e in EVENTS:
    setattr(CallbackHandler, _e, _fan_out(_e))
