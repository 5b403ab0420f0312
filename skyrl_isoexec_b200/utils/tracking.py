"""Step timers and experiment tracking (reference: R/train/utils/utils.py:33 ``Timer``;
R/train/utils/tracking.py:33-113 ``Tracking`` with wandb / mlflow / swanlab / tensorboard / console
backends). Backends that need a package which is not installed raise at construction, not at
the first log call."""

from __future__ import annotations

import json
import os
import time
import traceback


class Timer:
    """``with Timer("generate", timings):`` adds the elapsed seconds under ``timings["generate"]``."""

    def __init__(self, name: str, sink: dict | None = None, cuda_sync: bool = False):
        self.name, self.sink, self.cuda_sync = name, sink, cuda_sync
        self.elapsed = 0.0

    nvtx = False        # process-wide switch: every timed phase is also an NVTX range

    def __enter__(self):
        if self.cuda_sync:
            import torch

            if torch.cuda.is_available():
                torch.cuda.synchronize()
        if Timer.nvtx:
            import torch

            if torch.cuda.is_available():
                torch.cuda.nvtx.range_push(self.name)
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda_sync:
            import torch

            if torch.cuda.is_available():
                torch.cuda.synchronize()
        self.elapsed = time.perf_counter() - self.t0
        if Timer.nvtx:
            import torch

            if torch.cuda.is_available():
                torch.cuda.nvtx.range_pop()
        if self.sink is not None:
            self.sink[self.name] = self.sink.get(self.name, 0.0) + self.elapsed
        return False


_ANSI = {"green": "\033[32m", "yellow": "\033[33m", "cyan": "\033[36m"}


def log_example(prompt, response, reward=None, stream=None, color: bool | None = None) -> str:
    """Print one rollout (reference: R/train/utils/logging_utils.py:35-84): the prompt in cyan, the response in green when
    its total reward is positive and yellow otherwise, line by line so that a pager or a log collector that cuts at line
    ends keeps the colours. ``reward`` may be a number or per-token rewards (summed). Returns the text that was written."""
    import sys

    stream = stream or sys.stdout
    if color is None:
        color = bool(getattr(stream, "isatty", lambda: False)())
    total = None if reward is None else float(sum(reward)) if isinstance(reward, (list, tuple)) else float(reward)

    def block(text, name):
        lines = str(text).splitlines() or [""]
        return "\n".join(f"{_ANSI[name]}{ln}\033[0m" if color else ln for ln in lines)

    text = (f"Example:\n  Input: {block(prompt, 'cyan')}\n  Output (Total Reward: {'N/A' if total is None else format(total, '.4f')}):\n"
            f"{block(response, 'green' if total is not None and total > 0 else 'yellow')}\n")
    stream.write(text)
    return text


class ConsoleLogger:
    def log(self, data: dict, step: int):
        keys = sorted(data)
        parts = [f"{k}={data[k]:.6g}" if isinstance(data[k], float) else f"{k}={data[k]}" for k in keys]
        print(f"[step {step}] " + " ".join(parts), flush=True)

    def finish(self):
        pass


class JsonlLogger:
    def __init__(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
        self.f = open(path, "a")

    def log(self, data: dict, step: int):
        self.f.write(json.dumps({"step": step, **{k: (float(v) if hasattr(v, "__float__") else v) for k, v in data.items()}}) + "\n")
        self.f.flush()

    def finish(self):
        self.f.close()


class _TensorboardAdapter:
    def __init__(self, logdir: str):
        from torch.utils.tensorboard import SummaryWriter  # raises if tensorboard is missing

        self.w = SummaryWriter(logdir)

    def log(self, data: dict, step: int):
        for k, v in data.items():
            if isinstance(v, (int, float)):
                self.w.add_scalar(k, v, step)

    def finish(self):
        self.w.close()


class _WandbAdapter:
    def __init__(self, project, name, config):
        import wandb  # raises if wandb is missing

        self.wandb = wandb
        wandb.init(project=project, name=name, config=config)

    def log(self, data, step):
        self.wandb.log(data, step=step)

    def finish(self):
        self.wandb.finish()


class _MlflowAdapter:
    def __init__(self, project, name, config):
        import mlflow  # raises if mlflow is missing

        self.mlflow = mlflow
        mlflow.set_experiment(project)
        mlflow.start_run(run_name=name)
        mlflow.log_params({k: str(v)[:250] for k, v in (config or {}).items()})

    def log(self, data, step):
        self.mlflow.log_metrics({k: float(v) for k, v in data.items() if isinstance(v, (int, float))}, step=step)

    def finish(self):
        self.mlflow.end_run()


class _SwanlabAdapter:
    def __init__(self, project, name, config):
        import swanlab  # raises if swanlab is missing

        self.swanlab = swanlab
        swanlab.init(project=project, experiment_name=name, config=config)

    def log(self, data, step):
        self.swanlab.log({k: v for k, v in data.items() if isinstance(v, (int, float))}, step=step)

    def finish(self):
        self.swanlab.finish()


class Tracking:
    SUPPORTED = ("console", "jsonl", "tensorboard", "wandb", "mlflow", "swanlab")

    def __init__(self, project_name: str, experiment_name: str, backends="console", config: dict | None = None,
                 log_dir: str = "runs"):
        if isinstance(backends, str):
            backends = [b for b in backends.replace("[", "").replace("]", "").split(",") if b.strip()]
        self.loggers = {}
        for b in backends:
            b = b.strip().strip("'\"")
            if b not in self.SUPPORTED:
                raise ValueError(f"unsupported logger {b!r}; supported: {self.SUPPORTED}")
            if b == "console":
                self.loggers[b] = ConsoleLogger()
            elif b == "jsonl":
                self.loggers[b] = JsonlLogger(os.path.join(log_dir, project_name, experiment_name + ".jsonl"))
            elif b == "tensorboard":
                self.loggers[b] = _TensorboardAdapter(os.path.join(log_dir, project_name, experiment_name))
            elif b == "wandb":
                self.loggers[b] = _WandbAdapter(project_name, experiment_name, config)
            elif b == "mlflow":
                self.loggers[b] = _MlflowAdapter(project_name, experiment_name, config)
            elif b == "swanlab":
                self.loggers[b] = _SwanlabAdapter(project_name, experiment_name, config)

    def log(self, data: dict, step: int, commit: bool = True):
        for lg in self.loggers.values():
            lg.log(data, step)

    def log_exception(self, exc: BaseException, step: int = 0):
        """Push the traceback of a crash to every backend before the process dies."""
        tb = "".join(traceback.format_exception(type(exc), exc, exc.__traceback__))
        for lg in self.loggers.values():
            try:
                lg.log({"crash/traceback": tb[-4000:], "crash/type": type(exc).__name__}, step)
            except Exception:  # noqa: BLE001
                pass

    def finish(self):
        for lg in self.loggers.values():
            lg.finish()
