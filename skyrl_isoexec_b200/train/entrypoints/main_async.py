"""Asynchronous training entry points (reference: examples/train/async/main_async.py and R/train/entrypoints for the fully
asynchronous trainer):

    python -m skyrl_isoexec_b200.train.entrypoints.main_async --config run.yaml [--mode one_step_off | fully_async] [key=value ...]

``one_step_off`` (default): ``train/async_trainer.py``, generation of the next batch overlaps the update on the current one;
it needs ``generator.inference_engine.own_weights=true``. ``fully_async``: ``train/fully_async_trainer.py``, rollouts are
generated continuously by prompt group under a staleness bound (``--max-staleness-steps``, ``--generation-workers``).
"""

from __future__ import annotations

import argparse

from ..config import SkyRLTrainConfig
from .main_base import BasePPOExp


class AsyncPPOExp(BasePPOExp):
    def __init__(self, cfg, mode: str = "one_step_off", max_staleness_steps: int = 1, generation_workers: int = 4):
        super().__init__(cfg)
        self.mode, self.max_staleness_steps, self.generation_workers = mode, max_staleness_steps, generation_workers

    def get_trainer(self):
        kw = dict(ps=self.ps, device=self.device, dataset=self.get_train_dataset(), tokenizer=self.get_tokenizer(), tracker=self.get_tracker())
        if self.mode == "fully_async":
            from ..fully_async_trainer import AsyncConfig, FullyAsyncTrainer

            fa = self.cfg.trainer.fully_async
            acfg = AsyncConfig(max_staleness_steps=self.max_staleness_steps, num_parallel_generation_workers=self.generation_workers,
                               mini_batch_prompts=self.cfg.trainer.policy_mini_batch_size, simulate_training=fa.simulate_training,
                               simulate_training_step_seconds=fa.simulate_training_step_seconds,
                               simulate_weight_sync_seconds=fa.simulate_weight_sync_seconds)
            if fa.simulate_training:
                from ..fully_async_trainer import FullyAsyncTrainerSim

                return FullyAsyncTrainerSim(self.cfg, acfg, **kw)
            return FullyAsyncTrainer(self.cfg, acfg, **kw)
        from ..async_trainer import AsyncRayPPOTrainer

        return AsyncRayPPOTrainer(self.cfg, **kw)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="")
    ap.add_argument("--mode", default="", choices=["", "one_step_off", "fully_async"],
                    help="default: fully_async when trainer.fully_async.enabled, else one_step_off")
    ap.add_argument("--max-staleness-steps", type=int, default=None, help="default: trainer.fully_async.max_staleness_steps")
    ap.add_argument("--generation-workers", type=int, default=None, help="default: trainer.fully_async.num_parallel_generation_workers")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    cfg = SkyRLTrainConfig.from_file(a.config, a.overrides) if a.config else SkyRLTrainConfig.from_cli_overrides(a.overrides)
    fa = cfg.trainer.fully_async
    mode = a.mode or ("fully_async" if fa.enabled else "one_step_off")
    exp = AsyncPPOExp(cfg, mode, a.max_staleness_steps if a.max_staleness_steps is not None else fa.max_staleness_steps,
                      a.generation_workers if a.generation_workers is not None else fa.num_parallel_generation_workers)
    return exp.run()


if __name__ == "__main__":
    main()
