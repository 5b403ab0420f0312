"""Callbacks: stop a run once the mean reward has not improved for a few steps, checkpoint on every new best, and add a
field of our own to what the tracker logs.

    python examples/callbacks_early_stop.py
"""

from skyrl_isoexec_b200.train.callbacks import TrainingCallback
from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
from skyrl_isoexec_b200.train.trainer import RayPPOTrainer


class BestRewardCheckpoint(TrainingCallback):
    def __init__(self, patience: int = 3, key: str = "reward/avg_raw_reward"):
        self.patience, self.key, self.best, self.since = patience, key, float("-inf"), 0

    def on_step_end(self, trainer, callback_input, control):
        r = float(callback_input.metrics.get(self.key, float("-inf")))
        if r > self.best:
            self.best, self.since = r, 0
            control.should_save = True           # read by the trainer right after this event
        else:
            self.since += 1
            control.should_stop = self.since >= self.patience

    def on_log(self, trainer, callback_input, control):
        callback_input.logs["early_stop/best_reward"] = self.best
        callback_input.logs["early_stop/steps_since_best"] = self.since


def main(ckpt_path: str = "ckpts/callbacks_example", num_steps: int = 20) -> RayPPOTrainer:
    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model=tiny-qwen3", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "generator.n_samples_per_prompt=2", "generator.sampling_params.max_generate_length=8",
        "generator.sampling_params.ignore_eos=true", "data.synthetic_prompt_len=8", "data.synthetic_prompts=64",
        "trainer.max_prompt_length=8", "generator.inference_engine.num_kv_pages=32", f"trainer.num_steps={num_steps}",
        f"trainer.ckpt_path={ckpt_path}", "trainer.ckpt_interval=0", "trainer.logger=console"])
    trainer = RayPPOTrainer(cfg, callbacks=[BestRewardCheckpoint()])
    trainer.train()
    return trainer


if __name__ == "__main__":
    main()
