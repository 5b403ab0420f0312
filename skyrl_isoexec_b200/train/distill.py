"""On-policy distillation (reference: examples/train/on_policy_distillation/main_on_policy_distill.py): the student samples,
a frozen teacher scores the student's own tokens, and the per-token reward is the negative reverse-KL sample
``-(log p_student - log p_teacher)``; with the ``no_op`` estimator those rewards are the advantages as they are.

    python -m skyrl_isoexec_b200.train.distill trainer.policy.model=tiny-qwen3 trainer.ref.model=tiny-qwen3 trainer.ref.seed=7 ...

The teacher is ``trainer.ref`` (a preset with the policy's vocabulary; ``trainer.ref.hf_path`` loads its weights). The
environment's reward is ignored."""

from __future__ import annotations

import sys

from .config import SkyRLTrainConfig
from .entrypoints.main_base import BasePPOExp
from .trainer import RayPPOTrainer


class OnPolicyDistillationTrainer(RayPPOTrainer):
    def __init__(self, cfg: SkyRLTrainConfig, **kw):
        a = cfg.trainer.algorithm
        a.use_kl_in_reward = True           # builds the frozen reference model and routes through the seam below
        a.use_kl_loss = False
        if a.advantage_estimator == "grpo":  # the default estimator would collapse the dense signal to one scalar per sample
            a.advantage_estimator = "no_op"
        super().__init__(cfg, **kw)

    def apply_reward_kl_penalty(self, batch):
        mask = batch["loss_mask"]
        gap = (batch["action_log_probs"] - batch["base_action_log_probs"]) * mask
        batch["rewards"] = -gap
        self.all_metrics["distill/reverse_kl"] = float(gap.sum() / mask.sum().clamp(min=1))
        return batch


class OnPolicyDistillationExp(BasePPOExp):
    def get_trainer(self) -> RayPPOTrainer:
        return OnPolicyDistillationTrainer(self.cfg, ps=self.ps, device=self.device, dataset=self.get_train_dataset(),
                                           tokenizer=self.get_tokenizer(), tracker=self.get_tracker())


def main(argv=None) -> None:
    OnPolicyDistillationExp(SkyRLTrainConfig.from_cli_overrides(list(sys.argv[1:] if argv is None else argv))).run()


if __name__ == "__main__":
    main()
