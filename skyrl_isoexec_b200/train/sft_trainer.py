"""Supervised fine-tuning on (prompt, response) pairs (reference: R/train/sft_trainer.py, R/train/main_sft.py).

Runs through the same policy worker as RL: sequences are packed without padding, the loss is the
negative log-likelihood of the response tokens (``policy_loss_type=cross_entropy``), micro-batches
are cut by a token budget, and checkpoints use the same directory layout.
"""

from __future__ import annotations

import random
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..models.config import get_config
from ..models.decoder import DecoderLM
from ..parallel.state import ParallelState
from ..utils.tracking import Timer, Tracking
from . import algorithms as alg
from . import checkpoint as ckpt
from .batch import TrainingInputBatch, build_sequences
from .policy_worker import OptimizerConfig, PolicyWorker, WorkerConfig


@dataclass
class SFTConfig:
    model: str = "tiny-qwen3"
    model_overrides: dict = field(default_factory=dict)
    batch_size: int = 32                  # sequences per optimizer step (global)
    max_tokens_per_microbatch: int = 8192
    epochs: int = 1
    num_steps: int = -1
    max_seq_len: int = 4096
    loss_reduction: str = "token_mean"    # token_mean | sequence_mean
    optimizer: OptimizerConfig = field(default_factory=lambda: OptimizerConfig(lr=1e-5))
    ckpt_path: str = ""
    ckpt_interval: int = 0
    resume_mode: str = "latest"
    seed: int = 0
    logger: str = "console"
    project_name: str = "skyrl_isoexec_b200_sft"
    run_name: str = "sft"


class SFTTrainer:
    def __init__(self, cfg: SFTConfig, examples: list[dict], ps: ParallelState | None = None, device: str | None = None):
        """``examples``: dicts with ``prompt_ids`` and ``response_ids`` (token lists)."""
        self.cfg = cfg
        self.ps = ps or ParallelState.single()
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        mcfg = get_config(cfg.model, **cfg.model_overrides)
        self.model = DecoderLM(mcfg, self.ps, self.device, seed=cfg.seed)
        algo = alg.AlgorithmConfig(policy_loss_type="cross_entropy", loss_reduction=cfg.loss_reduction)
        self.worker = PolicyWorker(self.model, WorkerConfig(max_tokens_per_microbatch=cfg.max_tokens_per_microbatch,
                                                            optimizer=cfg.optimizer), algo)
        self.examples = [e for e in examples if len(e["prompt_ids"]) + len(e["response_ids"]) <= cfg.max_seq_len]
        self.global_step = 0
        self.tracker = Tracking(cfg.project_name, cfg.run_name, cfg.logger) if self.rank == 0 else None
        self.cursor, self.epoch = 0, 0

    def _order(self):
        idx = list(range(len(self.examples)))
        random.Random(self.cfg.seed + self.epoch).shuffle(idx)
        return idx

    def _global_sum(self, x: float) -> float:
        if self.ps.dp > 1:
            t = torch.tensor([x], dtype=torch.float64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, group=self.ps.dp_group)
            return float(t.item())
        return x

    def train_step(self, rows: list[dict]) -> dict:
        timings: dict = {}
        with Timer("step", timings):
            seq, att, rmask = build_sequences([r["prompt_ids"] for r in rows], [r["response_ids"] for r in rows])
            batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone()})
            # cross_entropy sums -logp over masked tokens; the mean comes from scaling afterwards via the advantages slot
            ntok = self._global_sum(float(rmask.sum()))
            batch["advantages"] = torch.zeros_like(rmask)
            m = self.worker.forward_backward(batch)
            scale = 1.0 / max(1.0, ntok) if self.cfg.loss_reduction == "token_mean" else 1.0 / max(1.0, self._global_sum(len(rows)))
            self.worker.opt.main_grad.mul_(scale)
            gn = self.worker.optim_step()
        self.global_step += 1
        out = {"sft/loss": self._global_sum(m["policy_loss"]) * scale, "sft/grad_norm": gn, "sft/tokens": ntok,
               "timing/step": timings["step"]}
        if self.tracker is not None:
            self.tracker.log(out, self.global_step)
        return out

    def train(self) -> None:
        c = self.cfg
        per_rank = max(1, c.batch_size // max(1, self.ps.dp))
        if c.ckpt_path and c.resume_mode != "none":
            path = ckpt.resolve_resume_path(c.ckpt_path, c.resume_mode)
            if path is not None:
                data_state, st = ckpt.load_checkpoint(path, self.worker, self.ps)
                self.global_step, self.cursor, self.epoch = st["global_step"], data_state["cursor"], data_state["epoch"]
        while self.epoch < c.epochs:
            order = self._order()
            shard = order[self.ps.dp_rank::max(1, self.ps.dp)]
            while self.cursor + per_rank <= len(shard):
                rows = [self.examples[i] for i in shard[self.cursor:self.cursor + per_rank]]
                self.cursor += per_rank
                self.train_step(rows)
                if c.ckpt_path and c.ckpt_interval > 0 and self.global_step % c.ckpt_interval == 0:
                    ckpt.save_checkpoint(c.ckpt_path, self.global_step, self.worker, {"cursor": self.cursor, "epoch": self.epoch},
                                         {"global_step": self.global_step}, self.ps)
                if 0 < c.num_steps <= self.global_step:
                    return
            self.cursor, self.epoch = 0, self.epoch + 1
