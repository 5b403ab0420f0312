"""Supervised fine-tuning on (prompt, response) pairs (reference: R/train/sft_trainer.py, R/train/main_sft.py).

Runs through the same policy worker as RL: sequences are packed without padding, the loss is the
negative log-likelihood of the response tokens (``policy_loss_type=cross_entropy``), micro-batches
are cut by a token budget, and checkpoints use the same directory layout.

Records may be token rows, alpaca-style or chat messages with tool calls (``train/sft_data.py``; ``train_on`` selects the
assistant turns that carry loss, tokenized rows can be cached on disk). Beyond the step loop: an evaluation pass over a
held-out set every ``eval_interval`` steps (mean negative log-likelihood per loss token, no gradient), the trainer
callbacks of the RL controller (``train/callbacks.py``), a Hugging Face export at the end or every ``hf_save_interval``
steps, length statistics of the tokenized set, and ``dummy_steps`` for timing runs on synthetic rows.
"""

from __future__ import annotations

import json
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
    train_on: str = "last"                # chat records: loss on the "last" assistant turn or on "all" of them
    tokenize_cache_dir: str = ""
    eval_interval: int = 0                # every N steps (and at the end) when an eval set was given
    eval_batch_size: int = 32
    export_path: str = ""
    hf_save_interval: int = 0             # every N steps; 0 with export_path set: once, at the end
    lora_rank: int = 0                    # > 0: train low-rank adapters (train/lora.py), the base weights stay as they are
    lora_alpha: float = 16.0
    hf_path: str = ""                     # initial weights: a Hugging Face style directory (models/hf_export.py); default: random init
    dummy_steps: int = 0                  # > 0: ignore the data, train on synthetic rows of max_seq_len tokens (timing runs)

    @classmethod
    def from_file(cls, path: str, overrides: list[str] | None = None) -> "SFTConfig":
        """A YAML or JSON file of these fields (nested under ``optimizer:`` for the optimizer's), then ``key=value``
        overrides with dotted keys (``optimizer.lr=3e-6``), the same forms the RL trainer's config takes."""
        from .config import _flatten, set_by_path

        with open(path, encoding="utf-8") as f:
            text = f.read()
        if path.endswith(".json"):
            tree = json.loads(text)
        else:
            import yaml

            tree = yaml.safe_load(text) or {}
        cfg = cls()
        for key, val in _flatten(tree):
            if isinstance(val, (dict, list)):
                val = json.dumps(val)
            set_by_path(cfg, key, "none" if val is None else str(val))
        for ov in overrides or []:
            if "=" not in ov:
                raise ValueError(f"override {ov!r} is not key=value")
            key, val = ov.split("=", 1)
            set_by_path(cfg, key.lstrip("+"), val)
        return cfg


class SFTTrainer:
    def __init__(self, cfg: SFTConfig, examples: list[dict], ps: ParallelState | None = None, device: str | None = None,
                 tokenizer=None, eval_examples: list[dict] | None = None, callbacks: list | None = None):
        """``examples`` / ``eval_examples``: token rows (``prompt_ids``, ``response_ids``, optional ``loss_mask``), alpaca
        records or chat records; the text forms need ``tokenizer``."""
        from . import sft_data

        self.cfg = cfg
        self.callbacks = list(callbacks or [])
        examples, self.data_stats = sft_data.tokenize_dataset(examples, tokenizer, cfg.max_seq_len, cfg.train_on, cfg.tokenize_cache_dir)
        self.eval_examples = sft_data.tokenize_dataset(eval_examples, tokenizer, cfg.max_seq_len, cfg.train_on, cfg.tokenize_cache_dir)[0] \
            if eval_examples else []
        self.ps = ps or ParallelState.single()
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        mcfg = get_config(cfg.model, **cfg.model_overrides)
        self.model = DecoderLM(mcfg, self.ps, self.device, seed=cfg.seed)
        algo = alg.AlgorithmConfig(policy_loss_type="cross_entropy", loss_reduction=cfg.loss_reduction)
        self.worker = PolicyWorker(self.model, WorkerConfig(max_tokens_per_microbatch=cfg.max_tokens_per_microbatch,
                                                            optimizer=cfg.optimizer), algo)
        if cfg.hf_path:
            from ..models import hf_export

            hf_export.load_hf(self.model, cfg.hf_path)
            if self.worker.opt.low_precision:
                self.worker.opt.master.copy_(self.model.store.flat[self.worker.opt.lo:self.worker.opt.hi].float())
        self.lora_store = None
        if cfg.lora_rank > 0:
            from .lora import AdapterStore, LoRAAdapter, LoRAConfig, LoRATrainer

            if self.ps.tp > 1 or self.ps.pp > 1:
                raise ValueError("LoRA fine-tuning needs tensor- and pipeline-parallel degrees of 1")
            self.lora_store = AdapterStore(self.model)
            self.lora_store.register("sft", LoRAAdapter.init(self.model, LoRAConfig(rank=cfg.lora_rank, alpha=cfg.lora_alpha, lr=cfg.optimizer.lr,
                                                                                    seed=cfg.seed)))
            self.lora_store.activate("sft")
            self.worker.lora = LoRATrainer(self.worker, self.lora_store, "sft")
        self.examples = examples
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

    def _fire(self, event: str, **fields) -> None:
        for cb in self.callbacks:
            fn = getattr(cb, event, None)
            if fn is not None:
                fn(trainer=self, global_step=self.global_step, **fields)

    @staticmethod
    def _batch(rows: list[dict]) -> TrainingInputBatch:
        seq, att, rmask = build_sequences([r["prompt_ids"] for r in rows], [r["response_ids"] for r in rows])
        lmask = rmask.clone()
        for i, r in enumerate(rows):
            m = r.get("loss_mask")
            if m is not None:
                lmask[i, :len(m)] = torch.tensor(m, dtype=lmask.dtype)
        return TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": lmask})

    @torch.no_grad()
    def evaluate(self) -> dict:
        """Mean negative log-likelihood per loss token over the eval set (this rank's share, summed over data parallelism)."""
        rows = self.eval_examples[self.ps.dp_rank::max(1, self.ps.dp)]
        nll, ntok = 0.0, 0.0
        for lo in range(0, len(rows), max(1, self.cfg.eval_batch_size)):
            b = self._batch(rows[lo:lo + self.cfg.eval_batch_size])
            lp = self.worker.forward(b)
            nll -= float((lp * b["loss_mask"]).sum())
            ntok += float(b["loss_mask"].sum())
        nll, ntok = self._global_sum(nll), self._global_sum(ntok)
        out = {"eval/loss": nll / max(1.0, ntok), "eval/tokens": ntok, "eval/examples": self._global_sum(float(len(rows)))}
        if self.tracker is not None:
            self.tracker.log(out, self.global_step)
        self._fire("on_eval_end", metrics=out)
        return out

    def export_hf(self) -> str | None:
        import os

        from ..models import hf_export

        if not self.cfg.export_path or self.ps.pp > 1 or (self.ps.ep == 1 and self.ps.dp_rank != 0):
            return None
        path = os.path.join(self.cfg.export_path, f"global_step_{self.global_step}")
        hf_export.save_hf(self.model, path, write=self.rank == 0)
        return path

    def _dummy_rows(self, n: int) -> list[dict]:
        g = torch.Generator().manual_seed(self.cfg.seed + self.global_step)
        L, V = self.cfg.max_seq_len, self.model.cfg.vocab_size
        return [{"prompt_ids": torch.randint(0, V, (L // 4,), generator=g).tolist(),
                 "response_ids": torch.randint(0, V, (L - L // 4,), generator=g).tolist()} for _ in range(n)]

    def train_step(self, rows: list[dict]) -> dict:
        timings: dict = {}
        self._fire("on_step_begin")
        with Timer("step", timings):
            batch = self._batch(rows)
            rmask = batch["loss_mask"]
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
        self._fire("on_step_end", metrics=out)
        return out

    def _after_step(self) -> None:
        c = self.cfg
        if self.eval_examples and c.eval_interval > 0 and self.global_step % c.eval_interval == 0:
            self.evaluate()
        if c.export_path and c.hf_save_interval > 0 and self.global_step % c.hf_save_interval == 0:
            self.export_hf()

    def train(self) -> None:
        self._fire("on_train_begin")
        try:
            self._train()
        finally:
            if self.eval_examples:
                self.last_eval = self.evaluate()
            if self.cfg.export_path and self.cfg.hf_save_interval <= 0:
                self.export_hf()
            self._fire("on_train_end")

    def _train(self) -> None:
        c = self.cfg
        per_rank = max(1, c.batch_size // max(1, self.ps.dp))
        if c.dummy_steps > 0:
            for _ in range(c.dummy_steps):
                self.train_step(self._dummy_rows(per_rank))
            return
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
                self._after_step()
                if c.ckpt_path and c.ckpt_interval > 0 and self.global_step % c.ckpt_interval == 0:
                    ckpt.save_checkpoint(c.ckpt_path, self.global_step, self.worker, {"cursor": self.cursor, "epoch": self.epoch},
                                         {"global_step": self.global_step}, self.ps)
                if 0 < c.num_steps <= self.global_step:
                    return
            self.cursor, self.epoch = 0, self.epoch + 1
