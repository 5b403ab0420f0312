"""Training entry point (reference: R/train/entrypoints/main_base.py:134-452).

    python -m skyrl_isoexec_b200.train.entrypoints.main_base trainer.policy.model=qwen3-8b key=value ...
    torchrun --nproc-per-node 8 -m skyrl_isoexec_b200.train.entrypoints.main_base ... (one process per GPU)

``BasePPOExp`` keeps the reference's extension hooks (``get_trainer``, ``get_generator``,
``get_inference_client``, ``get_train_dataset``, ``get_tracker``) so an experiment subclass can swap a piece
without touching the loop. No Ray: under torchrun every rank runs the same program.
"""

from __future__ import annotations

import sys

import torch

from ...parallel.state import ParallelState, init_distributed
from ..config import SkyRLTrainConfig, validate_cfg
from ..trainer import RayPPOTrainer


class BasePPOExp:
    def __init__(self, cfg: SkyRLTrainConfig):
        self.cfg = cfg
        self.rank, self.world, self.local_rank = init_distributed()
        validate_cfg(cfg, self.world)
        p = cfg.trainer.policy.parallel
        kv_rep = 1
        if self.world > 1 and p.tensor_model_parallel_size > 1:
            from ...models.config import get_config

            # more tensor-parallel ranks than KV heads: consecutive ranks share (replicate) a KV head
            m = get_config(cfg.trainer.policy.model, **cfg.trainer.policy.model_overrides)
            kv_rep = max(1, p.tensor_model_parallel_size // m.num_kv_heads)
        self.ps = ParallelState.build(tp=p.tensor_model_parallel_size, pp=p.pipeline_model_parallel_size,
                                      ep=p.expert_model_parallel_size, cp=p.context_parallel_size, kv_rep=kv_rep) if self.world > 1 \
            else ParallelState.single()
        self.device = f"cuda:{self.local_rank}" if torch.cuda.is_available() else "cpu"
        if torch.cuda.is_available():
            torch.cuda.set_device(self.local_rank)

    # ---- hooks
    def get_tokenizer(self):
        """``trainer.policy.tokenizer_path``: nothing, the built-in byte tokenizer, or a Hugging Face tokenizer directory."""
        path = self.cfg.trainer.policy.tokenizer_path
        if not path:
            return None
        if getattr(self, "_tok", None) is None:
            if path == "byte":
                from ...utils.tokenizer import ByteTokenizer

                self._tok = ByteTokenizer()
            else:
                from transformers import AutoTokenizer

                self._tok = AutoTokenizer.from_pretrained(path)
        return self._tok

    def get_train_dataset(self):
        from ..dataset import PromptDataset

        d = self.cfg.data
        if d.train_data:
            return PromptDataset(d.train_data, tokenizer=self.get_tokenizer(), max_prompt_length=self.cfg.trainer.max_prompt_length,
                                 env_class=self.cfg.environment.env_class)
        return None   # the trainer falls back to synthetic prompts

    def get_eval_dataset(self):
        from ..dataset import PromptDataset

        d = self.cfg.data
        if d.val_data:
            return PromptDataset(d.val_data, tokenizer=self.get_tokenizer(), max_prompt_length=self.cfg.trainer.max_prompt_length,
                                 env_class=self.cfg.environment.env_class)
        return None   # evaluation then uses the first training prompts

    def get_tracker(self):
        return None

    def get_trainer(self) -> RayPPOTrainer:
        if self.cfg.trainer.fully_async.enabled and type(self) is BasePPOExp:
            # trainer.fully_async.enabled=true on the plain entry point means the fully asynchronous trainer, as in the reference
            from .main_async import AsyncPPOExp

            fa = self.cfg.trainer.fully_async
            exp = AsyncPPOExp.__new__(AsyncPPOExp)
            exp.__dict__.update(self.__dict__)
            exp.mode, exp.max_staleness_steps, exp.generation_workers = "fully_async", fa.max_staleness_steps, fa.num_parallel_generation_workers
            return exp.get_trainer()
        return RayPPOTrainer(self.cfg, ps=self.ps, device=self.device, dataset=self.get_train_dataset(),
                             tokenizer=self.get_tokenizer(), tracker=self.get_tracker())

    def run(self):
        trainer = self.get_trainer()
        ev = self.get_eval_dataset()
        if ev is not None:
            trainer.eval_dataset = ev
        trainer.build_models()
        if self.world > 1 and torch.cuda.is_available() and self.ps.dp > 1:
            from ...parallel.symm_runtime import SymmGroup

            SymmGroup(self.ps.dp_group)
        trainer.train()
        return trainer


def main(argv=None) -> None:
    """``main_base [--config file.yaml] key=value ...``: an optional YAML / JSON config file, then overrides."""
    args = list(sys.argv[1:] if argv is None else argv)
    path = None
    if args and args[0] in ("--config", "-c"):
        path, args = args[1], args[2:]
    elif args and args[0].startswith("--config="):
        path, args = args[0].split("=", 1)[1], args[1:]
    cfg = SkyRLTrainConfig.from_file(path, args) if path else SkyRLTrainConfig.from_cli_overrides(args)
    BasePPOExp(cfg).run()


if __name__ == "__main__":
    main()
