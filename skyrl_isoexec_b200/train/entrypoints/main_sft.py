"""Supervised fine-tuning entry point (reference: R/train/main_sft.py).

    python -m skyrl_isoexec_b200.train.entrypoints.main_sft --data sft.jsonl [--model qwen3-8b] [--batch-size 32] [--epochs 1]
        [--lr 1e-5] [--ckpt-path DIR --ckpt-interval N] [--max-tokens 8192] [--num-steps N]
        [--eval-data eval.jsonl --eval-interval N] [--tokenizer DIR --train-on last|all --cache-dir DIR]
        [--export-path DIR --hf-save-interval N] [--dummy-steps N]

``--data`` is a JSONL file with one record per line: ``{"prompt_ids": [...], "response_ids": [...]}`` (token ids), an
alpaca record (``instruction`` / ``input`` / ``output``) or a chat record (``messages`` with optional ``tool_calls`` and
``tools``). Text records need ``--tokenizer`` (a directory ``transformers.AutoTokenizer`` can load; its chat template is
used when it has one). Loss is taken on the response / assistant tokens. Under ``torchrun`` the ranks form one
data-parallel group.
"""

from __future__ import annotations

import argparse
import json

import torch

from ...parallel.state import ParallelState, init_distributed
from ..policy_worker import OptimizerConfig
from ..sft_trainer import SFTConfig, SFTTrainer


def main(argv=None) -> SFTTrainer:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True)
    ap.add_argument("--model", default="tiny-qwen3")
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--num-steps", type=int, default=-1)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--max-tokens", type=int, default=8192)
    ap.add_argument("--max-seq-len", type=int, default=4096)
    ap.add_argument("--ckpt-path", default="")
    ap.add_argument("--ckpt-interval", type=int, default=0)
    ap.add_argument("--resume-mode", default="latest")
    ap.add_argument("--logger", default="console")
    ap.add_argument("--eval-data", default="")
    ap.add_argument("--eval-interval", type=int, default=0)
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--train-on", default="last", choices=["last", "all"])
    ap.add_argument("--cache-dir", default="")
    ap.add_argument("--export-path", default="")
    ap.add_argument("--hf-save-interval", type=int, default=0)
    ap.add_argument("--dummy-steps", type=int, default=0)
    a = ap.parse_args(argv)
    rank, world, local = init_distributed()
    device = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    ps = ParallelState.build() if world > 1 else ParallelState.single()
    def read(path):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]

    examples = read(a.data)
    eval_examples = read(a.eval_data) if a.eval_data else None
    tokenizer = None
    if a.tokenizer:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(a.tokenizer)
    cfg = SFTConfig(model=a.model, batch_size=a.batch_size, epochs=a.epochs, num_steps=a.num_steps, max_tokens_per_microbatch=a.max_tokens,
                    max_seq_len=a.max_seq_len, optimizer=OptimizerConfig(lr=a.lr), ckpt_path=a.ckpt_path, ckpt_interval=a.ckpt_interval,
                    resume_mode=a.resume_mode, logger=a.logger, train_on=a.train_on, tokenize_cache_dir=a.cache_dir,
                    eval_interval=a.eval_interval, export_path=a.export_path, hf_save_interval=a.hf_save_interval, dummy_steps=a.dummy_steps)
    tr = SFTTrainer(cfg, examples, ps=ps, device=device, tokenizer=tokenizer, eval_examples=eval_examples)
    tr.train()
    return tr


if __name__ == "__main__":
    main()
