"""Supervised fine-tuning entry point (reference: R/train/main_sft.py).

    python -m skyrl_isoexec_b200.train.entrypoints.main_sft --data sft.jsonl [--model qwen3-8b] [--batch-size 32] [--epochs 1]
        [--lr 1e-5] [--ckpt-path DIR --ckpt-interval N] [--max-tokens 8192] [--num-steps N]

``--data`` is a JSONL file with one ``{"prompt_ids": [...], "response_ids": [...]}`` per line (token ids); loss is taken
on the response tokens. Under ``torchrun`` the ranks form one data-parallel group.
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
    a = ap.parse_args(argv)
    rank, world, local = init_distributed()
    device = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    ps = ParallelState.build() if world > 1 else ParallelState.single()
    with open(a.data) as f:
        examples = [json.loads(line) for line in f if line.strip()]
    cfg = SFTConfig(model=a.model, batch_size=a.batch_size, epochs=a.epochs, num_steps=a.num_steps, max_tokens_per_microbatch=a.max_tokens,
                    max_seq_len=a.max_seq_len, optimizer=OptimizerConfig(lr=a.lr), ckpt_path=a.ckpt_path, ckpt_interval=a.ckpt_interval,
                    resume_mode=a.resume_mode, logger=a.logger)
    tr = SFTTrainer(cfg, examples, ps=ps, device=device)
    tr.train()
    return tr


if __name__ == "__main__":
    main()
