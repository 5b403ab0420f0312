"""Supervised fine-tuning entry point (reference: R/train/main_sft.py).

    python -m skyrl_isoexec_b200.train.entrypoints.main_sft --data sft.jsonl [--model qwen3-8b] [--batch-size 32] [--epochs 1]
        [--lr 1e-5] [--ckpt-path DIR --ckpt-interval N] [--max-tokens 8192] [--num-steps N]
        [--eval-data eval.jsonl --eval-interval N] [--tokenizer DIR --train-on last|all --cache-dir DIR]
        [--export-path DIR --hf-save-interval N] [--dummy-steps N] [--lora-rank R --lora-alpha A] [--hf-path DIR]
        [--config sft.yaml] [key=value ...]

``--data`` is a JSONL file with one record per line: ``{"prompt_ids": [...], "response_ids": [...]}`` (token ids), an
alpaca record (``instruction`` / ``input`` / ``output``) or a chat record (``messages`` with optional ``tool_calls`` and
``tools``). Text records need ``--tokenizer`` (a directory ``transformers.AutoTokenizer`` can load; its chat template is
used when it has one). Loss is taken on the response / assistant tokens. Under ``torchrun`` the ranks form one
data-parallel group.

``--config`` names a YAML or JSON file of ``SFTConfig`` fields; trailing ``key=value`` words override it with dotted
keys (``optimizer.lr=3e-6``), and an option given on the command line overrides both.
"""

from __future__ import annotations

import argparse
import json

import torch

from ...parallel.state import ParallelState, init_distributed
from ..config import set_by_path
from ..sft_trainer import SFTConfig, SFTTrainer


def main(argv=None) -> SFTTrainer:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True)
    ap.add_argument("--config", default="")
    ap.add_argument("overrides", nargs="*", help="key=value overrides of the config (dotted keys)")
    # options that map onto SFTConfig fields: no default here, so that only the ones given override the file
    opts = {"model": ("--model", str), "batch_size": ("--batch-size", int), "epochs": ("--epochs", int), "num_steps": ("--num-steps", int),
            "optimizer.lr": ("--lr", float), "max_tokens_per_microbatch": ("--max-tokens", int), "max_seq_len": ("--max-seq-len", int),
            "ckpt_path": ("--ckpt-path", str), "ckpt_interval": ("--ckpt-interval", int), "resume_mode": ("--resume-mode", str),
            "logger": ("--logger", str), "eval_interval": ("--eval-interval", int), "train_on": ("--train-on", str),
            "tokenize_cache_dir": ("--cache-dir", str), "export_path": ("--export-path", str),
            "hf_save_interval": ("--hf-save-interval", int), "dummy_steps": ("--dummy-steps", int), "lora_rank": ("--lora-rank", int),
            "lora_alpha": ("--lora-alpha", float), "hf_path": ("--hf-path", str)}
    for key, (flag, tp) in opts.items():
        ap.add_argument(flag, type=tp, default=None, dest="f_" + key.replace(".", "__"),
                        **({"choices": ["last", "all"]} if key == "train_on" else {}))
    ap.add_argument("--eval-data", default="")
    ap.add_argument("--tokenizer", default="")
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
    cfg = SFTConfig.from_file(a.config, a.overrides) if a.config else SFTConfig()
    if not a.config:
        for ov in a.overrides:
            set_by_path(cfg, *ov.split("=", 1))
    for key in opts:
        val = getattr(a, "f_" + key.replace(".", "__"))
        if val is not None:
            set_by_path(cfg, key, str(val))
    tr = SFTTrainer(cfg, examples, ps=ps, device=device, tokenizer=tokenizer, eval_examples=eval_examples)
    tr.train()
    return tr


if __name__ == "__main__":
    main()
