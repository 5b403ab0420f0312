"""Chunked LM-head log-probabilities: time and peak memory against the chunk size, forward and forward+backward
(reference: R/benchmarks/ chunked-logprobs benchmark).

    python -m skyrl_isoexec_b200.benchmarks.bench_logprobs [--model qwen3-8b] [--rows 8192] [--chunks 1024,4096,8192]

The [rows, vocab] logits tensor is never kept: each chunk is a GEMM into a scratch tile, a fused row-invariant
log-softmax/gather, and (in the backward) a recompute. Memory is therefore linear in the chunk, not in the rows.
"""

from __future__ import annotations

import argparse
import time

import torch

from ..models.config import get_config
from ..models.decoder import DecoderLM
from ..train.policy_worker import lm_head_logprobs


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--chunks", default="1024,4096,8192")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    cfg = get_config(args.model, num_layers=1)
    model = DecoderLM(cfg, device=args.device)
    hidden = torch.randn(args.rows, cfg.hidden_size, device=args.device).to(cfg.torch_dtype)
    targets = torch.randint(0, cfg.vocab_size, (args.rows,), device=args.device)
    cuda = args.device != "cpu"
    for chunk in [int(c) for c in args.chunks.split(",")]:
        for mode in ("forward", "forward+backward"):
            if cuda:
                torch.cuda.reset_peak_memory_stats()
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            if mode == "forward":
                with torch.no_grad():
                    lp, _ = lm_head_logprobs(model, hidden, targets, chunk)
            else:
                h = hidden.clone().requires_grad_()
                lp, _ = lm_head_logprobs(model, h, targets, chunk)
                lp.sum().backward()
                model.zero_grad(set_to_none=True)
            if cuda:
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            peak = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else float("nan")
            print(f"chunk {chunk:6d} {mode:17s} {dt * 1e3:9.1f} ms   peak {peak:6.2f} GiB   {args.rows / dt:9.0f} rows/s")


if __name__ == "__main__":
    main()
