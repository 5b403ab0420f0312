"""Peak training memory against the micro-batch size (reference: R/benchmarks/ memory sweep): one forward_backward of
the policy worker per token budget, peak allocator bytes and tokens per second for each.

    python -m skyrl_isoexec_b200.benchmarks.memory_sweep [--model qwen3-8b] [--layers 4] [--tokens 2048,4096,8192] [--seq-len 1024]

The sweep is bounded: before each point the activation estimate of ``PolicyWorker.activation_bytes_per_layer`` is
checked against the free memory, and a point that would not fit under ``--limit-frac`` of it is skipped, not tried.
"""

from __future__ import annotations

import argparse
import json
import time

import torch

from ..models.config import get_config
from ..models.decoder import DecoderLM
from ..train.batch import TrainingInputBatch, build_sequences
from ..train.policy_worker import PolicyWorker, WorkerConfig


def run(model: str, layers: int, tokens: list[int], seq_len: int, device: str, limit_frac: float = 0.8, recompute: bool = True) -> list[dict]:
    cfg = get_config(model, num_layers=layers) if layers else get_config(model)
    m = DecoderLM(cfg, device=device)
    rows = []
    w = PolicyWorker(m, WorkerConfig(checkpoint_layers=recompute))     # one worker: its gradient hooks live on the parameters
    for budget in tokens:
        w.cfg.max_tokens_per_microbatch = budget
        est = w.activation_bytes_per_layer(budget) * (1 if recompute else len(m.layer_ids)) + budget * cfg.vocab_size * 4 // 8
        if device != "cpu":
            free, _ = torch.cuda.mem_get_info()
            if est > limit_frac * free:
                rows.append({"tokens": budget, "skipped": f"estimate {est / 2**30:.1f} GiB exceeds {limit_frac:.0%} of the free {free / 2**30:.1f} GiB"})
                continue
            torch.cuda.reset_peak_memory_stats()
        n_seq = max(1, budget // seq_len)
        g = torch.Generator().manual_seed(0)
        half = max(1, min(seq_len, budget) // 2)
        prompts = [torch.randint(0, cfg.vocab_size, (half,), generator=g).tolist() for _ in range(n_seq)]
        resp = [torch.randint(0, cfg.vocab_size, (half,), generator=g).tolist() for _ in range(n_seq)]
        seq, att, rmask = build_sequences(prompts, resp)
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.ones(rmask.shape)})
        t0 = time.perf_counter()
        w.forward_backward(batch)
        if device != "cpu":
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        w.opt.zero_grad()
        rows.append({"tokens": budget, "sequences": n_seq, "seconds": round(dt, 4), "tokens_per_s": round(n_seq * 2 * half / dt, 1),
                     "peak_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2) if device != "cpu" else None,
                     "estimate_gib": round(est / 2**30, 2)})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", default="2048,4096,8192")
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--limit-frac", type=float, default=0.8)
    ap.add_argument("--no-recompute", action="store_true")
    a = ap.parse_args(argv)
    for r in run(a.model, a.layers, [int(x) for x in a.tokens.split(",")], a.seq_len, a.device, a.limit_frac, not a.no_recompute):
        print(json.dumps(r))


if __name__ == "__main__":
    main()
