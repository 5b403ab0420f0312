"""One engine decode workload, bracketed for a per-kernel launch list.

    python -m skyrl_isoexec_b200.benchmarks.profile_decode_step [--model qwen3-8b] [--seqs 64] [--prompt-len 1536]
                                                                [--warm 6] [--steps 4] [--leaves 2] [--eager]

Random-initialised weights of the named model, ``--seqs`` prompts of ``--prompt-len`` random tokens. After prefill and
``--warm`` decode steps (graph capture included) it runs ``--steps`` decode steps between cudaProfilerStart / Stop and
prints the wall time per step. Under
``ncu --metrics gpu__time_duration.sum --profile-from-start off --clock-control none --csv --log-file out.csv`` the
bracket yields every kernel of those steps with its device time (one pass: nothing is saved or restored); kernels are
serialised and cache-cold there, so compare shares, and take absolute step time from the plain run.
"""

from __future__ import annotations

import argparse
import time

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1536)
    ap.add_argument("--warm", type=int, default=6)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--leaves", type=int, default=2)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--eager", action="store_true")
    args = ap.parse_args(argv)
    from ..engine.llm_engine import EngineConfig, LLMEngine
    from ..engine.sampler import SamplingParams
    from ..models.config import get_config
    from ..models.decoder import DecoderLM
    from ..ops import _native

    _native.lib().ix_init()
    ov = {"dtype": "bfloat16"}
    if args.leaves > 1:
        ov.update(tp_invariant=True, pik_leaves=args.leaves)
    if args.layers:
        ov["num_layers"] = args.layers
    cfg = get_config(args.model, **ov)
    model = DecoderLM(cfg, device="cuda:0", seed=0)
    # sequences admitted by an early prefill chunk decode while the later chunks prefill: leave room for those tokens so
    # that nobody finishes (and the batch, hence the graph, stays the same) before the measured steps are over
    lead = (args.seqs * args.prompt_len + 8191) // 8192 + 2
    total = args.prompt_len + args.warm + args.steps + lead + 8
    eng = LLMEngine(model, EngineConfig(max_num_seqs=args.seqs, num_kv_pages=args.seqs * (total // 128 + 2), max_model_len=total,
                                        max_num_batched_tokens=8192, use_cuda_graph=not args.eager))
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(max_generate_length=args.warm + args.steps + lead + 4, ignore_eos=True)
    for i in range(args.seqs):
        eng.add_request(torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist(), sp, i)

    def decoded():
        sch = eng.scheduler
        return min(len(s.output_ids) for s in sch.running) if sch.running and not sch.waiting else 0

    while decoded() < args.warm:               # prefill chunks, then warm decode steps (the first replays capture)
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    t0 = time.perf_counter()
    n0 = decoded()
    while decoded() < n0 + args.steps:
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    torch.cuda.profiler.stop()
    n = decoded() - n0
    assert _native.read_status() == 0 and len(eng.scheduler.running) == args.seqs, "the batch changed during the measurement"
    print(f"decode: {args.seqs} sequences, ~{args.prompt_len + n0} cached keys, {n} steps, {dt / n * 1e3:.3f} ms per step "
          f"({'eager' if args.eager else 'CUDA graph'}), {args.seqs * n / dt:.0f} tok/s")


if __name__ == "__main__":
    main()
