"""Headline benchmark: full GRPO steps of Qwen3-8B (rollout + scoring + policy update + weight
sync) through the framework's public trainer API, one process per GPU.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0. ``value`` is the whole-job aggregate of response tokens per
second through complete GRPO steps, timed on the device with CUDA events (max over ranks);
``e2e`` is the same quantity from the host clock around ``RayPPOTrainer.train_step`` (prompts
enter from pinned host memory, sampled tokens / logprobs / loss come back to the host every
step). Weak scaling: each GPU keeps 8 prompts x 8 samples, 512-token prompts, 2048-token responses,
so 8 GPUs run the named configuration (64 prompts x 8 samples).

Layout per GPU count (``--tp`` / ``--engine-tp`` override it, ``--layout dp`` forces plain data parallelism):

    1 GPU    one trainer, one engine on the trainer's weights
    2 GPUs   trainer TP2,        two engines at TP1
    4 GPUs   trainer TP4,        two engines at TP2
    8 GPUs   trainer TP4 x DP2,  four engines at TP2      (the named configuration)

With more than one GPU the engines have their own layout and every step ends with a resharding weight sync
(trainer shards -> engine shards over peer memory), reported as ``sync_ms_per_step``.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--prompts-per-gpu", type=int, default=8)
    ap.add_argument("--samples", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--response-len", type=int, default=2048)
    ap.add_argument("--micro-tokens", type=int, default=8192)
    ap.add_argument("--tp", type=int, default=0, help="trainer tensor-parallel degree (0 = by GPU count: 1, 2, 4, 4)")
    ap.add_argument("--engine-tp", type=int, default=0, help="engine tensor-parallel degree (0 = by GPU count: 1, 1, 2, 2)")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel degree (MoE models; trainer and engines share it, tp = 1)")
    ap.add_argument("--layout", default="named", choices=["named", "dp"], help="dp: plain data parallelism, engines on the trainer's weights")
    ap.add_argument("--keep-last-layers", type=int, default=-1,
                    help="layers not recomputed in the backward (uses spare HBM); -1 = as many as the first step's measured peak leaves room for")
    ap.add_argument("--reuse-rollout-logprobs", action="store_true",
                    help="variant, not the headline: skip the scoring forward and take the engine's logprobs as the old-policy "
                         "logprobs (same bits under the contract); the gate then compares the training forward with the rollout")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the run invalid)")
    return ap.parse_args()


def reference_arm(args) -> None:
    """The reference's entry point (skyrl.train.entrypoints.main_base) imports ray, omegaconf and
    megatron.core at module import; none of them is installed or installable offline here."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    why = None
    try:
        import skyrl.train.entrypoints.main_base  # noqa: F401
    except Exception as e:  # noqa: BLE001
        why = f"reference entrypoint not importable offline: {type(e).__name__}: {str(e)[:120]}"
    if why is None:
        why = ("reference imports, but its IsoExec path admits only sm90 implementations and needs pinned nightly "
               "vLLM/Megatron/FA3 wheels that are not in the offline wheelhouse")
    print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self.stop_flag = index, [], False

    def run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([x.strip() for x in out.split(",")])
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.2)

    def summary(self) -> dict:
        sm = sorted(int(float(r[0])) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = max((int(float(r[1])) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()), default=0)
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for name, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else 0, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def main():
    args = parse()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_arm(args)
        return
    # NCCL only carries bootstrap, metrics and fallback byte movement here; the collectives on the hot paths are this
    # framework's own peer-memory kernels. Every multi-GPU run of this code so far had NCCL's in-switch reduction off,
    # so that stays the default (set NCCL_NVLS_ENABLE yourself to override).
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    from skyrl_isoexec_b200.ops import _native
    from skyrl_isoexec_b200.parallel.state import ParallelState, init_distributed
    from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
    from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

    rank, world, local = init_distributed()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    _native.lib().ix_init()
    if args.ep > 1:
        args.tp, args.engine_tp, args.layout = 1, 1, "dp"
    if args.layout == "dp":
        args.tp = args.tp or 1
        args.engine_tp = args.engine_tp or args.tp
    else:
        args.tp = args.tp or {1: 1, 2: 2, 4: 4}.get(world, 4)
        args.engine_tp = args.engine_tp or {1: 1, 2: 1}.get(world, 2)
    if world > 1:
        from skyrl_isoexec_b200.models.config import get_config as _gc

        ps = ParallelState.build(tp=args.tp, ep=args.ep, kv_rep=max(1, args.tp // _gc(args.model).num_kv_heads))
    else:
        ps = ParallelState.single()
    P, S = args.prompts_per_gpu * args.tp, args.samples
    per_engine = P * S // max(1, args.tp // args.engine_tp)       # sequences one engine serves per step
    ov = [
        f"trainer.policy.model={args.model}", f"trainer.train_batch_size={P * ps.dp}",
        f"trainer.policy_mini_batch_size={P * ps.dp}", f"generator.n_samples_per_prompt={S}",
        f"generator.sampling_params.max_generate_length={args.response_len}", "generator.sampling_params.ignore_eos=true",
        f"data.synthetic_prompt_len={args.prompt_len}", f"data.synthetic_prompts={P * ps.dp * (args.steps + args.warmup + 1)}",
        f"trainer.max_prompt_length={args.prompt_len}", f"trainer.max_tokens_per_microbatch={args.micro_tokens}",
        f"generator.inference_engine.max_num_seqs={per_engine}", "generator.inference_engine.max_num_batched_tokens=8192",
        f"generator.inference_engine.num_kv_pages={per_engine * ((args.prompt_len + args.response_len) // 128 + 2)}",
        "trainer.policy.optimizer_config.lr=1e-6", "trainer.logger=console" if os.environ.get("BENCH_VERBOSE") else "trainer.logger=jsonl",
        "environment.env_class=even_tokens", "trainer.resume_mode=none", f"trainer.policy.keep_last_layers={args.keep_last_layers}",
    ]
    if args.reuse_rollout_logprobs:
        ov.append("trainer.isoexec.reuse_rollout_logprobs=true")
    mo = {}
    if args.layers:
        mo["num_layers"] = args.layers
    # leaves of the TP-invariant reduction tree: the largest tensor-parallel degree of the deployment (a contract pin
    # shared by trainer and engines; fewer leaves mean wider GEMM tiles on every rank), and at least 2 everywhere: the
    # tree is a K split whose order is part of the contract, so a decode-sized row-parallel GEMM (o, down) gives each
    # leaf its own CTA and folds them through a cluster's shared memory instead of walking all of K in one CTA
    mo["tp_invariant"] = True
    mo["pik_leaves"] = max(2, args.tp, args.engine_tp)
    ov.append(f"generator.inference_engine.tensor_parallel_size={args.engine_tp}")
    if mo:
        ov.append("trainer.policy.model_overrides=" + json.dumps(mo))
    cfg = SkyRLTrainConfig.from_cli_overrides(ov)
    trainer = RayPPOTrainer(cfg, ps=ps, device=f"cuda:{local}")
    trainer.build_models()
    trainer.sync_weights()
    it = iter(trainer.loader)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.train_step(next(it))
    sync_all()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = _native.launch_count()
    h2d0, d2h0 = trainer.engine.stats.get("h2d_bytes", 0), trainer.engine.stats.get("d2h_bytes", 0)
    tokens = 0
    mism = 0
    gen_s = sync_s = 0.0
    sync_bytes = 0
    phases = {"generate": 0.0, "fwd_logprobs": 0.0, "policy_train": 0.0, "sync_weights": 0.0, "convert": 0.0, "advantages": 0.0}
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        m = trainer.train_step(next(it))
        tokens += int(m["generate/response_tokens"])
        mism += int(m["policy/rollout_train_logprob_bit_mismatches"])
        gen_s += float(m["timing/generate"])
        sync_s += float(m["timing/sync_weights"])
        sync_bytes = int(m.get("sync/bytes", 0))
        for k in phases:
            phases[k] += float(m.get(f"timing/{k}", 0.0))
    e1.record()
    sync_all()
    wall = time.perf_counter() - t0
    sampler.stop_flag = True
    sampler.join(timeout=2)
    dev_ms = e0.elapsed_time(e1)
    stats = torch.tensor([dev_ms, wall * 1e3, float(tokens), float(mism), gen_s, sync_s], dtype=torch.float64, device="cuda")
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        dev_ms, wall_ms, gen_s, sync_s = float(mx[0]), float(mx[1]), float(mx[4]), float(mx[5])
        tokens, mism = float(sm[2]) / args.tp, float(sm[3]) / args.tp   # every rank of a TP group reports the same sequences
    else:
        wall_ms = wall * 1e3
    status = _native.read_status()
    if rank == 0:
        launches = _native.launch_count() - launches0
        h2d = (trainer.engine.stats.get("h2d_bytes", 0) - h2d0) / args.steps
        d2h = (trainer.engine.stats.get("d2h_bytes", 0) - d2h0) / args.steps
        out = {
            "metric": "GRPO step throughput: response tokens/s through full steps (rollout+score+update+sync)",
            "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform-random prompt tokens, even-token reward, random-init weights)",
            "grpo_steps_per_s": args.steps / (dev_ms / 1e3), "rollout_tok_per_s": tokens / max(1e-9, gen_s),
            "logprob_mismatches": int(mism), "kernel_status": status,
            "sync_ms_per_step": 1e3 * sync_s / args.steps, "sync_bytes_per_rank": sync_bytes,
            "phase_s_per_step_rank0": {k: round(v / args.steps, 3) for k, v in phases.items()},
            "config": {"model": args.model + (f"[layers={args.layers} INVALID-DEBUG]" if args.layers else ""),
                       "global_batch": P * S * ps.dp, "prompts": P * ps.dp, "samples_per_prompt": S,
                       "prompt_len": args.prompt_len, "seq_len": args.prompt_len + args.response_len,
                       "parallelism": (f"dp{ps.dp}" + (f"xtp{args.tp}" if args.tp > 1 else "") + (f"xep{args.ep}" if args.ep > 1 else "")) if world > 1 else "single",
                       "engine": (f"colocated, {world // args.engine_tp} engines x TP{args.engine_tp}, own layout, resharding weight sync every step"
                                  if trainer.separate_engine else f"colocated, {world // args.tp} engines x TP{args.tp} on the trainer's weights"),
                       "pik_leaves": mo.get("pik_leaves", 0), "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", ""),
                       "scoring_forward": "skipped: rollout logprobs reused (VARIANT, not the reference's step)" if args.reuse_rollout_logprobs else "run",
                       "l2": "working set (16 GB of weights per pass) exceeds L2; no explicit flush"},
            "clocks": sampler.summary(),
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
            "peak_reserved_gb": round(torch.cuda.max_memory_reserved() / 2**30, 1),
            "layers_not_recomputed": int(trainer.policy.keep_layers()), "optimizer_sharded": trainer.policy.opt.shard is not None,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
