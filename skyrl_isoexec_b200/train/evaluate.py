"""Evaluation: generate on a validation set with the eval sampling parameters and report reward
statistics and pass@k (reference: R/train/evaluate.py)."""

from __future__ import annotations

import asyncio
from collections import defaultdict

from .generator import GeneratorInput


def pass_at_k(n: int, c: int, k: int) -> float:
    """Unbiased estimator of pass@k from n samples with c correct (Chen et al., 2021)."""
    if n - c < k:
        return 1.0
    p = 1.0
    for i in range(n - c + 1, n + 1):
        p *= 1.0 - k / i
    return 1.0 - p


def evaluate(generator, rows: list[dict], sampling_params: dict, n_samples: int = 1, ks=(1,), batch_size: int = 1024,
             dump_path: str = "", decode=None) -> dict:
    """rows: dataset rows ({prompt, env_class, env_extras, uid}). Returns eval/* metrics. ``dump_path``: a JSONL file that
    gets one line per evaluated sample (uid, environment, prompt and response as ids and, with ``decode``, as text, reward,
    stop reason), the reference's ``dump_eval_results``."""
    by_uid: dict = defaultdict(list)
    lens = []
    dump = []
    for lo in range(0, len(rows), batch_size):
        chunk = rows[lo:lo + batch_size]
        gi: GeneratorInput = {"prompts": [r["prompt"] for r in chunk for _ in range(n_samples)],
                              "env_classes": [r["env_class"] for r in chunk for _ in range(n_samples)],
                              "env_extras": [r.get("env_extras") or {} for r in chunk for _ in range(n_samples)],
                              "sampling_params": sampling_params, "trajectory_ids": None, "batch_metadata": {"eval": True}}
        go = asyncio.run(generator.generate(gi))
        uids = [r["uid"] for r in chunk for _ in range(n_samples)]
        if go.get("step_source") is not None:
            # step-wise output (one row per model turn; R/train/evaluate.py ``evaluate_step_wise``): a trajectory is scored by
            # its LAST step's reward, and its length is the sum over its turns
            total = defaultdict(int)
            for src, resp in zip(go["step_source"], go["response_ids"]):
                total[src] += len(resp)
            for src, rew, last in zip(go["step_source"], go["rewards"], go["is_last_step"]):
                if last:
                    by_uid[uids[src]].append(float(sum(rew)) if isinstance(rew, (list, tuple)) else float(rew))
                    lens.append(total[src])
        else:
            for uid, rew, resp in zip(uids, go["rewards"], go["response_ids"]):
                by_uid[uid].append(float(sum(rew)) if isinstance(rew, (list, tuple)) else float(rew))
                lens.append(len(resp))
        if dump_path:
            envs = gi["env_classes"]
            for i, resp in enumerate(go["response_ids"]):
                src = go["step_source"][i] if go.get("step_source") is not None else i
                rew = go["rewards"][i]
                rec = {"uid": uids[src], "env_class": envs[src], "prompt_ids": list(go["prompt_token_ids"][i]), "response_ids": list(resp),
                       "reward": float(sum(rew)) if isinstance(rew, (list, tuple)) else float(rew),
                       "stop_reason": (go.get("stop_reasons") or [None] * len(go["response_ids"]))[i]}
                if decode is not None:
                    rec["prompt"], rec["response"] = decode(rec["prompt_ids"]), decode(rec["response_ids"])
                dump.append(rec)
    if dump_path:
        import json

        from ..utils import io as uio

        with uio.open_file(dump_path, "w") as f:
            for rec in dump:
                f.write(json.dumps(rec) + "\n")
    allr = [r for v in by_uid.values() for r in v]
    out = {"eval/avg_reward": sum(allr) / max(1, len(allr)), "eval/num_prompts": len(by_uid),
           "eval/avg_response_length": sum(lens) / max(1, len(lens))}
    for k in ks:
        if k <= n_samples:
            out[f"eval/pass_at_{k}"] = sum(pass_at_k(len(v), sum(1 for r in v if r > 0), k) for v in by_uid.values()) / max(1, len(by_uid))
    return out
