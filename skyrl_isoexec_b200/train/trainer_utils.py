"""Trainer helpers: dynamic sampling (DAPO-style filter / replace), checkpoint directory hygiene,
batch dumps (reference: R/train/utils/trainer_utils.py:343-443 checkpoint cleanup/validation,
:618-842 dynamic sampling)."""

from __future__ import annotations

import json
import os
import random
import shutil
from collections import defaultdict


# ------------------------------------------------------------------ dynamic sampling
def _groups(uids: list) -> dict:
    g = defaultdict(list)
    for i, u in enumerate(uids):
        g[u].append(i)
    return g


def _score(r) -> float:
    return float(sum(r)) if isinstance(r, (list, tuple)) else float(r)


def _take(go: dict, idx: list[int]) -> dict:
    out = {}
    for k, v in go.items():
        out[k] = [v[i] for i in idx] if isinstance(v, list) and len(v) == len(go["response_ids"]) else v
    return out


def _cat(a: dict | None, b: dict) -> dict:
    if a is None:
        return b
    n = len(a["response_ids"])
    return {k: (a[k] + b[k]) if isinstance(a[k], list) and len(a[k]) == n else a[k] for k in a}


def informative_groups(go: dict, uids: list) -> tuple[list, list]:
    """uids of prompt groups whose samples do not all have the same reward (a zero-variance group has zero
    GRPO advantage everywhere and teaches nothing), and the rest."""
    good, bad = [], []
    for u, idx in _groups(uids).items():
        scores = [_score(go["rewards"][i]) for i in idx]
        (good if max(scores) - min(scores) > 1e-12 else bad).append(u)
    return good, bad


def handle_dynamic_sampling(go: dict, uids: list, cfg, state: dict, prompts_needed: int, n_samples: int, seed: int = 0):
    """Returns (generator_output, uids, keep_sampling).

    ``filter``  : keep only informative groups, accumulating over successive sample batches in ``state``
                  until ``prompts_needed`` groups are there (or ``max_sample_batches`` is hit, which raises);
    ``replace`` : if at least ``min_replace_ratio`` of the groups are informative, overwrite each
                  uninformative group with a copy of a randomly chosen informative one (new uid); else keep all.
    """
    kind = cfg.dynamic_sampling_type
    if not kind:
        return go, uids, False
    good, bad = informative_groups(go, uids)
    grp = _groups(uids)
    if kind == "replace":
        if not bad or len(good) < cfg.dynamic_sampling_min_replace_ratio * len(grp):
            return go, uids, False
        rng = random.Random(seed)
        idx, new_uids = [], []
        for u in grp:
            src = u if u in good else rng.choice(good)
            idx += grp[src]
            new_uids += [u if u in good else f"{src}#for#{u}"] * len(grp[src])
        return _take(go, idx), new_uids, False
    if kind != "filter":
        raise ValueError(f"unknown dynamic sampling type {kind!r} (filter | replace)")
    keep_idx = [i for u in good for i in grp[u]]
    state["batches"] = state.get("batches", 0) + 1
    state["go"] = _cat(state.get("go"), _take(go, keep_idx))
    state["uids"] = state.get("uids", []) + [uids[i] for i in keep_idx]
    have = len(_groups(state["uids"]))
    if have >= prompts_needed:
        order = list(_groups(state["uids"]).items())[:prompts_needed]
        idx = [i for _, ix in order for i in ix]
        out, out_uids = _take(state["go"], idx), [state["uids"][i] for i in idx]
        state.clear()
        return out, out_uids, False
    if state["batches"] >= cfg.dynamic_sampling_max_sample_batches:
        raise RuntimeError(f"dynamic sampling: only {have} of {prompts_needed} informative prompt groups after "
                           f"{state['batches']} sample batches; the task is too easy or too hard for this policy")
    return None, None, True


# ------------------------------------------------------------------ checkpoints on disk
def list_checkpoints(root: str) -> list[int]:
    if not os.path.isdir(root):
        return []
    steps = []
    for name in os.listdir(root):
        if name.startswith("global_step_") and name[len("global_step_"):].isdigit():
            steps.append(int(name[len("global_step_"):]))
    return sorted(steps)


def cleanup_old_checkpoints(root: str, max_to_keep: int) -> list[int]:
    """Delete all but the newest ``max_to_keep`` step directories (-1 keeps everything)."""
    steps = list_checkpoints(root)
    if max_to_keep < 0 or len(steps) <= max_to_keep:
        return []
    victims = steps[:len(steps) - max_to_keep]
    for s in victims:
        shutil.rmtree(os.path.join(root, f"global_step_{s}"), ignore_errors=True)
    return victims


def validate_consistency_for_latest_checkpoint(root: str) -> int | None:
    """The step named by ``latest_ckpt_global_step.txt`` must exist and be complete; returns it (or None)."""
    marker = os.path.join(root, "latest_ckpt_global_step.txt")
    if not os.path.exists(marker):
        return None
    step = int(open(marker).read().strip())
    d = os.path.join(root, f"global_step_{step}")
    need = ["policy", "trainer_state.pt", "data.pt"]
    missing = [n for n in need if not os.path.exists(os.path.join(d, n))]
    if missing:
        raise RuntimeError(f"checkpoint {d} is named as latest but lacks {missing}; remove the marker or the partial directory")
    return step


def dump_per_dataset_eval_results(path: str, rows: list[dict], metrics: dict) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    with open(os.path.splitext(path)[0] + ".metrics.json", "w") as f:
        json.dump(metrics, f, indent=1, sort_keys=True)
