"""Helpers around generator outputs and chat rendering (reference: R/train/generators/utils.py: trajectory metrics, overlong
filtering, per-turn token counts, custom chat templates, the generation-prompt ids of a tokenizer, turning a finished
conversation into response ids with an assistant-only loss mask, merging step-wise outputs back into trajectories).

Everything here is host-side list processing; tokenizers are duck-typed (``encode`` and, when present,
``apply_chat_template``), as in ``train/sft_data.py``.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import os
from collections import defaultdict

from .sft_data import _ids


# ------------------------------------------------------------------------------------ metrics
def get_metrics_from_generator_output(generator_output: dict, uids: list) -> dict:
    """``avg_score`` (mean trajectory reward), ``pass_at_n`` (share of prompts with at least one positive trajectory; n is
    the number of trajectories per prompt) and ``mean_positive_reward``. Rewards are per trajectory (floats) or per token
    (lists): a token-level trajectory scores the sum of its tokens, and its LAST token decides the pass."""
    rewards = generator_output["rewards"]
    if not len(rewards):
        raise ValueError("`rewards` must not be empty")
    if len(rewards) != len(uids):
        raise ValueError(f"{len(rewards)} rewards for {len(uids)} uids")
    per_uid = defaultdict(list)
    if isinstance(rewards[0], (list, tuple)):
        if any(len(r) == 0 for r in rewards):
            raise ValueError("token-level rewards of a trajectory must not be empty")
        totals = [float(sum(r)) for r in rewards]
        positives = [float(sum(max(x, 0.0) for x in r)) for r in rewards]
        for u, r in zip(uids, rewards):
            per_uid[u].append(float(r[-1]))
    else:
        totals = [float(r) for r in rewards]
        positives = [max(t, 0.0) for t in totals]
        for u, r in zip(uids, totals):
            per_uid[u].append(r)
    n = len(totals)
    return {"avg_score": sum(totals) / n, "mean_positive_reward": sum(positives) / n,
            "pass_at_n": sum(1 for v in per_uid.values() if any(x > 0 for x in v)) / len(per_uid)}


def apply_overlong_filtering(loss_masks: list[list[int]], stop_reasons: list[str]) -> list[list[int]]:
    """DAPO overlong filtering: a response that did not end by itself (stop reason other than ``"stop"``) carries no
    loss at all. Decided from the engine's stop reasons, so no end-of-sequence id has to be known."""
    if len(loss_masks) != len(stop_reasons):
        raise ValueError("loss_masks and stop_reasons must have the same length")
    return [list(m) if why == "stop" else [0] * len(m) for m, why in zip(loss_masks, stop_reasons)]


def compute_turn_token_counts(loss_masks: list[list[int]]) -> list[int]:
    """Token counts of the model's turns over a batch: a turn is a maximal run of non-zero mask entries (observation
    tokens are masked 0 and separate the turns). One entry per turn, trajectories without loss contribute none."""
    out = []
    for mask in loss_masks:
        run = 0
        for m in mask:
            if m:
                run += 1
            elif run:
                out.append(run)
                run = 0
        if run:
            out.append(run)
    return out


# ------------------------------------------------------------------------------------ chat templates
CUSTOM_CHAT_TEMPLATES = {
    # keeps earlier assistant turns' reasoning blocks (a stock template may strip them, which breaks prefix stability)
    "qwen3_with_thinking": (
        "{% for message in messages %}{{ '<|im_start|>' + message['role'] + '\\n' + message['content'] + '<|im_end|>\\n' }}{% endfor %}"
        "{% if add_generation_prompt %}{{ '<|im_start|>assistant\\n' }}{% endif %}"),
    # drops everything up to and including </think> from assistant turns
    "qwen3_without_thinking": (
        "{% for message in messages %}{% set c = message['content'] %}"
        "{% if message['role'] == 'assistant' and '</think>' in c %}{% set c = c.split('</think>')[-1].lstrip('\\n') %}{% endif %}"
        "{{ '<|im_start|>' + message['role'] + '\\n' + c + '<|im_end|>\\n' }}{% endfor %}"
        "{% if add_generation_prompt %}{{ '<|im_start|>assistant\\n' }}{% endif %}"),
}


def get_custom_chat_template(cfg: dict | None) -> str | None:
    """``{"source": "name", "name_or_path": <key of CUSTOM_CHAT_TEMPLATES>}`` or ``{"source": "file", "name_or_path":
    <path of a Jinja template file>}``; ``None`` / empty keeps the tokenizer's own template."""
    if not cfg or not cfg.get("name_or_path"):
        return None
    src, ref = cfg.get("source", "name"), cfg["name_or_path"]
    if src == "name":
        if ref not in CUSTOM_CHAT_TEMPLATES:
            raise ValueError(f"unknown chat template {ref!r}; known: {sorted(CUSTOM_CHAT_TEMPLATES)}")
        return CUSTOM_CHAT_TEMPLATES[ref]
    if src == "file":
        path = os.path.abspath(os.path.expanduser(ref))
        if not os.path.isfile(path):
            raise FileNotFoundError(f"chat template file {path} does not exist")
        with open(path, encoding="utf-8") as f:
            return f.read()
    raise ValueError(f"chat template source {src!r} must be 'name' or 'file'")


def get_generation_prompt_ids(tokenizer) -> list[int]:
    """The ids a template appends to open an assistant turn (``add_generation_prompt=True`` minus ``False``)."""
    if not hasattr(tokenizer, "apply_chat_template"):
        return list(tokenizer.encode("<|assistant|>\n"))
    msgs = [{"role": "user", "content": ""}]
    a = chat_ids(tokenizer, msgs, False)
    b = chat_ids(tokenizer, msgs, True)
    if b[:len(a)] != a:
        raise ValueError("the tokenizer's template is not prefix-stable under add_generation_prompt")
    return b[len(a):]


def encode_messages_subset(messages: list[dict], tokenizer) -> list[int]:
    """Ids of ``messages`` as they appear INSIDE a longer conversation: rendered after a fixed dummy first turn, whose
    ids are cut off again, so that a template's start-of-conversation preamble (system prompt injection, BOS) is not
    repeated for every appended observation."""
    base = [{"role": "user", "content": "."}]
    head = _ids(tokenizer, base)
    full = _ids(tokenizer, base + list(messages))
    if full[:len(head)] != head:
        raise ValueError("the tokenizer's template is not prefix-stable: cannot encode a slice of a conversation")
    return full[len(head):]


def get_response_ids_and_loss_mask_from_messages(messages: list[dict], tokenizer, assistant_logprobs: list[list[float]] | None = None):
    """A finished conversation AFTER the initial prompt -> (response ids, loss mask, rollout logprobs or None). Assistant
    turns are split into the generation prompt (mask 0), the generated tokens (mask 1) and whatever the template
    appends after them (mask 0); every other role is mask 0. ``assistant_logprobs``: one list per assistant turn with a
    logprob per GENERATED token; non-generated positions get 0.0."""
    gen = get_generation_prompt_ids(tokenizer)
    ids, mask, lps = [], [], [] if assistant_logprobs is not None else None
    a_i = 0
    for m in messages:
        cur = encode_messages_subset([m], tokenizer)
        if m["role"] != "assistant":
            ids += cur
            mask += [0] * len(cur)
            if lps is not None:
                lps += [0.0] * len(cur)
            continue
        start = len(gen) if cur[:len(gen)] == gen else 0
        body = list(tokenizer.encode(m.get("content") or "")) if not hasattr(tokenizer, "apply_chat_template") else None
        n_gen = len(cur) - start
        if assistant_logprobs is not None:
            n_gen = min(n_gen, len(assistant_logprobs[a_i]))         # what follows the generated tokens is the template's
        elif body is not None:
            n_gen = min(n_gen, len(body))
        ids += cur
        mask += [0] * start + [1] * n_gen + [0] * (len(cur) - start - n_gen)
        if lps is not None:
            lps += [0.0] * start + list(assistant_logprobs[a_i][:n_gen]) + [0.0] * (len(cur) - start - n_gen)
        a_i += 1
    return ids, mask, lps


# ------------------------------------------------------------------------------------ step-wise outputs
def merge_stepwise_output(generator_output: dict) -> dict:
    """Step-wise rollouts (one row per model turn, ``trajectory_ids`` + ``is_last_step``) back to one row per trajectory:
    a later step's prompt extends the earlier step's prompt + response, so the merged response is what follows the FIRST
    step's prompt in the LAST step's full sequence; tokens that were observations get mask 0 and logprob 0, the reward
    is the last step's."""
    tids = generator_output["trajectory_ids"]
    order: dict = {}
    for i, t in enumerate(tids):
        order.setdefault(t, []).append(i)
    keys = ("prompt_token_ids", "response_ids", "rewards", "loss_masks", "stop_reasons", "rollout_logprobs")
    out = {k: [] for k in keys if generator_output.get(k) is not None}
    for t, rows in order.items():
        first, last = rows[0], rows[-1]
        p0 = list(generator_output["prompt_token_ids"][first])
        resp, mask, lps, rew = [], [], [], []
        per_token = isinstance(generator_output["rewards"][first], (list, tuple))
        pos = len(p0)
        for i in rows:
            p, r = list(generator_output["prompt_token_ids"][i]), list(generator_output["response_ids"][i])
            if p[:pos] != (p0 + resp)[:pos] or len(p) < pos:
                raise ValueError(f"trajectory {t!r}: step {i} does not extend the steps before it")
            gap = p[pos:]                                           # observation tokens appended since the previous step
            resp += gap + r
            mask += [0] * len(gap) + list(generator_output["loss_masks"][i])
            if "rollout_logprobs" in out:
                lps += [0.0] * len(gap) + list(generator_output["rollout_logprobs"][i])
            if per_token:
                rew += [0.0] * len(gap) + list(generator_output["rewards"][i])
            pos = len(p) + len(r)
        out["prompt_token_ids"].append(p0)
        out["response_ids"].append(resp)
        out["loss_masks"].append(mask)
        out["rewards"].append(rew if per_token else generator_output["rewards"][last])
        if "stop_reasons" in out:
            out["stop_reasons"].append(generator_output["stop_reasons"][last])
        if "rollout_logprobs" in out:
            out["rollout_logprobs"].append(lps)
    out["trajectory_ids"] = list(order)
    return out
