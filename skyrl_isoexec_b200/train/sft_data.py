"""Turning SFT records into token rows (reference: R/train/sft_trainer.py:80-630, its chat / alpaca tokenizers, the
tool-call normalisation and the on-disk tokenization cache).

A row is ``{"prompt_ids", "response_ids", "loss_mask"}``: the sequence is ``prompt_ids + response_ids``, the loss is taken
on the response tokens whose ``loss_mask`` entry is 1. Three record shapes are understood:

* ``{"prompt_ids": [...], "response_ids": [...]}``                     already tokenized
* ``{"instruction", "input"?, "output"}``                              alpaca style
* ``{"messages": [{"role", "content", "tool_calls"?}, ...], "tools"?}``  chat style; ``train_on`` selects which
  assistant turns carry loss: ``"last"`` (everything before the last assistant turn is prompt) or ``"all"`` (the first
  assistant turn starts the response; user / tool / system tokens inside it get mask 0).

The tokenizer is anything with ``encode(text) -> list[int]``; when it also has ``apply_chat_template`` that is used to
render messages, otherwise a plain ``<|role|>\\ncontent<|end|>\\n`` rendering is. Chat tokenization is PREFIX-BASED: the
ids of the first k messages must be a prefix of the ids of the first k+1 (true of the templates in use; checked, and a
record whose template breaks it is dropped with a count), which is what lets the mask be cut at message boundaries.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import hashlib
import json
import os
import pickle
import tempfile


def _render(messages: list[dict], tools=None) -> str:
    out = []
    if tools:
        out.append("<|tools|>\n" + json.dumps(tools, sort_keys=True) + "<|end|>\n")
    for m in messages:
        body = m.get("content") or ""
        if m.get("tool_calls"):
            body += "".join("\n<tool_call>" + json.dumps(tc, sort_keys=True) + "</tool_call>" for tc in m["tool_calls"])
        out.append(f"<|{m['role']}|>\n{body}<|end|>\n")
    return "".join(out)


def _ids(tokenizer, messages: list[dict], tools=None) -> list[int]:
    if hasattr(tokenizer, "apply_chat_template"):
        kw = {"tools": tools} if tools else {}
        return chat_ids(tokenizer, messages, False, **kw)
    return list(tokenizer.encode(_render(messages, tools)))


def normalize_tools(tools):
    """``tools`` may arrive as a JSON string, a single dict or a list; returns a list of dicts or None."""
    if tools is None or tools == "":
        return None
    if isinstance(tools, str):
        try:
            tools = json.loads(tools)
        except json.JSONDecodeError:
            return None
    if isinstance(tools, dict):
        tools = [tools]
    return [t for t in tools if isinstance(t, dict)] or None


def normalize_messages(messages: list[dict]) -> list[dict]:
    """Roles lower-cased, ``None`` contents made empty, tool calls given as a JSON string or a single dict made a list of
    ``{"name", "arguments"}`` dicts with the arguments decoded."""
    out = []
    for m in messages:
        role = str(m.get("role", "user")).lower()
        d = {"role": role, "content": m.get("content") or ""}
        tcs = m.get("tool_calls")
        if tcs:
            if isinstance(tcs, str):
                try:
                    tcs = json.loads(tcs)
                except json.JSONDecodeError:
                    tcs = None
            if isinstance(tcs, dict):
                tcs = [tcs]
            norm = []
            for tc in tcs or []:
                fn = tc.get("function", tc)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except json.JSONDecodeError:
                        args = {"_raw": args}
                norm.append({"name": fn.get("name", ""), "arguments": args})
            if norm:
                d["tool_calls"] = norm
        if role == "tool" and m.get("name"):
            d["name"] = m["name"]
        out.append(d)
    return out


def tokenize_alpaca(rec: dict, tokenizer, max_length: int) -> dict | None:
    prompt = rec["instruction"] + ("\n\n" + rec["input"] if rec.get("input") else "")
    p = _ids(tokenizer, [{"role": "user", "content": prompt}])
    full = _ids(tokenizer, [{"role": "user", "content": prompt}, {"role": "assistant", "content": rec["output"]}])
    if full[:len(p)] != p or len(full) <= len(p) or len(full) > max_length:
        return None
    r = full[len(p):]
    return {"prompt_ids": p, "response_ids": r, "loss_mask": [1] * len(r)}


def tokenize_chat(rec: dict, tokenizer, max_length: int, train_on: str = "last") -> dict | None:
    msgs = normalize_messages(rec["messages"])
    tools = normalize_tools(rec.get("tools"))
    a_idx = [i for i, m in enumerate(msgs) if m["role"] == "assistant"]
    if not a_idx:
        return None
    first = a_idx[-1] if train_on == "last" else a_idx[0]
    pre = [_ids(tokenizer, msgs[:k], tools) if k else [] for k in range(first, len(msgs) + 1)]
    full = pre[-1]
    if len(full) > max_length or any(full[:len(p)] != p for p in pre):
        return None                                  # too long, or the template is not prefix-stable for this record
    cuts = [len(p) for p in pre]
    mask = []
    for j, k in enumerate(range(first, len(msgs))):
        n = cuts[j + 1] - cuts[j]
        mask += [1 if msgs[k]["role"] == "assistant" else 0] * n
    r = full[cuts[0]:]
    if not r or not any(mask):
        return None
    return {"prompt_ids": full[:cuts[0]], "response_ids": r, "loss_mask": mask}


def tokenize_record(rec: dict, tokenizer, max_length: int, train_on: str = "last") -> dict | None:
    if "prompt_ids" in rec and "response_ids" in rec:
        if len(rec["prompt_ids"]) + len(rec["response_ids"]) > max_length or not rec["response_ids"]:
            return None
        return {"prompt_ids": list(rec["prompt_ids"]), "response_ids": list(rec["response_ids"]),
                "loss_mask": list(rec.get("loss_mask") or [1] * len(rec["response_ids"]))}
    if tokenizer is None:
        raise ValueError("text records need a tokenizer")
    if "messages" in rec:
        return tokenize_chat(rec, tokenizer, max_length, train_on)
    if "instruction" in rec and "output" in rec:
        return tokenize_alpaca(rec, tokenizer, max_length)
    raise ValueError(f"unrecognised SFT record with keys {sorted(rec)}")


def cache_key(records_fingerprint: str, tokenizer, max_length: int, train_on: str) -> str:
    tok = getattr(tokenizer, "name_or_path", None) or type(tokenizer).__name__
    h = hashlib.sha256(json.dumps([records_fingerprint, tok, getattr(tokenizer, "vocab_size", 0), max_length, train_on, 1]).encode())
    return h.hexdigest()[:24]


def fingerprint(records: list[dict]) -> str:
    h = hashlib.sha256()
    for r in records:
        h.update(json.dumps(r, sort_keys=True, default=str).encode())
    return h.hexdigest()


def tokenize_dataset(records: list[dict], tokenizer, max_length: int, train_on: str = "last", cache_dir: str = "") -> tuple[list[dict], dict]:
    """(rows, stats). With ``cache_dir`` the rows are stored under a key of (records, tokenizer, max_length, train_on) and
    a later call with the same inputs reads them back instead of tokenizing (written to a temporary file and renamed, so
    a crash never leaves a half-written cache entry)."""
    path = None
    if cache_dir:
        os.makedirs(cache_dir, exist_ok=True)
        path = os.path.join(cache_dir, cache_key(fingerprint(records), tokenizer, max_length, train_on) + ".pkl")
        if os.path.exists(path):
            try:
                with open(path, "rb") as f:
                    rows, stats = pickle.load(f)
                stats = dict(stats, cache="hit")
                return rows, stats
            except Exception:  # noqa: BLE001 - a damaged entry is recomputed
                pass
    rows, dropped = [], 0
    for rec in records:
        row = tokenize_record(rec, tokenizer, max_length, train_on)
        if row is None:
            dropped += 1
        else:
            rows.append(row)
    lens = sorted(len(r["prompt_ids"]) + len(r["response_ids"]) for r in rows)
    pct = lambda p: lens[min(len(lens) - 1, int(p * len(lens)))] if lens else 0
    stats = {"rows": len(rows), "dropped": dropped, "tokens": sum(lens), "loss_tokens": sum(sum(r["loss_mask"]) for r in rows),
             "len_p50": pct(0.5), "len_p90": pct(0.9), "len_max": lens[-1] if lens else 0, "cache": "miss" if path else "off"}
    if path:
        fd, tmp = tempfile.mkstemp(dir=cache_dir, suffix=".tmp")
        with os.fdopen(fd, "wb") as f:
            pickle.dump((rows, stats), f)
        os.replace(tmp, path)
    return rows, stats
