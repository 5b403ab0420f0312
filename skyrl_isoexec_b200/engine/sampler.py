"""Token sampling and the rollout log-probabilities.

The log-probability reported for a sampled token is always the one of the RAW logits
(vLLM's ``raw_logprobs`` mode, which the reference forces under IsoExec,
ISO/runtimes/vllm/vllm_patches.py:388), computed by the same fixed-leaf kernel the trainer
scores with (ops/functional.token_logprobs). Temperature / top-k / top-p / min-p only shape
the distribution the token is drawn from; drawing uses the Gumbel-max trick so one
generator seed fixes the whole rollout.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops import functional as F


@dataclass
class SamplingParams:
    max_generate_length: int = 1024
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    repetition_penalty: float = 1.0     # > 1: logits of tokens seen in prompt or output are divided (if positive) or multiplied by it
    presence_penalty: float = 0.0       # subtracted once from the logit of every token generated so far
    frequency_penalty: float = 0.0      # subtracted per occurrence among the generated tokens
    min_tokens: int = 0                 # end-of-sequence and stop tokens cannot be drawn before this many tokens were generated
    logit_bias: dict | None = None      # {token id: additive bias}
    logprobs: int | None = 1
    prompt_logprobs: int | None = None  # not None: also report the log-probability of every prompt token given the tokens before it
    stop_token_ids: tuple[int, ...] = ()
    stop: tuple[str, ...] = ()          # stop strings (need a detokenizer on the engine: ``LLMEngine.detokenize``)
    ignore_eos: bool = False
    seed: int | None = None
    n: int = 1
    additional_kwargs: dict = field(default_factory=dict)

    @staticmethod
    def from_dict(d: dict | None) -> "SamplingParams":
        d = dict(d or {})
        if "max_tokens" in d:
            d["max_generate_length"] = d.pop("max_tokens")
        if "stop" in d:
            st = d.pop("stop")
            d["stop"] = () if not st else ((st,) if isinstance(st, str) else tuple(st))
        if d.get("logit_bias"):
            d["logit_bias"] = {int(k): float(v) for k, v in d["logit_bias"].items()}
        known = {k: v for k, v in d.items() if k in SamplingParams.__dataclass_fields__}
        if "stop_token_ids" in known and known["stop_token_ids"] is not None:
            known["stop_token_ids"] = tuple(known["stop_token_ids"])
        return SamplingParams(**known)


def needs_history(p: SamplingParams) -> bool:
    """Whether drawing a token for this request depends on the tokens of its own sequence (penalties, ``min_tokens``)."""
    return bool((p.repetition_penalty not in (1.0, None)) or p.presence_penalty or p.frequency_penalty or p.min_tokens > 0)


def shapes_logits(p: SamplingParams) -> bool:
    return needs_history(p) or bool(p.logit_bias)


def isoexec_sampling_constraints(p: SamplingParams) -> SamplingParams:
    """Under the execution contract the importance ratio is exactly 1 only if the behaviour policy
    is the raw model distribution: temperature 1, no truncation, no penalties or biases."""
    if p.temperature != 1.0 or p.top_p != 1.0 or p.top_k not in (-1, 0) or p.min_p != 0.0 or shapes_logits(p):
        raise ValueError("IsoExec rollouts require temperature=1.0, top_p=1.0, top_k=-1, min_p=0.0 and no penalties, min_tokens or logit_bias")
    return p


class Sampler:
    def __init__(self, device, seed: int = 0, leaves: int = F.DEFAULT_LEAVES):
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.leaves = leaves
        self.seed = int(seed)
        self.calls = 0
        self._temp_cache: dict = {}

    def reseed(self, seed: int) -> None:
        self.gen.manual_seed(seed)
        self.seed, self.calls = int(seed), 0

    def _fused(self, logits: torch.Tensor, params: list[SamplingParams]):
        """One pass over the bf16 logits (csrc/sampler.cu): Gumbel-max with counter-based noise, then the chosen tokens'
        log-probabilities from the row-invariant kernel the trainer uses."""
        from ..ops import _native

        n, V = logits.shape
        p0 = params[0]
        # the usual batch shares one parameter object: one identity pass instead of reading every request's temperature
        same = all(p is p0 for p in params)
        key = ("same", p0.temperature, n) if same else tuple(p.temperature for p in params)
        inv = self._temp_cache.get(key)
        if inv is None:
            if len(self._temp_cache) > 64:
                self._temp_cache.clear()
            temps = [p0.temperature] * n if same else [p.temperature for p in params]
            inv = torch.tensor([0.0 if t == 0.0 else 1.0 / t for t in temps], dtype=torch.float32, device=logits.device)
            self._temp_cache[key] = inv
        L = _native.lib()
        m = L.ix_sampler_scratch_elems(n)
        sv = torch.empty(m, dtype=torch.float32, device=logits.device)
        si = torch.empty(m, dtype=torch.int32, device=logits.device)
        tokens = torch.empty(n, dtype=torch.int64, device=logits.device)
        self.calls += 1
        _native.check(L.ix_sample_gumbel(logits.data_ptr(), logits.stride(0), n, V, inv.data_ptr(), self.seed & 0xFFFFFFFFFFFFFFFF,
                                         self.calls & 0xFFFFFFFF, sv.data_ptr(), si.data_ptr(), tokens.data_ptr(), _native.stream()),
                      "ix_sample_gumbel")
        logprobs, _ = F.token_logprobs(logits, tokens, self.leaves)
        return tokens, logprobs

    @staticmethod
    def _shape_row(row: torch.Tensor, p: SamplingParams, history, eos_token_id) -> torch.Tensor:
        """Penalties, bias and the ``min_tokens`` mask on one row of fp32 logits (before the temperature, as vLLM does)."""
        prompt_ids, output_ids = history if history is not None else ((), ())
        dev = row.device
        if p.repetition_penalty not in (1.0, None) and (prompt_ids or output_ids):
            seen = torch.tensor(sorted(set(prompt_ids) | set(output_ids)), dtype=torch.long, device=dev)
            v = row[seen]
            row[seen] = torch.where(v > 0, v / p.repetition_penalty, v * p.repetition_penalty)
        if (p.presence_penalty or p.frequency_penalty) and output_ids:
            ids, counts = torch.tensor(output_ids, dtype=torch.long, device=dev).unique(return_counts=True)
            row[ids] -= p.frequency_penalty * counts.to(row.dtype) + p.presence_penalty
        if p.logit_bias:
            ids = torch.tensor(list(p.logit_bias), dtype=torch.long, device=dev)
            row[ids] += torch.tensor(list(p.logit_bias.values()), dtype=row.dtype, device=dev)
        if p.min_tokens > 0 and len(output_ids) < p.min_tokens:
            stop = set(p.stop_token_ids) | ({eos_token_id} if eos_token_id is not None and not p.ignore_eos else set())
            if stop:
                row[torch.tensor(sorted(stop), dtype=torch.long, device=dev)] = float("-inf")
        return row

    @torch.no_grad()
    def __call__(self, logits: torch.Tensor, params: list[SamplingParams], histories: list | None = None, eos_token_id: int | None = None):
        """logits [n, V] -> (token ids int64 [n], raw logprobs fp32 [n]). ``histories``: per row ``(prompt ids, generated
        ids)``, needed by requests whose parameters look at their own sequence (``needs_history``)."""
        n, V = logits.shape
        p0 = params[0]
        if all(p is p0 for p in params):                     # one shared parameter object: decide once, not per request
            plain = p0.top_p >= 1.0 and p0.top_k <= 0 and p0.min_p <= 0.0 and not shapes_logits(p0)
            if plain and logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
                return self._fused(logits, params)
        shaped = [shapes_logits(p) for p in params]
        if any(needs_history(p) for p in params) and histories is None:
            raise ValueError("penalties and min_tokens need the sequences' token histories")
        untruncated = all(p.top_p >= 1.0 and p.top_k <= 0 and p.min_p <= 0.0 for p in params) and not any(shaped)
        if untruncated and logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
            return self._fused(logits, params)
        x = logits.float()
        uniform = all(p.temperature == 1.0 and p.top_p >= 1.0 and p.top_k <= 0 and p.min_p <= 0.0 for p in params) and not any(shaped)
        if not uniform:
            x = x.clone()
            for i, p in enumerate(params):
                if shaped[i]:
                    x[i] = self._shape_row(x[i], p, histories[i] if histories is not None else None, eos_token_id)
                if p.temperature == 0.0:
                    continue
                row = x[i] / p.temperature
                if p.top_k and p.top_k > 0 and p.top_k < V:
                    kth = torch.topk(row, p.top_k).values[-1]
                    row = row.masked_fill(row < kth, float("-inf"))
                if p.min_p > 0.0:
                    probs = torch.softmax(row, -1)
                    row = row.masked_fill(probs < p.min_p * probs.max(), float("-inf"))
                if p.top_p < 1.0:
                    sp, si = torch.sort(torch.softmax(row, -1), descending=True)
                    keep = (sp.cumsum(-1) - sp) < p.top_p
                    mask = torch.ones_like(row, dtype=torch.bool)
                    mask[si[keep]] = False
                    row = row.masked_fill(mask, float("-inf"))
                x[i] = row
        u = torch.rand(x.shape, device=x.device, dtype=torch.float32, generator=self.gen)
        expo = -torch.log(u.clamp_min(1e-20))          # Exp(1) samples
        gumbel = -torch.log(expo.clamp_min(1e-20))     # Gumbel(0, 1) samples
        greedy = torch.tensor([p.temperature == 0.0 for p in params], device=x.device)
        noisy = torch.where(greedy[:, None], x, x + gumbel)
        tokens = noisy.argmax(-1)
        logprobs, _ = F.token_logprobs(logits, tokens, self.leaves)
        return tokens, logprobs
