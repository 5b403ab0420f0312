"""RL algorithm core: advantage estimators, policy / critic losses, KL estimators and
controllers, loss-reduction scaling, off-policy correction.

Semantics follow the reference (B/utils/ppo_utils.py): losses are SUMS over masked tokens and
the mean-type reductions are obtained by pre-scaling the advantages (:1080-1148); GRPO
normalises per prompt group with the unbiased std (:1271-1321); the policy loss is the PPO
clip objective with optional dual clip (:541-571). Estimators and losses are looked up by
name in two registries that user code can extend with the decorators below.

The regular / dual-clip policy loss has a fused CUDA path (csrc/loss_optim.cu) that produces
the per-token loss and its gradient in one pass; every other loss is written with torch ops.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

import torch

from ..ops import _native

# ------------------------------------------------------------------------------------ registries
ADVANTAGE_ESTIMATORS: dict[str, Callable] = {}
POLICY_LOSSES: dict[str, Callable] = {}


def register_advantage_estimator(name: str):
    def deco(fn):
        ADVANTAGE_ESTIMATORS[str(name)] = fn
        return fn
    return deco


def register_policy_loss(name: str):
    def deco(fn):
        POLICY_LOSSES[str(name)] = fn
        return fn
    return deco


def get_advantage_estimator(name: str) -> Callable:
    if name not in ADVANTAGE_ESTIMATORS:
        raise KeyError(f"unknown advantage estimator {name!r}; registered: {sorted(ADVANTAGE_ESTIMATORS)}")
    return ADVANTAGE_ESTIMATORS[name]


def get_policy_loss(name: str) -> Callable:
    if name not in POLICY_LOSSES:
        raise KeyError(f"unknown policy loss {name!r}; registered: {sorted(POLICY_LOSSES)}")
    return POLICY_LOSSES[name]


# ------------------------------------------------------------------------------------ config
@dataclass
class OffPolicyCorrection:
    tis_ratio_type: str | None = None      # None | "token" | "sequence"
    token_tis_ratio_clip_high: float = 2.0
    sequence_tis_ratio_clip_high: float = 5.0
    sequence_mask_metric: str | None = None  # None | "geometric" | "product"
    geo_mask_high: float = 1.01
    geo_mask_low: float = 0.99
    product_mask_high: float = 2.0
    product_mask_low: float = 0.5
    outlier_token_is_threshold_low: float | None = None
    outlier_token_is_threshold_high: float | None = None


@dataclass
class AlgorithmConfig:
    advantage_estimator: str = "grpo"
    policy_loss_type: str = "regular"
    loss_reduction: str = "token_mean"
    eps_clip_low: float = 0.2
    eps_clip_high: float = 0.2
    clip_ratio_c: float = 3.0
    grpo_norm_by_std: bool = True
    gamma: float = 1.0
    lambd: float = 1.0
    use_kl_loss: bool = False
    use_kl_in_reward: bool = False
    kl_loss_coef: float = 0.001
    kl_estimator_type: str = "k3"
    use_entropy_loss: bool = False
    entropy_loss_coef: float = 0.0
    value_clip: float = 0.2
    kl_ctrl_type: str = "fixed"
    kl_target: float = 0.1
    kl_horizon: int = 10000
    init_kl_coef: float = 0.001
    sapo_tau_pos: float = 1.0
    sapo_tau_neg: float = 1.05
    cispo_eps_clip_low: float = 0.0
    cispo_eps_clip_high: float = 5.0
    dppo_type: str = "binary_tv"           # binary_tv | binary_kl
    dppo_delta_low: float = 0.2
    dppo_delta_high: float = 0.2
    clip_cov_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0
    clip_cov_seed: int = 0
    kl_cov_frac: float = 0.2
    kl_cov_ppo_kl_coef: float = 1.0
    dynamic_sampling_type: str = ""        # "" | filter | replace
    dynamic_sampling_max_sample_batches: int = 30
    dynamic_sampling_min_replace_ratio: float = 0.3
    max_seq_len: int = 0
    temperature: float | None = None           # None = the rollout's sampling temperature; logprobs are taken at this temperature
    advantage_batch_normalize: bool = False    # z-score the advantages over all response tokens of the (global) batch
    zero_variance_filter: bool = False         # prompts whose samples all got the same outcome reward carry no loss
    zero_variance_filter_tol: float = 1e-6
    off_policy_correction: OffPolicyCorrection = field(default_factory=OffPolicyCorrection)


# ------------------------------------------------------------------------------------ masked stats
def masked_mean(x, mask, dim=None):
    if mask is None:
        return x.mean(dim) if dim is not None else x.mean()
    if dim is None:
        return (x * mask).sum() / mask.sum().clamp(min=1)
    return (x * mask).sum(dim) / mask.sum(dim).clamp(min=1)


def masked_var(x, mask, unbiased=True):
    mean = masked_mean(x, mask)
    var = masked_mean((x - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n == 0:
            raise ValueError("masked_var: empty mask")
        if n == 1:
            return torch.zeros_like(var)
        var = var * (n / (n - 1))
    return var


def masked_whiten(x, mask, shift_mean=True):
    mean, var = masked_mean(x, mask), masked_var(x, mask)
    w = (x - mean) * torch.rsqrt(var + 1e-8)
    return w if shift_mean else w + mean


# ------------------------------------------------------------------------------------ KL
def compute_approx_kl(log_probs, log_probs_base, loss_mask=None, kl_estimator_type: str = "k3"):
    """Per-token KL estimate between the policy and a base policy (k1 / abs / k2 / k3)."""
    lr = log_probs.float() - log_probs_base.float()
    if loss_mask is not None:
        lr = lr * loss_mask
    if kl_estimator_type == "k1":
        return lr
    if kl_estimator_type == "abs":
        return lr.abs()
    if kl_estimator_type == "k2":
        return 0.5 * lr.square()
    if kl_estimator_type == "k3":
        r = torch.clamp(-lr, min=-20, max=20)
        return torch.clamp(torch.exp(r) - r - 1, min=-10, max=10)
    raise ValueError(f"unknown KL estimator {kl_estimator_type!r}")


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current, n_steps):
        pass

    def state_dict(self):
        return {"value": self.value}

    def load_state_dict(self, sd):
        self.value = float(sd["value"])


class AdaptiveKLController:
    """Proportional controller on the observed KL (Ziegler et al.), clipped to +-20% per update."""

    def __init__(self, init_kl_coef: float, target: float, horizon: int):
        self.value, self.target, self.horizon = init_kl_coef, target, horizon

    def update(self, current, n_steps):
        err = min(max(current / self.target - 1, -0.2), 0.2)
        self.value *= 1 + err * n_steps / self.horizon

    def state_dict(self):
        return {"value": self.value}

    def load_state_dict(self, sd):
        self.value = float(sd["value"])


def get_kl_controller(cfg: AlgorithmConfig):
    if cfg.kl_ctrl_type == "fixed":
        return FixedKLController(cfg.kl_loss_coef)
    if cfg.kl_ctrl_type == "adaptive":
        return AdaptiveKLController(cfg.init_kl_coef, cfg.kl_target, cfg.kl_horizon)
    raise ValueError(f"unknown kl_ctrl_type {cfg.kl_ctrl_type!r}")


# ------------------------------------------------------------------------------------ advantage estimators
def _group_ids(index) -> torch.Tensor:
    uniq: dict = {}
    return torch.tensor([uniq.setdefault(u, len(uniq)) for u in index], dtype=torch.long)


def _group_stats(scores: torch.Tensor, gid: torch.Tensor):
    n_groups = int(gid.max().item()) + 1
    cnt = torch.zeros(n_groups, dtype=scores.dtype).index_add_(0, gid, torch.ones_like(scores))
    mean = torch.zeros(n_groups, dtype=scores.dtype).index_add_(0, gid, scores) / cnt
    sq = torch.zeros(n_groups, dtype=scores.dtype).index_add_(0, gid, (scores - mean[gid]) ** 2)
    std = torch.sqrt(sq / (cnt - 1).clamp(min=1))
    return cnt, mean, std


@register_advantage_estimator("grpo")
def grpo_advantage(token_level_rewards, response_mask, index, epsilon=1e-6, grpo_norm_by_std=True, **kw):
    """(score - group mean) / (group std + eps); a single-sample group keeps its raw score (mean 0, std 1)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(-1).float().cpu()
        gid = _group_ids(index)
        cnt, mean, std = _group_stats(scores, gid)
        single = cnt[gid] == 1
        mean_i = torch.where(single, torch.zeros_like(scores), mean[gid])
        std_i = torch.where(single, torch.ones_like(scores), std[gid])
        adv = scores - mean_i
        if grpo_norm_by_std:
            adv = adv / (std_i + epsilon)
        adv = adv.to(response_mask.device)[:, None] * response_mask
    return adv, adv


@register_advantage_estimator("rloo")
def rloo_advantage(token_level_rewards, response_mask, index, **kw):
    """Leave-one-out baseline: score - mean of the other samples of the same prompt."""
    with torch.no_grad():
        scores = token_level_rewards.sum(-1).float().cpu()
        gid = _group_ids(index)
        cnt, mean, _ = _group_stats(scores, gid)
        n = cnt[gid]
        # a group of one has no "others": its advantage is 0 (R/backends/skyrl_train/utils/ppo_utils.py:1231-1234)
        adv = torch.where(n > 1, scores * n / (n - 1).clamp(min=1) - mean[gid] * n / (n - 1).clamp(min=1), torch.zeros_like(scores))
        adv = adv.to(response_mask.device)[:, None] * response_mask
    return adv, adv


@register_advantage_estimator("no_op")
def no_op_advantage(token_level_rewards, response_mask, index=None, **kw):
    """The token-level rewards ARE the advantages (dense per-token signals such as a distillation reward)."""
    adv = (token_level_rewards * response_mask).detach()
    return adv, adv


@register_advantage_estimator("maxrl")
def maxrl_advantage(token_level_rewards, response_mask, index, epsilon=1e-6, **kw):
    """(score - group mean) / (group mean + eps)."""
    with torch.no_grad():
        scores = token_level_rewards.sum(-1).float().cpu()
        gid = _group_ids(index)
        cnt, mean, _ = _group_stats(scores, gid)
        multi = cnt[gid] > 1
        adv = torch.where(multi, (scores - mean[gid]) / (mean[gid] + epsilon), scores)
        adv = adv.to(response_mask.device)[:, None] * response_mask
    return adv, adv


@register_advantage_estimator("reinforce++")
def reinforce_pp_advantage(token_level_rewards, response_mask, gamma=1.0, **kw):
    with torch.no_grad():
        returns = torch.zeros_like(token_level_rewards)
        run = torch.zeros_like(token_level_rewards[:, 0])
        for t in reversed(range(token_level_rewards.shape[1])):
            run = token_level_rewards[:, t] + gamma * run
            returns[:, t] = run
            run = run * response_mask[:, t]
        adv = masked_whiten(returns, response_mask) * response_mask
    return adv, returns


@register_advantage_estimator("gae")
def gae_advantage(token_level_rewards, response_mask, values, gamma=1.0, lambd=1.0, **kw):
    with torch.no_grad():
        T = token_level_rewards.shape[1]
        last = torch.zeros_like(token_level_rewards[:, 0])
        adv_rev = []
        for t in reversed(range(T)):
            nxt = values[:, t + 1] if t < T - 1 else torch.zeros_like(last)
            delta = token_level_rewards[:, t] + gamma * nxt - values[:, t]
            last = delta + gamma * lambd * last
            adv_rev.append(last)
        adv = torch.stack(adv_rev[::-1], dim=1)
        returns = adv + values
        adv = masked_whiten(adv, response_mask)
    return adv, returns


def compute_advantages_and_returns(token_level_rewards, response_mask, index, adv_estimator: str,
                                   cfg: AlgorithmConfig, values=None):
    fn = get_advantage_estimator(adv_estimator)
    return fn(token_level_rewards=token_level_rewards, response_mask=response_mask, index=index, values=values,
              gamma=cfg.gamma, lambd=cfg.lambd, grpo_norm_by_std=cfg.grpo_norm_by_std)


# ------------------------------------------------------------------------------------ loss reduction (by advantage scaling)
def apply_loss_reduction_to_advantages(advantages, loss_mask, loss_reduction: str, micro_batch_size: int = 0,
                                       max_seq_len: int = 0, prompt_boundaries=None, total_scale: float = 1.0):
    """Scale advantages so that SUMMING the token losses of a mini-batch yields the named mean."""
    B = advantages.shape[0]
    if loss_reduction == "token_mean":
        out = advantages / loss_mask.sum().clamp(min=1)
    elif loss_reduction == "token_mean_legacy":
        out = torch.zeros_like(advantages)
        nmb = max(1, B // max(1, micro_batch_size))
        for i in range(nmb):
            sl = slice(i * micro_batch_size, (i + 1) * micro_batch_size)
            out[sl] = advantages[sl] / loss_mask[sl].sum().clamp(min=1) / nmb
    elif loss_reduction == "sequence_mean":
        out = advantages / (B * loss_mask.sum(-1, keepdim=True).clamp(min=1))
    elif loss_reduction == "seq_mean_token_sum_norm":
        out = advantages / (B * max_seq_len)
    elif loss_reduction == "prompt_mean":
        if prompt_boundaries is None:
            raise ValueError("prompt_mean loss reduction requires prompt_boundaries")
        out = torch.zeros_like(advantages)
        for lo, hi in prompt_boundaries:
            out[lo:hi] = advantages[lo:hi] / (len(prompt_boundaries) * loss_mask[lo:hi].sum().clamp(min=1))
    else:
        raise ValueError(f"invalid loss reduction {loss_reduction!r}")
    return out * total_scale


# ------------------------------------------------------------------------------------ off-policy correction
def compute_off_policy_correction(old_log_probs, rollout_logprobs, loss_mask, opc: OffPolicyCorrection):
    """Truncated importance sampling weights and sequence / outlier masks from the gap between
    the trainer's old logprobs and the rollout engine's. Returns (weights|None, new_mask, metrics)."""
    metrics: dict[str, float] = {}
    if rollout_logprobs is None or (opc.tis_ratio_type is None and opc.sequence_mask_metric is None
                                    and opc.outlier_token_is_threshold_low is None
                                    and opc.outlier_token_is_threshold_high is None):
        return None, loss_mask, metrics
    with torch.no_grad():
        lr = (old_log_probs.float() - rollout_logprobs.float()) * loss_mask
        weights = None
        if opc.tis_ratio_type == "token":
            weights = torch.exp(lr).clamp(max=opc.token_tis_ratio_clip_high)
        elif opc.tis_ratio_type == "sequence":
            weights = torch.exp(lr.sum(-1, keepdim=True)).clamp(max=opc.sequence_tis_ratio_clip_high).expand_as(lr)
        mask = loss_mask
        if opc.sequence_mask_metric == "geometric":
            geo = torch.exp(lr.sum(-1) / loss_mask.sum(-1).clamp(min=1))
            keep = (geo <= opc.geo_mask_high) & (geo >= opc.geo_mask_low)
            mask = mask * keep[:, None]
        elif opc.sequence_mask_metric == "product":
            prod = torch.exp(lr.sum(-1))
            keep = (prod <= opc.product_mask_high) & (prod >= opc.product_mask_low)
            mask = mask * keep[:, None]
        if opc.outlier_token_is_threshold_low is not None or opc.outlier_token_is_threshold_high is not None:
            r = torch.exp(lr)
            bad = torch.zeros_like(r, dtype=torch.bool)
            if opc.outlier_token_is_threshold_low is not None:
                bad |= r < opc.outlier_token_is_threshold_low
            if opc.outlier_token_is_threshold_high is not None:
                bad |= r > opc.outlier_token_is_threshold_high
            keep = ~((bad & (loss_mask > 0)).any(-1))
            mask = mask * keep[:, None]
        if weights is not None:
            metrics["tis_weight_mean"] = masked_mean(weights, loss_mask).item()
        metrics["off_policy_masked_frac"] = 1.0 - (mask.sum() / loss_mask.sum().clamp(min=1)).item()
    return weights, mask, metrics


# ------------------------------------------------------------------------------------ policy losses
_KL_KIND = {"k1": 0, "abs": 1, "k2": 2, "k3": 3}


class _FusedPPOLoss(torch.autograd.Function):
    """Per-token PPO loss + gradient from one CUDA kernel; backward only rescales the stored gradient."""

    @staticmethod
    def forward(ctx, log_probs, old, adv, mask, tis, eps_lo, eps_hi, clip_c, dual):
        n = log_probs.numel()
        lp = log_probs.contiguous().float()
        loss = torch.empty_like(lp)
        grad = torch.empty_like(lp)
        clip = torch.empty_like(lp)
        L = _native.lib()
        _native.check(L.ix_ppo_loss(lp.data_ptr(), old.contiguous().float().data_ptr(), adv.contiguous().float().data_ptr(),
                                    mask.contiguous().float().data_ptr(), None,
                                    None if tis is None else tis.contiguous().float().data_ptr(), loss.data_ptr(),
                                    grad.data_ptr(), clip.data_ptr(), None, n, eps_lo, eps_hi, clip_c, int(dual), 0.0, 3,
                                    _native.stream()), "ix_ppo_loss")
        ctx.save_for_backward(grad)
        ctx.mark_non_differentiable(clip)
        return loss, clip

    @staticmethod
    def backward(ctx, g_loss, _g_clip):
        (grad,) = ctx.saved_tensors
        return (g_loss * grad).to(g_loss.dtype), None, None, None, None, None, None, None, None


def _ppo_clip(log_probs, old_log_probs, advantages, cfg: AlgorithmConfig, loss_mask, rollout_logprobs, dual: bool):
    weights, mask, metrics = compute_off_policy_correction(old_log_probs, rollout_logprobs, loss_mask,
                                                           cfg.off_policy_correction)
    if log_probs.is_cuda:
        loss_tok, clip_tok = _FusedPPOLoss.apply(log_probs, old_log_probs, advantages, mask, weights,
                                                 cfg.eps_clip_low, cfg.eps_clip_high, cfg.clip_ratio_c, dual)
        loss = loss_tok.sum()
        metrics["clip_ratio"] = (clip_tok.sum() / mask.sum().clamp(min=1)).detach()
        return loss, metrics
    ratio = torch.exp(torch.clamp(log_probs - old_log_probs, -20.0, 20.0))
    l1 = -advantages * ratio
    l2 = -advantages * ratio.clamp(1 - cfg.eps_clip_low, 1 + cfg.eps_clip_high)
    loss = torch.max(l1, l2)
    clipped = (l2 > l1).float()
    if dual:
        l3 = -advantages * cfg.clip_ratio_c
        use3 = (advantages < 0) & (l3 < loss)
        loss = torch.where(use3, l3, loss)
        clipped = torch.where(use3, torch.ones_like(clipped), clipped)
    if weights is not None:
        loss = loss * weights
    metrics["clip_ratio"] = masked_mean(clipped, mask).detach()
    return (loss * mask).sum(), metrics


@register_policy_loss("regular")
def ppo_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    return _ppo_clip(log_probs, old_log_probs, advantages, cfg, loss_mask, rollout_logprobs, dual=False)


@register_policy_loss("dual_clip")
def dual_clip_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    return _ppo_clip(log_probs, old_log_probs, advantages, cfg, loss_mask, rollout_logprobs, dual=True)


def _finish(loss, old_log_probs, rollout_logprobs, loss_mask, cfg, metrics):
    weights, mask, m2 = compute_off_policy_correction(old_log_probs, rollout_logprobs, loss_mask, cfg.off_policy_correction)
    if weights is not None:
        loss = loss * weights
    metrics.update(m2)
    return (loss * mask).sum(), metrics


@register_policy_loss("sapo")
def sapo_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Soft adaptive gate sigma(tau (r - 1)) * 4 / tau instead of a hard clip."""
    ratio = torch.exp(torch.clamp(log_probs - old_log_probs, -20.0, 20.0))
    tau = torch.where(advantages > 0, torch.full_like(advantages, cfg.sapo_tau_pos),
                      torch.full_like(advantages, cfg.sapo_tau_neg))
    gates = torch.sigmoid(tau * (ratio - 1.0)) * (4.0 / tau)
    return _finish(-gates * advantages, old_log_probs, rollout_logprobs, loss_mask, cfg, {"clip_ratio": 0.0})


@register_policy_loss("gspo")
def gspo_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Sequence-level importance weight (mean token log-ratio) applied to every token (GSPO-token)."""
    log_w = masked_mean(log_probs - old_log_probs, loss_mask, dim=-1).unsqueeze(-1)
    ratio = torch.exp(torch.clamp(log_probs - log_probs.detach() + log_w.detach(), max=10))
    s1 = ratio * advantages
    s2 = ratio.clamp(1 - cfg.eps_clip_low, 1 + cfg.eps_clip_high) * advantages
    metrics = {"clip_ratio": masked_mean((-s2 > -s1).float(), loss_mask).detach()}
    return _finish(-torch.min(s1, s2), old_log_probs, rollout_logprobs, loss_mask, cfg, metrics)


@register_policy_loss("cispo")
def cispo_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Clip the importance weight in the gradient coefficient, not in the objective."""
    ratio = torch.exp(torch.clamp(log_probs - old_log_probs, -20.0, 20.0))
    lo, hi = 1 - cfg.cispo_eps_clip_low, 1 + cfg.cispo_eps_clip_high
    loss = -advantages * ratio.clamp(lo, hi).detach() * log_probs
    metrics = {"clip_ratio": masked_mean(((ratio < lo) | (ratio > hi)).float(), loss_mask).detach()}
    return _finish(loss, old_log_probs, rollout_logprobs, loss_mask, cfg, metrics)


@register_policy_loss("rollout_is")
def rollout_is_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """CISPO against the ROLLOUT distribution, with a hard zero outside (1-eps_low, 1+eps_high): usable when
    the trainer's own old logprobs do not exist (asynchronous training).
    Reference: B/utils/ppo_utils.py:752-792."""
    if rollout_logprobs is None:
        raise ValueError("rollout_is needs the rollout logprobs")
    ratio = torch.exp(torch.clamp(log_probs - rollout_logprobs, -20.0, 20.0))
    keep = (ratio > 1 - cfg.eps_clip_low) & (ratio < 1 + cfg.eps_clip_high)
    coef = torch.where(keep, ratio, torch.zeros_like(ratio)).detach()
    metrics = {"clip_ratio": masked_mean((~keep).float(), loss_mask).detach()}
    return _finish(-coef * advantages * log_probs, old_log_probs, rollout_logprobs, loss_mask, cfg, metrics)


@register_policy_loss("dppo")
def dppo_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Divergence-proximal PPO: a token leaves the objective when moving its PROBABILITY further in the
    direction the advantage asks for would exceed a divergence budget (binary total-variation or binary KL
    between behaviour and current token probability). Reference: B/utils/ppo_utils.py:794-864."""
    mu = rollout_logprobs if rollout_logprobs is not None else old_log_probs
    ratio = torch.exp(torch.clamp(log_probs - mu, -20.0, 20.0))
    with torch.no_grad():
        p, q = torch.exp(log_probs), torch.exp(mu)
        diff = p - q
        up, down = advantages > 0, advantages < 0
        if cfg.dppo_type == "binary_tv":
            drop = (up & (diff > cfg.dppo_delta_high)) | (down & (-diff > cfg.dppo_delta_low))
        elif cfg.dppo_type == "binary_kl":
            eps = 1e-8
            bkl = q * (mu - log_probs) + (1 - q) * torch.log((1 - q + eps) / (1 - p + eps))
            drop = (up & (diff > 0) & (bkl > cfg.dppo_delta_high)) | (down & (diff < 0) & (bkl > cfg.dppo_delta_low))
        else:
            raise ValueError(f"unknown dppo_type {cfg.dppo_type!r} (binary_tv | binary_kl)")
        keep = (~drop).to(ratio.dtype)
    metrics = {"clip_ratio": masked_mean(1.0 - keep, loss_mask).detach()}
    return _finish(-ratio * advantages * keep, old_log_probs, rollout_logprobs, loss_mask, cfg, metrics)


def _token_covariance(log_probs, advantages, loss_mask):
    return (advantages - masked_mean(advantages, loss_mask)) * (log_probs.detach() - masked_mean(log_probs.detach(), loss_mask))


@register_policy_loss("clip_cov")
def clip_cov_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """PPO clip plus covariance clipping: among tokens the ratio clip left alone, a random sample (a fixed
    fraction of the batch) of those whose advantage/logprob covariance lies in [lb, ub] is detached from
    the objective. The sample is drawn from a generator seeded by ``cfg.clip_cov_seed`` so DP ranks and
    re-runs agree. Reference: B/utils/ppo_utils.py:866-927."""
    ratio = torch.exp(log_probs - old_log_probs)
    l1 = -advantages * ratio
    l2 = -advantages * ratio.clamp(1 - cfg.eps_clip_low, 1 + cfg.eps_clip_high)
    valid = loss_mask > 0
    clipped = (l2 > l1) & valid
    cov = _token_covariance(log_probs, advantages, loss_mask)
    cand = valid & ~clipped & (cov > cfg.clip_cov_lb) & (cov < cfg.clip_cov_ub)
    budget = max(1, int(cfg.clip_cov_ratio * float(loss_mask.sum())))
    flat = torch.nonzero(cand.reshape(-1)).squeeze(-1)
    corr = torch.ones_like(advantages).reshape(-1)
    if flat.numel():
        g = torch.Generator().manual_seed(int(cfg.clip_cov_seed))
        pick = flat[torch.randperm(flat.numel(), generator=g)[:budget].to(flat.device)]
        corr[pick] = 0.0
    corr = corr.view_as(advantages)
    metrics = {"clip_ratio": masked_mean((corr == 0).float(), loss_mask).detach()}
    return (torch.maximum(l1, l2) * corr * loss_mask).sum(), metrics


@register_policy_loss("kl_cov")
def kl_cov_policy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Unclipped policy gradient, with a |log ratio| penalty on the ``kl_cov_frac`` of tokens whose
    advantage/logprob covariance is largest. Reference: B/utils/ppo_utils.py:929-982."""
    delta = log_probs - old_log_probs
    base = -advantages * torch.exp(delta)
    valid = loss_mask > 0
    n = int(valid.sum())
    if n == 0:
        return (base * loss_mask).sum(), {"clip_ratio": 0.0}
    cov = _token_covariance(log_probs, advantages, loss_mask).masked_fill(~valid, float("-inf")).reshape(-1)
    k = max(1, min(n, int(n * cfg.kl_cov_frac)))
    top = torch.topk(cov, k, largest=True).indices
    pen = torch.zeros_like(cov)
    pen[top] = 1.0
    loss = base + cfg.kl_cov_ppo_kl_coef * delta.abs() * pen.view_as(base)
    return (loss * loss_mask).sum(), {"clip_ratio": 0.0}


@register_policy_loss("cross_entropy")
def cross_entropy_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Negative log-likelihood of the masked tokens (SFT through the RL path)."""
    return (-log_probs * loss_mask).sum(), {"clip_ratio": 0.0}


@register_policy_loss("importance_sampling")
def importance_sampling_loss(log_probs, old_log_probs, advantages, cfg, loss_mask=None, rollout_logprobs=None):
    """Unclipped importance-weighted policy gradient against the rollout distribution."""
    base = rollout_logprobs if rollout_logprobs is not None else old_log_probs
    ratio = torch.exp(torch.clamp(log_probs - base, -20.0, 20.0))
    return (-ratio * advantages * loss_mask).sum(), {"clip_ratio": 0.0}


def ppo_critic_loss(values, old_values, returns, cfg: AlgorithmConfig, loss_mask=None):
    """Clipped value loss 0.5 * max((v - R)^2, (clip(v) - R)^2)."""
    if cfg.value_clip is not None:
        vc = old_values + (values - old_values).clamp(-cfg.value_clip, cfg.value_clip)
        loss = torch.max((vc - returns) ** 2, (values - returns) ** 2)
        clipfrac = masked_mean(((vc - returns) ** 2 > (values - returns) ** 2).float(), loss_mask).detach()
    else:
        loss = (values - returns) ** 2
        clipfrac = torch.zeros(())
    return 0.5 * masked_mean(loss, loss_mask), clipfrac
