"""Reference-policy and critic workers (reference: B/workers/worker.py:1303 ``CriticWorkerBase``,
:1493 ``RefWorkerBase``).

  * ``RefWorker``    a frozen copy of the initial policy; its scoring forward gives ``base_action_log_probs`` for the
                     KL term (in the loss or in the reward). It runs the same kernels as the policy's scoring pass.
  * ``CriticWorker`` a decoder backbone with a scalar value head read at the rows that predict each response token;
                     trained with the clipped value loss; feeds GAE.
Both reuse the policy worker's packing (no padding) and micro-batching by token budget.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.decoder import DecoderLM
from . import algorithms as alg
from .batch import TrainingInputBatch
from .policy_worker import PolicyWorker, WorkerConfig, pack_microbatches


class RefWorker(PolicyWorker):
    def __init__(self, model: DecoderLM, cfg: WorkerConfig | None = None):
        self.model = model
        self.cfg = cfg or WorkerConfig()
        self.algo = alg.AlgorithmConfig()
        self.ps = model.ps
        self.device = model.device_
        self.opt = None
        for p in model.parameters():
            p.requires_grad_(False)

    @classmethod
    def from_policy(cls, policy_model: DecoderLM, cfg: WorkerConfig | None = None) -> "RefWorker":
        """A second model with the policy's CURRENT weights (taken before the first update)."""
        ref = DecoderLM(policy_model.cfg, policy_model.ps, policy_model.device_, seed=0)
        ref.store.flat.copy_(policy_model.store.flat)
        return cls(ref, cfg)

    def forward_backward(self, batch):  # pragma: no cover - a frozen model has no update
        raise RuntimeError("the reference policy is frozen")

    def optim_step(self):  # pragma: no cover
        raise RuntimeError("the reference policy is frozen")


class CriticWorker:
    def __init__(self, model: DecoderLM, cfg: WorkerConfig | None = None, algo: alg.AlgorithmConfig | None = None):
        self.model = model
        self.cfg = cfg or WorkerConfig()
        self.algo = algo or alg.AlgorithmConfig()
        self.ps, self.device = model.ps, model.device_
        # a complete policy-style worker around the backbone: packing, recompute policy, the (possibly DP-sharded) flat
        # optimizer and the TP / KV-replica / DP gradient reductions are the policy worker's own
        self._policy_like = PolicyWorker(model, self.cfg, self.algo)
        self.opt = self._policy_like.opt
        g = torch.Generator().manual_seed(1234)
        h = model.cfg.hidden_size
        self.v_weight = torch.nn.Parameter((torch.randn(h, generator=g) * (1.0 / h ** 0.5)).to(self.device))
        self.v_bias = torch.nn.Parameter(torch.zeros(1, device=self.device))
        self.head_opt = torch.optim.AdamW([self.v_weight, self.v_bias], lr=self.cfg.optimizer.lr, weight_decay=0.0)

    def _values(self, mb, hidden) -> torch.Tensor:
        rows = mb.pred_rows.to(self.device, non_blocking=True)
        h = hidden.index_select(0, rows).float()
        return h @ self.v_weight.float() + self.v_bias.float()

    @torch.no_grad()
    def forward(self, batch: TrainingInputBatch) -> torch.Tensor:
        """Values at every response position, ``[B, max_response]`` fp32 (CPU)."""
        R = batch["response_mask"].shape[1]
        seqs, att = batch["sequences"], batch["attention_mask"]
        out = torch.zeros(seqs.shape[0], R, dtype=torch.float32)
        self._policy_like.set_images(batch)
        for mb in pack_microbatches(seqs, att, R, self.cfg.max_tokens_per_microbatch):
            hidden = PolicyWorker._run_model(self._policy_like, mb, "critic_score")
            v = self._values(mb, hidden)
            flat = torch.zeros(len(mb.seq_index) * R, dtype=torch.float32, device=v.device)
            flat[mb.out_index.to(v.device)] = v
            out[torch.tensor(mb.seq_index)] = flat.view(-1, R).cpu()
        return out

    def forward_backward(self, batch: TrainingInputBatch) -> dict:
        R = batch["response_mask"].shape[1]
        seqs, att = batch["sequences"], batch["attention_mask"]
        dev = self.device
        tot_mask = float(batch["response_mask"].sum().clamp(min=1))
        if self.ps.dp > 1:
            t = torch.tensor([tot_mask], dtype=torch.float64, device=dev if dev.type == "cuda" else "cpu")
            dist.all_reduce(t, group=self.ps.dp_group)
            tot_mask = float(t)
        tot = {"loss": 0.0, "clip": 0.0, "n": 0}
        self._policy_like.set_images(batch)
        for mb in pack_microbatches(seqs, att, R, self.cfg.max_tokens_per_microbatch):
            idx = torch.tensor(mb.seq_index)
            hidden = PolicyWorker._run_model(self._policy_like, mb, "critic_fwd")
            v = self._values(mb, hidden)
            nb = len(mb.seq_index)
            v2d = torch.zeros(nb * R, dtype=torch.float32, device=dev).index_put((mb.out_index.to(dev),), v).view(nb, R)
            mask = batch["response_mask"][idx].to(dev).float()
            loss, clipfrac = alg.ppo_critic_loss(v2d, batch["values"][idx].to(dev), batch["returns"][idx].to(dev), self.algo, mask)
            # masked_mean over this micro-batch -> weight by its share of the global mask so the sum is the global mean
            (loss * (mask.sum() / tot_mask)).backward()
            tot["loss"] += float(loss.detach()) * float(mask.sum()) / tot_mask
            tot["clip"] += float(clipfrac)
            tot["n"] += 1
        return {"critic_loss": tot["loss"], "values_clip_ratio": tot["clip"] / max(1, tot["n"])}

    def optim_step(self) -> float:
        self._policy_like.reduce_gradients()          # TP sums of per-head norm weights, KV replicas, then DP
        if self.ps.dp > 1:
            for p in (self.v_weight, self.v_bias):
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.ps.dp_group)
        norm = self.opt.step(self.ps)
        self.head_opt.step()
        self.head_opt.zero_grad(set_to_none=True)
        return float(norm.item())

    # ---------------------------------------------------------------- checkpoint
    def state_dict(self) -> dict:
        """This rank's critic state: backbone shard, value head, both optimizers (reference: the ``critic/`` folder of a
        step directory, R/train/trainer.py:1858-1930)."""
        cpu = lambda t: t.detach().cpu().clone()
        return {"model": {n: cpu(t) for n, t in self.model.named_weights()},
                "optimizer": {k: (cpu(v) if torch.is_tensor(v) else v) for k, v in self.opt.state_dict().items()},
                "head": {"weight": cpu(self.v_weight), "bias": cpu(self.v_bias)}, "head_optimizer": self.head_opt.state_dict()}

    def load_state_dict(self, sd: dict) -> None:
        with torch.no_grad():
            for n, dst in self.model.named_weights():
                dst.copy_(sd["model"][n].to(dst.dtype))
            self.v_weight.copy_(sd["head"]["weight"])
            self.v_bias.copy_(sd["head"]["bias"])
        dev = self.opt.master.device
        self.opt.load_state_dict({k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in sd["optimizer"].items()})
        self.head_opt.load_state_dict(sd["head_optimizer"])
