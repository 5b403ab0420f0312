"""LoRA adapters over the flat-parameter model and a multi-tenant adapter store (reference:
B/workers/megatron/adapter_store.py multi-tenant LoRA; R/tx/layers/lora.py).

The model computes with ONE weight buffer (shared with the colocated engine), so an adapter is applied by merging
``W += (alpha / r) * B @ A`` into the target weights and removed by restoring the saved base rows exactly; the
engine needs no LoRA-aware kernel and rollouts under an adapter stay bitwise equal to the trainer's scoring.
Training an adapter: the base weights are frozen; the dense weight gradient dW that the backward already
produces is projected onto the factors, dA = (alpha/r) * B^T dW, dB = (alpha/r) * dW A^T, and only A, B step.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

DEFAULT_TARGETS = ("attn.qkv.weight", "attn.q_b.weight", "attn.kv_b.weight", "attn.o.weight", "mlp.gate_up.weight", "mlp.down.weight")


@dataclass
class LoRAConfig:
    rank: int = 8
    alpha: float = 16.0
    targets: tuple = DEFAULT_TARGETS
    lr: float = 1e-4
    seed: int = 0


@dataclass
class LoRAAdapter:
    cfg: LoRAConfig
    A: dict = field(default_factory=dict)     # name -> [r, in]   (fp32)
    B: dict = field(default_factory=dict)     # name -> [out, r]  (fp32, zeros at init: the adapter starts as a no-op)

    @property
    def scale(self) -> float:
        return self.cfg.alpha / self.cfg.rank

    @staticmethod
    def init(model, cfg: LoRAConfig) -> "LoRAAdapter":
        ad = LoRAAdapter(cfg)
        g = torch.Generator().manual_seed(cfg.seed)
        for name, w in model.named_weights():
            if w.dim() == 2 and name.endswith(tuple(cfg.targets)):
                out, inn = w.shape
                ad.A[name] = (torch.randn(cfg.rank, inn, generator=g) / math.sqrt(inn)).to(w.device)
                ad.B[name] = torch.zeros(out, cfg.rank, device=w.device)
        if not ad.A:
            raise ValueError(f"no parameter matches the LoRA targets {cfg.targets}")
        return ad

    def delta(self, name: str) -> torch.Tensor:
        return self.scale * (self.B[name] @ self.A[name])

    def num_parameters(self) -> int:
        return sum(a.numel() + b.numel() for a, b in zip(self.A.values(), self.B.values()))

    def state_dict(self) -> dict:
        return {"cfg": vars(self.cfg), "A": {k: v.cpu() for k, v in self.A.items()}, "B": {k: v.cpu() for k, v in self.B.items()}}

    @staticmethod
    def from_state_dict(sd: dict, device="cpu") -> "LoRAAdapter":
        ad = LoRAAdapter(LoRAConfig(**{**sd["cfg"], "targets": tuple(sd["cfg"]["targets"])}))
        ad.A = {k: v.to(device) for k, v in sd["A"].items()}
        ad.B = {k: v.to(device) for k, v in sd["B"].items()}
        return ad


class AdapterStore:
    """Named adapters for one base model; at most one is merged into the weights at a time."""

    def __init__(self, model):
        self.model = model
        self.adapters: dict[str, LoRAAdapter] = {}
        self.active: str | None = None
        self._base: dict[str, torch.Tensor] = {}

    def register(self, tenant: str, adapter: LoRAAdapter) -> None:
        if tenant in self.adapters:
            raise ValueError(f"adapter {tenant!r} already registered")
        self.adapters[tenant] = adapter

    def remove(self, tenant: str) -> None:
        if self.active == tenant:
            self.deactivate()
        del self.adapters[tenant]

    @torch.no_grad()
    def activate(self, tenant: str) -> None:
        """Merge ``tenant``'s delta into the model weights (after un-merging whichever adapter was active)."""
        if self.active == tenant:
            return
        self.deactivate()
        ad = self.adapters[tenant]
        views = dict(self.model.named_weights())
        for name in ad.A:
            w = views[name]
            self._base[name] = w.detach().clone()
            w.copy_((w.float() + ad.delta(name).to(w.device)).to(w.dtype))
        self.active = tenant

    @torch.no_grad()
    def deactivate(self) -> None:
        """Restore the base weights bit for bit."""
        if self.active is None:
            return
        views = dict(self.model.named_weights())
        for name, base in self._base.items():
            views[name].copy_(base)
        self._base.clear()
        self.active = None

    @torch.no_grad()
    def refresh(self) -> None:
        """Re-merge the active adapter after its factors changed (an optimizer step)."""
        t = self.active
        if t is not None:
            self.deactivate()
            self.activate(t)


class LoRATrainer:
    """Adam on the factors of one adapter, fed by the dense main gradients of a ``PolicyWorker``."""

    def __init__(self, worker, store: AdapterStore, tenant: str):
        self.worker, self.store, self.tenant = worker, store, tenant
        self.ad = store.adapters[tenant]
        params = []
        for name in self.ad.A:
            self.ad.A[name].requires_grad_(False)
            self.ad.B[name].requires_grad_(False)
            params += [self.ad.A[name], self.ad.B[name]]
        self.opt = torch.optim.Adam(params, lr=self.ad.cfg.lr)

    @torch.no_grad()
    def optim_step(self) -> float:
        """Project the accumulated dense gradients onto (A, B), step them, re-merge; the base weights never move."""
        model, opt = self.worker.model, self.worker.opt
        sq = 0.0
        for name in self.ad.A:
            s = model.store.specs[name]
            n = 1
            for d in s.shape:
                n *= d
            dW = opt.main_grad[s.offset:s.offset + n].view(s.shape).float()
            A, B = self.ad.A[name], self.ad.B[name]
            A.grad = self.ad.scale * (B.t() @ dW)
            B.grad = self.ad.scale * (dW @ A.t())
            sq += float(A.grad.square().sum() + B.grad.square().sum())
        self.opt.step()
        opt.zero_grad()
        self.store.refresh()
        return math.sqrt(sq)
