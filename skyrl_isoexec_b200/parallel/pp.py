"""Pipeline parallelism for the trainer: contiguous layer ranges per stage, activations and their
gradients travel between neighbouring stages by point-to-point send/recv (NCCL on GPUs, gloo on CPU),
micro-batches follow the one-forward-one-backward (1F1B) schedule.

The reference delegates this to Megatron's ``get_forward_backward_func`` (B/workers/megatron/
megatron_model_wrapper.py:205,383) and pins PP = 1 under the execution contract (ISO/models/qwen3_5.py:68);
here too the contract refuses PP > 1 for the bitwise path, and this module serves ordinary (non-gated) training.

What crosses a stage boundary is the (x, residual) pair of the residual stream, two ``[tokens, hidden]`` tensors.
Every stage packs the same micro-batches from the same batch (the data-parallel shard is replicated over the
pipeline ranks), so shapes are known without a handshake. The last stage owns final norm, LM head and loss.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.decoder import DecoderLM, ForwardCtx
from ..ops import functional as F
from ..train import algorithms as alg
from ..train.batch import TrainingInputBatch
from ..train.policy_worker import PolicyWorker, WorkerConfig, lm_head_logprobs, pack_microbatches


def stage_layers(num_layers: int, pp: int, pp_rank: int) -> range:
    """Contiguous, as even as possible; earlier stages get the extra layers."""
    base, extra = divmod(num_layers, pp)
    lo = pp_rank * base + min(pp_rank, extra)
    return range(lo, lo + base + (1 if pp_rank < extra else 0))


def build_stage_model(cfg, ps, device, seed: int = 0) -> DecoderLM:
    return DecoderLM(cfg, ps, device, seed=seed, layer_range=stage_layers(cfg.num_layers, ps.pp, ps.pp_rank))


class _P2P:
    def __init__(self, ps, device, dtype, hidden):
        self.ps, self.device, self.dtype, self.hidden = ps, device, dtype, hidden
        self.prev = ps.pp_ranks[ps.pp_rank - 1] if not ps.is_first_pp else None
        self.next = ps.pp_ranks[ps.pp_rank + 1] if not ps.is_last_pp else None
        self.pending: list = []

    def _pair(self, T):
        return torch.empty(2, T, self.hidden, dtype=self.dtype, device=self.device)

    def send(self, x, res, dst):
        """Non-blocking: in 1F1B a stage sends activations forward while its neighbour sends gradients back, and two
        blocking sends facing each other would never complete. ``drain`` waits for everything issued."""
        buf = torch.stack([x, res]).contiguous()
        self.pending.append((dist.isend(buf, dst), buf))

    def drain(self):
        for work, _buf in self.pending:
            work.wait()
        self.pending.clear()

    def recv(self, T, src):
        buf = self._pair(T)
        dist.recv(buf, src)
        return buf[0], buf[1]


class PipelinePolicyWorker(PolicyWorker):
    """Same verbs as ``PolicyWorker``; every pipeline rank calls them with the same batch. Log-probabilities and
    loss metrics are valid on the last stage and broadcast to the others."""

    def __init__(self, model: DecoderLM, cfg: WorkerConfig | None = None, algo=None):
        super().__init__(model, cfg, algo)
        assert self.ps.pp > 1
        self.p2p = _P2P(self.ps, self.device, model.cfg.torch_dtype, model.cfg.hidden_size)

    # ------------------------------------------------------------------ one micro-batch through this stage
    def _stage_forward(self, mb, site: str, hidden_in):
        dev = self.device
        fc = ForwardCtx(positions=mb.positions.to(dev), meta=F.AttnMeta.packed(mb.seq_lens, self.model.hq, self.model.hkv, dev), site=site)
        if self.model.cfg.has_gdn:
            from ..ops.gdn import GDNMeta

            fc.gdn_meta = GDNMeta.packed(mb.seq_lens, dev)
        ids = mb.ids.to(dev) if self.ps.is_first_pp else None
        return self.model(ids, fc, hidden_in=hidden_in, checkpoint_layers=self._ckpt_arg())

    def reduce_gradients(self) -> None:
        """A tied embedding lives on every stage (input on the first, LM head on the last): its gradient is their sum."""
        if self.model.cfg.tie_embeddings:
            s = self.model.store.specs["embed.weight"]
            n = 1
            for d in s.shape:
                n *= d
            dist.all_reduce(self.opt.main_grad[s.offset:s.offset + n], group=self.ps.pp_group)
        super().reduce_gradients()

    def _bcast_from_last(self, t: torch.Tensor) -> torch.Tensor:
        dist.broadcast(t, src=self.ps.pp_ranks[-1], group=self.ps.pp_group)
        return t

    # ------------------------------------------------------------------ scoring: forward-only pipeline
    @torch.no_grad()
    def forward(self, batch: TrainingInputBatch) -> torch.Tensor:
        R = batch["response_mask"].shape[1]
        out = torch.zeros(batch["sequences"].shape[0], R, dtype=torch.float32)
        for mb in pack_microbatches(batch["sequences"], batch["attention_mask"], R, self.cfg.max_tokens_per_microbatch):
            T = int(mb.ids.numel())
            hin = None if self.ps.is_first_pp else self.p2p.recv(T, self.p2p.prev)
            y = self._stage_forward(mb, "trainer_score", hin)
            if not self.ps.is_last_pp:
                x, res = y
                self.p2p.send(x, res if res is not None else torch.zeros_like(x), self.p2p.next)
            else:
                lp, _, _ = self._logprobs(mb, y, False)
                flat = torch.zeros(len(mb.seq_index) * R, dtype=torch.float32, device=lp.device)
                flat[mb.out_index.to(lp.device)] = lp
                out[torch.tensor(mb.seq_index)] = flat.view(-1, R).cpu()
        self.p2p.drain()
        dev_out = out.to(self.device)
        return self._bcast_from_last(dev_out).cpu()

    # ------------------------------------------------------------------ training: 1F1B
    def forward_backward(self, batch: TrainingInputBatch) -> dict:
        algo, ps = self.algo, self.ps
        R = batch["response_mask"].shape[1]
        mbs = pack_microbatches(batch["sequences"], batch["attention_mask"], R, self.cfg.max_tokens_per_microbatch)
        loss_fn = alg.get_policy_loss(algo.policy_loss_type)
        n_mb, dev = len(mbs), self.device
        warm = min(ps.pp - ps.pp_rank - 1, n_mb)
        live: list = []                  # per in-flight micro-batch: (inputs needing grad, outputs)
        tot = {"loss": 0.0, "tokens": 0.0, "clip_num": 0.0}

        def fwd(i):
            mb = mbs[i]
            T = int(mb.ids.numel())
            hin = None
            if not ps.is_first_pp:
                x, res = self.p2p.recv(T, self.p2p.prev)
                hin = (x.requires_grad_(), res.requires_grad_())
            y = self._stage_forward(mb, "trainer_fwd", hin)
            if ps.is_last_pp:
                lp_flat, _ = lm_head_logprobs(self.model, y.index_select(0, mb.pred_rows.to(dev)), mb.targets.to(dev),
                                              self.cfg.logprob_chunk_rows, False)
                nb, idx = len(mb.seq_index), torch.tensor(mb.seq_index)
                lp2d = torch.zeros(nb * R, dtype=torch.float32, device=dev).index_put((mb.out_index.to(dev),), lp_flat).view(nb, R)
                get = lambda k: (batch[k][idx].to(dev).float() if batch.get(k) is not None else None)  # noqa: E731
                mask = get("loss_mask") if batch.get("loss_mask") is not None else get("response_mask")
                old = get("action_log_probs")
                loss, m = loss_fn(lp2d, old if old is not None else lp2d.detach(), get("advantages"), algo, loss_mask=mask,
                                  rollout_logprobs=get("rollout_logprobs"))
                tot["loss"] += float(loss.detach())
                tot["tokens"] += float(mask.sum())
                tot["clip_num"] += float(m.get("clip_ratio", 0.0)) * float(mask.sum())
                live.append((hin, loss))
            else:
                x, res = y
                self.p2p.send(x.detach(), res.detach() if res is not None else torch.zeros_like(x), self.p2p.next)
                live.append((hin, (x, res)))

        def bwd():
            hin, out = live.pop(0)
            if ps.is_last_pp:
                out.backward()
            else:
                x, res = out
                gx, gres = self.p2p.recv(x.shape[0], self.p2p.next)
                torch.autograd.backward([x] + ([res] if res is not None else []), [gx] + ([gres] if res is not None else []))
            if hin is not None:
                gx = hin[0].grad if hin[0].grad is not None else torch.zeros_like(hin[0])
                gr = hin[1].grad if hin[1].grad is not None else torch.zeros_like(hin[1])
                self.p2p.send(gx, gr, self.p2p.prev)

        i = 0
        for _ in range(warm):                # warm-up: fill the pipeline
            fwd(i)
            i += 1
        for _ in range(n_mb - warm):         # steady state: one forward, one backward
            fwd(i)
            i += 1
            bwd()
        for _ in range(warm):                # cool-down: drain
            bwd()
        self.p2p.drain()
        stats = torch.tensor([tot["loss"], tot["tokens"], tot["clip_num"]], dtype=torch.float64, device=dev)
        self._bcast_from_last(stats)
        n = max(1.0, float(stats[1]))
        return {"policy_loss": float(stats[0]), "ppo_clip_ratio": float(stats[2]) / n, "loss_tokens": float(stats[1]),
                "policy_entropy": 0.0, "policy_kl": 0.0}
