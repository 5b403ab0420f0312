"""Trainer-side worker: owns the policy model, its flat optimizer state and the three verbs
the controller drives (``forward`` for scoring, ``forward_backward`` per mini-batch,
``optim_step``), like the reference's ``PolicyWorkerBase`` (B/workers/worker.py:776-1073) and
its Megatron wrapper (B/workers/megatron/megatron_model_wrapper.py:185-711) - without Megatron:
padding is removed and sequences are packed back to back, micro-batches are cut by a token
budget, and the LM head + log-softmax run chunked and are recomputed in the backward so a
[tokens, vocab] tensor is never kept alive.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..models.decoder import DecoderLM, ForwardCtx
from ..ops import _native
from ..ops import functional as F
from ..parallel.state import ParallelState
from . import algorithms as alg
from .batch import TrainingInputBatch


@dataclass
class OptimizerConfig:
    lr: float = 1e-6
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    num_warmup_steps: int = 0
    scheduler: str = "constant_with_warmup"  # | "cosine" | "linear"
    total_steps: int = 0
    min_lr_ratio: float = 0.0


@dataclass
class WorkerConfig:
    max_tokens_per_microbatch: int = 8192
    logprob_chunk_rows: int = 8192
    freeze_moe_router: bool = False    # the routers' weights (and selection biases) are put back after every optimizer step
    moe_aux_loss_coeff: float = 0.0    # > 0: every MoE layer's load-balancing term enters the gradient with this weight (ops/moe.py)
    temperature: float = 1.0           # != 1: logprobs of the distribution the rollout sampled from, softmax(logits / T): the rows
                                       # entering the LM head are divided by T (no contract run: that pins T = 1)
    checkpoint_layers: bool = True
    keep_last_layers: int = 0          # do not recompute the last n layers (trades activation memory for one forward of
                                       # them); -1 = as many as the free HBM allows (only with a sharded optimizer)
    want_entropy: bool = False
    overlap_grad_reduce: bool = True   # sum gradient buckets over DP during the last micro-batch's backward
    shard_optimizer: bool = True       # fp32 master weights and Adam moments are cut over the data-parallel group
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)


# ------------------------------------------------------------------------------------ LM head + logprob (chunked, recomputed)
class _LMHeadLogprob(torch.autograd.Function):
    """logprob/entropy of ``targets`` from hidden rows, one vocabulary GEMM chunk at a time.
    Saves only the hidden rows and the per-row lse; the backward recomputes each logits chunk,
    turns it into d(logits) in place and feeds the NN / TN gradient GEMMs."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, leaves, chunk, want_entropy):
        n = hidden.shape[0]
        lp = torch.empty(n, device=hidden.device, dtype=torch.float32)
        lse = torch.empty_like(lp)
        ent = torch.empty_like(lp) if want_entropy else None
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            logits = F.gemm_nt(hidden[lo:hi], weight)
            a, b, c = F.logprob_fused_fwd(logits, targets[lo:hi], leaves, want_entropy)
            lp[lo:hi], lse[lo:hi] = a, b
            if want_entropy:
                ent[lo:hi] = c
            del logits
        ctx.save_for_backward(hidden, weight, targets, lse, ent if want_entropy else lse)
        ctx.cfg = (leaves, chunk, want_entropy)
        if not want_entropy:
            ent = torch.zeros_like(lp)
            ctx.mark_non_differentiable(ent)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, targets, lse, ent = ctx.saved_tensors
        leaves, chunk, want_entropy = ctx.cfg
        n = hidden.shape[0]
        g_lp = g_lp.contiguous().float()
        ge = g_ent.contiguous().float() if want_entropy and g_ent is not None else None
        dh = torch.empty_like(hidden)
        # the weight gradient of all chunks is summed in fp32 by the TN GEMM's accumulating epilogue (GPU, bf16)
        own = hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
        dwf = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if own else None
        dw = None if own else torch.zeros_like(weight)
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            logits = F.gemm_nt(hidden[lo:hi], weight)
            d = F.logprob_bwd(logits, targets[lo:hi], lse[lo:hi], g_lp[lo:hi], None if ge is None else ge[lo:hi],
                              ent[lo:hi] if ge is not None else None, inplace=True)
            dh[lo:hi] = F.gemm_nn(d, weight)
            if dwf is not None:
                F.gemm_tn(d, hidden[lo:hi], out=dwf, accumulate=True)
            else:
                dw.addmm_(d.t(), hidden[lo:hi])
            del logits, d
        return dh, (dwf.to(weight.dtype) if dwf is not None else dw), None, None, None, None


def lm_head_logprobs(model: DecoderLM, hidden_rows, targets, chunk: int, want_entropy: bool = False):
    w = model.lm_head_weight()
    leaves = model.cfg.logprob_leaves
    if model.ps.tp > 1:
        from ..parallel.vocab_parallel import vocab_parallel_logprobs

        return vocab_parallel_logprobs(model, hidden_rows, targets, chunk, want_entropy)
    if torch.is_grad_enabled() and (hidden_rows.requires_grad or w.requires_grad):
        return _LMHeadLogprob.apply(hidden_rows, w, targets, leaves, chunk, want_entropy)
    n = hidden_rows.shape[0]
    lp = torch.empty(n, device=hidden_rows.device, dtype=torch.float32)
    ent = torch.zeros_like(lp)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        a, _, c = F.logprob_fused_fwd(F.gemm_nt(hidden_rows[lo:hi], w), targets[lo:hi], leaves, want_entropy)
        lp[lo:hi] = a
        if want_entropy:
            ent[lo:hi] = c
    return lp, ent


# ------------------------------------------------------------------------------------ packing
@dataclass
class PackedMicroBatch:
    seq_index: list[int]          # rows of the mini-batch in this micro-batch
    ids: torch.Tensor             # int64 [T]
    positions: torch.Tensor       # int32 [T]
    seq_lens: list[int]
    pred_rows: torch.Tensor       # int64 [Nr] hidden rows that predict a response token
    targets: torch.Tensor         # int64 [Nr]
    out_index: torch.Tensor       # int64 [Nr] flat index into [len(seq_index) * R]
    packed_rows: list[int] | None = None   # the mini-batch row behind every entry of seq_lens (empty sequences are not packed)


def pack_microbatches(sequences: torch.Tensor, attention_mask: torch.Tensor, num_actions: int,
                      max_tokens: int, min_groups: int = 0) -> list[PackedMicroBatch]:
    """Remove padding, pack sequences back to back and cut micro-batches by a token budget. ``min_groups``: produce at
    least that many micro-batches (ranks that share collectives per layer must run the same number of them)."""
    B, S = sequences.shape
    P = S - num_actions
    att = attention_mask.bool()
    lens = att.sum(1).tolist()
    first = att.float().argmax(1).tolist()
    groups, cur, cur_tok = [], [], 0
    for b in range(B):
        if cur and cur_tok + lens[b] > max_tokens:
            groups.append(cur)
            cur, cur_tok = [], 0
        cur.append(b)
        cur_tok += lens[b]
    if cur:
        groups.append(cur)
    while len(groups) < min_groups:
        big = max(range(len(groups)), key=lambda i: len(groups[i]))
        if len(groups[big]) < 2:
            raise ValueError(f"cannot cut {B} sequences into {min_groups} micro-batches; give every rank at least that many sequences")
        g = groups.pop(big)
        groups[big:big] = [g[:len(g) // 2], g[len(g) // 2:]]
    out = []
    for grp in groups:
        ids, pos, pred, tgt, oidx, seq_lens, packed = [], [], [], [], [], [], []
        base = 0
        for j, b in enumerate(grp):
            n, f = lens[b], first[b]
            if n == 0:
                continue
            packed.append(b)
            ids.append(sequences[b, f:f + n])
            pos.append(torch.arange(n, dtype=torch.int32))
            plen = P - f                      # real prompt tokens
            rlen = n - plen                   # real response tokens
            if rlen > 0 and plen > 0:
                k = torch.arange(rlen)
                pred.append(base + plen - 1 + k)
                tgt.append(sequences[b, P:P + rlen])
                oidx.append(j * num_actions + k)
            seq_lens.append(n)
            base += n
        z = torch.zeros(0, dtype=torch.long)
        out.append(PackedMicroBatch(grp, torch.cat(ids), torch.cat(pos), seq_lens,
                                    torch.cat(pred) if pred else z, torch.cat(tgt) if tgt else z,
                                    torch.cat(oidx) if oidx else z, packed))
    return out


# ------------------------------------------------------------------------------------ optimizer
class FlatAdamW:
    """AdamW over the model's flat parameter buffer: fp32 master weights, moments and main
    gradients are four flat buffers, updated by one kernel launch (csrc/loss_optim.cu). Gradient
    norm and clip coefficient are computed on the device in a fixed order; nothing syncs with
    the host unless the caller reads the norm."""

    def __init__(self, model: DecoderLM, cfg: OptimizerConfig, shard: tuple | None = None):
        """``shard = (index, count, process group)``: this rank keeps the fp32 master weights and both moments of one
        contiguous slice of the flat buffer only (the distributed optimizer of the reference's Megatron backend,
        B/distributed/megatron/megatron_strategy.py:281-323, and what FSDP2 does to optimizer state). Gradients are still
        summed in full, so the norm, the clip coefficient and every updated weight have the bits of the unsharded run;
        after the update each rank broadcasts its slice of the new low-precision weights."""
        self.model, self.cfg = model, cfg
        flat = model.store.flat
        self.n = flat.numel()
        dev = flat.device
        self.low_precision = flat.dtype != torch.float32
        self.shard = shard if shard is not None and shard[1] > 1 else None
        if self.shard is not None:
            idx, cnt, _ = self.shard
            per = (-(-self.n // cnt) + 63) // 64 * 64          # slices start on 256-byte boundaries
            self.slices = [(min(self.n, r * per), min(self.n, (r + 1) * per)) for r in range(cnt)]
            self.lo, self.hi = self.slices[idx]
        else:
            self.slices, self.lo, self.hi = [(0, self.n)], 0, self.n
        own = flat.detach()[self.lo:self.hi]
        self.master = own.float().clone() if self.low_precision else own
        self.exp_avg = torch.zeros(self.hi - self.lo, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.hi - self.lo, dtype=torch.float32, device=dev)
        self.main_grad = torch.zeros(self.n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self._sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._coef = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._scratch = None
        self._hooks = []
        for name in model.store.order:
            spec = model.store.specs[name]
            p = model.p(name)
            view = self.main_grad[spec.offset:spec.offset + p.numel()].view(p.shape)
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(view, name)))
        self._ov = None

    # ---- data-parallel reduction overlapped with the backward -------------------------------------------------
    def setup_overlap(self, ps, bucket_elems: int = 64 << 20) -> None:
        """Cut the flat gradient buffer into buckets of whole parameters (storage order). During the LAST micro-batch's
        backward a bucket is summed over the data-parallel group, on a side stream, as soon as its last gradient has
        been accumulated, so the reduction hides behind the remaining backward instead of following it."""
        buckets, cur_lo, cur_names, end = [], None, [], 0
        for name in self.model.store.order:
            s = self.model.store.specs[name]
            if cur_lo is None:
                cur_lo = s.offset
            cur_names.append(name)
            end = s.offset + math.prod(s.shape)
            if end - cur_lo >= bucket_elems:
                buckets.append((cur_lo, end, cur_names))
                cur_lo, cur_names = None, []
        if cur_names:
            buckets.append((cur_lo, end, cur_names))
        self._ov = {"ps": ps, "buckets": buckets, "of": {n: i for i, b in enumerate(buckets) for n in b[2]},
                    "pending": [0] * len(buckets), "done": set(), "active": False,
                    "side": torch.cuda.Stream() if self.main_grad.is_cuda else None}

    def begin_overlap(self) -> None:
        ov = self._ov
        if ov is None:
            return
        ov["pending"] = [len(b[2]) for b in ov["buckets"]]
        ov["done"], ov["active"] = set(), True

    def _bucket_ready(self, i: int) -> None:
        from ..parallel.dp import reduce_main_grads

        ov = self._ov
        lo, hi, _ = ov["buckets"][i]
        if ov["side"] is not None:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(ov["side"]):
                ov["side"].wait_event(ev)
                reduce_main_grads(self.main_grad, ov["ps"], ranges=[(lo, hi)])
        else:
            reduce_main_grads(self.main_grad, ov["ps"], ranges=[(lo, hi)])
        ov["done"].add(i)

    def finish_overlap(self) -> bool:
        """Reduce whatever the backward did not trigger, join the side stream. False if no overlap was running."""
        ov = self._ov
        if ov is None or not ov["active"]:
            return False
        for i in range(len(ov["buckets"]) - 1, -1, -1):      # same order on every rank
            if i not in ov["done"]:
                self._bucket_ready(i)
        if ov["side"] is not None:
            torch.cuda.current_stream().wait_stream(ov["side"])
        ov["active"] = False
        return True

    def _make_hook(self, view, name):
        def hook(p):
            g = p.grad
            if g is None:          # another optimizer on the same parameters has already taken it
                return
            if g.is_cuda and g.dtype == torch.bfloat16 and g.is_contiguous() and g.numel() % 8 == 0:
                # main_grad += float(grad), vectorised (csrc/loss_optim.cu); torch's mixed-dtype add_ runs at a quarter of the bandwidth
                _native.check(_native.lib().ix_accum_bf16_to_f32(view.data_ptr(), g.data_ptr(), g.numel(), 1, _native.stream()),
                              "ix_accum_bf16_to_f32")
            else:
                view.add_(g)
            p.grad = None
            ov = self._ov
            if ov is not None and ov["active"]:
                b = ov["of"][name]
                ov["pending"][b] -= 1
                if ov["pending"][b] == 0:
                    self._bucket_ready(b)
        return hook

    def zero_grad(self):
        self.main_grad.zero_()

    def lr_at(self, step: int) -> float:
        c = self.cfg
        if c.num_warmup_steps and step < c.num_warmup_steps:
            return c.lr * (step + 1) / c.num_warmup_steps
        if c.scheduler == "cosine" and c.total_steps > c.num_warmup_steps:
            t = (step - c.num_warmup_steps) / (c.total_steps - c.num_warmup_steps)
            return c.lr * (c.min_lr_ratio + (1 - c.min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * min(1.0, t))))
        if c.scheduler == "linear" and c.total_steps > c.num_warmup_steps:
            t = (step - c.num_warmup_steps) / (c.total_steps - c.num_warmup_steps)
            return c.lr * max(c.min_lr_ratio, 1 - t)
        return c.lr

    def grad_sq_norm(self, ps: ParallelState) -> torch.Tensor:
        """Squared L2 norm of the full gradient. Replicated parameters are counted once."""
        self._sq = F.reduce_sum_fixed(self.main_grad, square=True, out=self._sq, scratch=self._scratch)
        if ps.tp > 1:
            # sharded parameters add across TP; replicated ones are identical on every rank, so
            # count them on TP rank 0 only
            rep = torch.zeros_like(self._sq)
            for name in self.model.store.order:
                s = self.model.store.specs[name]
                if s.shard_dim is None:
                    g = self.main_grad[s.offset:s.offset + math.prod(s.shape)]
                    rep += g.square().sum()
            local = self._sq - (rep if ps.tp_rank != 0 else 0)
            if getattr(ps, "kvr_rank", 0) != 0:
                # copies of a replicated KV head: counted once, on the first rank of the sharing group
                from ..models.decoder import kv_rows

                for name in self.model.store.order:
                    s = self.model.store.specs[name]
                    if s.kv_rep > 1:
                        r0, nr = kv_rows(s)
                        lo = s.offset + r0 * s.shape[1]
                        local = local - self.main_grad[lo:lo + nr * s.shape[1]].square().sum()
            dist.all_reduce(local, group=ps.tp_group)
            self._sq = local
        if ps.ep > 1 and self.model.cfg.has_moe:
            # expert shards are distinct parameters on every rank of the EP group: add them up; the rest is replicated
            ex = torch.zeros_like(self._sq)
            for name in self.model.store.order:
                s = self.model.store.specs[name]
                if s.ep_sharded:
                    ex += self.main_grad[s.offset:s.offset + math.prod(s.shape)].square().sum()
            tot = ex.clone()
            dist.all_reduce(tot, group=ps.ep_group)
            self._sq = self._sq - ex + tot
        if ps.pp > 1:
            # every pipeline stage holds its own layers: the global norm is the sum over stages (a tied embedding sits on
            # the first and the last stage with the same, already summed, gradient: counted on the first only)
            local = self._sq.clone()
            if self.model.cfg.tie_embeddings and ps.is_last_pp and not ps.is_first_pp and "embed.weight" in self.model.store.specs:
                s = self.model.store.specs["embed.weight"]
                local = local - self.main_grad[s.offset:s.offset + math.prod(s.shape)].square().sum()
            dist.all_reduce(local, group=ps.pp_group)
            self._sq = local
        return self._sq

    def step(self, ps: ParallelState) -> torch.Tensor:
        """Clip by global norm and apply AdamW. Returns the gradient norm (device scalar)."""
        c = self.cfg
        sq = self.grad_sq_norm(ps)
        self.step_count += 1
        lr = self.lr_at(self.step_count - 1)
        flat = self.model.store.flat
        if flat.is_cuda:
            L = _native.lib()
            _native.check(L.ix_clip_coef(sq.data_ptr(), c.max_grad_norm, self._coef.data_ptr(), self._norm.data_ptr(),
                                         _native.stream()), "ix_clip_coef")
            if self.hi > self.lo:
                _native.check(L.ix_adamw(self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                                         self.main_grad.data_ptr() + 4 * self.lo,
                                         flat.data_ptr() + flat.element_size() * self.lo if self.low_precision else None,
                                         self.hi - self.lo, 1, lr, c.beta1, c.beta2, c.eps, c.weight_decay, self.step_count,
                                         self._coef.data_ptr(), _native.stream()), "ix_adamw")
        else:
            norm = sq.sqrt()
            self._norm.copy_(norm)
            coef = torch.clamp(c.max_grad_norm / (norm + 1e-6), max=1.0) if c.max_grad_norm > 0 else torch.ones(1)
            g = self.main_grad[self.lo:self.hi] * coef
            self.exp_avg.mul_(c.beta1).add_(g, alpha=1 - c.beta1)
            self.exp_avg_sq.mul_(c.beta2).addcmul_(g, g, value=1 - c.beta2)
            bc1, bc2 = 1 - c.beta1 ** self.step_count, 1 - c.beta2 ** self.step_count
            with torch.no_grad():
                self.master.mul_(1 - lr * c.weight_decay)
                self.master.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt() + c.eps, value=-lr)
                if self.low_precision:
                    flat[self.lo:self.hi].copy_(self.master.to(flat.dtype))
        self._gather_weights()
        self.zero_grad()
        return self._norm

    def _gather_weights(self) -> None:
        """Sharded optimizer: every rank sends the slice it has just updated to the others."""
        if self.shard is None:
            return
        _, cnt, group = self.shard
        flat = self.model.store.flat.detach()
        for r in range(cnt):
            lo, hi = self.slices[r]
            if hi > lo:
                dist.broadcast(flat[lo:hi], src=dist.get_global_rank(group, r) if group is not None else r, group=group)

    def state_dict(self) -> dict:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq,
                "step": self.step_count, "slice": (self.lo, self.hi, self.n)}

    def load_state_dict(self, sd: dict) -> None:
        """Accepts the state of the same slice, or a full (unsharded) state, which is cut to this rank's slice."""
        lo, hi, n = sd.get("slice", (0, self.n, self.n))
        if n != self.n or not (lo <= self.lo and self.hi <= hi):
            raise ValueError(f"optimizer state covers [{lo}, {hi}) of {n}; this rank needs [{self.lo}, {self.hi}) of {self.n}")
        cut = slice(self.lo - lo, self.hi - lo)
        with torch.no_grad():
            self.master.copy_(sd["master"][cut])
            self.exp_avg.copy_(sd["exp_avg"][cut])
            self.exp_avg_sq.copy_(sd["exp_avg_sq"][cut])
            self.step_count = int(sd["step"])
            if self.low_precision:
                flat = self.model.store.flat
                flat[self.lo:self.hi].copy_(self.master.to(flat.dtype))
        self._gather_weights()

    def offload(self):
        """Move optimizer state to pinned host memory (the colocated rollout phase needs the HBM)."""
        for n in ("master", "exp_avg", "exp_avg_sq", "main_grad"):
            t = getattr(self, n)
            if t.is_cuda and not (n == "master" and not self.low_precision):
                setattr(self, n, t.to("cpu", non_blocking=False).pin_memory())

    def backload(self, device):
        for n in ("master", "exp_avg", "exp_avg_sq", "main_grad"):
            t = getattr(self, n)
            if not t.is_cuda and torch.device(device).type == "cuda":
                setattr(self, n, t.to(device, non_blocking=True))


def layers_that_fit(headroom_bytes: int, bytes_per_layer: int, num_layers: int, margin_bytes: int = 10 << 30,
                    safety: float = 1.25) -> int:
    """How many layers' activations fit into HBM that a whole step never touched: the estimate per layer is inflated
    by ``safety`` and ``margin_bytes`` stay free for fragmentation and for anything the first step did not show."""
    if bytes_per_layer <= 0:
        return 0
    return max(0, min(num_layers, int((headroom_bytes - margin_bytes) // int(safety * bytes_per_layer))))


# ------------------------------------------------------------------------------------ worker
class PolicyWorker:
    def __init__(self, model: DecoderLM, cfg: WorkerConfig | None = None, algo: alg.AlgorithmConfig | None = None):
        self.model = model
        self.cfg = cfg or WorkerConfig()
        self.algo = algo or alg.AlgorithmConfig()
        self.ps = model.ps
        self.device = model.device_
        ps = self.ps
        shard = None
        if self.cfg.shard_optimizer and ps.dp > 1 and ps.ep == 1 and ps.pp == 1 and dist.is_initialized():
            shard = (ps.dp_rank, ps.dp, ps.dp_group)
        self.opt = FlatAdamW(model, self.cfg.optimizer, shard=shard)
        self._auto_keep = None
        self.launch_count = 0

    # ---------------------------------------------------------------- forward pieces
    def _ckpt_arg(self):
        if not (self.cfg.checkpoint_layers and torch.is_grad_enabled()):
            return False
        keep = self.keep_layers()
        return True if keep <= 0 else max(0, len(self.model.layer_ids) - keep)

    def keep_layers(self) -> int:
        """Layers whose activations stay alive for the backward instead of being recomputed. ``-1`` in the config means
        "what the spare HBM allows": 0 until one whole step has run with full recompute, then fixed from that step's
        measured peak (see ``_calibrate_keep``)."""
        keep = getattr(self.cfg, "keep_last_layers", 0)
        if keep >= 0:
            return keep
        return self._auto_keep or 0

    def activation_bytes_per_layer(self, tokens: int) -> int:
        """What autograd keeps alive for one dense layer that is not recomputed: layer input, both residual sums, both
        normed inputs, the o-projection output, fused QKV, rotated Q/K, attention output, gate|up and the activation."""
        c = self.model.cfg
        tp = max(1, self.ps.tp)
        qkv = (c.num_q_heads * (2 if c.attn_output_gate else 1) + 2 * c.num_kv_heads) * c.head_dim // tp
        qk = (c.num_q_heads + c.num_kv_heads) * c.head_dim // tp
        attn = c.num_q_heads * c.head_dim // tp
        per_token = 6 * c.hidden_size + qkv + qk + attn + 3 * c.ffn_size // tp
        return 2 * per_token * tokens

    def _calibrate_keep(self) -> None:
        """After the first full step (rollout, scoring and update have each run once with full recompute): the HBM the
        step never touched, less a margin, is given to activations of the last layers. Dense attention models on a
        GPU only; every data-parallel rank takes the smallest answer so that steps stay balanced."""
        if getattr(self.cfg, "keep_last_layers", 0) >= 0 or self._auto_keep is not None:
            return
        n = 0
        c = self.model.cfg
        if self.device.type == "cuda" and not c.has_moe and not c.has_gdn and self.cfg.checkpoint_layers:
            total = torch.cuda.get_device_properties(self.device).total_memory
            free_now, _ = torch.cuda.mem_get_info(self.device)
            outside = total - free_now - torch.cuda.memory_reserved(self.device)   # context, NCCL, symmetric memory
            if getattr(self, "_peak_armed", False):
                # the peak of the scoring and training phases alone: a colocated engine's KV pools (asleep by now, their
                # blocks back in the allocator's cache) set the step's overall peak but never coexist with activations
                headroom = total - outside - torch.cuda.max_memory_allocated(self.device)
            else:
                headroom = total - outside - torch.cuda.max_memory_reserved(self.device)
            n = layers_that_fit(headroom, self.activation_bytes_per_layer(self.cfg.max_tokens_per_microbatch),
                                len(self.model.layer_ids))
        if dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([n], dtype=torch.int64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            n = int(t.item())
        self._auto_keep = n

    def _arm_peak(self) -> None:
        """First scoring / training call of a run that sizes the kept layers itself: start the peak-memory statistics
        here, so that ``_calibrate_keep`` sees what these phases need, not what the rollout before them needed."""
        if (self.device.type == "cuda" and getattr(self.cfg, "keep_last_layers", 0) < 0 and self._auto_keep is None
                and not getattr(self, "_peak_armed", False)):
            torch.cuda.reset_peak_memory_stats(self.device)
            self._peak_armed = True

    def _run_model(self, mb: PackedMicroBatch, site: str):
        dev = self.device
        if self.ps.cp > 1:
            return self._run_model_cp(mb, site)
        fc = ForwardCtx(positions=mb.positions.to(dev, non_blocking=True),
                        meta=F.AttnMeta.packed(mb.seq_lens, self.model.hq, self.model.hkv, dev), site=site)
        if self.model.cfg.has_gdn:
            from ..ops.gdn import GDNMeta

            fc.gdn_meta = GDNMeta.packed(mb.seq_lens, dev)
        fc.mm = self._image_rows(mb)
        hidden = self.model(mb.ids.to(dev, non_blocking=True), fc,
                            checkpoint_layers=self._ckpt_arg())
        return hidden

    def set_images(self, batch) -> None:
        """Remember the batch's ``pixel_values`` / ``image_grid_thw`` (per-sample lists) for the forwards that follow."""
        pv = batch.get("pixel_values") if batch is not None else None
        self._mm = None if pv is None else (pv, batch.get("image_grid_thw"), batch.get("mm_positions"))
        if self._mm is not None:
            if getattr(self.model, "vision", None) is None:
                raise ValueError(f"the batch carries images but model {self.model.cfg.name!r} has no vision tower")
            if self.ps.cp > 1 or self.ps.pp > 1:
                raise ValueError("image inputs are not supported with context or pipeline parallelism")

    def _image_rows(self, mb: PackedMicroBatch):
        """(rows, features) of the micro-batch's image placeholder tokens: the tower runs image by image, without gradient,
        exactly as the engine ran it for the rollout. Where the batch names the placeholder positions (``mm_positions``,
        counted from the first real token of a sequence) they are used; otherwise a sequence's FIRST placeholder-id
        tokens are taken, as many as its images give rows (a placeholder id the policy sampled later is plain text)."""
        mm = getattr(self, "_mm", None)
        if mm is None:
            return None
        tok = self.model.cfg.image_token_id
        rows, feats, base = [], [], 0
        for b, n in zip(mb.packed_rows if mb.packed_rows is not None else mb.seq_index, mb.seq_lens):
            if mm[0][b].shape[0] == 0:
                base += n
                continue
            f = self.model.vision.encode(mm[0][b], mm[1][b])
            if mm[2] is not None:
                r = mm[2][b].to(torch.long) + base
                if r.numel() != f.shape[0] or (r.numel() and (int(r.max()) >= base + n or bool((mb.ids[r] != tok).any()))):
                    raise ValueError(f"sample {b}: {r.numel()} image positions for {f.shape[0]} feature rows, or a position that is "
                                     f"not an image placeholder token (a prompt truncated inside an image?)")
            else:
                r = (mb.ids[base:base + n] == tok).nonzero(as_tuple=True)[0][:f.shape[0]] + base
                if r.numel() != f.shape[0]:
                    raise ValueError(f"sample {b}: {r.numel()} image placeholder tokens but the images give {f.shape[0]} feature rows "
                                     f"(a prompt truncated inside an image?)")
            rows.append(r)
            feats.append(f)
            base += n
        if not rows:
            return None
        return torch.cat(rows).to(self.device, non_blocking=True), torch.cat(feats, 0)

    # ---------------------------------------------------------------- context parallelism
    def _cp_span(self, mb: PackedMicroBatch) -> tuple[int, int, int]:
        """(padded token count, first token, one past the last token) of this rank's contiguous share of a micro-batch."""
        cp = self.ps.cp
        Tp = (int(mb.ids.numel()) + cp - 1) // cp * cp
        n = Tp // cp
        return Tp, self.ps.cp_rank * n, (self.ps.cp_rank + 1) * n

    def _run_model_cp(self, mb: PackedMicroBatch, site: str):
        """The packed micro-batch is padded to a multiple of cp tokens (the padding forms a sequence of its own, so no real
        token attends to it) and cut into cp contiguous shares; this rank runs the model on its share and the attention
        layers exchange heads for tokens (``parallel/cp.py::ulysses_attention``). Returns the hidden rows of the share.
        Reference: B/distributed/megatron/model_utils.py:1438-1540, B/distributed/ulysses/utils.py:66-240."""
        c = self.model.cfg
        if c.has_gdn:
            raise ValueError("context parallelism cuts sequences across ranks; GatedDeltaNet layers scan a sequence in order and are not supported with it")
        cp, dev = self.ps.cp, self.device
        if self.model.hq % cp or self.model.hkv % cp:
            raise ValueError(f"context_parallel_size={cp} must divide the local query ({self.model.hq}) and KV ({self.model.hkv}) head counts")
        T = int(mb.ids.numel())
        Tp, lo, hi = self._cp_span(mb)
        ids, pos, lens = mb.ids, mb.positions, list(mb.seq_lens)
        if Tp > T:
            ids = torch.cat([ids, ids.new_zeros(Tp - T)])
            pos = torch.cat([pos, torch.arange(Tp - T, dtype=pos.dtype)])
            lens.append(Tp - T)
        fc = ForwardCtx(positions=pos[lo:hi].contiguous().to(dev, non_blocking=True),
                        meta=F.AttnMeta.packed(lens, self.model.hq // cp, self.model.hkv // cp, dev), site=site)
        return self.model(ids[lo:hi].contiguous().to(dev, non_blocking=True), fc, checkpoint_layers=self._ckpt_arg())

    def _pack(self, seqs, att, R):
        """Micro-batches of this rank. Under expert parallelism every rank of the EP group runs the same number of them
        (each MoE layer is a collective), so the count is agreed on first."""
        mbs = pack_microbatches(seqs, att, R, self.cfg.max_tokens_per_microbatch)
        if self.ps.ep > 1 and self.model.cfg.has_moe:
            n = torch.tensor([len(mbs)], dtype=torch.int64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(n, op=dist.ReduceOp.MAX, group=self.ps.ep_group)
            if int(n) > len(mbs):
                mbs = pack_microbatches(seqs, att, R, self.cfg.max_tokens_per_microbatch, min_groups=int(n))
        return mbs

    def _logprobs(self, mb: PackedMicroBatch, hidden, want_entropy: bool):
        """(logprobs, entropies, flat output index) of the response tokens this rank predicts: all of the micro-batch's, or
        under context parallelism those whose predicting row lies in this rank's share of the tokens."""
        dev = self.device
        rows, tg, oi = mb.pred_rows, mb.targets, mb.out_index
        if self.ps.cp > 1:
            _, lo, hi = self._cp_span(mb)
            mine = (rows >= lo) & (rows < hi)
            rows, tg, oi = rows[mine] - lo, tg[mine], oi[mine]
        rows = rows.to(dev, non_blocking=True)
        tg = tg.to(dev, non_blocking=True)
        h = hidden.index_select(0, rows)
        if self.cfg.temperature != 1.0:
            h = h * (1.0 / self.cfg.temperature)            # logits are linear in these rows: (h / T) W = (h W) / T
        lp, ent = lm_head_logprobs(self.model, h, tg, self.cfg.logprob_chunk_rows, want_entropy)
        return lp, ent, oi.to(dev)

    # ---------------------------------------------------------------- verbs
    @torch.no_grad()
    def forward(self, batch: TrainingInputBatch) -> torch.Tensor:
        """Scoring forward: log-probabilities of the response tokens, ``[B, max_response]`` fp32 (CPU)."""
        self._arm_peak()
        R = batch["response_mask"].shape[1] if batch.get("response_mask") is not None else batch.metadata["response_length"]
        seqs, att = batch["sequences"], batch["attention_mask"]
        self.set_images(batch)
        out = torch.zeros(seqs.shape[0], R, dtype=torch.float32)
        for mb in self._pack(seqs, att, R):
            hidden = self._run_model(mb, "trainer_score")
            lp, _, oi = self._logprobs(mb, hidden, False)
            flat = torch.zeros(len(mb.seq_index) * R, dtype=torch.float32, device=lp.device)
            flat[oi] = lp
            out[torch.tensor(mb.seq_index)] = flat.view(-1, R).cpu()
        if self.ps.cp > 1:
            # every rank filled the tokens of its own share and left zeros elsewhere: a sum is an exact merge
            t = out.to(self.device) if self.device.type == "cuda" else out
            dist.all_reduce(t, group=self.ps.cp_group)
            out = t.cpu()
        return out

    def forward_backward(self, batch: TrainingInputBatch) -> dict:
        """Accumulate the gradient of the (sum-reduced, advantage-pre-scaled) policy loss of a
        mini-batch shard. Returns metrics (python floats)."""
        algo = self.algo
        self._arm_peak()
        R = batch["response_mask"].shape[1]
        seqs, att = batch["sequences"], batch["attention_mask"]
        self.set_images(batch)
        loss_fn = alg.get_policy_loss(algo.policy_loss_type)
        want_ent = self.cfg.want_entropy or algo.use_entropy_loss
        tot = {"loss": 0.0, "clip_ratio_num": 0.0, "tokens": 0.0, "entropy_sum": 0.0, "kl_sum": 0.0}
        # optional: compare this forward's logprobs with the rollout's, bit for bit (the forward gate when the scoring
        # forward is skipped)
        check_bits = bool(batch.metadata.get("check_rollout_bits")) and batch.get("rollout_logprobs") is not None
        bits = {"mismatches": 0, "abs_sum": 0.0, "abs_max": 0.0, "tokens": 0.0}
        post = {"sum": 0.0, "sq": 0.0, "max": 0.0, "tokens": 0.0}
        dev = self.device
        mbs = self._pack(seqs, att, R)
        for mi, mb in enumerate(mbs):
            if mi == len(mbs) - 1 and self._overlap_ok():
                self.opt.begin_overlap()          # gradients of this backward are final: reduce them bucket by bucket
            idx = torch.tensor(mb.seq_index)
            if self.cfg.moe_aux_loss_coeff > 0 and self.model.cfg.has_moe:
                from ..ops import moe as _moe

                # the policy loss is a sum pre-divided by the global token count; the balance term of a micro-batch gets
                # the share of that count its own loss tokens have, so that the total is a token-weighted mean over micro-batches
                share = float(batch.metadata.get("aux_loss_scale", 0.0)) * float((batch["loss_mask"] if batch.get("loss_mask") is not None
                                                                                    else batch["response_mask"])[idx].sum())
                _moe.AUX_LOSS.update(coeff=self.cfg.moe_aux_loss_coeff, scale=share if share > 0 else 1.0 / max(1, len(mbs)))
                if mi == 0:
                    _moe.AUX_LOSS.update(sum=0.0, layers=0)
            hidden = self._run_model(mb, "trainer_fwd")
            lp_flat, ent_flat, oi = self._logprobs(mb, hidden, want_ent)
            nb = len(mb.seq_index)

            def to2d(x):
                return torch.zeros(nb * R, dtype=torch.float32, device=dev).index_put((oi,), x).view(nb, R)

            lp2d = to2d(lp_flat)
            get = lambda k: (batch[k][idx].to(dev).float() if batch.get(k) is not None else None)
            mask = get("loss_mask") if batch.get("loss_mask") is not None else get("response_mask")
            if self.ps.cp > 1:
                # the loss is a sum over tokens: each context-parallel rank takes the tokens it predicted, the gradient
                # sum over the cp group (reduce_gradients) puts the pieces together
                if algo.policy_loss_type in ("gspo", "sapo"):
                    raise ValueError(f"policy_loss_type={algo.policy_loss_type!r} needs whole-sequence statistics and is not supported with context parallelism")
                mask = mask * to2d(torch.ones_like(lp_flat))
            old = get("action_log_probs")
            if old is None:
                old = lp2d.detach()
            loss, m = loss_fn(lp2d, old, get("advantages"), algo, loss_mask=mask, rollout_logprobs=get("rollout_logprobs"))
            ntok = mask.sum()
            if batch.get("rollout_logprobs") is not None and self.ps.cp == 1:
                # |logprob the loss optimises against - rollout logprob| over the trained tokens: the policy's drift since
                # the rollout once optimizer steps have happened between mini-batches (never the forward-identity gate;
                # R/backends/skyrl_train/workers/worker_utils.py:39-64)
                sel = mask > 0
                d_ = torch.where(sel, (lp2d.detach() - get("rollout_logprobs")).abs(), torch.zeros_like(lp2d))
                s_ = torch.stack([d_.sum(), (d_ * d_).sum(), d_.max() if d_.numel() else d_.sum(), sel.sum().to(d_.dtype)]).tolist()
                post["sum"] += s_[0]
                post["sq"] += s_[1]
                post["max"] = max(post["max"], s_[2])
                post["tokens"] += s_[3]
            if check_bits:
                from ..core.testing import count_bit_mismatches

                rm = get("response_mask")
                if batch.get("loss_mask") is not None:     # trained tokens only: observation tokens carry no rollout logprob
                    rm = rm * (get("loss_mask") > 0).to(rm.dtype)
                z_ = torch.zeros_like(rm)
                a_, b_ = torch.where(rm > 0, lp2d.detach(), z_).contiguous(), torch.where(rm > 0, get("rollout_logprobs"), z_).contiguous()
                d_ = (a_ - b_).abs()
                bits["mismatches"] += count_bit_mismatches(a_, b_)
                bits["abs_sum"] += float(d_.sum())
                bits["abs_max"] = max(bits["abs_max"], float(d_.max()) if d_.numel() else 0.0)
                bits["tokens"] += float(rm.sum())
            if algo.use_kl_loss and batch.get("base_action_log_probs") is not None:
                kl = alg.compute_approx_kl(lp2d, get("base_action_log_probs"), mask, algo.kl_estimator_type)
                scale = batch.metadata.get("aux_loss_scale", 1.0)
                loss = loss + algo.kl_loss_coef * scale * (kl * mask).sum()
                tot["kl_sum"] += float((kl * mask).sum().detach())
            if want_ent:
                ent2d = to2d(ent_flat)
                tot["entropy_sum"] += float((ent2d * mask).sum().detach())
                if algo.use_entropy_loss:
                    scale = batch.metadata.get("aux_loss_scale", 1.0)
                    loss = loss - algo.entropy_loss_coef * scale * (ent2d * mask).sum()
            loss.backward()
            tot["loss"] += float(loss.detach())
            tot["clip_ratio_num"] += float(m.get("clip_ratio", 0.0)) * float(ntok)
            tot["tokens"] += float(ntok)
        if self.ps.cp > 1:
            keys = sorted(tot)
            t = torch.tensor([tot[k] for k in keys], dtype=torch.float64, device=dev if dev.type == "cuda" else "cpu")
            dist.all_reduce(t, group=self.ps.cp_group)
            tot = {k: float(v) for k, v in zip(keys, t.tolist())}
        n = max(1.0, tot["tokens"])
        out = {"policy_loss": tot["loss"], "ppo_clip_ratio": tot["clip_ratio_num"] / n, "loss_tokens": tot["tokens"],
               "policy_entropy": tot["entropy_sum"] / n, "policy_kl": tot["kl_sum"] / n}
        if self.cfg.moe_aux_loss_coeff > 0 and self.model.cfg.has_moe:
            from ..ops import moe as _moe

            out["moe_aux_loss"] = _moe.AUX_LOSS["sum"] / max(1, _moe.AUX_LOSS["layers"])      # mean balance term per layer and micro-batch
            _moe.AUX_LOSS.update(coeff=0.0)                                                    # forwards outside the update carry none
        if check_bits:
            out["rollout_bits"] = bits
        if post["tokens"] > 0:
            out["post_update_diff"] = post
        return out

    def _overlap_ok(self) -> bool:
        """Overlap applies to plain data parallelism (no TP/EP-specific reductions to order before the DP sum)."""
        ps = self.ps
        if not (ps.dp > 1 and ps.tp == 1 and ps.ep == 1 and self.cfg.overlap_grad_reduce):
            return False
        if self.opt._ov is None:
            self.opt.setup_overlap(ps)
        return True

    @staticmethod
    def _kv_range(s) -> tuple[int, int]:
        """(first element, count) of the replicated k|v rows of a fused-QKV shard inside the flat buffer."""
        from ..models.decoder import kv_rows

        r0, nr = kv_rows(s)
        return s.offset + r0 * s.shape[1], nr * s.shape[1]

    def reduce_gradients(self) -> None:
        """Sum the main gradients over the data-parallel group (fixed bucket order); before that,
        weights that are replicated over TP but only see the local heads get their gradient summed over TP."""
        if self.opt.finish_overlap():
            return
        if self.ps.tp > 1:
            store = self.model.store
            sp = bool(getattr(self.model.cfg, "sequence_parallel", False))
            for name in store.order:
                s = store.specs[name]
                # under sequence parallelism the norm weights between the tensor-parallel regions saw this rank's rows only
                sp_partial = sp and s.shard_dim is None and name.endswith(("ln1.weight", "ln2.weight", "final_norm.weight"))
                if s.tp_grad_sum or sp_partial:
                    dist.all_reduce(self.opt.main_grad[s.offset:s.offset + math.prod(s.shape)], group=self.ps.tp_group)
                if s.kv_rep > 1:
                    # the ranks that share a KV head each saw the gradient from their own query heads only
                    lo, n = self._kv_range(s)
                    dist.all_reduce(self.opt.main_grad[lo:lo + n], group=self.ps.kvr_group)
        if self.ps.cp > 1:
            # every context-parallel rank saw a share of the tokens: parameter gradients are partial sums
            from ..parallel.dp import reduce_main_grads

            reduce_main_grads(self.opt.main_grad, self.ps, group=self.ps.cp_group)
        if self.ps.dp > 1:
            from ..parallel.dp import reduce_main_grads, split_ranges_by_expert_sharding

            if self.ps.ep > 1 and self.model.cfg.has_moe:
                # expert shards differ from rank to rank inside an EP group: only ranks holding the same shard sum them
                dense, expert = split_ranges_by_expert_sharding(self.model.store)
                reduce_main_grads(self.opt.main_grad, self.ps, ranges=dense)
                reduce_main_grads(self.opt.main_grad, self.ps, ranges=expert, group=self.ps.edp_group)
            else:
                reduce_main_grads(self.opt.main_grad, self.ps)

    def optim_step(self) -> float:
        self.reduce_gradients()
        if getattr(self, "lora", None) is not None:
            # adapters: the dense gradients are projected onto the factors, the factors step, the merged weights are
            # rebuilt; master weights and Adam moments of the base parameters never move
            return self.lora.optim_step()
        frozen = None
        if self.cfg.freeze_moe_router and self.model.cfg.has_moe:
            frozen = [(t, t.detach().clone()) for n, t in self.model.named_weights() if ".moe.router." in n]
        norm = self.opt.step(self.ps)
        if frozen:
            with torch.no_grad():
                for t, old in frozen:
                    t.copy_(old)
                if self.opt.low_precision:          # the fp32 master copy follows, or the next step would bring the change back
                    for n, t in self.model.named_weights():
                        if ".moe.router." in n:
                            sp = self.model.store.specs[n]
                            a, b = max(self.opt.lo, sp.offset), min(self.opt.hi, sp.offset + t.numel())
                            if a < b:
                                self.opt.master[a - self.opt.lo:b - self.opt.lo].copy_(t.reshape(-1)[a - sp.offset:b - sp.offset].float())
        out = float(norm.item())
        self._calibrate_keep()
        return out

    # ---------------------------------------------------------------- memory residency (colocated runs)
    def offload_optimizer(self):
        self.opt.offload()

    def backload_optimizer(self):
        self.opt.backload(self.device)
