"""The RL controller: one GRPO/PPO step = generate -> score -> advantages -> update -> sync.

Mirrors ``RayPPOTrainer.train`` (R/train/trainer.py:309-635) as an SPMD program: every rank (one
process per GPU) runs this loop on its own shard of the prompts with a colocated rollout engine
and policy worker; prompt groups never straddle ranks, so advantages need no communication, and
the only cross-rank traffic of a step is the token-count / metric all-reduce and the gradient
reduction. Ray is not needed.

IsoExec hooks, as in the reference: contract built and installed on both sides at model
construction (R/train/trainer.py:223), hash exchanged on the weight-sync init message and
checked again on every sync, rollout-vs-train logprob gate after scoring (trainer.py:455-475,
1540-1588; R/train/utils/trainer_utils.py:199-267).
"""

from __future__ import annotations

import asyncio
import os
import random
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..core import ledger as L
from ..core import observe as _observe
from ..core import process as P
from ..core.adapter import ContractAdapter, served_ops_of
from ..core.testing import count_bit_mismatches
from ..engine.interface import NativeInferenceEngine
from ..engine.llm_engine import EngineConfig, LLMEngine
from ..models.config import get_config
from ..models.decoder import DecoderLM
from ..parallel.state import ParallelState
from ..sync import strategies as S
from ..utils.tracking import Timer, Tracking
from . import algorithms as alg
from . import checkpoint as ckpt
from .batch import TrainingInputBatch, build_sequences, pad_training_input_batch
from .config import SkyRLTrainConfig, validate_cfg
from .generator import GeneratorInput, GeneratorOutput, SkyRLGymGenerator
from .policy_worker import PolicyWorker, WorkerConfig


class ForwardGateError(RuntimeError):
    pass


def validate_isoexec_forward_gate(diff_abs: torch.Tensor, mask: torch.Tensor, mismatches: int, cfg) -> dict:
    """Rollout-vs-train logprob gate. Under the contract the tolerance claim is zero, so any bit
    mismatch refuses; the reference's mean/max envelope (1e-5 / 1e-4) is kept as a second line."""
    n = mask.sum().clamp(min=1)
    mean = float((diff_abs * mask).sum() / n)
    mx = float((diff_abs * mask).max()) if diff_abs.numel() else 0.0
    ok = mean <= cfg.gate_mean_limit and mx <= cfg.gate_max_limit and (mismatches == 0 or not cfg.require_bitwise)
    return {"ok": ok, "mean": mean, "max": mx, "mismatches": mismatches}


class SyntheticPromptDataset:
    """Uniform-random token prompts with a fixed seed (the benchmark configurations use synthetic data)."""

    def __init__(self, num_prompts: int, prompt_len: int, vocab_size: int, seed: int, env_class: str):
        g = torch.Generator().manual_seed(seed)
        self.prompts = [torch.randint(0, vocab_size, (prompt_len,), generator=g).tolist() for _ in range(num_prompts)]
        self.env_class = env_class

    def __len__(self):
        return len(self.prompts)

    def __getitem__(self, i):
        return {"prompt": self.prompts[i], "env_class": self.env_class, "env_extras": {}, "uid": f"p{i}"}


class PromptDataLoader:
    """Shuffling batch iterator with a resumable state (epoch, cursor, seed).

    Data parallelism: every rank walks the SAME global order (one seed for the job) and takes slice ``part`` of
    ``parts`` out of each global batch of ``batch_size * parts`` prompts, so the shards of one step are disjoint, an
    epoch visits every prompt once across the job, and the state is identical on every rank (one rank saves it for all)."""

    def __init__(self, dataset, batch_size: int, seed: int, shuffle: bool = True, drop_last: bool = True,
                 part: int = 0, parts: int = 1):
        self.ds, self.bs, self.seed, self.shuffle, self.drop_last = dataset, batch_size, seed, shuffle, drop_last
        self.part, self.parts = part, max(1, parts)
        self.epoch, self.cursor = 0, 0
        self._order = self._make_order()

    def _make_order(self):
        idx = list(range(len(self.ds)))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        return idx

    @property
    def _global_bs(self) -> int:
        return self.bs * self.parts

    def __len__(self):
        g = self._global_bs
        return len(self.ds) // g if self.drop_last else (len(self.ds) + g - 1) // g

    def __iter__(self):
        g = self._global_bs
        while self.cursor + (g if self.drop_last else 1) <= len(self._order):
            whole = self._order[self.cursor:self.cursor + g]
            batch = [self.ds[i] for i in whole[self.part * self.bs:(self.part + 1) * self.bs]]
            self.cursor += g
            yield batch
        self.epoch += 1
        self.cursor = 0
        self._order = self._make_order()

    def state_dict(self):
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed, "parts": self.parts, "batch_size": self.bs}

    def load_state_dict(self, sd):
        self.epoch, self.seed = sd["epoch"], sd["seed"]
        # the cursor counts prompts of the global order, so it survives a change of the data-parallel degree as long
        # as the global batch is the same
        self.cursor = sd["cursor"]
        self._order = self._make_order()


class RayPPOTrainer:
    """Name kept for API parity; no Ray involved."""

    def __init__(self, cfg: SkyRLTrainConfig, ps: ParallelState | None = None, device: str | None = None,
                 dataset=None, tokenizer=None, tracker: Tracking | None = None, callbacks=None):
        from .callbacks import CallbackHandler, TrainingControl

        self.callbacks = CallbackHandler(callbacks)
        self.control = TrainingControl()
        self.epoch = 0
        self.cfg = cfg
        self.ps = ps or ParallelState.single()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        if ps is not None:        # the process groups that exist are the truth; the config follows them
            pc = cfg.trainer.policy.parallel
            pc.tensor_model_parallel_size, pc.pipeline_model_parallel_size = self.ps.tp, self.ps.pp
            pc.context_parallel_size, pc.expert_model_parallel_size = self.ps.cp, self.ps.ep
        validate_cfg(cfg, self.world)
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.tokenizer = tokenizer
        self.global_step = 0
        self.all_metrics: dict = {}
        self.all_timings: dict = {}
        t = cfg.trainer
        self.tracker = tracker or (Tracking(t.project_name, t.run_name, t.logger, cfg.to_dict()) if self.rank == 0 else None)
        self.dataset = dataset
        self.policy: PolicyWorker | None = None
        self.engine: LLMEngine | None = None
        self.generator: SkyRLGymGenerator | None = None
        self.kl_ctrl = alg.get_kl_controller(t.algorithm)

    def _fire(self, event: str, **fields) -> None:
        """Dispatch one callback event (R/train/utils/callbacks.py:117-162) with a fresh snapshot of the run's position."""
        if not self.callbacks:
            return
        from .callbacks import CallbackInput

        per_epoch = len(self.loader) if getattr(self, "loader", None) is not None else 0
        t = self.cfg.trainer
        total = t.num_steps if t.num_steps > 0 else per_epoch * t.epochs
        getattr(self.callbacks, event)(self, CallbackInput(self.global_step, self.epoch, total, per_epoch, **fields), self.control)

    # ------------------------------------------------------------------ build
    def _engine_layout(self, mcfg):
        """Decide how the rollout engines are laid out. Same tensor-parallel degree as the trainer: the engine computes
        with the trainer's own flat buffer (one engine per trainer TP group). Another degree (for instance "trainer TP4 x
        DP2 feeding four TP2 engines"): every GPU also holds a shard of an engine of that degree, engines nest inside
        trainer TP groups, and each sync reshards the weights (sync/reshard.py). Collective: every rank calls it."""
        ie = self.cfg.generator.inference_engine
        tp_e = ie.tensor_parallel_size or self.ps.tp
        self.separate_engine = tp_e != self.ps.tp or bool(getattr(ie, "own_weights", False))
        self.engine_ps = self.ps
        self.engines_per_replica = 1
        self.replica_group, self.replica_size, self.replica_rank = self.ps.tp_group, self.ps.tp, self.ps.tp_rank
        self._every_rank_leads = False
        if self.ps.cp > 1 and self.ps.pp == 1:
            # context-parallel trainer: parameters are not cut by cp, so every cp rank runs an engine on the trainer's own
            # weights; the cp engines of a replica split its requests and swap rollouts inside the cp group
            if tp_e != self.ps.tp:
                raise ValueError("a context-parallel trainer feeds engines of its own tensor-parallel degree")
            self.engines_per_replica = self.ps.cp
            self.replica_group, self.replica_size, self.replica_rank = self.ps.cp_group, self.ps.cp, self.ps.cp_rank
            self._every_rank_leads = True
            return tp_e
        if self.ps.pp > 1:
            self._every_rank_leads = True
            # pipelined trainer: every rank also holds an un-pipelined engine of the trainer's TP degree; the pp engines of
            # a replica split its requests and swap rollouts inside the pipeline group; the sync gathers the stages
            if tp_e != self.ps.tp or self.ps.cp > 1:
                raise ValueError("a pipelined trainer feeds engines of its own tensor-parallel degree (cp = 1)")
            import copy

            self.separate_engine = True
            self.engine_ps = copy.copy(self.ps)
            self.engine_ps.pp, self.engine_ps.pp_rank, self.engine_ps.pp_group, self.engine_ps.pp_ranks = 1, 0, None, [self.ps.rank]
            self.engines_per_replica = self.ps.pp
            self.replica_group, self.replica_size, self.replica_rank = self.ps.pp_group, self.ps.pp, self.ps.pp_rank
            return tp_e
        if self.separate_engine:
            if self.ps.tp % tp_e or self.ps.pp > 1 or self.ps.cp > 1 or self.ps.ep > 1:
                raise ValueError(f"engine TP {tp_e} must divide trainer TP {self.ps.tp}, with pp = cp = ep = 1")
            if tp_e == self.ps.tp:
                self.engine_ps = self.ps                  # own_weights: the trainer's layout, a second copy of the shards
            else:
                self.engine_ps = ParallelState.build(tp=tp_e, kv_rep=max(1, tp_e // mcfg.num_kv_heads)) if tp_e > 1 or self.world > 1 \
                    else ParallelState.single()
            self.engines_per_replica = self.ps.tp // tp_e
        return tp_e

    def _engine_index(self) -> int:
        """Global index of the engine this rank belongs to (all ranks of one engine share a sampler stream)."""
        if self.ps.pp > 1:
            return self.ps.dp_rank * self.ps.pp + self.ps.pp_rank
        if self.ps.cp > 1:
            return self.ps.dp_rank * self.ps.cp + self.ps.cp_rank
        return self.engine_ps.dp_rank if self.separate_engine else self.ps.dp_rank

    def _setup_transports(self, mcfg) -> None:
        """Peer-memory transports for every group this job computes over (GPUs with peer access only)."""
        self.transports = {}
        t = self.cfg.trainer
        if self.world == 1 or self.device.type != "cuda" or not getattr(t.policy, "peer_transports", True):
            return
        from ..parallel import tp_fused
        from ..parallel.transports import setup_transports

        if tp_fused.get(self.ps.tp_group) is None:          # a caller may have registered them already
            self.transports["trainer"] = setup_transports(self.ps, mcfg, max_tokens=t.max_tokens_per_microbatch)
        if self.separate_engine and self.engine_ps.tp > 1 and tp_fused.get(self.engine_ps.tp_group) is None:
            from ..parallel.state import ParallelState as _PS

            only_tp = _PS(tp=self.engine_ps.tp, tp_rank=self.engine_ps.tp_rank, tp_group=self.engine_ps.tp_group,
                          tp_ranks=self.engine_ps.tp_ranks)
            self.transports["engine"] = setup_transports(only_tp, mcfg, max_tokens=self.cfg.generator.inference_engine.max_num_batched_tokens)

    def build_models(self) -> None:
        t, g = self.cfg.trainer, self.cfg.generator
        mo = dict(t.policy.model_overrides)
        tp_e_cfg = g.inference_engine.tensor_parallel_size or self.ps.tp
        if tp_e_cfg != self.ps.tp:
            mo.setdefault("tp_invariant", True)     # two degrees, one set of bits: the K reductions use the leaf tree
        if (t.policy.parallel.sequence_parallel or os.environ.get("SKYRL_ISOEXEC_TRAINER_SP", "0") == "1") and self.ps.tp > 1:
            mo.setdefault("sequence_parallel", True)
        mcfg = get_config(t.policy.model, **mo)
        if mcfg.sequence_parallel and (mcfg.has_moe or mcfg.has_gdn or mcfg.is_mla):
            raise ValueError("sequence_parallel=true is built for dense attention models; this model has MoE, GatedDeltaNet or "
                             "latent-attention layers")
        if t.isoexec.debug_trace:
            # region digests of both sides of every forward, one file per rank, for debug/compare.py
            from ..debug import trace as _trace

            _trace.install("trainer", self.rank, t.isoexec.debug_trace)
        tp_e = self._engine_layout(mcfg)
        self._setup_transports(mcfg)
        flat_alloc = self._flat_rendezvous = None
        if self.separate_engine and self.device.type == "cuda" and self.ps.tp > 1 and g.inference_engine.weight_sync_backend != "nccl_gather":
            from ..parallel import nccl_runtime

            if nccl_runtime.capabilities()["symmetric_memory"]:
                from ..sync.reshard import symmetric_flat_allocator

                flat_alloc, self._flat_rendezvous = symmetric_flat_allocator(self.ps.tp_group)
        if self.ps.pp > 1:
            from ..parallel.pp import build_stage_model

            model = build_stage_model(mcfg, self.ps, self.device, seed=t.policy.seed)
        else:
            model = DecoderLM(mcfg, self.ps, self.device, seed=t.policy.seed, flat_alloc=flat_alloc)
        if os.path.isdir(t.policy.model) and self.ps.pp == 1:
            # trainer.policy.model names a checkpoint directory: its config.json gave the architecture, its weights are the
            # starting point (a directory with a config only starts from the seeded random init)
            from ..models import hf_export

            if hf_export.has_hf_weights(t.policy.model):
                hf_export.load_hf(model, t.policy.model)
        wcfg = WorkerConfig(max_tokens_per_microbatch=t.max_tokens_per_microbatch, optimizer=t.policy.optimizer_config,
                            keep_last_layers=t.policy.keep_last_layers, shard_optimizer=t.policy.shard_optimizer,
                            want_entropy=t.algorithm.use_entropy_loss, logprob_chunk_rows=t.logprobs_chunk_size,
                            moe_aux_loss_coeff=t.policy.moe_aux_loss_coeff, freeze_moe_router=t.policy.freeze_moe_router,
                            temperature=(t.algorithm.temperature if t.algorithm.temperature is not None else g.sampling_params.temperature) or 1.0)
        from .config import COMPAT_NOTES

        if COMPAT_NOTES and self.rank == 0 and not getattr(RayPPOTrainer, "_compat_said", False):
            RayPPOTrainer._compat_said = True
            print(f"[config] {len(COMPAT_NOTES)} keys of the reference's config tree were accepted without effect here "
                  f"(machinery this framework does not have), e.g. {COMPAT_NOTES[0].split(':')[0]}")
        algo = t.algorithm
        if not algo.max_seq_len:
            algo.max_seq_len = t.max_prompt_length + g.sampling_params.max_generate_length
        if self.ps.pp > 1:
            from ..parallel.pp import PipelinePolicyWorker

            self.policy = PipelinePolicyWorker(model, wcfg, algo)
        else:
            self.policy = PolicyWorker(model, wcfg, algo)
        self.ref = self.critic = None
        self.lora_store = None
        if t.policy.lora.rank > 0:
            from .lora import DEFAULT_TARGETS, AdapterStore, LoRAAdapter, LoRAConfig, LoRATrainer

            ls = t.policy.lora
            targets = DEFAULT_TARGETS if ls.target_modules in ("all-linear", "", "all") else tuple(x.strip() for x in ls.target_modules.split(",") if x.strip())
            self.lora_store = AdapterStore(model)
            self.lora_store.register("policy", LoRAAdapter.init(model, LoRAConfig(rank=ls.rank, alpha=ls.alpha, targets=targets,
                                                                                  lr=ls.lr or t.policy.optimizer_config.lr, seed=ls.seed)))
            self.lora_store.activate("policy")
            self.policy.lora = LoRATrainer(self.policy, self.lora_store, "policy")
        if algo.use_kl_loss or algo.use_kl_in_reward:
            from .ref_critic import RefWorker

            if t.ref.model or t.ref.hf_path:   # a different frozen model (a teacher): same vocabulary, its own weights
                from ..models import hf_export

                rcfg = get_config(t.ref.model, **t.ref.model_overrides) if t.ref.model else \
                    (mcfg.with_(**t.ref.model_overrides) if t.ref.model_overrides else mcfg)
                assert rcfg.vocab_size == mcfg.vocab_size, "the reference / teacher model must share the policy's vocabulary"
                rmodel = DecoderLM(rcfg, self.ps, self.device, seed=t.ref.seed)
                if t.ref.hf_path:
                    hf_export.load_hf(rmodel, t.ref.hf_path)
                self.ref = RefWorker(rmodel, wcfg)
            else:
                self.ref = RefWorker.from_policy(model, wcfg)
        if algo.advantage_estimator == "gae":
            from .ref_critic import CriticWorker

            ccfg = get_config(t.critic.model, **t.critic.model_overrides) if t.critic.model else \
                (mcfg.with_(**t.critic.model_overrides) if t.critic.model_overrides else mcfg)
            cmodel = DecoderLM(ccfg, self.ps, self.device, seed=t.policy.seed + 1)
            if t.critic.hf_path:
                from ..models import hf_export

                hf_export.load_hf(cmodel, t.critic.hf_path)
            import dataclasses as _dc

            self.critic = CriticWorker(cmodel, _dc.replace(wcfg, optimizer=t.critic.optimizer_config), algo)
        # the controller drives its workers through one dispatch object (verbs + residency of optimizer state)
        from .worker_dispatch import WorkerDispatch

        self.dispatch = WorkerDispatch({"policy": self.policy, "critic": self.critic, "ref": self.ref},
                                       colocate_all=bool(t.placement.colocate_all and t.placement.offload_optimizer),
                                       sync_fn=self.sync_weights)
        ie = g.inference_engine
        ecfg = EngineConfig(max_num_seqs=ie.max_num_seqs, max_num_batched_tokens=ie.max_num_batched_tokens,
                            num_kv_pages=ie.num_kv_pages, gpu_memory_utilization=ie.gpu_memory_utilization,
                            # one sampler stream per engine; the ranks of one engine share it
                            seed=t.seed + 7919 * self._engine_index(),
                            enable_prefix_caching=ie.enable_prefix_caching,
                            use_cuda_graph=not ie.enforce_eager, share_prompt_pages=ie.share_prompt_pages, share_recurrent_state=ie.share_recurrent_state,
                            # a multi-turn context grows to generator.max_input_length before its last turn
                            max_model_len=min(mcfg.max_position, (max(t.max_prompt_length, g.max_input_length) if (g.max_turns > 1 or not g.batched)
                                                                  else t.max_prompt_length) + g.sampling_params.max_generate_length + 1))
        self.remote_engines = not ie.run_engines_locally
        if self.remote_engines:
            # rollouts on servers this job does not own: generation over HTTP, weights through a shared directory
            from .remote_engines import RemoteEngines

            wdir = ie.remote_weights_dir or os.path.join(t.ckpt_path, "remote_weights")
            self.engine = RemoteEngines(list(ie.remote_urls), wdir, rank=self.rank)
            self.infer = self.engine.client
            self.separate_engine = False
        elif self.separate_engine:
            # engines of their own layout: a second set of (sharded) weights per GPU, filled by the resharding sync
            emodel = DecoderLM(mcfg, self.engine_ps, self.device, seed=t.policy.seed, init=False)
            self.engine = LLMEngine(emodel, ecfg)
        else:
            # colocated, same TP layout: the engine computes with the trainer's flat parameter buffer
            self.engine = LLMEngine(model, ecfg)
        self.http_server, self.http_endpoint_url = None, ""
        if not self.remote_engines:
            self.infer = NativeInferenceEngine(self.engine, self.tokenizer)
            if ie.enable_http_endpoint:
                # the engine behind HTTP: a server thread steps it whenever requests are queued; the trainer's generator is
                # one more client of that endpoint (reference: enable_http_endpoint of the inference engine client)
                from ..engine.server import InferenceServer, RemoteInferenceClient

                if self.engines_per_replica > 1 or self.engine_ps.tp > 1:
                    raise ValueError("enable_http_endpoint serves a single-rank engine (tensor_parallel_size = 1)")
                self.http_server = InferenceServer(self.engine, self.tokenizer, ie.http_endpoint_host, ie.http_endpoint_port,
                                                   model_name=mcfg.name).start()
                self.http_endpoint_url = self.http_server.url
                self.infer = RemoteInferenceClient([self.http_endpoint_url])
        if g.chat_template and self.tokenizer is not None:
            from .generator_utils import get_custom_chat_template

            tpl = get_custom_chat_template(g.chat_template)
            if tpl is not None:
                if not hasattr(self.tokenizer, "chat_template"):
                    raise ValueError("generator.chat_template needs a tokenizer with a settable chat template (a Hugging Face tokenizer)")
                self.tokenizer.chat_template = tpl
        # a multi-turn trajectory stops taking turns once its context reaches this many tokens (stop reason "length"): the
        # configured bound, but never more than the engine can hold
        mil = min(max(g.max_input_length, t.max_prompt_length), int(getattr(self.engine, "max_len", 1 << 30)) - 1)
        if g.multimodal:
            from .vlm_generator import SkyRLVLMGymGenerator

            if not mcfg.has_vision:
                raise ValueError(f"generator.multimodal=true but model {mcfg.name!r} has no vision tower")
            self.generator = SkyRLVLMGymGenerator(self.infer, self.tokenizer, max_turns=g.max_turns,
                                                  append_eos_after_stop_str=g.append_eos_token_after_stop_str_in_multi_turn,
                                                  env_config=self.cfg.environment.env_kwargs,
                                                  zero_reward_on_non_stop=g.zero_reward_on_non_stop,
                                                  apply_overlong_filtering=g.apply_overlong_filtering, rate_limit=g.rate_limit or None, max_input_length=mil)
        elif g.rlm:
            from .rlm_generator import RLMGymGenerator

            self.generator = RLMGymGenerator(self.infer, self.tokenizer, max_turns=g.max_turns, max_depth=g.rlm_max_depth,
                                             lm_max_tokens=g.rlm_lm_max_tokens, train_children=g.rlm_train_children,
                                             env_config=self.cfg.environment.env_kwargs, zero_reward_on_non_stop=g.zero_reward_on_non_stop,
                                             apply_overlong_filtering=g.apply_overlong_filtering, rate_limit=g.rate_limit or None, max_input_length=mil)
        else:
            self.generator = SkyRLGymGenerator(self.infer, self.tokenizer, max_turns=g.max_turns, batched=g.batched,
                                               env_config=self.cfg.environment.env_kwargs,
                                               zero_reward_on_non_stop=g.zero_reward_on_non_stop,
                                               apply_overlong_filtering=g.apply_overlong_filtering,
                                               rate_limit=g.rate_limit or None, max_input_length=mil, step_wise=g.step_wise_trajectories)
        self.generator.chat_template_kwargs = dict(g.chat_template_kwargs or {})
        if t.isoexec.enabled:
            self.adapter_trainer = ContractAdapter("trainer", model, self.rank, trainer_tp=self.ps.tp, engine_tp=tp_e, trainer_pp=self.ps.pp)
            self.adapter_trainer.run_install()
            self.adapter_engine = ContractAdapter("engine", self.engine.model, self.rank, trainer_tp=self.ps.tp, engine_tp=tp_e,
                                                  trainer_pp=self.ps.pp)
            self.adapter_engine.run_install()
            if t.isoexec.contract_path and self.rank == 0:
                # the frozen contract as an artifact beside the run (R/.../isoexec/core/process.py write_contract)
                from ..core import process as _process

                _process.write_contract(self.adapter_trainer.contract, t.isoexec.contract_path)
            # the admitted steady-state signature of this (model, contract, arch): under the contract the band of the
            # mean |rollout - train| logprob difference is exactly zero (R/.../isoexec/core/signatures.py:48-131)
            from ..core.signatures import bitwise_table

            self._sig_key = (mcfg.name, self.adapter_trainer.contract.identities.numerical_policy, self.adapter_trainer.arch)
            self.signatures = bitwise_table(*self._sig_key, proof_ref="tests/test_train_cpu.py::test_grpo_loop_is_bitwise_on_policy_and_resumes")
        if t.isoexec.enabled and t.isoexec.mm_admission and self.device.type == "cuda":
            from ..core import mm_admission

            self.mm_admitted = {}
            for deg in sorted({self.ps.tp, self.engine_ps.tp if self.separate_engine else self.ps.tp}):
                rep = mm_admission.admit(mcfg, str(self.device), tp=deg, ep=self.ps.ep)
                self.mm_admitted[deg] = rep
                bad = mm_admission.refused(rep)
                if bad:
                    raise RuntimeError(f"GEMM admission refused at tp={deg}: rows of {bad} depend on the batch they are computed in")
        if self.dataset is None:
            d = self.cfg.data
            n = d.synthetic_prompts or t.train_batch_size * 4
            self.dataset = SyntheticPromptDataset(n, d.synthetic_prompt_len, mcfg.vocab_size, t.seed,
                                                  self.cfg.environment.env_class)
        per_rank = t.train_batch_size // self.ps.dp if self.ps.dp > 1 else t.train_batch_size
        self.loader = PromptDataLoader(self.dataset, per_rank, t.seed, part=self.ps.dp_rank, parts=self.ps.dp)
        self.init_weight_sync_state()
        self._census0 = _observe.snapshot()

    def init_weight_sync_state(self) -> None:
        """Stamp the trainer's contract hash on the init message; the engine's receiver refuses a mismatch."""
        iso = self.cfg.trainer.isoexec.enabled
        self.resharder = None
        if self.separate_engine:
            from ..sync import reshard as R

            info = S.ReshardInitInfo(contract_hash=P.contract_hash() if iso else None, engine_tp=self.engine_ps.tp, trainer_tp=self.ps.tp)
            if iso:
                P.assert_init_info_contract(info)          # engine side of the handshake
            if self.ps.pp > 1:
                self.resharder = R.PipelineStageSync(self.policy.model, self.engine.model, self.ps)
            elif self._flat_rendezvous is not None:
                ptrs, self._flat_handle = self._flat_rendezvous(self.policy.model.store.flat)
                self.resharder = R.PeerPullResharder(self.policy.model, self.engine.model, self.ps.tp_group, self.ps.tp_rank, ptrs)
            else:
                self.resharder = R.CollectiveResharder(self.policy.model, self.engine.model, self.ps.tp_group, self.ps.tp_rank)
            self.sync_info = info
            return
        info = S.create_init_info("shared") if iso else S.SharedInitInfo(contract_hash=None)
        self.sync_info = info
        if iso:
            self.receiver = S.create_receiver(info, self.engine.model)
        self.sender = S.create_sender(info, self.policy.model)

    # ------------------------------------------------------------------ one step, phase by phase
    def prepare_generator_input(self, rows: list[dict]) -> tuple[GeneratorInput, list[str]]:
        n = self.cfg.generator.n_samples_per_prompt
        sp = self.cfg.generator.sampling_params
        prompts, envs, extras, uids = [], [], [], []
        for r in rows:
            for _ in range(n):
                prompts.append(r["prompt"])
                envs.append(r["env_class"])
                extras.append(r.get("env_extras") or {})
                uids.append(r["uid"])
        gi: GeneratorInput = {"prompts": prompts, "env_classes": envs, "env_extras": extras,
                              "sampling_params": {"max_generate_length": sp.max_generate_length, "temperature": sp.temperature,
                                                  "top_p": sp.top_p, "top_k": sp.top_k, "min_p": sp.min_p,
                                                  "ignore_eos": sp.ignore_eos},
                              "trajectory_ids": None, "batch_metadata": {"global_step": self.global_step}}
        return gi, uids

    def generate(self, gi: GeneratorInput) -> GeneratorOutput:
        if self.engines_per_replica == 1:
            return asyncio.run(self.generator.generate(gi))
        # several engines serve one trainer replica: each takes a contiguous slice of the replica's requests, then the
        # slices are exchanged inside the trainer's tensor-parallel group so that every rank trains on the whole batch
        from .generator import get_rollout_metrics
        from .trainer_utils import _cat, _take

        k, n = self.engines_per_replica, len(gi["prompts"])
        e = self.replica_rank if self._every_rank_leads else self.ps.tp_rank // self.engine_ps.tp
        lo, hi = e * n // k, (e + 1) * n // k
        part = dict(gi)
        for key in ("prompts", "env_classes", "env_extras", "trajectory_ids"):
            if isinstance(gi.get(key), list):
                part[key] = gi[key][lo:hi]
        go = asyncio.run(self.generator.generate(part))
        go.pop("rollout_metrics", None)
        box = [None] * self.replica_size
        lead = True if self._every_rank_leads else self.engine_ps.tp_rank == 0      # one copy per engine
        dist.all_gather_object(box, go if lead else None, group=self.replica_group)
        merged = None
        for g_ in box:
            if g_ is not None:
                merged = _cat(merged, g_)
        assert merged is not None and len(merged["response_ids"]) == n or self.cfg.generator.step_wise_trajectories
        last = merged.get("is_last_step") or [True] * len(merged["response_ids"])
        sel = [i for i, f in enumerate(last) if f]
        merged["rollout_metrics"] = get_rollout_metrics([merged["response_ids"][i] for i in sel], [merged["rewards"][i] for i in sel],
                                                        [merged["env_metrics"][i] for i in sel] if merged.get("env_metrics") else None)
        return merged

    def balance_rollouts(self, go: GeneratorOutput, uids: list[str]):
        """Length-balanced data parallelism (reference: B/utils/ep_balance.py, DP row striping by length): the rollouts of
        all data-parallel ranks are pooled, whole prompt groups (the samples of one prompt stay together, as the group
        statistics of the advantage need them) are dealt out longest first in a serpentine, and every rank continues
        with its share: same number of groups everywhere, nearly the same number of tokens. Returns (go, uids)."""
        from .moe_utils import balanced_dp_assignment, imbalance

        ps = self.ps
        if ps.dp == 1 or go.get("step_source") is not None:
            return go, uids
        B = len(uids)
        cols = {k: v for k, v in go.items() if isinstance(v, list) and len(v) == B}
        pooled: list = [None] * ps.dp
        dist.all_gather_object(pooled, (cols, list(uids)), group=ps.dp_group)
        groups: dict = {}
        for r, (c, u) in enumerate(pooled):
            for i, uid in enumerate(u):
                groups.setdefault((r, uid), []).append((r, i))                 # uids repeat across ranks: keep the origin
        keys = list(groups)
        lens = [sum(len(pooled[r][0]["prompt_token_ids"][i]) + len(pooled[r][0]["response_ids"][i]) for r, i in groups[k]) for k in keys]
        if len(keys) % ps.dp:
            return go, uids
        assign = balanced_dp_assignment(lens, ps.dp)
        before = imbalance(lens, [[j for j, k in enumerate(keys) if k[0] == r] for r in range(ps.dp)])
        mine = sorted(assign[ps.dp_rank])
        out = dict(go)
        for k in cols:
            out[k] = [pooled[r][0][k][i] for j in mine for r, i in groups[keys[j]]]
        new_uids = [f"{keys[j][0]}:{keys[j][1]}" for j in mine for _ in groups[keys[j]]]
        self.all_metrics["generate/dp_token_imbalance_before"] = before
        self.all_metrics["generate/dp_token_imbalance_after"] = imbalance(lens, assign)
        return out, new_uids

    def convert_to_training_input(self, go: GeneratorOutput, uids: list[str]) -> TrainingInputBatch:
        cfg = getattr(self, "cfg", None)
        if go.get("step_source") is not None and cfg is not None and cfg.generator.merge_stepwise_output and cfg.generator.step_wise_trajectories:
            # step-wise rollouts, trained as whole trajectories: the turns of a trajectory are joined again (observation
            # tokens get loss mask 0), one row and one uid per trajectory
            from .generator_utils import merge_stepwise_output

            go = dict(go)
            if go.get("trajectory_ids") is None:
                go["trajectory_ids"] = list(go["step_source"])
            first = {}
            for tid, src in zip(go["trajectory_ids"], go["step_source"]):
                first.setdefault(tid, src)
            go = merge_stepwise_output(go)
            uids = [uids[first[tid]] for tid in go["trajectory_ids"]]
        seq, att, rmask = build_sequences(go["prompt_token_ids"], go["response_ids"])
        B, R = rmask.shape
        loss_mask = torch.zeros(B, R)
        rewards = torch.zeros(B, R)
        rollout_lp = torch.zeros(B, R)
        for i in range(B):
            n = len(go["response_ids"][i])
            loss_mask[i, :n] = torch.tensor(go["loss_masks"][i], dtype=torch.float32)
            r = go["rewards"][i]
            if isinstance(r, (list, tuple)):
                rewards[i, :n] = torch.tensor(r, dtype=torch.float32)
            elif n > 0:
                rewards[i, n - 1] = float(r)     # outcome reward sits on the last response token
            if go.get("rollout_logprobs") is not None:
                rollout_lp[i, :n] = torch.tensor(go["rollout_logprobs"][i], dtype=torch.float32)
        fields = {"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": loss_mask,
                  "rewards": rewards, "rollout_logprobs": rollout_lp}
        if go.get("pixel_values") is not None:
            # vision-language rollouts: per sample, the patches and grids of its images and where the placeholder tokens
            # are (reference: R/train/trainer.py:913-966). Positions count from the first prompt token, which is where the
            # packed forward starts a sequence, so a prompt must not have been cut from the left
            from .batch import TensorList

            if go.get("image_grid_thw") is None or len(go["pixel_values"]) != B or len(go["image_grid_thw"]) != B:
                raise ValueError("pixel_values and image_grid_thw must both be given, one entry per sample")
            fields["pixel_values"] = TensorList(list(go["pixel_values"]))
            fields["image_grid_thw"] = TensorList(list(go["image_grid_thw"]))
            if go.get("mm_positions") is not None:
                fields["mm_positions"] = TensorList([torch.as_tensor(p, dtype=torch.int64) for p in go["mm_positions"]])
        b = TrainingInputBatch(fields)
        lens = rmask.sum(1)
        b.metadata = {"uids": list(uids), "response_length": R, "avg_response_length": float(lens.mean()),
                      "max_response_length": int(lens.max())}
        if go.get("step_source") is not None:       # step-wise: one row per model turn; a row inherits its trajectory's uid
            b.metadata["uids"] = [uids[i] for i in go["step_source"]]
            b.metadata["is_last_step"] = list(go["is_last_step"])
        return b

    def _reuse_rollout_logprobs(self) -> bool:
        """The scoring forward may be dropped only when the rollout policy IS the policy being updated: contract
        enforced, one optimizer step per rollout batch."""
        t = self.cfg.trainer
        return bool(t.isoexec.enabled and t.isoexec.reuse_rollout_logprobs and t.update_epochs_per_batch == 1
                    and t.policy_mini_batch_size >= t.train_batch_size)

    def fwd_logprobs_values_reward(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        self._gate_in_update = self._reuse_rollout_logprobs()
        if self._gate_in_update:
            # old-policy logprobs = the engine's, which the contract makes the trainer's bit for bit; the gate runs on the
            # training forward (train_critic_and_policy), before the optimizer step
            lp = batch["rollout_logprobs"].clone()
        else:
            lp = self.dispatch.forward("policy", batch)
        batch["action_log_probs"] = lp
        rmask = batch["response_mask"]
        # the gate and the diff metrics look at the tokens the loss trains on (R/train/trainer.py:1544-1546): observation
        # tokens of a multi-turn rollout sit inside response_mask with a placeholder rollout logprob of 0 and loss mask 0
        lm = batch.get("loss_mask")
        mask = ((lm > 0) & (rmask > 0)).to(lp.dtype) if lm is not None else rmask
        ro = batch["rollout_logprobs"]
        diff = (lp - ro).abs() * mask
        nsel = float(mask.sum())
        n = mask.sum().clamp(min=1)
        mean = diff.sum() / n
        std = ((diff - mean).pow(2) * mask).sum().div(n).sqrt()
        sel = mask > 0            # select, do not multiply: -x * 0 is -0.0, whose bits differ from the placeholder +0.0
        z = torch.zeros_like(lp)
        mism = count_bit_mismatches(torch.where(sel, lp, z).contiguous(), torch.where(sel, ro, z).contiguous()) if nsel > 0 else 0
        self.all_metrics.update({
            "policy/rollout_train_logprobs_abs_diff_max": float(diff.max()) if diff.numel() and nsel > 0 else 0.0,
            "policy/rollout_train_logprobs_abs_diff_min": float(diff[mask > 0].min()) if nsel > 0 else 0.0,
            "policy/rollout_train_logprobs_abs_diff_mean": float(mean),
            "policy/rollout_train_logprobs_abs_diff_std": float(std),
            "policy/rollout_train_logprob_bit_mismatches": mism,
        })
        a = self.cfg.trainer.algorithm
        if getattr(self, "ref", None) is not None:
            batch["base_action_log_probs"] = self.dispatch.forward("ref", batch)
            if a.use_kl_in_reward:
                batch["action_log_probs"] = lp
                batch = self.apply_reward_kl_penalty(batch)
        if getattr(self, "critic", None) is not None:
            batch["values"] = self.dispatch.forward("critic", batch) * rmask
        iso = self.cfg.trainer.isoexec
        if iso.enabled and not self._gate_in_update:
            gate = validate_isoexec_forward_gate(diff, mask, mism, iso)
            if iso.require_bitwise and getattr(self, "signatures", None) is not None:
                sig_ok, why = self.signatures.check(*self._sig_key, gate["mean"])
                if not sig_ok:
                    gate["ok"] = False
                    gate["signature"] = why
            if self.global_step <= 1 and hasattr(self, "adapter_trainer"):
                self.adapter_trainer.on_gate(gate["ok"], f"mean={gate['mean']:.3e} max={gate['max']:.3e} "
                                                           f"mismatches={gate['mismatches']}")
            if not gate["ok"]:
                msg = (f"IsoExec forward gate refused at step {self.global_step}: mean={gate['mean']:.3e} "
                       f"max={gate['max']:.3e} bit mismatches={gate['mismatches']}")
                if iso.strict:
                    raise ForwardGateError(msg)
                print("[warn] " + msg)
        return batch

    def apply_reward_kl_penalty(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        """Subtract ``kl_coef * KL(policy || reference)`` per token from the rewards (R/train/trainer.py
        ``apply_reward_kl_penalty``); a seam that subclasses replace (on-policy distillation makes it THE reward)."""
        a = self.cfg.trainer.algorithm
        lp, mask = batch["action_log_probs"], batch["response_mask"]
        kl = alg.compute_approx_kl(lp, batch["base_action_log_probs"], mask, a.kl_estimator_type) * mask
        batch["rewards"] = batch["rewards"] - self.kl_ctrl.value * kl
        cur = float(kl.sum() / mask.sum().clamp(min=1))
        self.kl_ctrl.update(cur, int(mask.shape[0]))
        self.all_metrics.update({"reward/kl": cur, "reward/kl_coef": self.kl_ctrl.value})
        return batch

    def compute_advantages_and_returns(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        a = self.cfg.trainer.algorithm
        last = batch.metadata.get("is_last_step")
        if last is not None:
            # step-wise (R/train/trainer.py:1179-1218): the advantage of a trajectory comes from its LAST step's reward,
            # compared within the prompt's group, and is given to every response token of every step of that trajectory
            is_last = torch.tensor(last, dtype=torch.bool)
            assert bool(is_last[-1]), "the last row must close a trajectory"
            uids = batch.metadata["uids"]
            adv_l, ret_l = alg.compute_advantages_and_returns(
                batch["rewards"][is_last], torch.ones_like(batch["response_mask"][is_last], dtype=torch.float32),
                [u for u, f in zip(uids, last) if f], a.advantage_estimator, a, values=None)
            traj = torch.cat([torch.zeros(1, dtype=torch.bool), is_last[:-1]]).long().cumsum(0)
            assert int(traj[-1]) + 1 == adv_l.shape[0]
            rm = batch["response_mask"].to(adv_l.dtype)
            adv, ret = adv_l[traj] * rm, ret_l[traj] * rm
        else:
            adv, ret = alg.compute_advantages_and_returns(batch["rewards"], batch["response_mask"], batch.metadata["uids"],
                                                          a.advantage_estimator, a, values=batch.get("values"))
        m = batch["response_mask"]
        if a.zero_variance_filter and last is None:
            # groups whose samples all scored the same teach nothing under a group baseline: their loss mask goes to zero
            # (reference: R/train/trainer.py:1123-1138)
            tot = batch["rewards"].sum(-1)
            by_uid: dict = {}
            for i, u in enumerate(batch.metadata["uids"]):
                by_uid.setdefault(u, []).append(i)
            dead = [i for idx in by_uid.values() if len(idx) > 1 and float(tot[idx].max() - tot[idx].min()) <= a.zero_variance_filter_tol for i in idx]
            if dead and batch.get("loss_mask") is not None:
                batch["loss_mask"][torch.tensor(dead)] = 0
            self.all_metrics["reward/num_zero_variance_filtered"] = len({batch.metadata["uids"][i] for i in dead})
        if a.advantage_batch_normalize:
            # z-score over every response token of the global batch (reference: R/train/trainer.py:1659-1664)
            mf = m.to(adv.dtype)
            n = max(1.0, self._global_sum(float(mf.sum())))
            mean = self._global_sum(float((adv * mf).sum())) / n
            var = self._global_sum(float((((adv - mean) ** 2) * mf).sum())) / n
            adv = (adv - mean) * (max(var, 1e-8) ** -0.5) * mf
        batch["advantages"], batch["returns"] = adv, ret
        scores = batch["rewards"].sum(-1)
        if last is not None:
            scores = scores[torch.tensor(last, dtype=torch.bool)]
        self.all_metrics.update({"reward/avg_raw_reward": float(scores.mean()),
                                 "reward/avg_pass_rate": float((scores > 0).float().mean()),
                                 "policy/avg_advantage_abs": float((adv.abs() * m).sum() / m.sum().clamp(min=1))})
        return batch

    def update_ref_with_policy(self) -> None:
        """The reference model takes the policy's current weights (``trainer.update_ref_every_epoch``; reference:
        R/train/trainer.py ``update_ref_with_policy``). Both must have the same architecture and layout."""
        src, dst = self.policy.model.store.flat, self.ref.model.store.flat
        if src.shape != dst.shape:
            raise ValueError("update_ref_every_epoch needs a reference model of the policy's own architecture")
        with torch.no_grad():
            dst.copy_(src)

    def _global_sum(self, x: float) -> float:
        if self.ps.dp > 1:
            t = torch.tensor([x], dtype=torch.float64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, group=self.ps.dp_group)
            return float(t.item())
        return x

    def _global_max(self, x: float) -> float:
        if self.ps.dp > 1:
            t = torch.tensor([x], dtype=torch.float64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.ps.dp_group)
            return float(t.item())
        return x

    def train_critic_and_policy(self, batch: TrainingInputBatch) -> dict:
        t, a = self.cfg.trainer, self.cfg.trainer.algorithm
        n_samples = self.cfg.generator.n_samples_per_prompt
        mb_seqs = (t.policy_mini_batch_size * n_samples) // max(1, self.ps.dp)
        B = batch.batch_size
        out = {"policy_loss": 0.0, "ppo_clip_ratio": 0.0, "grad_norm": 0.0, "policy_entropy": 0.0, "policy_kl": 0.0}
        post = {"sum": 0.0, "sq": 0.0, "max": 0.0, "tokens": 0.0}
        n_updates = 0
        if getattr(self, "critic", None) is not None:
            closs = 0.0
            cmb = (t.critic_mini_batch_size * n_samples) // max(1, self.ps.dp) if t.critic_mini_batch_size > 0 else mb_seqs
            for lo in range(0, B, cmb):
                cm = self.dispatch.forward_backward("critic", batch.slice(lo, min(B, lo + cmb)))
                self.dispatch.optim_step("critic")
                closs += cm["critic_loss"]
            self.all_metrics["critic/critic_loss"] = closs / max(1, (B + cmb - 1) // cmb)
        for _epoch in range(t.update_epochs_per_batch):
            for lo in range(0, B, mb_seqs):
                mb = batch.slice(lo, min(B, lo + mb_seqs))
                lm = mb["loss_mask"]
                # mean-type reductions by advantage pre-scaling, with GLOBAL mini-batch statistics
                if a.loss_reduction == "token_mean":
                    tot = self._global_sum(float(lm.sum()))
                    mb["advantages"] = mb["advantages"] / max(1.0, tot)
                    mb.metadata["aux_loss_scale"] = 1.0 / max(1.0, tot)
                else:
                    gB = int(self._global_sum(float(mb.batch_size)))
                    pb = None
                    if a.loss_reduction == "prompt_mean":
                        from .dataset import compute_prompt_boundaries

                        pb = compute_prompt_boundaries(batch.metadata["uids"][lo:min(B, lo + mb_seqs)])
                    scaled = alg.apply_loss_reduction_to_advantages(mb["advantages"], lm, a.loss_reduction,
                                                                    t.micro_train_batch_size_per_gpu, a.max_seq_len,
                                                                    prompt_boundaries=pb)
                    mb["advantages"] = scaled * (mb.batch_size / max(1, gB))
                    mb.metadata["aux_loss_scale"] = 1.0 / max(1.0, self._global_sum(float(lm.sum())))
                if getattr(self, "_gate_in_update", False):
                    mb.metadata["check_rollout_bits"] = True
                if t.recompute_old_logprobs_per_minibatch and n_updates > 0:
                    # the policy has moved since the batch was scored: take the old-policy logprobs of this mini-batch
                    # from the CURRENT weights, so the ratio of its first update is exactly 1 (R/train/trainer.py:1610-1640)
                    mb["action_log_probs"] = self.dispatch.forward("policy", mb)
                m = self.dispatch.forward_backward("policy", mb)
                if getattr(self, "_gate_in_update", False):
                    self._gate_on_training_forward(m["rollout_bits"])      # raises before the weights move
                gn = self.dispatch.optim_step("policy")
                out["policy_loss"] += m["policy_loss"]
                out["ppo_clip_ratio"] += m["ppo_clip_ratio"]
                out["policy_entropy"] += m["policy_entropy"]
                out["policy_kl"] += m["policy_kl"]
                out["grad_norm"] += gn
                n_updates += 1
                if "moe_aux_loss" in m:
                    out["moe_aux_loss"] = out.get("moe_aux_loss", 0.0) + m["moe_aux_loss"]
                if m.get("post_update_diff"):
                    for k_ in ("sum", "sq", "tokens"):
                        post[k_] += m["post_update_diff"][k_]
                    post["max"] = max(post["max"], m["post_update_diff"]["max"])
        for k in out:
            out[k] /= max(1, n_updates)
        out["policy_loss"] = self._global_sum(out["policy_loss"])
        self.all_metrics.update({f"policy/{k}": v for k, v in out.items()})
        ntok = self._global_sum(post["tokens"])
        if ntok > 0:
            mean = self._global_sum(post["sum"]) / ntok
            var = max(0.0, self._global_sum(post["sq"]) / ntok - mean * mean)
            self.all_metrics.update({"policy/post_update_rollout_logprobs_abs_diff_mean": mean,
                                     "policy/post_update_rollout_logprobs_abs_diff_std": var ** 0.5,
                                     "policy/post_update_rollout_logprobs_abs_diff_max": self._global_max(post["max"])})
        self.all_metrics["policy/policy_lr"] = self.policy.opt.lr_at(max(0, self.policy.opt.step_count - 1))
        return out

    def _gate_on_training_forward(self, bits: dict) -> None:
        """Forward gate when the scoring forward is skipped: the training forward's logprobs against the rollout's."""
        iso = self.cfg.trainer.isoexec
        mism = int(self._global_sum(float(bits["mismatches"])))
        ntok = max(1.0, self._global_sum(bits["tokens"]))
        mean = self._global_sum(bits["abs_sum"]) / ntok
        mx = bits["abs_max"]
        if self.ps.dp > 1:
            t = torch.tensor([mx], dtype=torch.float64, device=self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.ps.dp_group)
            mx = float(t)
        self.all_metrics.update({"policy/rollout_train_logprob_bit_mismatches": mism,
                                 "policy/rollout_train_logprobs_abs_diff_mean": mean,
                                 "policy/rollout_train_logprobs_abs_diff_max": mx,
                                 "policy/scoring_forward_skipped": 1})
        ok = mean <= iso.gate_mean_limit and mx <= iso.gate_max_limit and (mism == 0 or not iso.require_bitwise)
        if self.global_step <= 1 and hasattr(self, "adapter_trainer"):
            self.adapter_trainer.on_gate(ok, f"mean={mean:.3e} max={mx:.3e} mismatches={mism} (training forward)")
        if not ok:
            msg = (f"IsoExec forward gate refused at step {self.global_step} (training forward vs rollout): mean={mean:.3e} "
                   f"max={mx:.3e} bit mismatches={mism}")
            if iso.strict:
                raise ForwardGateError(msg)
            print("[warn] " + msg)

    def sync_weights(self) -> None:
        """Trainer -> rollout. Same process and layout: the flat buffer is shared, so the transfer is
        the handshake, the state invalidation and the verification that the alias still holds."""
        iso = self.cfg.trainer.isoexec.enabled
        if getattr(self, "remote_engines", False):
            # every rank takes part in the gather of the shards; one rank writes the file and tells the servers
            self.all_metrics["sync/bytes"] = self.engine.push_weights(self.policy.model, write=self.rank == 0)
            if dist.is_initialized():
                dist.barrier()
            return
        before = self.engine.invalidation_counts()
        if self.separate_engine:
            self.all_metrics["sync/bytes"] = self.resharder.sync()
            self.all_metrics["sync/bytes_from_peers"] = self.resharder.remote_bytes
        else:
            req = self.sender.send_chunks(S.extract_native_weights(self.policy.model, None))
            if iso:
                n = S.load_weights(self.engine.model, ((k, v) for k, v in self.receiver.receive_weights(req)))
                assert n == len(req.names)
        self.engine.reset_prefix_cache()
        if iso:
            # what the invalidation hooks themselves counted during this sync, per state claim of the contract
            after = self.engine.invalidation_counts()
            observed = {s.state_id: after.get(s.state_id, {}).get("weight_sync", 0) > before.get(s.state_id, {}).get("weight_sync", 0)
                        for s in self.adapter_engine.contract.claims.state if "weight_sync" in s.invalidated_by}
            self.adapter_engine.on_weight_sync(self.sync_info.contract_hash, observed)
            self.adapter_trainer.on_weight_sync(P.contract_hash(self.adapter_engine.contract))

    # ------------------------------------------------------------------ the loop
    def _observability(self):
        """Profiler window, NVTX ranges and allocator history, as configured (all off by default)."""
        if getattr(self, "_prof", None) is None:
            from ..utils.profiler import Profiler, start_memory_history

            t = self.cfg.trainer
            self._prof = Profiler(t.profiler, self.rank)
            Timer.nvtx = bool(t.nvtx)
            if t.record_memory:
                start_memory_history()
            self._gpu_mon = None
            if t.gpu_monitor and self.device.type == "cuda":
                from ..utils.gpu_monitor import GpuMonitor

                self._gpu_mon = GpuMonitor(self.device.index or 0, period_s=0.5)
                self._gpu_mon.start()
        return self._prof

    def _ops_of_other_stages(self) -> tuple:
        """Contract ops that this pipeline stage does not execute because the layers that use them live elsewhere."""
        if self.ps.pp == 1:
            return ()
        cfg, ids = self.policy.model.cfg, self.policy.model.layer_ids
        out = []
        if not self.ps.is_last_pp:
            out += ["logprobs.log_softmax", "logprobs.lm_head_slice"]
        kinds = {cfg.layer_type(i) for i in ids}
        if "attn" not in kinds:
            out += ["attention.varlen", "rope.rope", "norms.qk", "activation.attn_gate"]
        if "gdn" not in kinds:
            out += ["gdn.core", "gdn.conv", "gdn.gating", "gdn.state", "norms.gated_out"]
        return tuple(out)

    def _extra_prompts(self, n: int) -> list[dict]:
        """More prompts for dynamic sampling, drawn from a stream of their own (the epoch iterator that feeds
        ``train()`` is not touched): a seeded walk over the dataset, disjoint across data-parallel ranks, that wraps around."""
        if getattr(self, "_extra_rng", None) is None:
            self._extra_rng = random.Random(self.cfg.trainer.seed + 7_654_321)
            self._extra_pool: list[int] = []
        out = []
        while len(out) < n:
            if len(self._extra_pool) < self.ps.dp:
                idx = list(range(len(self.dataset)))
                self._extra_rng.shuffle(idx)
                self._extra_pool += idx
            take = self._extra_pool[:self.ps.dp]           # every rank draws the same numbers and keeps its own column
            del self._extra_pool[:self.ps.dp]
            out.append(self.dataset[take[self.ps.dp_rank]])
        return out

    def train_step(self, rows: list[dict]) -> dict:
        """One full RL step on this rank's prompt shard. Returns the step's metrics."""
        self.all_metrics, self.all_timings = {}, {}
        self._observability().step()
        self.global_step += 1
        T = self.all_timings
        with Timer("step", T):
            with Timer("prepare_input", T):
                gi, uids = self.prepare_generator_input(rows)
            with Timer("wake", T):
                if self.dispatch.colocate_all:
                    self.dispatch.offload_all()           # rollout gets the HBM the optimizer states held
                self.engine.wake_up()
            with Timer("generate", T):
                go = self.generate(gi)
                a = self.cfg.trainer.algorithm
                if a.dynamic_sampling_type:
                    from .trainer_utils import handle_dynamic_sampling

                    state: dict = {}
                    while True:
                        go2, uids2, more = handle_dynamic_sampling(go, uids, a, state, len(rows), self.cfg.generator.n_samples_per_prompt,
                                                                   seed=self.cfg.trainer.seed + self.global_step)
                        if not more:
                            go, uids = go2, uids2
                            break
                        gi, uids = self.prepare_generator_input(self._extra_prompts(len(rows)))
                        go = self.generate(gi)
            with Timer("sleep", T):
                self.engine.sleep()
            every = self.cfg.trainer.log_example_interval
            if every > 0 and self.rank == 0 and self.global_step % every == 0 and go["response_ids"]:
                from ..utils.tracking import log_example

                dec = self.tokenizer.decode if self.tokenizer is not None else str
                log_example(dec(list(go["prompt_token_ids"][0])), dec(list(go["response_ids"][0])), go["rewards"][0])
            with Timer("convert", T):
                if self.cfg.trainer.balance_dp_by_length:
                    go, uids = self.balance_rollouts(go, uids)
                batch = self.convert_to_training_input(go, uids)
            if self.cfg.trainer.dump_data_batch and self.cfg.trainer.ckpt_path:
                from ..utils import io as uio

                with uio.open_file(self.cfg.trainer.ckpt_path.rstrip("/") + f"/dumped_data/global_step_{self.global_step}_rank{self.rank}.pt", "wb") as f:
                    torch.save({"tensors": {k: v for k, v in batch.items() if torch.is_tensor(v)}, "uids": list(uids)}, f)
            if self.global_step == 1 and hasattr(self, "adapter_engine"):
                # everything the op layer ran since the models were built was the engine's (generation)
                self.adapter_engine.on_first_forward(_observe.diff(self._census0))
            c1 = _observe.snapshot()
            with Timer("fwd_logprobs", T):
                batch = self.fwd_logprobs_values_reward(batch)
            if self.global_step == 1 and hasattr(self, "adapter_trainer"):
                if self._reuse_rollout_logprobs():
                    # no scoring forward on this configuration: the trainer's first forward is the training forward,
                    # judged after the update below
                    self._pending_trainer_census = c1
                else:
                    self.adapter_trainer.on_first_forward(_observe.diff(c1), self._ops_of_other_stages())
            with Timer("advantages", T):
                batch = self.compute_advantages_and_returns(batch)
            with Timer("policy_train", T):
                self.train_critic_and_policy(batch)
            if getattr(self, "_pending_trainer_census", None) is not None:
                self.adapter_trainer.on_first_forward(_observe.diff(self._pending_trainer_census), self._ops_of_other_stages())
                self._pending_trainer_census = None
            if self.cfg.trainer.record_memory:
                from ..utils.profiler import save_memory_snapshot

                save_memory_snapshot(self.cfg.trainer.record_memory, f"step{self.global_step}_policy_train", self.rank)
            with Timer("sync_weights", T):
                self.sync_weights()
        t = self.cfg.trainer
        if t.ckpt_path and t.ckpt_interval > 0 and self.global_step % t.ckpt_interval == 0:
            with Timer("save_checkpoints", T):
                self.save_checkpoints()
        self.all_metrics.update(go.get("rollout_metrics") or {})
        ntok = sum(len(r) for r in go["response_ids"])
        self.all_metrics["generate/response_tokens"] = ntok
        self.all_metrics["generate/tokens_per_s"] = ntok / max(1e-9, T["generate"])
        self.all_metrics.update({f"timing/{k}": v for k, v in T.items()})
        if getattr(self, "_gpu_mon", None) is not None:
            g = self._gpu_mon.summary(reset=True)
            self.all_metrics.update({f"gpu/{k}": (",".join(v) if isinstance(v, list) else v) for k, v in g.items()})
        self._fire("on_log", logs=self.all_metrics)
        if self.tracker is not None:
            self.tracker.log(self.all_metrics, self.global_step)
        return dict(self.all_metrics)

    def train(self) -> None:
        if self.policy is None:
            self.build_models()
        t = self.cfg.trainer
        if t.ckpt_path and t.resume_mode != "none":
            self.load_checkpoints()
        self.sync_weights()
        try:
            self._fire("on_train_start")
            if t.eval_before_train:
                self.eval()
            done = False
            for self.epoch in range(getattr(self, "_start_epoch", 0), t.epochs):
                self._fire("on_epoch_start")
                for rows in self.loader:
                    self._fire("on_step_start", batch=rows)
                    metrics = self.train_step(rows)
                    self._fire("on_step_end", batch=rows, metrics=metrics)
                    # the control flags are read once per step, here, and cleared
                    want_save, want_eval = self.control.should_save, self.control.should_evaluate
                    self.control.reset()
                    if want_save and t.ckpt_path and not (t.ckpt_interval > 0 and self.global_step % t.ckpt_interval == 0):
                        self.save_checkpoints()
                    if want_eval or (t.eval_interval > 0 and self.global_step % t.eval_interval == 0):
                        self.eval()
                    if t.export_path and t.hf_save_interval > 0 and self.global_step % t.hf_save_interval == 0:
                        self.export_hf()
                    if t.export_path and t.dcp_save_interval > 0 and self.global_step % t.dcp_save_interval == 0:
                        self.export_dcp()
                    if 0 < t.num_steps <= self.global_step or self.control.should_stop:
                        done = True
                        break
                self._fire("on_epoch_end")
                if t.update_ref_every_epoch and getattr(self, "ref", None) is not None:
                    self.update_ref_with_policy()
                if done:
                    break
            self._fire("on_train_end")
        except BaseException as e:  # noqa: BLE001
            if self.tracker is not None:
                self.tracker.log_exception(e, self.global_step)
            raise
        finally:
            if t.isoexec.enabled and t.ckpt_path and hasattr(self, "adapter_trainer"):
                self.adapter_trainer.ledger.write_verdict(t.ckpt_path)
                self.adapter_engine.ledger.write_verdict(t.ckpt_path)

    # ------------------------------------------------------------------ evaluation / export
    def eval(self) -> dict:
        """Generate on the validation prompts (``eval_dataset`` or the first ``eval_batch_size`` training prompts) with the
        eval sampling parameters and log reward statistics and pass@k."""
        from .evaluate import evaluate

        g = self.cfg.generator
        ds = getattr(self, "eval_dataset", None) or self.dataset
        rows = [ds[i] for i in range(min(len(ds), self.cfg.trainer.eval_batch_size))]
        sp = g.eval_sampling_params
        params = {"max_generate_length": sp.max_generate_length, "temperature": sp.temperature, "top_p": sp.top_p, "top_k": sp.top_k,
                  "min_p": sp.min_p, "ignore_eos": sp.ignore_eos}
        was_asleep = self.engine.asleep
        if was_asleep:
            self.engine.wake_up()
        n = max(1, g.eval_n_samples_per_prompt)
        self._fire("on_eval_start")
        t = self.cfg.trainer
        dump = ""
        if t.dump_eval_results and (t.export_path or t.ckpt_path) and self.rank == 0:
            dump = (t.export_path or t.ckpt_path).rstrip("/") + f"/dumped_evals/global_step_{self.global_step}.jsonl"
        out = evaluate(self.generator, rows, params, n_samples=n, ks=tuple(sorted({1, n})), dump_path=dump,
                       decode=self.tokenizer.decode if self.tokenizer is not None else None)
        if was_asleep:
            self.engine.sleep()
        if self.tracker is not None:
            self.tracker.log(out, self.global_step)
        self.last_eval = out
        self._fire("on_eval_end", metrics=out)
        return out

    def export_hf(self) -> str | None:
        """Write the policy in the Hugging Face layout under ``export_path/global_step_N``. Tensor-parallel shards are
        and expert-parallel shards are gathered (collectives over those groups), global rank 0 writes; pipeline-parallel
        runs are not exported."""
        from ..models import hf_export

        if self.ps.pp > 1:
            return None
        if self.ps.ep == 1 and self.ps.dp_rank != 0:      # plain data-parallel replicas hold copies: one is enough
            return None
        path = os.path.join(self.cfg.trainer.export_path, f"global_step_{self.global_step}")
        hf_export.save_hf(self.policy.model, path, write=self.rank == 0)
        return path if self.rank == 0 else None

    def export_dcp(self) -> str:
        """Policy weights and optimizer state at full shapes as a ``torch.distributed.checkpoint`` directory
        (``export_path/global_step_N/dcp``), readable by torch's own tools and loadable at any layout
        (``trainer.resume_mode=from_path`` with that directory resumes weights, optimizer and the step counter)."""
        from . import dcp_checkpoint

        path = self.cfg.trainer.export_path.rstrip("/") + f"/global_step_{self.global_step}/dcp"
        return dcp_checkpoint.save_dcp(self.policy, path, self.ps, step=self.global_step)

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoints(self) -> str:
        t = self.cfg.trainer
        extra = {"critic": self.critic.state_dict()} if getattr(self, "critic", None) is not None else None
        if self.lora_store is not None:
            # the weights in the checkpoint are the MERGED ones; the factors and the rows of the base under them go beside
            ad = self.lora_store.adapters["policy"]
            extra = dict(extra or {}, lora={"adapter": ad.state_dict(), "base": {k: v.cpu() for k, v in self.lora_store._base.items()},
                                            "opt": self.policy.lora.opt.state_dict()})
        path = ckpt.save_checkpoint(t.ckpt_path, self.global_step, self.policy, self.loader.state_dict(),
                                    {"global_step": self.global_step, "epoch": self.epoch, "kl_ctrl": self.kl_ctrl.state_dict(),
                                     "config": self.cfg.to_dict()}, self.ps,
                                    max_to_keep=t.max_ckpts_to_keep, extra_shards=extra)
        self._fire("on_save", ckpt_path=path)
        return path

    def load_checkpoints(self) -> int:
        t = self.cfg.trainer
        path = ckpt.resolve_resume_path(t.ckpt_path, t.resume_mode, t.resume_path)
        if path is None:
            return 0
        if os.path.exists(os.path.join(path, ".metadata")):
            # a torch.distributed.checkpoint directory: weights, optimizer state and the step; the data order restarts
            from . import dcp_checkpoint

            info = dcp_checkpoint.load_dcp(self.policy, path)
            self.global_step = int(info["global_step"])
            return self.global_step
        data_state, trainer_state = ckpt.load_checkpoint(path, self.policy, self.ps)
        self.loader.load_state_dict(data_state)
        self.global_step = int(trainer_state["global_step"])
        self.epoch = self._start_epoch = int(trainer_state.get("epoch", data_state.get("epoch", 0)))
        if trainer_state.get("kl_ctrl") is not None:
            self.kl_ctrl.load_state_dict(trainer_state["kl_ctrl"])
        if self.lora_store is not None:
            sd = ckpt.load_extra_shard(path, "lora")
            if sd is None:
                raise FileNotFoundError(f"{path} holds no adapter state: it was not written by a run with trainer.policy.lora")
            ad = self.lora_store.adapters["policy"]
            for k in ad.A:
                ad.A[k].copy_(sd["adapter"]["A"][k])
                ad.B[k].copy_(sd["adapter"]["B"][k])
            self.lora_store._base = {k: v.to(self.device) for k, v in sd["base"].items()}       # the loaded weights are merged already
            self.policy.lora.opt.load_state_dict(sd["opt"])
        if getattr(self, "critic", None) is not None:
            sd = ckpt.load_extra_shard(path, "critic")
            if sd is None:
                print("[warn] checkpoint has no critic state for this rank: the critic restarts from its initial weights")
            else:
                self.critic.load_state_dict(sd)
        return self.global_step
