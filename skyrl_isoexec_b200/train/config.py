"""Typed configuration tree with ``key=value`` dotted CLI overrides.

Shape and defaults follow the reference's ``SkyRLTrainConfig`` (R/train/config/config.py:29-1056:
``trainer.*``, ``generator.*``, ``data.*``, ``environment.*``; defaults at :244-259,421-487,561-639,
719-833) so existing launch lines carry over. Parsing needs no OmegaConf: a dotted key walks the
dataclass tree and the value is coerced to the field's type; unknown keys are errors.
"""

from __future__ import annotations

import dataclasses
import json
import typing
from dataclasses import dataclass, field, fields, is_dataclass

from ..utils.profiler import ProfilerConfig
from .algorithms import AlgorithmConfig, OffPolicyCorrection
from .policy_worker import OptimizerConfig


@dataclass
class PlacementConfig:
    colocate_all: bool = True
    offload_optimizer: bool = False     # colocated jobs: at most one model's optimizer state on the GPU at a time, and none of
                                        # them during rollout (parked in pinned host memory; costs a PCIe round trip per switch)
    policy_num_gpus_per_node: int = 1
    policy_num_nodes: int = 1


@dataclass
class ParallelConfig:
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    sequence_parallel: bool = False


@dataclass
class RefConfig:
    """The frozen reference / teacher model. Empty ``model``: a copy of the policy's initial weights."""
    model: str = ""                     # preset name; must share the policy's vocabulary
    model_overrides: dict = field(default_factory=dict)
    seed: int = 0                       # random init seed when no weights are given
    hf_path: str = ""                   # directory with model.safetensors in the Hugging Face layout


@dataclass
class LoRASettings:
    """Low-rank adapters on the policy (``train/lora.py``): the base weights are frozen, only the factors step; the adapter is
    merged into the weight buffer, so the engine needs no adapter-aware kernel. ``rank = 0``: full fine-tuning."""
    rank: int = 0
    alpha: float = 16.0
    lr: float = 0.0                     # 0 = the policy optimizer's learning rate
    target_modules: str = "all-linear"  # "all-linear" or a comma-separated list of parameter-name suffixes (e.g. "attn.qkv.weight")
    seed: int = 0


@dataclass
class PolicyConfig:
    model: str = "tiny-qwen3"           # preset name or path of a saved config
    model_overrides: dict = field(default_factory=dict)
    lora: LoRASettings = field(default_factory=LoRASettings)
    freeze_moe_router: bool = False     # MoE models: the routers do not train
    moe_aux_loss_coeff: float = 0.0     # MoE models: weight of the router's load-balancing term in the update (0 = none)
    tokenizer_path: str = ""            # "" = none (token-id prompts and environments); "byte" = the built-in byte tokenizer;
                                        # else a directory transformers.AutoTokenizer loads (text prompts, chat templates, stop strings)
    optimizer_config: OptimizerConfig = field(default_factory=OptimizerConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    seed: int = 0
    keep_last_layers: int = 0           # layers whose activations are kept instead of recomputed in the backward;
                                        # -1 = as many as the first step's measured memory peak leaves room for
    shard_optimizer: bool = True        # dp > 1: fp32 master weights and Adam moments are cut over the data-parallel ranks
    peer_transports: bool = True        # GPUs with peer access: fused TP GEMM+collective kernels, peer-memory DP / EP transports


@dataclass
class CriticConfig:
    """The value model (built when ``advantage_estimator=gae``). Empty ``model``: the policy's architecture."""
    model: str = ""
    model_overrides: dict = field(default_factory=dict)
    hf_path: str = ""                   # initial weights in the Hugging Face layout (default: seeded random init)
    optimizer_config: OptimizerConfig = field(default_factory=lambda: OptimizerConfig(lr=5e-6))


@dataclass
class FullyAsyncConfig:
    """``train/fully_async_trainer.py`` (run through ``train/entrypoints/main_async.py --mode fully_async``, or implied by
    ``enabled``)."""
    enabled: bool = False
    max_staleness_steps: int = 4
    num_parallel_generation_workers: int = 768
    simulate_training: bool = False
    simulate_training_step_seconds: float = 0.0
    simulate_weight_sync_seconds: float = 0.0


@dataclass
class SamplingConfig:
    max_generate_length: int = 1024
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    min_p: float = 0.0
    top_k: int = -1
    logprobs: int = 1
    stop: list | None = None
    ignore_eos: bool = False
    additional_kwargs: dict = field(default_factory=dict)


@dataclass
class InferenceEngineConfig:
    backend: str = "native"
    num_engines: int = 0                # 0 = as many as fit the job: world size / tensor_parallel_size
    tensor_parallel_size: int = 0       # 0 = the trainer's tensor-parallel degree (engine computes with the trainer's buffer);
                                        # another degree gives colocated engines of their own layout, fed by a resharding sync
    data_parallel_size: int = 1
    gpu_memory_utilization: float = 0.8
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 1024
    num_kv_pages: int = 0
    enforce_eager: bool = False
    enable_prefix_caching: bool = False
    own_weights: bool = False           # the engine computes with a copy of the weights of its own (filled by every weight sync) even
                                        # when its layout is the trainer's: what lets generation run WHILE the trainer updates
    share_prompt_pages: bool = True     # the n samples of a prompt read one copy of its full KV pages (same bits; not a cache)
    share_recurrent_state: bool = False # GatedDeltaNet models: the samples also start from one snapshot of the recurrent state
    weight_sync_backend: str = "nccl"   # nccl | gloo | cuda_ipc | shared
    run_engines_locally: bool = True
    enable_http_endpoint: bool = False  # the in-process engine also answers HTTP (OpenAI-style and token-level routes of engine/server.py) and
                                        # the trainer's own generator goes through that endpoint; external agent harnesses can use it too
    http_endpoint_host: str = "127.0.0.1"
    http_endpoint_port: int = 0         # 0 = any free port (trainer.http_endpoint_url tells which)
    remote_urls: list = field(default_factory=list)   # run_engines_locally=false: base URLs of running inference servers (train/remote_engines.py)
    remote_weights_dir: str = ""        # a directory the trainer writes and every server reads (default: ckpt_path/remote_weights)


@dataclass
class GeneratorConfig:
    inference_engine: InferenceEngineConfig = field(default_factory=InferenceEngineConfig)
    n_samples_per_prompt: int = 5
    sampling_params: SamplingConfig = field(default_factory=SamplingConfig)
    eval_sampling_params: SamplingConfig = field(default_factory=lambda: SamplingConfig(temperature=0.0))
    eval_n_samples_per_prompt: int = 1
    max_input_length: int = 512
    batched: bool = True
    max_turns: int = 1
    use_conversation_multi_turn: bool = True
    zero_reward_on_non_stop: bool = False
    apply_overlong_filtering: bool = False
    step_wise_trajectories: bool = False   # every model turn of a multi-turn trajectory is a training sample of its own
    chat_template: dict = field(default_factory=dict)          # {"source": "name" | "file", "name_or_path": ...}: train/generator_utils.py
    chat_template_kwargs: dict = field(default_factory=dict)   # passed to the tokenizer's apply_chat_template
    merge_stepwise_output: bool = False    # step-wise rollouts are merged back into one row per trajectory before training
    multimodal: bool = False               # conversations may hold images: the vision-language generator (train/vlm_generator.py)
    append_eos_token_after_stop_str_in_multi_turn: bool = False
    rlm: bool = False                      # REPL environments whose blocks query the policy and spawn child trajectories (train/rlm_generator.py)
    rlm_max_depth: int = 1
    rlm_lm_max_tokens: int = 256
    rlm_train_children: bool = False       # child trajectories become samples of their own, rewarded with their root's outcome
    rate_limit: dict = field(default_factory=dict)   # enabled / trajectories_per_second / max_concurrency (multi-turn trajectories)


@dataclass
class DataConfig:
    train_data: list = field(default_factory=list)
    val_data: list = field(default_factory=list)
    synthetic_prompts: int = 0          # >0: uniform-random token prompts (no dataset needed)
    synthetic_prompt_len: int = 32


@dataclass
class EnvironmentConfig:
    env_class: str = "even_tokens"
    env_kwargs: dict = field(default_factory=dict)


@dataclass
class IsoExecConfig:
    enabled: bool = True
    gate_mean_limit: float = 1.0e-5     # forward-gate limits of the reference (R/train/utils/trainer_utils.py:45-46)
    gate_max_limit: float = 1.0e-4
    require_bitwise: bool = True        # the contract claims tolerance 0: any nonzero diff refuses
    strict: bool = True
    # Strictly on-policy steps (one optimizer step per rollout batch): take the engine's sampled-token logprobs as the
    # old-policy logprobs instead of recomputing them with a scoring forward. Under the contract the two are the same
    # bits; the forward gate then compares the TRAINING forward's logprobs with the rollout's, before the optimizer
    # step. Off by default (the reference always runs the scoring forward).
    reuse_rollout_logprobs: bool = False
    # At start-up on a GPU, prove on every GEMM shape of the model's census that the provider's rows do not depend on
    # the batch they are computed in (and that the two leaf-tree forms agree); a shape that fails refuses the launch.
    mm_admission: bool = True
    contract_path: str = ""
    debug_trace: str = ""


@dataclass
class TrainerConfig:
    placement: PlacementConfig = field(default_factory=PlacementConfig)
    policy: PolicyConfig = field(default_factory=PolicyConfig)
    ref: RefConfig = field(default_factory=RefConfig)
    critic: CriticConfig = field(default_factory=CriticConfig)
    fully_async: FullyAsyncConfig = field(default_factory=FullyAsyncConfig)
    algorithm: AlgorithmConfig = field(default_factory=AlgorithmConfig)
    isoexec: IsoExecConfig = field(default_factory=IsoExecConfig)
    strategy: str = "native"
    epochs: int = 1
    train_batch_size: int = 1024
    policy_mini_batch_size: int = 256
    micro_train_batch_size_per_gpu: int = 1
    micro_forward_batch_size_per_gpu: int = 1
    max_tokens_per_microbatch: int = 8192
    logprobs_chunk_size: int = 8192     # rows of the LM head scored at a time (bounds the [rows, vocabulary] logits in flight)
    critic_mini_batch_size: int = 0     # 0 = policy_mini_batch_size
    dump_eval_results: bool = False     # every evaluation also writes its samples to export_path (or ckpt_path)/dumped_evals/global_step_N.jsonl
    update_ref_every_epoch: bool = False  # the reference model takes the policy's weights at the end of every epoch
    update_epochs_per_batch: int = 1
    max_prompt_length: int = 512
    eval_batch_size: int = 1024
    eval_before_train: bool = False
    eval_interval: int = -1
    ckpt_path: str = ""
    ckpt_interval: int = 10
    max_ckpts_to_keep: int = -1
    resume_mode: str = "latest"         # none | latest | from_path
    resume_path: str = ""
    export_path: str = ""
    hf_save_interval: int = -1
    dcp_save_interval: int = -1         # every N steps: a torch.distributed.checkpoint directory under export_path/global_step_N/dcp
    logger: str = "console"
    project_name: str = "skyrl_isoexec_b200"
    run_name: str = "run"
    seed: int = 42
    recompute_old_logprobs_per_minibatch: bool = False
    dump_data_batch: bool = False
    balance_dp_by_length: bool = False   # after generation, deal whole prompt groups out over the data-parallel ranks so that
                                         # every rank scores and trains on about the same number of tokens
    num_steps: int = -1                 # stop after this many global steps (-1: run the epochs out)
    profiler: ProfilerConfig = field(default_factory=ProfilerConfig)    # torch.profiler over a window of steps
    nvtx: bool = False                  # NVTX range around every phase of a step (for timeline tools)
    record_memory: str = ""             # directory: allocator history on, one snapshot after each policy update
    log_example_interval: int = 0        # > 0: print the first rollout of the step every this many steps
    gpu_monitor: bool = False           # poll nvidia-smi (read-only) and log gpu/* per step: clocks, power, throttle reasons


@dataclass
class SkyRLTrainConfig:
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    generator: GeneratorConfig = field(default_factory=GeneratorConfig)
    data: DataConfig = field(default_factory=DataConfig)
    environment: EnvironmentConfig = field(default_factory=EnvironmentConfig)

    @classmethod
    def from_cli_overrides(cls, argv: list[str]) -> "SkyRLTrainConfig":
        cfg = cls()
        for arg in argv:
            if "=" not in arg:
                raise ValueError(f"override {arg!r} is not key=value")
            if arg.startswith("+"):
                raise ValueError("the '+key=value' syntax is not supported; every key already exists in the config tree")
            key, val = arg.split("=", 1)
            _apply(cfg, LEGACY_KEYS.get(key.strip(), key.strip()), val.strip())
        return cfg

    @classmethod
    def from_file(cls, path: str, overrides: list[str] | None = None) -> "SkyRLTrainConfig":
        """A YAML or JSON file with the nested config tree (any subset of keys), then ``key=value`` overrides on top.
        Keys of older config files are translated first (``LEGACY_KEYS``; reference: the legacy YAML translation of
        R/train/config/config.py:1001-1056)."""
        with open(path) as f:
            text = f.read()
        if path.endswith(".json"):
            tree = json.loads(text)
        else:
            import yaml

            tree = yaml.safe_load(text) or {}
        if not isinstance(tree, dict):
            raise ValueError(f"{path}: the top level of a config file must be a mapping")
        cfg = cls()
        for key, val in _flatten(tree):
            key = LEGACY_KEYS.get(key, key)
            text_val = val if isinstance(val, str) else json.dumps(val)
            if text_val == "null":
                text_val = "none"
            _apply(cfg, key, text_val)
        for arg in overrides or []:
            if "=" not in arg:
                raise ValueError(f"override {arg!r} is not key=value")
            k, v = arg.split("=", 1)
            _apply(cfg, LEGACY_KEYS.get(k.strip(), k.strip()), v.strip())
        return cfg

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def dumps(self) -> str:
        return json.dumps(self.to_dict(), indent=1, sort_keys=True, default=str)


# ----------------------------------------------------------------------------- keys of the reference's config tree
# A launch line or YAML file written for the reference names keys of its FSDP / Megatron / vLLM / Ray machinery and nests
# some settings differently. ``translate_key`` maps those that have a counterpart here, accepts (and notes) those that
# configure machinery this framework does not have, and refuses, with a message that says what is missing, those whose
# value would change what is trained if it were dropped silently.
RENAMED_KEYS = {
    "trainer.max_training_steps": "trainer.num_steps",
    "trainer.enable_ray_gpu_monitor": "trainer.gpu_monitor",
    "trainer.policy.sequence_parallel_size": "trainer.policy.parallel.context_parallel_size",       # Ulysses
    "trainer.policy.megatron_config.tensor_model_parallel_size": "trainer.policy.parallel.tensor_model_parallel_size",
    "trainer.policy.megatron_config.pipeline_model_parallel_size": "trainer.policy.parallel.pipeline_model_parallel_size",
    "trainer.policy.megatron_config.context_parallel_size": "trainer.policy.parallel.context_parallel_size",
    "trainer.policy.megatron_config.expert_model_parallel_size": "trainer.policy.parallel.expert_model_parallel_size",
    "trainer.policy.megatron_config.moe_aux_loss_coeff": "trainer.policy.moe_aux_loss_coeff",
    "trainer.policy.megatron_config.freeze_moe_router": "trainer.policy.freeze_moe_router",
    "trainer.ref.model.path": "trainer.ref.hf_path",
    "trainer.critic.model.path": "trainer.critic.hf_path",
    "trainer.algorithm.kl_ctrl.type": "trainer.algorithm.kl_ctrl_type",
    "trainer.algorithm.kl_ctrl.kl_target": "trainer.algorithm.kl_target",
    "trainer.algorithm.kl_ctrl.horizon": "trainer.algorithm.kl_horizon",
    "trainer.algorithm.sapo.tau_pos": "trainer.algorithm.sapo_tau_pos",
    "trainer.algorithm.sapo.tau_neg": "trainer.algorithm.sapo_tau_neg",
    "trainer.algorithm.dynamic_sampling.type": "trainer.algorithm.dynamic_sampling_type",
    "trainer.algorithm.dynamic_sampling.max_sample_batches": "trainer.algorithm.dynamic_sampling_max_sample_batches",
    "trainer.algorithm.dynamic_sampling.min_replace_ratio": "trainer.algorithm.dynamic_sampling_min_replace_ratio",
    "trainer.algorithm.clip_cov.clip_ratio": "trainer.algorithm.clip_cov_ratio",
    "trainer.algorithm.clip_cov.clip_cov_lb": "trainer.algorithm.clip_cov_lb",
    "trainer.algorithm.clip_cov.clip_cov_ub": "trainer.algorithm.clip_cov_ub",
    "trainer.algorithm.kl_cov.kl_cov_frac": "trainer.algorithm.kl_cov_frac",
    "trainer.algorithm.kl_cov.ppo_kl_coef": "trainer.algorithm.kl_cov_ppo_kl_coef",
    "trainer.algorithm.cispo.cispo_eps_clip_low": "trainer.algorithm.cispo_eps_clip_low",
    "trainer.algorithm.cispo.cispo_eps_clip_high": "trainer.algorithm.cispo_eps_clip_high",
    "trainer.algorithm.dppo.dppo_type": "trainer.algorithm.dppo_type",
    "trainer.algorithm.dppo.delta_low": "trainer.algorithm.dppo_delta_low",
    "trainer.algorithm.dppo.delta_high": "trainer.algorithm.dppo_delta_high",
    "trainer.algorithm.off_policy_correction.token_mask_is_threshold_low": "trainer.algorithm.off_policy_correction.outlier_token_is_threshold_low",
    "trainer.algorithm.off_policy_correction.token_mask_is_threshold_high": "trainer.algorithm.off_policy_correction.outlier_token_is_threshold_high",
    "trainer.algorithm.tis_imp_ratio_cap": "trainer.algorithm.off_policy_correction.token_tis_ratio_clip_high",
    "generator.vision_language_generator": "generator.multimodal",
    "generator.chat_template.source": "generator.chat_template.source",
    "generator.chat_template.name_or_path": "generator.chat_template.name_or_path",
    "environment.skyrl_gym.text2sql.db_path": "environment.env_kwargs.db_path",
    "environment.skyrl_gym.llm_as_a_judge.model": "environment.env_kwargs.model",
    "environment.skyrl_gym.llm_as_a_judge.base_url": "environment.env_kwargs.base_url",
}
# environment.skyrl_gym.<environment>.<key> -> environment.env_kwargs.<key>
_ENV_PREFIX = "environment.skyrl_gym."
# machinery that does not exist here: accepted, noted, without effect
INERT_PREFIXES = (
    "data.dataloader.", "trainer.placement.colocate_policy_ref", "trainer.placement.critic_num_", "trainer.placement.ref_num_",
    "trainer.use_expandable_segments", "trainer.sequence_parallel_backend", "trainer.policy.fsdp_config.", "trainer.ref.fsdp_config.",
    "trainer.critic.fsdp_config.", "trainer.policy.use_torch_compile", "trainer.policy.megatron_config.ddp_config.",
    "trainer.policy.megatron_config.torch_profiler_config.", "trainer.policy.megatron_config.moe_token_dispatcher_type",
    "trainer.policy.megatron_config.moe_grouped_gemm", "trainer.policy.megatron_config.moe_per_layer_logging",
    "trainer.policy.megatron_config.moe_router_dtype", "trainer.policy.megatron_config.optimizer_config_kwargs",
    "trainer.policy.megatron_config.transformer_config_kwargs", "trainer.policy.megatron_config.model_config_kwargs",
    "trainer.policy.megatron_config.empty_cuda_cache", "trainer.policy.megatron_config.dist_ckpt_optim_fully_reshardable",
    "trainer.policy.megatron_config.moe_router_load_balancing_type", "trainer.policy.megatron_config.moe_router_score_function",
    "trainer.policy.megatron_config.moe_router_enable_expert_bias", "trainer.ref.megatron_config.", "trainer.ref.sequence_parallel_size",
    "trainer.critic.sequence_parallel_size", "trainer.policy.model_config_kwargs", "trainer.ref.model_config_kwargs",
    "trainer.critic.model_config_kwargs", "trainer.policy.inference_only_init", "trainer.policy.optimizer_config.offload_after_step",
    "trainer.critic.optimizer_config.offload_after_step", "trainer.gradient_checkpointing_use_reentrant", "trainer.log_path", "trainer.tags",
    "trainer.remove_microbatch_padding", "trainer.flash_attn", "trainer.disable_fast_tokenizer",
    "trainer.max_tokens_per_microbatch_forward", "trainer.fully_async.sample_full_batch", "trainer.fully_async.clear_kv_cache_on_weight_sync",
    "trainer.algorithm.value_head_prefix", "trainer.policy.megatron_config.lora_config.",
    "generator.inference_engine.model_dtype",
    "generator.inference_engine.weight_transfer_threshold_cuda_ipc_GB", "generator.inference_engine.async_engine",
    "generator.inference_engine.vllm_v1_disable_multiproc", "generator.inference_engine.enable_chunked_prefill",
    "generator.inference_engine.fully_sharded_loras", "generator.inference_engine.enable_ray_prometheus_stats",
    "generator.inference_engine.use_expandable_segments", "generator.inference_engine.distributed_executor_backend",
    "generator.inference_engine.engine_init_kwargs", "generator.inference_engine.override_existing_update_group",
    "generator.inference_engine.router_init_kwargs", "generator.inference_engine.served_model_name",
    "environment.skyrl_gym.max_env_workers",
)
# (key or prefix, values that are fine, what is missing): a value outside the fine ones would change what is trained
UNSUPPORTED_IF_SET = (
    ("trainer.ref.model.lora.rank", ("0",), "LoRA adapters exist for the policy only (trainer.policy.lora); the reference model is frozen"),
    ("trainer.critic.model.lora.rank", ("0",), "LoRA adapters exist for the policy only (trainer.policy.lora); the critic trains in full"),
    ("trainer.policy.megatron_config.expert_tensor_parallel_size", ("1", "none", "null"), "experts are sharded over expert parallelism only"),
    ("trainer.policy.megatron_config.moe_enable_routing_replay", ("false",), "router replay has no consumer here: both sides route with the same kernel on the same bits"),
    ("trainer.policy.language_model_only", ("false",), "the vision tower is frozen already; there is no switch"),
    ("trainer.ref.language_model_only", ("false",), "the vision tower is frozen already; there is no switch"),
    ("generator.inference_engine.language_model_only", ("false",), "the vision tower is frozen already; there is no switch"),
    ("trainer.bf16", ("true",), "compute is bf16 (or the preset's dtype); fp32 training is chosen with trainer.policy.model_overrides.dtype"),
    ("generator.inference_engine.pipeline_parallel_size", ("1",), "engines are not pipelined"),
    ("generator.inference_engine.expert_parallel_size", ("1",), "engine expert parallelism follows the trainer's"),
    ("generator.inference_engine.enable_return_routed_experts", ("false",), "router replay has no consumer here"),
    ("generator.inference_engine.enable_pd", ("false",), "prefill / decode disaggregation is not implemented"),
    ("generator.inference_engine.num_prefill", ("0",), "prefill / decode disaggregation is not implemented"),
)
COMPAT_NOTES: list[str] = []


def translate_key(key: str, val: str):
    """(key here, value) for a key of this tree or of the reference's; None when the key is accepted without effect."""
    low = val.strip().strip("\"'").lower() if isinstance(val, str) else str(val).lower()
    for k, fine, why in UNSUPPORTED_IF_SET:
        if key == k or (k.endswith(".") and key.startswith(k)):
            if fine is None or low not in fine:
                raise ValueError(f"config key {key}={val} cannot be honoured: {why}")
            return None
    if key == "trainer.algorithm.use_tis":
        return ("trainer.algorithm.off_policy_correction.tis_ratio_type", "token") if low == "true" else None
    if key == "trainer.gradient_checkpointing":
        return ("trainer.policy.keep_last_layers", "0" if low == "true" else "-1")       # off = keep what fits instead of recomputing
    if key in ("trainer.rope_theta", "generator.rope_theta"):
        return None if low in ("none", "null") else ("trainer.policy.model_overrides.rope_theta", val)
    if key in ("trainer.rope_scaling", "generator.rope_scaling"):
        return None if low in ("none", "null", "{}") else ("trainer.policy.model_overrides.rope_scaling", val)
    if key == "generator.inference_engine.external_server_urls":
        return None if low in ("[]", "none", "null", "") else ("generator.inference_engine.remote_urls", val)
    if key == "generator.inference_engine.external_proxy_url":      # one router in front of the servers (engine/router.py) is one URL
        return None if low in ("none", "null", "") else ("generator.inference_engine.remote_urls", json.dumps([val.strip().strip("\"'")]))
    if key == "trainer.policy.record_memory":
        return ("trainer.record_memory", "memory_snapshots" if low == "true" else "")
    if key in ("trainer.policy.optimizer_config.adam_betas", "trainer.critic.optimizer_config.adam_betas"):
        if low in ("none", "null"):
            return None
        b = json.loads(val.replace("(", "[").replace(")", "]"))
        return [(key.replace("adam_betas", "beta1"), str(b[0])), (key.replace("adam_betas", "beta2"), str(b[1]))]
    if key.startswith("trainer.policy.model.lora."):
        leaf = key.rsplit(".", 1)[1]
        if leaf in ("rank", "alpha"):
            return f"trainer.policy.lora.{leaf}", val
        if leaf == "target_modules":
            return "trainer.policy.lora.target_modules", val
        return None                                          # dropout, init method, adapter paths: no counterpart, no effect on the maths here
    if key.startswith("trainer.ref.model.lora.") or key.startswith("trainer.critic.model.lora."):
        return None                                          # the adapter's other settings mean nothing at rank 0
    if key in RENAMED_KEYS:
        return RENAMED_KEYS[key], ("" if key.endswith("dynamic_sampling.type") and low in ("none", "null") else val)
    if key.startswith(_ENV_PREFIX) and not any(key.startswith(p) for p in INERT_PREFIXES):
        rest = key[len(_ENV_PREFIX):].split(".", 1)
        if len(rest) == 2:
            return "environment.env_kwargs." + rest[1], val
        return "environment.env_kwargs." + rest[0], val      # a whole mapping for one environment
    if any(key == p or key.startswith(p) for p in INERT_PREFIXES):
        note = f"{key}: accepted for compatibility, without effect here"
        if note not in COMPAT_NOTES:
            COMPAT_NOTES.append(note)
        return None
    return key, val


def _apply(cfg, key: str, val: str) -> None:
    tr = translate_key(key, val)
    for k, v in ([] if tr is None else tr if isinstance(tr, list) else [tr]):
        set_by_path(cfg, k, v)


# old key -> current key (files written for earlier layouts of the tree keep working)
LEGACY_KEYS = {
    "trainer.policy.model.path": "trainer.policy.model",
    "trainer.policy_mini_batch": "trainer.policy_mini_batch_size",
    "trainer.algorithm.eps_clip": "trainer.algorithm.eps_clip_low",
    "generator.num_samples": "generator.n_samples_per_prompt",
    "generator.max_generate_length": "generator.sampling_params.max_generate_length",
    "generator.temperature": "generator.sampling_params.temperature",
    "trainer.keep_last_layers": "trainer.policy.keep_last_layers",
}


def _flatten(tree: dict, prefix: str = ""):
    """Nested mapping -> (dotted key, leaf) pairs. A mapping under a key whose config field is itself a dict (for
    instance ``trainer.policy.model_overrides``) is a leaf."""
    for k, v in tree.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict) and not key.endswith(("model_overrides", "additional_kwargs", "env_extras", "env_kwargs", "chat_template_kwargs",
                                                     "engine_init_kwargs", "router_init_kwargs", "optimizer_config_kwargs",
                                                     "transformer_config_kwargs", "model_config_kwargs", "rope_scaling")):
            yield from _flatten(v, key + ".")
        else:
            yield key, v


def _coerce(val: str, tp):
    origin = typing.get_origin(tp)
    if origin is typing.Union or str(origin) == "types.UnionType" or origin is getattr(__import__("types"), "UnionType", None):
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if val.lower() in ("null", "none"):
            return None
        return _coerce(val, args[0])
    if tp is bool:
        if val.lower() in ("true", "1", "yes"):
            return True
        if val.lower() in ("false", "0", "no"):
            return False
        raise ValueError(f"{val!r} is not a bool")
    if tp is int:
        return int(val)
    if tp is float:
        return float(val)
    if tp is str:
        return val.strip("\"'")
    if tp in (list, dict) or origin in (list, dict, tuple):
        try:
            out = json.loads(val.replace("'", '"'))
        except json.JSONDecodeError:
            if tp is dict or origin is dict:
                raise
            out = [v.strip().strip("\"'") for v in val.strip("[]()").split(",") if v.strip()]   # a bare value or a, b, c: a list of strings
        if (tp is list or origin in (list, tuple)) and not isinstance(out, (list, tuple)):
            out = [out]
        return tuple(out) if origin is tuple else out
    return val


def set_by_path(cfg, key: str, val: str) -> None:
    parts = key.split(".")
    obj = cfg
    for p in parts[:-1]:
        if not is_dataclass(obj) or p not in {f.name for f in fields(obj)}:
            raise KeyError(f"unknown config key {key!r} (at {p!r})")
        obj = getattr(obj, p)
    leaf = parts[-1]
    if isinstance(obj, dict):
        try:
            obj[leaf] = None if val.lower() in ("none", "null") else json.loads(val)
        except ValueError:
            obj[leaf] = val
        return
    fmap = {f.name: f for f in fields(obj)} if is_dataclass(obj) else {}
    if leaf not in fmap:
        raise KeyError(f"unknown config key {key!r}")
    hints = typing.get_type_hints(type(obj))
    tp = hints[leaf]
    optional = type(None) in typing.get_args(tp)
    if val.lower() in ("none", "null") and not optional and tp is not str:
        return                                  # "no value" for a field that always has one: the default stays
    setattr(obj, leaf, _coerce(val, tp))


def validate_cfg(cfg: SkyRLTrainConfig, world_size: int = 1) -> None:
    """Cross-field checks done before anything is built (reference: R/train/utils/utils.py:230)."""
    t, g = cfg.trainer, cfg.generator
    p = t.policy.parallel
    mp = p.tensor_model_parallel_size * p.pipeline_model_parallel_size * p.context_parallel_size
    if world_size % mp:
        raise ValueError(f"world size {world_size} is not divisible by tp*pp*cp={mp}")
    dp = world_size // mp
    if g.multimodal:
        if g.batched or g.step_wise_trajectories:
            raise ValueError("generator.multimodal renders every trajectory on its own: it needs generator.batched=false and "
                             "generator.step_wise_trajectories=false")
        if p.pipeline_model_parallel_size > 1 or p.context_parallel_size > 1:
            raise ValueError("generator.multimodal is not supported with pipeline or context parallelism")
    temp = t.algorithm.temperature if t.algorithm.temperature is not None else g.sampling_params.temperature
    if temp not in (1.0, 0.0) and t.isoexec.enabled:
        raise ValueError("a training temperature other than 1 needs trainer.isoexec.enabled=false (the contract pins the raw distribution)")
    if t.policy.lora.rank > 0 and mp * p.expert_model_parallel_size > 1:
        raise ValueError("trainer.policy.lora needs tensor-, pipeline-, context- and expert-parallel degrees of 1 (data parallelism is fine)")
    if g.rlm and (g.multimodal or g.step_wise_trajectories):
        raise ValueError("generator.rlm cannot be combined with generator.multimodal or generator.step_wise_trajectories")
    if g.step_wise_trajectories:
        if g.batched and g.max_turns == 1:
            raise ValueError("generator.step_wise_trajectories needs the multi-turn agent loop (generator.batched=false)")
        if t.algorithm.advantage_estimator not in ("grpo", "rloo", "maxrl"):
            raise ValueError("step-wise trajectories take their advantage from the last step's outcome reward: "
                             "advantage_estimator must be grpo, rloo or maxrl")
    if t.train_batch_size % t.policy_mini_batch_size:
        raise ValueError("train_batch_size must be a multiple of policy_mini_batch_size")
    if (t.policy_mini_batch_size * g.n_samples_per_prompt) % dp:
        raise ValueError(f"policy_mini_batch_size * n_samples_per_prompt must be divisible by the DP size {dp}")
    if t.algorithm.policy_loss_type not in __import__("skyrl_isoexec_b200.train.algorithms", fromlist=["x"]).POLICY_LOSSES:
        raise ValueError(f"unknown policy_loss_type {t.algorithm.policy_loss_type!r}")
    if t.algorithm.advantage_estimator not in __import__("skyrl_isoexec_b200.train.algorithms", fromlist=["x"]).ADVANTAGE_ESTIMATORS:
        raise ValueError(f"unknown advantage_estimator {t.algorithm.advantage_estimator!r}")
    tp = p.tensor_model_parallel_size
    if tp > 1:
        from ..models.config import PRESETS, get_config

        if t.policy.model in PRESETS:
            m = get_config(t.policy.model, **t.policy.model_overrides)
            hkv, hq = m.num_kv_heads, m.num_q_heads
            if hq % tp:
                raise ValueError(f"tensor parallel size {tp} does not divide the {hq} query heads of {t.policy.model}")
            if hkv % tp and (tp % hkv or (hq // hkv) % (tp // hkv)):
                raise ValueError(f"tensor parallel size {tp} must divide the {hkv} KV heads, or be a multiple of them that "
                                 f"also divides each group of {hq // hkv} query heads (KV heads are then replicated)")
    if t.resume_mode not in ("none", "latest", "from_path"):
        raise ValueError(f"resume_mode {t.resume_mode!r} must be none|latest|from_path")
    if t.isoexec.enabled:
        s = g.sampling_params
        if s.temperature != 1.0 or s.top_p != 1.0 or s.top_k not in (-1, 0) or s.min_p != 0.0:
            raise ValueError("isoexec.enabled requires temperature=1.0, top_p=1.0, top_k=-1, min_p=0.0 for rollouts")
        # enable_prefix_caching is allowed: this engine's reuse is page-granular and bitwise prefix-invariant, and the cached
        # pages fall under the contract's engine_kv_cache state claim (dropped at every weight sync, which is observed)
    ie = g.inference_engine
    if ie.tensor_parallel_size < 0 or ie.num_engines < 0:
        raise ValueError("inference engine sizes must be >= 0 (0 = derived from the trainer layout)")
    etp = ie.tensor_parallel_size or tp
    if etp != tp:
        if tp % etp:
            raise ValueError(f"colocated engines of tensor-parallel size {etp} must nest inside the trainer's tensor-parallel "
                             f"groups of size {tp} (the trainer degree has to be a multiple of the engine degree)")
        if p.pipeline_model_parallel_size > 1 or p.context_parallel_size > 1 or p.expert_model_parallel_size > 1:
            raise ValueError("engines with their own tensor-parallel degree need pp = cp = ep = 1 on the trainer")
    if p.pipeline_model_parallel_size > 1 and (p.context_parallel_size > 1 or p.expert_model_parallel_size > 1):
        raise ValueError("a pipelined trainer (pipeline_model_parallel_size > 1) supports tensor and data parallelism only")
    # keys of the reference's config that have no meaning in a one-process-per-GPU job: refuse values that would be ignored
    if p.sequence_parallel and (p.pipeline_model_parallel_size > 1 or p.context_parallel_size > 1 or p.expert_model_parallel_size > 1):
        raise ValueError("sequence_parallel=true goes with tensor parallelism only (pp = cp = ep = 1)")
    if ie.data_parallel_size != 1:
        raise ValueError("inference_engine.data_parallel_size: engines are replicated by num_engines, not by an inner data-parallel degree")
    if not ie.run_engines_locally:
        if not ie.remote_urls:
            raise ValueError("run_engines_locally=false needs generator.inference_engine.remote_urls (servers started with train/entrypoints/serve.py)")
        if t.isoexec.enabled:
            raise ValueError("remote engines: the execution contract's hand-shake and ledger do not reach across HTTP; set "
                             "trainer.isoexec.enabled=false (the bit-mismatch metrics are still reported)")
        if p.pipeline_model_parallel_size > 1 or p.context_parallel_size > 1 or p.expert_model_parallel_size > 1 or g.multimodal:
            raise ValueError("remote engines are supported with tensor and data parallelism, text-only")
        if not (ie.remote_weights_dir or t.ckpt_path):
            raise ValueError("remote engines need generator.inference_engine.remote_weights_dir (or trainer.ckpt_path) for the weight files")
    if not g.use_conversation_multi_turn:
        raise ValueError("use_conversation_multi_turn=false (token-append multi-turn without re-rendering) is not supported; "
                         "observations are always appended as rendered turns")
    pl = t.placement
    if world_size > 1 and pl.policy_num_nodes * pl.policy_num_gpus_per_node not in (1, world_size):
        raise ValueError(f"placement asks for {pl.policy_num_nodes} x {pl.policy_num_gpus_per_node} policy GPUs but the job has {world_size} ranks")
    if t.micro_forward_batch_size_per_gpu != 1:
        import warnings

        warnings.warn("micro_forward_batch_size_per_gpu is ignored: micro-batches are cut by trainer.max_tokens_per_microbatch", stacklevel=2)
    if ie.num_engines not in (0, 1) and ie.num_engines * etp != world_size:
        raise ValueError(f"num_engines={ie.num_engines} x tensor_parallel_size={etp} must cover the {world_size} GPUs of a colocated job")
