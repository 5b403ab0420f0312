"""The single table of environment flags, with who reads each one and whether it can move bits.

The reference catalogues 189 ``SKYRL_ISOEXEC_*`` flags with a *disposition* per flag (reference:
ISO/core/flags.py:14-47,1969-2010): ``function`` flags change arithmetic and therefore must be
visible in the execution contract; ``deployment`` flags change placement or transport but not bits;
``diagnostic`` flags only observe; ``dead`` flags are recognised and ignored. Most of the reference's
flags select between alternative implementations; this framework has exactly one implementation per
op, so the table is short. What is kept is the machinery: every flag is declared here, each names the
sides that read it, ``snapshot()`` records the live values, and ``latent_split_brain()`` reports a
function flag that is set on one side only (the handshake would catch the consequence; this names the cause).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

TRAIN, ENGINE = "trainer", "engine"
DISPOSITIONS = ("function", "deployment", "diagnostic", "dead")


@dataclass(frozen=True)
class Flag:
    name: str
    default: str
    sides: tuple[str, ...]
    disposition: str
    doc: str
    selects: str = ""          # the contract pin / behaviour the flag controls

    def get(self, env=None) -> str:
        return (env if env is not None else os.environ).get(self.name, self.default)


FLAGS: tuple[Flag, ...] = (
    Flag("SKYRL_ISOEXEC", "1", (TRAIN, ENGINE), "function", "master switch: build, exchange and enforce the execution contract",
         "trainer.isoexec.enabled"),
    Flag("SKYRL_ISOEXEC_MANIFEST_STRICT", "1", (TRAIN, ENGINE), "deployment", "0 demotes contract refusals to warnings"),
    Flag("SKYRL_ISOEXEC_DEBUG_TRACE", "", (TRAIN, ENGINE), "diagnostic", "directory for per-region digest traces (also demotes refusals)"),
    Flag("SKYRL_ISOEXEC_GDN_KERNEL", "recurrent", (TRAIN, ENGINE), "function", "recurrent | cpr: bf16 snapshots of the GDN state at chunk boundaries (read by models/config.py::get_config)",
         "gdn.core:kernel"),
    Flag("SKYRL_ISOEXEC_PIK_LEAVES", "8", (TRAIN, ENGINE), "function", "number of K leaves of the TP-invariant reduction tree (read by models/config.py::get_config)",
         "collectives.tree_all_reduce:leaves"),
    Flag("SKYRL_ISOEXEC_LOGPROB_LEAVES", "8", (TRAIN, ENGINE), "function", "number of vocabulary leaves of the log-softmax (read by models/config.py::get_config)",
         "logprobs.log_softmax:leaves"),
    Flag("SKYRL_ISOEXEC_TRAINER_SP", "0", (TRAIN,), "deployment", "1: sequence parallelism in the tensor-parallel trainer (rows of the residual stream cut over the ranks; the logprob "
         "bits do not change, so this is a deployment choice, not a numerical pin; read by train/trainer.py::build_models)"),
    Flag("ISOEXEC_CONTRACT_PATH", "", (TRAIN, ENGINE), "deployment", "write the built contract here (artifact)"),
    Flag("ISOEXEC_CONTRACT_HASH", "", (TRAIN, ENGINE), "deployment", "expected numerical_policy; a different built or loaded contract is refused"),
    Flag("ISOEXEC_HANDSHAKE_NEGATIVE_CONTROL", "0", (TRAIN,), "diagnostic", "corrupt the stamped hash so the handshake must refuse"),
    Flag("ISOEXEC_B200_FORCE_CPU", "0", (TRAIN, ENGINE), "deployment", "treat the process as GPU-less (tests)"),
    Flag("SKYRL_WORKER_NCCL_TIMEOUT_IN_S", "600", (TRAIN, ENGINE), "deployment", "process-group timeout"),
    Flag("NCCL_NVLS_ENABLE", "", (TRAIN, ENGINE), "deployment", "NVLS on/off for NCCL; no NCCL reduction is on the logprob path"),
    Flag("SKYRL_ISOEXEC_PIK_P2P", "1", (TRAIN, ENGINE), "deployment", "0 forces the NCCL all-gather transport for tree reductions (same bits; read by parallel/transports.py)"),
    Flag("VLLM_BATCH_INVARIANT", "", (ENGINE,), "dead", "vLLM switch of the reference; there is no vLLM here"),
)

_BY_NAME = {f.name: f for f in FLAGS}


def flag(name: str) -> Flag:
    return _BY_NAME[name]


def snapshot(env=None) -> dict[str, str]:
    return {f.name: f.get(env) for f in FLAGS}


def function_flags() -> list[Flag]:
    return [f for f in FLAGS if f.disposition == "function"]


def actor_forwarding_list(side: str) -> list[str]:
    """Names of the flags a launcher must forward to processes of ``side``."""
    return [f.name for f in FLAGS if side in f.sides and f.disposition != "dead"]


def latent_split_brain(trainer_env: dict, engine_env: dict) -> list[str]:
    """Function flags that both sides read but whose values differ between the two environments."""
    out = []
    for f in function_flags():
        if TRAIN in f.sides and ENGINE in f.sides and f.get(trainer_env) != f.get(engine_env):
            out.append(f"{f.name}: trainer={f.get(trainer_env)!r} engine={f.get(engine_env)!r}")
    return out


def check_table() -> list[str]:
    """Self-consistency of the table (used by the tests)."""
    errs = []
    seen = set()
    for f in FLAGS:
        if f.name in seen:
            errs.append(f"duplicate flag {f.name}")
        seen.add(f.name)
        if f.disposition not in DISPOSITIONS:
            errs.append(f"{f.name}: unknown disposition {f.disposition}")
        if not f.sides:
            errs.append(f"{f.name}: no side reads it")
        if f.disposition == "function" and not f.selects:
            errs.append(f"{f.name}: a function flag must name the contract pin it selects")
    return errs
