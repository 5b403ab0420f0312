"""ctypes binding to ``lib/libisoexec_b200.so`` (built by ``skyrl_isoexec_b200.build``).

Every launcher returns 0 on success; anything else raises ``NativeError`` with the
library's message. On a box with a GPU a missing library is an error, never a silent
fallback: ``lib()`` raises and the CUDA ops built on it raise with it.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libisoexec_b200.so"
_lib = None


class NativeError(RuntimeError):
    pass


_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_SIGS = {
    "ix_init": [],
    "ix_set_pdl": [_I],
    "ix_read_status": [],
    "ix_version": [],
    "ix_gemm_bf16_nt": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "ix_gemm_bf16_nn": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "ix_gemm_bf16_tn": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "ix_rmsnorm": [_P, _P, _P, _P, _P, _P, _I, _I, _F, _I, _L, _L, _P],
    "ix_qk_norm_rope": [_P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "ix_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "ix_qk_norm_rope_bwd": [_P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "ix_bwd_num_partials": [],
    "ix_swiglu": [_P, _P, _L, _I, _L, _P],
    "ix_swiglu_bwd": [_P, _P, _P, _L, _I, _L, _P],
    "ix_sigmoid_gate": [_P, _P, _L, _P, _L, _I, _I, _I, _P],
    "ix_gated_outnorm": [_P, _P, _P, _P, _L, _I, _F, _I, _P],
    "ix_logprob_fused": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _I, _P],
    "ix_logprob_rowmax": [_P, _L, _I, _I, _P, _I, _P],
    "ix_logprob_leafsum": [_P, _L, _I, _I, _I, _I, _I, _P, _P, _P, _I, _P],
    "ix_logprob_gather_target": [_P, _L, _I, _I, _I, _P, _P, _I, _P],
    "ix_logprob_finalize": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P],
    "ix_logprob_bwd": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _L, _I, _P],
    "ix_ppo_loss": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _F, _F, _F, _I, _F, _I, _P],
    "ix_reduce_sum": [_P, _L, _I, _I, _P, _P, _I, _P],
    "ix_clip_coef": [_P, _F, _P, _P, _P],
    "ix_adamw": [_P, _P, _P, _P, _P, _L, _I, _F, _F, _F, _F, _F, _I, _P, _P],
    "ix_accum_bf16_to_f32": [_P, _P, _L, _I, _P],
    "ix_router_topk": [_P, _L, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P],
    "ix_moe_combine": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "ix_scale_rows": [_P, _P, _L, _I, _P],
    "ix_sampler_scratch_elems": [_I],
    "ix_sample_gumbel": [_P, _L, _I, _I, _P, C.c_ulonglong, C.c_uint, _P, _P, _P, _P],
    "ix_moe_grouped_gemm": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "ix_gdn_conv": [_P, _L, _P, _P, _P, _P, _P, _L, _I, _I, _I, _P],
    "ix_gdn_conv_state": [_P, _L, _P, _P, _I, _I, _I, _I, _P],
    "ix_gdn_gate": [_P, _P, _L, _P, _P, _P, _P, _L, _I, _I, _P],
    "ix_gdn_l2norm": [_P, _L, _P, _P, _L, _I, _I, _F, _F, _I, _P],
    "ix_gdn_scan": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "ix_attention_fwd": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _I, _F, _P, _P],
    "ix_enable_peer_access": [_I],
    "ix_ipc_open": [_P, _P],
    "ix_ipc_close": [_P],
    "ix_pointer_device": [_P],
    "ix_attention_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _P],
}
_RESTYPE = {"ix_reduce_scratch_elems": C.c_longlong}


def available() -> bool:
    return _LIB_PATH.exists()


def lib():
    """Load the library once. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise NativeError(
            f"{_LIB_PATH} is missing: run `python -m skyrl_isoexec_b200.build` (the CUDA ops have no fallback)"
        )
    h = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL if hasattr(C, "RTLD_GLOBAL") else 0)
    h.ix_last_error.restype = C.c_char_p
    h.ix_status_ptr.restype = C.c_void_p
    h.ix_reduce_scratch_elems.restype = C.c_longlong
    h.ix_reduce_scratch_elems.argtypes = [C.c_longlong]
    for name, sig in _SIGS.items():
        fn = getattr(h, name, None)
        if fn is None:
            continue
        fn.argtypes = sig
        fn.restype = C.c_int
    if os.environ.get("ISOEXEC_B200_PDL", "1") == "0" and hasattr(h, "ix_set_pdl"):
        h.ix_set_pdl(0)          # plain stream order instead of programmatic dependent launches
    _lib = h
    return h


_launches = 0


def launch_count() -> int:
    """Number of native launcher calls made by this process (every launcher result passes through ``check``)."""
    return _launches


def check(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        msg = lib().ix_last_error()
        raise NativeError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def read_status() -> int:
    """Synchronise and return the kernel status word (0 = no bounded wait ran out)."""
    return lib().ix_read_status()


def on_gpu() -> bool:
    return torch.cuda.is_available() and os.environ.get("ISOEXEC_B200_FORCE_CPU", "0") != "1"
