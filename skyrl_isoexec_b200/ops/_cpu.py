"""ctypes binding to ``lib/libisoexec_cpu.so``: the CPU restatement of every kernel with the
same reduction orders (the oracle of the GPU tests and the compute path of the CPU/gloo
configuration)."""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libisoexec_cpu.so"
_lib = None

_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_longlong, C.c_float
_SIGS = {
    "ixc_gemm_nt": [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _I],
    "ixc_leaftree_gemm": [_P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _I],
    "ixc_rmsnorm": [_P, _P, _P, _P, _P, _P, _I, _I, _F, _I, _L, _L, _I],
    "ixc_qk_norm_rope": [_P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I],
    "ixc_swiglu": [_P, _P, _L, _I, _L, _I],
    "ixc_sigmoid_gate": [_P, _P, _L, _P, _L, _I, _I, _I, _I],
    "ixc_gated_outnorm": [_P, _P, _P, _P, _L, _I, _F, _I, _I],
    "ixc_logprob_fused": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _I],
    "ixc_logprob_rowmax": [_P, _L, _I, _I, _P, _I],
    "ixc_logprob_leafsum": [_P, _L, _I, _I, _I, _I, _I, _P, _P, _P, _I],
    "ixc_logprob_finalize": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I],
    "ixc_router_topk": [_P, _L, _P, _I, _I, _I, _I, _I, _P, _P, _P],
    "ixc_gdn_conv": [_P, _L, _P, _P, _P, _P, _P, _L, _I, _I, _I],
    "ixc_gdn_conv_state": [_P, _L, _P, _P, _I, _I, _I, _I],
    "ixc_gdn_gate": [_P, _P, _L, _P, _P, _P, _P, _L, _I, _I],
    "ixc_gdn_l2norm": [_P, _L, _P, _P, _L, _I, _I, _F, _F, _I],
    "ixc_gdn_scan": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I],
    "ixc_attention_fwd": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I],
}


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        from .. import build as _b

        _b.build_cpu()
    h = C.CDLL(str(_LIB_PATH))
    for name, sig in _SIGS.items():
        fn = getattr(h, name)
        fn.argtypes = sig
        fn.restype = None
    h.ixc_reduce_sum.argtypes = [_P, _L, _I, _I]
    h.ixc_reduce_sum.restype = C.c_float
    _lib = h
    return h


def dt(t: torch.Tensor) -> int:
    """dtype code of the library: 0 = bf16, 1 = fp32."""
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise TypeError(f"unsupported dtype {t.dtype}: the kernels take bf16 or fp32 activations")


def ptr(t):
    return None if t is None else t.data_ptr()
