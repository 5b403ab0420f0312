"""Order-invariant tensor digests for region tracing (reference scheme: ISO/debug/thash.py:106-307).

digest_k(x) = sum_i  w(i) * (bits(x_i) & mask_k)   mod 2^64

* ``bits`` is the integer view of the element, so +0/-0 and NaN payloads count;
* ``w(i)`` is a fixed odd 64-bit weight derived from the element's index inside its ROW, so the
  digest does not depend on the order rows are visited in, nor on how a tensor is tiled;
* ``mask_k`` clears the k lowest mantissa bits: the *ladder* k = 0, 1, 2, 4, 8 tells how large a
  difference is (two tensors whose digests differ at k=0 but agree at k=2 differ only in the last
  two mantissa bits);
* row digests: one digest per row (last dim flattened), so two runtimes that batch tokens
  differently can still be compared token by token.
On a GPU all ladder levels come from one kernel pass over the tensor (csrc/thash.cu); on the CPU, and for levels
outside the ladder, from integer torch ops (int64 arithmetic wraps mod 2^64). Both give the same numbers.
"""

from __future__ import annotations

import torch

LADDER = (0, 1, 2, 4, 8)
_INT = {torch.float32: (torch.int32, 32), torch.bfloat16: (torch.int16, 16), torch.float16: (torch.int16, 16),
        torch.float64: (torch.int64, 64)}
_weights_cache: dict = {}


def _splitmix64(n: int) -> torch.Tensor:
    """n odd 64-bit weights, as int64 (two's complement)."""
    MASK = (1 << 64) - 1
    out = []
    x = 0x9E3779B97F4A7C15
    for _ in range(n):
        x = (x + 0x9E3779B97F4A7C15) & MASK
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        z = (z ^ (z >> 31)) | 1
        out.append(z - (1 << 64) if z >= (1 << 63) else z)
    return torch.tensor(out, dtype=torch.int64)


def weights(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    if key not in _weights_cache:
        _weights_cache[key] = _splitmix64(n).to(device)
    return _weights_cache[key]


_ks_cache: dict = {}


def _ladder_kernel(x: torch.Tensor) -> torch.Tensor:
    """int64 [len(LADDER), rows]: every ladder level of every row in one pass (GPU tensors)."""
    import ctypes as C

    from ..ops import _native

    lib = _native.lib()
    if not getattr(lib, "_thash_sig", False):
        lib.ix_row_digests.argtypes = [C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        lib._thash_sig = True
    key = str(x.device)
    if key not in _ks_cache:
        _ks_cache[key] = torch.tensor(LADDER, dtype=torch.int32, device=x.device)
    x = x.contiguous()
    rows = x.shape[0] if x.dim() > 0 else 1
    out = torch.zeros(len(LADDER), rows, dtype=torch.int64, device=x.device)
    if x.numel():
        _native.check(lib.ix_row_digests(x.data_ptr(), rows, x.numel() // rows, x.element_size(), _ks_cache[key].data_ptr(),
                                         out.data_ptr(), _native.stream()), "ix_row_digests")
    return out


def row_digests(x: torch.Tensor, k: int = 0) -> torch.Tensor:
    """int64 [rows] digests of a [rows, ...] tensor with the k lowest mantissa bits cleared."""
    if x.dtype not in _INT:
        x = x.float()
    if x.is_cuda and k in LADDER:
        return _ladder_kernel(x)[LADDER.index(k)]
    it, nbits = _INT[x.dtype]
    rows = x.shape[0] if x.dim() > 0 else 1
    b = x.contiguous().view(it).reshape(rows, -1).to(torch.int64)
    if nbits < 64:
        b = b & ((1 << nbits) - 1)
    if k:
        b = b & ~((1 << k) - 1)
    return (b * weights(b.shape[1], x.device)[None, :]).sum(dim=1)


def digest(x: torch.Tensor, k: int = 0) -> int:
    """Whole-tensor digest = wrapping sum of its row digests (order-invariant over rows)."""
    d = int(row_digests(x, k).sum().item())
    return d & ((1 << 64) - 1)


def ladder(x: torch.Tensor) -> dict[str, str]:
    if x.is_cuda:
        if x.dtype not in _INT:
            x = x.float()
        tot = _ladder_kernel(x).sum(dim=1).tolist()
        return {str(k): f"{v & ((1 << 64) - 1):016x}" for k, v in zip(LADDER, tot)}
    return {str(k): f"{digest(x, k):016x}" for k in LADDER}


def row_ladder(x: torch.Tensor) -> dict[str, list[str]]:
    out = {}
    if x.is_cuda:
        if x.dtype not in _INT:
            x = x.float()
        allk = _ladder_kernel(x).tolist()
        return {str(k): [f"{v & ((1 << 64) - 1):016x}" for v in allk[i]] for i, k in enumerate(LADDER)}
    for k in LADDER:
        d = row_digests(x, k).tolist()
        out[str(k)] = [f"{v & ((1 << 64) - 1):016x}" for v in d]
    return out
