"""The op layer both runtimes call: one function per contract op, one implementation per
device. CUDA tensors go to the hand-written sm_100a kernels (``_native``); CPU tensors go
to the C++ restatement with the same reduction orders (``_cpu``). There is no eager
fallback on a GPU: a missing native library raises.

Forward passes are the bitwise-gated half (trainer == engine). Backward passes are outside
the contract (as in the reference, whose backward runs on stock cuBLAS,
ISO/ops/mm/mm_fwd_scope.py:75-147); their GEMMs are the NN / TN tcgen05 kernels of
csrc/gemm_bwd_tcgen05.cu on a GPU and torch ops on CPU.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..core import observe as _obs
from . import _cpu, _native

PAGE = 128  # keys per attention block == slots per KV page


def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


# --------------------------------------------------------------------------- GEMM
def gemm_nt(x: torch.Tensor, w: torch.Tensor, out_f32: bool = False, bn: int = 0) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T`` with the batch-invariant kernel (no autograd)."""
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], (x.shape, w.shape)
    M, K = x.shape
    N = w.shape[0]
    if x.stride(1) != 1:
        x = x.contiguous()
    if w.stride(1) != 1:
        w = w.contiguous()
    if _is_cuda(x):
        out = torch.empty(M, N, device=x.device, dtype=torch.float32 if out_f32 else torch.bfloat16)
        if M == 0:
            return out
        _obs.note("mm", "tcgen05_batch_invariant")
        L = _native.lib()
        _native.check(
            L.ix_gemm_bf16_nt(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                              int(out_f32), bn, 0, _native.stream()),
            "ix_gemm_bf16_nt",
        )
        return out
    out_dtype = torch.float32 if (out_f32 or x.dtype == torch.float32) else torch.bfloat16
    out = torch.empty(M, N, dtype=out_dtype)
    if M == 0:
        return out
    _obs.note("mm", "cpu_sequential_k")
    _cpu.lib().ixc_gemm_nt(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                           _cpu.dt(x), int(out_dtype == torch.float32))
    return out


def _bwd_gemm_ok(*ts) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 for t in ts)


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    """``a[M,R] @ b[R,N]`` (the input gradient ``dY @ W``): tcgen05 kernel reading ``b`` M/N-major, no transposed copy
    (csrc/gemm_bwd_tcgen05.cu). CPU tensors and odd shapes use torch."""
    M, R = a.shape
    N = b.shape[1]
    if not (_bwd_gemm_ok(a, b) and M > 0 and R % 8 == 0 and N % 8 == 0):
        return torch.matmul(a, b).to(torch.float32 if out_f32 else a.dtype)
    if a.stride(1) != 1 or a.stride(0) % 8:
        a = a.contiguous()
    if b.stride(1) != 1 or b.stride(0) % 8:
        b = b.contiguous()
    out = torch.empty(M, N, device=a.device, dtype=torch.float32 if out_f32 else torch.bfloat16)
    _native.check(_native.lib().ix_gemm_bf16_nn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, R, a.stride(0), b.stride(0), N,
                                                int(out_f32), _native.stream()), "ix_gemm_bf16_nn")
    return out


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
            out_f32: bool = False) -> torch.Tensor:
    """``a[R,M]^T @ b[R,N]`` (the weight gradient ``dY^T @ X``): both operands read M/N-major by the tcgen05 kernel.
    ``out`` (fp32, contiguous [M,N]) with ``accumulate=True``: the product is ADDED to it in the epilogue."""
    R, M = a.shape
    N = b.shape[1]
    ok = _bwd_gemm_ok(a, b) and R > 0 and M % 8 == 0 and N % 8 == 0
    if out is not None:
        assert out.dtype == torch.float32 and out.shape == (M, N) and out.is_contiguous()
    if not ok:
        res = torch.matmul(a.t(), b)
        if out is None:
            return res.to(torch.float32 if out_f32 else a.dtype)
        if accumulate:
            out.add_(res)
        else:
            out.copy_(res)
        return out
    if a.stride(1) != 1 or a.stride(0) % 8:
        a = a.contiguous()
    if b.stride(1) != 1 or b.stride(0) % 8:
        b = b.contiguous()
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.float32 if out_f32 else torch.bfloat16)
        mode = int(out_f32)
    else:
        mode = 2 if accumulate else 1
    _native.check(_native.lib().ix_gemm_bf16_tn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, R, a.stride(0), b.stride(0), N, mode,
                                                _native.stream()), "ix_gemm_bf16_tn")
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, out_f32):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        ctx.save_for_backward(x2, w)
        ctx.shp = shp
        return gemm_nt(x2, w, out_f32).reshape(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(w.dtype)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, w).reshape(ctx.shp)
        if ctx.needs_input_grad[1]:
            dw = gemm_tn(dy2, x2)
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    """``x[..., K] @ w[N, K]^T``. Forward: batch-invariant GEMM. Backward: the NN / TN tcgen05 GEMMs."""
    if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad):
        return _Linear.apply(x, w, out_f32)
    shp = x.shape
    return gemm_nt(x.reshape(-1, shp[-1]), w, out_f32).reshape(*shp[:-1], w.shape[0])


# --------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x, w, eps, zero_centered=False, residual=None, want_rstd=False):
    """Returns (y, residual_out or None, rstd or None). x: [rows, N] (row stride free)."""
    assert x.dim() == 2 and x.stride(1) == 1
    rows, N = x.shape
    y = torch.empty(rows, N, device=x.device, dtype=x.dtype)
    res_out = torch.empty(rows, N, device=x.device, dtype=x.dtype) if residual is not None else None
    rstd = torch.empty(rows, device=x.device, dtype=torch.float32) if want_rstd else None
    if rows == 0:
        return y, res_out, rstd
    if residual is not None:
        residual = residual.contiguous()
    if _is_cuda(x):
        _obs.note("norms.rms", "fused_add_rmsnorm")
        L = _native.lib()
        _native.check(
            L.ix_rmsnorm(x.data_ptr(), _native.ptr(residual), w.data_ptr(), y.data_ptr(), _native.ptr(res_out),
                         _native.ptr(rstd), rows, N, eps, int(zero_centered), x.stride(0), N, _native.stream()),
            "ix_rmsnorm",
        )
    else:
        _obs.note("norms.rms", "cpu_add_rmsnorm")
        _cpu.lib().ixc_rmsnorm(x.data_ptr(), _cpu.ptr(residual), w.data_ptr(), y.data_ptr(), _cpu.ptr(res_out),
                               _cpu.ptr(rstd), rows, N, eps, int(zero_centered), x.stride(0), N, _cpu.dt(x))
    return y, res_out, rstd


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, eps, zero_centered):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        r2 = residual.reshape(-1, shp[-1]) if residual is not None else None
        y, res_out, rstd = rmsnorm_fwd(x2, w, eps, zero_centered, r2, want_rstd=True)
        h = res_out if res_out is not None else x2
        ctx.save_for_backward(h, w, rstd)
        ctx.zero_centered = zero_centered
        ctx.has_res = residual is not None
        ctx.shp = shp
        if residual is not None:
            return y.reshape(shp), res_out.reshape(shp)
        return y.reshape(shp), None

    @staticmethod
    def backward(ctx, dy, dres):
        h, w, rstd = ctx.saved_tensors
        N = h.shape[-1]
        if _is_cuda(h) and h.dtype == torch.bfloat16 and N % 8 == 0 and N <= 8192:
            # one pass over the activations (csrc/norm_rope_bwd.cu); weight gradient folded in a fixed order
            L = _native.lib()
            rows = h.shape[0]
            dy2 = dy.reshape(-1, N).contiguous()
            dr2 = dres.reshape(-1, N).contiguous() if dres is not None else None
            dh = torch.empty_like(h)
            part = torch.empty(L.ix_bwd_num_partials(), N, dtype=torch.float32, device=h.device)
            dw = torch.empty_like(w) if ctx.needs_input_grad[1] else None
            _native.check(L.ix_rmsnorm_bwd(h.data_ptr(), w.data_ptr(), rstd.data_ptr(), dy2.data_ptr(), _native.ptr(dr2), dh.data_ptr(),
                                           part.data_ptr(), _native.ptr(dw), rows, N, int(ctx.zero_centered), _native.stream()), "ix_rmsnorm_bwd")
            dh = dh.reshape(ctx.shp)
            return dh, dw, (dh if ctx.has_res else None), None, None
        hf = h.float()
        g = w.float()
        if ctx.zero_centered:
            g = (1.0 + g).to(w.dtype).float()
        n = hf * rstd[:, None]
        dyf = dy.reshape(-1, N).float()
        dw = (dyf * n.to(h.dtype).float()).sum(0).to(w.dtype) if ctx.needs_input_grad[1] else None
        dn = dyf * g
        dh = rstd[:, None] * (dn - n * (dn * n).mean(-1, keepdim=True))
        if dres is not None:
            dh = dh + dres.reshape(-1, N).float()
        dh = dh.to(h.dtype).reshape(ctx.shp)
        return dh, dw, (dh if ctx.has_res else None), None, None


def rmsnorm(x, w, eps=1e-6, zero_centered=False, residual=None):
    """(y, new_residual). With ``residual`` the kernel first forms h = x + residual (rounded to
    the activation dtype), returns it as the new residual stream and normalises h."""
    if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or (residual is not None and residual.requires_grad)):
        return _RMSNorm.apply(x, w, residual, eps, zero_centered)
    shp = x.shape
    y, res_out, _ = rmsnorm_fwd(x.reshape(-1, shp[-1]), w, eps, zero_centered,
                                residual.reshape(-1, shp[-1]) if residual is not None else None)
    return y.reshape(shp), (res_out.reshape(shp) if res_out is not None else None)


# --------------------------------------------------------------------------- RoPE table
def scaled_inv_freq(rot_dim: int, theta: float, scaling: dict | None, max_pos: int):
    """(inverse frequencies fp64 [rot_dim / 2], factor on cos and sin) under a Hugging Face style ``rope_scaling`` mapping:

    * ``linear``   every frequency divided by ``factor`` (positions are compressed);
    * ``llama3``   wavelengths beyond ``original_max_position_embeddings / low_freq_factor`` are divided by ``factor``, those
                   below ``.. / high_freq_factor`` are kept, the band between is blended linearly in the wavelength's inverse;
    * ``yarn``     per dimension a blend of the original frequency (dimensions that turn more than ``beta_fast`` times over
                   the original context) and the interpolated one (fewer than ``beta_slow`` turns), linear ramp between;
                   cos and sin are multiplied by ``attention_factor`` (default ``0.1 ln(factor) + 1``, or the
                   ``mscale`` / ``mscale_all_dim`` ratio of the DeepSeek configs)."""
    import math

    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if not scaling:
        return inv, 1.0
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind in ("default", None):
        return inv, 1.0
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return inv / factor, 1.0
    orig = float(scaling.get("original_max_position_embeddings") or max_pos)
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        wavelen = 2 * math.pi / inv
        smooth = ((orig / wavelen) - lo) / (hi - lo)
        blended = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > orig / lo, inv / factor, torch.where(wavelen < orig / hi, inv, blended))
        return out, 1.0
    if kind == "yarn":
        beta_fast, beta_slow = float(scaling.get("beta_fast") or 32.0), float(scaling.get("beta_slow") or 1.0)

        def dim_of(turns):                     # the (fractional) dimension pair that makes ``turns`` rotations over ``orig`` positions
            return rot_dim * math.log(orig / (turns * 2 * math.pi)) / (2 * math.log(theta))

        low, high = dim_of(beta_fast), dim_of(beta_slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, rot_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        keep = 1 - ramp                        # 1 where the original frequency stays
        out = (inv / factor) * (1 - keep) + inv * keep
        att = scaling.get("attention_factor")
        if att is None:
            def mscale(f, m=1.0):
                return 1.0 if f <= 1 else 0.1 * m * math.log(f) + 1.0

            if scaling.get("mscale") and scaling.get("mscale_all_dim"):
                att = mscale(factor, float(scaling["mscale"])) / mscale(factor, float(scaling["mscale_all_dim"]))
            else:
                att = mscale(factor)
        return out, float(att)
    raise ValueError(f"rope_scaling type {kind!r} is not implemented (linear | llama3 | yarn)")


class RopeTable:
    """cos/sin of ``pos * theta^(-2i/rot_dim)`` as fp32 ``[max_pos, rot_dim/2]``, computed once in
    fp64 on the host so trainer and engine hold byte-identical tables. ``scaling``: a ``rope_scaling`` mapping
    (``scaled_inv_freq``); context extension changes only this table, the kernels read it as before."""

    def __init__(self, rot_dim: int, max_pos: int, theta: float, device, scaling: dict | None = None):
        inv, att = scaled_inv_freq(rot_dim, theta, scaling, max_pos)
        ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = (ang.cos() * att).float().to(device).contiguous()
        self.sin = (ang.sin() * att).float().to(device).contiguous()
        self.rot_dim = rot_dim
        self.max_pos = max_pos
        self.attention_factor = att


# --------------------------------------------------------------------------- QK-norm + RoPE + KV write
def qk_norm_rope_fwd(qkv, positions, slots, rope: RopeTable, qw, kw, k_out, v_out, Hq, Hkv, D, eps, qk_norm=True,
                     zero_centered=False, q_gate=False):
    """qkv: [T, (Hq*(2 if q_gate else 1) + 2*Hkv) * D]. Writes k/v into k_out/v_out ([slots, Hkv, D]) at
    ``slots[t]`` (or t when slots is None) and returns q [T, Hq, D]."""
    T = qkv.shape[0]
    assert qkv.stride(1) == 1
    q = torch.empty(T, Hq, D, device=qkv.device, dtype=qkv.dtype)
    if T == 0:
        return q
    assert positions.dtype == torch.int32 and (slots is None or slots.dtype == torch.int64)
    _obs.note("rope.rope", "fused_qknorm_rope_kvwrite" if _is_cuda(qkv) else "cpu_fused_qknorm_rope")
    if _is_cuda(qkv):
        L = _native.lib()
        _native.check(
            L.ix_qk_norm_rope(qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), _native.ptr(slots),
                              rope.cos.data_ptr(), rope.sin.data_ptr(), _native.ptr(qw), _native.ptr(kw), q.data_ptr(),
                              k_out.data_ptr(), v_out.data_ptr(), T, Hq, Hkv, D, rope.rot_dim, eps, int(qk_norm),
                              int(zero_centered), int(q_gate), _native.stream()),
            "ix_qk_norm_rope",
        )
    else:
        _cpu.lib().ixc_qk_norm_rope(qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), _cpu.ptr(slots),
                                    rope.cos.data_ptr(), rope.sin.data_ptr(), _cpu.ptr(qw), _cpu.ptr(kw),
                                    q.data_ptr(), k_out.data_ptr(), v_out.data_ptr(), T, Hq, Hkv, D, rope.rot_dim, eps,
                                    int(qk_norm), int(zero_centered), int(q_gate), _cpu.dt(qkv))
    return q


def _rope_apply_f32(y, cos, sin, rot_dim, transpose=False):
    """y: [T, H, D] fp32. Forward rotate-half (or its transpose for the backward)."""
    half = rot_dim // 2
    y1, y2, rest = y[..., :half], y[..., half:rot_dim], y[..., rot_dim:]
    c, s = cos[:, None, :], sin[:, None, :]
    if not transpose:
        o1 = y1 * c - y2 * s
        o2 = y2 * c + y1 * s
    else:
        o1 = y1 * c + y2 * s
        o2 = y2 * c - y1 * s
    return torch.cat([o1, o2, rest], dim=-1)


class _QKNormRope(torch.autograd.Function):
    """Training-side op: returns (q, k, v) as fresh packed tensors [T, H, D]."""

    @staticmethod
    def forward(ctx, qkv, positions, rope, qw, kw, Hq, Hkv, D, eps, qk_norm, zero_centered, q_gate):
        T = qkv.shape[0]
        k = torch.empty(T, Hkv, D, device=qkv.device, dtype=qkv.dtype)
        v = torch.empty(T, Hkv, D, device=qkv.device, dtype=qkv.dtype)
        q = qk_norm_rope_fwd(qkv, positions, None, rope, qw, kw, k, v, Hq, Hkv, D, eps, qk_norm, zero_centered, q_gate)
        ctx.save_for_backward(qkv, positions, qw, kw)
        ctx.rope = rope
        ctx.cfg = (Hq, Hkv, D, eps, qk_norm, zero_centered, q_gate)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, positions, qw, kw = ctx.saved_tensors
        Hq, Hkv, D, eps, qk_norm, zero_centered, q_gate = ctx.cfg
        rope = ctx.rope
        T = qkv.shape[0]
        if _is_cuda(qkv) and qkv.dtype == torch.bfloat16 and D % 8 == 0 and D <= 256 and rope.rot_dim % 16 == 0 and qkv.stride(1) == 1:
            L = _native.lib()
            dqkv = torch.zeros_like(qkv) if q_gate else torch.empty_like(qkv)
            part = torch.empty(L.ix_bwd_num_partials(), 2, D, dtype=torch.float32, device=qkv.device)
            dw = torch.empty(2, D, dtype=qw.dtype, device=qkv.device) if qk_norm else None
            _native.check(L.ix_qk_norm_rope_bwd(qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), rope.cos.data_ptr(), rope.sin.data_ptr(),
                                                _native.ptr(qw), _native.ptr(kw), dq.contiguous().data_ptr(), dk.contiguous().data_ptr(),
                                                dv.contiguous().data_ptr(), dqkv.data_ptr(), part.data_ptr(), _native.ptr(dw),
                                                (dw[1].data_ptr() if dw is not None else None), T, Hq, Hkv, D, rope.rot_dim, eps,
                                                int(qk_norm), int(zero_centered), int(q_gate), _native.stream()), "ix_qk_norm_rope_bwd")
            return (dqkv, None, None, (dw[0] if dw is not None else None), (dw[1] if dw is not None else None),
                    None, None, None, None, None, None, None)
        qs = 2 * D if q_gate else D
        pos = positions.long()
        cos, sin = rope.cos[pos], rope.sin[pos]
        G = Hq // Hkv
        dqkv = torch.zeros_like(qkv)
        grp = qkv.view(T, Hkv, G * qs + 2 * D)  # KV-group major: [G query blocks | k | v]
        dgrp = dqkv.view(T, Hkv, G * qs + 2 * D)
        xq = grp[..., : G * qs].reshape(T, Hkv, G, qs)[..., :D].reshape(T, Hq, D).float()
        xk = grp[..., G * qs: G * qs + D].float()
        dwq = dwk = None

        def one(x, dout, w):
            dy = _rope_apply_f32(dout.float(), cos, sin, rope.rot_dim, transpose=True)
            if not qk_norm:
                return dy, None
            g = w.float()
            if zero_centered:
                g = (1.0 + g).to(w.dtype).float()
            rstd = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
            n = x * rstd
            dw = (dy * n).sum((0, 1)).to(w.dtype)
            dn = dy * g
            dx = rstd * (dn - n * (dn * n).mean(-1, keepdim=True))
            return dx, dw

        dxq, dwq = one(xq, dq, qw)
        dxk, dwk = one(xk, dk, kw)
        dgrp[..., : G * qs].view(T, Hkv, G, qs)[..., :D] = dxq.to(qkv.dtype).view(T, Hkv, G, D)
        dgrp[..., G * qs: G * qs + D] = dxk.to(qkv.dtype)
        dgrp[..., G * qs + D:] = dv
        return dqkv, None, None, dwq, dwk, None, None, None, None, None, None, None


def qk_norm_rope_train(qkv, positions, rope, qw, kw, Hq, Hkv, D, eps, qk_norm=True, zero_centered=False, q_gate=False):
    return _QKNormRope.apply(qkv, positions, rope, qw, kw, Hq, Hkv, D, eps, qk_norm, zero_centered, q_gate)


# --------------------------------------------------------------------------- attention
@dataclass
class AttnMeta:
    """Work list of the attention kernel. ``items`` is int32 [n, 8]:
    (q_start, q_len, q_pos0, kv_len, bt_row | -1, kv_start, 0, 0)."""

    items: torch.Tensor
    block_table: torch.Tensor | None = None
    seq_lens: list[int] = field(default_factory=list)  # packed training layout only (for the backward)
    _bwd: tuple | None = None

    def bwd_items(self, Hq: int, Hkv: int, device):
        """Work lists of the backward kernels (int32 [n, 8]: first row, sequence start, sequence end, 0...): one item
        per query tile of 128 / G tokens for dQ, one per block of 128 keys for dK / dV; the heaviest items come first
        so that the long ones do not start last."""
        if self._bwd is None:
            tq = PAGE // (Hq // Hkv)
            qi, ki = [], []
            start = 0
            for n in self.seq_lens:
                for t0 in range(0, n, tq):
                    qi.append((-(t0 + min(tq, n - t0)), start + t0, start, start + n))
                for k0 in range(0, n, PAGE):
                    ki.append((-(n - k0), start + k0, start, start + n))
                start += n
            mk = lambda rows: torch.tensor([(a, b, c, 0, 0, 0, 0, 0) for _, a, b, c in sorted(rows)],
                                           dtype=torch.int32).reshape(-1, 8).to(device)
            self._bwd = (mk(qi), mk(ki))
        return self._bwd

    @staticmethod
    def packed(seq_lens, Hq, Hkv, device) -> "AttnMeta":
        """Trainer / full-sequence layout: sequences packed back to back, keys contiguous."""
        tq = PAGE // (Hq // Hkv)
        rows = []
        start = 0
        for n in seq_lens:
            for t0 in range(0, n, tq):
                rows.append((start + t0, min(tq, n - t0), t0, n, -1, start, 0, 0))
            start += n
        items = torch.tensor(rows, dtype=torch.int32).reshape(-1, 8).to(device)
        return AttnMeta(items=items, block_table=None, seq_lens=list(seq_lens))


def attention_fwd(q, k, v, meta: AttnMeta, scale: float, want_lse: bool = False):
    """q: [T, Hq, D]; k, v: slot pools [num_slots, Hkv, D]. Returns (out [T,Hq,D], lse or None)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty(T, Hq, device=q.device, dtype=torch.float32) if want_lse else None
    n_items = meta.items.shape[0]
    if T == 0 or n_items == 0:
        return out, lse
    bt = meta.block_table
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and meta.items.is_contiguous()
    _obs.note("attention.varlen", "tcgen05_unified" if _is_cuda(q) else "cpu_blockwise")
    if _is_cuda(q):
        L = _native.lib()
        _native.check(
            L.ix_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), meta.items.data_ptr(), _native.ptr(bt),
                               out.data_ptr(), _native.ptr(lse), None, n_items, T, Hq, Hkv, D,
                               0 if bt is None else bt.stride(0), k.shape[0], 0, scale, None, _native.stream()),
            "ix_attention_fwd",
        )
    else:
        _cpu.lib().ixc_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), meta.items.data_ptr(), _cpu.ptr(bt),
                                     out.data_ptr(), _cpu.ptr(lse), n_items, Hq, Hkv, D,
                                     0 if bt is None else bt.stride(0), scale, _cpu.dt(q))
    return out, lse


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta, scale):
        native = _is_cuda(q) and q.dtype == torch.bfloat16
        out, lse = attention_fwd(q, k, v, meta, scale, want_lse=native)
        if native:
            ctx.save_for_backward(q, k, v, out, lse)
        else:
            ctx.save_for_backward(q, k, v)
        ctx.native = native
        ctx.meta = meta
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        if ctx.native:
            # csrc/attention_bwd_tcgen05.cu: delta, dK/dV (key-stationary) and dQ (query-stationary), no atomics
            q, k, v, out, lse = ctx.saved_tensors
            T, Hq, D = q.shape
            Hkv = k.shape[1]
            assert k.shape[0] == T and k.is_contiguous() and v.is_contiguous(), "the backward needs the packed contiguous layout"
            dout = dout.contiguous()
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            delta = torch.empty(T, Hq, device=q.device, dtype=torch.float32)
            iq, ik = ctx.meta.bwd_items(Hq, Hkv, q.device)
            _native.check(
                _native.lib().ix_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                               dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(),
                                               iq.data_ptr(), iq.shape[0], ik.data_ptr(), ik.shape[0], T, Hq, Hkv, D,
                                               ctx.scale, _native.stream()),
                "ix_attention_bwd",
            )
            return dq, dk, dv, None, None
        # CPU / fp32 configuration: recompute per sequence with the library attention and
        # differentiate it (right padding is harmless under a causal mask).
        q, k, v = ctx.saved_tensors
        lens = ctx.meta.seq_lens
        B, S = len(lens), max(lens)
        Hq, D = q.shape[1], q.shape[2]
        Hkv = k.shape[1]
        with torch.enable_grad():
            if all(n == S for n in lens):
                qp = q.view(B, S, Hq, D).transpose(1, 2).detach().requires_grad_(True)
                kp = k.view(B, S, Hkv, D).transpose(1, 2).detach().requires_grad_(True)
                vp = v.view(B, S, Hkv, D).transpose(1, 2).detach().requires_grad_(True)
                do = dout.view(B, S, Hq, D).transpose(1, 2)
            else:
                def pad(x):
                    H = x.shape[1]
                    o = x.new_zeros(B, S, H, D)
                    s = 0
                    for b, n in enumerate(lens):
                        o[b, :n] = x[s:s + n]
                        s += n
                    return o.transpose(1, 2)
                qp, kp, vp = (pad(t).detach().requires_grad_(True) for t in (q, k, v))
                do = pad(dout)
            o = torch.nn.functional.scaled_dot_product_attention(qp, kp, vp, is_causal=True, scale=ctx.scale,
                                                                 enable_gqa=(Hq != Hkv))
            gq, gk, gv = torch.autograd.grad(o, (qp, kp, vp), do)
        if all(n == S for n in lens):
            unp = lambda g, H: g.transpose(1, 2).reshape(B * S, H, D)
        else:
            def unp(g, H):
                g = g.transpose(1, 2)
                return torch.cat([g[b, :n] for b, n in enumerate(lens)], 0)
        return unp(gq, Hq), unp(gk, Hkv), unp(gv, Hkv), None, None


def attention(q, k, v, meta: AttnMeta, scale: float):
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _Attention.apply(q, k, v, meta, scale)
    return attention_fwd(q, k, v, meta, scale)[0]


# --------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(x):
    """x: [T, 2F] = [gate | up] -> [T, F]."""
    T, F2 = x.shape
    F = F2 // 2
    out = torch.empty(T, F, device=x.device, dtype=x.dtype)
    if T == 0:
        return out
    _obs.note("activation.swiglu", "fused_swiglu" if _is_cuda(x) else "cpu_swiglu")
    assert x.stride(1) == 1
    if _is_cuda(x):
        _native.check(_native.lib().ix_swiglu(x.data_ptr(), out.data_ptr(), T, F, x.stride(0), _native.stream()), "ix_swiglu")
    else:
        _cpu.lib().ixc_swiglu(x.data_ptr(), out.data_ptr(), T, F, x.stride(0), _cpu.dt(x))
    return out


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return swiglu_fwd(x)

    @staticmethod
    def backward(ctx, dout):
        (x,) = ctx.saved_tensors
        T, F2 = x.shape
        F = F2 // 2
        dout = dout.contiguous()
        if x.is_cuda and x.dtype == torch.bfloat16:
            dx = torch.empty(T, F2, device=x.device, dtype=x.dtype)
            _native.check(_native.lib().ix_swiglu_bwd(x.data_ptr(), dout.data_ptr(), dx.data_ptr(), T, F, x.stride(0),
                                                      _native.stream()), "ix_swiglu_bwd")
            return dx
        g, u = x[:, :F].float(), x[:, F:].float()
        d = dout.float()
        sig = torch.sigmoid(g)
        return torch.cat([d * u * (sig * (1 + g * (1 - sig))), d * g * sig], -1).to(x.dtype)


def swiglu(x):
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    y = _SwiGLU.apply(x2) if (torch.is_grad_enabled() and x.requires_grad) else swiglu_fwd(x2)
    return y.reshape(*shp[:-1], shp[-1] // 2)


# --------------------------------------------------------------------------- gated attention output / GDN out-norm
def sigmoid_gate(a, qkv, Hq, Hkv, D):
    """out[t,h,:] = a[t,h,:] * sigmoid(gate[t,h,:]) with gate read in place from the fused q block."""
    T = a.shape[0]
    _obs.note("activation.attn_gate", "fused_sigmoid_gate" if _is_cuda(a) else "cpu_sigmoid_gate")
    out = torch.empty_like(a)
    if T == 0:
        return out
    if _is_cuda(a):
        _native.check(_native.lib().ix_sigmoid_gate(a.data_ptr(), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), T, Hq, Hkv, D,
                                                    _native.stream()), "ix_sigmoid_gate")
    else:
        _cpu.lib().ixc_sigmoid_gate(a.data_ptr(), qkv.data_ptr(), qkv.stride(0), out.data_ptr(), T, Hq, Hkv, D, _cpu.dt(a))
    return out


def gated_outnorm(o, z, w, eps=1e-6, zero_centered=False):
    """rows = (token, value head): rms_norm(o) * g * silu(z), the GatedDeltaNet output norm."""
    shp = o.shape
    D = shp[-1]
    o2, z2 = o.reshape(-1, D).contiguous(), z.reshape(-1, D).contiguous()
    out = torch.empty_like(o2)
    if o2.shape[0] == 0:
        return out.reshape(shp)
    _obs.note("norms.gated_out", "fused_gated_outnorm" if _is_cuda(o2) else "cpu_gated_outnorm")
    if _is_cuda(o2):
        _native.check(_native.lib().ix_gated_outnorm(o2.data_ptr(), z2.data_ptr(), w.data_ptr(), out.data_ptr(),
                                                     o2.shape[0], D, eps, int(zero_centered), _native.stream()),
                      "ix_gated_outnorm")
    else:
        _cpu.lib().ixc_gated_outnorm(o2.data_ptr(), z2.data_ptr(), w.data_ptr(), out.data_ptr(), o2.shape[0], D, eps,
                                     int(zero_centered), _cpu.dt(o2))
    return out.reshape(shp)


# --------------------------------------------------------------------------- token log-probabilities (rowinv)
DEFAULT_LEAVES = 8


def logprob_fused_fwd(logits, targets, leaves=DEFAULT_LEAVES, want_entropy=False):
    """logits [rows, V] (bf16/fp32), targets int64 [rows] (negative = ignore -> 0).
    Returns (logprob, lse, entropy|None), all fp32 [rows]."""
    rows, V = logits.shape
    assert logits.stride(1) == 1
    lp = torch.empty(rows, device=logits.device, dtype=torch.float32)
    lse = torch.empty_like(lp)
    ent = torch.empty_like(lp) if want_entropy else None
    if rows == 0:
        return lp, lse, ent
    _obs.note("logprobs.log_softmax", "rowinv_leaftree" if _is_cuda(logits) else "cpu_rowinv_leaftree")
    targets = targets.to(torch.int64).contiguous()
    is_f32 = int(logits.dtype == torch.float32)
    if _is_cuda(logits):
        _native.check(_native.lib().ix_logprob_fused(logits.data_ptr(), logits.stride(0), rows, V, leaves,
                                                     targets.data_ptr(), lp.data_ptr(), lse.data_ptr(),
                                                     _native.ptr(ent), is_f32, _native.stream()), "ix_logprob_fused")
    else:
        _cpu.lib().ixc_logprob_fused(logits.data_ptr(), logits.stride(0), rows, V, leaves, targets.data_ptr(),
                                     lp.data_ptr(), lse.data_ptr(), _cpu.ptr(ent), _cpu.dt(logits))
    return lp, lse, ent


def logprob_bwd(logits, targets, lse, g_lp, g_ent=None, entropy=None, col_base=0, inplace=False):
    """d loss / d logits for the rowinv forward; ``inplace`` overwrites the logits buffer."""
    rows, V = logits.shape
    out = logits if inplace else torch.empty_like(logits)
    if rows == 0:
        return out
    if logits.is_cuda:
        _native.check(_native.lib().ix_logprob_bwd(logits.data_ptr(), logits.stride(0), rows, V, col_base,
                                                   targets.data_ptr(), lse.data_ptr(), _native.ptr(g_lp),
                                                   _native.ptr(g_ent), _native.ptr(entropy), out.data_ptr(),
                                                   out.stride(0), int(logits.dtype == torch.float32),
                                                   _native.stream()), "ix_logprob_bwd")
        return out
    x = logits.float()
    p = torch.exp(x - lse[:, None])
    g = torch.zeros_like(x)
    if g_lp is not None:
        oh = torch.zeros_like(x)
        t = targets - col_base
        ok = (t >= 0) & (t < V)
        oh[ok.nonzero()[:, 0], t[ok]] = 1.0
        g = g_lp[:, None] * (oh - p)
    if g_ent is not None:
        g = g + g_ent[:, None] * (-p * (x - lse[:, None] + entropy[:, None]))
    out.copy_(g.to(logits.dtype))
    return out


class _TokenLogprobs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, leaves, want_entropy):
        lp, lse, ent = logprob_fused_fwd(logits, targets, leaves, want_entropy)
        ctx.save_for_backward(logits, targets.to(torch.int64).contiguous(), lse, ent if ent is not None else lse)
        ctx.want_entropy = want_entropy
        if ent is None:
            ent = torch.zeros_like(lp)
            ctx.mark_non_differentiable(ent)
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        logits, targets, lse, ent = ctx.saved_tensors
        g_lp = g_lp.contiguous().float()
        ge = g_ent.contiguous().float() if (ctx.want_entropy and g_ent is not None) else None
        return logprob_bwd(logits, targets, lse, g_lp, ge, ent if ge is not None else None), None, None, None


def token_logprobs(logits, targets, leaves=DEFAULT_LEAVES, want_entropy=False):
    """(logprob, entropy) of ``targets`` under ``softmax(logits)`` with the fixed-leaf reduction."""
    if torch.is_grad_enabled() and logits.requires_grad:
        return _TokenLogprobs.apply(logits, targets, leaves, want_entropy)
    lp, _, ent = logprob_fused_fwd(logits, targets, leaves, want_entropy)
    return lp, (ent if ent is not None else torch.zeros_like(lp))


# --------------------------------------------------------------------------- fixed-order reductions / optimizer
def reduce_sum_fixed(x: torch.Tensor, square: bool = False, out: torch.Tensor | None = None,
                     accumulate: bool = False, scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Sum (or sum of squares) of a flat bf16/fp32 tensor in an order that depends only on its length."""
    x = x.reshape(-1)
    n = x.numel()
    if x.is_cuda:
        L = _native.lib()
        if out is None:
            out = torch.zeros(1, device=x.device, dtype=torch.float32)
        need = max(1, L.ix_reduce_scratch_elems(n))
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(need, device=x.device, dtype=torch.float32)
        _native.check(L.ix_reduce_sum(x.data_ptr(), n, int(x.dtype == torch.float32), int(square), scratch.data_ptr(),
                                      out.data_ptr(), int(accumulate), _native.stream()), "ix_reduce_sum")
        return out
    v = _cpu.lib().ixc_reduce_sum(x.data_ptr(), n, _cpu.dt(x), int(square)) if n else 0.0
    res = torch.tensor([v], dtype=torch.float32)
    if out is not None:
        out.copy_(out + res if accumulate else res)
        return out
    return res


def softmax_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
