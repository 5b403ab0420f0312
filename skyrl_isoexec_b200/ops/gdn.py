"""GatedDeltaNet layer: shared by trainer and engine (reference: ISO/ops/gdn/gdn_ops.py:74-316,1197-1210
for the math, ISO/ops/gdn/gdn_recurrent_state.py:628-869 for the engine-side prefill/decode flow).

Layer dataflow: in_proj -> [q | k | v | z | b | a]; width-4 causal conv + SiLU over q|k|v that
never crosses a sequence boundary; q, k L2-normalised per head (q scaled by Dk^-0.5);
g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b); gated delta-rule scan with an fp32
state per value head; gated output norm rms_norm(o) * gamma * silu(z); out_proj (row-parallel).

Forward = the kernels of csrc/gdn.cu (or their C++ restatement on CPU): one sequential scan per
(sequence chunk, value head), which is literally the same arithmetic whether the chunk is a whole
training sequence, a prefill chunk continuing from the state pool, or a single decode token.
Backward (outside the contract) = autograd through ``gdn_core_torch``, a chunked (WY / UT
transform) formulation of the same recurrence in plain torch.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..core import observe as _obs
from . import _cpu, _native
from . import functional as F

SCAN_CHUNK_DTYPE = np.dtype([("tok_start", "<i4"), ("n_tok", "<i4"), ("pos0", "<i4"), ("pad", "<i4"),
                             ("row_in", "<i8"), ("row_out", "<i8")])


@dataclass
class GDNMeta:
    """Sequence layout of one forward for the GDN layers.
    chunks     uint8 tensor holding ``ScanChunk`` records (one per sequence chunk in the batch)
    tok_back   int32 [T]: earlier tokens of the same sequence inside this batch
    state_row  int64 [T]: conv/ssm state row of the token's sequence (-1 = start from zeros)
    lens       chunk lengths (host list, used by the backward)"""

    chunks: torch.Tensor
    tok_back: torch.Tensor
    state_row: torch.Tensor | None
    lens: list[int]
    n_chunks: int
    uses_state: bool = False
    host_chunks: list | None = None       # the (tok_start, n_tok, pos0, row_in, row_out) tuples the tables were built from
    plan: dict | None = None              # index tensors of the chunked scan, built by the first GDN layer of a step

    @staticmethod
    def build(chunk_list, device) -> "GDNMeta":
        """chunk_list: [(tok_start, n_tok, pos0, row_in, row_out)]."""
        arr = np.zeros(len(chunk_list), dtype=SCAN_CHUNK_DTYPE)
        T = sum(c[1] for c in chunk_list)
        back = np.zeros(T, dtype=np.int32)
        srow = np.full(T, -1, dtype=np.int64)
        for i, (ts, n, pos0, rin, rout) in enumerate(chunk_list):
            arr[i] = (ts, n, pos0, 0, rin, rout)
            back[ts:ts + n] = np.arange(n)
            srow[ts:ts + n] = rin
        uses = any(c[3] >= 0 or c[4] >= 0 for c in chunk_list)
        ch = torch.from_numpy(arr.view(np.uint8).copy())
        return GDNMeta(ch.to(device), torch.from_numpy(back).to(device), torch.from_numpy(srow).to(device) if uses else None,
                       [c[1] for c in chunk_list], len(chunk_list), uses, host_chunks=[tuple(int(x) for x in c) for c in chunk_list])

    @staticmethod
    def packed(seq_lens, device) -> "GDNMeta":
        out, s = [], 0
        for n in seq_lens:
            out.append((s, n, 0, -1, -1))
            s += n
        return GDNMeta.build(out, device)


def _dims(cfg, tp):
    hk, hv, d = cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp, cfg.gdn_head_dim
    return hk, hv, d, hk * d, hv * d


# ------------------------------------------------------------------------------------ kernel wrappers
def _is_f32(t):
    return int(t.dtype == torch.float32)


def _chunk_plan(meta: GDNMeta, rows: int, device) -> dict:
    """Index tensors that lay the open chunk of every sequence (kept tokens since its last chunk boundary) in front of
    the sequence's new tokens, and that write the new open chunk back. Same for every GDN layer of a step."""
    if meta.plan is not None:
        return meta.plan
    T = sum(c[1] for c in meta.host_chunks)
    gather, segs, new_rows, keep_src, keep_dst = [], [], [], [], []
    base = 0
    for tok, n, pos0, rin, rout in meta.host_chunks:
        fill = pos0 % CHUNK
        row = rout if rout >= 0 else rin
        if fill and row < 0:
            raise ValueError("a sequence continues inside a chunk but has no state row holding its open chunk")
        gather += [row * CHUNK + j for j in range(fill)] + [rows * CHUNK + tok + j for j in range(n)]
        c0 = pos0 - fill
        segs.append((base, fill + n, rin if c0 > 0 else -1, rout))
        new_rows += [base + fill + j for j in range(n)]
        nfill = (pos0 + n) % CHUNK
        if rout >= 0 and nfill:
            keep_src += [base + fill + n - nfill + j for j in range(nfill)]
            keep_dst += [rout * CHUNK + j for j in range(nfill)]
        base += fill + n
    mk = lambda x: torch.tensor(x, dtype=torch.int64, device=device)
    meta.plan = {"gather": mk(gather), "segments": segs, "new_rows": mk(new_rows), "keep_src": mk(keep_src), "keep_dst": mk(keep_dst),
                 "identity": not meta.uses_state, "T": T}
    return meta.plan


def _chunked_core(qn, kn, vv, g, beta, meta: GDNMeta, ssm_state, chunk_buf):
    """The scan by the chunked tensor-core kernels. Trainer: packed whole sequences. Engine: every sequence's open chunk is
    kept in ``chunk_buf`` (post-conv q, k, v and the gates of up to 63 tokens) and is re-run in front of the new tokens,
    from the fp32 state at its chunk boundary, so a decode step computes the very row a whole-sequence scan computes."""
    if not meta.uses_state:
        segs, s0 = [], 0
        for n in meta.lens:
            segs.append((s0, n, -1, -1))
            s0 += n
        return gdn_chunk_scan(qn, kn, vv, g, beta, segs, None)
    rows = ssm_state.shape[0]
    plan = _chunk_plan(meta, rows, qn.device)
    names = ("q", "k", "v", "g", "b")
    new = dict(zip(names, (qn, kn, vv, g, beta)))
    full = {}
    for nm in names:
        buf = chunk_buf[nm]
        both = torch.cat([buf.reshape((rows * CHUNK,) + tuple(buf.shape[2:])), new[nm]], 0)
        full[nm] = both.index_select(0, plan["gather"]).contiguous()
    out = gdn_chunk_scan(full["q"], full["k"], full["v"], full["g"], full["b"], plan["segments"], ssm_state)
    if plan["keep_src"].numel():
        for nm in names:
            buf = chunk_buf[nm]
            buf.reshape((rows * CHUNK,) + tuple(buf.shape[2:])).index_copy_(0, plan["keep_dst"], full[nm].index_select(0, plan["keep_src"]))
    return out.index_select(0, plan["new_rows"])


def new_chunk_buffers(rows: int, hk: int, hv: int, d: int, dtype, device) -> dict:
    """Per state row: the tokens of the sequence's open chunk (q, k [64, Hk, D], v [64, Hv, D], log-decay and beta [64, Hv])."""
    z = lambda *shape, dt=dtype: torch.zeros(rows, CHUNK, *shape, dtype=dt, device=device)
    return {"q": z(hk, d), "k": z(hk, d), "v": z(hv, d), "g": z(hv, dt=torch.float32), "b": z(hv, dt=torch.float32)}


def chunked_ok(proj, d: int) -> bool:
    return proj.is_cuda and proj.dtype == torch.bfloat16 and d in (64, 128)


def gdn_core_fwd(proj, conv_w, A_log, dt_bias, meta: GDNMeta, cfg, tp, conv_state=None, ssm_state=None, chunk_buf=None):
    """proj: [T, 2kd+2vd+2Hv] (in_proj output). Returns o [T, Hv, Dv]. Updates the state pools in place
    when ``meta`` names state rows. On a GPU in bf16 the scan is the chunked tensor-core form (``_chunked_core``); with
    state rows it needs ``chunk_buf`` (``new_chunk_buffers``). CPU / fp32: the sequential scan."""
    hk, hv, d, kd, vd = _dims(cfg, tp)
    T = proj.shape[0]
    C, W = 2 * kd + vd, cfg.gdn_conv_kernel
    dev = proj.device
    qkv = torch.empty(T, C, dtype=proj.dtype, device=dev)
    g = torch.empty(T, hv, dtype=torch.float32, device=dev)
    beta = torch.empty_like(g)
    qn = torch.empty(T, hk, d, dtype=proj.dtype, device=dev)
    kn = torch.empty_like(qn)
    o = torch.empty(T, hv, d, dtype=proj.dtype, device=dev)
    if T == 0:
        return o
    ab = proj[:, C + vd:]                       # [b(Hv) | a(Hv)]
    snap = cfg.gdn_chunk if getattr(cfg, "gdn_snapshot", False) else 0
    if ssm_state is None:
        ssm_state = torch.empty(0, dtype=torch.float32, device=dev)
    args_cs = None if conv_state is None else conv_state.data_ptr()
    # one token per chunk with a state row behind it is the recurrent decode step; anything longer is the scan
    _obs.note("gdn.core", "cpr_recurrent_step" if (meta.uses_state and T == meta.n_chunks) else "cpr_chunk_scan")
    _obs.note("gdn.conv", "shifted_sum_conv")
    _obs.note("gdn.gating", "fp32_gating")
    if meta.uses_state:
        _obs.note("gdn.state", "slot_pool")
    if proj.is_cuda:
        L, s, f32 = _native.lib(), _native.stream(), _is_f32(proj)
        ck = _native.check
        ck(L.ix_gdn_conv(proj.data_ptr(), proj.stride(0), conv_w.data_ptr(), meta.tok_back.data_ptr(), _native.ptr(meta.state_row),
                         args_cs, qkv.data_ptr(), T, C, W, f32, s), "ix_gdn_conv")
        if meta.uses_state and conv_state is not None:
            ck(L.ix_gdn_conv_state(proj.data_ptr(), proj.stride(0), meta.chunks.data_ptr(), conv_state.data_ptr(), meta.n_chunks, C, W,
                                   f32, s), "ix_gdn_conv_state")
        ck(L.ix_gdn_gate(ab[:, hv:].data_ptr(), ab.data_ptr(), proj.stride(0), A_log.data_ptr(), dt_bias.data_ptr(), g.data_ptr(),
                         beta.data_ptr(), T, hv, f32, s), "ix_gdn_gate")
        ck(L.ix_gdn_l2norm(qkv.data_ptr(), C, qn.data_ptr(), kn.data_ptr(), T, hk, d, 1e-6, d ** -0.5, f32, s), "ix_gdn_l2norm")
        vv = qkv[:, 2 * kd:].contiguous()          # the scan indexes v as packed [T, Hv, Dv]
        if chunked_ok(proj, d) and (not meta.uses_state or chunk_buf is not None):
            o = _chunked_core(qn, kn, vv.view(T, hv, d), g, beta, meta, ssm_state if meta.uses_state else None, chunk_buf)
        else:
            ck(L.ix_gdn_scan(qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), g.data_ptr(), beta.data_ptr(), meta.chunks.data_ptr(),
                             ssm_state.data_ptr(), o.data_ptr(), meta.n_chunks, hk, hv, d, d, snap, f32, s), "ix_gdn_scan")
    else:
        L, dt = _cpu.lib(), _cpu.dt(proj)
        L.ixc_gdn_conv(proj.data_ptr(), proj.stride(0), conv_w.data_ptr(), meta.tok_back.data_ptr(), _cpu.ptr(meta.state_row), args_cs,
                       qkv.data_ptr(), T, C, W, dt)
        if meta.uses_state and conv_state is not None:
            L.ixc_gdn_conv_state(proj.data_ptr(), proj.stride(0), meta.chunks.data_ptr(), conv_state.data_ptr(), meta.n_chunks, C, W, dt)
        L.ixc_gdn_gate(ab[:, hv:].data_ptr(), ab.data_ptr(), proj.stride(0), A_log.data_ptr(), dt_bias.data_ptr(), g.data_ptr(),
                       beta.data_ptr(), T, hv, dt)
        L.ixc_gdn_l2norm(qkv.data_ptr(), C, qn.data_ptr(), kn.data_ptr(), T, hk, d, 1e-6, d ** -0.5, dt)
        # the v block of qkv is a strided view: the scan wants it packed
        vv = qkv[:, 2 * kd:].contiguous()
        L.ixc_gdn_scan(qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), g.data_ptr(), beta.data_ptr(), meta.chunks.data_ptr(),
                       ssm_state.data_ptr(), o.data_ptr(), meta.n_chunks, hk, hv, d, d, snap, dt)
    return o


# ------------------------------------------------------------------------------------ chunked scan on the tensor cores
CHUNK = 64
_CHUNK_DT = np.dtype([("tok_start", "<i4"), ("n_tok", "<i4")])
_CHAIN_DT = np.dtype([("chunk_begin", "<i4"), ("chunk_end", "<i4"), ("row_in", "<i8"), ("row_out", "<i8")])


def chunk_tables(segments, device):
    """Device tables for ``gdn_chunk_scan``. ``segments``: [(tok_start, n_tok, row_in, row_out)], one per sequence, each
    starting ON a chunk boundary of its sequence (position multiple of 64). Returns (chunks, chains, n_chunks, n_chains)."""
    ch, cn = [], []
    for ts, n, rin, rout in segments:
        b = len(ch)
        for lo in range(0, n, CHUNK):
            ch.append((ts + lo, min(CHUNK, n - lo)))
        cn.append((b, len(ch), rin, rout))
    a = np.array(ch, dtype=_CHUNK_DT)
    c = np.array(cn, dtype=_CHAIN_DT)
    return (torch.from_numpy(a.view(np.uint8).copy()).to(device), torch.from_numpy(c.view(np.uint8).copy()).to(device), len(ch), len(cn))


def gdn_chunk_scan(qn, kn, v, g, beta, segments, state=None):
    """Gated delta rule over packed sequences by the chunked tcgen05 kernels (csrc/gdn_chunk.cu).
    qn, kn: [T, Hk, D] bf16 (normalised), v: [T, Hv, D] bf16, g, beta: [T, Hv] fp32; ``segments`` as in ``chunk_tables``;
    ``state``: fp32 pool [rows, Hv, D, D] read at ``row_in`` and written at ``row_out`` (after the last complete chunk)."""
    import ctypes as C

    T, Hk, D = qn.shape
    Hv = v.shape[1]
    assert qn.dtype == torch.bfloat16 and qn.is_contiguous() and kn.is_contiguous() and v.is_contiguous()
    assert g.dtype == torch.float32 and g.is_contiguous() and beta.is_contiguous()
    out = torch.empty(T, Hv, D, dtype=torch.bfloat16, device=qn.device)
    if T == 0:
        return out
    chunks, chains, n_chunks, n_chains = chunk_tables(segments, qn.device)
    lib = _native.lib()
    if not getattr(lib, "_gdn_chunk_sig", False):
        lib.ix_gdn_chunk_scratch_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
        lib.ix_gdn_chunk_scratch_bytes.restype = C.c_longlong
        lib.ix_gdn_chunk_fwd.argtypes = [C.c_void_p] * 6 + [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 4
        lib._gdn_chunk_sig = True
    scratch = torch.empty(int(lib.ix_gdn_chunk_scratch_bytes(n_chunks, Hv, D)), dtype=torch.uint8, device=qn.device)
    _native.check(lib.ix_gdn_chunk_fwd(qn.data_ptr(), kn.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), chunks.data_ptr(),
                                       n_chunks, chains.data_ptr(), n_chains, Hk, Hv, D, scratch.data_ptr(), _native.ptr(state),
                                       out.data_ptr(), _native.stream()), "ix_gdn_chunk_fwd")
    return out


# ------------------------------------------------------------------------------------ torch formulation (backward only)
def chunk_gated_delta_rule_torch(q, k, v, g, beta, chunk: int = 64):
    """q, k: [H, T, Dk] (already normalised / scaled), v: [H, T, Dv], g, beta: [H, T] fp32.
    Chunked (UT-transform) evaluation of the gated delta rule, equal to the token recurrence up to
    fp32 rounding. Returns o [H, T, Dv]."""
    H, T, Dk = q.shape
    Dv = v.shape[-1]
    pad = (-T) % chunk
    if pad:
        zp = lambda x: torch.nn.functional.pad(x, (0, 0, 0, pad))
        q, k, v = zp(q), zp(k), zp(v)
        g, beta = torch.nn.functional.pad(g, (0, pad)), torch.nn.functional.pad(beta, (0, pad))
    n = (T + pad) // chunk
    q, k, v = (x.reshape(H, n, chunk, -1) for x in (q, k, v))
    g, beta = g.reshape(H, n, chunk), beta.reshape(H, n, chunk)
    G = g.cumsum(-1)                                              # cumulative log-decay inside the chunk
    decay = (G[..., :, None] - G[..., None, :]).tril().exp().tril()    # exp(G_i - G_j) for i >= j
    kb, vb = k * beta[..., None], v * beta[..., None]
    A = -((kb @ k.transpose(-1, -2)) * decay).tril(-1)            # strictly lower
    eye = torch.eye(chunk, dtype=q.dtype, device=q.device)
    Tm = torch.linalg.solve_triangular(eye - A, eye.expand(H, n, chunk, chunk), upper=False)   # (I - A)^-1
    W = Tm @ (kb * G.exp()[..., None])                            # [H, n, C, Dk]
    U = Tm @ vb                                                   # [H, n, C, Dv]
    S = q.new_zeros(H, Dk, Dv)
    outs = []
    qk = ((q @ k.transpose(-1, -2)) * decay).tril()
    for c in range(n):
        v_new = U[:, c] - W[:, c] @ S
        o_inter = (q[:, c] * G[:, c].exp()[..., None]) @ S
        outs.append(o_inter + qk[:, c] @ v_new)
        gl = G[:, c, -1]
        S = S * gl.exp()[:, None, None] + (k[:, c] * (gl[:, None] - G[:, c]).exp()[..., None]).transpose(-1, -2) @ v_new
    return torch.cat(outs, 1)[:, :T]


def gdn_core_torch(proj, conv_w, A_log, dt_bias, lens, cfg, tp):
    """Differentiable torch version of ``gdn_core_fwd`` for packed whole sequences (zero initial state)."""
    hk, hv, d, kd, vd = _dims(cfg, tp)
    C, W = 2 * kd + vd, cfg.gdn_conv_kernel
    rep = hv // hk
    outs, s = [], 0
    for n in lens:
        p = proj[s:s + n].float()
        x = torch.nn.functional.pad(p[:, :C].t(), (W - 1, 0))           # [C, n + W - 1]
        conv = (x.unfold(1, W, 1) * conv_w.float()[:, None, :]).sum(-1).t()   # [n, C]
        qkv = torch.nn.functional.silu(conv)
        qh = qkv[:, :kd].reshape(n, hk, d)
        kh = qkv[:, kd:2 * kd].reshape(n, hk, d)
        vh = qkv[:, 2 * kd:].reshape(n, hv, d)
        qh = qh * torch.rsqrt(qh.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        kh = kh * torch.rsqrt(kh.pow(2).sum(-1, keepdim=True) + 1e-6)
        b, a = p[:, C + vd:C + vd + hv], p[:, C + vd + hv:]
        g = -torch.exp(A_log.float()) * torch.nn.functional.softplus(a + dt_bias.float())
        beta = torch.sigmoid(b)
        o = chunk_gated_delta_rule_torch(qh.repeat_interleave(rep, 1).transpose(0, 1), kh.repeat_interleave(rep, 1).transpose(0, 1),
                                         vh.transpose(0, 1), g.t(), beta.t(), cfg.gdn_chunk)
        outs.append(o.transpose(0, 1))
        s += n
    return torch.cat(outs, 0).to(proj.dtype)


class _GDNCore(torch.autograd.Function):
    @staticmethod
    def forward(ctx, proj, conv_w, A_log, dt_bias, meta, cfg, tp):
        ctx.save_for_backward(proj, conv_w, A_log, dt_bias)
        ctx.cfgs = (meta.lens, cfg, tp)
        return gdn_core_fwd(proj, conv_w, A_log, dt_bias, meta, cfg, tp)

    @staticmethod
    def backward(ctx, do):
        proj, conv_w, A_log, dt_bias = ctx.saved_tensors
        lens, cfg, tp = ctx.cfgs
        with torch.enable_grad():
            ins = [t.detach().requires_grad_(True) for t in (proj, conv_w, A_log, dt_bias)]
            o = gdn_core_torch(*ins, lens, cfg, tp)
            grads = torch.autograd.grad(o, ins, do.to(o.dtype), allow_unused=True)
        return (*[None if g is None else g.to(t.dtype) for g, t in zip(grads, ins)], None, None, None)


# ------------------------------------------------------------------------------------ the layer
def gdn_block(y, model, i: int, fc, kv_idx: int):
    from ..parallel import tp as tp_ops

    cfg, ps = model.cfg, model.ps
    pfx = f"layers.{i}.gdn."
    hk, hv, d, kd, vd = _dims(cfg, ps.tp)
    C = 2 * kd + vd
    proj = F.linear(tp_ops.copy_to_tp(y, ps), model.p(pfx + "in_proj.weight"))
    meta = fc.gdn_meta
    assert meta is not None, "GDN layers need ForwardCtx.gdn_meta"
    conv_w, A_log, dt_bias = model.p(pfx + "conv.weight"), model.p(pfx + "A_log"), model.p(pfx + "dt_bias")
    if fc.kv is None:
        if torch.is_grad_enabled() and proj.requires_grad:
            o = _GDNCore.apply(proj, conv_w, A_log, dt_bias, meta, cfg, ps.tp)
        else:
            o = gdn_core_fwd(proj, conv_w, A_log, dt_bias, meta, cfg, ps.tp)
    else:
        st = fc.kv[kv_idx]
        conv_state, ssm_state = st[0], st[1]
        o = gdn_core_fwd(proj, conv_w, A_log, dt_bias, meta, cfg, ps.tp, conv_state, ssm_state, st[2] if len(st) > 2 else None)
    z = proj[:, C:C + vd].reshape(-1, hv, d)
    if torch.is_grad_enabled() and (o.requires_grad or proj.requires_grad):
        w = model.p(pfx + "out_norm.weight").float()
        gamma = (1.0 + w) if cfg.zero_centered_norm else w
        of = o.float()
        n = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + cfg.rms_eps)
        gated = (n * gamma * torch.nn.functional.silu(z.float())).to(o.dtype)
        # forward value must be the kernel's bits: take them from the kernel, keep the torch graph for the gradient
        with torch.no_grad():
            exact = F.gated_outnorm(o, z, model.p(pfx + "out_norm.weight"), cfg.rms_eps, cfg.zero_centered_norm)
        gated = gated + (exact - gated).detach()
    else:
        gated = F.gated_outnorm(o, z, model.p(pfx + "out_norm.weight"), cfg.rms_eps, cfg.zero_centered_norm)
    return tp_ops.row_parallel_linear(gated.reshape(-1, vd), model.p(pfx + "out_proj.weight"), ps, cfg)
