"""sm_100a kernels against (a) a plain PyTorch fp32 reference of the same op and (b) the C++ CPU
restatement with the same reduction order (bitwise where the chain has no transcendental
function). Also the invariance properties the execution contract claims."""
import math

import pytest
import torch

from skyrl_isoexec_b200.core.testing import bitwise_equal, count_bit_mismatches
from skyrl_isoexec_b200.ops import _native
from skyrl_isoexec_b200.ops import functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert _native.read_status() == 0, "a kernel's bounded wait ran out"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1000, 4096, 1024), (8, 4096, 4096), (333, 1000, 776), (1, 2048, 256)])
def test_gemm_matches_fp32_and_is_invariant(M, N, K):
    torch.manual_seed(0)
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    ref = x.float() @ w.float().T
    outs = {bn: F.gemm_nt(x, w, bn=bn) for bn in (32, 48, 64, 128, 208, 256)}
    for o in outs.values():
        assert (o.float() - ref).abs().max() <= 1e-2 * ref.abs().max() + 1e-3
    assert all(bitwise_equal(outs[32], outs[b]) for b in (48, 64, 128, 208, 256))       # N-tile invariance
    k = min(M, 3)
    assert bitwise_equal(F.gemm_nt(x[:k].contiguous(), w), outs[256][:k])        # row-count invariance
    f32 = F.gemm_nt(x, w, out_f32=True)
    assert (f32 - ref).abs().max() <= 2e-4 * max(1.0, ref.abs().max().item())
    assert bitwise_equal(f32.bfloat16(), outs[256])                               # bf16 out = one round of the fp32 acc


@pytest.mark.parametrize("M,N,R", [(300, 512, 1024), (8192, 4096, 1536), (1, 264, 64), (4097, 12288, 4096), (640, 72, 8)])
def test_input_gradient_gemm_nn_matches_fp32(M, N, R):
    """dX = dY[M,R] @ W[R,N]: W is read M/N-major by the MMA (no transposed copy), against an fp32 product."""
    torch.manual_seed(2)
    dy = (torch.randn(M, R, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(R, N, device=DEV) * 0.05).bfloat16()
    ref = dy.float() @ w.float()
    got = F.gemm_nn(dy, w, out_f32=True)
    assert (got - ref).abs().max() <= 2e-4 * max(1.0, ref.abs().max().item())
    assert bitwise_equal(F.gemm_nn(dy, w), got.bfloat16())
    assert bitwise_equal(F.gemm_nn(dy, w), F.gemm_nn(dy, w))
    big = torch.zeros(M, R + 64, device=DEV, dtype=torch.bfloat16)
    big[:, 32:32 + R] = dy
    assert bitwise_equal(F.gemm_nn(big[:, 32:32 + R], w), got.bfloat16()) if (R + 64) % 8 == 0 else True     # strided rows


@pytest.mark.parametrize("M,N,R", [(512, 1024, 300), (4096, 1536, 8192), (264, 64, 1), (12288, 4096, 4097), (72, 8, 640)])
def test_weight_gradient_gemm_tn_matches_fp32_and_accumulates(M, N, R):
    """dW[M,N] = dY[R,M]^T @ X[R,N] with both operands read M/N-major; R (the token count) need not be a multiple of
    anything. The accumulating form adds the product to an fp32 buffer in the epilogue."""
    torch.manual_seed(3)
    dy = (torch.randn(R, M, device=DEV) * 0.5).bfloat16()
    x = (torch.randn(R, N, device=DEV) * 0.25).bfloat16()
    ref = dy.float().T @ x.float()
    got = F.gemm_tn(dy, x, out_f32=True)
    tol = 2e-4 * max(1.0, ref.abs().max().item())
    assert (got - ref).abs().max() <= tol
    assert bitwise_equal(F.gemm_tn(dy, x), got.bfloat16())
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    F.gemm_tn(dy, x, out=acc, accumulate=True)
    assert bitwise_equal(acc, base + got)
    F.gemm_tn(dy, x, out=acc, accumulate=False)
    assert bitwise_equal(acc, got)


def test_linear_backward_uses_own_gemms_and_matches_fp32_autograd():
    torch.manual_seed(4)
    x = (torch.randn(777, 1024, device=DEV) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(2048, 1024, device=DEV) * 0.05).bfloat16().requires_grad_()
    g = (torch.randn(777, 2048, device=DEV) * 0.1).bfloat16()
    n0 = F._native.launch_count()
    F.linear(x, w).backward(g)
    assert F._native.launch_count() - n0 == 3                       # forward NT, input-gradient NN, weight-gradient TN
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xf @ wf.T).backward(g.float())
    assert (x.grad.float() - xf.grad).abs().max() <= 1e-2 * xf.grad.abs().max()
    assert (w.grad.float() - wf.grad).abs().max() <= 1e-2 * wf.grad.abs().max()


def test_gemm_strided_input_rows():
    torch.manual_seed(1)
    big = (torch.randn(64, 512, device=DEV)).bfloat16()
    x = big[:, 128:384]                      # row stride 512, K = 256
    w = (torch.randn(96, 256, device=DEV) * 0.1).bfloat16()
    assert bitwise_equal(F.gemm_nt(x, w), F.gemm_nt(x.contiguous(), w))


@pytest.mark.parametrize("N", [4096, 2560, 1000 * 8])
def test_rmsnorm_few_rows_kernel_equals_many_rows_kernel_bitwise(N):
    """Decode-sized launches use a CTA per row, large ones a warp per row: one reduction order, same bits."""
    torch.manual_seed(6)
    x = torch.randn(1500, N, device=DEV).bfloat16()
    r = torch.randn(1500, N, device=DEV).bfloat16()
    w = (torch.randn(N, device=DEV) * 0.1 + 1).bfloat16()
    y_big, res_big, rstd_big = F.rmsnorm_fwd(x, w, 1e-6, False, r, want_rstd=True)            # 1500 rows: warp per row
    y_small, res_small, rstd_small = F.rmsnorm_fwd(x[:64].contiguous(), w, 1e-6, False, r[:64].contiguous(), want_rstd=True)
    assert bitwise_equal(y_small, y_big[:64]) and bitwise_equal(res_small, res_big[:64]) and bitwise_equal(rstd_small, rstd_big[:64])
    y1, _, _ = F.rmsnorm_fwd(x[:3].contiguous(), w, 1e-6, True)
    y2, _, _ = F.rmsnorm_fwd(x[:1100].contiguous(), w, 1e-6, True)
    assert bitwise_equal(y1, y2[:3])


@pytest.mark.parametrize("zero_centered,with_res", [(False, True), (True, False)])
def test_rmsnorm_backward_kernel_matches_fp32_autograd(zero_centered, with_res):
    torch.manual_seed(2)
    rows, N = 333, 1024
    x = torch.randn(rows, N, device=DEV).bfloat16().requires_grad_()
    res = torch.randn(rows, N, device=DEV).bfloat16().requires_grad_() if with_res else None
    w = (torch.randn(N, device=DEV) * 0.2 + (0.0 if zero_centered else 1.0)).bfloat16().requires_grad_()
    gy, gr = torch.randn(rows, N, device=DEV).bfloat16(), torch.randn(rows, N, device=DEV).bfloat16()
    y, r = F.rmsnorm(x, w, 1e-6, zero_centered, res)
    loss = (y.float() * gy.float()).sum() + ((r.float() * gr.float()).sum() if with_res else 0.0)
    dx, dw = torch.autograd.grad(loss, [x, w])
    # fp32 reference of the same function
    xf = x.detach().float().requires_grad_()
    wf = w.detach().float().requires_grad_()
    h = (xf + res.detach().float()) if with_res else xf
    n = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6)
    yf = n * ((1.0 + wf) if zero_centered else wf)
    lf = (yf * gy.float()).sum() + ((h * gr.float()).sum() if with_res else 0.0)
    dxf, dwf = torch.autograd.grad(lf, [xf, wf])
    assert (dx.float() - dxf).abs().max() <= 2e-2 * dxf.abs().max()
    assert (dw.float() - dwf).abs().max() <= 2e-2 * dwf.abs().max()
    # fixed-order weight-gradient fold: two runs, same bits
    y2, r2 = F.rmsnorm(x, w, 1e-6, zero_centered, res)
    loss2 = (y2.float() * gy.float()).sum() + ((r2.float() * gr.float()).sum() if with_res else 0.0)
    assert bitwise_equal(torch.autograd.grad(loss2, [w])[0], dw)


@pytest.mark.parametrize("gate", [False, True])
def test_qk_norm_rope_backward_kernel_matches_cpu_composite(gate):
    torch.manual_seed(4)
    T, Hq, Hkv, D = 77, 8, 2, 128
    width = (Hq * (2 * D if gate else D)) + 2 * Hkv * D
    rope = {d: F.RopeTable(D, 256, 1e6, d) for d in ("cpu", DEV)}
    qkv0 = torch.randn(T, width).bfloat16()
    qw0, kw0 = (torch.randn(D) * 0.2 + 1).bfloat16(), (torch.randn(D) * 0.2 + 1).bfloat16()
    pos0 = torch.randint(0, 256, (T,), dtype=torch.int32)
    gq, gk, gv = torch.randn(T, Hq, D).bfloat16(), torch.randn(T, Hkv, D).bfloat16(), torch.randn(T, Hkv, D).bfloat16()
    grads = {}
    for d in ("cpu", DEV):
        qkv, qw, kw = (t.to(d).requires_grad_() for t in (qkv0, qw0, kw0))
        q, k, v = F.qk_norm_rope_train(qkv, pos0.to(d), rope[d], qw, kw, Hq, Hkv, D, 1e-6, True, False, gate)
        loss = (q.float() * gq.to(d).float()).sum() + (k.float() * gk.to(d).float()).sum() + (v.float() * gv.to(d).float()).sum()
        grads[d] = [g.cpu().float() for g in torch.autograd.grad(loss, [qkv, qw, kw])]
    for a, b in zip(grads[DEV], grads["cpu"]):
        assert (a - b).abs().max() <= 2e-2 * b.abs().max() + 1e-3


@pytest.mark.parametrize("T,E,k", [(7, 8, 2), (700, 16, 4)])
def test_grouped_expert_gemm_equals_per_expert_loop_bitwise(T, E, k):
    """One grouped launch (fc1 + SwiGLU + gate weight fused; fc2 with fp32 out, plain and scattered) gives the bits
    of the per-expert loop over the dense kernels, including empty experts and ragged last tiles."""
    from skyrl_isoexec_b200.ops import moe

    torch.manual_seed(5)
    H, Fd = 256, 192
    x = torch.randn(T, H, device=DEV).bfloat16()
    gate_up = (torch.randn(E, 2 * Fd, H, device=DEV) * 0.06).bfloat16()
    down = (torch.randn(E, H, Fd, device=DEV) * 0.06).bfloat16()
    idx = torch.stack([torch.randperm(E - 1, device=DEV)[:k] for _ in range(T)]).int()      # the last expert stays empty
    order, counts, pos = moe.build_dispatch(idx, E)
    assert int(counts[-1]) == 0
    x_rows = x.index_select(0, torch.div(order, k, rounding_mode="floor"))
    w_rows = torch.rand(T * k, device=DEV)
    with torch.no_grad():
        want = moe._expert_rows(x_rows, w_rows, counts.tolist(), gate_up, down)
        offs = moe.counts_to_offsets(counts)
        got = moe.expert_rows_grouped(x_rows, w_rows, offs, gate_up, down)
        assert bitwise_equal(got, want)
        for bn in (32, 64, 96):
            a = moe.grouped_gemm(x_rows, gate_up, offs, moe.EPI_GLU, w_rows=w_rows, bn=bn)
            assert bitwise_equal(moe.grouped_gemm(a, down, offs, moe.EPI_F32, bn=min(bn, 64)), want)
        # scattered epilogue: rows land at the addresses given, here a permutation of a local buffer
        a = moe.grouped_gemm(x_rows, gate_up, offs, moe.EPI_GLU, w_rows=w_rows)
        dest = torch.zeros(T * k, H, device=DEV)
        perm = torch.randperm(T * k, device=DEV)
        row_dst = dest.data_ptr() + perm * (H * 4)
        moe.grouped_gemm(a, down, offs, moe.EPI_F32, row_dst=row_dst)
        assert bitwise_equal(dest[perm], want)
        h1 = moe.grouped_gemm(x_rows, gate_up, offs, moe.EPI_BF16)
        lo = int(offs[1])
        assert bitwise_equal(h1[:lo], F.gemm_nt(x_rows[:lo].contiguous(), gate_up[0])) if lo else True


@pytest.mark.parametrize("M", [1, 64, 130, 256])
def test_leaf_parallel_gemm_over_a_cluster_equals_the_one_cta_form_bitwise(M):
    """Decode-sized leaf-tree GEMM with one CTA per leaf, folded through the cluster's shared memory: same bits as the
    form that keeps all leaves in one CTA's TMEM and as the leaf loop, for every leaf count, tile width and output type;
    a strided activation view is taken as it is."""
    from skyrl_isoexec_b200.ops import _native
    from skyrl_isoexec_b200.parallel.tp import tree_fold
    from skyrl_isoexec_b200.parallel.tp_fused import leaftree_gemm_fused

    torch.manual_seed(5)
    N, K = 512, 2048
    xs = torch.randn(M, K + 64, device=DEV).bfloat16()
    x = xs[:, :K]                                               # row stride K + 64
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    for L in (2, 4, 8):
        LK = K // L
        parts = torch.stack([F.gemm_nt(x[:, j * LK:(j + 1) * LK], w[:, j * LK:(j + 1) * LK], out_f32=True) for j in range(L)])
        want = tree_fold(parts)
        assert bitwise_equal(leaftree_gemm_fused(x, w, L, split=False), want)
        assert _native.lib().ix_leaf_split_bn(M, N, K, L) > 0
        assert bitwise_equal(leaftree_gemm_fused(x, w, L), want), f"default form, L={L}"
        for bn in (32, 64, 128):
            if bn // L < 4:
                continue
            assert bitwise_equal(leaftree_gemm_fused(x, w, L, bn=bn, split=True), want), f"L={L} bn={bn}"
            assert bitwise_equal(leaftree_gemm_fused(x, w, L, out_f32=False, bn=bn, split=True), want.bfloat16())
    assert _native.read_status() == 0
    assert _native.lib().ix_leaf_split_bn(4096, N, K, 2) == 0    # training sizes keep the one-CTA form


@pytest.mark.parametrize("M", [5, 300])
def test_leaftree_gemm_one_kernel_equals_leaf_loop_bitwise(M):
    """Leaves accumulate in separate TMEM accumulators and fold in the epilogue: same bits as one GEMM per
    leaf followed by the balanced tree in fp32, for every leaf count; one leaf is the plain GEMM."""
    from skyrl_isoexec_b200.parallel.tp import tree_fold
    from skyrl_isoexec_b200.parallel.tp_fused import leaftree_gemm_fused

    torch.manual_seed(3)
    N, K = 384, 1024
    x = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    assert bitwise_equal(leaftree_gemm_fused(x, w, 1), F.gemm_nt(x, w, out_f32=True))
    for L in (2, 4, 8):
        LK = K // L
        parts = torch.stack([F.gemm_nt(x[:, j * LK:(j + 1) * LK], w[:, j * LK:(j + 1) * LK], out_f32=True) for j in range(L)])
        want = tree_fold(parts)
        got = leaftree_gemm_fused(x, w, L)
        assert bitwise_equal(got, want), f"L={L}"
        assert bitwise_equal(leaftree_gemm_fused(x, w, L, out_f32=False), want.bfloat16())
    ref = x.float() @ w.float().T
    assert (leaftree_gemm_fused(x, w, 8) - ref).abs().max() <= 2e-4 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("zero_centered", [False, True])
@pytest.mark.parametrize("N", [128, 4096, 2560])
def test_rmsnorm_bitwise_vs_cpu_oracle(N, zero_centered):
    torch.manual_seed(2)
    x, r, w = (torch.randn(37, N) * 2).bfloat16(), torch.randn(37, N).bfloat16(), torch.randn(N).bfloat16()
    y_c, res_c, _ = F.rmsnorm_fwd(x, w, 1e-6, zero_centered, r)
    y_g, res_g, _ = F.rmsnorm_fwd(x.to(DEV), w.to(DEV), 1e-6, zero_centered, r.to(DEV))
    assert bitwise_equal(res_g.cpu(), res_c) and bitwise_equal(y_g.cpu(), y_c)
    h = x.float() + r.float()
    g = (1 + w.float()) if zero_centered else w.float()
    ref = h.bfloat16().float() * torch.rsqrt(h.bfloat16().float().pow(2).mean(-1, keepdim=True) + 1e-6) * g
    assert (y_g.cpu().float() - ref).abs().max() <= 0.05 * ref.abs().max()


@pytest.mark.parametrize("qk_norm", [True, False])
@pytest.mark.parametrize("Hq,Hkv,D,gate", [(8, 2, 128, False), (4, 2, 64, False), (4, 2, 128, True)])
def test_qk_norm_rope_bitwise_vs_cpu_oracle(Hq, Hkv, D, gate, qk_norm):
    torch.manual_seed(3)
    T = 53
    rows = (Hq * (2 if gate else 1) + 2 * Hkv) * D
    qkv = torch.randn(T, rows).bfloat16()
    qw, kw = torch.randn(D).bfloat16(), torch.randn(D).bfloat16()
    pos = torch.randint(0, 1000, (T,), dtype=torch.int32)
    slots = torch.randperm(256)[:T].to(torch.int64)
    outs = []
    for dev in ("cpu", DEV):
        rope = F.RopeTable(D, 1024, 1e6, dev)
        kp, vp = torch.zeros(256, Hkv, D, dtype=torch.bfloat16, device=dev), torch.zeros(256, Hkv, D, dtype=torch.bfloat16, device=dev)
        q = F.qk_norm_rope_fwd(qkv.to(dev), pos.to(dev), slots.to(dev), rope, qw.to(dev), kw.to(dev), kp, vp, Hq, Hkv, D, 1e-6,
                               qk_norm, False, gate)
        outs.append((q.cpu(), kp.cpu(), vp.cpu()))
    for a, b in zip(*outs):
        assert bitwise_equal(a, b)


def _attn_ref(q, k, v, lens, scale):
    outs, s = [], 0
    G = q.shape[1] // k.shape[1]
    for n in lens:
        qs = q[s:s + n].float().transpose(0, 1)
        ks = k[s:s + n].float().repeat_interleave(G, 1).transpose(0, 1)
        vs = v[s:s + n].float().repeat_interleave(G, 1).transpose(0, 1)
        sc = (qs @ ks.transpose(1, 2)) * scale
        sc = sc.masked_fill(~torch.ones(n, n, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        outs.append((sc.softmax(-1) @ vs).transpose(0, 1))
        s += n
    return torch.cat(outs, 0)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 2, 64), (32, 8, 128), (16, 2, 128)])
def test_attention_packed_vs_fp32_and_cpu_oracle(Hq, Hkv, D):
    torch.manual_seed(4)
    lens = [300, 17, 129, 128]
    T = sum(lens)
    q, k, v = (torch.randn(T, h, D, device=DEV).bfloat16() for h in (Hq, Hkv, Hkv))
    scale = 1 / math.sqrt(D)
    out, lse = F.attention_fwd(q, k, v, F.AttnMeta.packed(lens, Hq, Hkv, DEV), scale, want_lse=True)
    ref = _attn_ref(q, k, v, lens, scale)
    assert (out.float() - ref).abs().max() < 2e-2
    oc, lc = F.attention_fwd(q.cpu(), k.cpu(), v.cpu(), F.AttnMeta.packed(lens, Hq, Hkv, "cpu"), scale, want_lse=True)
    assert (out.cpu().float() - oc.float()).abs().max() < 2e-2 and (lse.cpu() - lc).abs().max() < 1e-3


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 2, 64), (32, 8, 128), (4, 4, 128)])
def test_attention_backward_kernels_match_fp32_autograd(Hq, Hkv, D):
    """dQ, dK, dV of the tcgen05 backward against autograd through the fp32 reference on the same bf16 inputs:
    ragged sequences (tiles that straddle a sequence end, a block with few keys), and determinism."""
    torch.manual_seed(14)
    lens = [300, 17, 129, 128, 513]
    T = sum(lens)
    q, k, v = (torch.randn(T, h, D, device=DEV).bfloat16().requires_grad_(True) for h in (Hq, Hkv, Hkv))
    dout = torch.randn(T, Hq, D, device=DEV).bfloat16()
    scale = 1 / math.sqrt(D)
    meta = F.AttnMeta.packed(lens, Hq, Hkv, DEV)
    out = F.attention(q, k, v, meta, scale)
    got = torch.autograd.grad(out, (q, k, v), dout)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = torch.autograd.grad(_attn_ref(qf, kf, vf, lens, scale), (qf, kf, vf), dout.float())
    for name, g, r in zip("qkv", got, ref):
        assert g.dtype == torch.bfloat16 and g.shape == r.shape
        err = (g.float() - r).abs().max().item()
        assert err < 2.5e-2 * max(1.0, r.abs().max().item()), (name, err, r.abs().max().item())
    again = torch.autograd.grad(F.attention(q, k, v, meta, scale), (q, k, v), dout)
    assert all(bitwise_equal(a, b) for a, b in zip(got, again))


@pytest.mark.parametrize("n", [8 * 1000, 8 * 1000 + 3, 1 << 22])
def test_gradient_accumulation_kernel_bf16_into_fp32(n):
    from skyrl_isoexec_b200.ops import _native

    torch.manual_seed(21)
    g = torch.randn(n, device=DEV).bfloat16()
    acc = torch.randn(n, device=DEV)
    want = acc + g.float()
    L = _native.lib()
    _native.check(L.ix_accum_bf16_to_f32(acc.data_ptr(), g.data_ptr(), n, 1, _native.stream()), "accum")
    assert bitwise_equal(acc, want)
    _native.check(L.ix_accum_bf16_to_f32(acc.data_ptr(), g.data_ptr(), n, 0, _native.stream()), "accum")
    assert bitwise_equal(acc, g.float())


def test_qk_norm_rope_many_tokens_path_equals_few_tokens_path_bitwise():
    """Above 1024 tokens a warp walks several heads of its token (per-token constants fetched once); a token's bits
    must not depend on which path ran."""
    torch.manual_seed(31)
    Hq, Hkv, D, T = 32, 8, 128, 1500
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    qw, kw = torch.randn(D, device=DEV).bfloat16(), torch.randn(D, device=DEV).bfloat16()
    pos = torch.randint(0, 1000, (T,), dtype=torch.int32, device=DEV)
    rope = F.RopeTable(D, 1024, 1e6, DEV)
    mk = lambda: (torch.zeros(T, Hkv, D, dtype=torch.bfloat16, device=DEV), torch.zeros(T, Hkv, D, dtype=torch.bfloat16, device=DEV))
    k1, v1 = mk()
    q1 = F.qk_norm_rope_fwd(qkv, pos, None, rope, qw, kw, k1, v1, Hq, Hkv, D, 1e-6)
    k2, v2 = mk()
    q2 = torch.empty_like(q1)
    for lo in range(0, T, 700):
        hi = min(T, lo + 700)
        slots = torch.arange(lo, hi, device=DEV, dtype=torch.int64)
        q2[lo:hi] = F.qk_norm_rope_fwd(qkv[lo:hi], pos[lo:hi], slots, rope, qw, kw, k2, v2, Hq, Hkv, D, 1e-6)
    assert bitwise_equal(q1, q2) and bitwise_equal(k1, k2) and bitwise_equal(v1, v2)


def test_descriptor_driven_push_copy_kernel_copies_and_casts_on_one_gpu():
    """The kernel behind the peer weight push, run on local memory: several ranges in one launch, bf16 -> bf16 byte
    equality and fp32 -> bf16 round-to-nearest, ragged tail included."""
    import ctypes as C
    import struct

    from skyrl_isoexec_b200.ops import _native

    torch.manual_seed(17)
    sizes = [4096, 8 * 1000 + 5, 128, 1 << 20]
    src_bf = [torch.randn(n, device=DEV).bfloat16() for n in sizes]
    src_f32 = [torch.randn(n, device=DEV) for n in sizes]
    dst_a = [torch.zeros(n, device=DEV, dtype=torch.bfloat16) for n in sizes]
    dst_b = [torch.zeros(n, device=DEV, dtype=torch.bfloat16) for n in sizes]
    recs = [struct.pack("<QQqii", s.data_ptr(), d.data_ptr(), s.numel(), 0, 0) for s, d in zip(src_bf, dst_a)]
    recs += [struct.pack("<QQqii", s.data_ptr(), d.data_ptr(), s.numel(), 1, 0) for s, d in zip(src_f32, dst_b)]
    descs = torch.frombuffer(bytearray(b"".join(recs)), dtype=torch.uint8).to(DEV)
    lib = _native.lib()
    lib.ix_push_copy.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    _native.check(lib.ix_push_copy(descs.data_ptr(), len(recs), _native.stream()), "ix_push_copy")
    torch.cuda.synchronize()
    for s_, d in zip(src_bf, dst_a):
        assert bitwise_equal(s_, d)
    for s_, d in zip(src_f32, dst_b):
        assert bitwise_equal(s_.bfloat16(), d)


def test_attention_decode_and_chunk_equal_prefill_bitwise_paged():
    torch.manual_seed(5)
    Hq, Hkv, D, S = 32, 8, 128, 700
    q, k, v = (torch.randn(S, h, D, device=DEV).bfloat16() for h in (Hq, Hkv, Hkv))
    scale = 1 / math.sqrt(D)
    full, _ = F.attention_fwd(q, k, v, F.AttnMeta.packed([S], Hq, Hkv, DEV), scale)
    nblk = (S + 127) // 128
    perm = torch.randperm(nblk + 4)[:nblk]
    kc = torch.zeros((nblk + 4) * 128, Hkv, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for b, p in enumerate(perm.tolist()):
        lo, hi = b * 128, min(S, b * 128 + 128)
        kc[p * 128:p * 128 + hi - lo], vc[p * 128:p * 128 + hi - lo] = k[lo:hi], v[lo:hi]
    bt = perm.to(torch.int32).view(1, -1).to(DEV)
    for t in (0, 127, 128, 511, S - 1):                       # single-token decode at several positions
        items = torch.tensor([[0, 1, t, t + 1, 0, 0, 0, 0]], dtype=torch.int32, device=DEV)
        o, _ = F.attention_fwd(q[t:t + 1].contiguous(), kc, vc, F.AttnMeta(items, bt), scale)
        assert bitwise_equal(o[0], full[t])
    items = torch.tensor([[0, 32, S - 45, S - 13, 0, 0, 0, 0], [32, 13, S - 13, S, 0, 0, 0, 0]], dtype=torch.int32, device=DEV)
    o, _ = F.attention_fwd(q[S - 45:].contiguous(), kc, vc, F.AttnMeta(items, bt), scale)   # chunked prefill
    assert bitwise_equal(o, full[S - 45:])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_logprobs_vs_fp32_cpu_oracle_and_row_invariance(dtype):
    torch.manual_seed(6)
    V = 151936
    logits = (torch.randn(9, V, device=DEV) * 3).to(dtype)
    tg = torch.randint(0, V, (9,), device=DEV)
    lp, lse, ent = F.logprob_fused_fwd(logits, tg, 8, want_entropy=True)
    ref = torch.log_softmax(logits.float(), -1)
    assert (lp - ref.gather(1, tg[:, None])[:, 0]).abs().max() < 3e-6
    assert (ent - (-(ref.exp() * ref).sum(-1))).abs().max() < 1e-3
    lp1, _, _ = F.logprob_fused_fwd(logits[4:5].contiguous(), tg[4:5], 8)
    assert bitwise_equal(lp1, lp[4:5])
    lpc, lsec, _ = F.logprob_fused_fwd(logits.cpu(), tg.cpu(), 8)
    assert (lp.cpu() - lpc).abs().max() < 2e-6 and (lse.cpu() - lsec).abs().max() < 2e-6


def test_logprob_staged_equals_fused_bitwise():
    """TP path: row max / leaf sums / finalize over two vocabulary shards == the fused kernel."""
    torch.manual_seed(7)
    V, G, rows = 4096, 8, 11
    logits = (torch.randn(rows, V, device=DEV) * 2).bfloat16()
    tg = torch.randint(0, V, (rows,), device=DEV)
    lp, lse, _ = F.logprob_fused_fwd(logits, tg, G)
    L = _native.lib()
    s = _native.stream()
    mx = torch.empty(2, rows, device=DEV)
    leaf = torch.empty(rows, G, device=DEV)
    tl = torch.zeros(2, rows, device=DEV)
    half = V // 2
    shards = [logits[:, :half].contiguous(), logits[:, half:].contiguous()]
    for r, sh in enumerate(shards):
        _native.check(L.ix_logprob_rowmax(sh.data_ptr(), half, rows, half, mx[r].data_ptr(), 0, s), "rowmax")
    m = torch.maximum(mx[0], mx[1])
    for r, sh in enumerate(shards):
        _native.check(L.ix_logprob_leafsum(sh.data_ptr(), half, rows, half, G // 2, G, r * (G // 2), m.data_ptr(),
                                           leaf.data_ptr(), None, 0, s), "leafsum")
        _native.check(L.ix_logprob_gather_target(sh.data_ptr(), half, rows, half, r * half, tg.data_ptr(), tl[r].data_ptr(), 0, s), "gather")
    t_logit = tl[0] + tl[1]
    lp2, lse2 = torch.empty(rows, device=DEV), torch.empty(rows, device=DEV)
    _native.check(L.ix_logprob_finalize(leaf.data_ptr(), None, m.data_ptr(), t_logit.data_ptr(), tg.data_ptr(), lp2.data_ptr(),
                                        lse2.data_ptr(), None, rows, G, s), "finalize")
    assert bitwise_equal(lp2, lp) and bitwise_equal(lse2, lse)


def test_logprob_backward_matches_autograd():
    torch.manual_seed(8)
    V = 4096
    logits = (torch.randn(7, V, device=DEV) * 2).bfloat16().requires_grad_()
    tg = torch.randint(0, V, (7,), device=DEV)
    lp, ent = F.token_logprobs(logits, tg, 8, want_entropy=True)
    w = torch.arange(1, 8.0, device=DEV)
    ((lp * w).sum() + 0.3 * ent.sum()).backward()
    l2 = logits.detach().float().requires_grad_()
    ls = torch.log_softmax(l2, -1)
    ((ls.gather(1, tg[:, None])[:, 0] * w).sum() + 0.3 * (-(ls.exp() * ls).sum(-1)).sum()).backward()
    assert (logits.grad.float() - l2.grad).abs().max() < 2e-2


def test_swiglu_and_reduce_and_adamw():
    torch.manual_seed(9)
    x = torch.randn(33, 512, device=DEV).bfloat16()
    y = F.swiglu_fwd(x)
    ref = torch.nn.functional.silu(x[:, :256].float()).bfloat16().float() * x[:, 256:].float()
    assert (y.float() - ref).abs().max() < 2e-2
    yc = F.swiglu_fwd(x.cpu())
    assert count_bit_mismatches(y.cpu(), yc) <= 0.001 * y.numel()          # expf implementations may differ in the last ulp
    g = torch.randn(100003, device=DEV)
    a = F.reduce_sum_fixed(g, square=True)
    assert bitwise_equal(a.cpu(), F.reduce_sum_fixed(g.cpu(), square=True))
    assert abs(a.item() - g.double().pow(2).sum().item()) < 1e-1


def test_ppo_loss_kernel_matches_torch():
    from skyrl_isoexec_b200.train import algorithms as alg

    torch.manual_seed(10)
    cfg = alg.AlgorithmConfig()
    lp = (torch.randn(6, 40) * 0.3 - 2).requires_grad_()
    old = lp.detach() + torch.randn(6, 40) * 0.2
    adv, mask = torch.randn(6, 40), (torch.rand(6, 40) > 0.2).float()
    for name in ("regular", "dual_clip"):
        fn = alg.get_policy_loss(name)
        l_cpu, m_cpu = fn(lp, old, adv, cfg, loss_mask=mask)
        (g_cpu,) = torch.autograd.grad(l_cpu, lp)
        lpg = lp.detach().to(DEV).requires_grad_()
        l_gpu, m_gpu = fn(lpg, old.to(DEV), adv.to(DEV), cfg, loss_mask=mask.to(DEV))
        (g_gpu,) = torch.autograd.grad(l_gpu, lpg)
        assert abs(l_cpu.item() - l_gpu.item()) < 1e-3 * max(1.0, abs(l_cpu.item()))
        assert (g_cpu - g_gpu.cpu()).abs().max() < 1e-4
        assert abs(float(m_cpu["clip_ratio"]) - float(m_gpu["clip_ratio"])) < 1e-6


def test_engine_and_trainer_logprobs_bitwise_on_gpu_and_step():
    """The flagship claim on the GPU: rollout logprobs == trainer scoring logprobs, bit for bit,
    with chunked prefill and a batch mix that changes every step; then one optimizer step and again."""
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config("tiny-qwen3-bf16")
    model = DecoderLM(cfg, device=DEV, seed=0)
    eng = LLMEngine(model, EngineConfig(max_num_seqs=16, num_kv_pages=64, max_num_batched_tokens=96))
    worker = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=700))
    worker.cfg.optimizer.lr = 1e-3
    g = torch.Generator().manual_seed(0)
    for _round in range(2):
        prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in torch.randint(20, 200, (10,), generator=g)]
        outs = eng.generate(prompts, SamplingParams(max_generate_length=40, ignore_eos=True))
        seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.randn_like(rmask) / rmask.sum()})
        lp = worker.forward(batch)
        ro = torch.zeros_like(lp)
        for i, o in enumerate(outs):
            ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
        assert count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous()) == 0
        batch["action_log_probs"] = lp
        worker.forward_backward(batch)
        assert worker.optim_step() > 0


def test_run_ahead_decode_with_stops_and_mixed_lengths_stays_bitwise():
    """Graph decode runs one step ahead of the host. Sequences stop at different times (stop tokens, different
    length limits), so surplus tokens are computed and dropped and the batch keeps changing: what is reported must
    still be exactly the tokens up to the stop, and their logprobs must equal a clean scoring pass bit for bit."""
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config("tiny-qwen3-bf16")
    model = DecoderLM(cfg, device=DEV, seed=3)
    eng = LLMEngine(model, EngineConfig(max_num_seqs=12, num_kv_pages=64, max_num_batched_tokens=256, seed=5))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in torch.randint(5, 120, (12,), generator=g)]
    stops = tuple(range(0, cfg.vocab_size, 16))                       # one token in 16 ends a sequence
    params = [SamplingParams(max_generate_length=20 + 9 * i, stop_token_ids=stops if i % 3 else ()) for i in range(12)]
    outs = eng.generate(prompts, params)
    assert eng.stats["steps"] > 0 and not eng.scheduler.has_work() and eng._inflight is None
    assert eng.cache.allocator.num_free == 64
    n_stop = 0
    for o, p in zip(outs, params):
        assert len(o.response_ids) == len(o.response_logprobs) and 1 <= len(o.response_ids) <= p.max_generate_length
        body = o.response_ids[:-1]
        assert not any(t in stops for t in body) or not p.stop_token_ids        # nothing after a stop token
        if o.stop_reason == "stop":
            assert o.response_ids[-1] in stops
            n_stop += 1
        else:
            assert len(o.response_ids) == p.max_generate_length
    assert n_stop >= 3
    seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
    lp = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=600)).forward(
        TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask}))
    ro = torch.zeros_like(lp)
    for i, o in enumerate(outs):
        ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
    assert count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous()) == 0


def test_router_topk_matches_cpu_oracle_and_tie_rule():
    from skyrl_isoexec_b200.ops import moe

    torch.manual_seed(11)
    for E, k in ((128, 8), (8, 2), (256, 8)):
        lg = torch.randn(37, E)
        lg[0, 3] = lg[0, 5] = 9.0                        # exact tie at the top: the lower index must win
        ic, wc, pc = moe.router_topk_fwd(lg, k, None, False, True, want_probs=True)
        ig, wg, pg = moe.router_topk_fwd(lg.to(DEV), k, None, False, True, want_probs=True)
        assert ic[0, 0] == 3 and ic[0, 1] == 5
        assert torch.equal(ig.cpu(), ic)
        assert (wg.cpu() - wc).abs().max() < 1e-6 and (pg.cpu() - torch.softmax(lg, -1)).abs().max() < 1e-6
        one = moe.router_topk_fwd(lg[5:6].to(DEV).contiguous(), k, None, False, True)
        assert torch.equal(one[0], ig[5:6]) and bitwise_equal(one[1], wg[5:6])   # a token's routing ignores the batch


@pytest.mark.parametrize("name", ["tiny-moe", "tiny-hybrid"])
def test_moe_and_hybrid_engine_and_trainer_logprobs_bitwise_on_gpu(name):
    from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
    from skyrl_isoexec_b200.engine.sampler import SamplingParams
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.models.decoder import DecoderLM
    from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
    from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

    cfg = get_config(name, dtype="bfloat16")
    model = DecoderLM(cfg, device=DEV, seed=0)
    eng = LLMEngine(model, EngineConfig(max_num_seqs=16, num_kv_pages=64, max_num_batched_tokens=80))
    worker = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=300))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in torch.randint(20, 150, (8,), generator=g)]
    outs = eng.generate(prompts, SamplingParams(max_generate_length=24, ignore_eos=True))
    seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
    batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                "advantages": torch.randn_like(rmask) / rmask.sum()})
    lp = worker.forward(batch)
    ro = torch.tensor([o.response_logprobs for o in outs])
    assert count_bit_mismatches(lp.contiguous(), ro.contiguous()) == 0
    batch["action_log_probs"] = lp
    worker.forward_backward(batch)
    assert worker.optim_step() > 0


def test_gdn_scan_bitwise_vs_cpu_oracle_chunked_equals_recurrent():
    """The scan over a whole sequence equals the same sequence fed as chunks through the state pool
    (bitwise, on the GPU), and agrees with the C++ oracle wherever exp() agrees."""
    from skyrl_isoexec_b200.models.config import get_config
    from skyrl_isoexec_b200.ops import gdn

    torch.manual_seed(12)
    cfg = get_config("tiny-hybrid", dtype="bfloat16")
    hk, hv, d = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
    C = (2 * hk + hv) * d
    T = 200
    proj = (torch.randn(T, C + hv * d + 2 * hv) * 0.5).bfloat16()
    conv_w, A_log, dtb = (torch.randn(C, 4) * 0.3).bfloat16(), (torch.randn(hv) * 0.1).bfloat16(), (torch.randn(hv) * 0.1).bfloat16()
    whole = gdn.gdn_core_fwd(proj.to(DEV), conv_w.to(DEV), A_log.to(DEV), dtb.to(DEV), gdn.GDNMeta.packed([T], DEV), cfg, 1)
    cpu = gdn.gdn_core_fwd(proj, conv_w, A_log, dtb, gdn.GDNMeta.packed([T], "cpu"), cfg, 1)
    assert (whole.cpu().float() - cpu.float()).abs().max() < 2e-2 * max(1.0, cpu.float().abs().max().item())
    conv_state = torch.zeros(3, C, 3, dtype=torch.bfloat16, device=DEV)
    ssm = torch.zeros(3, hv, d, d, dtype=torch.float32, device=DEV)
    open_chunk = gdn.new_chunk_buffers(3, hk, hv, d, torch.bfloat16, DEV)      # tokens since the last chunk boundary, per state row
    outs, pos = [], 0
    for n in (70, 1, 1, 64, 1, 63):                       # prefill chunk, decode steps, more chunks
        meta = gdn.GDNMeta.build([(0, n, pos, 2 if pos > 0 else -1, 2)], DEV)
        outs.append(gdn.gdn_core_fwd(proj[pos:pos + n].to(DEV).contiguous(), conv_w.to(DEV), A_log.to(DEV), dtb.to(DEV), meta, cfg, 1,
                                     conv_state, ssm, open_chunk))
        pos += n
    assert bitwise_equal(torch.cat(outs, 0), whole)


def test_fused_gumbel_sampler_distribution_greedy_and_determinism():
    from skyrl_isoexec_b200.engine.sampler import Sampler, SamplingParams

    torch.manual_seed(0)
    V, n = 1000, 8192
    base = torch.full((V,), -30.0)
    hot = torch.tensor([5, 400, 998, 999])
    base[hot] = torch.tensor([2.0, 1.0, 0.0, 1.5])
    ld = 1008
    buf = torch.zeros(n, ld, device=DEV, dtype=torch.bfloat16)
    buf[:, :V] = base.to(DEV).bfloat16()
    logits = buf[:, :V]
    sm = Sampler(DEV, seed=11)
    toks, lps = sm(logits, [SamplingParams()] * n)
    p = torch.softmax(base.bfloat16().float(), -1)
    freq = torch.bincount(toks.cpu(), minlength=V).float() / n
    assert (freq[hot] - p[hot]).abs().max() < 0.02 and freq[hot].sum() > 0.999
    assert torch.allclose(lps.cpu(), torch.log_softmax(base.bfloat16().float(), -1)[toks.cpu()], atol=1e-4)
    # same seed and call counter -> same draws; the next call differs
    sm2 = Sampler(DEV, seed=11)
    toks2, _ = sm2(logits, [SamplingParams()] * n)
    toks3, _ = sm2(logits, [SamplingParams()] * n)
    assert torch.equal(toks, toks2) and not torch.equal(toks2, toks3)
    # rows are independent of the batch they sit in
    t_small, _ = Sampler(DEV, seed=11)(logits[:7], [SamplingParams()] * 7)
    assert torch.equal(t_small, toks[:7])
    # greedy rows (temperature 0) take the argmax, lower index on ties; temperature sharpens
    tie = buf.clone()
    tie[:, 7] = tie[:, 5]
    g, _ = Sampler(DEV, seed=1)(tie[:4, :V], [SamplingParams(temperature=0.0)] * 4)
    assert g.tolist() == [5, 5, 5, 5]
    cold, _ = Sampler(DEV, seed=3)(logits, [SamplingParams(temperature=0.25)] * n)
    assert (cold == 5).float().mean() > 0.85


def test_moe_dispatch_plan_is_the_stable_counting_sort():
    """The device-built routing tables equal the torch sort / bincount construction; with padding every expert's group
    starts on a multiple of 64 rows and the padding rows are marked empty."""
    from skyrl_isoexec_b200.ops import moe

    g = torch.Generator().manual_seed(5)
    for T, E, k in ((1, 8, 2), (333, 8, 2), (4096, 128, 8), (77, 16, 4)):
        idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int().to(DEV)
        order, counts, pos = moe.build_dispatch(idx, E)
        plan = moe.DispatchPlan(idx, E, 1)
        assert torch.equal(plan.src_of_row[:T * k].long(), order) and torch.equal(plan.pos, pos)
        assert torch.equal(plan.offs.long(), moe.counts_to_offsets(counts).long())
        pp = moe.DispatchPlan(idx, E, 64)
        offs = pp.offs.tolist()
        assert all(o % 64 == 0 for o in offs) and offs[-1] <= pp.r_cap
        src = pp.src_of_row.tolist()
        cl = counts.tolist()
        for e in range(E):
            seg = src[offs[e]:offs[e + 1]]
            assert seg[:cl[e]] == order[sum(cl[:e]):sum(cl[:e + 1])].tolist() and all(v == -1 for v in seg[cl[e]:])
        y = torch.randn(T, 64, device=DEV).bfloat16()
        w = torch.rand(T * k, device=DEV)
        xr, wr = pp.gather(y, w)
        for e in (0, E - 1):
            n = cl[e]
            rows = order[sum(cl[:e]):sum(cl[:e]) + n]
            assert torch.equal(xr[offs[e]:offs[e] + n], y[rows // k]) and torch.equal(wr[offs[e]:offs[e] + n], w[rows])
            assert not xr[offs[e] + n:offs[e + 1]].any() and not wr[offs[e] + n:offs[e + 1]].any()


def test_moe_experts_autograd_function_matches_fp32_autograd_and_the_fused_forward():
    """One MoE layer's experts as grouped kernels with a kernel VJP: the forward has the bits of the fused inference
    path, the gradients of input, gate weights and both expert weights agree with fp32 autograd of the same math."""
    from skyrl_isoexec_b200.ops import moe

    torch.manual_seed(7)
    T, E, k, H, Fd = 500, 8, 2, 256, 128
    y = (torch.randn(T, H, device=DEV) * 0.5).bfloat16().requires_grad_()
    gate_up = (torch.randn(E, 2 * Fd, H, device=DEV) * 0.05).bfloat16().requires_grad_()
    down = (torch.randn(E, H, Fd, device=DEV) * 0.05).bfloat16().requires_grad_()
    logits = torch.randn(T, E, device=DEV)
    idx, w0, _ = moe.router_topk_fwd(logits, k, None, False, True)
    w = w0.clone().requires_grad_()
    gout = (torch.randn(T, H, device=DEV) * 0.1).bfloat16()
    out = moe._ExpertsFn.apply(y, w, gate_up, down, idx, None)
    out.backward(gout)
    # forward bits: the inference path (fused GLU epilogue, unpadded plan)
    with torch.no_grad():
        plan = moe.DispatchPlan(idx, E, 1)
        xr, wr = plan.gather(y.detach(), w0.reshape(-1).contiguous())
        rows = moe.expert_rows_grouped(xr, wr, plan.offs, gate_up.detach(), down.detach())
        assert bitwise_equal(moe.combine_fixed_order(rows, plan.pos, torch.bfloat16), out.detach())
    # fp32 reference of the same function
    yf, wf = y.detach().float().requires_grad_(), w0.clone().requires_grad_()
    guf, df = gate_up.detach().float().requires_grad_(), down.detach().float().requires_grad_()
    ref = torch.zeros(T, H, device=DEV)
    for e in range(E):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = yf[tok] @ guf[e].T
        a = torch.nn.functional.silu(h[:, :Fd]) * h[:, Fd:] * wf[tok, slot][:, None]
        ref = ref.index_add(0, tok, a @ df[e].T)
    ref.backward(gout.float())
    rel = lambda a, b: float((a.float() - b).abs().max() / b.abs().max().clamp(min=1e-6))
    assert rel(out.detach(), ref.detach()) < 2e-2
    assert rel(y.grad, yf.grad) < 3e-2 and rel(w.grad, wf.grad) < 3e-2
    assert rel(gate_up.grad, guf.grad) < 3e-2 and rel(down.grad, df.grad) < 3e-2
    # an expert that received no token gets an exactly zero gradient
    empty = [e for e in range(E) if not bool((idx == e).any())]
    for e in empty:
        assert not gate_up.grad[e].any() and not down.grad[e].any()


def test_moe_experts_raw_form_equals_the_rows_of_the_combined_form():
    """The form an expert-parallel owner runs (one expert per received row, fp32 rows returned unrounded): summing its
    rows in the source's fixed order gives the bits of the single-rank experts function, and its gradients agree."""
    from skyrl_isoexec_b200.ops import moe

    torch.manual_seed(9)
    T, E, k, H, Fd = 300, 8, 2, 256, 128
    y0 = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    gu0 = (torch.randn(E, 2 * Fd, H, device=DEV) * 0.05).bfloat16()
    dn0 = (torch.randn(E, H, Fd, device=DEV) * 0.05).bfloat16()
    idx, w0, _ = moe.router_topk_fwd(torch.randn(T, E, device=DEV), k, None, False, True)
    gout = (torch.randn(T, H, device=DEV) * 0.1).bfloat16()
    y, w, gu, dn = y0.clone().requires_grad_(), w0.clone().requires_grad_(), gu0.clone().requires_grad_(), dn0.clone().requires_grad_()
    moe._ExpertsFn.apply(y, w, gu, dn, idx, None).backward(gout)
    want = moe._ExpertsFn.apply(y0, w0, gu0, dn0, idx, None)
    # the same work as an owner sees it: T*k rows in (token, slot) order, each naming its expert
    y2, w2, gu2, dn2 = y0.clone().requires_grad_(), w0.clone().requires_grad_(), gu0.clone().requires_grad_(), dn0.clone().requires_grad_()
    rows_in = y2.repeat_interleave(k, 0)
    raw = moe._ExpertsFn.apply(rows_in, w2.reshape(-1, 1), gu2, dn2, idx.reshape(-1, 1).contiguous(), None, True)
    assert raw.dtype == torch.float32 and raw.shape == (T * k, H)
    pos = torch.arange(T * k, device=DEV).view(T, k)
    got = moe.combine_fixed_order(raw, pos, torch.bfloat16)
    assert bitwise_equal(got.detach(), want)
    got.backward(gout)
    rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6))
    assert rel(gu2.grad, gu.grad) < 1e-2 and rel(dn2.grad, dn.grad) < 1e-2
    assert rel(y2.grad, y.grad) < 2e-2 and rel(w2.grad, w.grad) < 2e-2


def test_every_fused_region_equals_its_unfused_chain_on_hazard_inputs():
    """The fusion ledger's checkers on the GPU: everything except the multi-GPU kernels is decided here."""
    from skyrl_isoexec_b200.core import fusion_ledger as FL

    res = FL.run_checkers(DEV)
    multi = {"tp_gemm_fused (AR1/AR2/RS)", "tp_gemm_fused (AG)"}
    assert all(res[n] is True for n in res if n not in multi), res
    assert all(res[n] is not False for n in multi)


def _gdn_recurrence_fp32(q, k, v, g, beta):
    """Token-by-token gated delta rule in fp32: q, k [T, Hk, D], v [T, Hv, D], g, beta [T, Hv] -> o [T, Hv, D]."""
    T, Hk, D = q.shape
    Hv = v.shape[1]
    rep = Hv // Hk
    qf, kf = q.float().repeat_interleave(rep, 1), k.float().repeat_interleave(rep, 1)
    S = torch.zeros(Hv, D, D, device=q.device)                   # [Hv, Dv, Dk]
    out = torch.empty(T, Hv, D, device=q.device)
    for t in range(T):
        S = S * g[t].exp()[:, None, None]
        kv = torch.einsum("hvk,hk->hv", S, kf[t])
        d = (v[t].float() - kv) * beta[t][:, None]
        S = S + d[:, :, None] * kf[t][:, None, :]
        out[t] = torch.einsum("hvk,hk->hv", S, qf[t])
    return out


@pytest.mark.parametrize("D", [64, 128])
def test_gdn_chunked_tensor_core_scan_matches_the_fp32_recurrence_and_decode_is_bitwise(D):
    """The chunked tcgen05 form of the gated delta rule: close to the fp32 token recurrence, and bit-identical whether a
    sequence is scanned whole, or as a prefill piece, single decode tokens and further pieces that each re-run the open
    chunk from the state at the last chunk boundary."""
    from skyrl_isoexec_b200.ops import gdn

    torch.manual_seed(21)
    T, Hk, Hv = 300, 2, 4
    q = torch.nn.functional.normalize(torch.randn(T, Hk, D, device=DEV), dim=-1) * D ** -0.5
    k = torch.nn.functional.normalize(torch.randn(T, Hk, D, device=DEV), dim=-1)
    v = torch.randn(T, Hv, D, device=DEV) * 0.5
    g = -torch.rand(T, Hv, device=DEV) * 0.2
    beta = torch.rand(T, Hv, device=DEV)
    qb, kb, vb = q.bfloat16().contiguous(), k.bfloat16().contiguous(), v.bfloat16().contiguous()
    whole = gdn.gdn_chunk_scan(qb, kb, vb, g, beta, [(0, T, -1, -1)])
    ref = _gdn_recurrence_fp32(qb, kb, vb, g, beta)
    err = (whole.float() - ref).abs().max().item()
    assert err < 3e-2 * max(1.0, ref.abs().max().item()), err
    # two sequences packed back to back give the rows of each scanned alone
    both = gdn.gdn_chunk_scan(qb, kb, vb, g, beta, [(0, 130, -1, -1), (130, T - 130, -1, -1)])
    assert bitwise_equal(both[:130], whole[:130])
    alone = gdn.gdn_chunk_scan(qb[130:].contiguous(), kb[130:].contiguous(), vb[130:].contiguous(), g[130:].contiguous(),
                               beta[130:].contiguous(), [(0, T - 130, -1, -1)])
    assert bitwise_equal(both[130:], alone)
    # engine-style walk: every call re-runs the open chunk from the state at the last boundary (row 1 of a pool)
    state = torch.zeros(2, Hv, D, D, device=DEV)
    outs, pos, have_state = [], 0, False
    for n in (70, 1, 1, 57, 1, 100, 1, T - 231):
        c0 = pos // 64 * 64                                   # the open chunk starts here
        sl = slice(c0, pos + n)
        o = gdn.gdn_chunk_scan(qb[sl].contiguous(), kb[sl].contiguous(), vb[sl].contiguous(), g[sl].contiguous(), beta[sl].contiguous(),
                               [(0, pos + n - c0, 1 if have_state else -1, 1)], state)
        outs.append(o[pos - c0:])
        pos += n
        have_state = pos >= 64
    assert pos == T and bitwise_equal(torch.cat(outs, 0), whole)


@pytest.mark.parametrize("D,zc", [(64, True), (128, True), (128, False), (256, True)])
def test_gated_outnorm_matches_the_cpu_oracle_and_the_formula(D, zc):
    """rms_norm(o) * gamma * silu(z) per (token, head) row. Rows of up to 128 elements are handled two per warp; the result
    must equal the C++ restatement (same roundings; only exp() may differ in its last bit) and the fp32 formula."""
    torch.manual_seed(5)
    rows = 777
    o = torch.randn(rows, D).bfloat16()
    z = torch.randn(rows, D).bfloat16()
    w = (torch.randn(D) * 0.1).bfloat16()
    cpu = F.gated_outnorm(o, z, w, 1e-6, zc)
    gpu = F.gated_outnorm(o.to(DEV), z.to(DEV), w.to(DEV), 1e-6, zc).cpu()
    diff = (gpu.float() - cpu.float()).abs()
    assert float((diff > 0).float().mean()) < 0.02                      # exp() rounding only
    assert float((diff / cpu.float().abs().clamp(min=1e-3)).max()) < 2e-2
    of, zf = o.float(), z.float()
    ref = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + 1e-6) * ((1 + w.float()) if zc else w.float()) * torch.nn.functional.silu(zf)
    assert float((gpu.float() - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max()))
    # a row's bits do not depend on how many rows the launch has (odd counts leave half a warp idle)
    one = F.gated_outnorm(o[:1].to(DEV), z[:1].to(DEV), w.to(DEV), 1e-6, zc).cpu()
    assert bitwise_equal(one, gpu[:1])


def test_gemm_admission_on_the_model_census_and_its_negative_control(monkeypatch):
    """Start-up admission: every GEMM shape of a model's census gives batch-independent rows (and the two leaf-tree
    forms agree); a provider whose rows depend on the batch is refused by name."""
    from skyrl_isoexec_b200.core import mm_admission
    from skyrl_isoexec_b200.models.config import get_config

    cfg = get_config("qwen3-8b", dtype="bfloat16", tp_invariant=True, pik_leaves=2, num_layers=2, vocab_size=32768)
    rep = mm_admission.admit(cfg, "cuda")
    assert rep and all(v is True for v in rep.values()), rep
    assert {"attn.qkv", "attn.o", "mlp.fc1", "mlp.fc2", "lm_head"} <= set(rep)
    assert mm_admission.refused(rep) == []
    rep2 = mm_admission.admit(cfg, "cuda", tp=2)
    assert all(v is True for v in rep2.values()), rep2
    # negative control: a "provider" that picks a different summation for small batches
    real = F.gemm_nt
    monkeypatch.setattr(F, "gemm_nt", lambda a, w, out_f32=False, **kw: real(a, w, out_f32=out_f32, **kw) if a.shape[0] > 100
                        else (a.float() @ w.float().T).to(torch.float32 if out_f32 else torch.bfloat16))
    mm_admission._REPORTS.clear()
    bad = mm_admission.admit(cfg, "cuda")
    assert "mlp.fc2" in mm_admission.refused(bad) or "attn.qkv" in mm_admission.refused(bad)
    mm_admission._REPORTS.clear()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_trace_digest_kernel_equals_the_integer_torch_formulation(dtype):
    """Row digests of every ladder level from one kernel pass: the same 64-bit numbers as the CPU integer ops, so a
    trace taken on a GPU compares with one taken on a CPU; invariant to the order of the rows."""
    from skyrl_isoexec_b200.debug import thash

    torch.manual_seed(2)
    x = torch.randn(37, 5, 129).to(dtype)
    x[3, 0, 0], x[4, 1, 1] = 0.0, -0.0
    xg = x.to(DEV)
    for k in thash.LADDER:
        assert torch.equal(thash.row_digests(xg, k).cpu(), thash.row_digests(x, k)), k
    assert thash.ladder(xg) == thash.ladder(x) and thash.row_ladder(xg) == thash.row_ladder(x)
    perm = torch.randperm(37)
    assert thash.ladder(xg[perm.to(DEV)]) == thash.ladder(xg)
    y = xg.clone()
    y.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)[5, 2, 7] ^= 1      # flip the last mantissa bit of one element
    la, lb = thash.ladder(xg), thash.ladder(y)
    assert la["0"] != lb["0"] and la["1"] == lb["1"]


def test_gdn_conv_eight_channels_per_thread_equals_the_scalar_kernel_bitwise():
    """The vectorised causal conv (16-byte loads, taken when the row stride is a multiple of 8) and the scalar kernel (any
    stride) give the same bits, with taps that reach into the conv state and with a zero history."""
    from skyrl_isoexec_b200.ops import _native, gdn

    torch.manual_seed(4)
    T, C, W = 150, 256, 4
    lens = [70, 80]
    x = (torch.randn(T, C, device=DEV) * 0.7).bfloat16()
    w = (torch.randn(C, W, device=DEV) * 0.3).bfloat16()
    conv_state = (torch.randn(3, C, W - 1, device=DEV) * 0.5).bfloat16()
    # sequence 0 continues from state row 2 (its first taps read the state), sequence 1 starts from nothing
    meta = gdn.GDNMeta.build([(0, lens[0], 5, 2, 2), (lens[0], lens[1], 0, -1, 1)], DEV)
    lib = _native.lib()

    def run(xin, ldx):
        out = torch.empty(T, C, device=DEV, dtype=torch.bfloat16)
        _native.check(lib.ix_gdn_conv(xin.data_ptr(), ldx, w.data_ptr(), meta.tok_back.data_ptr(), _native.ptr(meta.state_row),
                                      conv_state.data_ptr(), out.data_ptr(), T, C, W, 0, _native.stream()), "ix_gdn_conv")
        return out

    wide = torch.zeros(T, C + 3, device=DEV, dtype=torch.bfloat16)            # row stride 259: the scalar kernel
    wide[:, :C] = x
    assert bitwise_equal(run(x, C), run(wide, C + 3))
    assert _native.read_status() == 0
