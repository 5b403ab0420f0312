"""CPU route of the op layer: invariance properties and agreement with plain PyTorch fp32."""
import math

import pytest
import torch

from skyrl_isoexec_b200.ops import functional as F

torch.manual_seed(0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_batch_invariant_and_close(dtype):
    x = torch.randn(37, 96).to(dtype)
    w = torch.randn(50, 96).to(dtype)
    full = F.gemm_nt(x, w)
    one = F.gemm_nt(x[5:6].contiguous(), w)
    assert torch.equal(full[5:6], one)  # a row's bits do not depend on the other rows
    ref = x.float() @ w.float().T
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (full.float() - ref).abs().max() < tol * ref.abs().max()


def test_linear_grad_matches_torch():
    x = torch.randn(9, 32, requires_grad=True)
    w = torch.randn(16, 32, requires_grad=True)
    y = F.linear(x, w)
    y.square().sum().backward()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    (x2 @ w2.T).square().sum().backward()
    assert torch.allclose(x.grad, x2.grad, atol=1e-4) and torch.allclose(w.grad, w2.grad, atol=1e-4)


@pytest.mark.parametrize("zero_centered", [False, True])
def test_rmsnorm_matches_formula_and_grad(zero_centered):
    x = torch.randn(11, 64, requires_grad=True)
    r = torch.randn(11, 64, requires_grad=True)
    w = torch.randn(64, requires_grad=True)
    y, res = F.rmsnorm(x, w, 1e-6, zero_centered, residual=r)
    (y.sum() + (res * 0.5).sum()).backward()
    x2, r2, w2 = (t.detach().clone().requires_grad_() for t in (x, r, w))
    h = x2 + r2
    g = (1 + w2) if zero_centered else w2
    y2 = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * g
    (y2.sum() + (h * 0.5).sum()).backward()
    assert torch.allclose(y, y2, atol=1e-5) and torch.allclose(res, h)
    for a, b in ((x, x2), (r, r2), (w, w2)):
        assert torch.allclose(a.grad, b.grad, atol=1e-4)


def _rope_ref(y, pos, rope):
    half = rope.rot_dim // 2
    c, s = rope.cos[pos.long()][:, None, :], rope.sin[pos.long()][:, None, :]
    y1, y2 = y[..., :half], y[..., half:rope.rot_dim]
    return torch.cat([y1 * c - y2 * s, y2 * c + y1 * s, y[..., rope.rot_dim:]], -1)


def test_qk_norm_rope_matches_formula_and_grad():
    T, Hq, Hkv, D = 13, 4, 2, 64
    rope = F.RopeTable(D, 128, 1e6, "cpu")
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, requires_grad=True)
    qw = torch.randn(D, requires_grad=True)
    kw = torch.randn(D, requires_grad=True)
    pos = torch.randint(0, 128, (T,), dtype=torch.int32)
    q, k, v = F.qk_norm_rope_train(qkv, pos, rope, qw, kw, Hq, Hkv, D, 1e-6)
    (q.square().sum() + k.sum() * 2 + v.sum() * 3).backward()
    a, b, c = (t.detach().clone().requires_grad_() for t in (qkv, qw, kw))
    G = Hq // Hkv  # rows are KV-group major: [G query heads | k | v] per KV head
    grp = a.view(T, Hkv, (G + 2) * D)
    xq = grp[..., :G * D].reshape(T, Hq, D)
    xk = grp[..., G * D:(G + 1) * D]
    xv = grp[..., (G + 1) * D:]
    nrm = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    q2, k2 = _rope_ref(nrm(xq, b), pos, rope), _rope_ref(nrm(xk, c), pos, rope)
    (q2.square().sum() + k2.sum() * 2 + xv.sum() * 3).backward()
    assert torch.allclose(q, q2, atol=1e-5) and torch.allclose(k, k2, atol=1e-5) and torch.equal(v, xv)
    assert torch.allclose(qkv.grad, a.grad, atol=1e-4)
    assert torch.allclose(qw.grad, b.grad, atol=1e-3) and torch.allclose(kw.grad, c.grad, atol=1e-3)


def _attn_ref(q, k, v, lens, scale):
    outs, s = [], 0
    G = q.shape[1] // k.shape[1]
    for n in lens:
        qs = q[s:s + n].transpose(0, 1)
        ks = k[s:s + n].repeat_interleave(G, 1).transpose(0, 1)
        vs = v[s:s + n].repeat_interleave(G, 1).transpose(0, 1)
        sc = (qs @ ks.transpose(1, 2)) * scale
        sc = sc.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), float("-inf"))
        outs.append((sc.softmax(-1) @ vs).transpose(0, 1))
        s += n
    return torch.cat(outs, 0)


def test_attention_packed_matches_reference_and_grad():
    Hq, Hkv, D = 4, 2, 64
    lens = [150, 37, 129]
    T = sum(lens)
    q = torch.randn(T, Hq, D, requires_grad=True)
    k = torch.randn(T, Hkv, D, requires_grad=True)
    v = torch.randn(T, Hkv, D, requires_grad=True)
    meta = F.AttnMeta.packed(lens, Hq, Hkv, "cpu")
    scale = 1 / math.sqrt(D)
    o = F.attention(q, k, v, meta, scale)
    o.square().sum().backward()
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
    o2 = _attn_ref(q2, k2, v2, lens, scale)
    o2.square().sum().backward()
    assert torch.allclose(o, o2, atol=2e-5)
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert torch.allclose(a.grad, b.grad, atol=2e-4)


def test_attention_decode_equals_prefill_bitwise_paged():
    Hq, Hkv, D, S = 4, 2, 64, 300
    q, k, v = torch.randn(S, Hq, D), torch.randn(S, Hkv, D), torch.randn(S, Hkv, D)
    scale = 1 / math.sqrt(D)
    full, _ = F.attention_fwd(q, k, v, F.AttnMeta.packed([S], Hq, Hkv, "cpu"), scale)
    pages = [4, 0, 2]
    kc, vc = torch.zeros(5 * 128, Hkv, D), torch.zeros(5 * 128, Hkv, D)
    for b, p in enumerate(pages):
        lo, hi = b * 128, min(S, b * 128 + 128)
        kc[p * 128:p * 128 + hi - lo], vc[p * 128:p * 128 + hi - lo] = k[lo:hi], v[lo:hi]
    bt = torch.tensor([pages], dtype=torch.int32)
    for t in (0, 127, 128, 299):
        items = torch.tensor([[0, 1, t, t + 1, 0, 0, 0, 0]], dtype=torch.int32)
        o, _ = F.attention_fwd(q[t:t + 1].contiguous(), kc, vc, F.AttnMeta(items, bt), scale)
        assert torch.equal(o[0], full[t])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_logprobs_close_and_row_invariant(dtype):
    V = 2048
    logits = (torch.randn(6, V) * 3).to(dtype)
    tg = torch.randint(0, V, (6,))
    lp, ent = F.token_logprobs(logits, tg, leaves=8, want_entropy=True)
    ref = torch.log_softmax(logits.float(), -1)
    assert torch.allclose(lp, ref.gather(1, tg[:, None])[:, 0], atol=2e-6)
    assert torch.allclose(ent, -(ref.exp() * ref).sum(-1), atol=1e-4)
    lp1, _ = F.token_logprobs(logits[3:4].contiguous(), tg[3:4], leaves=8)
    assert torch.equal(lp1, lp[3:4])


def test_token_logprobs_grad():
    V = 512
    logits = torch.randn(5, V, requires_grad=True)
    tg = torch.randint(0, V, (5,))
    lp, ent = F.token_logprobs(logits, tg, leaves=4, want_entropy=True)
    (lp * torch.arange(1, 6.0)).sum().add(ent.sum() * 0.3).backward()
    l2 = logits.detach().clone().requires_grad_()
    ls = torch.log_softmax(l2, -1)
    ((ls.gather(1, tg[:, None])[:, 0] * torch.arange(1, 6.0)).sum() + (-(ls.exp() * ls).sum(-1)).sum() * 0.3).backward()
    assert torch.allclose(logits.grad, l2.grad, atol=1e-5)


def test_swiglu_and_grad():
    x = torch.randn(7, 32, requires_grad=True)
    y = F.swiglu(x)
    y.sum().backward()
    x2 = x.detach().clone().requires_grad_()
    y2 = torch.nn.functional.silu(x2[:, :16]) * x2[:, 16:]
    y2.sum().backward()
    assert torch.allclose(y, y2, atol=1e-6) and torch.allclose(x.grad, x2.grad, atol=1e-5)


def test_reduce_sum_fixed_is_length_only():
    x = torch.randn(10000)
    a = F.reduce_sum_fixed(x, square=True)
    assert abs(a.item() - x.double().pow(2).sum().item()) < 1e-2
    assert torch.equal(a, F.reduce_sum_fixed(x.clone(), square=True))
