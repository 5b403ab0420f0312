"""Bitwise tests whose inputs are PROVEN to contain the hazard they claim to cover (the reference's hazard-exercised rule,
ISO/core/contracts.py:55-121): each case first asserts the hazard is present in its input population, then checks bits.
One case per hazard that a CPU implementation declares in the registry."""

import math

import torch

from skyrl_isoexec_b200.core.testing import assert_hazard_exercised, bitwise_equal
from skyrl_isoexec_b200.ops import functional as F
from skyrl_isoexec_b200.ops import moe as moe_ops
from skyrl_isoexec_b200.parallel import tp as tp_ops


def test_gemm_reads_a_strided_operand_like_a_packed_one():
    torch.manual_seed(0)
    big = torch.randn(9, 96)
    x = big[:, :64]                                      # row stride 96, 64 columns used
    assert_hazard_exercised("non_contiguous", x=x)
    w = torch.randn(24, 64)
    assert bitwise_equal(F.gemm_nt(x, w), F.gemm_nt(x.contiguous(), w))


def test_rmsnorm_keeps_subnormal_inputs_and_products():
    x = torch.full((3, 64), 1e-40)                       # subnormal in fp32: flushing them to zero would give y == 0
    x[1] = torch.linspace(-2e-39, 2e-39, 64)
    assert_hazard_exercised("subnormals", x=x)
    w = torch.ones(64)
    y, _ = F.rmsnorm(x, w, 1e-6)
    rstd = 1.0 / torch.sqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-6)
    ref = (x.double() * rstd).float()
    assert (y != 0).any() and torch.allclose(y.double(), ref.double(), rtol=1e-6, atol=1e-44)
    one = torch.cat([F.rmsnorm(x[i:i + 1].contiguous(), w, 1e-6)[0] for i in range(3)])
    assert bitwise_equal(y, one)


def test_rope_keeps_the_sign_of_zero():
    Hq, Hkv, D, T = 2, 1, 64, 5
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D)
    qkv[:, :D] = -0.0                                    # a whole query head of negative zeros
    assert_hazard_exercised("signed_zero", x=qkv)
    rope = F.RopeTable(D, 16, 1e4, "cpu")
    pos = torch.arange(T, dtype=torch.int32)
    k_out, v_out = torch.zeros(T, Hkv, D), torch.zeros(T, Hkv, D)
    q = F.qk_norm_rope_fwd(qkv, pos, None, rope, None, None, k_out, v_out, Hq, Hkv, D, 1e-6, False, False, False)
    # position 0 rotates by the identity: x*1 - y*0 with x = y = -0.0 is -0.0 - (-0.0) = +0.0 for the first half under IEEE,
    # and y*1 + x*0 = -0.0 for the second; what matters is that no NaN / non-zero appears and v passes through untouched
    assert bool((q[:, 0] == 0).all()) and bitwise_equal(v_out.view(T, -1), qkv[:, (Hq + Hkv) * D:].contiguous())
    again = F.qk_norm_rope_fwd(qkv.clone(), pos, None, rope, None, None, torch.zeros_like(k_out), torch.zeros_like(v_out),
                               Hq, Hkv, D, 1e-6, False, False, False)
    assert bitwise_equal(q, again)


def test_attention_with_a_padded_last_page_and_an_empty_batch():
    Hq, Hkv, D, S = 2, 1, 64, 130                        # 130 keys: the second 128-slot page holds 2 keys and 126 unused lanes
    q, k, v = torch.randn(S, Hq, D), torch.randn(S, Hkv, D), torch.randn(S, Hkv, D)
    scale = 1 / math.sqrt(D)
    full, _ = F.attention_fwd(q, k, v, F.AttnMeta.packed([S], Hq, Hkv, "cpu"), scale)
    kc, vc = torch.full((3 * 128, Hkv, D), float("nan")), torch.full((3 * 128, Hkv, D), float("nan"))
    kc[256:384], vc[256:384] = k[:128], v[:128]
    kc[0:2], vc[0:2] = k[128:], v[128:]
    assert_hazard_exercised("null_lanes", x=kc, has_padding=bool(torch.isnan(kc[2:128]).all()))
    bt = torch.tensor([[2, 0]], dtype=torch.int32)
    items = torch.tensor([[0, 1, S - 1, S, 0, 0, 0, 0]], dtype=torch.int32)
    o, _ = F.attention_fwd(q[S - 1:].contiguous(), kc, vc, F.AttnMeta(items, bt), scale)
    assert bitwise_equal(o[0], full[S - 1]), "the unused lanes of the last page (NaN here) never reach the softmax"
    assert_hazard_exercised("t_zero", x=None, num_tokens=0)
    empty, _ = F.attention_fwd(torch.zeros(0, Hq, D), k, v, F.AttnMeta.packed([], Hq, Hkv, "cpu"), scale)
    assert empty.shape == (0, Hq, D)


def test_logprobs_with_tied_maxima_are_row_invariant():
    V = 512
    logits = torch.randn(6, V)
    logits[:, 7] = logits[:, 300] = logits.max(-1).values + 1.0          # two equal maxima in every row
    assert_hazard_exercised("tie_boundaries", x=logits)
    tgt = torch.tensor([7, 300, 1, 2, 7, 300])
    lp, _ = F.token_logprobs(logits, tgt)
    one = torch.cat([F.token_logprobs(logits[i:i + 1].contiguous(), tgt[i:i + 1])[0] for i in range(6)])
    assert bitwise_equal(lp, one)
    assert torch.allclose(lp, torch.log_softmax(logits.double(), -1).gather(1, tgt[:, None])[:, 0].float(), atol=1e-5)


def test_router_breaks_ties_toward_the_lower_expert_index_and_experts_tolerate_empty_groups():
    E, k = 8, 2
    logits = torch.zeros(4, E)
    logits[:, 5] = logits[:, 2] = logits[:, 6] = 3.0                    # three equal top scores, two slots
    assert_hazard_exercised("tie_boundaries", x=logits)
    idx, w = moe_ops.route(logits, k, None, False, True)
    assert idx.sort(-1).values.tolist() == [[2, 5]] * 4 and torch.allclose(w.sum(-1), torch.ones(4))
    order, counts, pos = moe_ops.build_dispatch(idx, E)
    assert_hazard_exercised("e_mismatch", x=None, experts_unused=bool((counts == 0).any()))
    assert counts.tolist() == [0, 0, 4, 0, 0, 4, 0, 0]
    # fixed-order combine: equal expert outputs (a tie in the values being summed) fold the same whatever the batch
    rows = torch.randn(8, 16)
    rows[pos[:, 1]] = rows[pos[:, 0]]
    out = moe_ops.combine_fixed_order(rows, pos, torch.float32)
    one = torch.cat([moe_ops.combine_fixed_order(rows, pos[i:i + 1], torch.float32) for i in range(4)])
    assert bitwise_equal(out, one)
    idx0, w0 = moe_ops.route(torch.zeros(0, E), k, None, False, True)    # no tokens at all
    assert_hazard_exercised("t_zero", x=None, num_tokens=idx0.shape[0])
    assert moe_ops.build_dispatch(idx0, E)[1].tolist() == [0] * E


def test_tree_fold_keeps_negative_zero_and_its_fixed_order():
    parts = torch.zeros(8, 4, 16)
    parts[:, 0] = -0.0                                                   # every leaf contributes -0.0 to row 0
    parts[:, 1] = torch.randn(8, 16)
    assert_hazard_exercised("signed_zero", x=parts)
    out = tp_ops.tree_fold(parts)
    assert bool(torch.signbit(out[0]).all()), "-0.0 + -0.0 stays -0.0 through the whole tree"
    a = parts[:, 1]
    want = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]))
    assert bitwise_equal(out[1], want)
    assert tp_ops.combine_order(8)[:4] == [(0, 1), (2, 3), (4, 5), (6, 7)]
