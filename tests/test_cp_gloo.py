"""Sequence parallel attention (Ulysses all-to-all and all-gather forms) on CPU/gloo: same bits as one rank."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs():
    g = torch.Generator().manual_seed(0)
    lens = [40, 24, 64]                    # 128 tokens: divides by 2 and 4
    T, Hq, Hkv, D = sum(lens), 4, 2, 64
    q = torch.randn(T, Hq, D, generator=g)
    k = torch.randn(T, Hkv, D, generator=g)
    v = torch.randn(T, Hkv, D, generator=g)
    go = torch.randn(T, Hq, D, generator=g)
    return lens, q, k, v, go


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.ops import functional as F
        from skyrl_isoexec_b200.parallel import cp as CP
        from skyrl_isoexec_b200.parallel.state import ParallelState

        ps = ParallelState.build(cp=world)
        lens, q, k, v, go = _inputs()
        meta = F.AttnMeta.packed(lens, 4 // world, 2 // world, "cpu")     # the kernel sees H/cp heads of the whole batch
        ql, kl, vl = (CP.shard_sequence(t, rank, world).clone().requires_grad_() for t in (q, k, v))
        o = CP.ulysses_attention(ql, kl, vl, meta, 0.125, ps)
        (o * CP.shard_sequence(go, rank, world)).sum().backward()
        # all-gather form: K/V gathered, queries stay local; check the gather's forward and backward
        kg = CP.gather_sequence(kl.detach().clone().requires_grad_(), ps)
        ok_gather = torch.equal(kg, k)
        q_out.put((rank, o.detach().numpy(), ql.grad.numpy(), kl.grad.numpy(), vl.grad.numpy(), ok_gather))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(240)
def test_ulysses_attention_equals_single_rank():
    from skyrl_isoexec_b200.ops import functional as F

    world = 2
    ctx = mp.get_context("spawn")
    qq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, qq)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, o, gq, gk, gv, okg = qq.get(timeout=60)
        got[r] = tuple(torch.from_numpy(x) for x in (o, gq, gk, gv)) + (okg,)
    for p in procs:
        p.join(timeout=60)
    lens, q, k, v, go = _inputs()
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    o = F.attention(q, k, v, F.AttnMeta.packed(lens, 4, 2, "cpu"), 0.125)
    (o * go).sum().backward()
    n = q.shape[0] // world
    for r in range(world):
        sl = slice(r * n, (r + 1) * n)
        assert torch.equal(got[r][0], o.detach()[sl])                    # forward: bytes moved, same kernel per head
        for a, b in ((got[r][1], q.grad[sl]), (got[r][2], k.grad[sl]), (got[r][3], v.grad[sl])):
            assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)
        assert got[r][4]


def _ring_worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from skyrl_isoexec_b200.parallel import cp as CP
        from skyrl_isoexec_b200.parallel.state import ParallelState

        ps = ParallelState.build(cp=world)
        g = torch.Generator().manual_seed(3)
        S, Hq, Hkv, D = 96, 4, 2, 32
        q, k, v, go = (torch.randn(S, h, D, generator=g) for h in (Hq, Hkv, Hkv, Hq))
        ql, kl, vl = (CP.shard_sequence(t, rank, world).clone().requires_grad_() for t in (q, k, v))
        o = CP.ring_attention(ql, kl, vl, D ** -0.5, ps, causal=True)
        (o * CP.shard_sequence(go, rank, world)).sum().backward()
        q_out.put((rank, o.detach().numpy(), ql.grad.numpy(), kl.grad.numpy(), vl.grad.numpy()))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.timeout(240)
@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_matches_full_attention_forward_and_backward(world):
    ctx = mp.get_context("spawn")
    qq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ring_worker, args=(r, world, port, qq)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, o, gq, gk, gv = qq.get(timeout=90)
        got[r] = tuple(torch.from_numpy(x) for x in (o, gq, gk, gv))
    for p in procs:
        p.join(timeout=60)
    g = torch.Generator().manual_seed(3)
    S, Hq, Hkv, D = 96, 4, 2, 32
    q, k, v, go = (torch.randn(S, h, D, generator=g) for h in (Hq, Hkv, Hkv, Hq))
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    qs = q.transpose(0, 1)
    ks, vs = (t.repeat_interleave(Hq // Hkv, 1).transpose(0, 1) for t in (k, v))
    sc = (qs @ ks.transpose(1, 2)) * D ** -0.5
    sc = sc.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    o = (sc.softmax(-1) @ vs).transpose(0, 1)
    (o * go).sum().backward()
    n = S // world
    for r in range(world):
        sl = slice(r * n, (r + 1) * n)
        for a, b in ((got[r][0], o.detach()[sl]), (got[r][1], q.grad[sl]), (got[r][2], k.grad[sl]), (got[r][3], v.grad[sl])):
            assert torch.allclose(a, b, atol=2e-5, rtol=1e-4), (r, (a - b).abs().max())
