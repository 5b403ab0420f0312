"""Peer-memory collectives and tensor/data parallel paths on 2+ GPUs (skipped on smaller boxes).
Ranks are child processes, one per GPU, over NCCL on 127.0.0.1; every kernel-side wait is bounded."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from skyrl_isoexec_b200.core.testing import bitwise_equal
        from skyrl_isoexec_b200.ops import _native
        from skyrl_isoexec_b200.parallel.symm_runtime import SymmGroup
        from skyrl_isoexec_b200.parallel.tp import tree_fold

        _native.lib().ix_init()
        sg = SymmGroup(dist.group.WORLD, staging_bytes=64 << 20)
        res = {}
        # ---- one-shot tree all-reduce == all_gather + local fold in tree order, bit for bit, twice (both parities)
        ok = True
        for it in range(3):
            torch.manual_seed(100 * it + rank)
            part = torch.randn(77, 1024, device="cuda")
            got = sg.tree_all_reduce(part)
            gathered = torch.empty(world, 77, 1024, device="cuda")
            dist.all_gather_into_tensor(gathered, part)
            ok &= bitwise_equal(got, tree_fold(gathered))
        sg.check()
        res["tree_all_reduce_bitwise"] = bool(ok)
        # ---- two-shot bucketed sum == tree fold of the gathered buffers (bitwise) and ~= NCCL all-reduce
        torch.manual_seed(7 + rank)
        n = (64 << 20) // 4 // 2 * 3 + 40                     # spans several buckets, ragged tail
        flat = torch.randn(n, device="cuda")
        ref_in = flat.clone()
        sg.all_reduce_sum_(flat)
        sg.check()
        nccl = ref_in.clone()
        dist.all_reduce(nccl)
        res["all_reduce_close_to_nccl"] = bool((flat - nccl).abs().max() < 1e-4)
        probe = ref_in[:4096].clone()
        g = torch.empty(world, 4096, device="cuda")
        dist.all_gather_into_tensor(g, probe)
        res["all_reduce_bitwise_tree"] = bool(bitwise_equal(flat[:4096], tree_fold(g)))
        # ---- timing of the DP reduction (device time, max over ranks)
        big = torch.randn(256 << 20, device="cuda")           # 1 GiB of fp32
        for _ in range(2):
            sg.all_reduce_sum_(big)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sg.all_reduce_sum_(big)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e0.record()
        dist.all_reduce(big)
        e1.record()
        torch.cuda.synchronize()
        t2 = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        res["ours_ms_1GiB"], res["nccl_ms_1GiB"] = float(t), float(t2)
        res["status"] = _native.read_status()
        if rank == 0:
            q.put(res)
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_peer_collectives_two_ranks():
    world = 2 if _ngpu() < 4 else 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = q.get(timeout=500)
    for p in procs:
        p.join(timeout=120)
    print("peer collectives:", res)
    assert res["tree_all_reduce_bitwise"] and res["all_reduce_bitwise_tree"] and res["all_reduce_close_to_nccl"]
    assert res["status"] == 0


def test_bounded_wait_reports_instead_of_hanging():
    """A flag that nothing sets: the kernel gives up after its limit, the status word says so and the
    context stays usable (single GPU; the 'peer' is a slot of a local array that no one writes)."""
    import ctypes as C

    from skyrl_isoexec_b200.ops import _native

    lib = _native.lib()
    lib.ix_init()
    lib.ix_peer_handshake.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_void_p]
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    ptrs = (C.c_longlong * 2)(flags.data_ptr(), flags.data_ptr())
    assert _native.read_status() == 0
    _native.check(lib.ix_peer_handshake(ptrs, 0, 2, 1, _native.stream()), "handshake")   # rank 1's slot is never written
    torch.cuda.synchronize()
    assert _native.read_status() == 105                        # ST_TIMEOUT_FLAG
    assert _native.read_status() == 0                          # cleared by the read
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0                               # the context is still healthy
