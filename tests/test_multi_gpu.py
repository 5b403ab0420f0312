"""Peer-memory collectives and tensor/data parallel paths on 2+ GPUs (skipped on smaller boxes).
Ranks are child processes, one per GPU, over NCCL on 127.0.0.1; every kernel-side wait is bounded."""
import datetime
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

# a rank that raised leaves its peers in a collective: the process group gives up after this long instead of ten minutes
_PG_TIMEOUT = datetime.timedelta(seconds=120)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _collect(q, procs, n=1, timeout=500):
    """n results from the ranks' queue; gives up at once when a rank has died instead of waiting out the timeout."""
    import queue as _queue
    import time as _time

    out, t0 = [], _time.time()
    while len(out) < n:
        try:
            out.append(q.get(timeout=2))
        except _queue.Empty:
            if any((not p.is_alive()) and p.exitcode not in (0, None) for p in procs):
                raise AssertionError("a rank exited with an error: " + str([p.exitcode for p in procs]))
            if _time.time() - t0 > timeout:
                raise AssertionError("timed out waiting for the ranks")
    return out


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=_PG_TIMEOUT)
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
        from conftest import finish_rank

        finish_rank(dist)


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
    res = _collect(q, procs, 1, 500)[0]
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


def _tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=_PG_TIMEOUT)
    try:
        from skyrl_isoexec_b200.core.testing import bitwise_equal
        from skyrl_isoexec_b200.ops import _native, functional as F
        from skyrl_isoexec_b200.parallel.tp_fused import FusedTP, leaftree_gemm_fused

        _native.lib().ix_init()
        rt = FusedTP(dist.group.WORLD, stage_bytes=192 << 20, out_bytes=96 << 20, gather_bytes=96 << 20)
        res = {}
        G, N, K = 8, 512, 2048
        Kr = K // world
        ok = {"ar1": True, "ar2": True, "rs": True, "ag": True}
        for it in range(3):                                    # three rounds: both staging halves get reused
            g = torch.Generator(device="cuda").manual_seed(11 + it)
            w_full = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
            ws = w_full[:, rank * Kr:(rank + 1) * Kr].contiguous()
            for M, key in ((40, "ar1"), (640, "ar2"), (128 * world * 2, "rs")):
                x_full = torch.randn(M, K, device="cuda", generator=g).bfloat16()
                xs = x_full[:, rank * Kr:(rank + 1) * Kr].contiguous()
                want = leaftree_gemm_fused(x_full, w_full, G, out_f32=False)          # the single-rank member of the family
                got = rt.row_parallel(xs, ws, G // world, mode="reduce_scatter" if key == "rs" else "allreduce")
                if key == "rs":
                    want = want[rank * (M // world):(rank + 1) * (M // world)]
                ok[key] &= bool(bitwise_equal(got, want))
            # all-gather -> GEMM: every rank contributes different rows
            gl = torch.Generator(device="cuda").manual_seed(1000 * it + rank)
            x_loc = torch.randn(256, 1024, device="cuda", generator=gl).bfloat16()
            w_col = (torch.randn(384, 1024, device="cuda", generator=g) * 0.05).bfloat16()
            gathered = torch.empty(world * 256, 1024, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(gathered, x_loc)
            ok["ag"] &= bool(bitwise_equal(rt.allgather_linear(x_loc, w_col), F.gemm_nt(gathered, w_col)))
        rt.check()
        res.update({f"fused_{k}_bitwise": v for k, v in ok.items()})

        # ---- timing, device clock, max over ranks: down-projection of Qwen3-8B at TP=world, 8192 tokens
        def timed(fn, n=5):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / n], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        M, N, Kr = 8192, 4096, 12288 // world
        x = torch.randn(M, Kr, device="cuda").bfloat16()
        w = (torch.randn(N, Kr, device="cuda") * 0.02).bfloat16()

        def unfused():
            y = torch.matmul(x, w.t())
            dist.all_reduce(y)
            return y

        res["fused_ar2_ms"] = timed(lambda: rt.row_parallel(x, w, 1))
        res["fused_rs_ms"] = timed(lambda: rt.row_parallel(x, w, 1, mode="reduce_scatter"))
        res["cublas_nccl_allreduce_ms"] = timed(unfused)
        res["gemm_only_ms"] = timed(lambda: F.gemm_nt(x, w))
        xl = torch.randn(M // world, 4096, device="cuda").bfloat16()
        wq = (torch.randn(6144 // world, 4096, device="cuda") * 0.02).bfloat16()
        gath = torch.empty(M, 4096, device="cuda", dtype=torch.bfloat16)

        def unfused_ag():
            dist.all_gather_into_tensor(gath, xl)
            return torch.matmul(gath, wq.t())

        res["fused_ag_ms"] = timed(lambda: rt.allgather_linear(xl, wq))
        res["nccl_allgather_cublas_ms"] = timed(unfused_ag)
        xd = torch.randn(64, Kr, device="cuda").bfloat16()
        res["fused_ar1_decode_ms"] = timed(lambda: rt.row_parallel(xd, w, 1), n=20)

        def unfused_dec():
            y = torch.matmul(xd, w.t())
            dist.all_reduce(y)
            return y

        res["cublas_nccl_decode_ms"] = timed(unfused_dec, n=20)
        rt.check()
        res["status"] = _native.read_status()
        if rank == 0:
            q.put(res)
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_fused_tp_gemm_matches_single_rank_tree_bitwise():
    """GEMM -> all-reduce (one- and two-shot), GEMM -> reduce-scatter and all-gather -> GEMM, each one kernel
    over peer memory, reproduce the bits of the single-rank 8-leaf tree GEMM at TP = 2 (and 4)."""
    world = 2 if _ngpu() < 4 else 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = _collect(q, procs, 1, 500)[0]
    for p in procs:
        p.join(timeout=120)
    print("fused tp gemm:", res)
    assert res["fused_ar1_bitwise"] and res["fused_ar2_bitwise"] and res["fused_rs_bitwise"] and res["fused_ag_bitwise"]
    assert res["status"] == 0


def test_fused_tp_kernel_gives_up_when_a_peer_never_arrives():
    """One GPU plays rank 0 of 2; 'rank 1' is a set of local buffers that nothing writes. The reducer warps'
    wait for rank 1's tile flags runs out, the kernel frees its TMEM and returns, the status word reports it."""
    import ctypes as C

    from skyrl_isoexec_b200.ops import _native
    from skyrl_isoexec_b200.parallel import tp_fused

    lib = _native.lib()
    lib.ix_init()
    tp_fused._sig(lib)
    M, N, K, bn = 16, 256, 256, 32
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    nfl = int(lib.ix_tp_stage_floats(M, N, tp_fused.TP_AR1, 2, bn))
    stage = [torch.zeros(nfl, device="cuda") for _ in range(2)]
    flags = [torch.zeros(4096, dtype=torch.int32, device="cuda") for _ in range(2)]
    arr = lambda ts: (C.c_longlong * 2)(*[t.data_ptr() for t in ts])  # noqa: E731
    assert _native.read_status() == 0
    _native.check(lib.ix_tp_gemm_fused(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, K, K, N, tp_fused.TP_AR1, 1, bn, 0,
                                       0, 2, 1, arr(stage), arr(flags), None, None, None, None, 0, 0, _native.stream()), "tp_gemm")
    torch.cuda.synchronize()
    assert _native.read_status() == 105
    assert int(flags[1].view(-1, 2)[: N // bn, 0].min()) == 1        # rank 0 did publish its tiles to the 'peer'
    y = torch.ones(4, device="cuda")
    assert float(y.sum()) == 4.0


def _ep_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=_PG_TIMEOUT)
    try:
        from skyrl_isoexec_b200.core.testing import bitwise_equal
        from skyrl_isoexec_b200.ops import _native, moe
        from skyrl_isoexec_b200.ops.moe_ep import EPPeer

        _native.lib().ix_init()
        res = {}
        E, k, H, Fd, T = 16, 4, 256, 192, 300 + 17 * rank          # ranks hold different numbers of tokens
        g = torch.Generator(device="cuda").manual_seed(1)
        gate_up = (torch.randn(E, 2 * Fd, H, device="cuda", generator=g) * 0.06).bfloat16()
        down = (torch.randn(E, H, Fd, device="cuda", generator=g) * 0.06).bfloat16()
        e_loc = E // world
        gu_l, dn_l = gate_up[rank * e_loc:(rank + 1) * e_loc].contiguous(), down[rank * e_loc:(rank + 1) * e_loc].contiguous()
        rt = EPPeer(dist.group.WORLD, H, E, max_rows_local=400 * k)
        ok = True
        with torch.no_grad():
            for it in range(3):
                gl = torch.Generator(device="cuda").manual_seed(100 * it + rank)
                y = torch.randn(T, H, device="cuda", generator=gl).bfloat16()
                idx = torch.stack([torch.randperm(E, device="cuda", generator=gl)[:k] for _ in range(T)]).int()
                w = torch.rand(T, k, device="cuda", generator=gl)
                rows, pos = rt.forward(y, idx, w, gu_l, dn_l)
                got = moe.combine_fixed_order(rows, pos, torch.bfloat16)
                order, counts, pos1 = moe.build_dispatch(idx, E)
                x_rows = y.index_select(0, torch.div(order, k, rounding_mode="floor"))
                w_rows = w.reshape(-1).index_select(0, order)
                rows1 = moe.expert_rows_grouped(x_rows, w_rows, moe.counts_to_offsets(counts), gate_up, down)
                ok &= bool(bitwise_equal(got, moe.combine_fixed_order(rows1, pos1, torch.bfloat16)))
        res["ep_peer_equals_single_rank_bitwise"] = ok
        # ---- one Qwen3-30B-A3B-sized layer: 4096 tokens per rank, 128 experts, top-8 (device time, max over ranks)
        E, k, H, Fd, T = 128, 8, 2048, 768, 4096
        e_loc = E // world
        gu = (torch.randn(e_loc, 2 * Fd, H, device="cuda") * 0.03).bfloat16()
        dn = (torch.randn(e_loc, H, Fd, device="cuda") * 0.03).bfloat16()
        rt2 = EPPeer(dist.group.WORLD, H, E, max_rows_local=T * k, capacity_rows=T * k * 2)
        y = torch.randn(T, H, device="cuda").bfloat16()
        idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).int()
        w = torch.rand(T, k, device="cuda")
        with torch.no_grad():
            for _ in range(2):
                rt2.forward(y, idx, w, gu, dn)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                rows, pos = rt2.forward(y, idx, w, gu, dn)
                moe.combine_fixed_order(rows, pos, torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 5], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["ep_layer_ms_4096tok_per_rank"] = float(t)
        res["status"] = _native.read_status()
        if rank == 0:
            q.put(res)
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_expert_parallel_over_peer_memory_equals_single_rank_bitwise():
    world = 2 if _ngpu() < 4 else 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = _collect(q, procs, 1, 500)[0]
    for p in procs:
        p.join(timeout=120)
    print("expert parallel over peer memory:", res)
    assert res["ep_peer_equals_single_rank_bitwise"] and res["status"] == 0


def _tp_model_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=_PG_TIMEOUT)
    try:
        from skyrl_isoexec_b200.core.testing import count_bit_mismatches
        from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
        from skyrl_isoexec_b200.engine.sampler import SamplingParams
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.ops import _native
        from skyrl_isoexec_b200.parallel import tp_fused
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        _native.lib().ix_init()
        ps = ParallelState.build(tp=world)
        tp_fused.register(ps.tp_group, tp_fused.FusedTP(ps.tp_group, stage_bytes=64 << 20, out_bytes=32 << 20, gather_bytes=8 << 20))
        cfg = get_config("tiny-qwen3-bf16", hidden_size=1024, num_q_heads=8, num_kv_heads=4, head_dim=128, ffn_size=2048,
                         num_layers=2, tp_invariant=True, pik_leaves=8)
        model = DecoderLM(cfg, ps, "cuda", seed=2)
        eng = LLMEngine(model, EngineConfig(max_num_seqs=8, num_kv_pages=48, max_num_batched_tokens=512, seed=9))
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (300, 40, 150, 90, 210, 33)]
        outs = eng.generate(prompts, SamplingParams(max_generate_length=24, ignore_eos=True))
        seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.randn(rmask.shape, generator=g) * 1e-3})
        worker = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=700))
        lp = worker.forward(batch)
        ro = torch.zeros_like(lp)
        for i, o in enumerate(outs):
            ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
        res = {"engine_vs_trainer_mismatches_tp": count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous())}
        batch["action_log_probs"] = lp
        # the same weights with the residual stream cut over the two ranks (sequence parallelism): same logprob bits,
        # and the same gradients up to the order in which the norm weights' partial sums meet
        import dataclasses

        sp_model = DecoderLM(dataclasses.replace(cfg, sequence_parallel=True), ps, "cuda", seed=2)
        sp_worker = PolicyWorker(sp_model, WorkerConfig(max_tokens_per_microbatch=700))
        lp_sp = sp_worker.forward(batch)
        res["sp_mismatches"] = count_bit_mismatches((lp_sp * rmask).contiguous(), (lp * rmask).contiguous())
        sp_worker.forward_backward(batch)
        sp_worker.reduce_gradients()
        worker.forward_backward(batch)
        worker.reduce_gradients()
        ga, gb = worker.opt.main_grad, sp_worker.opt.main_grad
        res["sp_grad_rel_diff"] = float((ga - gb).abs().max() / ga.abs().max().clamp(min=1e-12))
        worker.opt.zero_grad()                                   # the step below reduces its own gradients
        worker.forward_backward(batch)
        res["grad_norm_tp"] = worker.optim_step()
        tp_fused.get(ps.tp_group).check()
        if rank == 0:
            # the same model on ONE rank (8 leaves in one kernel) scores the same sequences: TP must not change a bit
            single = DecoderLM(cfg, ParallelState.single(), "cuda", seed=2)
            w1 = PolicyWorker(single, WorkerConfig(max_tokens_per_microbatch=700))
            lp1 = w1.forward(batch)
            res["tp2_vs_tp1_mismatches"] = count_bit_mismatches((lp1 * rmask).contiguous(), (ro * rmask).contiguous())
            res["status"] = _native.read_status()
            from skyrl_isoexec_b200.parallel import tp as tp_ops

            res["census"] = tp_ops.transport_census()
            res["admitted"] = sorted(tp_ops.admitted_shapes().values())
            q.put(res)
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_tensor_parallel_model_with_fused_kernels_is_bitwise_tp_invariant():
    """Engine and trainer at TP=2, their row-parallel linears running as the fused GEMM->all-reduce kernel:
    rollout logprobs == trainer logprobs == the logprobs of the same model on a single rank, bit for bit."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_model_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = _collect(q, procs, 1, 500)[0]
    for p in procs:
        p.join(timeout=120)
    print("tp model:", res)
    assert res["engine_vs_trainer_mismatches_tp"] == 0 and res["tp2_vs_tp1_mismatches"] == 0
    assert res["sp_mismatches"] == 0 and res["sp_grad_rel_diff"] < 2e-2
    assert res["grad_norm_tp"] > 0 and res["status"] == 0
    # every row-parallel shape passed its bitwise admission probe and was then served by the fused kernel
    assert res["admitted"] and all(res["admitted"]), res["admitted"]
    assert res["census"].get("row_parallel/fused_peer", 0) > 0 and "row_parallel/refused" not in res["census"], res["census"]


def _ep_model_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=_PG_TIMEOUT)
    try:
        from skyrl_isoexec_b200.core.testing import count_bit_mismatches
        from skyrl_isoexec_b200.engine.llm_engine import EngineConfig, LLMEngine
        from skyrl_isoexec_b200.engine.sampler import SamplingParams
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.ops import _native
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.parallel.transports import setup_transports
        from skyrl_isoexec_b200.train.batch import TrainingInputBatch, build_sequences
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        _native.lib().ix_init()
        ps = ParallelState.build(ep=world)
        cfg = get_config("tiny-moe", dtype="bfloat16", hidden_size=512, num_q_heads=4, num_kv_heads=2,
                         head_dim=128, moe_ffn_size=256, num_experts=16, top_k=4)
        reg = setup_transports(ps, cfg, max_tokens=1024)
        model = DecoderLM(cfg, ps, "cuda", seed=4)
        eng = LLMEngine(model, EngineConfig(max_num_seqs=8, num_kv_pages=40, max_num_batched_tokens=512, seed=20 + rank))
        g = torch.Generator().manual_seed(rank)                      # every rank has its own prompts and its own lengths
        prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in torch.randint(20, 200, (4 + rank,), generator=g)]
        outs = eng.generate(prompts, SamplingParams(max_generate_length=12 + 7 * rank, ignore_eos=True))
        seq, att, rmask = build_sequences([o.prompt_ids for o in outs], [o.response_ids for o in outs])
        batch = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                                    "advantages": torch.randn(rmask.shape, generator=g) * 1e-3})
        worker = PolicyWorker(model, WorkerConfig(max_tokens_per_microbatch=300 if rank == 0 else 1000))
        lp = worker.forward(batch)
        ro = torch.zeros_like(lp)
        for i, o in enumerate(outs):
            ro[i, :len(o.response_logprobs)] = torch.tensor(o.response_logprobs)
        mism = count_bit_mismatches((lp * rmask).contiguous(), (ro * rmask).contiguous())
        batch["action_log_probs"] = lp
        batch["rollout_logprobs"] = ro                               # the backward pass's own forward is compared as well
        batch.metadata["check_rollout_bits"] = True
        fb = worker.forward_backward(batch)
        gn = worker.optim_step()
        from skyrl_isoexec_b200.ops import moe as moe_ops
        res = torch.tensor([float(mism), gn, float(_native.read_status()), float(fb["rollout_bits"]["mismatches"]),
                            float(moe_ops._SERVED["moe.experts/nccl_grouped_autograd"])], device="cuda", dtype=torch.float64)
        allr = [torch.zeros_like(res) for _ in range(world)]
        dist.all_gather(allr, res)
        if rank == 0:
            q.put({"registered": reg, "mismatches": [int(r[0]) for r in allr], "grad_norms": [float(r[1]) for r in allr],
                   "status": [int(r[2]) for r in allr], "train_mismatches": [int(r[3]) for r in allr],
                   "grouped_autograd_blocks": [int(r[4]) for r in allr]})
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_moe_model_with_expert_parallelism_over_peer_memory():
    """MoE engine and trainer at EP=2: dispatch / grouped GEMMs / return over peer memory in the no-grad passes, NCCL
    all-to-all under autograd; ranks hold different prompts and step in lockstep. Rollout == trainer, bit for bit."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_model_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = _collect(q, procs, 1, 500)[0]
    for p in procs:
        p.join(timeout=120)
    print("moe ep model:", res)
    assert res["registered"]["ep"] and res["mismatches"] == [0, 0] and res["status"] == [0, 0]
    assert res["train_mismatches"] == [0, 0] and min(res["grouped_autograd_blocks"]) > 0
    assert res["grad_norms"][0] == res["grad_norms"][1] > 0


def _separate_engine_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=_PG_TIMEOUT)
    try:
        import json

        from skyrl_isoexec_b200.ops import _native
        from skyrl_isoexec_b200.parallel.state import ParallelState
        from skyrl_isoexec_b200.sync.reshard import PeerPullResharder
        from skyrl_isoexec_b200.train.config import SkyRLTrainConfig
        from skyrl_isoexec_b200.train.trainer import RayPPOTrainer

        _native.lib().ix_init()
        ps = ParallelState.build(tp=world)
        mo = {"hidden_size": 1024, "num_q_heads": 8, "num_kv_heads": 4, "head_dim": 128, "ffn_size": 2048, "num_layers": 2, "pik_leaves": 8}
        cfg = SkyRLTrainConfig.from_cli_overrides([
            "trainer.policy.model=tiny-qwen3-bf16", "trainer.policy.model_overrides=" + json.dumps(mo),
            "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4", "generator.n_samples_per_prompt=4",
            "generator.sampling_params.max_generate_length=40", "generator.sampling_params.ignore_eos=true",
            "data.synthetic_prompt_len=200", "data.synthetic_prompts=32", "trainer.max_prompt_length=200",
            "generator.inference_engine.num_kv_pages=64", "generator.inference_engine.max_num_batched_tokens=1024",
            "trainer.max_tokens_per_microbatch=1024", "trainer.policy.optimizer_config.lr=1e-3", "trainer.logger=jsonl",
            f"generator.inference_engine.tensor_parallel_size={world // 2}"])
        tr = RayPPOTrainer(cfg, ps=ps, device=f"cuda:{rank}")
        tr.build_models()
        tr.sync_weights()
        it = iter(tr.loader)
        out = {"mism": [], "bytes": [], "far": [], "sync_s": [], "peer_pull": isinstance(tr.resharder, PeerPullResharder),
               "engines": tr.engines_per_replica}
        for _ in range(3):
            m = tr.train_step(next(it))
            out["mism"].append(int(m["policy/rollout_train_logprob_bit_mismatches"]))
            out["bytes"].append(int(m["sync/bytes"]))
            out["far"].append(int(m["sync/bytes_from_peers"]))
            out["sync_s"].append(float(m["timing/sync_weights"]))
        out["status"] = _native.read_status()
        q.put((rank, out))
    finally:
        from conftest import finish_rank

        finish_rank(dist)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_trainer_tp_feeds_engines_of_half_the_degree_through_the_peer_pull_sync():
    """Trainer at TP = all GPUs, engines at half that degree (TP2 -> two TP1 engines on 2 GPUs, TP4 -> two TP2 engines on
    4): three full GRPO steps; every step reshards the updated weights with ONE pull kernel over peer memory, and the
    engines' rollout logprobs equal the trainer's scoring forward bit for bit."""
    world = 2 if _ngpu() < 4 else 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_separate_engine_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(_collect(q, procs, world))
    for p in procs:
        p.join(timeout=120)
    print("separate engines:", res[0])
    for r in range(world):
        o = res[r]
        assert o["peer_pull"] and o["engines"] == 2 and o["status"] == 0
        assert o["mism"] == [0, 0, 0], (r, o["mism"])
        assert all(b > 0 for b in o["bytes"]) and all(0 < f < b for f, b in zip(o["far"], o["bytes"]))
