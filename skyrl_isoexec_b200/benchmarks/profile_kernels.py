"""Small, self-terminating kernel workloads for ncu captures (one kernel family per mode).

    python skyrl_isoexec_b200/benchmarks/profile_kernels.py attn_decode | attn_prefill | gemm_large | gemm_decode | logprob | rmsnorm |
                                   glu_decode | moe_grouped | rmsnorm_decode | sampler | rmsnorm_bwd | attn_bwd | train_small |
                                   gemm_bwd_dx | gemm_bwd_dw | moe_train | reshard | gdn_chunk | gated_outnorm | small_train

Each mode allocates well under 1 GB, launches the kernel a handful of times and exits.
"""
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch  # noqa: E402

from skyrl_isoexec_b200.ops import _native, functional as F  # noqa: E402


def main(mode: str = "attn_decode") -> None:
    dev = "cuda"
    _native.lib().ix_init()
    torch.manual_seed(0)
    if mode in ("attn_decode", "attn_prefill"):
        Hq, Hkv, D = 32, 8, 128
        if mode == "attn_decode":
            B, kv_len = 64, 1536
            npg = (kv_len + 127) // 128
            kc = torch.randn(B * npg * 128, Hkv, D, device=dev).bfloat16()
            vc = torch.randn_like(kc)
            q = torch.randn(B, Hq, D, device=dev).bfloat16()
            bt = torch.arange(B * npg, dtype=torch.int32, device=dev).view(B, npg)
            items = torch.tensor([[i, 1, kv_len - 1, kv_len, i, 0, 0, 0] for i in range(B)], dtype=torch.int32, device=dev)
            meta = F.AttnMeta(items, bt)
        else:
            lens = [2560, 2560, 2560, 512]
            T = sum(lens)
            q = torch.randn(T, Hq, D, device=dev).bfloat16()
            kc = torch.randn(T, Hkv, D, device=dev).bfloat16()
            vc = torch.randn_like(kc)
            meta = F.AttnMeta.packed(lens, Hq, Hkv, dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(4):
            if i == 1:
                e0.record()
            F.attention_fwd(q, kc, vc, meta, 1 / math.sqrt(D))
        e1.record()
        torch.cuda.synchronize()
        print(f"{mode}: {e0.elapsed_time(e1) / 3 * 1e3:.1f} us per call (3 calls back to back; K+V {2 * kc.numel() * 2 / 1e6:.0f} MB)")
    elif mode in ("gemm_large", "gemm_decode"):
        M, N, K = (8192, 4096, 4096) if mode == "gemm_large" else (64, 24576, 4096)
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        for _ in range(4):
            F.gemm_nt(x, w)
    elif mode == "logprob":
        V = 151936
        lg = torch.randn(1024, V, device=dev).bfloat16()
        tg = torch.randint(0, V, (1024,), device=dev)
        for _ in range(4):
            F.logprob_fused_fwd(lg, tg, 8)
    elif mode == "rmsnorm":
        x = torch.randn(16384, 4096, device=dev).bfloat16()
        r = torch.randn_like(x)
        w = torch.ones(4096, device=dev).bfloat16()
        for _ in range(4):
            F.rmsnorm_fwd(x, w, 1e-6, False, r)
    elif mode == "glu_decode":
        # dense MLP in a decode step: gate_up GEMM with the SwiGLU epilogue (grouped kernel, one group), 64 tokens
        from skyrl_isoexec_b200.ops import moe
        x = torch.randn(64, 4096, device=dev).bfloat16()
        w = (torch.randn(1, 24576, 4096, device=dev) * 0.02).bfloat16()
        with torch.no_grad():
            for _ in range(4):
                moe.grouped_gemm(x, w, None, moe.EPI_GLU)
    elif mode == "moe_grouped":
        # one Qwen3-30B-A3B expert layer: 4096 tokens x top-8 over 128 experts (fc1 + SwiGLU x gate weight, then fc2)
        from skyrl_isoexec_b200.ops import moe
        T, E, k, H, Fd = 4096, 128, 8, 2048, 768
        gate_up = (torch.randn(E, 2 * Fd, H, device=dev) * 0.03).bfloat16()
        down = (torch.randn(E, H, Fd, device=dev) * 0.03).bfloat16()
        y = torch.randn(T, H, device=dev).bfloat16()
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).int()
        order, counts, pos = moe.build_dispatch(idx, E)
        x_rows = y.index_select(0, torch.div(order, k, rounding_mode="floor"))
        w_rows = torch.rand(T * k, device=dev)
        offs = moe.counts_to_offsets(counts)
        with torch.no_grad():
            for _ in range(4):
                moe.expert_rows_grouped(x_rows, w_rows, offs, gate_up, down)
    elif mode == "rmsnorm_decode":
        x = torch.randn(64, 4096, device=dev).bfloat16()
        r = torch.randn_like(x)
        w = torch.ones(4096, device=dev).bfloat16()
        for _ in range(4):
            F.rmsnorm_fwd(x, w, 1e-6, False, r)
    elif mode == "rmsnorm_bwd":
        x = torch.randn(8192, 4096, device=dev).bfloat16().requires_grad_()
        r = torch.randn(8192, 4096, device=dev).bfloat16().requires_grad_()
        w = torch.ones(4096, device=dev).bfloat16().requires_grad_()
        for _ in range(3):
            y, h = F.rmsnorm(x, w, 1e-6, False, r)
            (y.float().sum() + h.float().sum()).backward()
    elif mode == "attn_bwd":
        # one micro-batch of the flagship step: 8192 packed tokens, Qwen3-8B heads; prints device time of the three
        # backward kernels together and, for scale, of the library path they replace (SDPA forward + backward on padded
        # [B, H, S, D])
        Hq, Hkv, D = 32, 8, 128
        lens = [2560, 2560, 2560, 512]
        T = sum(lens)
        q, kc, vc = (torch.randn(T, h, D, device=dev).bfloat16().requires_grad_(True) for h in (Hq, Hkv, Hkv))
        dout = torch.randn(T, Hq, D, device=dev).bfloat16()
        meta = F.AttnMeta.packed(lens, Hq, Hkv, dev)
        out = F.attention(q, kc, vc, meta, 1 / math.sqrt(D))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(4):
            if it == 1:
                e0.record()
            torch.autograd.grad(out, (q, kc, vc), dout, retain_graph=True)
        e1.record()
        torch.cuda.synchronize()
        print(f"attention backward (delta + dK/dV + dQ kernels): {e0.elapsed_time(e1) / 3 * 1000:.1f} us per call")
        if len(sys.argv) > 2 and sys.argv[2] == "compare":
            B, S = 3, 2560
            qp, kp, vp = (torch.randn(B, h, S, D, device=dev).bfloat16().requires_grad_(True) for h in (Hq, Hkv, Hkv))
            do = torch.randn(B, Hq, S, D, device=dev).bfloat16()
            for it in range(4):
                if it == 1:
                    e0.record()
                o = torch.nn.functional.scaled_dot_product_attention(qp, kp, vp, is_causal=True, enable_gqa=True)
                torch.autograd.grad(o, (qp, kp, vp), do)
            e1.record()
            torch.cuda.synchronize()
            print(f"library SDPA forward + backward, 3 x 2560 tokens (7680 of the 8192): {e0.elapsed_time(e1) / 3 * 1000:.1f} us per call")
    elif mode == "train_small":
        # elementwise kernels of one training micro-batch (8192 tokens, Qwen3-8B shapes): CUDA-event time and bytes moved
        T, Hq, Hkv, D = 8192, 32, 8, 128
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def timed(fn, n=5):
            for _ in range(2):
                fn()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n * 1000

        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).bfloat16().requires_grad_(True)
        qw, kw = (torch.randn(D, device=dev).bfloat16().requires_grad_(True) for _ in range(2))
        pos = (torch.arange(T, device=dev, dtype=torch.int32) % 2560).contiguous()
        rope = F.RopeTable(D, 4096, 1e6, dev)
        kc, vc = (torch.zeros(T, Hkv, D, device=dev, dtype=torch.bfloat16) for _ in range(2))
        us = timed(lambda: F.qk_norm_rope_fwd(qkv.detach(), pos, None, rope, qw.detach(), kw.detach(), kc, vc, Hq, Hkv, D, 1e-6))
        nbytes = 2 * qkv.numel() * 2
        print(f"qk_norm_rope forward: {us:.1f} us, {nbytes / us / 1e6:.2f} TB/s (read + write of the fused QKV)")
        q, k, v = F.qk_norm_rope_train(qkv, pos, rope, qw, kw, Hq, Hkv, D, 1e-6)
        gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
        us = timed(lambda: torch.autograd.grad((q, k, v), (qkv, qw, kw), (gq, gk, gv), retain_graph=True))
        print(f"qk_norm_rope backward (+ weight-gradient fold): {us:.1f} us, {3 * qkv.numel() * 2 / us / 1e6:.2f} TB/s (dq|dk|dv + qkv read, dqkv written)")
        n = 4096 * 12288
        g = torch.randn(n, device=dev).bfloat16()
        acc = torch.zeros(n, device=dev)
        L = _native.lib()
        us = timed(lambda: _native.check(L.ix_accum_bf16_to_f32(acc.data_ptr(), g.data_ptr(), n, 1, _native.stream()), "accum"))
        print(f"gradient accumulation bf16 -> fp32, {n} elements: {us:.1f} us, {n * 10 / us / 1e6:.2f} TB/s")
    elif mode in ("gemm_bwd_dx", "gemm_bwd_dw"):
        # the two gradients of the gate|up projection of Qwen3-8B for an 8192-token micro-batch
        M, N, K = 8192, 24576, 4096
        dy = torch.randn(M, N, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        x = torch.randn(M, K, device=dev).bfloat16()
        for _ in range(4):
            F.gemm_nn(dy, w) if mode == "gemm_bwd_dx" else F.gemm_tn(dy, x)
    elif mode == "moe_train":
        # one MoE layer of Qwen3-30B-A3B (128 experts, top-8, hidden 2048, expert FFN 768), 4096 tokens: forward and
        # backward through the grouped kernels (dispatch plan, fc1, GLU x weight, fc2, combine and their VJPs)
        from skyrl_isoexec_b200.ops import moe
        T, E, k, H, Fd = 4096, 128, 8, 2048, 768
        y = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_()
        gu = (torch.randn(E, 2 * Fd, H, device=dev) * 0.02).bfloat16().requires_grad_()
        dn = (torch.randn(E, H, Fd, device=dev) * 0.02).bfloat16().requires_grad_()
        idx, w0, _ = moe.router_topk_fwd(torch.randn(T, E, device=dev), k, None, False, True)
        g = (torch.randn(T, H, device=dev) * 0.1).bfloat16()
        for _ in range(3):
            w = w0.clone().requires_grad_()
            moe._ExpertsFn.apply(y, w, gu, dn, idx, None).backward(g)
            y.grad = gu.grad = dn.grad = None
    elif mode == "reshard":
        # the pull kernel of the resharding weight sync on local memory: column-split and row-split pieces of a 1 GB buffer
        import ctypes as C
        import struct
        lib = _native.lib()
        lib.ix_reshard_pull.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        src = torch.randn(512 << 20, device=dev).bfloat16()
        dst = torch.empty(256 << 20, device=dev, dtype=torch.bfloat16)
        recs, off = [], 0
        for i in range(64):          # 64 matrices [4096, 2048] taken as the left half of [4096, 4096] sources
            recs.append(struct.pack("<QQqqqqii", src.data_ptr() + i * 4096 * 4096 * 2, dst.data_ptr() + off, 4096, 2048 * 2, 4096 * 2, 2048 * 2, 0, 0))
            off += 4096 * 2048 * 2
        d = torch.frombuffer(bytearray(b"".join(recs)), dtype=torch.uint8).to(dev)
        for _ in range(4):
            _native.check(lib.ix_reshard_pull(d.data_ptr(), len(recs), _native.stream()), "ix_reshard_pull")
    elif mode == "gdn_chunk":
        # chunked gated delta rule: 8 sequences x 2048 tokens, 16 key heads, 32 value heads of 128 (the hybrid preset's shape)
        from skyrl_isoexec_b200.ops import gdn
        T, Hk, Hv, D = 16384, 16, 32, 128
        qn = torch.nn.functional.normalize(torch.randn(T, Hk, D, device=dev), dim=-1).bfloat16()
        kn = torch.nn.functional.normalize(torch.randn(T, Hk, D, device=dev), dim=-1).bfloat16()
        v = torch.randn(T, Hv, D, device=dev).bfloat16()
        g = -torch.rand(T, Hv, device=dev) * 0.1
        beta = torch.rand(T, Hv, device=dev)
        segs = [(i * 2048, 2048, -1, -1) for i in range(8)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(4):
            if i == 3:
                e0.record()
            gdn.gdn_chunk_scan(qn, kn, v, g, beta, segs)
        e1.record()
        torch.cuda.synchronize()
        print(f"gdn_chunk_scan T={T} Hk={Hk} Hv={Hv} D={D}: {e0.elapsed_time(e1) * 1e3:.1f} us (both kernels)")
        # the token-by-token scan the chunked form replaces on this path (fp32 state in registers, one CTA per head)
        meta = gdn.GDNMeta.packed([2048] * 8, dev)
        o = torch.empty(T, Hv, D, device=dev, dtype=torch.bfloat16)
        ssm = torch.empty(0, dtype=torch.float32, device=dev)
        lib = _native.lib()
        for i in range(3):
            if i == 2:
                e0.record()
            _native.check(lib.ix_gdn_scan(qn.data_ptr(), kn.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), meta.chunks.data_ptr(),
                                          ssm.data_ptr(), o.data_ptr(), meta.n_chunks, Hk, Hv, D, D, 0, 0, _native.stream()), "ix_gdn_scan")
        e1.record()
        torch.cuda.synchronize()
        print(f"sequential gdn_scan, same input: {e0.elapsed_time(e1) * 1e3:.1f} us")
    elif mode == "gated_outnorm":
        o, z = torch.randn(8192, 32, 128, device=dev).bfloat16(), torch.randn(8192, 32, 128, device=dev).bfloat16()
        w = (torch.randn(128, device=dev) * 0.1).bfloat16()
        for _ in range(4):
            F.gated_outnorm(o, z, w, 1e-6, True)
    elif mode == "small_train":
        # the small kernels of a training step at Qwen3-8B / 30B-A3B / hybrid sizes: router top-k, PPO loss forward +
        # backward, clip-norm + AdamW over a flat buffer, GatedDeltaNet conv / gating / L2 norm. CUDA-event times printed.
        from skyrl_isoexec_b200.models.config import get_config
        from skyrl_isoexec_b200.models.decoder import DecoderLM
        from skyrl_isoexec_b200.ops import gdn, moe
        from skyrl_isoexec_b200.train import algorithms as alg
        from skyrl_isoexec_b200.train.policy_worker import PolicyWorker, WorkerConfig

        def timed(name, fn, n=1 if os.environ.get("IX_PROFILE_ONCE") else 4):     # IX_PROFILE_ONCE=1: one launch each (ncu)
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            print(f"{name}: {e0.elapsed_time(e1) / n * 1e3:.1f} us")

        logits = torch.randn(8192, 128, device=dev)
        timed("router_topk 8192 tokens x 128 experts, top-8", lambda: moe.router_topk_fwd(logits, 8, None, False, True))
        acfg = alg.AlgorithmConfig()
        loss_fn = alg.get_policy_loss("regular")
        lp0 = torch.randn(64, 2048, device=dev) * 0.3 - 2
        old, adv = lp0 + torch.randn_like(lp0) * 0.1, torch.randn(64, 2048, device=dev)
        mask = (torch.rand(64, 2048, device=dev) > 0.1).float()

        def ppo():
            a = lp0.clone().requires_grad_()
            loss, _ = loss_fn(a, old, adv, acfg, loss_mask=mask)
            loss.backward()

        timed("ppo_loss forward + backward, 64 x 2048 tokens (with the autograd call)", ppo)
        cfg = get_config("qwen3-8b", dtype="bfloat16", num_layers=2, vocab_size=32768)
        w = PolicyWorker(DecoderLM(cfg, device=dev, seed=0), WorkerConfig())
        n = w.opt.n
        w.opt.main_grad.normal_()

        def adam():
            w.optim_step()
            w.opt.main_grad.normal_()

        timed(f"grad-norm + clip + AdamW + bf16 write-back over {n / 1e6:.0f} M parameters (incl. refilling the gradient)", adam)
        hcfg = get_config("qwen3.5-hybrid", dtype="bfloat16")
        hk, hv, d = hcfg.gdn_k_heads, hcfg.gdn_v_heads, hcfg.gdn_head_dim
        C = (2 * hk + hv) * d
        T = 8192
        proj = (torch.randn(T, C + hv * d + 2 * hv, device=dev) * 0.5).bfloat16()
        conv_w = (torch.randn(C, hcfg.gdn_conv_kernel, device=dev) * 0.3).bfloat16()
        A_log, dtb = (torch.randn(hv, device=dev) * 0.1).bfloat16(), (torch.randn(hv, device=dev) * 0.1).bfloat16()
        meta = gdn.GDNMeta.packed([2048] * 4, dev)
        timed(f"GatedDeltaNet core forward (conv + gate + l2norm + chunk scan), {T} tokens, {hk}/{hv} heads of {d}",
              lambda: gdn.gdn_core_fwd(proj, conv_w, A_log, dtb, meta, hcfg, 1))
    elif mode == "sampler":
        from skyrl_isoexec_b200.engine.sampler import Sampler, SamplingParams
        lg = torch.randn(64, 151936, device=dev).bfloat16()
        sm = Sampler(dev, 0)
        for _ in range(4):
            sm(lg, [SamplingParams()] * 64)
    torch.cuda.synchronize()
    assert _native.read_status() == 0
    print("ok", mode)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "attn_decode")
