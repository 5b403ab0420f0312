"""Kernel microbenchmarks against the roofline of THIS machine.

    python -m skyrl_isoexec_b200.benchmarks.bench_kernels [--model qwen3-8b] [--batch 64] [--json out.json]

Timing: CUDA events on the launching stream, 3 warm-ups, median of 10, an L2 flush (256 MB write) before every timed
launch of the decode-sized cases. Denominators: the copy bandwidth and cuBLAS bf16 rate measured here at start-up
(a 1 GiB copy and an 8192^3 matmul), so fractions read "of measured". Holds a few GB on the device.
"""

from __future__ import annotations

import argparse
import json
import math

import torch

from ..models.config import get_config
from ..ops import _native
from ..ops import functional as F


def _timer(flush):
    def timeit(fn, iters=10, warm=3, do_flush=True):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(iters):
            if do_flush:
                flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2] * 1e3   # us
    return timeit


def measure_peaks(timeit) -> dict:
    a = torch.empty(1 << 29, dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(a)
    t = timeit(lambda: b.copy_(a), do_flush=False)
    hbm = 2 * a.numel() * 2 / t / 1e6                      # TB/s, read + write
    del a, b
    x = torch.randn(8192, 8192, device="cuda").bfloat16()
    t = timeit(lambda: torch.matmul(x, x), do_flush=False)
    return {"hbm_tbs": hbm, "bf16_tflops": 2 * 8192 ** 3 / t / 1e6}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    _native.lib().ix_init()
    cfg = get_config(args.model)
    dev = "cuda"
    timeit = _timer(torch.empty(256 << 20, dtype=torch.uint8, device=dev))
    peaks = measure_peaks(timeit)
    print(f"measured here: copy {peaks['hbm_tbs']:.2f} TB/s, cuBLAS bf16 {peaks['bf16_tflops']:.0f} TFLOP/s")
    h, ffn, D = cfg.hidden_size, cfg.ffn_size, cfg.head_dim
    Hq, Hkv = cfg.num_q_heads, cfg.num_kv_heads
    shapes = [((Hq + 2 * Hkv) * D, h, "qkv"), (h, Hq * D, "o"), (2 * ffn, h, "gate_up"), (h, ffn, "down"), (cfg.vocab_size, h, "lm_head")]
    rows = []
    B, M = args.batch, args.tokens
    for N, K, name in shapes:
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        x = torch.randn(B, K, device=dev).bfloat16()
        t = timeit(lambda: F.gemm_nt(x, w))
        rows.append({"kernel": "gemm_decode", "case": f"{name} M={B} N={N} K={K}", "us": t, "tbs": N * K * 2 / t / 1e6,
                     "frac_of_measured": N * K * 2 / t / 1e6 / peaks["hbm_tbs"]})
        if name != "lm_head":
            # the same decode GEMM as the device sees it inside a step: launches queued back to back over enough weight
            # copies to exceed L2 (the row above times one call at a time and so includes the host's launch path)
            copies = [w] + [w.clone() for _ in range(max(1, (600 << 20) // (N * K * 2)))]

            def queue(fn):
                def run():
                    for c in copies:
                        fn(c)
                return run

            t = timeit(queue(lambda c: F.gemm_nt(x, c)), do_flush=False) / len(copies)
            rows.append({"kernel": "gemm_decode_queued", "case": f"{name} M={B} N={N} K={K}", "us": t, "tbs": N * K * 2 / t / 1e6,
                         "frac_of_measured": N * K * 2 / t / 1e6 / peaks["hbm_tbs"]})
            if name in ("o", "down") and K % 128 == 0:
                from ..parallel import tp_fused

                t = timeit(queue(lambda c: tp_fused.leaftree_gemm_fused(x, c, 2, out_f32=False)), do_flush=False) / len(copies)
                rows.append({"kernel": "gemm_decode_queued", "case": f"{name} M={B} N={N} K={K}, 2-leaf tree (one CTA per leaf)", "us": t,
                             "tbs": N * K * 2 / t / 1e6, "frac_of_measured": N * K * 2 / t / 1e6 / peaks["hbm_tbs"]})
            del copies
            xl = torch.randn(M, K, device=dev).bfloat16()
            t = timeit(lambda: F.gemm_nt(xl, w), do_flush=False)
            tf = 2 * M * N * K / t / 1e6
            rows.append({"kernel": "gemm_train", "case": f"{name} M={M} N={N} K={K}", "us": t, "tflops": tf, "frac_of_measured": tf / peaks["bf16_tflops"]})
            # the two gradients of the same layer: dX = dY @ W (NN), dW = dY^T @ X (TN); library time beside ours
            dy = torch.randn(M, N, device=dev).bfloat16()
            for kern, ours, lib in (("gemm_bwd_dx", lambda: F.gemm_nn(dy, w), lambda: torch.matmul(dy, w)),
                                    ("gemm_bwd_dw", lambda: F.gemm_tn(dy, xl), lambda: torch.matmul(dy.t(), xl))):
                t, tl = timeit(ours, do_flush=False), timeit(lib, do_flush=False)
                tf = 2 * M * N * K / t / 1e6
                rows.append({"kernel": kern, "case": f"{name} M={M} N={N} K={K}", "us": t, "tflops": tf,
                             "frac_of_measured": tf / peaks["bf16_tflops"], "library_us": tl})
            del dy
    for kv_len in (512, 1536, 2560):
        npg = (kv_len + 127) // 128
        kc = torch.randn(B * npg * 128, Hkv, D, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        q = torch.randn(B, Hq, D, device=dev).bfloat16()
        bt = torch.arange(B * npg, dtype=torch.int32, device=dev).view(B, npg)
        items = torch.tensor([[i, 1, kv_len - 1, kv_len, i, 0, 0, 0] for i in range(B)], dtype=torch.int32, device=dev)
        meta = F.AttnMeta(items, bt)
        t = timeit(lambda: F.attention_fwd(q, kc, vc, meta, 1 / math.sqrt(D)))
        tb = B * kv_len * Hkv * D * 2 * 2 / t / 1e6
        rows.append({"kernel": "attention_decode", "case": f"B={B} kv={kv_len}", "us": t, "tbs": tb, "frac_of_measured": tb / peaks["hbm_tbs"]})
    lens = [2560, 2560, 2560, 512]
    T = sum(lens)
    q = torch.randn(T, Hq, D, device=dev).bfloat16()
    k = torch.randn(T, Hkv, D, device=dev).bfloat16()
    v = torch.randn_like(k)
    meta = F.AttnMeta.packed(lens, Hq, Hkv, dev)
    t = timeit(lambda: F.attention_fwd(q, k, v, meta, 1 / math.sqrt(D)), do_flush=False)
    fl = 4 * D * sum(n * n for n in lens) / 2 * Hq
    rows.append({"kernel": "attention_prefill", "case": f"packed {lens}", "us": t, "tflops": fl / t / 1e6, "frac_of_measured": fl / t / 1e6 / peaks["bf16_tflops"]})
    x = torch.randn(M, h, device=dev).bfloat16()
    r = torch.randn_like(x)
    w = torch.ones(h, device=dev).bfloat16()
    t = timeit(lambda: F.rmsnorm_fwd(x, w, 1e-6, False, r), do_flush=False)
    tb = 4 * M * h * 2 / t / 1e6
    rows.append({"kernel": "rmsnorm+residual", "case": f"{M}x{h}", "us": t, "tbs": tb, "frac_of_measured": tb / peaks["hbm_tbs"]})
    xs = x[:B].contiguous()
    t = timeit(lambda: F.rmsnorm_fwd(xs, w, 1e-6, False, r[:B].contiguous()))
    rows.append({"kernel": "rmsnorm+residual", "case": f"{B}x{h} (decode)", "us": t})
    for row in rows:
        extra = f"{row['tbs']:.2f} TB/s" if "tbs" in row else (f"{row['tflops']:.0f} TFLOP/s" if "tflops" in row else "")
        frac = f"  {row['frac_of_measured']:.2f} of measured" if "frac_of_measured" in row else ""
        if "library_us" in row:
            frac += f"  (torch.matmul {row['library_us']:.1f} us)"
        print(f"{row['kernel']:18s} {row['case']:36s} {row['us']:9.1f} us  {extra}{frac}")
    assert _native.read_status() == 0
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"peaks": peaks, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
