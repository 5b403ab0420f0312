"""Kernel-level comparison arms: this framework's kernels beside the reference's OWN, unmodified kernels on the same
shapes and the same GPU.

    python -m skyrl_isoexec_b200.benchmarks.bench_reference_kernels [--json out.json]

The reference's training entry point cannot run offline (it imports ray, megatron.core, omegaconf), but several of its
kernels are self-contained modules that import with what this image has (torch, triton, vllm):

  rowinv_logprob    skyrl/backends/skyrl_train/isoexec/ops/logprobs/rowinv.py::rowinv_sampled_logprobs   (Triton)
  add_rmsnorm       .../ops/norms/fused_add_rmsnorm.py::fused_add_rms_norm_gamma                          (Triton)
  rope              .../ops/rope/rope_fused.py::fused_rope_bshd                                           (Triton)
  gated_outnorm     .../ops/norms/fused_outnorm.py::fused_gated_out_norm                                  (Triton)
  leaftree_gemm     .../ops/collectives/pik/gemm.py::ti_gemm  (its Triton / cuBLAS leaf schedules, 8 leaves, tp = 1)
  matmul_invariant  vllm.model_executor.layers.batch_invariant::matmul_persistent  (what the reference's engine runs)

They are loaded from the offline install of the reference under ``baseline/_ref`` (nothing of this package is on
their path) and called through their public functions. A kernel that does not import or run prints
``unavailable: <reason>`` and the table goes on. Timing: CUDA events around 12 calls queued back to back, median of 3
such groups after warm-up; inputs exceed L2, and the decode-sized GEMMs cycle over enough weight copies to exceed it. Each row reports both times and ours / theirs (below 1 = this framework is faster).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.path.join(ROOT, "baseline", "_ref")


def _time(fn, copies=1, calls=12, warm=3):
    """Device time per call: ``calls`` launches queued back to back between two events (so the host's launch path is
    hidden, as it is inside a step), ``fn(i)`` with i cycling over ``copies`` operand sets when one set would stay in L2."""
    for i in range(max(warm, copies)):
        fn(i % copies)
    torch.cuda.synchronize()
    ts = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(calls):
            fn(i % copies)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / calls)
    ts.sort()
    return ts[1] * 1e3


def _ref_module(name: str):
    import importlib

    os.environ.setdefault("SKYRL_ISOEXEC", "1")        # the reference's kernels admit inputs only when its master switch is on
    for extra in (REF, os.path.join(REF, "skyrl", "backends", "skyrl_train", "isoexec", "ops", "collectives")):
        if extra not in sys.path:                       # its pik package imports itself as top-level ``pik``
            sys.path.insert(0, extra)
    return importlib.import_module(name)


def _row(rows, kernel, case, ours_fn, theirs_fn, note="", copies=1):
    """ours_fn / theirs_fn take the index of the operand set to use."""
    rec = {"kernel": kernel, "case": case, "note": note}
    try:
        rec["ours_us"] = _time(ours_fn, copies)
    except Exception as e:  # noqa: BLE001
        rec["ours_error"] = f"{type(e).__name__}: {str(e)[:160]}"
    try:
        if theirs_fn is None:
            raise RuntimeError(note or "not importable")
        rec["theirs_us"] = _time(theirs_fn, copies)
    except Exception as e:  # noqa: BLE001
        rec["unavailable"] = f"{type(e).__name__}: {str(e)[:200]}"
    if "ours_us" in rec and "theirs_us" in rec:
        rec["ours_over_theirs"] = rec["ours_us"] / rec["theirs_us"]
    rows.append(rec)
    return rec


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    from ..ops import _native
    from ..ops import functional as F
    from ..parallel import tp_fused

    _native.lib().ix_init()
    dev = "cuda"
    rows: list = []
    P = "skyrl.backends.skyrl_train.isoexec.ops."

    # ---- sampled-token logprob over the full vocabulary
    R, V = 1024, 151936
    logits = (torch.randn(R, V, device=dev) * 2).bfloat16()
    tg = torch.randint(0, V, (R,), device=dev)
    try:
        m = _ref_module(P + "logprobs.rowinv")
        ref = lambda: torch.log_softmax(logits.float(), -1).gather(1, tg[:, None])[:, 0]   # the incumbent its probe compares with

        def theirs(_i):
            out = m.rowinv_sampled_logprobs(logits, tg, vocab_start_index=0, vocab_end_index=V, group=None, src_dtype=torch.bfloat16,
                                            reference=ref)
            if out is None:
                raise RuntimeError("the reference's admission declined this input")
            return out
    except Exception as e:  # noqa: BLE001
        theirs = None
        why = f"{type(e).__name__}: {str(e)[:160]}"
    _row(rows, "rowinv_logprob", f"{R}x{V} bf16", lambda _i: F.logprob_fused_fwd(logits, tg, 8), theirs,
         "" if theirs else why)
    del logits

    # ---- residual add + RMSNorm (zero-centred gamma), widths 2048 (the width the reference admits) and 4096
    for N in (2048, 4096):
        M = 16384
        x, r = torch.randn(M, N, device=dev).bfloat16(), torch.randn(M, N, device=dev).bfloat16()
        w = (torch.randn(N, device=dev) * 0.1).bfloat16()
        try:
            m = _ref_module(P + "norms.fused_add_rmsnorm")
            theirs = lambda _i: m.fused_add_rms_norm_gamma(x, r, w, 1e-6)
        except Exception as e:  # noqa: BLE001
            theirs, why = None, f"{type(e).__name__}: {str(e)[:160]}"
        _row(rows, "add_rmsnorm", f"{M}x{N} bf16", lambda _i: F.rmsnorm_fwd(x, w, 1e-6, True, r), theirs, "" if theirs else why)

    # ---- rotary embedding. Ours also applies the per-head QK RMSNorm and writes K/V to their slots in the same pass.
    S, Hq, Hkv, D = 8192, 32, 8, 128
    qkv = torch.randn(S, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
    pos = torch.arange(S, dtype=torch.int32, device=dev) % 4096
    rope = F.RopeTable(D, 4096, 1e6, torch.device(dev))
    qw, kw = torch.ones(D, device=dev).bfloat16(), torch.ones(D, device=dev).bfloat16()
    kp, vp = torch.empty(S, Hkv, D, device=dev, dtype=torch.bfloat16), torch.empty(S, Hkv, D, device=dev, dtype=torch.bfloat16)
    try:
        m = _ref_module(P + "rope.rope_fused")
        t = torch.randn(S, 1, Hq + Hkv, D, device=dev).bfloat16()          # q and k heads, as the reference rotates them
        ang = torch.randn(S, 1, 1, D, device=dev)
        cos_, sin_ = ang.cos().bfloat16().contiguous(), ang.sin().bfloat16().contiguous()
        theirs = lambda _i: m.fused_rope_bshd(t, cos_, sin_)
    except Exception as e:  # noqa: BLE001
        theirs, why = None, f"{type(e).__name__}: {str(e)[:160]}"
    _row(rows, "rope", f"{S} tokens x ({Hq}+{Hkv}) heads x {D}",
         lambda _i: F.qk_norm_rope_fwd(qkv, pos, None, rope, qw, kw, kp, vp, Hq, Hkv, D, 1e-6), theirs,
         "ours = QK-norm + rotary + K/V write; theirs = rotary only" if theirs else why)

    # ---- GatedDeltaNet output norm: rms_norm(o) * (1 + w) * silu(z)
    T, HV, N = 8192, 32, 128
    o, z = torch.randn(T, HV, N, device=dev).bfloat16(), torch.randn(T, HV, N, device=dev).bfloat16()
    w = (torch.randn(N, device=dev) * 0.1).bfloat16()
    try:
        m = _ref_module(P + "norms.fused_outnorm")
        theirs = lambda _i: m.fused_gated_out_norm(o, z, w, 1e-6)
    except Exception as e:  # noqa: BLE001
        theirs, why = None, f"{type(e).__name__}: {str(e)[:160]}"
    _row(rows, "gated_outnorm", f"{T}x{HV}x{N} bf16", lambda _i: F.gated_outnorm(o, z, w, 1e-6, True), theirs, "" if theirs else why)

    def _copies(nbytes):
        return 1 if nbytes > (256 << 20) else max(2, (600 << 20) // nbytes)

    # ---- TP-invariant leaf-tree GEMM, one rank (down projection of Qwen3-8B), training and decode sizes. The reference's
    # default is 8 leaves; 2 is what a single-GPU deployment of this framework runs.
    for M, G in ((8192, 8), (8192, 2), (64, 8), (64, 2)):
        Nn, K = 4096, 12288
        nc = _copies(Nn * K * 2) if M <= 256 else 1
        x = torch.randn(M, K, device=dev).bfloat16()
        wts = [(torch.randn(Nn, K, device=dev) * 0.02).bfloat16() for _ in range(nc)]
        try:
            m = _ref_module(P + "collectives.pik.gemm")
            plan = m.ReductionPlan(num_leaves=G)
            theirs = lambda i, plan=plan: m.ti_gemm(x, wts[i], plan=plan)
        except Exception as e:  # noqa: BLE001
            theirs, why = None, f"{type(e).__name__}: {str(e)[:160]}"
        _row(rows, "leaftree_gemm", f"M={M} N={Nn} K={K} {G} leaves", lambda i, G=G: tp_fused.leaftree_gemm_fused(x, wts[i], G, out_f32=True),
             theirs, "" if theirs else why, copies=nc)
        del wts

    # ---- batch-invariant matmul of the reference's engine (vLLM), against the tcgen05 GEMM
    for M, Nn, K in ((8192, 4096, 4096), (64, 6144, 4096), (64, 24576, 4096)):
        nc = _copies(Nn * K * 2) if M <= 256 else 1
        x = torch.randn(M, K, device=dev).bfloat16()
        wts = [(torch.randn(Nn, K, device=dev) * 0.02).bfloat16() for _ in range(nc)]
        try:
            import importlib

            bi = importlib.import_module("vllm.model_executor.layers.batch_invariant")
            theirs = lambda i: bi.matmul_persistent(x, wts[i].t())
        except Exception as e:  # noqa: BLE001
            theirs, why = None, f"{type(e).__name__}: {str(e)[:160]}"
        _row(rows, "matmul_invariant", f"M={M} N={Nn} K={K}", lambda i: F.gemm_nt(x, wts[i]), theirs, "" if theirs else why, copies=nc)
        del wts

    for r_ in rows:
        a = f"{r_['ours_us']:10.1f} us" if "ours_us" in r_ else f"ours failed: {r_.get('ours_error')}"
        if "theirs_us" in r_:
            b = f"{r_['theirs_us']:10.1f} us   ours/theirs {r_['ours_over_theirs']:.2f}"
        else:
            b = f"unavailable: {r_['unavailable']}"
        print(f"{r_['kernel']:17s} {r_['case']:38s} ours {a}   reference {b}" + (f"   [{r_['note']}]" if r_.get("note") and "theirs_us" in r_ else ""))
    assert _native.read_status() == 0
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
