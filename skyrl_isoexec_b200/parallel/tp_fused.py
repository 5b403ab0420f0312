"""Host side of the fused tensor-parallel GEMMs (csrc/tp_gemm_fused.cu): symmetric-memory buffers,
epochs, tile-width choice and the five entry points.

  * ``leaftree_gemm_fused(x, w, leaves)``           single rank: G-leaf tree GEMM in one launch;
  * ``FusedTP.row_parallel(x, w, leaves, ...)``     GEMM -> all-reduce (one-shot for decode-sized M,
                                                    two-shot otherwise) or GEMM -> reduce-scatter;
  * ``FusedTP.allgather_linear(x_local, w)``        all-gather -> GEMM for a sequence-parallel input.

Every rank of the group calls the same methods in the same order; each call advances a shared epoch
and flips the staging half.

CUDA graphs: a recorded kernel argument would repeat the same epoch at every replay, so while a graph is being
captured (``begin_capture`` .. ``end_capture``) the decode-sized GEMM -> all-reduce is recorded in a form that reads
its epoch from a device word: epoch = word + position of the call in the graph. ``before_replay(n)`` sets the word to
the epoch reached so far (a one-thread kernel on the stream, outside the graph) and accounts for the n calls of the
replay, so eager calls and replays can be mixed freely and every rank stays on the same count.

Why a buffer half is free again two calls later: a rank finishes call e+1 only after it has waited
for data that EVERY peer produced in call e+1, and a peer launches e+1 after its own kernel e (and the
copy-out that follows it on the same stream) has completed; so when a rank starts call e+2 and writes
into the halves of parity e, no peer still reads them.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _native

TP_LOCAL, TP_AR1, TP_AR2, TP_RS, TP_AG = 0, 1, 2, 3, 4
_SMS = 148


def _sig(lib):
    if getattr(lib, "_tp_sig", False):
        return
    lib.ix_tp_gemm_fused.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 6 + [C.c_int] * 6 + [C.c_uint] + \
        [C.c_void_p] * 4 + [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.ix_tp_stage_floats.argtypes = [C.c_int] * 5
    lib.ix_tp_stage_floats.restype = C.c_longlong
    lib.ix_tp_gemm_ar1_graph.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int] * 6 + [C.c_int] * 5 + \
        [C.c_void_p, C.c_uint, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_void_p]
    lib.ix_tp_set_epoch.argtypes = [C.c_void_p, C.c_uint, C.c_void_p]
    lib.ix_leaftree_gemm_add.argtypes = [C.c_void_p] * 3 + [C.c_int] * 9 + [C.c_void_p, C.c_int, C.c_void_p]
    lib.ix_leaf_split_bn.argtypes = [C.c_int] * 4
    lib.ix_leaf_split_gemm.argtypes = [C.c_void_p] * 3 + [C.c_int] * 9 + [C.c_void_p]
    lib._tp_sig = True


def pick_bn(M: int, N: int, leaves: int, peers: bool = False) -> int:
    """Widest tile that still gives most SMs a tile. Single rank: the ``leaves`` accumulators may fill all 512 TMEM
    columns (a tcgen05.mma of 128 columns costs what one of 32 does, so width beats keeping a second accumulator set for
    epilogue overlap: 843 us against 1640 us at 4 leaves, 8192 x 4096 x 12288). With peers the epilogue also pushes the
    tile over NVLink, the overlap matters as much as the width (measured equal at 2 ranks), and the rule stays at two
    accumulator sets (2 * leaves * bn <= 512)."""
    bn = min(256, (256 if peers else 512) // leaves)
    tiles_m = (M + 127) // 128
    while bn > 32 and (N % bn or tiles_m * (N // bn) * 5 < _SMS * 3):
        bn //= 2
    if N % bn:
        raise ValueError(f"N={N} is not a multiple of the narrowest tile (32)")
    return bn


def fused_ok(M: int, N: int, K: int, leaves: int) -> bool:
    return leaves in (1, 2, 4, 8) and K % (64 * leaves) == 0 and N % 32 == 0 and M > 0


def leaftree_gemm_fused(x: torch.Tensor, w: torch.Tensor, leaves: int, out_f32: bool = True, bn: int | None = None,
                        split: bool | None = None) -> torch.Tensor:
    """[M,N] = balanced fp32 tree over ``leaves`` equal K slices of x @ w^T, one kernel, no peers. Decode-sized M runs
    the leaf-parallel form (one CTA per leaf, folded through a cluster's shared memory; csrc/leaf_split_gemm.cu), larger
    M the form that keeps every leaf's accumulator in one CTA's TMEM; both give the same bits. ``bn`` / ``split``
    override the choice (benchmarks and tests)."""
    lib = _native.lib()
    _sig(lib)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    out = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    if split is None:
        split = bn is None and N % 4 == 0 and lib.ix_leaf_split_bn(M, N, K, leaves) > 0
    if split:
        _native.check(lib.ix_leaf_split_gemm(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                                             leaves, bn or 0, int(out_f32), _native.stream()), "ix_leaf_split_gemm")
        return out
    if leaves == 8 and bn is None and M > 256 and N % 128 == 0 and K % 512 == 0:
        # training sizes: 8 accumulators in one CTA's TMEM leave 64 columns each. The two halves of the tree as two
        # launches of 4 leaves keep 128-wide tiles; the second adds the first's fp32 result before its store, which is
        # the root of the same balanced tree
        half = K // 2
        esz = x.element_size()
        low = torch.empty(M, N, dtype=torch.float32, device=x.device)
        _native.check(lib.ix_tp_gemm_fused(x.data_ptr(), w.data_ptr(), low.data_ptr(), M, N, half, x.stride(0), w.stride(0), N,
                                           TP_LOCAL, 4, 128, 1, 0, 1, 0, None, None, None, None, None, None, 0, 0,
                                           _native.stream()), "ix_tp_gemm_fused")
        _native.check(lib.ix_leaftree_gemm_add(x.data_ptr() + half * esz, w.data_ptr() + half * esz, out.data_ptr(), M, N, half,
                                               x.stride(0), w.stride(0), N, 4, 128, int(out_f32), low.data_ptr(), N,
                                               _native.stream()), "ix_leaftree_gemm_add")
        return out
    bn = bn or pick_bn(M, N, leaves)
    _native.check(lib.ix_tp_gemm_fused(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                                       TP_LOCAL, leaves, bn, int(out_f32), 0, 1, 0, None, None, None, None, None, None, 0, 0,
                                       _native.stream()), "ix_tp_gemm_fused")
    return out


class FusedTP:
    def __init__(self, group, stage_bytes: int = 160 << 20, out_bytes: int = 80 << 20, gather_bytes: int = 80 << 20, device=None):
        import torch.distributed._symmetric_memory as sm

        self.group = group
        self.rank = dist.get_rank(group)
        self.W = dist.get_world_size(group)
        assert self.W & (self.W - 1) == 0 and self.W <= 8, "fused TP kernels support 1, 2, 4 or 8 ranks"
        self.device = torch.device(device or f"cuda:{torch.cuda.current_device()}")
        self.stage_floats = stage_bytes // 4
        self.out_elems = out_bytes // 2           # bf16 elements per half
        self.gather_elems = gather_bytes // 2
        self.n_flags = 1 << 16
        name = group.group_name if group is not None else dist.group.WORLD.group_name
        self.stage = sm.empty(2 * self.stage_floats, dtype=torch.float32, device=self.device)
        self.outring = sm.empty(2 * self.out_elems, dtype=torch.bfloat16, device=self.device)
        self.gather = sm.empty(2 * self.gather_elems, dtype=torch.bfloat16, device=self.device)
        self.flags = sm.empty(2 * self.n_flags + 64, dtype=torch.int32, device=self.device)   # [2 halves of tile flags | done flags]
        self.flags.zero_()
        self.ctr = torch.zeros(4, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize()
        hs = [sm.rendezvous(t, group=name) for t in (self.stage, self.outring, self.gather, self.flags)]
        dist.barrier(group=group)
        self.p_stage, self.p_out, self.p_gather, self.p_flags = ([int(p) for p in h.buffer_ptrs] for h in hs)
        self._handles = hs
        self.calls = 0
        self.epoch = 0
        self.lib = _native.lib()
        _sig(self.lib)
        self.epoch_word = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._cap = None            # while a CUDA graph is being captured: {"n": calls recorded so far}
        self._base_stage = (C.c_longlong * self.W)(*self.p_stage)
        self._base_flags = (C.c_longlong * self.W)(*self.p_flags)

    # ------------------------------------------------------------------ CUDA-graph capture
    def begin_capture(self) -> None:
        self._cap = {"n": 0}

    def end_capture(self) -> int:
        """Number of fused calls the captured graph contains."""
        n, self._cap = self._cap["n"], None
        return n

    def before_replay(self, n_calls: int) -> None:
        """Call on the replay's stream right before ``graph.replay()``."""
        if n_calls <= 0:
            return
        _native.check(self.lib.ix_tp_set_epoch(self.epoch_word.data_ptr(), self.epoch, _native.stream()), "ix_tp_set_epoch")
        self.epoch += n_calls
        self.calls += n_calls

    def _arr(self, ptrs, off_bytes):
        return (C.c_longlong * self.W)(*[p + off_bytes for p in ptrs])

    def _next(self):
        parity = self.calls & 1
        self.calls += 1
        self.epoch += 1
        return parity

    def check(self) -> None:
        st = _native.read_status()
        if st != 0:
            raise RuntimeError(f"a fused tensor-parallel kernel gave up on a wait (kernel status {st}): a rank of the group did not arrive")

    # ------------------------------------------------------------------ GEMM -> all-reduce / reduce-scatter
    def row_parallel(self, x: torch.Tensor, w: torch.Tensor, leaves: int = 1, mode: str = "auto",
                     out_dtype=torch.bfloat16) -> torch.Tensor:
        """x [M, K/W], w [N, K/W] (this rank's K slice). Returns the tree-ordered sum over ranks:
        ``allreduce``/``auto`` -> [M, N] on every rank; ``reduce_scatter`` -> this rank's [M/W, N] row block."""
        M, K = x.shape
        N = w.shape[0]
        W = self.W
        if mode == "auto":
            mode = "allreduce"
        code = TP_RS if mode == "reduce_scatter" else (TP_AR1 if M <= 256 else TP_AR2)
        bn = pick_bn(M, N, leaves, peers=True)
        need = int(self.lib.ix_tp_stage_floats(M, N, code, W, bn))
        tiles = ((M + 127) // 128) * (N // bn)
        if need > self.stage_floats or tiles * W > self.n_flags:
            raise ValueError(f"row_parallel {M}x{N}: needs {need * 4} B of staging (have {self.stage_floats * 4})")
        out_f32 = out_dtype == torch.float32
        if self._cap is not None:
            if code != TP_AR1:
                raise ValueError(f"a CUDA graph can record the decode-sized GEMM -> all-reduce only (M <= 256); got M={M}, mode={mode}")
            self._cap["n"] += 1
            ret = torch.empty(M, N, dtype=out_dtype, device=x.device)
            _native.check(self.lib.ix_tp_gemm_ar1_graph(x.data_ptr(), w.data_ptr(), ret.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                                                        leaves, bn, int(out_f32), self.rank, W, self.epoch_word.data_ptr(), self._cap["n"],
                                                        self._base_stage, self._base_flags, self.stage_floats, self.n_flags,
                                                        _native.stream()), "ix_tp_gemm_ar1_graph")
            return ret
        parity = self._next()
        esz = 4 if out_f32 else 2
        stage = self._arr(self.p_stage, parity * self.stage_floats * 4)
        flags = self._arr(self.p_flags, parity * self.n_flags * 4)
        done = self._arr(self.p_flags, (2 * self.n_flags + parity * 16) * 4)
        peer_out, out_local, ret = None, None, None
        if code == TP_AR2:
            if M * N * esz > self.out_elems * 2:
                raise ValueError(f"row_parallel {M}x{N}: output exceeds the symmetric output ring")
            peer_out = self._arr(self.p_out, parity * self.out_elems * 2)
            ring = self.outring[parity * self.out_elems:(parity + 1) * self.out_elems]
            view = (ring.view(torch.float32) if out_f32 else ring)[:M * N].view(M, N)
        elif code == TP_RS:
            ret = torch.empty(M // W, N, dtype=out_dtype, device=x.device)
            out_local = ret.data_ptr()
        else:
            ret = torch.empty(M, N, dtype=out_dtype, device=x.device)
            out_local = ret.data_ptr()
        _native.check(self.lib.ix_tp_gemm_fused(x.data_ptr(), w.data_ptr(), out_local, M, N, K, x.stride(0), w.stride(0), N,
                                                code, leaves, bn, int(out_f32), self.rank, W, self.epoch, stage, flags, peer_out, done,
                                                self.ctr.data_ptr(), None, 0, 0, _native.stream()), "ix_tp_gemm_fused")
        if code == TP_AR2:
            ret = view.clone()       # the ring half is rewritten two calls from now
        return ret

    # ------------------------------------------------------------------ all-gather -> GEMM
    def allgather_linear(self, x_local: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        """x_local [M/W, K] (this rank's rows), w [N_local, K]. Returns [M, N_local] = all_gather(x) @ w^T."""
        Ml, K = x_local.shape
        N = w.shape[0]
        W = self.W
        M = Ml * W
        if M * K > self.gather_elems:
            raise ValueError(f"allgather_linear: gathered input {M}x{K} exceeds the symmetric gather buffer")
        bn = pick_bn(M, N, 1)
        parity = self._next()
        flags = self._arr(self.p_flags, parity * self.n_flags * 4)
        gat = self._arr(self.p_gather, parity * self.gather_elems * 2)
        a_gathered = self.p_gather[self.rank] + parity * self.gather_elems * 2
        out = torch.empty(M, N, dtype=out_dtype, device=x_local.device)
        _native.check(self.lib.ix_tp_gemm_fused(a_gathered, w.data_ptr(), out.data_ptr(), M, N, K, K, w.stride(0), N, TP_AG, 1, bn,
                                                int(out_dtype == torch.float32), self.rank, W, self.epoch, None, flags, gat, None,
                                                None, x_local.data_ptr(), x_local.stride(0), Ml, _native.stream()), "ix_tp_gemm_fused")
        return out


_registry: dict = {}


def register(group, rt: FusedTP) -> None:
    _registry[group] = rt


def get(group):
    return _registry.get(group)
