// Tensor-parallel GEMMs fused with their collective over NVLink peer memory, one kernel per rank
// (the reference runs a leaf GEMM and a separate NCCL/Triton all-reduce: ISO/ops/collectives/pik/
// allreduce.py:1018-1168 and layers.py:180-240).
//
//   C = A[M,K] * B[N,K]^T with K sharded over W ranks (row-parallel) or M sharded (sequence-parallel input).
//
// Modes
//   LOCAL  W = 1: the K range is cut into L equal leaves, each accumulated in its own TMEM accumulator and
//          folded by a balanced fp32 tree in the epilogue. This is the single-rank member of the family:
//          TP = W with L = G / W leaves per rank gives the same bits as LOCAL with L = G.
//   AR1    one-shot all-reduce (decode-sized M): every rank pushes its folded partial tile to EVERY rank's
//          staging slot; every rank's reducer warps fold all tiles over ranks in the same tree order.
//   AR2    two-shot all-reduce: tile t is owned by rank t % W; partials are pushed to the owner only, the
//          owner folds and pushes the bf16 result tile to every rank's output.
//   RS     reduce-scatter (sequence-parallel output): rank o owns the o-th block of rows; as AR2 without the
//          second push.
//   AG     all-gather -> GEMM (sequence-parallel input of a column-parallel linear): copier warps push this
//          rank's rows of A into every rank's gathered buffer, 128-row block by block, each with a flag; the
//          TMA producer waits for a block's flag before it loads that block's tiles, own rows first.
//
// Per CTA (persistent, one per SM, 320 threads):
//   warp 0      TMA producer        warp 1      tcgen05.mma issuer
//   warps 2..5  epilogue: tcgen05.ld, leaf fold, store/push of the partial tile + release flag
//   warps 6..9  reducer (AR1/AR2/RS): wait for a tile's W flags, fold over ranks, write/push the result
//               copier  (AG): push local rows to the peers' gathered buffers
// Remote traffic is plain st.global / ld.global on peer-mapped memory; TMA only ever reads this GPU's memory
// Flags are st.release.sys / ld.acquire.sys epochs; every wait is bounded.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 320;
constexpr int kMaxRanks = 16;
constexpr int kMaxStages = 16;
constexpr int kCopySplit = 4;   // AG: a 128-row block travels as four 32-row pieces, each with its own flag
constexpr int kSmemLimit = 227 * 1024 - 64;     // dynamic shared memory a CTA may ask for, minus this kernel's static bytes
constexpr int kFixedBytes = 1024 /*align*/ + 512 /*barriers*/;
constexpr int kTbufFloatsPerWarp = 32 * 36;   // epilogue transpose buffer: 32 rows x (32 + 4 pad) floats per warp

enum Mode { TP_LOCAL = 0, TP_AR1 = 1, TP_AR2 = 2, TP_RS = 3, TP_AG = 4 };

struct TpParams {
  float* stage[kMaxRanks];      // AR/RS: rank d's partial staging; slot (i*W + src) holds a [128][BN] fp32 tile
  uint32_t* flags[kMaxRanks];   // rank d's flags: AR/RS [slot]; AG [src*nb + block]
  void* peer_out[kMaxRanks];    // AR2: rank d's output (bf16/fp32 [M, ldc]); AG: rank d's gathered A (bf16 [W*Ml, K])
  uint32_t* done[kMaxRanks];    // AR2: rank d's completion flags [W]
  unsigned int* local_ctr;      // AR2: CTA arrival counter in local memory
  const void* a_local;          // AG: this rank's rows of A (bf16 [Ml, lda_local])
  int lda_local, m_local;       // AG
  int rank, W, mode, out_f32;
  uint32_t epoch;               // the call's epoch; with epoch_word set, an OFFSET added to the value of that word
  // A call recorded in a CUDA graph cannot carry its epoch as an argument (a replay would repeat it). Such a call
  // passes the address of a device word that the host sets before every replay, the call's position in the graph as
  // `epoch`, BASE addresses of the double-buffered staging and flag arrays, and the sizes of one half; the kernel
  // derives the epoch and the half from the word. One-shot all-reduce (AR1) only.
  const uint32_t* epoch_word;
  long long stage_half;         // floats per staging half
  long long flags_half;         // flags per half
  // LOCAL: an fp32 [M, ld_add] tensor added to the folded tile before the store (the lower half of a leaf tree that was
  // computed by an earlier launch: out = lower + fold(this launch's leaves), the root of the same balanced tree)
  const float* addend;
  int ld_add;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ void named_bar(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// Bounded wait until *p has reached `epoch`. False if it gave up (abort flag and status are then set).
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t epoch, volatile int* abort_flag, int* status) {
  if (static_cast<int>(ld_acquire_sys(p) - epoch) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t it = 0;
  while (static_cast<int>(ld_acquire_sys(p) - epoch) < 0) {
    if (((++it) & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, ST_TIMEOUT_FLAG);
        return false;
      }
    }
  }
  return true;
}

struct TileMap {
  int tiles_m, tiles_n, T, W, rank, mode, rows_per, nb;
  __device__ int num_q() const {
    if (mode == TP_AR2) return ((T + W - 1) / W) * W;
    return T;
  }
  // q-th tile in this rank's compute order -> (m_blk, n_blk, owner, slot at the owner). False: q names no tile.
  __device__ bool decode(int q, int& m_blk, int& n_blk, int& owner, int& slot) const {
    if (mode == TP_AR2) {
      const int i = q / W, o = (rank + 1 + q % W) % W;
      const int t = i * W + o;
      if (t >= T) return false;
      m_blk = t % tiles_m, n_blk = t / tiles_m, owner = o, slot = i;
      return true;
    }
    if (mode == TP_RS) {
      const int i = q / W, o = (rank + 1 + q % W) % W;
      m_blk = o * rows_per + i % rows_per, n_blk = i / rows_per, owner = o, slot = i;
      return true;
    }
    if (mode == TP_AG) {
      const int per = nb * tiles_n;
      const int src = (rank + q / per) % W, rem = q % per;
      m_blk = src * nb + rem % nb, n_blk = rem / nb, owner = src, slot = rem % nb;
      return true;
    }
    m_blk = q % tiles_m, n_blk = q / tiles_m, owner = -1, slot = q;   // LOCAL, AR1
    return true;
  }
  // i-th tile this rank reduces -> (m_blk, n_blk). False past the end.
  __device__ bool owned(int i, int& m_blk, int& n_blk) const {
    if (mode == TP_AR2) {
      const int t = i * W + rank;
      if (t >= T) return false;
      m_blk = t % tiles_m, n_blk = t / tiles_m;
      return true;
    }
    if (mode == TP_RS) {
      if (i >= rows_per * tiles_n) return false;
      m_blk = rank * rows_per + i % rows_per, n_blk = i / rows_per;
      return true;
    }
    if (i >= T) return false;
    m_blk = i % tiles_m, n_blk = i / tiles_m;
    return true;
  }
};

template <int W>
__device__ __forceinline__ void fold_ranks(float4 (&v)[W]) {
#pragma unroll
  for (int stride = 1; stride < W; stride <<= 1)
#pragma unroll
    for (int i = 0; i < W; i += 2 * stride) {
      v[i].x = __fadd_rn(v[i].x, v[i + stride].x);
      v[i].y = __fadd_rn(v[i].y, v[i + stride].y);
      v[i].z = __fadd_rn(v[i].z, v[i + stride].z);
      v[i].w = __fadd_rn(v[i].w, v[i + stride].w);
    }
}


// 32 lanes x CW columns of one accumulator
template <int CW>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[CW]);
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) {
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait_dep(r);
}
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) {
  // load and wait in one statement: the results cannot be read before the wait
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Balanced fp32 tree over NL leaf accumulators that sit `leaf_stride` TMEM columns apart, lower leaf on the left:
// ((l0 + l1) + (l2 + l3)) + ((l4 + l5) + (l6 + l7)).
template <int NL, int CW>
__device__ __forceinline__ void fold_leaves(uint32_t taddr, int leaf_stride, float (&out)[CW]) {
  if constexpr (NL == 1) {
    uint32_t r[CW];
    tmem_ld_cols<CW>(taddr, r);
#pragma unroll
    for (int e = 0; e < CW; ++e) out[e] = __uint_as_float(r[e]);
  } else {
    float hi[CW];
    fold_leaves<NL / 2, CW>(taddr, leaf_stride, out);
    fold_leaves<NL / 2, CW>(taddr + (NL / 2) * leaf_stride, leaf_stride, hi);
#pragma unroll
    for (int e = 0; e < CW; ++e) out[e] = __fadd_rn(out[e], hi[e]);
  }
}

// Reducer body for one tile, W ranks: out = tree over ranks of the W staged partials.
template <int BN, int W>
__device__ __forceinline__ void reduce_tile(const TpParams& p, size_t st_off, int slot, int m_blk, int n_blk, int M, int ldc,
                                            void* c_local, int tid) {
  const float* base = p.stage[p.rank] + st_off + static_cast<size_t>(slot) * W * (BM * BN);
  constexpr int kVecPerRow = BN / 4;
  const int row_base = (p.mode == TP_RS) ? (m_blk - p.rank * ((M + BM - 1) / BM / W)) * BM : m_blk * BM;
  const int rows_valid = min(BM, M - m_blk * BM);
#pragma unroll 2
  for (int idx = tid; idx < rows_valid * kVecPerRow; idx += 128) {
    const int r = idx / kVecPerRow, c4 = idx % kVecPerRow;
    float4 v[W];
#pragma unroll
    for (int s = 0; s < W; ++s) v[s] = __ldcs(reinterpret_cast<const float4*>(base + static_cast<size_t>(s) * (BM * BN)) + idx);
    fold_ranks<W>(v);
    const size_t off = static_cast<size_t>(row_base + r) * ldc + n_blk * BN + c4 * 4;
    if (p.mode == TP_AR2) {
#pragma unroll 1
      for (int d = 0; d < W; ++d) {
        if (p.out_f32) {
          *reinterpret_cast<float4*>(static_cast<float*>(p.peer_out[d]) + off) = v[0];
        } else {
          uint2 w;
          w.x = pack_bf2(v[0].x, v[0].y);
          w.y = pack_bf2(v[0].z, v[0].w);
          *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.peer_out[d]) + off) = w;
        }
      }
    } else if (p.out_f32) {
      *reinterpret_cast<float4*>(static_cast<float*>(c_local) + off) = v[0];
    } else {
      uint2 w;
      w.x = pack_bf2(v[0].x, v[0].y);
      w.y = pack_bf2(v[0].z, v[0].w);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(c_local) + off) = w;
    }
  }
}

template <int BN, int L>
__global__ void __launch_bounds__(kThreads, 1)
tp_gemm_fused_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                     const __grid_constant__ CUtensorMap tmB, const __grid_constant__ TpParams p, void* __restrict__ c_local, int M, int N, int K, int ldc, int a_rows,
                     int S, int* __restrict__ status) {
  constexpr int kAccCols = L * BN;
  constexpr int kNumAcc = (2 * kAccCols <= 512) ? 2 : 1;
  constexpr int kTmemCols = (kNumAcc * kAccCols < 32) ? 32 : kNumAcc * kAccCols;
  static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns must be a power of two <= 512");
  const int stage_bytes_a = a_rows * BK * 2;
  const int stage_bytes = stage_bytes_a + BN * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [S stages][tail: what the last stage's MMA may read beyond a short A box][barriers 512 B][epilogue transpose buffers]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * stage_bytes + (BM - a_rows) * BK * 2);
  // bars: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty, [2S+4] tile stored
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* tbuf_all = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 512);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  TileMap tm;
  tm.tiles_m = (M + BM - 1) / BM;
  tm.tiles_n = N / BN;
  tm.T = tm.tiles_m * tm.tiles_n;
  tm.W = p.W, tm.rank = p.rank, tm.mode = p.mode;
  tm.rows_per = tm.tiles_m / p.W;
  tm.nb = p.m_local / BM;
  const int num_q = tm.num_q();
  // epoch and staging half of this call (see TpParams::epoch_word); the half of call e is (e - 1) & 1 in both forms
  const uint32_t epoch = p.epoch_word ? (*p.epoch_word + p.epoch) : p.epoch;
  const size_t st_off = p.epoch_word ? static_cast<size_t>((epoch - 1u) & 1u) * static_cast<size_t>(p.stage_half) : 0;
  const size_t fl_off = p.epoch_word ? static_cast<size_t>((epoch - 1u) & 1u) * static_cast<size_t>(p.flags_half) : 0;
  const int num_kb = K / BK;
  const int kb_per_leaf = num_kb / L;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[S + i]), 1);
    }
    mbar_init(smem_u32(&bars[2 * S + 0]), 1);
    mbar_init(smem_u32(&bars[2 * S + 1]), 1);
    mbar_init(smem_u32(&bars[2 * S + 2]), 4);
    mbar_init(smem_u32(&bars[2 * S + 3]), 4);
    mbar_init(smem_u32(&bars[2 * S + 4]), 4);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<kTmemCols>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int q = blockIdx.x; q < num_q && ok; q += gridDim.x) {
        int m_blk, n_blk, owner, slot;
        if (!tm.decode(q, m_blk, n_blk, owner, slot)) continue;
        const bool local_rows = p.mode == TP_AG && owner == p.rank;   // AG: own rows come straight from a_local (tmA2)
        if (p.mode == TP_AG && !local_rows) {
          // rows of this block were pushed by rank `owner`'s copier warps (generic proxy, remote) in kCopySplit pieces
          bool arrived = true;
          for (int sub = 0; sub < kCopySplit && arrived; ++sub)
            arrived = wait_flag(p.flags[p.rank] + fl_off + (owner * tm.nb + slot) * kCopySplit + sub, epoch, abort_flag, status);
          if (!arrived) break;
          fence_proxy_async_global();
        }
        const CUtensorMap* ta = local_rows ? &tmA2 : &tmA;
        const int a_row = local_rows ? slot * BM : m_blk * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[S + stage]), phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars[stage]);
          mbar_arrive_expect_tx(full, stage_bytes);
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          tma_load_2d(sa, ta, full, kb * BK, a_row);
          tma_load_2d(sa + stage_bytes_a, &tmB, full, kb * BK, n_blk * BN);
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: leaf j accumulates in columns [j*BN, (j+1)*BN)
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int q = blockIdx.x; q < num_q && ok; q += gridDim.x) {
        int m_blk, n_blk, owner, slot;
        if (!tm.decode(q, m_blk, n_blk, owner, slot)) continue;
        if (!mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[stage]), phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int leaf = kb / kb_per_leaf;
          const uint32_t d_tmem = tmem_base + acc * kAccCols + leaf * BN;
          const uint32_t first = (kb - leaf * kb_per_leaf) == 0 ? 0u : 1u;
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint64_t da = make_sw128_desc(sa, 16, 1024);
          const uint64_t db = make_sw128_desc(sa + stage_bytes_a, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_f16_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, (first | k) != 0 ? 1u : 0u);
          umma_commit(smem_u32(&bars[S + stage]));
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bars[2 * S + acc]));
        if (kNumAcc == 2) {
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1;
        } else {
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5): fold leaves, store / push
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0, tile_phase = 0;
    for (int q = blockIdx.x; q < num_q; q += gridDim.x) {
      int m_blk, n_blk, owner, slot;
      if (!tm.decode(q, m_blk, n_blk, owner, slot)) continue;
      if (!mbar_wait(smem_u32(&bars[2 * S + acc]), acc_phase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row_in = quad * 32 + lane;
      const int row = m_blk * BM + row_in;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kAccCols;
      constexpr int CW = (L >= 8) ? 16 : 32;   // chunk width: keeps the fold's live registers bounded
#pragma unroll 1
      for (int c = 0; c < BN / CW; ++c) {
        float f[CW];
        fold_leaves<L, CW>(taddr + c * CW, BN, f);
        const int col0 = n_blk * BN + c * CW;
        if (p.mode == TP_LOCAL || p.mode == TP_AG) {
          if (row < M) {
            if (p.addend != nullptr) {
              const float4* ad = reinterpret_cast<const float4*>(p.addend + static_cast<size_t>(row) * p.ld_add + col0);
#pragma unroll
              for (int j = 0; j < CW / 4; ++j) {
                const float4 a = __ldcs(ad + j);
                f[4 * j] = __fadd_rn(a.x, f[4 * j]);
                f[4 * j + 1] = __fadd_rn(a.y, f[4 * j + 1]);
                f[4 * j + 2] = __fadd_rn(a.z, f[4 * j + 2]);
                f[4 * j + 3] = __fadd_rn(a.w, f[4 * j + 3]);
              }
            }
            if (p.out_f32) {
              float* dst = static_cast<float*>(c_local) + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
              for (int j = 0; j < CW / 4; ++j) reinterpret_cast<float4*>(dst)[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
            } else {
              __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(c_local) + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
              for (int j = 0; j < CW / 8; ++j) {
                uint4 v;
                v.x = pack_bf2(f[8 * j + 0], f[8 * j + 1]);
                v.y = pack_bf2(f[8 * j + 2], f[8 * j + 3]);
                v.z = pack_bf2(f[8 * j + 4], f[8 * j + 5]);
                v.w = pack_bf2(f[8 * j + 6], f[8 * j + 7]);
                reinterpret_cast<uint4*>(dst)[j] = v;
              }
            }
          }
        } else {
          // partial tile -> staging slot (slot*W + rank) at the owner (AR2/RS) or at every rank (AR1). A lane holds CW
          // columns of ONE row; through a per-warp shared-memory transpose the warp instead stores whole row segments
          // (CW*4 contiguous bytes each), which is what NVLink and DRAM want.
          constexpr int kUnits = CW / 4;            // float4 per row segment
          constexpr int kRowsPerIt = 32 / kUnits;
          float* tb = tbuf_all + (warp - 2) * kTbufFloatsPerWarp;
          __syncwarp();
#pragma unroll
          for (int j = 0; j < kUnits; ++j)
            *reinterpret_cast<float4*>(tb + lane * 36 + 4 * j) = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
          __syncwarp();
          const size_t tile_off = (static_cast<size_t>(slot) * p.W + p.rank) * (BM * BN) + c * CW;
          const int d0 = (p.mode == TP_AR1) ? 0 : owner, d1 = (p.mode == TP_AR1) ? p.W : owner + 1;
          const int u = lane % kUnits, rs = lane / kUnits;
#pragma unroll
          for (int it = 0; it < kUnits; ++it) {
            const int r = it * kRowsPerIt + rs;     // row within this warp's 32
            const float4 v = *reinterpret_cast<const float4*>(tb + r * 36 + 4 * u);
            if (m_blk * BM + quad * 32 + r < M) {
              const size_t off = tile_off + static_cast<size_t>(quad * 32 + r) * BN + 4 * u;
#pragma unroll 1
              for (int d = d0; d < d1; ++d) __stcs(reinterpret_cast<float4*>(p.stage[d] + st_off + off), v);   // streaming: keep A/B tiles in L2
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[2 * S + 2 + acc]));
      if (p.mode == TP_AR1 || p.mode == TP_AR2 || p.mode == TP_RS) {
        // "all four epilogue warps have stored their rows of this tile": an mbarrier rather than bar.sync, so that a
        // warp that gave up on a wait can never leave the others parked at a barrier without a limit
        const uint32_t tile_bar = smem_u32(&bars[2 * S + 4]);
        if (lane == 0) mbar_arrive(tile_bar);
        if (warp == 2) {
          const bool stored = mbar_wait(tile_bar, tile_phase, abort_flag, status, ST_TIMEOUT_MISC);
          const int d0 = (p.mode == TP_AR1) ? 0 : owner, d1 = (p.mode == TP_AR1) ? p.W : owner + 1;
          if (stored && lane < d1 - d0) {
            __threadfence_system();
            st_release_sys(p.flags[d0 + lane] + fl_off + slot * p.W + p.rank, epoch);
          }
          if (!stored) break;
        }
        tile_phase ^= 1;
      }
      if (kNumAcc == 2) {
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      } else {
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ warps 6..9: reducer or copier
    const int tid = threadIdx.x - 192;
    if (p.mode == TP_AG) {
      // units of (128-row block, quarter, destination peer); own rows are not copied (the GEMM reads them in place)
      constexpr int kRows = BM / kCopySplit;
      const int units = tm.nb * kCopySplit * (p.W - 1);
      const int vec_per_row = K / 8;
      const int n_vec = kRows * vec_per_row;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int d = (p.rank + 1 + u / (tm.nb * kCopySplit)) % p.W;
        const int b = (u / kCopySplit) % tm.nb, sub = u % kCopySplit;
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.a_local) + (static_cast<size_t>(b) * BM + sub * kRows) * p.lda_local;
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.peer_out[d]) + (static_cast<size_t>(p.rank) * p.m_local + b * BM + sub * kRows) * K;
        for (int base = tid; base < n_vec; base += 128 * 8) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {      // eight loads in flight per thread before the first remote store
            const int idx = base + j * 128;
            if (idx < n_vec) v[j] = reinterpret_cast<const uint4*>(src + static_cast<size_t>(idx / vec_per_row) * p.lda_local)[idx % vec_per_row];
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int idx = base + j * 128;
            if (idx < n_vec) reinterpret_cast<uint4*>(dst + static_cast<size_t>(idx / vec_per_row) * K)[idx % vec_per_row] = v[j];
          }
        }
        named_bar(2, 128);
        if (tid == 0) {
          __threadfence_system();
          st_release_sys(p.flags[d] + fl_off + (p.rank * tm.nb + b) * kCopySplit + sub, epoch);
        }
      }
    } else if (p.mode != TP_LOCAL) {
      __shared__ int s_ok;
      for (int i = blockIdx.x;; i += gridDim.x) {
        int m_blk, n_blk;
        if (!tm.owned(i, m_blk, n_blk)) break;
        if (tid == 0) s_ok = 1;
        named_bar(2, 128);
        if (tid < p.W && !wait_flag(p.flags[p.rank] + fl_off + i * p.W + tid, epoch, abort_flag, status)) s_ok = 0;
        named_bar(2, 128);
        if (!s_ok) break;
        switch (p.W) {
          case 1: reduce_tile<BN, 1>(p, st_off, i, m_blk, n_blk, M, ldc, c_local, tid); break;
          case 2: reduce_tile<BN, 2>(p, st_off, i, m_blk, n_blk, M, ldc, c_local, tid); break;
          case 4: reduce_tile<BN, 4>(p, st_off, i, m_blk, n_blk, M, ldc, c_local, tid); break;
          case 8: reduce_tile<BN, 8>(p, st_off, i, m_blk, n_blk, M, ldc, c_local, tid); break;
          default: break;
        }
      }
      if (p.mode == TP_AR2) {
        // every CTA's result pushes are out; the last CTA to arrive tells all ranks, CTA 0 waits for all ranks
        named_bar(2, 128);
        if (tid == 0) {
          __threadfence_system();
          const unsigned int arrived = atomicAdd(p.local_ctr, 1u);
          if (arrived + 1 == gridDim.x) {
            *p.local_ctr = 0;
            __threadfence_system();
            for (int d = 0; d < p.W; ++d) st_release_sys(p.done[d] + p.rank, epoch);
          }
        }
        if (blockIdx.x == 0 && tid < p.W) wait_flag(p.done[p.rank] + tid, epoch, abort_flag, status);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

int g_sms[64] = {0};
int sm_count(int dev) {
  if (dev < 0 || dev >= 64) return 148;
  if (g_sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

template <int BN, int L>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmA2, const CUtensorMap& tmB, const TpParams& p, void* c_local, int M, int N, int K, int ldc,
           int a_rows, int num_q, cudaStream_t stream, int dev) {
  const int stage_bytes = a_rows * BK * 2 + BN * BK * 2;
  const int tail = (BM - a_rows) * BK * 2;
  const int tbuf = 4 * kTbufFloatsPerWarp * 4;
  int S = (kSmemLimit - kFixedBytes - tail - tbuf) / stage_bytes;
  if (S > kMaxStages) S = kMaxStages;
  const int kSmem = S * stage_bytes + tail + kFixedBytes + tbuf;
  auto kern = tp_gemm_fused_kernel<BN, L>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    attr_set[dev & 63] = true;
  }
  int grid = sm_count(dev);
  if (num_q < grid) grid = num_q;
  kern<<<grid, kThreads, kSmem, stream>>>(tmA, tmA2, tmB, p, c_local, M, N, K, ldc, a_rows, S, ixh::status_word(dev));
  IX_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

// Bytes of fp32 staging one rank needs for a row-parallel call of the given shape (per parity half).
IX_API long long ix_tp_stage_floats(int M, int N, int mode, int W, int bn) {
  const long long tiles = static_cast<long long>((M + BM - 1) / BM) * (N / bn);
  long long slots = tiles;                                   // AR1: every rank holds all tiles
  if (mode == TP_AR2) slots = (tiles + W - 1) / W;
  if (mode == TP_RS) slots = tiles / W;
  return slots * W * BM * bn;
}

// The fused tensor-parallel GEMM. A: this rank's operand (row-parallel modes: [M, K] with K = this rank's slice;
// AG: ignored, rows come from a_local through the gathered buffers), B: this rank's weight shard [N, K].
// stage/flags/peer_out/done: W device addresses each (as mapped in THIS process), already offset to the call's
// parity half. leaves: L (K / 64 must be divisible by L). bn: 32/64/128/256 with L*bn <= 512
// (two accumulator sets, so that the epilogue of one tile overlaps the MMAs of the next, when 2*L*bn <= 512).
static int tp_gemm_fused_impl(const void* A, const void* B, void* c_local, int M, int N, int K, int lda, int ldb, int ldc,
                            int mode, int leaves, int bn, int out_f32, int rank, int W, unsigned epoch,
                            const long long* stage, const long long* flags, const long long* peer_out, const long long* done,
                            void* local_ctr, const void* a_local, int lda_local, int m_local, void* stream,
                            const void* epoch_word, long long stage_half, long long flags_half, const void* addend = nullptr,
                            int ld_add = 0) {
  if (addend != nullptr && (mode != TP_LOCAL || (ld_add & 3)))
    return ixh::fail(ixh::IX_EARG, "tp_gemm: an addend is taken by the single-rank leaf-tree GEMM only (ld_add a multiple of 4)");
  if (epoch_word != nullptr && mode != TP_AR1)
    return ixh::fail(ixh::IX_EARG, "tp_gemm: a device epoch word (graph capture) is supported by the one-shot all-reduce only");
  if (M <= 0 || N <= 0 || K <= 0) return ixh::fail(ixh::IX_EARG, "tp_gemm: empty problem");
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || leaves < 1 || (K % (BK * leaves)) != 0) return ixh::fail(ixh::IX_EARG, "tp_gemm: K=%d must split into %d leaves of whole 64-blocks", K, leaves);
  if (N % bn) return ixh::fail(ixh::IX_EARG, "tp_gemm: N=%d not a multiple of the tile width %d", N, bn);
  if (W < 1 || W > kMaxRanks || (W & (W - 1))) return ixh::fail(ixh::IX_EARG, "tp_gemm: world size %d must be a power of two <= 16", W);
  if (mode == TP_LOCAL && W != 1) return ixh::fail(ixh::IX_EARG, "tp_gemm: LOCAL mode is single-rank");
  const int tiles_m = (M + BM - 1) / BM;
  if (mode == TP_RS && (M % (BM * W)) != 0) return ixh::fail(ixh::IX_EARG, "tp_gemm: reduce-scatter needs M a multiple of %d", BM * W);
  if (mode == TP_AG && (m_local % BM != 0 || M != m_local * W || (lda_local & 7)))
    return ixh::fail(ixh::IX_EARG, "tp_gemm: all-gather mode needs M = W * m_local with m_local a multiple of 128");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  TpParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < W; ++r) {
    p.stage[r] = stage ? reinterpret_cast<float*>(stage[r]) : nullptr;
    p.flags[r] = flags ? reinterpret_cast<uint32_t*>(flags[r]) : nullptr;
    p.peer_out[r] = peer_out ? reinterpret_cast<void*>(peer_out[r]) : nullptr;
    p.done[r] = done ? reinterpret_cast<uint32_t*>(done[r]) : nullptr;
  }
  p.local_ctr = static_cast<unsigned int*>(local_ctr);
  p.a_local = a_local, p.lda_local = lda_local, p.m_local = m_local > 0 ? m_local : BM;
  p.rank = rank, p.W = W, p.mode = mode, p.out_f32 = out_f32, p.epoch = epoch;
  p.epoch_word = static_cast<const uint32_t*>(epoch_word), p.stage_half = stage_half, p.flags_half = flags_half;
  p.addend = static_cast<const float*>(addend), p.ld_add = ld_add;
  int a_rows = (M + 7) & ~7;
  if (a_rows > BM) a_rows = BM;
  CUtensorMap tmA, tmA2, tmB;
  int rc = ixh::make_tmap_bf16_2d(&tmA, A, M, K, lda, a_rows);
  if (rc) return rc;
  if (mode == TP_AG) rc = ixh::make_tmap_bf16_2d(&tmA2, a_local, m_local, K, lda_local, a_rows);
  else tmA2 = tmA;
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmB, B, N, K, ldb, bn);
  if (rc) return rc;
  const int T = tiles_m * (N / bn);
  const int num_q = (mode == TP_AR2) ? ((T + W - 1) / W) * W : T;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define IX_TP(BN_, L_) \
  if (bn == BN_ && leaves == L_) return launch<BN_, L_>(tmA, tmA2, tmB, p, c_local, M, N, K, ldc, a_rows, num_q, s, dev);
  IX_TP(256, 1) IX_TP(128, 1) IX_TP(128, 2) IX_TP(64, 1) IX_TP(64, 2) IX_TP(64, 4) IX_TP(32, 1) IX_TP(32, 2) IX_TP(32, 4) IX_TP(32, 8)
  IX_TP(256, 2) IX_TP(128, 4) IX_TP(64, 8)   // all 512 columns hold ONE tile's leaves: wider MMAs, no overlap of epilogue and next tile
#undef IX_TP
  return ixh::fail(ixh::IX_EARG, "tp_gemm: no kernel for bn=%d leaves=%d (need leaves*bn <= 512)", bn, leaves);
}

IX_API int ix_tp_gemm_fused(const void* A, const void* B, void* c_local, int M, int N, int K, int lda, int ldb, int ldc,
                            int mode, int leaves, int bn, int out_f32, int rank, int W, unsigned epoch,
                            const long long* stage, const long long* flags, const long long* peer_out, const long long* done,
                            void* local_ctr, const void* a_local, int lda_local, int m_local, void* stream) {
  return tp_gemm_fused_impl(A, B, c_local, M, N, K, lda, ldb, ldc, mode, leaves, bn, out_f32, rank, W, epoch, stage, flags, peer_out,
                            done, local_ctr, a_local, lda_local, m_local, stream, nullptr, 0, 0);
}

// Single-rank leaf-tree GEMM whose folded tile is added to `addend` (fp32 [M, ld_add]) before the store: the upper half
// of a tree whose lower half an earlier launch left in `addend`. Two launches of 4 leaves with 128-wide tiles are the
// 8-leaf tree, bit for bit, at twice the tile width the 8 accumulators of one launch would allow.
IX_API int ix_leaftree_gemm_add(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int leaves,
                                int bn, int out_f32, const void* addend, int ld_add, void* stream) {
  return tp_gemm_fused_impl(A, B, C, M, N, K, lda, ldb, ldc, TP_LOCAL, leaves, bn, out_f32, 0, 1, 0, nullptr, nullptr, nullptr, nullptr,
                            nullptr, nullptr, 0, 0, stream, nullptr, 0, 0, addend, ld_add);
}

// One-shot GEMM -> all-reduce in a form that a CUDA graph can record: the epoch of the call is
// *epoch_word + epoch_offset, read on the device; stage/flags are the BASE addresses of the double-buffered arrays
// (W each) and stage_half / flags_half the element counts of one half. The host sets the word (ix_tp_set_epoch) to the
// epoch of the last call made before the replay and then accounts for the calls the graph contains.
IX_API int ix_tp_gemm_ar1_graph(const void* A, const void* B, void* c_local, int M, int N, int K, int lda, int ldb, int ldc,
                                int leaves, int bn, int out_f32, int rank, int W, const void* epoch_word, unsigned epoch_offset,
                                const long long* stage, const long long* flags, long long stage_half, long long flags_half,
                                void* stream) {
  if (epoch_word == nullptr) return ixh::fail(ixh::IX_EARG, "tp_gemm_ar1_graph: no epoch word");
  return tp_gemm_fused_impl(A, B, c_local, M, N, K, lda, ldb, ldc, TP_AR1, leaves, bn, out_f32, rank, W, epoch_offset, stage, flags,
                            nullptr, nullptr, nullptr, nullptr, 0, 0, stream, epoch_word, stage_half, flags_half);
}

namespace {
__global__ void set_word_kernel(uint32_t* w, uint32_t v) { *w = v; }
}  // namespace

IX_API int ix_tp_set_epoch(void* epoch_word, unsigned value, void* stream) {
  if (epoch_word == nullptr) return ixh::fail(ixh::IX_EARG, "tp_set_epoch: null word");
  set_word_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t*>(epoch_word), value);
  IX_CUDA(cudaGetLastError());
  return 0;
}
