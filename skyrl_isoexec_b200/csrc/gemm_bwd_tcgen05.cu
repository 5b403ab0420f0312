// Backward-pass GEMMs for sm_100a. The forward kernel (gemm_tcgen05.cu) computes C = A * B^T with both operands
// K-major. The two gradients of a linear layer need the other operand orders:
//
//   NN   dX[M,K] = dY[M,N] * W[N,K]        A = dY is K-major (reduction over its inner dim N),
//                                          B = W is read "M/N-major": the reduction runs over W's ROWS
//   TN   dW[N,K] (+)= dY[M,N]^T * X[M,K]   both operands M/N-major: the reduction runs over the rows of dY and of X
//
// An M/N-major operand is brought in by TMA as 64-column chunks ([64 reduction rows x 64 columns] boxes, 128-byte
// swizzle); the shared-memory descriptor then names the chunk stride as its leading-dimension byte offset and the
// instruction descriptor marks the operand as M/N-major, so tcgen05.mma transposes on the fly and no transposed copy
// of an activation or a weight is ever written. (The reference leaves both products to cuBLAS,
// ISO/ops/mm/mm_fwd_scope.py:75-147.)
//
// TN can ACCUMULATE into an fp32 destination (the optimizer's main-gradient buffer): the epilogue adds the tile to
// what is there, which replaces "write a bf16 gradient, then add it to the fp32 buffer" by one pass.
//
// Structure as in the forward kernel: persistent CTAs, warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 epilogue,
// two TMEM accumulators, bounded waits. Reduction order: 64-row blocks ascending, four K=16 steps each; no split-K, so
// results do not depend on the grid.
#include "bw_common.cuh"
#include "host_util.h"

namespace {

using namespace bw;

constexpr int BM = 128;
constexpr int BK = 64;            // reduction elements per pipeline stage
constexpr int kThreads = 192;
constexpr int kChunkBytes = BK * 128;   // one [64 rows x 64 cols] bf16 chunk of an M/N-major operand

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ACC = 2 };

template <int BN>
struct Cfg {
  static constexpr int kBytesA = BM * BK * 2;      // 16 KB either way ([128 x 64] K-major or two chunks)
  static constexpr int kBytesB = BN * BK * 2;
  static constexpr int kStage = kBytesA + kBytesB;
  static constexpr int kStages = (200 * 1024) / kStage > 8 ? 8 : (200 * 1024) / kStage;
  static constexpr int kTmemCols = tmem_cols_pow2(2 * BN);
  static constexpr int kSmemBytes = kStages * kStage + 1024 + 512;
};

// A_MN: A is given as [Kred, M] row-major (else [M, Kred]); B is always given as [Kred, N] row-major.
template <int BN, bool A_MN, int OUT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cout,
                int M, int N, int Kred, int ldc, int* __restrict__ status) {
  using C = Cfg<BN>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * C::kStage);
  // bars: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (Kred + BK - 1) / BK;

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
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<C::kTmemCols>(smem_u32(tmem_holder));
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
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // tiles that share a block of B columns run on neighbouring CTAs at the same time, so B chunks hit in L2
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % tiles_m, n_blk = t / tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[S + stage]), phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars[stage]);
          const uint32_t sa = smem_u32(smem + stage * C::kStage);
          mbar_arrive_expect_tx(full, C::kStage);
          if constexpr (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * kChunkBytes, &tmA, full, m_blk * BM + c * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmA, full, kb * BK, m_blk * BM);
          }
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_2d(sa + C::kBytesA + c * kChunkBytes, &tmB, full, n_blk * BN + c * 64, kb * BK);
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[stage]), phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStage);
          // K-major: +32 bytes per K=16 step inside the swizzle atom. M/N-major: 16 reduction rows = 2048 bytes,
          // 64-column chunks kChunkBytes apart (leading-dimension offset), 8-row groups 1024 bytes apart.
          const uint64_t da = A_MN ? make_sw128_desc(sa, kChunkBytes, 1024) : make_sw128_desc(sa, 16, 1024);
          const uint64_t db = make_sw128_desc(sa + C::kBytesA, kChunkBytes, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16_ss(d_tmem, da + static_cast<uint64_t>(A_MN ? 128 * k : 2 * k), db + static_cast<uint64_t>(128 * k), idesc,
                        (kb | k) != 0 ? 1u : 0u);
          umma_commit(smem_u32(&bars[S + stage]));
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bars[2 * S + acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int m_blk = t % tiles_m, n_blk = t / tiles_m;
      if (!mbar_wait(smem_u32(&bars[2 * S + acc]), acc_phase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m_blk * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait_dep(r);
        const int col0 = n_blk * BN + c * 32;
        if (row < M && col0 < N) {
          const bool whole = col0 + 32 <= N;
          if constexpr (OUT == OUT_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * ldc + col0;
            if (whole && (ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                reinterpret_cast<uint4*>(dst)[j] = v;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) dst[j] = f2bf(__uint_as_float(r[j]));
            }
          } else {
            float* dst = reinterpret_cast<float*>(Cout) + static_cast<size_t>(row) * ldc + col0;
            if (whole && (ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                       __uint_as_float(r[4 * j + 3]));
                if constexpr (OUT == OUT_F32_ACC) {
                  const float4 o = reinterpret_cast<const float4*>(dst)[j];
                  v.x = __fadd_rn(o.x, v.x), v.y = __fadd_rn(o.y, v.y), v.z = __fadd_rn(o.z, v.z), v.w = __fadd_rn(o.w, v.w);
                }
                reinterpret_cast<float4*>(dst)[j] = v;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) dst[j] = (OUT == OUT_F32_ACC) ? __fadd_rn(dst[j], __uint_as_float(r[j])) : __uint_as_float(r[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[2 * S + 2 + acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
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
    tmem_dealloc<C::kTmemCols>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------------------ grouped (MoE experts)
// Rows are sorted by expert; offs[e] .. offs[e+1] (device memory) delimits expert e's rows, every group padded with
// zero rows to a multiple of 64 (see moe_dispatch.cu), so a 64-row reduction block never mixes two experts.
//
//   GROUPED_NN   dX[rows of e, :] = dY[rows of e, :] * W_e          W_e [Nred, Kout] read M/N-major
//   GROUPED_TN   dW_e[Mo, No] (+)= dY[rows of e, :]^T * X[rows of e, :]   both read M/N-major, reduction over e's rows
//
// (The reference: a hand-written Triton expert VJP, ISO/ops/moe/moe_backward_kernel.py:254-401.)
constexpr int kMaxExperts = 512;

template <int BN, bool TN, int OUT>
__global__ void __launch_bounds__(kThreads, 1)
grouped_bwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cout,
                   const int* __restrict__ offs, int E, int M, int N, int Kred, int ldc, long long c_expert_stride,
                   int* __restrict__ status) {
  // NN: M unused (rows come from offs), N = output columns, Kred = reduction (fixed per expert), B rows of expert e
  //     start at e * Kred.   TN: M x N = per-expert output, reduction over the expert's rows, C of expert e at
  //     Cout + e * c_expert_stride elements.
  using C = Cfg<BN>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * C::kStage);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  __shared__ int s_row_start[kMaxExperts + 1];
  __shared__ int s_tile_start[kMaxExperts + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e <= E; e += kThreads) s_row_start[e] = offs[e];
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
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<C::kTmemCols>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  __syncthreads();
  const int tiles_n = (N + BN - 1) / BN;
  const int tiles_m_tn = (M + BM - 1) / BM;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_tile_start[e] = acc;
      acc += TN ? tiles_m_tn : (s_row_start[e + 1] - s_row_start[e] + BM - 1) / BM;
    }
    s_tile_start[E] = acc;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int total_mt = s_tile_start[E];
  const int num_tiles = total_mt * tiles_n;

  // tile -> expert, first output row (NN: dispatch row; TN: row of the expert's matrix), end row, n block, reduction blocks
  auto decode = [&](int t, int& e, int& row0, int& row_end, int& n_blk, int& num_kb, int& red0) {
    const int mt = t % total_mt;
    n_blk = t / total_mt;
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_tile_start[mid] <= mt) lo = mid; else hi = mid;
    }
    e = lo;
    if (TN) {
      row0 = (mt - s_tile_start[e]) * BM;
      row_end = min(row0 + BM, M);
      red0 = s_row_start[e];
      num_kb = (s_row_start[e + 1] - s_row_start[e] + BK - 1) / BK;
    } else {
      row0 = s_row_start[e] + (mt - s_tile_start[e]) * BM;
      row_end = min(row0 + BM, s_row_start[e + 1]);
      red0 = e * Kred;
      num_kb = (Kred + BK - 1) / BK;
    }
  };

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int e, row0, row_end, n_blk, num_kb, red0;
        decode(t, e, row0, row_end, n_blk, num_kb, red0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[S + stage]), phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars[stage]);
          const uint32_t sa = smem_u32(smem + stage * C::kStage);
          mbar_arrive_expect_tx(full, C::kStage);
          if constexpr (TN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * kChunkBytes, &tmA, full, row0 + c * 64, red0 + kb * BK);
          } else {
            tma_load_2d(sa, &tmA, full, kb * BK, row0);
          }
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_2d(sa + C::kBytesA + c * kChunkBytes, &tmB, full, n_blk * BN + c * 64, red0 + kb * BK);
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, TN ? 1 : 0, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int e, row0, row_end, n_blk, num_kb, red0;
        decode(t, e, row0, row_end, n_blk, num_kb, red0);
        if (num_kb == 0) continue;       // an expert without rows: the epilogue writes zeros on its own
        if (!mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[stage]), phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::kStage);
          const uint64_t da = TN ? make_sw128_desc(sa, kChunkBytes, 1024) : make_sw128_desc(sa, 16, 1024);
          const uint64_t db = make_sw128_desc(sa + C::kBytesA, kChunkBytes, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16_ss(d_tmem, da + static_cast<uint64_t>(TN ? 128 * k : 2 * k), db + static_cast<uint64_t>(128 * k), idesc,
                        (kb | k) != 0 ? 1u : 0u);
          umma_commit(smem_u32(&bars[S + stage]));
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bars[2 * S + acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int e, row0, row_end, n_blk, num_kb, red0;
      decode(t, e, row0, row_end, n_blk, num_kb, red0);
      const bool empty = num_kb == 0;
      if (!empty) {
        if (!mbar_wait(smem_u32(&bars[2 * S + acc]), acc_phase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
      }
      const int row = row0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const size_t cbase = TN ? static_cast<size_t>(e) * static_cast<size_t>(c_expert_stride) : 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        if (!empty) {
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait_dep(r);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col0 = n_blk * BN + c * 32;
        if (row < row_end && col0 < N) {
          const bool whole = col0 + 32 <= N;
          if constexpr (OUT == OUT_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cout) + cbase + static_cast<size_t>(row) * ldc + col0;
            if (whole && (ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                reinterpret_cast<uint4*>(dst)[j] = v;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) dst[j] = f2bf(__uint_as_float(r[j]));
            }
          } else {
            float* dst = reinterpret_cast<float*>(Cout) + cbase + static_cast<size_t>(row) * ldc + col0;
            if (whole && (ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                       __uint_as_float(r[4 * j + 3]));
                if constexpr (OUT == OUT_F32_ACC) {
                  const float4 o = reinterpret_cast<const float4*>(dst)[j];
                  v.x = __fadd_rn(o.x, v.x), v.y = __fadd_rn(o.y, v.y), v.z = __fadd_rn(o.z, v.z), v.w = __fadd_rn(o.w, v.w);
                }
                reinterpret_cast<float4*>(dst)[j] = v;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) dst[j] = (OUT == OUT_F32_ACC) ? __fadd_rn(dst[j], __uint_as_float(r[j])) : __uint_as_float(r[j]);
            }
          }
        }
      }
      if (!empty) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[2 * S + 2 + acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<C::kTmemCols>(tmem_base);
  }
}

int sm_count(int dev) {
  static int n[64] = {0};
  if (dev < 0 || dev >= 64) return 148;
  if (n[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

template <int BN, bool A_MN, int OUT>
int launch(const void* A, const void* B, void* Cp, int M, int N, int Kred, int lda, int ldb, int ldc, cudaStream_t stream, int dev) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB;
  // A K-major: tensor [M rows, Kred cols], box [64 cols x 128 rows]; A M/N-major: tensor [Kred rows, M cols], box [64 x 64]
  int rc = A_MN ? ixh::make_tmap_bf16_2d(&tmA, A, Kred, M, lda, 64) : ixh::make_tmap_bf16_2d(&tmA, A, M, Kred, lda, BM);
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmB, B, Kred, N, ldb, 64);
  if (rc) return rc;
  auto kern = gemm_bwd_kernel<BN, A_MN, OUT>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = sm_count(dev);
  if (tiles < grid) grid = tiles;
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(tmA, tmB, Cp, M, N, Kred, ldc, ixh::status_word(dev));
  IX_CUDA(cudaGetLastError());
  return ixh::IX_OK;
}

template <bool A_MN>
int dispatch(const void* A, const void* B, void* C, int M, int N, int Kred, int lda, int ldb, int ldc, int out_mode, cudaStream_t s, int dev) {
  // the widest tile that still gives most SMs a tile
  const int tm = (M + BM - 1) / BM;
  int bn = 256;
  while (bn > 64 && tm * ((N + bn - 1) / bn) * 5 < sm_count(dev) * 3) bn >>= 1;
#define IX_CASE(BN_, OUT_) \
  if (bn == BN_ && out_mode == OUT_) return launch<BN_, A_MN, OUT_>(A, B, C, M, N, Kred, lda, ldb, ldc, s, dev);
  IX_CASE(256, OUT_BF16) IX_CASE(256, OUT_F32) IX_CASE(256, OUT_F32_ACC)
  IX_CASE(128, OUT_BF16) IX_CASE(128, OUT_F32) IX_CASE(128, OUT_F32_ACC)
  IX_CASE(64, OUT_BF16) IX_CASE(64, OUT_F32) IX_CASE(64, OUT_F32_ACC)
#undef IX_CASE
  return ixh::fail(ixh::IX_EARG, "gemm_bwd: unsupported output mode %d", out_mode);
}

}  // namespace

// C[M,N] = A[M,Kred] * B[Kred,N]   (input gradient: A = dY, B = W as stored, [out_features, in_features]).
// A, B bf16 row-major with leading dims lda, ldb (multiples of 8 elements); N a multiple of 8.
// out_mode: 0 bf16, 1 fp32, 2 fp32 accumulate (C += ...).
IX_API int ix_gemm_bf16_nn(const void* A, const void* B, void* C, int M, int N, int Kred, int lda, int ldb, int ldc, int out_mode,
                           void* stream) {
  if (M <= 0 || N <= 0 || Kred <= 0) return ixh::fail(ixh::IX_EARG, "gemm_nn: empty problem %dx%dx%d", M, N, Kred);
  if ((lda & 7) || (ldb & 7) || (Kred & 7) || (N & 7)) return ixh::fail(ixh::IX_EARG, "gemm_nn: N, K, lda, ldb must be multiples of 8");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  return dispatch<false>(A, B, C, M, N, Kred, lda, ldb, ldc, out_mode, reinterpret_cast<cudaStream_t>(stream), dev);
}

// C[M,N] (+)= A[Kred,M]^T * B[Kred,N]   (weight gradient: A = dY [tokens, out_features], B = X [tokens, in_features]).
// M, N multiples of 8; Kred (the token count) is free: rows past the end read as zero.
IX_API int ix_gemm_bf16_tn(const void* A, const void* B, void* C, int M, int N, int Kred, int lda, int ldb, int ldc, int out_mode,
                           void* stream) {
  if (M <= 0 || N <= 0 || Kred <= 0) return ixh::fail(ixh::IX_EARG, "gemm_tn: empty problem %dx%dx%d", M, N, Kred);
  if ((lda & 7) || (ldb & 7) || (M & 7) || (N & 7)) return ixh::fail(ixh::IX_EARG, "gemm_tn: M, N, lda, ldb must be multiples of 8");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  return dispatch<true>(A, B, C, M, N, Kred, lda, ldb, ldc, out_mode, reinterpret_cast<cudaStream_t>(stream), dev);
}

namespace {
template <int BN, bool TN, int OUT>
int launch_grouped(const void* A, const void* B, void* Cp, const int* offs, int R, int E, int M, int N, int Kred, int lda, int ldb,
                   int ldc, long long cstride, cudaStream_t stream, int dev) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (TN) {
    rc = ixh::make_tmap_bf16_2d(&tmA, A, R, M, lda, 64);          // dY [R rows, M cols], chunks [64 x 64]
    if (rc) return rc;
    rc = ixh::make_tmap_bf16_2d(&tmB, B, R, N, ldb, 64);          // X [R rows, N cols]
  } else {
    rc = ixh::make_tmap_bf16_2d(&tmA, A, R, Kred, lda, BM);       // dY [R rows, Kred cols], K-major box [64 x 128]
    if (rc) return rc;
    rc = ixh::make_tmap_bf16_2d(&tmB, B, static_cast<uint64_t>(E) * Kred, N, ldb, 64);   // W [E * Kred rows, N cols]
  }
  if (rc) return rc;
  auto kern = grouped_bwd_kernel<BN, TN, OUT>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  kern<<<sm_count(dev), kThreads, C::kSmemBytes, stream>>>(tmA, tmB, Cp, offs, E, M, N, Kred, ldc, cstride, ixh::status_word(dev));
  IX_CUDA(cudaGetLastError());
  return ixh::IX_OK;
}
}  // namespace

// Grouped input gradient: C[r, :] = A[r, :] * W_e for every dispatch row r of expert e.
// A bf16 [R, Kred] (lda), W bf16 [E, Kred, N] contiguous, C [R, N] (out_mode 0 bf16 / 1 fp32), offs int32 [E+1] on the device.
IX_API int ix_moe_grouped_gemm_nn(const void* A, const void* W, void* C, const void* offs, int R, int E, int N, int Kred, int lda,
                                  int ldc, int out_mode, void* stream) {
  if (R <= 0) return 0;
  if (E < 1 || E > kMaxExperts) return ixh::fail(ixh::IX_EARG, "grouped_nn: E=%d unsupported", E);
  if ((lda & 7) || (N & 7) || (Kred & 7)) return ixh::fail(ixh::IX_EARG, "grouped_nn: N, K, lda must be multiples of 8");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int* o = static_cast<const int*>(offs);
  const int bn = (N % 256 == 0) ? 256 : (N % 128 == 0 ? 128 : 64);
#define IX_G(BN_, OUT_) if (bn == BN_ && out_mode == OUT_) return launch_grouped<BN_, false, OUT_>(A, W, C, o, R, E, 0, N, Kred, lda, N, ldc, 0, s, dev);
  IX_G(256, OUT_BF16) IX_G(256, OUT_F32) IX_G(128, OUT_BF16) IX_G(128, OUT_F32) IX_G(64, OUT_BF16) IX_G(64, OUT_F32)
#undef IX_G
  return ixh::fail(ixh::IX_EARG, "grouped_nn: unsupported output mode %d", out_mode);
}

// Grouped weight gradient: C_e[M, N] (+)= A[rows of e, :]^T * B[rows of e, :].
// A bf16 [R, M] (lda), B bf16 [R, N] (ldb), C [E, M, N] contiguous (out_mode 0 bf16 / 1 fp32 / 2 fp32 accumulate).
// Every group must start on a multiple of 64 rows and its padding rows must be zero in A.
IX_API int ix_moe_grouped_gemm_tn(const void* A, const void* B, void* C, const void* offs, int R, int E, int M, int N, int lda, int ldb,
                                  int out_mode, void* stream) {
  if (E < 1 || E > kMaxExperts) return ixh::fail(ixh::IX_EARG, "grouped_tn: E=%d unsupported", E);
  if ((lda & 7) || (ldb & 7) || (M & 7) || (N & 7) || R <= 0) return ixh::fail(ixh::IX_EARG, "grouped_tn: M, N, lda, ldb must be multiples of 8, R > 0");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int* o = static_cast<const int*>(offs);
  const int bn = (N % 256 == 0) ? 256 : (N % 128 == 0 ? 128 : 64);
  const long long cs = static_cast<long long>(M) * N;
#define IX_G(BN_, OUT_) if (bn == BN_ && out_mode == OUT_) return launch_grouped<BN_, true, OUT_>(A, B, C, o, R, E, M, N, 0, lda, ldb, N, cs, s, dev);
  IX_G(256, OUT_BF16) IX_G(256, OUT_F32) IX_G(256, OUT_F32_ACC) IX_G(128, OUT_BF16) IX_G(128, OUT_F32) IX_G(128, OUT_F32_ACC)
  IX_G(64, OUT_BF16) IX_G(64, OUT_F32) IX_G(64, OUT_F32_ACC)
#undef IX_G
  return ixh::fail(ixh::IX_EARG, "grouped_tn: unsupported output mode %d", out_mode);
}
