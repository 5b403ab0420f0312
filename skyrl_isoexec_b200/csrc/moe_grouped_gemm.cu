// Grouped expert GEMM for mixture-of-experts layers on sm_100a: ONE launch computes, for every expert e,
//   C[rows of e, :] = A[rows of e, :] * B_e^T
// where the rows of A are already sorted by expert and `offs[e] .. offs[e+1]` (device memory, no host
// round trip) delimits expert e's rows. The reference loops over experts with one library GEMM each
// (ISO/ops/moe/moe_batched_experts.py:152-298).
//
// Numerics are those of the dense GEMM (gemm_tcgen05.cu): every output element is the sum over K in
// ascending 64-blocks, four K=16 tcgen05.mma steps each, into one fp32 TMEM cell. A row's result does
// not depend on which expert group it sits in, how large the group is, or which CTA computes it.
//
// Epilogues
//   EPI_BF16 / EPI_F32   plain store, optionally SCATTERED: row r goes to the address row_dst[r], which may be
//                        another GPU's memory (the combine all-to-all of expert parallelism happens inside
//                        the GEMM epilogue as peer stores);
//   EPI_GLU              B_e = [gate rows | up rows]; a tile multiplies both halves at once (one MMA of
//                        width 2*BN) and the epilogue applies the same three roundings as the separate
//                        kernels do: h = bf16(acc), a = bf16(bf16(silu(g)) * u), out = bf16(a * w_row).
//
// Structure as the dense kernel: persistent CTAs, warp 0 TMA, warp 1 MMA, warps 2..5 epilogue, double
// TMEM accumulators, all waits bounded. The (expert, m-tile) table is built in shared memory from `offs`.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kMaxStages = 12;
constexpr int kSmemLimit = 227 * 1024 - 4352;   // dynamic shared memory budget: the CTA limit minus this kernel's static tables
constexpr int kMaxExperts = 512;

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_GLU = 2 };

__device__ __forceinline__ float silu_f32(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))); }

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    void* __restrict__ Cout, const int* __restrict__ offs, const float* __restrict__ w_rows,
                    const long long* __restrict__ row_dst, int R, int E, int N, int K, int ldc, int rows_b_per_expert,
                    int a_rows, int S, int* __restrict__ status) {
  constexpr int kMmaN = (EPI == EPI_GLU) ? 2 * BN : BN;
  constexpr int kTmemCols = tmem_cols_pow2(2 * kMmaN);
  static_assert(kTmemCols <= 512, "accumulators exceed TMEM");
  const int stage_bytes_a = a_rows * BK * 2;
  const int stage_bytes = stage_bytes_a + kMmaN * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [S stages][tail: what the last stage's MMA may read past a short A box][barriers]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * stage_bytes + (BM - a_rows) * BK * 2);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  __shared__ int s_tile_start[kMaxExperts + 1];   // first m-tile index of each expert; [E] = total m-tiles
  __shared__ int s_row_start[kMaxExperts + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_n = N / BN;
  const int num_kb = K / BK;

  pdl_launch_dependents();
  if (offs != nullptr) pdl_wait();   // the row offsets come from the routing kernels that precede this one
  // offs == nullptr: one group made of all R rows (the dense MLP uses this kernel for its fused GLU epilogue)
  for (int e = threadIdx.x; e <= E; e += kThreads) s_row_start[e] = offs ? offs[e] : (e == 0 ? 0 : R);
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
    tmem_alloc<kTmemCols>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_tile_start[e] = acc;
      acc += (s_row_start[e + 1] - s_row_start[e] + BM - 1) / BM;
    }
    s_tile_start[E] = acc;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int total_mt = s_tile_start[E];
  const int num_tiles = total_mt * tiles_n;

  // tile t -> (expert, first row, end row, n block). m-tiles vary fastest so that CTAs running together share B tiles in L2.
  auto decode = [&](int t, int& e, int& row0, int& row_end, int& n_blk) {
    const int mt = t % total_mt;
    n_blk = t / total_mt;
    int lo = 0, hi = E;           // largest e with s_tile_start[e] <= mt
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_tile_start[mid] <= mt) lo = mid; else hi = mid;
    }
    e = lo;
    row0 = s_row_start[e] + (mt - s_tile_start[e]) * BM;
    row_end = min(row0 + BM, s_row_start[e + 1]);
  };

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      // weights of the first stages of this CTA's first tile go out before the wait for the previous kernel
      int pre = 0;
      if (static_cast<int>(blockIdx.x) < num_tiles) {
        int e, row0, row_end, n_blk;
        decode(blockIdx.x, e, row0, row_end, n_blk);
        const int b_row = e * rows_b_per_expert + n_blk * BN;
        pre = num_kb < S ? num_kb : S;
        for (int kb = 0; kb < pre; ++kb) {
          const uint32_t full = smem_u32(&bars[kb]);
          mbar_arrive_expect_tx(full, stage_bytes);
          const uint32_t sb = smem_u32(smem + kb * stage_bytes) + stage_bytes_a;
          tma_load_2d(sb, &tmB, full, kb * BK, b_row);
          if (EPI == EPI_GLU) tma_load_2d(sb + BN * BK * 2, &tmB, full, kb * BK, b_row + N);
        }
      }
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int e, row0, row_end, n_blk;
        decode(t, e, row0, row_end, n_blk);
        const int b_row = e * rows_b_per_expert + n_blk * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t full = smem_u32(&bars[stage]);
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          if (pre > 0) {
            --pre;
            tma_load_2d(sa, &tmA, full, kb * BK, row0);
            if (++stage == S) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          if (!mbar_wait(smem_u32(&bars[S + stage]), phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full, stage_bytes);
          tma_load_2d(sa, &tmA, full, kb * BK, row0);
          tma_load_2d(sa + stage_bytes_a, &tmB, full, kb * BK, b_row);
          if (EPI == EPI_GLU) tma_load_2d(sa + stage_bytes_a + BN * BK * 2, &tmB, full, kb * BK, b_row + N);
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, kMmaN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kMmaN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars[stage]), phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint64_t da = make_sw128_desc(sa, 16, 1024);
          const uint64_t db = make_sw128_desc(sa + stage_bytes_a, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_f16_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
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
    pdl_wait();   // outputs (and the per-row weights / destinations) belong to the previous kernels until they finish
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int e, row0, row_end, n_blk;
      decode(t, e, row0, row_end, n_blk);
      if (!mbar_wait(smem_u32(&bars[2 * S + acc]), acc_phase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = row0 + quad * 32 + lane;
      const bool valid = row < row_end;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kMmaN;
      float wr = 1.0f;
      if (EPI == EPI_GLU && valid && w_rows != nullptr) wr = w_rows[row];   // no weights: x 1.0 leaves the bf16 value as it is
      uint8_t* dst_row = nullptr;
      if (valid) {
        if (row_dst != nullptr) dst_row = reinterpret_cast<uint8_t*>(row_dst[row]);
        else dst_row = static_cast<uint8_t*>(Cout) + static_cast<size_t>(row) * ldc * (EPI == EPI_F32 ? 4 : 2);
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait_dep(r);
        const int col0 = n_blk * BN + c * 32;
        if constexpr (EPI == EPI_GLU) {
          uint32_t u[32];
          tmem_ld_32x32(taddr + BN + c * 32, u);
          tmem_ld_wait_dep(u);
          if (valid) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(dst_row) + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float a2[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int i = 8 * j + 2 * q + h;
                  const float g = round_bf(__uint_as_float(r[i]));            // what the fc1 GEMM would have stored
                  const float up = round_bf(__uint_as_float(u[i]));
                  const float s = round_bf(silu_f32(g));
                  const float a = round_bf(__fmul_rn(s, up));                 // SwiGLU output in bf16
                  a2[h] = __fmul_rn(a, wr);                                   // gate weight, rounded by the pack below
                }
                o[q] = pack_bf2(a2[0], a2[1]);
              }
              reinterpret_cast<uint4*>(dst)[j] = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        } else if (valid) {
          if constexpr (EPI == EPI_F32) {
            float* dst = reinterpret_cast<float*>(dst_row) + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(dst_row) + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              reinterpret_cast<uint4*>(dst)[j] = v;
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
    if (row_dst != nullptr) __threadfence_system();   // scattered rows may be peer memory: make them visible before the kernel ends
  }

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

int g_sms2[64] = {0};
int sms_of(int dev) {
  if (dev < 0 || dev >= 64) return 148;
  if (g_sms2[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms2[dev] = n;
  }
  return g_sms2[dev];
}

template <int BN, int EPI>
int launch_grouped(const void* A, const void* B, void* C, const int* offs, const float* w_rows, const long long* row_dst,
                   int R, int E, int N, int K, int lda, int ldb, int ldc, int max_tiles, cudaStream_t stream, int dev) {
  constexpr int kMmaN = (EPI == EPI_GLU) ? 2 * BN : BN;
  constexpr int kFixed = 1024 /*align*/ + 512 /*barriers*/;
  int a_rows = (R + 7) & ~7;
  if (a_rows > BM) a_rows = BM;
  const int stage_bytes = a_rows * BK * 2 + kMmaN * BK * 2;
  const int tail = (BM - a_rows) * BK * 2;
  int S = (kSmemLimit - kFixed - tail) / stage_bytes;
  if (S > kMaxStages) S = kMaxStages;
  const int rows_b = (EPI == EPI_GLU) ? 2 * N : N;
  CUtensorMap tmA, tmB;
  int rc = ixh::make_tmap_bf16_2d(&tmA, A, R, K, lda, a_rows);
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmB, B, static_cast<uint64_t>(E) * rows_b, K, ldb, BN);
  if (rc) return rc;
  auto kern = grouped_gemm_kernel<BN, EPI>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    attr_set[dev & 63] = true;
  }
  int grid = sms_of(dev);
  if (max_tiles > 0 && max_tiles < grid) grid = max_tiles;
  const int kSmem = S * stage_bytes + tail + kFixed;
  IX_CUDA(ixh::launch_pdl(kern, dim3(grid), dim3(kThreads), static_cast<size_t>(kSmem), stream, tmA, tmB, C, offs, w_rows, row_dst, R, E, N, K, ldc,
                          rows_b, a_rows, S, ixh::status_word(dev)));
  return 0;
}

}  // namespace

// A [R, K] bf16 rows sorted by expert; offs int32 [E+1] on the device; B [E, rows_b, K] bf16 contiguous
// (rows_b = N, or 2N = [gate | up] for epi 2). C [R, N] (bf16 for epi 0/2, fp32 for epi 1), or, when row_dst
// is given (int64 [R] of device addresses), row r is stored at row_dst[r] instead. w_rows fp32 [R] for epi 2.
IX_API int ix_moe_grouped_gemm(const void* A, const void* B, void* C, const void* offs, const void* w_rows, const void* row_dst,
                               int R, int E, int N, int K, int lda, int ldc, int epi, int bn, void* stream) {
  if (R <= 0) return 0;
  if (E < 1 || E > kMaxExperts) return ixh::fail(ixh::IX_EARG, "grouped gemm: E=%d unsupported (1..%d)", E, kMaxExperts);
  if ((K % BK) || (lda & 7) || (ldc & 7)) return ixh::fail(ixh::IX_EARG, "grouped gemm: K must be a multiple of 64, lda/ldc of 8");
  if (offs == nullptr && E != 1) return ixh::fail(ixh::IX_EARG, "grouped gemm: row offsets may only be omitted for a single group");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  if (bn == 0) {
    // an upper bound of the m-tiles: every expert may add one ragged tile (exact for a single group)
    const long long mt = (static_cast<long long>(R) + BM - 1) / BM + (offs ? E : 0);
    const int sms = sms_of(dev);
    const int cand[4] = {128, 96, 64, 32};
    double util[4], best = -1.0;
    for (int i = 0; i < 4; ++i) {
      util[i] = -1.0;
      if (N % cand[i]) continue;
      const long long tiles = mt * (N / cand[i]);
      const long long waves = (tiles + sms - 1) / sms;
      util[i] = static_cast<double>(tiles) / static_cast<double>(waves * sms);
      if (util[i] > best) best = util[i];
    }
    // the widest tile within 5% of the best whole-wave utilisation: narrow tiles only where they fill the machine
    bn = 32;
    for (int i = 0; i < 4; ++i) {
      if (util[i] >= 0.0 && util[i] >= best - 0.05) {
        bn = cand[i];
        break;
      }
    }
  }
  if (N % bn) return ixh::fail(ixh::IX_EARG, "grouped gemm: N=%d is not a multiple of the tile width %d", N, bn);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int* o = static_cast<const int*>(offs);
  const float* w = static_cast<const float*>(w_rows);
  const long long* rd = static_cast<const long long*>(row_dst);
  const long long max_tiles_ll = ((static_cast<long long>(R) + BM - 1) / BM + E) * (N / bn);
  const int max_tiles = max_tiles_ll > 1 << 30 ? 1 << 30 : static_cast<int>(max_tiles_ll);
#define IX_GG(BN_, EPI_) \
  if (bn == BN_ && epi == EPI_) return launch_grouped<BN_, EPI_>(A, B, C, o, w, rd, R, E, N, K, lda, K, ldc, max_tiles, s, dev);
  IX_GG(128, 0) IX_GG(96, 0) IX_GG(64, 0) IX_GG(32, 0) IX_GG(128, 1) IX_GG(96, 1) IX_GG(64, 1) IX_GG(32, 1)
  IX_GG(128, 2) IX_GG(96, 2) IX_GG(64, 2) IX_GG(32, 2)
#undef IX_GG
  return ixh::fail(ixh::IX_EARG, "grouped gemm: no kernel for bn=%d epi=%d", bn, epi);
}
