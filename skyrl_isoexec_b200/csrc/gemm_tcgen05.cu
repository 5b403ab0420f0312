// Batch-invariant dense GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T   (bf16 in, fp32
// accumulate in TMEM, bf16 or fp32 out).
//
// Invariance contract (the reason this kernel exists; the reference pins a cuBLASLt
// algorithm per (K,N) and proves two M-buckets equal, ISO/ops/mm/csrc/cublaslt_pinned.cpp:58-118):
//   * every output element is the sum over K of a_k*b_k taken in ONE order: 64-wide
//     K blocks in ascending order, each block as four tcgen05.mma K=16 steps that
//     accumulate into the same fp32 TMEM cell. No split-K, no stream-K.
//   * that order does not depend on M, on the tile the element falls in, on the CTA
//     that computes it, or on how many rows the call has, so one token's row is the
//     same bits in a 1-row decode and in a 16k-row training forward.
//   * the N tile width (template BN) only changes which elements share a CTA.
//
// Structure: persistent CTAs (one per SM), 192 threads:
//   warp 0      TMA producer  (one elected lane; 128B-swizzled 128x64 A and BNx64 B boxes)
//   warp 1      MMA issuer    (one elected lane; tcgen05.mma cta_group::1, M=128, N=BN, K=16)
//   warps 2..5  epilogue      (tcgen05.ld 32x32b -> registers -> bf16/fp32 -> global)
// TMEM holds two accumulators (2*BN columns) so the epilogue of tile i overlaps the
// main loop of tile i+1. All waits are bounded (bw_common.cuh).
#include <stdarg.h>

#include "bw_common.cuh"
#include "host_util.h"

namespace {

using namespace bw;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;

constexpr int kMaxStages = 16;
constexpr int kPipeBytes = 200 * 1024;   // shared memory given to the TMA pipeline

// The A stage holds only the rows that exist: a_rows = min(128, M rounded up to 8). The MMA still
// reads 128 rows (whatever follows in shared memory, never stored), so a decode-sized M spends its
// shared memory on more weight stages in flight instead of on zero padding.
template <int BN>
struct GemmCfg {
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kTmemCols = tmem_cols_pow2(2 * BN);
  static constexpr int kSmemBytes = kPipeBytes + BM * BK * 2 /*tail the last stage's MMA may read*/ + 1024 /*align*/ + 512 /*barriers*/;
  static int stage_bytes(int a_rows) { return a_rows * BK * 2 + kStageBytesB; }
  static int stages(int a_rows) {
    int s = kPipeBytes / stage_bytes(a_rows);
    return s > kMaxStages ? kMaxStages : s;
  }
};

template <int BN, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    void* __restrict__ Cout, int M, int N, int K, int ldc, int a_rows, int S,
                    int* __restrict__ status) {
  using Cfg = GemmCfg<BN>;
  const int stage_bytes_a = a_rows * BK * 2;
  const int stage_bytes = stage_bytes_a + Cfg::kStageBytesB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPipeBytes + BM * BK * 2);
  // bars: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

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
    tmem_alloc<Cfg::kTmemCols>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      // Before waiting for the previous kernel: the WEIGHT half of the first stages of this CTA's first tile (nothing
      // in a step writes weights). The activation half follows after pdl_wait().
      int pre = 0;
      if (static_cast<int>(blockIdx.x) < num_tiles) {
        pre = num_kb < S ? num_kb : S;
        const int n_blk0 = blockIdx.x / tiles_m;
        for (int kb = 0; kb < pre; ++kb) {
          const uint32_t full = smem_u32(&bars[kb]);
          mbar_arrive_expect_tx(full, stage_bytes);
          tma_load_2d(smem_u32(smem + kb * stage_bytes) + stage_bytes_a, &tmB, full, kb * BK, n_blk0 * BN);
        }
      }
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % tiles_m, n_blk = t / tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t full = smem_u32(&bars[stage]);
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          if (pre > 0) {
            // this stage's barrier is armed and its weights are on their way: add the activations
            --pre;
            tma_load_2d(sa, &tmA, full, kb * BK, m_blk * BM);
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
          tma_load_2d(sa, &tmA, full, kb * BK, m_blk * BM);
          tma_load_2d(sa + stage_bytes_a, &tmB, full, kb * BK, n_blk * BN);
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
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars[2 * S + 2 + acc]), acc_phase ^ 1, abort_flag, status,
                       ST_TIMEOUT_TMEM_EMPTY)) {
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
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint64_t da = make_sw128_desc(sa, 16, 1024);
          const uint64_t db = make_sw128_desc(sa + stage_bytes_a, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // +32 bytes per K=16 step inside the 128-byte swizzle atom (address field is >>4)
            umma_f16_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bars[S + stage]));  // frees the smem stage when the MMAs retire
          if (++stage == S) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bars[2 * S + acc]));  // accumulator ready for the epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    pdl_wait();                 // C may still be read by the previous kernel
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int m_blk = t % tiles_m, n_blk = t / tiles_m;
      if (!mbar_wait(smem_u32(&bars[2 * S + acc]), acc_phase, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m_blk * BM + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      constexpr int CW = (BN % 32 == 0) ? 32 : 16;   // columns per TMEM load (tiles of 48, 208, ... columns use 16)
#pragma unroll 1
      for (int c = 0; c < BN / CW; ++c) {
        uint32_t r[CW];
        if constexpr (CW == 32) {
          tmem_ld_32x32(taddr + c * CW, r);
          tmem_ld_wait_dep(r);
        } else {
          tmem_ld_32x16_sync(taddr + c * CW, r);
        }
        const int col0 = n_blk * BN + c * CW;
        if (row < M) {
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(Cout) + static_cast<size_t>(row) * ldc + col0;
            if (col0 + CW <= N && (ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < CW / 4; ++j)
                reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            } else {
              for (int j = 0; j < CW; ++j)
                if (col0 + j < N) dst[j] = __uint_as_float(r[j]);
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * ldc + col0;
            if (col0 + CW <= N && (ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < CW / 8; ++j) {
                uint4 v;
                v.x = pack_bf2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                reinterpret_cast<uint4*>(dst)[j] = v;
              }
            } else {
              for (int j = 0; j < CW; ++j)
                if (col0 + j < N) dst[j] = f2bf(__uint_as_float(r[j]));
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
    // give copies that may still be in flight time to land before the CTA's smem goes away
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<Cfg::kTmemCols>(tmem_base);
  }
}

int g_num_sms[64] = {0};

int num_sms(int dev) {
  if (dev < 0 || dev >= 64) return 148;
  if (g_num_sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_num_sms[dev] = n;
  }
  return g_num_sms[dev];
}

template <int BN, bool OUT_F32>
int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                int max_ctas, cudaStream_t stream, int dev) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int a_rows = (M + 7) & ~7;
  if (a_rows > BM) a_rows = BM;
  const int S = Cfg::stages(a_rows);
  int rc = ixh::make_tmap_bf16_2d(&tmA, A, M, K, lda, a_rows);
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmB, B, N, K, ldb, BN);
  if (rc) return rc;
  auto kern = gemm_bf16_nt_kernel<BN, OUT_F32>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = num_sms(dev);
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  IX_CUDA(ixh::launch_pdl(kern, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, tmA, tmB, C, M, N, K, ldc, a_rows, S, ixh::status_word(dev)));
  return ixh::IX_OK;
}

}  // namespace

// C[M,N] = A[M,K] * B[N,K]^T. A, B bf16 row-major with leading dims lda/ldb (elements,
// multiples of 8); C bf16 (out_f32=0) or fp32 (out_f32=1) with leading dim ldc.
// bn selects the N tile (32/48/64/128/208/256; 0 = choose from the shape).
IX_API int ix_gemm_bf16_nt(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                           int ldc, int out_f32, int bn, int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return ixh::fail(ixh::IX_EARG, "gemm: empty problem %dx%dx%d", M, N, K);
  if ((lda & 7) || (ldb & 7) || (K & 7)) return ixh::fail(ixh::IX_EARG, "gemm: K, lda, ldb must be multiples of 8");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0) {
    // Tile choice is a pure function of (M-bucket, N): wide tiles once they fill the
    // machine, narrow ones for decode-sized M so that all SMs stream weights.
    const int sms = num_sms(dev);
    const int tm = (M + BM - 1) / BM;
    bn = 256;
    if (tm > 1) {
      // training / prefill sizes: the widest tile that still gives >= 0.6 CTAs per SM
      while (bn > 32 && tm * ((N + bn - 1) / bn) * 5 < sms * 3) bn >>= 1;
    } else {
      // decode sizes (one row of tiles, weight streaming): of the widths below, the one that keeps the most SMs busy
      // over whole waves; ties go to the wider tile, which re-reads the activations least. A pure function of N.
      const int cand[6] = {256, 208, 128, 64, 48, 32};
      double util[6], best = -1.0;
      for (int i = 0; i < 6; ++i) {
        const long long tiles = (N + cand[i] - 1) / cand[i];
        const long long waves = (tiles + sms - 1) / sms;
        util[i] = static_cast<double>(tiles) / static_cast<double>(waves * sms);
        if (util[i] > best) best = util[i];
      }
      for (int i = 0; i < 6; ++i) {
        if (util[i] >= best - 0.05) {   // the widest tile within 5% of the best utilisation
          bn = cand[i];
          break;
        }
      }
    }
  }
#define IX_GEMM_CASE(BN_)                                                                                     \
  case BN_:                                                                                                   \
    return out_f32 ? launch_gemm<BN_, true>(A, B, C, M, N, K, lda, ldb, ldc, max_ctas, s, dev)                \
                   : launch_gemm<BN_, false>(A, B, C, M, N, K, lda, ldb, ldc, max_ctas, s, dev);
  switch (bn) {
    IX_GEMM_CASE(32)
    IX_GEMM_CASE(48)
    IX_GEMM_CASE(64)
    IX_GEMM_CASE(128)
    IX_GEMM_CASE(208)
    IX_GEMM_CASE(256)
    default:
      return ixh::fail(ixh::IX_EARG, "gemm: unsupported bn=%d", bn);
  }
#undef IX_GEMM_CASE
}
