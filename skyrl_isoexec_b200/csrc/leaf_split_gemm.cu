// Leaf-parallel form of the TP-invariant leaf-tree GEMM for decode-sized M (sm_100a):
//
//     C[M,N] = tree_{j<L} ( A[:, Kj] * B[:, Kj]^T ),   Kj = the j-th of L equal K slices, fp32, balanced tree
//
// Same bits as the single-CTA form in tp_gemm_fused.cu (every leaf is the same ascending walk over its 64-wide K
// blocks into a zeroed fp32 TMEM accumulator; the leaves are folded in the same order,
// ((l0 + l1) + (l2 + l3)) + ((l4 + l5) + (l6 + l7)), with round-to-nearest fp32 adds). What changes is WHERE the
// leaves run. A tcgen05.mma of up to 128 columns takes ~63 clocks whatever its width, so a CTA that walks the whole
// K of a decode GEMM spends K/16 x 63 clocks however few rows there are, and N/BN tiles cannot fill 148 SMs either.
// The leaf tree is a K split whose order is fixed by the contract, so it costs no invariance to give each leaf its
// own CTA: the L CTAs of one output tile form a thread-block CLUSTER, each walks K/L, parks its fp32 partial in its
// own shared memory, and after one cluster barrier every CTA folds 1/L of the tile's columns, reading the L partials
// through distributed shared memory in tree order. No global scratch, no atomics, no second launch.
// (reference: the leaf GEMM schedules of ISO/ops/collectives/pik/gemm.py; there the leaves are separate launches.)
//
// 192 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 drain TMEM to the staging tile; all six warps fold.
// Every mbarrier wait is bounded; a CTA that gives up still arrives at both cluster barriers (the fold then writes
// nothing), so its partners are never left waiting on it.
#include "bw_common.cuh"
#include "host_util.h"

namespace {

using namespace bw;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kMaxStages = 12;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kBarBytes = 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_addr, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

template <int BN, int L, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
leaf_split_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cout,
                  int M, int N, int K, int ldc, int a_rows, int S, int* __restrict__ status) {
  constexpr int kTmemCols = BN < 32 ? 32 : BN;
  constexpr int kStride = BN + 4;                       // floats per staged row (+4: rows do not share a bank phase)
  const int stage_bytes_a = a_rows * BK * 2;
  const int stage_bytes = stage_bytes_a + BN * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // [S stages][tail: rows the MMA reads beyond a short A box][barriers][staging: a_rows x kStride fp32]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * stage_bytes + (BM - a_rows) * BK * 2);
  // bars: [0,S) full, [S,2S) empty, [2S] accumulator complete
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* staging = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + kBarBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int leaf = static_cast<int>(cluster_ctarank());          // cluster = (L, 1, 1): rank in cluster = leaf
  const int tile = blockIdx.x / L;
  const int tiles_m = (M + BM - 1) / BM;
  const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
  const int kb_per_leaf = K / BK / L;
  const int kb0 = leaf * kb_per_leaf;
  const int rows_valid = min(BM, M - m_blk * BM);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2 * S + 1; ++i) mbar_init(smem_u32(&bars[i]), 1);
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
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      // weights first (no kernel of a step writes them), activations after the previous kernel has finished
      const int pre = kb_per_leaf < S ? kb_per_leaf : S;
      for (int kb = 0; kb < pre; ++kb) {
        const uint32_t full = smem_u32(&bars[kb]);
        mbar_arrive_expect_tx(full, stage_bytes);
        tma_load_2d(smem_u32(smem + kb * stage_bytes) + stage_bytes_a, &tmB, full, (kb0 + kb) * BK, n_blk * BN);
      }
      pdl_wait();
      for (int kb = 0; kb < pre; ++kb)
        tma_load_2d(smem_u32(smem + kb * stage_bytes), &tmA, smem_u32(&bars[kb]), (kb0 + kb) * BK, m_blk * BM);
      int stage = pre == S ? 0 : pre;
      uint32_t phase = pre == S ? 1 : 0;
      for (int kb = pre; kb < kb_per_leaf; ++kb) {
        if (!mbar_wait(smem_u32(&bars[S + stage]), phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t full = smem_u32(&bars[stage]);
        const uint32_t sa = smem_u32(smem + stage * stage_bytes);
        mbar_arrive_expect_tx(full, stage_bytes);
        tma_load_2d(sa, &tmA, full, (kb0 + kb) * BK, m_blk * BM);
        tma_load_2d(sa + stage_bytes_a, &tmB, full, (kb0 + kb) * BK, n_blk * BN);
        if (++stage == S) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer: this CTA's leaf only
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < kb_per_leaf; ++kb) {
        if (!mbar_wait(smem_u32(&bars[stage]), phase, abort_flag, status, ST_TIMEOUT_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * stage_bytes);
        const uint64_t da = make_sw128_desc(sa, 16, 1024);
        const uint64_t db = make_sw128_desc(sa + stage_bytes_a, 16, 1024);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) umma_f16_ss(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(smem_u32(&bars[S + stage]));
        if (++stage == S) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(smem_u32(&bars[2 * S]));
    }
  } else {
    // ------------------------------------------------------------ warps 2..5: TMEM -> staging tile (fp32, unrounded)
    const int quad = warp & 3;
    const bool done = mbar_wait(smem_u32(&bars[2 * S]), 0, abort_flag, status, ST_TIMEOUT_TMEM_FULL);
    tc_fence_after();
    if (done && quad * 32 < rows_valid) {                        // warp-uniform: the loads below are .sync.aligned
      const int row = quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait_dep(r);
        if (row < a_rows) {
          float4* dst = reinterpret_cast<float4*>(staging + row * kStride + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                 __uint_as_float(r[4 * j + 3]));
        }
      }
    }
  }

  // ---------------------------------------------------------------- fold across the cluster
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  int bad = *abort_flag;
  if (threadIdx.x == 0 && bad) staging[0] = __int_as_float(0x7fc00000);    // a partner never reads a half-written tile as data
  cluster_sync_all();                                            // every CTA's partial is staged (or its CTA gave up)
  if (!bad) {
    pdl_wait();                                                  // C may still be read by the previous kernel
    constexpr int kColsPer = BN / L;                             // columns of the tile this CTA folds
    constexpr int kVec = kColsPer / 4;
    const uint32_t st_addr = smem_u32(staging);
    for (int idx = threadIdx.x; idx < rows_valid * kVec; idx += kThreads) {
      const int r = idx / kVec, c = leaf * kColsPer + (idx % kVec) * 4;
      const uint32_t off = st_addr + static_cast<uint32_t>(r * kStride + c) * 4u;
      float4 v[L];
#pragma unroll
      for (int l = 0; l < L; ++l) v[l] = ld_dsmem_f4(off, static_cast<uint32_t>(l));
#pragma unroll
      for (int s = 1; s < L; s *= 2)
#pragma unroll
        for (int i = 0; i + s < L; i += 2 * s) v[i] = add4(v[i], v[i + s]);
      const size_t o = static_cast<size_t>(m_blk * BM + r) * ldc + n_blk * BN + c;
      if constexpr (OUT_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(Cout) + o) = v[0];
      } else {
        uint2 w;
        w.x = pack_bf2(v[0].x, v[0].y);
        w.y = pack_bf2(v[0].z, v[0].w);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(Cout) + o) = w;
      }
    }
  } else {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);              // copies that may still be in flight land first
  }
  cluster_sync_all();                                            // nobody leaves while a partner may read its staging tile
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

template <int BN, int L, bool OUT_F32>
int launch_split(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, cudaStream_t stream, int dev) {
  CUtensorMap tmA, tmB;
  int a_rows = (M + 7) & ~7;
  if (a_rows > BM) a_rows = BM;
  const int stage_bytes = a_rows * BK * 2 + BN * BK * 2;
  const int tail = (BM - a_rows) * BK * 2;
  const int staging = a_rows * (BN + 4) * 4;
  int S = (kSmemLimit - 1024 - kBarBytes - tail - staging) / stage_bytes;
  if (S > kMaxStages) S = kMaxStages;
  if (S < 2) return ixh::fail(ixh::IX_EARG, "leaf_split: no room for a pipeline (bn=%d rows=%d)", BN, a_rows);
  const int smem = S * stage_bytes + tail + kBarBytes + staging + 1024;
  int rc = ixh::make_tmap_bf16_2d(&tmA, A, M, K, lda, a_rows);
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmB, B, N, K, ldb, BN);
  if (rc) return rc;
  auto kern = leaf_split_kernel<BN, L, OUT_F32>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    attr_set[dev & 63] = true;
  }
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * L);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = L;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ixh::pdl_enabled() ? 2 : 1;
  IX_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, C, M, N, K, ldc, a_rows, S, ixh::status_word(dev)));
  return ixh::IX_OK;
}

}  // namespace

// Tile width the leaf-parallel form uses for a shape: the widest of 128 / 64 / 32 that divides N, leaves every CTA at
// least one float4 of columns to fold and still gives about one CTA per SM; 0 = this form does not apply.
IX_API int ix_leaf_split_bn(int M, int N, int K, int leaves) {
  if (leaves < 2 || leaves > 8 || (leaves & (leaves - 1)) || M <= 0 || M > 2 * BM || (K % (BK * leaves)) != 0) return 0;
  const int tiles_m = (M + BM - 1) / BM;
  int pick = 0;
  for (int bn = 128; bn >= 32; bn >>= 1) {
    if (N % bn || bn / leaves < 4) continue;
    pick = bn;
    if (tiles_m * (N / bn) * leaves >= 100) break;
  }
  return pick;
}

// C[M,N] (bf16, or fp32 when out_f32) = balanced fp32 tree over `leaves` equal K slices of A[M,K] * B[N,K]^T, one
// cluster of `leaves` CTAs per 128 x bn tile. bn: 32 / 64 / 128 (0 = ix_leaf_split_bn's choice).
IX_API int ix_leaf_split_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int leaves,
                              int bn, int out_f32, void* stream) {
  if (bn == 0) bn = ix_leaf_split_bn(M, N, K, leaves);
  if (bn == 0 || M <= 0 || N % bn || (K % (BK * leaves)) != 0 || bn / leaves < 4)
    return ixh::fail(ixh::IX_EARG, "leaf_split: unsupported shape M=%d N=%d K=%d leaves=%d bn=%d", M, N, K, leaves, bn);
  if ((lda & 7) || (ldb & 7) || (ldc & 3) || (!out_f32 && (ldc & 3))) return ixh::fail(ixh::IX_EARG, "leaf_split: leading dimensions must be multiples of 8 (ldc: 4)");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define IX_LS(BN_, L_)                                                                                           \
  if (bn == BN_ && leaves == L_)                                                                                 \
    return out_f32 ? launch_split<BN_, L_, true>(A, B, C, M, N, K, lda, ldb, ldc, s, dev)                        \
                   : launch_split<BN_, L_, false>(A, B, C, M, N, K, lda, ldb, ldc, s, dev);
  IX_LS(128, 2) IX_LS(64, 2) IX_LS(32, 2) IX_LS(128, 4) IX_LS(64, 4) IX_LS(32, 4) IX_LS(128, 8) IX_LS(64, 8) IX_LS(32, 8)
#undef IX_LS
  return ixh::fail(ixh::IX_EARG, "leaf_split: no kernel for bn=%d leaves=%d", bn, leaves);
}
