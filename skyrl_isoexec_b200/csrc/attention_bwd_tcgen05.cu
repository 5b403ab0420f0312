// Causal GQA attention backward for sm_100a (packed varlen training layout), the counterpart of
// attention_tcgen05.cu. The reference differentiates FlashAttention-3 through torch's varlen op
// (ISO/ops/attention/megatron_varlen_attn.py:38-228); the backward is outside the bitwise contract on both sides,
// but it is deterministic here: no atomics, every sum has one order.
//
//   P  = exp2(S * scale * log2e - lse * log2e)        S = Q K^T, lse saved by the forward (natural log)
//   dV = P^T dO          dP = dO V^T          dS = P * (dP - delta) * scale,  delta = rowsum(dO * O)
//   dQ = dS K            dK = dS^T Q
//
// Four kernels:
//   attn_delta_kernel        delta[t, h] (half a warp per row)
//   attn_dq_kernel           one CTA per (query tile, KV head), key blocks of 128 streamed through two stages:
//                            S and dP by tcgen05 into TMEM, softmax warps -> dS (bf16, shared memory), dQ += dS K in TMEM
//   attn_dkv_kernel<.., DV>  one CTA per (key block, KV head), query tiles streamed: S -> P -> dV += P^T dO
//   attn_dkv_kernel<.., DK>  same loop: S, dP -> dS -> dK += dS^T Q
// P / dS are written once, row-major, and read by the tensor core as the M-major A operand, so no transpose is ever
// materialised; the sum over the G query heads of a KV head happens inside the MMA because tile rows are
// (token, head-in-group) pairs. dV and dK are separate kernels because one CTA cannot hold K, V, two stages of Q
// and dO, P and dS (256 KB) at once; apart, every operand is double-buffered and the extra S = Q K^T is hidden.
//
// Overlap: the softmax warps copy a tile's S (and dP) from TMEM to registers and say so at once; the MMA warp then
// issues the next tile's S / dP into the same columns while the exponentials of this tile are being computed, and
// the accumulating MMA of this tile follows as soon as its P / dS is in shared memory. The tensor pipe only waits
// when the softmax (exp2 on the SFU, ~1k clocks per 128 x 128 tile) is the longer of the two.
//
// Tile rows are GQA-packed exactly as in the forward: row r = (token r / G, head kvh*G + r % G), fetched with one 4D
// TMA box over [T, Hkv, G, D]. Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 softmax
// and epilogue (thread = row x one half of the 128 score columns; two warps share a TMEM quadrant, so every
// scheduler has two softmax warps to interleave). Every wait is bounded; a timeout raises the status word and the
// CTA drains.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kRows = 128;
constexpr int kBlkN = 128;
constexpr int kThreads = 320;
constexpr int kSoftmaxThreads = 256;
constexpr int kChunk = kRows * 128;   // 128 rows x 128 B (64 bf16) = 16 KB
constexpr float kLog2e = 1.4426950408889634f;

struct BwdItem {
  int tok0;        // dq: first query token of the tile; dkv: first key token of the block (row of the packed tensors)
  int seq_start;   // row of position 0 of the sequence
  int seq_end;     // one past the last row of the sequence
  int pad[5];
};

// ------------------------------------------------------------------------------------------------ delta
// delta[row] = sum_d out[row, d] * dout[row, d]; half a warp per row, 16-byte loads.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, long long rows, int D) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const int l16 = threadIdx.x & 15;
  float acc = 0.f;
  if (row < rows) {
    for (int i = l16 * 8; i < D; i += 128) {
      const uint4 a = *reinterpret_cast<const uint4*>(out + row * D + i);
      const uint4 b = *reinterpret_cast<const uint4*>(dout + row * D + i);
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        acc = __fadd_rn(acc, __fadd_rn(__fmul_rn(__low2float(pa[q]), __low2float(pb[q])), __fmul_rn(__high2float(pa[q]), __high2float(pb[q]))));
    }
  }
#pragma unroll
  for (int off = 8; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
  if (row < rows && l16 == 0) delta[row] = acc;
}

// One 32-column chunk of a score row -> p (bf16 pairs). s: raw TMEM words of S. Columns >= lim are masked.
__device__ __forceinline__ void chunk_p(const uint32_t (&s)[32], int col0, int lim, float scale_log2, float neg_lse2,
                                        uint32_t (&pk)[16]) {
  if (lim >= col0 + 32) {
#pragma unroll
    for (int i = 0; i < 32; i += 2)
      pk[i >> 1] = pack_bf2(ex2_approx(__fmaf_rn(__uint_as_float(s[i]), scale_log2, neg_lse2)),
                            ex2_approx(__fmaf_rn(__uint_as_float(s[i + 1]), scale_log2, neg_lse2)));
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float p0 = col0 + i < lim ? ex2_approx(__fmaf_rn(__uint_as_float(s[i]), scale_log2, neg_lse2)) : 0.f;
      const float p1 = col0 + i + 1 < lim ? ex2_approx(__fmaf_rn(__uint_as_float(s[i + 1]), scale_log2, neg_lse2)) : 0.f;
      pk[i >> 1] = pack_bf2(p0, p1);
    }
  }
}
// Same chunk -> ds = p * (dp * scale - delta * scale) (bf16 pairs).
__device__ __forceinline__ void chunk_ds(const uint32_t (&s)[32], const uint32_t (&dp)[32], int col0, int lim,
                                         float scale_log2, float neg_lse2, float scale, float neg_dscale, uint32_t (&dk)[16]) {
  if (lim >= col0 + 32) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const float p0 = ex2_approx(__fmaf_rn(__uint_as_float(s[i]), scale_log2, neg_lse2));
      const float p1 = ex2_approx(__fmaf_rn(__uint_as_float(s[i + 1]), scale_log2, neg_lse2));
      dk[i >> 1] = pack_bf2(__fmul_rn(p0, __fmaf_rn(__uint_as_float(dp[i]), scale, neg_dscale)),
                            __fmul_rn(p1, __fmaf_rn(__uint_as_float(dp[i + 1]), scale, neg_dscale)));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const bool v0 = col0 + i < lim, v1 = col0 + i + 1 < lim;
      const float p0 = v0 ? ex2_approx(__fmaf_rn(__uint_as_float(s[i]), scale_log2, neg_lse2)) : 0.f;
      const float p1 = v1 ? ex2_approx(__fmaf_rn(__uint_as_float(s[i + 1]), scale_log2, neg_lse2)) : 0.f;
      const float d0 = v0 ? __fmul_rn(p0, __fmaf_rn(__uint_as_float(dp[i]), scale, neg_dscale)) : 0.f;
      const float d1 = v1 ? __fmul_rn(p1, __fmaf_rn(__uint_as_float(dp[i + 1]), scale, neg_dscale)) : 0.f;
      dk[i >> 1] = pack_bf2(d0, d1);
    }
  }
}

// 32 bf16 of row r, columns [c*32, c*32+32) of a [128 rows x 128 cols] K-major SW128 tile (two 64-column chunks)
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int r, int c, const uint32_t (&pk)[16]) {
  uint8_t* rowp = tile + (c >> 1) * kChunk + r * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
    *reinterpret_cast<uint4*>(rowp + chunk * 16) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
  }
}

// TMEM accumulator row (W fp32 columns at `taddr`) -> bf16 in global memory
template <int W>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, __nv_bfloat16* dst, bool valid) {
#pragma unroll 1
  for (int c = 0; c < W / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c * 32, v);
    tmem_ld_wait_dep(v);
    if (valid) {
      uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 w;
        w.x = pack_bf2(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
        w.y = pack_bf2(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
        w.z = pack_bf2(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
        w.w = pack_bf2(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
        d4[i] = w;
      }
    }
  }
}

// A shared-memory descriptor is linear in the start address (field = address >> 4, 14 bits, and all of shared memory
// fits in them), so the descriptors of a tile's K steps are the tile's base descriptor plus constants: one 64-bit add
// per operand instead of rebuilding the descriptor in the single thread that issues every MMA.
__device__ __forceinline__ uint64_t desc_k(uint32_t smem_addr) { return make_sw128_desc(smem_addr, 16, 1024); }          // K-major
__device__ __forceinline__ uint64_t desc_mn(uint32_t smem_addr) { return make_sw128_desc(smem_addr, kChunk, 1024); }     // M/N-major

// S (or dP) = A[128 x D] B[128 x D]^T, both K-major tiles of ND 64-wide chunks
template <int ND>
__device__ __forceinline__ void mma_nt_128(uint32_t d_tmem, uint64_t dA, uint64_t dB, uint32_t idesc) {
#pragma unroll
  for (int dc = 0; dc < ND; ++dc)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t off = static_cast<uint64_t>((dc * kChunk + k * 32) >> 4);
      umma_f16_ss(d_tmem, dA + off, dB + off, idesc, (dc | k) != 0 ? 1u : 0u);
    }
}
// acc (+)= A^T-ish[128 x 128 rows] B[128 rows x N]: both operands M/N-major, the reduction runs over the 128 tile rows
// in 8 steps of 16 rows (2048 B)
__device__ __forceinline__ void mma_tn_128(uint32_t d_tmem, uint64_t dA, uint64_t dB, uint32_t idesc, bool first) {
#pragma unroll
  for (int k = 0; k < 8; ++k) umma_f16_ss(d_tmem, dA + static_cast<uint64_t>(k * 128), dB + static_cast<uint64_t>(k * 128), idesc, (first && k == 0) ? 0u : 1u);
}

// ------------------------------------------------------------------------------------------------ dQ
template <int ND>
struct DqSmem {
  static constexpr int kT = ND * kChunk;               // one [128 x D] tile
  static constexpr int offQ = 0;
  static constexpr int offdO = offQ + kT;
  static constexpr int offK = offdO + kT;              // two stages
  static constexpr int offV = offK + 2 * kT;           // two stages
  static constexpr int offdS = offV + 2 * kT;          // [128 rows x 128 keys] bf16
  static constexpr int offBar = offdS + 2 * kChunk;
  static constexpr int kBytes = offBar + 256 + 1024;
};
// SF: S and dP of a block are in TMEM; SR: the softmax warps have them in registers; DSF: dS is in shared memory;
// DQF: dQ += dS K of a block is done (dS buffer and K stage free)
enum { Q_QF = 0, Q_KF = 1, Q_KE = 3, Q_VF = 5, Q_VE = 7, Q_SF = 9, Q_SR = 10, Q_DSF = 11, Q_DQF = 12, kDqBars = 13 };

template <int ND>
__global__ void __launch_bounds__(kThreads, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const BwdItem* __restrict__ items, const float* __restrict__ lse, const float* __restrict__ delta,
               __nv_bfloat16* __restrict__ dq, int Hq, int Hkv, int G, float scale, int* __restrict__ status) {
  using SM = DqSmem<ND>;
  constexpr int D = 64 * ND;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::offBar);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + kDqBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TQ = kRows / G;
  const BwdItem it = items[blockIdx.x / Hkv];
  const int kvh = blockIdx.x % Hkv;
  int q_valid = it.seq_end - it.tok0;
  if (q_valid > TQ) q_valid = TQ;
  const int kv_hi = it.tok0 - it.seq_start + q_valid;        // the last valid row sees positions < kv_hi
  const int nb = (kv_hi + kBlkN - 1) / kBlkN;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kDqBars; ++i) mbar_init(smem_u32(&bars[i]), (i == Q_DSF || i == Q_SR) ? kSoftmaxThreads : 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<512>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dQ = tmem_base + 256;

  if (warp == 0) {
    if (elect_one() && nb > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const uint32_t bq = smem_u32(&bars[Q_QF]);
      mbar_arrive_expect_tx(bq, 2 * SM::kT);
#pragma unroll
      for (int dc = 0; dc < ND; ++dc) {
        tma_load_4d(smem_u32(smem + SM::offQ + dc * kChunk), &tmQ, bq, dc * 64, 0, kvh, it.tok0);
        tma_load_4d(smem_u32(smem + SM::offdO + dc * kChunk), &tmdO, bq, dc * 64, 0, kvh, it.tok0);
      }
      for (int j = 0; j < nb; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = it.seq_start + j * kBlkN;
        if (!mbar_wait(smem_u32(&bars[Q_KE + st]), ph ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t bk = smem_u32(&bars[Q_KF + st]);
        mbar_arrive_expect_tx(bk, SM::kT);
#pragma unroll
        for (int dc = 0; dc < ND; ++dc)
          tma_load_2d(smem_u32(smem + SM::offK + st * SM::kT + dc * kChunk), &tmK, bk, kvh * D + dc * 64, row);
        if (!mbar_wait(smem_u32(&bars[Q_VE + st]), ph ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t bv = smem_u32(&bars[Q_VF + st]);
        mbar_arrive_expect_tx(bv, SM::kT);
#pragma unroll
        for (int dc = 0; dc < ND; ++dc)
          tma_load_2d(smem_u32(smem + SM::offV + st * SM::kT + dc * kChunk), &tmV, bv, kvh * D + dc * 64, row);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nb > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kRows, kBlkN, 0, 0);
      constexpr uint32_t idesc_q = make_idesc_bf16(kRows, D, 0, 1);       // B = K read MN-major (keys are the reduction)
      const uint64_t dQd = desc_k(smem_u32(smem + SM::offQ)), ddO = desc_k(smem_u32(smem + SM::offdO));
      const uint64_t ddS = desc_k(smem_u32(smem + SM::offdS));
      // S and dP of block j into TMEM (their columns are free once the softmax warps hold block j-1 in registers)
      auto front = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&bars[Q_KF + st]), ph, abort_flag, status, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(smem_u32(&bars[Q_VF + st]), ph, abort_flag, status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        mma_nt_128<ND>(tmem_S, dQd, desc_k(smem_u32(smem + SM::offK + st * SM::kT)), idesc_s);
        mma_nt_128<ND>(tmem_dP, ddO, desc_k(smem_u32(smem + SM::offV + st * SM::kT)), idesc_s);
        umma_commit(smem_u32(&bars[Q_VE + st]));
        umma_commit(smem_u32(&bars[Q_SF]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&bars[Q_QF]), 0, abort_flag, status, ST_TIMEOUT_FULL);
      if (ok) ok = front(0);
      for (int j = 0; j < nb && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < nb) {
          if (!mbar_wait(smem_u32(&bars[Q_SR]), j & 1, abort_flag, status, ST_TIMEOUT_MISC)) break;
          if (!front(j + 1)) break;
        }
        if (!mbar_wait(smem_u32(&bars[Q_DSF]), j & 1, abort_flag, status, ST_TIMEOUT_MISC)) break;
        tc_fence_after();
        // A = dS, K-major (two 64-key chunks); B = K block read M/N-major (16 keys = 2048 B per step)
        const uint64_t dKm = desc_mn(smem_u32(smem + SM::offK + st * SM::kT));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tmem_dQ, ddS + static_cast<uint64_t>(((k >> 2) * kChunk + (k & 3) * 32) >> 4), dKm + static_cast<uint64_t>(k * 128),
                      idesc_q, (j | k) != 0 ? 1u : 0u);
        umma_commit(smem_u32(&bars[Q_KE + st]));
        umma_commit(smem_u32(&bars[Q_DQF]));
      }
    }
  } else {
    const int quad = warp & 3;                 // TMEM quadrant this warp may read
    const int chalf = (warp - 2) >> 2;         // which 64 of the 128 score columns
    const int r = quad * 32 + lane;
    const int tok = r / G;
    const int hq = kvh * G + (r % G);
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const bool row_valid = tok < q_valid;
    const size_t orow = static_cast<size_t>(it.tok0 + (row_valid ? tok : 0)) * Hq + hq;
    const float scale_log2 = scale * kLog2e;
    const float neg_lse2 = row_valid ? -lse[orow] * kLog2e : 0.f;
    const float neg_dscale = row_valid ? -delta[orow] * scale : 0.f;
    const int q_pos = it.tok0 - it.seq_start + tok;
    const int seq_len = it.seq_end - it.seq_start;
    uint8_t* sdS = smem + SM::offdS;
    bool ok = nb > 0;
    for (int j = 0; j < nb && ok; ++j) {
      if (!mbar_wait(smem_u32(&bars[Q_SF]), j & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * kBlkN;
      int lim = q_pos - key0 + 1;
      if (seq_len - key0 < lim) lim = seq_len - key0;
      if (!row_valid) lim = 0;
      uint32_t s0[32], s1[32], d0[32], d1[32], dk[16], dk2[16];
      tmem_ld_32x32(tmem_S + lane_off + chalf * 64, s0);
      tmem_ld_32x32(tmem_S + lane_off + chalf * 64 + 32, s1);
      tmem_ld_32x32(tmem_dP + lane_off + chalf * 64, d0);
      tmem_ld_32x32(tmem_dP + lane_off + chalf * 64 + 32, d1);
      tmem_ld_wait_dep(s0);
      tmem_ld_wait_dep(s1);
      tmem_ld_wait_dep(d0);
      tmem_ld_wait_dep(d1);
      tc_fence_before();
      mbar_arrive(smem_u32(&bars[Q_SR]));       // S and dP are in registers: the next block's MMAs may overwrite them
      // both chunks are computed before the first store, so the wait for the buffer comes as late as possible
      chunk_ds(s0, d0, chalf * 64, lim, scale_log2, neg_lse2, scale, neg_dscale, dk);
      chunk_ds(s1, d1, chalf * 64 + 32, lim, scale_log2, neg_lse2, scale, neg_dscale, dk2);
      if (j > 0) {
        // the dS buffer is still the A operand of dQ += dS K of block j-1
        if (!mbar_wait(smem_u32(&bars[Q_DQF]), (j - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
      }
      store_row_chunk(sdS, r, chalf * 2, dk);
      store_row_chunk(sdS, r, chalf * 2 + 1, dk2);
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(smem_u32(&bars[Q_DSF]));
    }
    if (ok && mbar_wait(smem_u32(&bars[Q_DQF]), (nb - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      store_acc_row<D / 2>(tmem_dQ + lane_off + chalf * (D / 2), dq + orow * D + chalf * (D / 2), row_valid);
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------------------ dV and dK
// WHICH = 0: dV += P^T dO (needs K, Q, dO; no V, no delta). WHICH = 1: dK += dS^T Q (needs K, V, Q, dO).
template <int ND>
struct DkvSmem {
  static constexpr int kT = ND * kChunk;
  static constexpr int offK = 0;
  static constexpr int offV = offK + kT;               // unused by the dV kernel
  static constexpr int offQ = offV + kT;               // two stages
  static constexpr int offdO = offQ + 2 * kT;          // two stages
  static constexpr int offP = offdO + 2 * kT;          // P (dV) or dS (dK): [128 rows x 128 keys] bf16
  static constexpr int offBar = offP + 2 * kChunk;
  static constexpr int kBytes = offBar + 256 + 1024;
};
// SF / SR as above; PF: P or dS is in shared memory; PE: the accumulating MMA that read it is done
enum { K_KVF = 0, K_QF = 1, K_QE = 3, K_OF = 5, K_OE = 7, K_SF = 9, K_SR = 10, K_PF = 11, K_PE = 12, kDkvBars = 13 };

template <int ND, int WHICH>
__global__ void __launch_bounds__(kThreads, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const BwdItem* __restrict__ items, const float* __restrict__ lse, const float* __restrict__ delta,
                __nv_bfloat16* __restrict__ dst, int Hq, int Hkv, int G, float scale, int* __restrict__ status) {
  using SM = DkvSmem<ND>;
  constexpr int D = 64 * ND;
  constexpr bool kDK = WHICH == 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::offBar);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + kDkvBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TQ = kRows / G;
  const BwdItem it = items[blockIdx.x / Hkv];
  const int kvh = blockIdx.x % Hkv;
  int n_keys = it.seq_end - it.tok0;
  const int nq = (n_keys + TQ - 1) / TQ;                 // query tiles from the block's first key to the end of the sequence
  if (n_keys > kBlkN) n_keys = kBlkN;
  const int key_pos0 = it.tok0 - it.seq_start;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kDkvBars; ++i) mbar_init(smem_u32(&bars[i]), (i == K_PF || i == K_SR) ? kSoftmaxThreads : 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<512>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_acc = tmem_base + 256;

  if (warp == 0) {
    if (elect_one() && nq > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmdO);
      tma_prefetch_desc(&tmK);
      if (kDK) tma_prefetch_desc(&tmV);
      const uint32_t bkv = smem_u32(&bars[K_KVF]);
      mbar_arrive_expect_tx(bkv, (kDK ? 2 : 1) * SM::kT);
#pragma unroll
      for (int dc = 0; dc < ND; ++dc) {
        tma_load_2d(smem_u32(smem + SM::offK + dc * kChunk), &tmK, bkv, kvh * D + dc * 64, it.tok0);
        if (kDK) tma_load_2d(smem_u32(smem + SM::offV + dc * kChunk), &tmV, bkv, kvh * D + dc * 64, it.tok0);
      }
      for (int i = 0; i < nq; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int t0 = it.tok0 + i * TQ;
        if (!mbar_wait(smem_u32(&bars[K_QE + st]), ph ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t bq = smem_u32(&bars[K_QF + st]);
        mbar_arrive_expect_tx(bq, SM::kT);
#pragma unroll
        for (int dc = 0; dc < ND; ++dc)
          tma_load_4d(smem_u32(smem + SM::offQ + st * SM::kT + dc * kChunk), &tmQ, bq, dc * 64, 0, kvh, t0);
        if (!mbar_wait(smem_u32(&bars[K_OE + st]), ph ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t bo = smem_u32(&bars[K_OF + st]);
        mbar_arrive_expect_tx(bo, SM::kT);
#pragma unroll
        for (int dc = 0; dc < ND; ++dc)
          tma_load_4d(smem_u32(smem + SM::offdO + st * SM::kT + dc * kChunk), &tmdO, bo, dc * 64, 0, kvh, t0);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nq > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kRows, kBlkN, 0, 0);
      constexpr uint32_t idesc_t = make_idesc_bf16(kRows, D, 1, 1);       // A = P^T / dS^T and B = dO / Q, both M/N-major
      const uint64_t dKd = desc_k(smem_u32(smem + SM::offK)), dVd = desc_k(smem_u32(smem + SM::offV));
      const uint64_t dPm = desc_mn(smem_u32(smem + SM::offP));
      // S (and dP) of tile i; dV: Q is free after S. dK: dO is free after dP.
      auto front = [&](int i) -> bool {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(smem_u32(&bars[K_QF + st]), ph, abort_flag, status, ST_TIMEOUT_FULL)) return false;
        if (kDK && !mbar_wait(smem_u32(&bars[K_OF + st]), ph, abort_flag, status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        mma_nt_128<ND>(tmem_S, desc_k(smem_u32(smem + SM::offQ + st * SM::kT)), dKd, idesc_s);
        if (kDK) {
          mma_nt_128<ND>(tmem_dP, desc_k(smem_u32(smem + SM::offdO + st * SM::kT)), dVd, idesc_s);
          umma_commit(smem_u32(&bars[K_OE + st]));
        } else {
          umma_commit(smem_u32(&bars[K_QE + st]));
        }
        umma_commit(smem_u32(&bars[K_SF]));
        return true;
      };
      // acc += (P or dS of tile i)^T (dO or Q of tile i)
      auto back = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(smem_u32(&bars[K_PF]), i & 1, abort_flag, status, ST_TIMEOUT_MISC)) return false;
        if (!kDK && !mbar_wait(smem_u32(&bars[K_OF + st]), (i >> 1) & 1, abort_flag, status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        mma_tn_128(tmem_acc, dPm, desc_mn(smem_u32(smem + (kDK ? SM::offQ : SM::offdO) + st * SM::kT)), idesc_t, i == 0);
        umma_commit(smem_u32(&bars[(kDK ? K_QE : K_OE) + st]));
        umma_commit(smem_u32(&bars[K_PE]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&bars[K_KVF]), 0, abort_flag, status, ST_TIMEOUT_FULL);
      if (ok) ok = front(0);
      for (int i = 0; i < nq && ok; ++i) {
        if (i + 1 < nq) {
          if (!mbar_wait(smem_u32(&bars[K_SR]), i & 1, abort_flag, status, ST_TIMEOUT_MISC)) break;
          if (!front(i + 1)) break;
        }
        if (!back(i)) break;
      }
    }
  } else {
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int tok = r / G;
    const int hq = kvh * G + (r % G);
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float scale_log2 = scale * kLog2e;
    uint8_t* sP = smem + SM::offP;
    bool ok = nq > 0;
    // row statistics of tile i + 1 are fetched while tile i is being processed (a global load per tile would
    // otherwise sit in front of every tile's exponentials)
    auto row_stats = [&](int i, float& l2, float& ds) {
      const int t = it.tok0 + i * TQ + tok;
      const bool valid = i < nq && t < it.seq_end;
      const size_t srow = static_cast<size_t>(valid ? t : it.tok0) * Hq + hq;
      l2 = valid ? -lse[srow] * kLog2e : 0.f;
      ds = (kDK && valid) ? -delta[srow] * scale : 0.f;
    };
    float nxt_lse2 = 0.f, nxt_dscale = 0.f;
    row_stats(0, nxt_lse2, nxt_dscale);
    for (int i = 0; i < nq && ok; ++i) {
      const int t = it.tok0 + i * TQ + tok;                 // this row's token
      const bool row_valid = t < it.seq_end;
      const float neg_lse2 = nxt_lse2, neg_dscale = nxt_dscale;
      row_stats(i + 1, nxt_lse2, nxt_dscale);
      int lim = (t - it.seq_start) - key_pos0 + 1;          // keys [0, lim) of the block are visible to this row
      if (n_keys < lim) lim = n_keys;
      if (!row_valid) lim = 0;
      if (!mbar_wait(smem_u32(&bars[K_SF]), i & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t s0[32], s1[32], pk[16], pk2[16];
      tmem_ld_32x32(tmem_S + lane_off + chalf * 64, s0);
      tmem_ld_32x32(tmem_S + lane_off + chalf * 64 + 32, s1);
      if (kDK) {
        uint32_t d0[32], d1[32];
        tmem_ld_32x32(tmem_dP + lane_off + chalf * 64, d0);
        tmem_ld_32x32(tmem_dP + lane_off + chalf * 64 + 32, d1);
        tmem_ld_wait_dep(s0);
        tmem_ld_wait_dep(s1);
        tmem_ld_wait_dep(d0);
        tmem_ld_wait_dep(d1);
        tc_fence_before();
        mbar_arrive(smem_u32(&bars[K_SR]));
        chunk_ds(s0, d0, chalf * 64, lim, scale_log2, neg_lse2, scale, neg_dscale, pk);
        chunk_ds(s1, d1, chalf * 64 + 32, lim, scale_log2, neg_lse2, scale, neg_dscale, pk2);
        if (i > 0) {
          if (!mbar_wait(smem_u32(&bars[K_PE]), (i - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        }
        store_row_chunk(sP, r, chalf * 2, pk);
        store_row_chunk(sP, r, chalf * 2 + 1, pk2);
      } else {
        tmem_ld_wait_dep(s0);
        tmem_ld_wait_dep(s1);
        tc_fence_before();
        mbar_arrive(smem_u32(&bars[K_SR]));
        chunk_p(s0, chalf * 64, lim, scale_log2, neg_lse2, pk);
        chunk_p(s1, chalf * 64 + 32, lim, scale_log2, neg_lse2, pk2);
        if (i > 0) {
          if (!mbar_wait(smem_u32(&bars[K_PE]), (i - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        }
        store_row_chunk(sP, r, chalf * 2, pk);
        store_row_chunk(sP, r, chalf * 2 + 1, pk2);
      }
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(smem_u32(&bars[K_PF]));
    }
    if (ok && mbar_wait(smem_u32(&bars[K_PE]), (nq - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      // accumulator lanes are keys; each of the two warps of a quadrant writes half of the D columns
      const bool key_valid = r < n_keys;
      const size_t krow = static_cast<size_t>(it.tok0 + (key_valid ? r : 0)) * Hkv + kvh;
      store_acc_row<D / 2>(tmem_acc + lane_off + chalf * (D / 2), dst + krow * D + chalf * (D / 2), key_valid);
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

template <int ND>
int launch_bwd(const void* q, const void* k, const void* v, const void* out, const void* lse, const void* dout, void* dq,
               void* dk, void* dv, void* delta, const void* items_q, int n_q, const void* items_kv, int n_kv, int T, int Hq,
               int Hkv, float scale, cudaStream_t stream, int dev) {
  constexpr int D = 64 * ND;
  const int G = Hq / Hkv;
  const int TQ = kRows / G;
  {
    const long long rows = static_cast<long long>(T) * Hq;
    const int rpb = 16;                                   // rows per block (256 threads, 16 lanes per row)
    attn_delta_kernel<<<static_cast<unsigned>((rows + rpb - 1) / rpb), rpb * 16, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), static_cast<float*>(delta), rows, D);
    IX_CUDA(cudaGetLastError());
  }
  CUtensorMap tmQ, tmdO, tmK, tmV;
  {
    uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(G), static_cast<uint64_t>(Hkv), static_cast<uint64_t>(T)};
    uint64_t strides[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(G) * D * 2, static_cast<uint64_t>(Hq) * D * 2};
    uint32_t box[4] = {64, static_cast<uint32_t>(G), 1, static_cast<uint32_t>(TQ)};
    int rc = ixh::make_tmap(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, q, dims, strides, box);
    if (rc) return rc;
    rc = ixh::make_tmap(&tmdO, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dout, dims, strides, box);
    if (rc) return rc;
  }
  int rc = ixh::make_tmap_bf16_2d(&tmK, k, T, static_cast<uint64_t>(Hkv) * D, static_cast<uint64_t>(Hkv) * D, kBlkN);
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmV, v, T, static_cast<uint64_t>(Hkv) * D, static_cast<uint64_t>(Hkv) * D, kBlkN);
  if (rc) return rc;
  auto kq = attn_dq_kernel<ND>;
  auto kdv = attn_dkv_kernel<ND, 0>;
  auto kdk = attn_dkv_kernel<ND, 1>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<ND>::kBytes));
    IX_CUDA(cudaFuncSetAttribute(kdv, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<ND>::kBytes));
    IX_CUDA(cudaFuncSetAttribute(kdk, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<ND>::kBytes));
    attr_set[dev & 63] = true;
  }
  int* status = ixh::status_word(dev);
  const float* lsep = static_cast<const float*>(lse);
  const float* dlt = static_cast<const float*>(delta);
  if (n_kv > 0) {
    const unsigned grid = static_cast<unsigned>(n_kv) * Hkv;
    kdv<<<grid, kThreads, DkvSmem<ND>::kBytes, stream>>>(tmQ, tmdO, tmK, tmV, static_cast<const BwdItem*>(items_kv), lsep, dlt,
                                                         static_cast<__nv_bfloat16*>(dv), Hq, Hkv, G, scale, status);
    IX_CUDA(cudaGetLastError());
    kdk<<<grid, kThreads, DkvSmem<ND>::kBytes, stream>>>(tmQ, tmdO, tmK, tmV, static_cast<const BwdItem*>(items_kv), lsep, dlt,
                                                         static_cast<__nv_bfloat16*>(dk), Hq, Hkv, G, scale, status);
    IX_CUDA(cudaGetLastError());
  }
  if (n_q > 0) {
    kq<<<static_cast<unsigned>(n_q) * Hkv, kThreads, DqSmem<ND>::kBytes, stream>>>(
        tmQ, tmdO, tmK, tmV, static_cast<const BwdItem*>(items_q), lsep, dlt, static_cast<__nv_bfloat16*>(dq), Hq, Hkv, G, scale, status);
    IX_CUDA(cudaGetLastError());
  }
  return 0;
}

}  // namespace

// Backward of the packed varlen causal attention. q, out, dout, dq: [T, Hq, D] bf16; k, v, dk, dv: [T, Hkv, D] bf16
// (contiguous keys: row of position p of a sequence = seq_start + p); lse: [T, Hq] fp32 from the forward; delta:
// [T, Hq] fp32 scratch. items_q: one BwdItem per query tile of 128 / (Hq / Hkv) tokens; items_kv: one per block of 128
// keys; both int32 [n, 8], heaviest first. Every row of dq, dk, dv that belongs to a sequence is written.
IX_API int ix_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* lse, const void* dout,
                            void* dq, void* dk, void* dv, void* delta, const void* items_q, int n_q, const void* items_kv,
                            int n_kv, int T, int Hq, int Hkv, int D, float scale, void* stream) {
  if (T <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv) return ixh::fail(ixh::IX_EARG, "attention bwd: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  const int G = Hq / Hkv;
  if (G > 128 || (128 % G)) return ixh::fail(ixh::IX_EARG, "attention bwd: group size %d must divide 128", G);
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_bwd<2>(q, k, v, out, lse, dout, dq, dk, dv, delta, items_q, n_q, items_kv, n_kv, T, Hq, Hkv, scale, s, dev);
  if (D == 64) return launch_bwd<1>(q, k, v, out, lse, dout, dq, dk, dv, delta, items_q, n_q, items_kv, n_kv, T, Hq, Hkv, scale, s, dev);
  return ixh::fail(ixh::IX_EARG, "attention bwd: head dim %d unsupported (64 or 128)", D);
}
