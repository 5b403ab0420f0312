// Causal GQA attention forward for sm_100a: ONE kernel for the trainer's packed varlen
// forward, the engine's (chunked) prefill and the engine's paged decode, so the three
// sites produce the same bits per (token, head) by construction.
//
// Invariance rules (what the reference gets from FlashAttention-3 pinned to num_splits=1 on
// both sides, ISO/ops/attention/_register.py:15-77):
//   * keys are consumed in blocks of 128 aligned to position 0 of the sequence, in
//     ascending order, never split across CTAs; the online-softmax state of a row
//     (m, l, O) is updated once per block in that order;
//   * a row of the 128-row tile belongs to one (token, query head); the tcgen05 MMAs and
//     the per-row softmax never mix rows, so a token's result is the same whether its tile
//     holds 127 other real rows (prefill / training) or padding (decode);
//   * a block that is entirely masked for a row leaves that row's state untouched
//     (alpha = 1, p = 0).
//
// Tile rows are GQA-packed: row r = (token r / G, head g0*G + r % G) for one KV head g0,
// fetched with one 4D TMA box over Q viewed as [T, Hkv, G, D]. K and V come from a slot
// pool [num_slots, Hkv, D] through a block table (page = 128 slots) or contiguously.
//
// Persistent CTAs (one per SM) walk the (tile, KV head) work list; the producer runs ahead across work items.
// Roles (192 threads): warp 0 TMA producer, warp 1 tcgen05.mma issuer, warps 2..5 softmax
// (thread = row). TMEM: two S buffers (128 cols each) + one O buffer (D cols).
// Pipeline: S_{j+1} = Q K_{j+1}^T is issued while the softmax of block j runs; O += P V_j
// accumulates in TMEM. The exponent reference m of a row moves lazily (only when the running
// maximum grew by more than 8 in log2 units), so the softmax threads rescale O in TMEM rarely
// and otherwise only read the scores once, exponentiate and hand P to the tensor core.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kRows = 128;   // tile rows (queries x heads-in-group)
constexpr int kBlkN = 128;   // keys per block == page size
constexpr int kAttnThreads = 192;

struct WorkItem {
  int q_start;   // first query token (row of Q / out)
  int q_len;     // query tokens in this tile (<= 128 / G)
  int q_pos0;    // position of the first query token inside its sequence
  int kv_len;    // keys visible to the sequence (positions 0 .. kv_len-1 exist)
  int bt_row;    // row of the block table, or -1 for contiguous keys
  int kv_start;  // contiguous mode: slot of position 0
  int pad0, pad1;
};

template <int ND>  // head dim = 64 * ND
struct AttnSmem {
  static constexpr int kChunk = kRows * 128;                 // 128 rows x 128 B = 16 KB
  static constexpr int kQ = ND * kChunk;
  static constexpr int kKV = ND * kChunk;                    // one K or V block
  static constexpr int kP = 2 * kChunk;                      // 128 rows x 128 keys bf16
  static constexpr int offQ = 0;                             // two Q tiles: the next work item's Q loads during this one
  static constexpr int offK = offQ + 2 * kQ;
  static constexpr int offV = offK + 2 * kKV;
  static constexpr int offP = offV + 2 * kKV;
  static constexpr int offBar = offP + kP;
  static constexpr int kBytes = offBar + 256 + 1024;
};

// Barriers. Stage rings (K, V, S) and the once-per-block barriers (P, O_full) are indexed by a block counter that
// runs across the work items of a CTA; Q and O_empty by the item counter.
enum { B_QF = 0, B_QE = 2, B_KF = 4, B_KE = 6, B_VF = 8, B_VE = 10, B_SF = 12, B_PF = 14, B_OF = 15, B_OE = 16, kNumBars = 17 };

struct ItemGeom {
  WorkItem it;
  int kvh, q_valid, nb;
};

__device__ __forceinline__ ItemGeom item_geom(const WorkItem* items, int w, int num_items, int TQ) {
  ItemGeom g;
  g.it = items[w % num_items];      // items vary fastest: neighbouring CTAs work on the same KV head of neighbouring tiles
  g.kvh = w / num_items;
  g.q_valid = g.it.q_len < TQ ? g.it.q_len : TQ;
  int kv_hi = g.it.q_pos0 + g.q_valid;  // causal: last row sees positions < q_pos0 + q_valid
  if (kv_hi > g.it.kv_len) kv_hi = g.it.kv_len;
  g.nb = (kv_hi + kBlkN - 1) / kBlkN;
  return g;
}

// Persistent: a CTA walks the (tile, KV head) work list with stride gridDim.x. The producer runs ahead across work
// items (the next item's Q and first K/V blocks load while the current item's last blocks and epilogue run), so an SM
// keeps streaming K/V instead of draining and refilling its pipeline for every item.
template <int ND>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const WorkItem* __restrict__ items, int num_items,
                     const int* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ out,
                     float* __restrict__ lse_out, int Hq, int Hkv, int G, float scale_log2, int* __restrict__ status) {
  using SM = AttnSmem<ND>;
  constexpr int D = 64 * ND;
  constexpr int kTmemCols = 512;  // S0 | S1 | O  (2*128 + D <= 512, power of two)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::offBar);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TQ = kRows / G;
  const int total = num_items * Hkv;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kNumBars; ++i) mbar_init(smem_u32(&bars[i]), (i == B_PF || i == B_OE) ? 128 : 1);
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
  const uint32_t tmem_S0 = tmem_base, tmem_O = tmem_base + 256;
  pdl_launch_dependents();
  pdl_wait();   // Q, the K/V slots of this step and the work list come from the kernels before this one

  if (warp == 0) {
    // -------------------------------------------------------------- producer
    if (elect_one()) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      uint32_t jb = 0, qi = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const ItemGeom g = item_geom(items, w, num_items, TQ);
        if (g.nb == 0) continue;
        const int qs = qi & 1;
        if (!mbar_wait(smem_u32(&bars[B_QE + qs]), ((qi >> 1) & 1) ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) break;
        const uint32_t bq = smem_u32(&bars[B_QF + qs]);
        mbar_arrive_expect_tx(bq, SM::kQ);
#pragma unroll
        for (int dc = 0; dc < ND; ++dc)
          tma_load_4d(smem_u32(smem + SM::offQ + qs * SM::kQ + dc * SM::kChunk), &tmQ, bq, dc * 64, 0, g.kvh, g.it.q_start);
        for (int j = 0; j < g.nb; ++j, ++jb) {
          const int st = jb & 1;
          const uint32_t ph = (jb >> 1) & 1;
          int row;
          if (g.it.bt_row >= 0) row = block_table[static_cast<size_t>(g.it.bt_row) * bt_stride + j] * kBlkN;
          else row = g.it.kv_start + j * kBlkN;
          if (!mbar_wait(smem_u32(&bars[B_KE + st]), ph ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t bk = smem_u32(&bars[B_KF + st]);
          mbar_arrive_expect_tx(bk, SM::kKV);
#pragma unroll
          for (int dc = 0; dc < ND; ++dc)
            tma_load_2d(smem_u32(smem + SM::offK + st * SM::kKV + dc * SM::kChunk), &tmK, bk, g.kvh * D + dc * 64, row);
          if (!mbar_wait(smem_u32(&bars[B_VE + st]), ph ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          const uint32_t bv = smem_u32(&bars[B_VF + st]);
          mbar_arrive_expect_tx(bv, SM::kKV);
#pragma unroll
          for (int dc = 0; dc < ND; ++dc)
            tma_load_2d(smem_u32(smem + SM::offV + st * SM::kKV + dc * SM::kChunk), &tmV, bv, g.kvh * D + dc * 64, row);
        }
        ++qi;
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kRows, kBlkN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(kRows, D, 0, 1);  // V is MN-major
      const uint32_t sP = smem_u32(smem + SM::offP);
      uint32_t jb0 = 0, qi = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        const ItemGeom g = item_geom(items, w, num_items, TQ);
        if (g.nb == 0) continue;
        const int nb = g.nb;
        const int qs = qi & 1;
        const uint32_t sQ = smem_u32(smem + SM::offQ + qs * SM::kQ);
        ok = mbar_wait(smem_u32(&bars[B_QF + qs]), (qi >> 1) & 1, abort_flag, status, ST_TIMEOUT_FULL);
        auto issue_qk = [&](int j) -> bool {
          const uint32_t b = jb0 + j;
          const int st = b & 1;
          if (!mbar_wait(smem_u32(&bars[B_KF + st]), (b >> 1) & 1, abort_flag, status, ST_TIMEOUT_FULL)) return false;
          tc_fence_after();
          const uint32_t sK = smem_u32(smem + SM::offK + st * SM::kKV);
#pragma unroll
          for (int dc = 0; dc < ND; ++dc)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_ss(tmem_S0 + st * 128, make_sw128_desc(sQ + dc * SM::kChunk + k * 32, 16, 1024),
                          make_sw128_desc(sK + dc * SM::kChunk + k * 32, 16, 1024), idesc_s, (dc | k) != 0 ? 1u : 0u);
          umma_commit(smem_u32(&bars[B_KE + st]));   // K stage free
          umma_commit(smem_u32(&bars[B_SF + st]));   // S ready
          if (j == nb - 1) umma_commit(smem_u32(&bars[B_QE + qs]));   // last use of this Q tile
          return true;
        };
        // S[b & 1] was last read by the softmax of block b - 2, which finished before P_full(b - 2): waited below
        if (ok) ok = issue_qk(0);
        for (int j = 0; j < nb && ok; ++j) {
          if (j + 1 < nb) {
            if (!issue_qk(j + 1)) { ok = false; break; }
          }
          const uint32_t b = jb0 + j;
          const int st = b & 1;
          if (!mbar_wait(smem_u32(&bars[B_PF]), b & 1, abort_flag, status, ST_TIMEOUT_MISC)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&bars[B_VF + st]), (b >> 1) & 1, abort_flag, status, ST_TIMEOUT_FULL)) { ok = false; break; }
          if (j == 0 && qi > 0) {
            // the first P V of an item overwrites O: the previous item's epilogue must have read it out
            if (!mbar_wait(smem_u32(&bars[B_OE]), (qi - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t sV = smem_u32(smem + SM::offV + st * SM::kKV);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            // A = P (K-major): 64-key atoms 16 KB apart, 32 B per K=16 step inside an atom
            const uint64_t da = make_sw128_desc(sP + (k >> 2) * SM::kChunk + (k & 3) * 32, 16, 1024);
            // B = V (MN-major): 16 keys = 2 groups of 8 rows (SBO 1024 B); 64-wide d chunks LBO apart
            const uint64_t db = make_sw128_desc(sV + k * 2048, SM::kChunk, 1024);
            umma_f16_ss(tmem_O, da, db, idesc_o, (j | k) != 0 ? 1u : 0u);   // O accumulates over the item's blocks in TMEM
          }
          umma_commit(smem_u32(&bars[B_VE + st]));  // V stage free
          umma_commit(smem_u32(&bars[B_OF]));       // O_blk ready, P buffer free
        }
        jb0 += nb;
        ++qi;
      }
    }
  } else {
    // -------------------------------------------------------------- softmax / epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;             // tile row
    const int tok = r / G;                      // token inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* sP = smem + SM::offP;
    uint32_t jb0 = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      const ItemGeom g = item_geom(items, w, num_items, TQ);
      if (g.nb == 0) continue;
      const WorkItem& it = g.it;
      const int nb = g.nb, q_valid = g.q_valid;
      const int hq = g.kvh * G + (r % G);
      const bool row_valid = tok < q_valid;
      const int q_pos = it.q_pos0 + (row_valid ? tok : q_valid - 1);
      // m is the exponent reference of the row. It follows the running maximum lazily: it only moves
      // when the maximum has grown by more than 8 (log2 units) since it was last set, so O (which
      // accumulates in TMEM) is rescaled rarely. p = exp2(t - m) is then at most 2^8; l and O are
      // both relative to the same m, so O / l is exact softmax. The rule is per row.
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < nb && ok; ++j) {
        const uint32_t b = jb0 + j;
        const int st = b & 1;
        if (!mbar_wait(smem_u32(&bars[B_SF + st]), (b >> 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tS = tmem_S0 + st * 128 + lane_off;
        const int key0 = j * kBlkN;
        int lim = q_pos - key0 + 1;               // keys [0, lim) of this block are visible
        const int lim2 = it.kv_len - key0;
        if (lim2 < lim) lim = lim2;
        // the whole score row goes to registers once: four loads in flight, then the waits
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_32x32(tS, s0);
        tmem_ld_32x32(tS + 32, s1);
        tmem_ld_32x32(tS + 64, s2);
        tmem_ld_32x32(tS + 96, s3);
        tmem_ld_wait_dep(s0);
        tmem_ld_wait_dep(s1);
        tmem_ld_wait_dep(s2);
        tmem_ld_wait_dep(s3);
        // Row maximum on the raw scores (scale > 0, so max(s)*scale == max(s*scale)); a block that is
        // fully visible to every row of the warp skips the per-element mask test.
        const bool full_blk = __all_sync(0xffffffffu, lim >= kBlkN);
        float mraw = -INFINITY;
        if (full_blk) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            mraw = fmaxf(mraw, fmaxf(fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])),
                                     fmaxf(__uint_as_float(s2[i]), __uint_as_float(s3[i]))));
          }
        } else {
#define IX_MASK_MAX(S_, C_)                                                         \
  _Pragma("unroll") for (int i = 0; i < 32; ++i) {                                  \
    if ((C_) * 32 + i >= lim) S_[i] = 0xff800000u; /* -inf */                       \
    mraw = fmaxf(mraw, __uint_as_float(S_[i]));                                     \
  }
          IX_MASK_MAX(s0, 0)
          IX_MASK_MAX(s1, 1)
          IX_MASK_MAX(s2, 2)
          IX_MASK_MAX(s3, 3)
#undef IX_MASK_MAX
        }
        const float mb = __fmul_rn(mraw, scale_log2);
        const float m_new = fmaxf(m, mb);
        float alpha = 1.f;
        if (__fsub_rn(m_new, m) > 8.0f) {         // also true for the first visible block (m = -inf)
          alpha = (m == -INFINITY) ? 0.f : ex2_approx(__fsub_rn(m, m_new));
          m = m_new;
        }
        const bool any_rescale = __any_sync(0xffffffffu, alpha != 1.f);
        // P V of block j-1 must have finished: the P buffer is reused and O may be rescaled. (For j == 0 the buffer
        // was last read by the previous item's last P V, which this thread waited for in that item's epilogue.)
        if (j > 0) {
          if (!mbar_wait(smem_u32(&bars[B_OF]), (b - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          if (any_rescale) {
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t v[32];
              tmem_ld_32x32(tmem_O + lane_off + c * 32, v);
              tmem_ld_wait_dep(v);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__fmul_rn(__uint_as_float(v[i]), alpha));
              tmem_st_32x32(tmem_O + lane_off + c * 32, v);
            }
            tmem_st_wait();
          }
        }
        if (alpha != 1.f) l = __fmul_rn(l, alpha);
        // p = exp2(s*scale - m): one FMA and one ex2.approx per element (masked scores are -inf -> p = 0);
        // the row sum adds the pair (p_i + p_{i+1}) left to right
        const float neg_m = -m;
#define IX_EXP_STORE(S_, C_)                                                                         \
  {                                                                                                  \
    uint32_t pk[16];                                                                                 \
    _Pragma("unroll") for (int i = 0; i < 32; i += 2) {                                              \
      const float p0 = ex2_approx(__fmaf_rn(__uint_as_float(S_[i]), scale_log2, neg_m));             \
      const float p1 = ex2_approx(__fmaf_rn(__uint_as_float(S_[i + 1]), scale_log2, neg_m));         \
      l = __fadd_rn(l, __fadd_rn(p0, p1));                                                           \
      pk[i >> 1] = pack_bf2(p0, p1);                                                                 \
    }                                                                                                \
    uint8_t* rowp = sP + ((C_) >> 1) * SM::kChunk + r * 128;                                         \
    _Pragma("unroll") for (int q = 0; q < 4; ++q) {                                                  \
      const int chunk = (((C_) & 1) * 4 + q) ^ (r & 7);                                              \
      *reinterpret_cast<uint4*>(rowp + chunk * 16) =                                                 \
          make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);                        \
    }                                                                                                \
  }
        IX_EXP_STORE(s0, 0)
        IX_EXP_STORE(s1, 1)
        IX_EXP_STORE(s2, 2)
        IX_EXP_STORE(s3, 3)
#undef IX_EXP_STORE
        tc_fence_before();
        fence_proxy_async();  // make the generic-proxy writes of P visible to the tensor core
        mbar_arrive(smem_u32(&bars[B_PF]));
      }
      if (!ok) break;
      if (!mbar_wait(smem_u32(&bars[B_OF]), (jb0 + nb - 1) & 1, abort_flag, status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const float inv = __fdiv_rn(1.0f, l);
      const size_t orow = static_cast<size_t>(it.q_start + (row_valid ? tok : 0)) * Hq + hq;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_off + c * 32, v);
        tmem_ld_wait_dep(v);
        if (c == D / 32 - 1) {
          // O is in registers: the next item's first P V may overwrite the accumulator
          tc_fence_before();
          mbar_arrive(smem_u32(&bars[B_OE]));
        }
        if (row_valid) {
          uint4* dst = reinterpret_cast<uint4*>(out + orow * D + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 wv;
            wv.x = pack_bf2(__fmul_rn(__uint_as_float(v[8 * i + 0]), inv), __fmul_rn(__uint_as_float(v[8 * i + 1]), inv));
            wv.y = pack_bf2(__fmul_rn(__uint_as_float(v[8 * i + 2]), inv), __fmul_rn(__uint_as_float(v[8 * i + 3]), inv));
            wv.z = pack_bf2(__fmul_rn(__uint_as_float(v[8 * i + 4]), inv), __fmul_rn(__uint_as_float(v[8 * i + 5]), inv));
            wv.w = pack_bf2(__fmul_rn(__uint_as_float(v[8 * i + 6]), inv), __fmul_rn(__uint_as_float(v[8 * i + 7]), inv));
            dst[i] = wv;
          }
        }
      }
      if (row_valid) {
        if (lse_out) lse_out[orow] = (m + log2f(l)) * 0.6931471805599453f;
      }
      jb0 += nb;
    }
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

template <int ND>
int launch_attn(const void* q, const void* k, const void* v, const void* items, const void* block_table, void* out,
                void* lse, int num_items, int T, int Hq, int Hkv, int bt_stride, long long num_slots, float scale,
                cudaStream_t stream, int dev) {
  using SM = AttnSmem<ND>;
  constexpr int D = 64 * ND;
  const int G = Hq / Hkv;
  const int TQ = kRows / G;
  CUtensorMap tmQ, tmK, tmV;
  {
    uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(G), static_cast<uint64_t>(Hkv),
                        static_cast<uint64_t>(T)};
    uint64_t strides[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(G) * D * 2,
                           static_cast<uint64_t>(Hq) * D * 2};
    uint32_t box[4] = {64, static_cast<uint32_t>(G), 1, static_cast<uint32_t>(TQ)};
    int rc = ixh::make_tmap(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, q, dims, strides, box);
    if (rc) return rc;
  }
  int rc = ixh::make_tmap_bf16_2d(&tmK, k, num_slots, static_cast<uint64_t>(Hkv) * D, static_cast<uint64_t>(Hkv) * D, kBlkN);
  if (rc) return rc;
  rc = ixh::make_tmap_bf16_2d(&tmV, v, num_slots, static_cast<uint64_t>(Hkv) * D, static_cast<uint64_t>(Hkv) * D, kBlkN);
  if (rc) return rc;
  auto kern = attention_fwd_kernel<ND>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kBytes));
    attr_set[dev & 63] = true;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const long long total = static_cast<long long>(num_items) * Hkv;
  const int grid = static_cast<int>(total < sms ? total : sms);       // persistent: one CTA per SM walks the work list
  const float scale_log2 = scale * 1.4426950408889634f;
  IX_CUDA(ixh::launch_pdl(kern, dim3(grid), dim3(kAttnThreads), static_cast<size_t>(SM::kBytes), stream, tmQ, tmK, tmV,
                          static_cast<const WorkItem*>(items), num_items, static_cast<const int*>(block_table), bt_stride,
                          static_cast<__nv_bfloat16*>(out), static_cast<float*>(lse), Hq, Hkv, G, scale_log2, ixh::status_word(dev)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

// q: [T, Hq, D] bf16; k, v: [num_slots, Hkv, D] bf16 slot pools (zero-initialised: a masked key
// still enters P*V with weight 0, so its bytes must be finite); items: [num_items, 8] int32
// (WorkItem); block_table: [*, bt_stride] int32 page ids (page = 128 slots) or null;
// out: [T, Hq, D] bf16; lse: [T, Hq] fp32 or null.
IX_API int ix_attention_fwd(const void* q, const void* k, const void* v, const void* items, const void* block_table,
                            void* out, void* lse, void* /*reserved*/, int num_items, int T, int Hq, int Hkv, int D,
                            int bt_stride, long long num_slots, int /*flags*/, float scale, void* /*reserved2*/,
                            void* stream) {
  if (num_items <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv) return ixh::fail(ixh::IX_EARG, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  const int G = Hq / Hkv;
  if (G > 128 || (128 % G)) return ixh::fail(ixh::IX_EARG, "attention: group size %d must divide 128", G);
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_attn<2>(q, k, v, items, block_table, out, lse, num_items, T, Hq, Hkv, bt_stride, num_slots, scale, s, dev);
  if (D == 64) return launch_attn<1>(q, k, v, items, block_table, out, lse, num_items, T, Hq, Hkv, bt_stride, num_slots, scale, s, dev);
  return ixh::fail(ixh::IX_EARG, "attention: head dim %d unsupported (64 or 128)", D);
}
