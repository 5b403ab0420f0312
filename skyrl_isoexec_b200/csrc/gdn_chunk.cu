// Chunk-parallel gated delta rule on the tensor cores (sm_100a), the training / prefill form of the GatedDeltaNet core
// and, by construction, also its decode form.
//
// Per (sequence, value head), with tokens cut into chunks of C = 64 anchored at sequence position 0, G_t the running
// sum of the log-decays g inside the chunk, S0 the state entering the chunk:
//
//   L_ts = exp(G_t - G_s) (k_t . k_s)  (s < t)          T = (I + diag(beta) L)^-1     (unit lower triangular, fp32 solve)
//   W = T (beta e^G k)      U = T (beta v)               (independent of the state: computed for ALL chunks in parallel)
//   D = U - W bf16(S0)^T                                  (the "new values" d_s of the delta rule)
//   O = e^G (Q bf16(S0)^T) + P D,   P_ts = exp(G_t - G_s)(q_t . k_s)  (s <= t)
//   S1 = e^{G_C} S0 + D^T (e^{G_C - G} k)                 (fp32 chain; the chunk reads the bf16 SNAPSHOT of S0)
//
// which is the reference's CPR recipe (fp32 boundary chain, in-chunk results from the bf16 snapshot of the boundary
// state: ISO/ops/gdn/gdn_cpr.py:104-292, math of ISO/ops/gdn/gdn_ops.py:261-316) with every product on tcgen05:
//
//   gdn_chunk_prep_kernel   one CTA per (chunk, value head), all chunks at once: [Q;K] K^T as one M=128 MMA, the decay
//                           masks, the 64x64 triangular solve in fp32, then [W | U] = T [beta e^G K | beta V] as one MMA
//   gdn_chunk_state_kernel  one CTA per (sequence, value head) walking its chunks: state in TMEM (fp32), per chunk
//                           [W;Q] S^T, then P D and the state update D^T Kd
//
// Row independence is what makes decode bitwise equal to training: row t of every product depends only on tokens
// s <= t of its chunk (masked entries are exact zeros), so running these kernels on a chunk that holds only the tokens
// seen so far yields, for the newest token, the bits the full chunk yields for that row. The engine keeps the tokens of
// the open chunk and re-runs it every step; there is no separate recurrent kernel whose rounding could differ.
//
// Operands reach shared memory through plain loads and are written in the 128-byte swizzled layout the MMA reads
// (no TMA: the tiles are small and produced by arithmetic). All waits are bounded.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int C = 64;             // tokens per chunk
constexpr int kThreads = 128;

struct GdnChunk {
  int tok_start;    // first token row in the packed tensors
  int n_tok;        // tokens present (1..64); rows beyond are treated as empty
};
struct GdnChain {
  int chunk_begin, chunk_end;   // chunks [begin, end) of this sequence, in order
  long long row_in;             // state-pool row holding the state entering chunk_begin, or -1 for zeros
  long long row_out;            // state-pool row that receives the state after the last COMPLETE chunk, or -1
};

// byte offset of (row r, byte b of the 128-byte row) inside one swizzled [rows x 128 B] block
__device__ __forceinline__ uint32_t sw(int r, int b) { return r * 128 + ((((b >> 4) ^ (r & 7)) << 4) | (b & 15)); }

__device__ __forceinline__ uint64_t desc_k(uint32_t a) { return make_sw128_desc(a, 16, 1024); }
__device__ __forceinline__ uint64_t desc_mn(uint32_t a, uint32_t lbo) { return make_sw128_desc(a, lbo, 1024); }

// one thread: wait for the MMAs committed to `bar` (parity `ph`)
__device__ __forceinline__ bool mma_done(uint32_t bar, uint32_t ph, volatile int* abort_flag, int* status) {
  return mbar_wait(bar, ph, abort_flag, status, ST_TIMEOUT_MISC);
}

// 16 bytes (8 bf16) of row `r`, 16-byte unit `u` of a row-major [rows x ld] bf16 matrix, or zeros
__device__ __forceinline__ uint4 ld8(const __nv_bfloat16* base, long long row, long long ld, int u, bool valid) {
  return valid ? *reinterpret_cast<const uint4*>(base + row * ld + u * 8) : make_uint4(0u, 0u, 0u, 0u);
}

template <int D>
struct PrepSmem {
  static constexpr int kQK = 0;                          // [128 rows x D cols] K-major: rows 0..63 = K, 64..127 = Q
  static constexpr int kT = kQK + (D / 64) * 16384;      // [128 rows x 64 cols] K-major: rows 0..63 = T, 64..127 = 0
  static constexpr int kB2 = kT + 16384;                 // [64 rows x 2D cols] M/N-major: [beta e^G K | beta V]
  static constexpr int kA = kB2 + (2 * D / 64) * 8192;   // fp32 [64][65]: beta L (strictly lower)
  static constexpr int kG = kA + 64 * 65 * 4;            // fp32 G[64], beta[64]
  static constexpr int kBar = kG + 2 * 64 * 4;
  static constexpr int kBytes = kBar + 64 + 1024;
};

// q, k: [T, Hk, D] bf16 (normalised), v: [T, Hv, D] bf16, g, beta: [T, Hv] fp32.
// Scratch outputs, indexed by ch = chunk * Hv + hv: Wb, Ub, Kd [ch][64][D] bf16, Pm [ch][64][64] bf16, eG [ch][64] fp32,
// eGlast [ch] fp32.
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
gdn_chunk_prep_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                      const float* __restrict__ g, const float* __restrict__ beta, const GdnChunk* __restrict__ chunks, int Hk, int Hv,
                      __nv_bfloat16* __restrict__ Wb, __nv_bfloat16* __restrict__ Ub, __nv_bfloat16* __restrict__ Kd,
                      __nv_bfloat16* __restrict__ Pm, float* __restrict__ eG, float* __restrict__ eGlast, int* __restrict__ status) {
  using SM = PrepSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sA = reinterpret_cast<float*>(smem + SM::kA);
  float* sG = reinterpret_cast<float*>(smem + SM::kG);
  float* sBeta = sG + 64;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + SM::kBar);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  constexpr int kTmemCols = (2 * D < 64) ? 64 : 2 * D;     // acc0 (64 cols) and acc1 (2D cols) use the same columns in turn

  const GdnChunk ck = chunks[blockIdx.x];
  const int hv = blockIdx.y, hk = hv / (Hv / Hk);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long ch = static_cast<long long>(blockIdx.x) * Hv + hv;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(bar), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<kTmemCols>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  // decay prefix sums and beta (one thread: 64 adds in a fixed order)
  if (tid == 32) {
    float acc = 0.f;
    for (int t = 0; t < C; ++t) {
      const bool ok = t < ck.n_tok;
      acc = __fadd_rn(acc, ok ? g[static_cast<long long>(ck.tok_start + t) * Hv + hv] : 0.f);
      sG[t] = acc;
      sBeta[t] = ok ? beta[static_cast<long long>(ck.tok_start + t) * Hv + hv] : 0.f;
    }
  }
  // [K; Q] tile: 128 rows x (D / 8) units of 16 bytes
  constexpr int kUnits = D / 8;
  for (int i = tid; i < 128 * kUnits; i += kThreads) {
    const int r = i / kUnits, u = i % kUnits;
    const int t = r & 63;
    const bool ok = t < ck.n_tok;
    const __nv_bfloat16* src = (r < 64) ? k : q;
    const uint4 val = ld8(src, static_cast<long long>(ck.tok_start + t) * Hk + hk, D, u, ok);
    *reinterpret_cast<uint4*>(smem + SM::kQK + (u >> 3) * 16384 + sw(r, (u & 7) * 16)) = val;
  }
  // T tile rows 64..127 are zero
  for (int i = tid; i < 64 * 8; i += kThreads) *reinterpret_cast<uint4*>(smem + SM::kT + 64 * 128 + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;
  uint32_t ph = 0;

  // ---- (a) acc[128 x 64] = [K; Q] K^T
  if (tid == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, 64, 0, 0);
#pragma unroll
    for (int cc = 0; cc < D / 64; ++cc) {
      const uint64_t d = desc_k(smem_u32(smem + SM::kQK + cc * 16384));
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_f16_ss(tmem, d + 2 * ks, d + 2 * ks, idesc, (cc | ks) != 0 ? 1u : 0u);
    }
    umma_commit(smem_u32(bar));
  }
  const bool ok_a = __syncthreads_and(mma_done(smem_u32(bar), ph, abort_flag, status)) != 0;
  ph ^= 1;
  tc_fence_after();
  {
    const int r = tid;                    // TMEM lane = row of the product
    const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    uint32_t a0[32], a1[32];
    tmem_ld_32x32(taddr, a0);
    tmem_ld_32x32(taddr + 32, a1);
    tmem_ld_wait_dep(a0);
    tmem_ld_wait_dep(a1);
    const int t = r & 63;
    const float Gt = sG[t];
    if (r < 64) {
      const float bt = sBeta[t];
#pragma unroll
      for (int s = 0; s < 64; ++s) {
        const float kk = __uint_as_float(s < 32 ? a0[s] : a1[s - 32]);
        sA[t * 65 + s] = (s < t && ok_a) ? __fmul_rn(__fmul_rn(bt, expf(__fsub_rn(Gt, sG[s]))), kk) : 0.f;
      }
    } else {
      __nv_bfloat16* dst = Pm + (ch * 64 + t) * 64;
#pragma unroll
      for (int s = 0; s < 64; s += 2) {
        const float q0 = __uint_as_float(s < 32 ? a0[s] : a1[s - 32]);
        const float q1 = __uint_as_float(s + 1 < 32 ? a0[s + 1] : a1[s + 1 - 32]);
        const float p0 = (s <= t) ? __fmul_rn(expf(__fsub_rn(Gt, sG[s])), q0) : 0.f;
        const float p1 = (s + 1 <= t) ? __fmul_rn(expf(__fsub_rn(Gt, sG[s + 1])), q1) : 0.f;
        *reinterpret_cast<uint32_t*>(dst + s) = pack_bf2(p0, p1);
      }
    }
  }
  tc_fence_before();
  __syncthreads();

  // ---- T = (I + A)^-1 by forward substitution; thread c owns column c (fp32, ascending s)
  if (tid < 64) {
    const int c = tid;
    float Tc[64];
#pragma unroll
    for (int t = 0; t < 64; ++t) {
      float acc = (t == c) ? 1.f : 0.f;
#pragma unroll
      for (int s = 0; s < t; ++s) acc = __fmaf_rn(-sA[t * 65 + s], Tc[s], acc);
      Tc[t] = (t >= c) ? acc : 0.f;
    }
#pragma unroll
    for (int t = 0; t < 64; ++t)
      *reinterpret_cast<__nv_bfloat16*>(smem + SM::kT + sw(t, c * 2)) = f2bf(Tc[t]);
  } else {
    // meanwhile: B2 = [beta e^G K | beta V] as [64 rows x 2D cols] (M/N-major), Kd = e^{G_C - G} K, eG
    const int w = tid - 64;               // 64 threads
    const float Glast = sG[63];
    for (int i = w; i < 64 * kUnits; i += 64) {
      const int s = i / kUnits, u = i % kUnits;
      const bool ok = s < ck.n_tok;
      const float bs = sBeta[s], es = expf(sG[s]), ed = expf(__fsub_rn(Glast, sG[s]));
      uint4 kv = ld8(k, static_cast<long long>(ck.tok_start + s) * Hk + hk, D, u, ok);
      uint4 vv = ld8(v, static_cast<long long>(ck.tok_start + s) * Hv + hv, D, u, ok);
      const __nv_bfloat16* ke = reinterpret_cast<const __nv_bfloat16*>(&kv);
      const __nv_bfloat16* ve = reinterpret_cast<const __nv_bfloat16*>(&vv);
      uint4 kb, vb, kd;
      uint32_t* kbp = reinterpret_cast<uint32_t*>(&kb);
      uint32_t* vbp = reinterpret_cast<uint32_t*>(&vb);
      uint32_t* kdp = reinterpret_cast<uint32_t*>(&kd);
      const float bes = __fmul_rn(bs, es);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float k0 = bf2f(ke[2 * j]), k1 = bf2f(ke[2 * j + 1]);
        kbp[j] = pack_bf2(__fmul_rn(bes, k0), __fmul_rn(bes, k1));
        vbp[j] = pack_bf2(__fmul_rn(bs, bf2f(ve[2 * j])), __fmul_rn(bs, bf2f(ve[2 * j + 1])));
        kdp[j] = pack_bf2(__fmul_rn(ed, k0), __fmul_rn(ed, k1));
      }
      *reinterpret_cast<uint4*>(smem + SM::kB2 + (u >> 3) * 8192 + sw(s, (u & 7) * 16)) = kb;
      *reinterpret_cast<uint4*>(smem + SM::kB2 + ((kUnits + u) >> 3) * 8192 + sw(s, ((kUnits + u) & 7) * 16)) = vb;
      *reinterpret_cast<uint4*>(Kd + (ch * 64 + s) * D + u * 8) = kd;
    }
    for (int s = w; s < 64; s += 64) eG[ch * 64 + s] = expf(sG[s]);
    if (w == 0) eGlast[ch] = expf(Glast);
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- (b) acc[128 x 2D] = T [beta e^G K | beta V]   (rows 64..127 of T are zero)
  if (tid == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, 2 * D, 0, 1);
    const uint64_t da = desc_k(smem_u32(smem + SM::kT));
    const uint64_t db = desc_mn(smem_u32(smem + SM::kB2), 8192);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) umma_f16_ss(tmem, da + 2 * ks, db + 128 * ks, idesc, ks != 0 ? 1u : 0u);
    umma_commit(smem_u32(bar));
  }
  const bool ok_b = __syncthreads_and(mma_done(smem_u32(bar), ph, abort_flag, status)) != 0;
  tc_fence_after();
  if (tid < 64 && ok_b) {
    const int t = tid;
    const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < 2 * D; c0 += 32) {
      uint32_t a[32];
      tmem_ld_32x32(taddr + c0, a);
      tmem_ld_wait_dep(a);
      __nv_bfloat16* dst = (c0 < D) ? (Wb + (ch * 64 + t) * D + c0) : (Ub + (ch * 64 + t) * D + (c0 - D));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 o;
        o.x = pack_bf2(__uint_as_float(a[8 * j + 0]), __uint_as_float(a[8 * j + 1]));
        o.y = pack_bf2(__uint_as_float(a[8 * j + 2]), __uint_as_float(a[8 * j + 3]));
        o.z = pack_bf2(__uint_as_float(a[8 * j + 4]), __uint_as_float(a[8 * j + 5]));
        o.w = pack_bf2(__uint_as_float(a[8 * j + 6]), __uint_as_float(a[8 * j + 7]));
        reinterpret_cast<uint4*>(dst)[j] = o;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem);
  }
}


template <int D>
struct StateSmem {
  static constexpr int kS = 0;                               // [128 rows (Dv, padded) x D cols (Dk)] K-major: bf16 snapshot of the state
  static constexpr int kWQ = kS + (D / 64) * 16384;          // [128 rows x D cols] K-major: rows 0..63 = W, 64..127 = Q
  static constexpr int kD = kWQ + (D / 64) * 16384;          // [64 rows (s) x 128 cols (Dv, padded)] M/N-major: D = U - W S^T
  static constexpr int kP = kD + 2 * 8192;                   // [128 rows x 64 cols] K-major: rows 0..63 = 0, 64..127 = P
  static constexpr int kKd = kP + 16384;                     // [64 rows (s) x D cols (Dk)] M/N-major: e^{G_C - G} K
  static constexpr int kBar = kKd + (D / 64) * 8192;
  static constexpr int kBytes = kBar + 64 + 1024;
};

// state: fp32 pool [rows][Hv][D (Dv)][D (Dk)]. out: [T, Hv, D] bf16.
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
gdn_chunk_state_kernel(const __nv_bfloat16* __restrict__ q, const GdnChunk* __restrict__ chunks, const GdnChain* __restrict__ chains,
                       int Hk, int Hv, const __nv_bfloat16* __restrict__ Wb, const __nv_bfloat16* __restrict__ Ub,
                       const __nv_bfloat16* __restrict__ Kd, const __nv_bfloat16* __restrict__ Pm, const float* __restrict__ eG,
                       const float* __restrict__ eGlast, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
                       int* __restrict__ status) {
  using SM = StateSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + SM::kBar);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  constexpr int kTmemCols = (3 * D <= 256) ? 256 : 512;      // accS (D cols) | accX (D) | accO (D)
  constexpr int kUnits = D / 8;

  const GdnChain cn = chains[blockIdx.x];
  const int hv = blockIdx.y, hk = hv / (Hv / Hk);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid;                                          // TMEM lane handled by this thread

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(bar), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc<kTmemCols>(smem_u32(tmem_holder));
    tmem_relinquish();
  }
  // zero everything once: padding rows / columns of the tiles stay zero for the whole walk
  for (int i = tid; i < SM::kBar / 16; i += kThreads) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t accS = lane_addr, accX = lane_addr + D, accO = lane_addr + 2 * D;

  // initial state into TMEM: row r of S is value dim r (rows >= D stay zero)
  {
    const float* sp = (cn.row_in >= 0 && r < D) ? state + ((cn.row_in * Hv + hv) * D + r) * D : nullptr;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t a[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] = sp ? __float_as_uint(sp[c0 + j]) : 0u;
      tmem_st_32x32(accS + c0, a);
    }
    tmem_st_wait();
  }
  uint32_t ph = 0;
  bool ok = true;
  // the last chunk of a chain may be open (fewer than 64 tokens): the state to continue from is the one after the last
  // complete chunk
  const int last_complete = (cn.chunk_end > cn.chunk_begin && chunks[cn.chunk_end - 1].n_tok == C) ? cn.chunk_end - 1 : cn.chunk_end - 2;

  for (int c = cn.chunk_begin; c < cn.chunk_end && ok; ++c) {
    const GdnChunk ck = chunks[c];
    const long long ch = static_cast<long long>(c) * Hv + hv;
    const float egl = eGlast[ch];
    // (1) snapshot the state to bf16 (B operand of this chunk) and scale the fp32 state by e^{G_C} in place
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t a[32];
      tmem_ld_32x32(accS + c0, a);
      tmem_ld_wait_dep(a);
      if (r < D) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          o.x = pack_bf2(__uint_as_float(a[8 * j + 0]), __uint_as_float(a[8 * j + 1]));
          o.y = pack_bf2(__uint_as_float(a[8 * j + 2]), __uint_as_float(a[8 * j + 3]));
          o.z = pack_bf2(__uint_as_float(a[8 * j + 4]), __uint_as_float(a[8 * j + 5]));
          o.w = pack_bf2(__uint_as_float(a[8 * j + 6]), __uint_as_float(a[8 * j + 7]));
          const int col = c0 + 8 * j;                          // first of 8 key-dim columns
          *reinterpret_cast<uint4*>(smem + SM::kS + (col >> 6) * 16384 + sw(r, (col & 63) * 2)) = o;
        }
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] = __float_as_uint(__fmul_rn(__uint_as_float(a[j]), egl));
      tmem_st_32x32(accS + c0, a);
    }
    tmem_st_wait();
    // (2) operands of the chunk: [W; Q], P, Kd
    for (int i = tid; i < 128 * kUnits; i += kThreads) {
      const int row = i / kUnits, u = i % kUnits, t = row & 63;
      uint4 val;
      if (row < 64) val = *reinterpret_cast<const uint4*>(Wb + (ch * 64 + t) * D + u * 8);
      else val = ld8(q, static_cast<long long>(ck.tok_start + t) * Hk + hk, D, u, t < ck.n_tok);
      *reinterpret_cast<uint4*>(smem + SM::kWQ + (u >> 3) * 16384 + sw(row, (u & 7) * 16)) = val;
    }
    for (int i = tid; i < 64 * 8; i += kThreads) {
      const int t = i >> 3, u = i & 7;
      *reinterpret_cast<uint4*>(smem + SM::kP + sw(64 + t, u * 16)) = *reinterpret_cast<const uint4*>(Pm + (ch * 64 + t) * 64 + u * 8);
    }
    for (int i = tid; i < 64 * kUnits; i += kThreads) {
      const int sr = i / kUnits, u = i % kUnits;
      *reinterpret_cast<uint4*>(smem + SM::kKd + (u >> 3) * 8192 + sw(sr, (u & 7) * 16)) =
          *reinterpret_cast<const uint4*>(Kd + (ch * 64 + sr) * D + u * 8);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // (3) accX[128 x D] = [W; Q] S^T
    if (tid == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, D, 0, 0);
#pragma unroll
      for (int cc = 0; cc < D / 64; ++cc) {
        const uint64_t da = desc_k(smem_u32(smem + SM::kWQ + cc * 16384));
        const uint64_t db = desc_k(smem_u32(smem + SM::kS + cc * 16384));
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_f16_ss(tmem + D, da + 2 * ks, db + 2 * ks, idesc, (cc | ks) != 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(bar));
    }
    ok = __syncthreads_and(mma_done(smem_u32(bar), ph, abort_flag, status)) != 0;   // one answer for the whole CTA
    ph ^= 1;
    tc_fence_after();
    // (4) rows 0..63: D_t = U_t - X_t, rounded to bf16, into the M/N-major tile
    if (tid < 64 && ok) {
      const int t = tid;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t a[32];
        tmem_ld_32x32(accX + c0, a);
        tmem_ld_wait_dep(a);
        const uint4* up = reinterpret_cast<const uint4*>(Ub + (ch * 64 + t) * D + c0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 uv = up[j];
          const __nv_bfloat16* ue = reinterpret_cast<const __nv_bfloat16*>(&uv);
          uint4 o;
          uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            op[e] = pack_bf2(__fsub_rn(bf2f(ue[2 * e]), __uint_as_float(a[8 * j + 2 * e])),
                             __fsub_rn(bf2f(ue[2 * e + 1]), __uint_as_float(a[8 * j + 2 * e + 1])));
          const int col = c0 + 8 * j;
          *reinterpret_cast<uint4*>(smem + SM::kD + (col >> 6) * 8192 + sw(t, (col & 63) * 2)) = o;
        }
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // (5) accO[128 x D] = [0; P] D      accS[128 x D] += D^T Kd
    if (tid == 0) {
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);
      constexpr uint32_t idesc_s = make_idesc_bf16(128, D, 1, 1);
      const uint64_t dp = desc_k(smem_u32(smem + SM::kP));
      const uint64_t dd = desc_mn(smem_u32(smem + SM::kD), 8192);
      const uint64_t dk = desc_mn(smem_u32(smem + SM::kKd), 8192);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_f16_ss(tmem + 2 * D, dp + 2 * ks, dd + 128 * ks, idesc_o, ks != 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_f16_ss(tmem, dd + 128 * ks, dk + 128 * ks, idesc_s, 1u);
      umma_commit(smem_u32(bar));
    }
    ok = __syncthreads_and(mma_done(smem_u32(bar), ph, abort_flag, status)) != 0;   // one answer for the whole CTA
    ph ^= 1;
    tc_fence_after();
    // (6) rows 64..127: o_t = e^{G_t} (Q S^T)_t + (P D)_t. The TMEM loads are warp-wide instructions: every lane of the
    // two warps executes them, only the stores are predicated on the row holding a token.
    if (tid >= 64 && ok) {
      const int t = tid - 64;
      const bool live = t < ck.n_tok;
      const float eg = eG[ch * 64 + t];
      __nv_bfloat16* dst = out + (static_cast<long long>(ck.tok_start + (live ? t : 0)) * Hv + hv) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t x[32], o[32];
        tmem_ld_32x32(accX + c0, x);
        tmem_ld_32x32(accO + c0, o);
        tmem_ld_wait_dep(x);
        tmem_ld_wait_dep(o);
        if (live) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 w;
            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wp[e] = pack_bf2(__fmaf_rn(eg, __uint_as_float(x[8 * j + 2 * e]), __uint_as_float(o[8 * j + 2 * e])),
                               __fmaf_rn(eg, __uint_as_float(x[8 * j + 2 * e + 1]), __uint_as_float(o[8 * j + 2 * e + 1])));
            reinterpret_cast<uint4*>(dst + c0)[j] = w;
          }
        }
      }
    }
    // the state after a COMPLETE chunk is what a later call continues from
    if (c == last_complete && cn.row_out >= 0 && ok) {
      float* sp = (r < D) ? state + ((cn.row_out * Hv + hv) * D + r) * D : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t a[32];
        tmem_ld_32x32(accS + c0, a);
        tmem_ld_wait_dep(a);
        if (sp) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            reinterpret_cast<float4*>(sp + c0)[j] = make_float4(__uint_as_float(a[4 * j]), __uint_as_float(a[4 * j + 1]),
                                                                __uint_as_float(a[4 * j + 2]), __uint_as_float(a[4 * j + 3]));
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<kTmemCols>(tmem);
  }
}

template <int D>
int launch_chunk(const void* q, const void* k, const void* v, const void* g, const void* beta, const void* chunks, int n_chunks,
                 const void* chains, int n_chains, int Hk, int Hv, void* scratch, void* state, void* out, cudaStream_t s, int dev) {
  // scratch layout (bytes), ch = n_chunks * Hv: Wb, Ub, Kd [ch][64][D] bf16 | Pm [ch][64][64] bf16 | eG [ch][64] f32 | eGlast [ch] f32
  const size_t chn = static_cast<size_t>(n_chunks) * Hv;
  uint8_t* base = static_cast<uint8_t*>(scratch);
  __nv_bfloat16* Wb = reinterpret_cast<__nv_bfloat16*>(base);
  __nv_bfloat16* Ub = Wb + chn * 64 * D;
  __nv_bfloat16* Kd = Ub + chn * 64 * D;
  __nv_bfloat16* Pm = Kd + chn * 64 * D;
  float* eG = reinterpret_cast<float*>(Pm + chn * 64 * 64);
  float* eGl = eG + chn * 64;
  auto k1 = gdn_chunk_prep_kernel<D>;
  auto k2 = gdn_chunk_state_kernel<D>;
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    IX_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, PrepSmem<D>::kBytes));
    IX_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, StateSmem<D>::kBytes));
    attr_set[dev & 63] = true;
  }
  int* st = ixh::status_word(dev);
  k1<<<dim3(n_chunks, Hv), kThreads, PrepSmem<D>::kBytes, s>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      static_cast<const float*>(g), static_cast<const float*>(beta), static_cast<const GdnChunk*>(chunks), Hk, Hv, Wb, Ub, Kd, Pm, eG, eGl, st);
  IX_CUDA(cudaGetLastError());
  k2<<<dim3(n_chains, Hv), kThreads, StateSmem<D>::kBytes, s>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const GdnChunk*>(chunks), static_cast<const GdnChain*>(chains), Hk, Hv, Wb, Ub, Kd,
      Pm, eG, eGl, static_cast<float*>(state), static_cast<__nv_bfloat16*>(out), st);
  IX_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

// Bytes of scratch the chunked scan needs for n_chunks chunks of Hv value heads with head width D.
IX_API long long ix_gdn_chunk_scratch_bytes(int n_chunks, int Hv, int D) {
  const long long ch = static_cast<long long>(n_chunks) * Hv;
  return ch * (3LL * 64 * D * 2 + 64 * 64 * 2 + 64 * 4 + 4) + 256;
}

// Chunked gated delta rule. q, k: [T, Hk, D] bf16 (L2-normalised, q scaled), v: [T, Hv, D] bf16, g (log decay), beta: [T, Hv]
// fp32. chunks: n_chunks records {tok_start, n_tok}; chains: n_chains records {chunk_begin, chunk_end, row_in, row_out}
// (both device arrays). state: fp32 pool [rows][Hv][D][D] (may be null when no chain names a row). out: [T, Hv, D] bf16.
IX_API int ix_gdn_chunk_fwd(const void* q, const void* k, const void* v, const void* g, const void* beta, const void* chunks,
                            int n_chunks, const void* chains, int n_chains, int Hk, int Hv, int D, void* scratch, void* state,
                            void* out, void* stream) {
  if (n_chunks <= 0 || n_chains <= 0) return 0;
  if (D != 64 && D != 128) return ixh::fail(ixh::IX_EARG, "gdn_chunk: head width %d unsupported (64 | 128)", D);
  if (Hk < 1 || Hv % Hk) return ixh::fail(ixh::IX_EARG, "gdn_chunk: Hv=%d not a multiple of Hk=%d", Hv, Hk);
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_chunk<128>(q, k, v, g, beta, chunks, n_chunks, chains, n_chains, Hk, Hv, scratch, state, out, s, dev);
  return launch_chunk<64>(q, k, v, g, beta, chunks, n_chunks, chains, n_chains, Hk, Hv, scratch, state, out, s, dev);
}
