// Backward kernels of RMSNorm(+residual) and of the fused QK-norm + RoPE (training only; the forward
// kernels are in norm_rope.cu). Memory-bound, one pass over the activations, fp32 arithmetic.
//
// Weight gradients are reduced in a fixed order: a thread (rmsnorm) or warp (qk-norm) accumulates the rows it owns
// sequentially in registers, the CTA writes one partial row, and a second kernel adds the partial rows in CTA order. No atomics, so two runs give the same bits.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

struct alignas(16) BF8 {
  __nv_bfloat16 v[8];
};

constexpr int kBwdCtas = 592;      // rmsnorm backward: 4 CTAs per SM
constexpr int kQkBwdCtas = 2368;   // qk-norm/rope backward: 16 small CTAs per SM, each item is latency-bound

// dh = rstd * (dn - n * mean(dn * n)) + dres, dn = dy * g, n = h * rstd;  dw_partial[cta] = sum_rows dy * bf16(n)
// One CTA per row at a time (rows strided over the grid); thread t owns the 8-element vectors t, t+128, ... of the
// row (at most kVecPerThread of them), so the weight-gradient accumulators stay in registers and are summed over the
// CTA's rows in row order. N <= 8192, multiple of 8.
// kVecPerThread: 4 covers N <= 4096 (128 threads x 4 vectors x 8 elements), 8 covers N <= 8192
template <bool ZERO_CENTERED, bool HAS_DRES, int kVecPerThread>
__global__ void __launch_bounds__(128)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dres,
                   __nv_bfloat16* __restrict__ dh, float* __restrict__ dw_partial, int rows, int N) {
  __shared__ float s_red[2][4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nvec = N >> 3;
  const float inv_n = 1.0f / static_cast<float>(N);
  float acc[kVecPerThread][8];
  float g[kVecPerThread][8];
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int v = tid + i * 128;
    BF8 g8;
    if (v < nvec) g8 = reinterpret_cast<const BF8*>(w)[v];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[i][j] = 0.f;
      float gg = v < nvec ? bf2f(g8.v[j]) : 0.f;
      if (ZERO_CENTERED) gg = round_bf(1.0f + gg);
      g[i][j] = gg;
    }
  }
  int parity = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
    const BF8* hr = reinterpret_cast<const BF8*>(h + static_cast<size_t>(row) * N);
    const BF8* dyr = reinterpret_cast<const BF8*>(dy + static_cast<size_t>(row) * N);
    const float rs = rstd[row];
    BF8 a[kVecPerThread], d[kVecPerThread], r8[kVecPerThread];
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
      const int v = tid + i * 128;
      if (v < nvec) {
        a[i] = hr[v];
        d[i] = dyr[v];
        if (HAS_DRES) r8[i] = reinterpret_cast<const BF8*>(dres + static_cast<size_t>(row) * N)[v];
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
      if (tid + i * 128 < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += bf2f(d[i].v[j]) * g[i][j] * (bf2f(a[i].v[j]) * rs);
      }
    }
    dot = warp_sum_butterfly(dot);
    if (lane == 0) s_red[parity][warp] = dot;
    __syncthreads();            // one barrier per row: the buffer alternates, so the next row's writes cannot overtake these reads
    dot = (((s_red[parity][0] + s_red[parity][1]) + s_red[parity][2]) + s_red[parity][3]) * inv_n;
#pragma unroll
    for (int i = 0; i < kVecPerThread; ++i) {
      const int v = tid + i * 128;
      if (v < nvec) {
        BF8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = bf2f(a[i].v[j]) * rs;
          const float dyf = bf2f(d[i].v[j]);
          float dx = rs * (dyf * g[i][j] - n * dot);
          if (HAS_DRES) dx += bf2f(r8[i].v[j]);
          o.v[j] = f2bf(dx);
          acc[i][j] += dyf * round_bf(n);
        }
        reinterpret_cast<BF8*>(dh + static_cast<size_t>(row) * N)[v] = o;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int v = tid + i * 128;
    if (v < nvec) {
      float* dst = dw_partial + static_cast<size_t>(blockIdx.x) * N + v * 8;
      reinterpret_cast<float4*>(dst)[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
  }
}

// out[c] = sum over p (ascending) of partial[p][c], written as bf16
__global__ void __launch_bounds__(256) fold_partials_kernel(const float* __restrict__ partial, int P, int N, __nv_bfloat16* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[static_cast<size_t>(p) * N + c];
  out[c] = f2bf(s);
}

// Backward of qk_norm_rope. dq [T,Hq,D], dk/dv [T,Hkv,D] -> dqkv in the KV-group-major fused layout; the gate half of
// a gated query block is not touched here (its gradient comes from the gate op). Work layout as in the forward
// (csrc/norm_rope.cu): a head takes nact = D / 8 lanes, hpw heads share a warp when nact is a power of two, wpt warps
// share a token and walk its heads, fetching the rotation constants once per token and the norm weights once.
template <bool QK_NORM, bool ZERO_CENTERED>
__global__ void __launch_bounds__(128)
qk_norm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ldqkv, const int* __restrict__ positions,
                        const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                        const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                        const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                        const __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dw_partial,
                        int T, int Hq, int Hkv, int D, int rot_dim, float eps, int q_gate, int wpt, int hpw, int red_width) {
  __shared__ float s_w[4][2][256];            // per warp: [q | k][D] weight-gradient accumulators
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Htot = Hq + 2 * Hkv;
  const int nact = D >> 3;
  const int sub = lane / nact, sl = lane - sub * nact;
  const bool lane_on = sub < hpw;
  const int e0 = sl * 8;
  float accq[8], acck[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) accq[j] = acck[j] = 0.f;
  const int q_stride = q_gate ? 2 * D : D;
  const int G = Hq / Hkv;
  const long long grp_stride = static_cast<long long>(G) * q_stride + 2 * D;
  const int half = rot_dim >> 1, half_lanes = half >> 3;
  const bool in_rot = lane_on && e0 < rot_dim, first_half = e0 < half;
  const int partner = sub * nact + (first_half ? sl + half_lanes : sl - half_lanes);
  float gq[8], gk[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) gq[j] = gk[j] = 0.f;
  if (QK_NORM && lane_on) {
    const BF8 a = reinterpret_cast<const BF8*>(qw)[sl], b = reinterpret_cast<const BF8*>(kw)[sl];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gq[j] = bf2f(a.v[j]);
      gk[j] = bf2f(b.v[j]);
      if (ZERO_CENTERED) gq[j] = round_bf(1.0f + gq[j]), gk[j] = round_bf(1.0f + gk[j]);
    }
  }
  // sum over the lanes of one head (group-local butterfly)
  auto group_sum = [&](float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
      if (off < red_width) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
  };
  const long long total = static_cast<long long>(T) * wpt;
  for (long long wid = static_cast<long long>(blockIdx.x) * 4 + warp; wid < total; wid += static_cast<long long>(gridDim.x) * 4) {
    const int t = static_cast<int>(wid / wpt), h0 = static_cast<int>(wid % wpt);
    const int pos = positions[t];
    float cs[8], sn[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      cs[j] = 1.f;
      sn[j] = 0.f;
      if (in_rot) {
        const int fi = (first_half ? e0 : e0 - half) + j;
        cs[j] = cos_tab[static_cast<size_t>(pos) * half + fi];
        sn[j] = sin_tab[static_cast<size_t>(pos) * half + fi];
      }
    }
    for (int hb = h0; hb < Htot; hb += wpt * hpw) {       // the same trip count for every lane of the warp
      const int h = hb + sub * wpt;
      const bool on = lane_on && h < Htot;
      const bool is_v = h >= Hq + Hkv;
      long long off = 0;
      if (h < Hq) off = (h / G) * grp_stride + static_cast<long long>(h % G) * q_stride;
      else if (!is_v) off = (h - Hq) * grp_stride + static_cast<long long>(G) * q_stride;
      else off = (h - Hq - Hkv) * grp_stride + static_cast<long long>(G) * q_stride + D;
      float d[8], x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) d[j] = x[j] = 0.f;
      if (on) {
        __nv_bfloat16* dst = dqkv + static_cast<size_t>(t) * ldqkv + off;
        if (is_v) {
          reinterpret_cast<BF8*>(dst)[sl] = reinterpret_cast<const BF8*>(dv + (static_cast<size_t>(t) * Hkv + (h - Hq - Hkv)) * D)[sl];
        } else {
          const __nv_bfloat16* dsrc = (h < Hq) ? dq + (static_cast<size_t>(t) * Hq + h) * D : dk + (static_cast<size_t>(t) * Hkv + (h - Hq)) * D;
          const BF8 a = reinterpret_cast<const BF8*>(dsrc)[sl];
          const BF8 b = reinterpret_cast<const BF8*>(qkv + static_cast<size_t>(t) * ldqkv + off)[sl];
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = bf2f(a.v[j]), x[j] = bf2f(b.v[j]);
        }
      }
      // transpose of the rotation: dy_i = do_i c + do_{i+half} s ; dy_{i+half} = do_{i+half} c - do_i s
      float dy[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float other = __shfl_sync(0xffffffffu, d[j], (in_rot ? partner : lane) & 31);
        if (in_rot) {
          const float c = cs[j], s = sn[j];
          dy[j] = first_half ? d[j] * c + other * s : d[j] * c - other * s;
        } else {
          dy[j] = d[j];
        }
      }
      float dx[8];
      if (QK_NORM) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
        ss = group_sum(ss);
        const float rs = rsqrtf(ss / static_cast<float>(D) + eps);
        const bool is_q = h < Hq;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += dy[j] * (is_q ? gq[j] : gk[j]) * (x[j] * rs);
        dot = group_sum(dot) / static_cast<float>(D);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = x[j] * rs;
          dx[j] = rs * (dy[j] * (is_q ? gq[j] : gk[j]) - n * dot);
          if (on && !is_v) {
            if (is_q) accq[j] += dy[j] * n; else acck[j] += dy[j] * n;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) dx[j] = dy[j];
      }
      if (on && !is_v) {
        BF8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = f2bf(dx[j]);
        reinterpret_cast<BF8*>(dqkv + static_cast<size_t>(t) * ldqkv + off)[sl] = o;
      }
    }
  }
  if (QK_NORM) {
    // the head slots of a warp accumulated the same elements: fold them into slot 0
    if (hpw > 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        for (int o2 = nact; o2 < 32; o2 <<= 1) {
          accq[j] += __shfl_xor_sync(0xffffffffu, accq[j], o2);
          acck[j] += __shfl_xor_sync(0xffffffffu, acck[j], o2);
        }
      }
    }
    if (lane < nact) {
#pragma unroll
      for (int j = 0; j < 8; ++j) s_w[warp][0][e0 + j] = accq[j], s_w[warp][1][e0 + j] = acck[j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * D; c += 128) {
      const int which = c / D, e = c % D;
      dw_partial[static_cast<size_t>(blockIdx.x) * 2 * D + c] = ((s_w[0][which][e] + s_w[1][which][e]) + s_w[2][which][e]) + s_w[3][which][e];
    }
  }
}

}  // namespace

IX_API int ix_bwd_num_partials() { return kQkBwdCtas; }

// h: the normalised input ([rows, N] bf16: x + residual when there was a residual), rstd fp32 [rows], dy bf16.
// dres: gradient arriving on the residual output (or null). dh: gradient of h (bf16). dw_partial: fp32
// [ix_bwd_num_partials(), N] scratch; dw: bf16 [N] (or null to skip the fold).
IX_API int ix_rmsnorm_bwd(const void* h, const void* w, const void* rstd, const void* dy, const void* dres, void* dh, void* dw_partial,
                          void* dw, int rows, int N, int zero_centered, void* stream) {
  if (rows <= 0) return 0;
  if ((N & 7) || N > 8192) return ixh::fail(ixh::IX_EARG, "rmsnorm_bwd: N=%d must be a multiple of 8, at most 8192", N);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int grid = rows;
  if (grid > kBwdCtas) grid = kBwdCtas;
#define IX_RB(ZC, DR)                                                                                                   \
  {                                                                                                                     \
    auto kern = N <= 4096 ? rmsnorm_bwd_kernel<ZC, DR, 4> : rmsnorm_bwd_kernel<ZC, DR, 8>;                              \
    kern<<<grid, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w),           \
                                 static_cast<const float*>(rstd), static_cast<const __nv_bfloat16*>(dy),                \
                                 static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dh),              \
                                 static_cast<float*>(dw_partial), rows, N);                                             \
  }
  if (zero_centered) {
    if (dres) IX_RB(true, true) else IX_RB(true, false)
  } else {
    if (dres) IX_RB(false, true) else IX_RB(false, false)
  }
#undef IX_RB
  IX_CUDA(cudaGetLastError());
  if (dw) {
    fold_partials_kernel<<<(N + 255) / 256, 256, 0, s>>>(static_cast<const float*>(dw_partial), grid, N, static_cast<__nv_bfloat16*>(dw));
    IX_CUDA(cudaGetLastError());
  }
  return 0;
}

// dw_partial: fp32 [ix_bwd_num_partials(), 2, D] scratch; dwq/dwk: bf16 [D] outputs (only with qk_norm).
IX_API int ix_qk_norm_rope_bwd(const void* qkv, long long ldqkv, const void* positions, const void* cos_tab, const void* sin_tab,
                               const void* qw, const void* kw, const void* dq, const void* dk, const void* dv, void* dqkv,
                               void* dw_partial, void* dwq, void* dwk, int T, int Hq, int Hkv, int D, int rot_dim, float eps,
                               int qk_norm, int zero_centered, int q_gate, void* stream) {
  if (T <= 0) return 0;
  if ((D & 7) || D > 256 || (rot_dim & 15) || rot_dim > D) return ixh::fail(ixh::IX_EARG, "qk_norm_rope_bwd: D=%d rot_dim=%d unsupported", D, rot_dim);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int Htot = Hq + 2 * Hkv;
  const int nact = D >> 3;
  const bool pow2 = (nact & (nact - 1)) == 0;
  const int hpw = (pow2 && nact <= 16) ? 32 / nact : 1;
  int red_width = 1;
  while (red_width < nact) red_width <<= 1;
  int wpt = (Htot + hpw - 1) / hpw;
  if (wpt > 8) wpt = 8;
  const long long total = static_cast<long long>(T) * wpt;
  int grid = static_cast<int>((total + 3) / 4 > kQkBwdCtas ? kQkBwdCtas : (total + 3) / 4);
#define IX_QB(QN, ZC)                                                                                                          \
  qk_norm_rope_bwd_kernel<QN, ZC><<<grid, 128, 0, s>>>(                                                                        \
      static_cast<const __nv_bfloat16*>(qkv), ldqkv, static_cast<const int*>(positions), static_cast<const float*>(cos_tab),   \
      static_cast<const float*>(sin_tab), static_cast<const __nv_bfloat16*>(qw), static_cast<const __nv_bfloat16*>(kw),        \
      static_cast<const __nv_bfloat16*>(dq), static_cast<const __nv_bfloat16*>(dk), static_cast<const __nv_bfloat16*>(dv),     \
      static_cast<__nv_bfloat16*>(dqkv), static_cast<float*>(dw_partial), T, Hq, Hkv, D, rot_dim, eps, q_gate, wpt, hpw, red_width);
  if (qk_norm) {
    if (zero_centered) IX_QB(true, true) else IX_QB(true, false)
  } else {
    IX_QB(false, false)
  }
#undef IX_QB
  IX_CUDA(cudaGetLastError());
  if (qk_norm && dwq && dwk) {
    // partial rows are [q(D) | k(D)]: fold both halves in one launch, then split
    fold_partials_kernel<<<(2 * D + 255) / 256, 256, 0, s>>>(static_cast<const float*>(dw_partial), grid, 2 * D, static_cast<__nv_bfloat16*>(dwq));
    IX_CUDA(cudaGetLastError());
  }
  return 0;
}
