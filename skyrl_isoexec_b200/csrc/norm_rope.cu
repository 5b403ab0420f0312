// Row-wise normalisation / activation kernels shared by the trainer and the rollout
// engine. One warp owns one row (or one (token, head) pair), so a row's bits never
// depend on how many rows the launch has.
//
// Rounding chains (each step is one explicit round-to-nearest op, no FMA contraction):
//   RMSNorm   h = bf16(x + r)                          (only with a residual input)
//             ss = sum over the row of fp32(h*h): lane l keeps four chains, chain u over the 8-element
//                  vectors l+32u, l+32u+128, ... in ascending order, folds them as (c0+c1)+(c2+c3),
//                  then a 5-step xor butterfly (16,8,4,2,1) over the lanes. The same order is produced
//                  by the warp-per-row kernel and by the CTA-per-row kernel used for few rows.
//             rstd = 1 / sqrt(ss / N + eps)            (div.rn, sqrt.rn)
//             n = bf16(h * rstd);  y = bf16(n * g),  g = w or bf16(1 + w) (zero-centred)
//   RoPE      a = bf16(y*cos)  b = bf16(rot(y)*sin)  out = bf16(a + b)   (three rounds;
//             the reference pins the same three-round chain, ISO/ops/rope/rope_fused.py:49-105)
//   SwiGLU    s = bf16(g / (1 + exp(-g)));  out = bf16(s * u)
//   gated out-norm (GatedDeltaNet): n,y as RMSNorm; out = bf16(y * bf16(silu(z)))
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

struct alignas(16) BF8 {
  __nv_bfloat16 v[8];
};

__device__ __forceinline__ float silu_f32(float g) {
  return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
}

// ------------------------------------------------------------------ RMSNorm (+residual)
template <bool HAS_RES, bool ZERO_CENTERED>
__global__ void __launch_bounds__(128)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
               __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int rows, int N, float eps,
               long long ldx, long long ldy) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nvec = N >> 3;
  const BF8* xr = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * ldx);
  const BF8* rr = HAS_RES ? reinterpret_cast<const BF8*>(res + static_cast<size_t>(row) * N) : nullptr;
  BF8* ro = HAS_RES ? reinterpret_cast<BF8*>(res_out + static_cast<size_t>(row) * N) : nullptr;
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  // four vectors per lane are loaded before any is consumed (memory-level parallelism); vector u of a
  // batch feeds chain u
  for (int v0 = lane; v0 < nvec; v0 += 128) {
    BF8 a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        a[u] = xr[v];
        if (HAS_RES) b[u] = rr[v];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        if (HAS_RES) {
#pragma unroll
          for (int j = 0; j < 8; ++j) a[u].v[j] = f2bf(__fadd_rn(bf2f(a[u].v[j]), bf2f(b[u].v[j])));
          ro[v] = a[u];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = bf2f(a[u].v[j]);
          c[u] = __fadd_rn(c[u], __fmul_rn(f, f));
        }
      }
    }
  }
  const float ss = warp_sum_butterfly(__fadd_rn(__fadd_rn(c[0], c[1]), __fadd_rn(c[2], c[3])));
  const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(N)), eps)));
  if (rstd_out && lane == 0) rstd_out[row] = rstd;
  const BF8* hr = HAS_RES ? reinterpret_cast<const BF8*>(res_out + static_cast<size_t>(row) * N) : xr;
  const BF8* wr = reinterpret_cast<const BF8*>(w);
  BF8* yr = reinterpret_cast<BF8*>(y + static_cast<size_t>(row) * ldy);
  for (int v0 = lane; v0 < nvec; v0 += 128) {
    BF8 a[4], g[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        a[u] = hr[v];  // same lane wrote it above (HAS_RES), so no cross-thread hazard
        g[u] = wr[v];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        BF8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = round_bf(__fmul_rn(bf2f(a[u].v[j]), rstd));
          float gg = bf2f(g[u].v[j]);
          if (ZERO_CENTERED) gg = round_bf(__fadd_rn(1.0f, gg));
          o.v[j] = f2bf(__fmul_rn(n, gg));
        }
        yr[v] = o;
      }
    }
  }
}

// Same function and the same bits, for launches with few rows (decode): one CTA of 128 threads per row, warp u
// computes chain u of every lane, the row stays in registers between the two phases. N <= 8192.
template <bool HAS_RES, bool ZERO_CENTERED>
__global__ void __launch_bounds__(128)
rmsnorm_cta_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                       __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int N, float eps,
                       long long ldx, long long ldy) {
  __shared__ float s_c[4][32];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int u = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = N >> 3;
  const BF8* xr = reinterpret_cast<const BF8*>(x + static_cast<size_t>(row) * ldx);
  BF8 a[8], g[8];
  float c = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {           // vector l + 32u + 128 i: chain u of lane l, ascending
    const int v = lane + 32 * u + 128 * i;
    if (v < nvec) {
      a[i] = xr[v];
      g[i] = reinterpret_cast<const BF8*>(w)[v];
      if (HAS_RES) {
        const BF8 b = reinterpret_cast<const BF8*>(res + static_cast<size_t>(row) * N)[v];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[i].v[j] = f2bf(__fadd_rn(bf2f(a[i].v[j]), bf2f(b.v[j])));
        reinterpret_cast<BF8*>(res_out + static_cast<size_t>(row) * N)[v] = a[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (lane + 32 * u + 128 * i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = bf2f(a[i].v[j]);
        c = __fadd_rn(c, __fmul_rn(f, f));
      }
    }
  }
  s_c[u][lane] = c;
  __syncthreads();
  const float ss = warp_sum_butterfly(__fadd_rn(__fadd_rn(s_c[0][lane], s_c[1][lane]), __fadd_rn(s_c[2][lane], s_c[3][lane])));
  const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(N)), eps)));
  if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
  BF8* yr = reinterpret_cast<BF8*>(y + static_cast<size_t>(row) * ldy);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int v = lane + 32 * u + 128 * i;
    if (v < nvec) {
      BF8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float n = round_bf(__fmul_rn(bf2f(a[i].v[j]), rstd));
        float gg = bf2f(g[i].v[j]);
        if (ZERO_CENTERED) gg = round_bf(__fadd_rn(1.0f, gg));
        o.v[j] = f2bf(__fmul_rn(n, gg));
      }
      yr[v] = o;
    }
  }
}

// ------------------------------------------------------------------ QK-norm + RoPE + KV write
// qkv: [T, (Hq + 2*Hkv) * D] as produced by the fused QKV projection (row stride ldqkv),
// KV-group major (see below).
// q heads -> q_out[T, Hq, D]; k heads -> k_out[slot, Hkv, D]; v heads -> v_out[slot, Hkv, D] with
// slot = slots ? slots[t] : t (paged cache or packed).
//
// Work layout. A head occupies nact = D / 8 lanes (8 elements each; the 8-per-lane split is part of the pinned
// summation order). hpw = 32 / nact heads share a warp when nact is a power of two (two heads for D = 128), each in
// its own aligned lane group; the row sum then runs over the group only, which gives the bits of the full-warp
// butterfly over one head padded with zero lanes, because the skipped steps only ever added +0. wpt warps share a
// token; the warp with index w takes heads w, w + wpt, w + 2 wpt, ..., hpw at a time, and fetches the rotation
// constants and norm weights of its lanes once. A head's arithmetic depends on neither hpw nor wpt.
template <bool QK_NORM, bool ZERO_CENTERED>
__global__ void __launch_bounds__(128)
qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ qkv, long long ldqkv, const int* __restrict__ positions,
                    const long long* __restrict__ slots, const float* __restrict__ cos_tab,
                    const float* __restrict__ sin_tab, const __nv_bfloat16* __restrict__ qw,
                    const __nv_bfloat16* __restrict__ kw, __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ v_out, int T, int Hq, int Hkv,
                    int D, int rot_dim, float eps, int q_gate, int wpt, int hpw, int red_width) {
  pdl_launch_dependents();
  pdl_wait();
  const int Htot = Hq + 2 * Hkv;
  const long long wid = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(T) * wpt) return;
  const int t = static_cast<int>(wid / wpt);
  const int h0 = static_cast<int>(wid % wpt);
  const int nact = D >> 3;                 // lanes per head
  const int sub = lane / nact;             // which of the warp's head slots this lane belongs to
  const int sl = lane - sub * nact;        // lane within the head
  const bool lane_on = sub < hpw;
  // Row layout is KV-group major: for each KV head g, [its G query heads | k_g | v_g], so a
  // tensor-parallel shard (whole groups) is a contiguous slice. With an output gate (gated
  // attention) the block of a query head is [q(D) | gate(D)].
  const int q_stride = q_gate ? 2 * D : D;
  const int G = Hq / Hkv;
  const long long grp_stride = static_cast<long long>(G) * q_stride + 2 * D;
  const long long slot = slots ? slots[t] : t;
  // rotate-half over the first rot_dim elements: element i pairs with i +- rot_dim/2
  const int half = rot_dim >> 1;
  const int half_lanes = half >> 3;  // lanes per half (rot_dim multiple of 16)
  const int pos = positions[t];
  const int e0 = sl * 8;
  const bool in_rot = lane_on && e0 < rot_dim;
  const bool first_half = e0 < half;
  const int partner = sub * nact + (first_half ? sl + half_lanes : sl - half_lanes);
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
  BF8 gq, gk;
#pragma unroll
  for (int j = 0; j < 8; ++j) gq.v[j] = gk.v[j] = f2bf(0.f);
  if (QK_NORM && lane_on) {
    gq = reinterpret_cast<const BF8*>(qw)[sl];
    gk = reinterpret_cast<const BF8*>(kw)[sl];
  }
  for (int hb = h0; hb < Htot; hb += wpt * hpw) {     // the same trip count for every lane of the warp
    const int h = hb + sub * wpt;
    const bool on = lane_on && h < Htot;
    const bool is_v = h >= Hq + Hkv;
    BF8 a;
#pragma unroll
    for (int j = 0; j < 8; ++j) a.v[j] = f2bf(0.f);
    if (on) {
      long long src_off;
      if (h < Hq) src_off = (h / G) * grp_stride + static_cast<long long>(h % G) * q_stride;
      else if (!is_v) src_off = (h - Hq) * grp_stride + static_cast<long long>(G) * q_stride;
      else src_off = (h - Hq - Hkv) * grp_stride + static_cast<long long>(G) * q_stride + D;
      a = reinterpret_cast<const BF8*>(qkv + static_cast<size_t>(t) * ldqkv + src_off)[sl];
      if (is_v && slot >= 0)   // a value head: copy (its lanes still take part in the shuffles below)
        reinterpret_cast<BF8*>(v_out + (static_cast<size_t>(slot) * Hkv + (h - Hq - Hkv)) * D)[sl] = a;
    }
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = bf2f(a.v[j]);
    if (QK_NORM) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(y[j], y[j]));
      // the steps of warp_sum_butterfly that stay inside the head's lane group, in the same order (16, 8, 4, 2, 1)
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1)
        if (off < red_width) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
      const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(D)), eps)));
      const BF8& g = (h < Hq) ? gq : gk;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float n = round_bf(__fmul_rn(y[j], rstd));
        float gg = bf2f(g.v[j]);
        if (ZERO_CENTERED) gg = round_bf(__fadd_rn(1.0f, gg));
        y[j] = round_bf(__fmul_rn(n, gg));
      }
    }
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float other = __shfl_sync(0xffffffffu, y[j], (in_rot ? partner : lane) & 31);
      if (in_rot) {
        const float rot = first_half ? __fmul_rn(other, -1.0f) : other;
        const float p1 = round_bf(__fmul_rn(y[j], cs[j]));
        const float p2 = round_bf(__fmul_rn(rot, sn[j]));
        o[j] = __fadd_rn(p1, p2);
      } else {
        o[j] = y[j];
      }
    }
    if (on && !is_v) {
      BF8 r;
#pragma unroll
      for (int j = 0; j < 8; ++j) r.v[j] = f2bf(o[j]);
      if (h < Hq) reinterpret_cast<BF8*>(q_out + (static_cast<size_t>(t) * Hq + h) * D)[sl] = r;
      else if (slot >= 0) reinterpret_cast<BF8*>(k_out + (static_cast<size_t>(slot) * Hkv + (h - Hq)) * D)[sl] = r;
    }
  }
}

// ------------------------------------------------------------------ SwiGLU
// in: [T, 2F] = [gate | up]; out: [T, F]
__global__ void __launch_bounds__(256)
swiglu_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long T, int F,
              long long ld_in) {
  const long long nvec_row = F >> 3;
  const long long total = T * nvec_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec_row;
    const long long v = i % nvec_row;
    const BF8 g = reinterpret_cast<const BF8*>(in + t * ld_in)[v];
    const BF8 u = reinterpret_cast<const BF8*>(in + t * ld_in + F)[v];
    BF8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = round_bf(silu_f32(bf2f(g.v[j])));
      o.v[j] = f2bf(__fmul_rn(s, bf2f(u.v[j])));
    }
    reinterpret_cast<BF8*>(out + t * F)[v] = o;
  }
}

// d(gate), d(up) from d(out); recomputes silu. din: [T, 2F]
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                  __nv_bfloat16* __restrict__ din, long long T, int F, long long ld_in) {
  const long long nvec_row = F >> 3;
  const long long total = T * nvec_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec_row;
    const long long v = i % nvec_row;
    const BF8 g = reinterpret_cast<const BF8*>(in + t * ld_in)[v];
    const BF8 u = reinterpret_cast<const BF8*>(in + t * ld_in + F)[v];
    const BF8 d = reinterpret_cast<const BF8*>(dout + t * F)[v];
    BF8 dg, du;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gf = bf2f(g.v[j]), uf = bf2f(u.v[j]), df = bf2f(d.v[j]);
      const float sig = 1.0f / (1.0f + expf(-gf));
      const float s = gf * sig;
      du.v[j] = f2bf(df * s);
      dg.v[j] = f2bf(df * uf * (sig * (1.0f + gf * (1.0f - sig))));
    }
    reinterpret_cast<BF8*>(din + t * 2 * F)[v] = dg;
    reinterpret_cast<BF8*>(din + t * 2 * F + F)[v] = du;
  }
}

// ------------------------------------------------------------------ gated multiply: out = bf16(a * bf16(sigmoid(g)))
// used for the output gate of gated attention. a: [T, H*D] ; g read from qkv block layout.
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ qkv, long long ldqkv,
                    __nv_bfloat16* __restrict__ out, long long T, int Hq, int Hkv, int D) {
  const int G = Hq / Hkv;
  const long long grp_stride = static_cast<long long>(G) * 2 * D + 2 * D;
  const long long nvec_row = static_cast<long long>(Hq) * D >> 3;
  const long long total = T * nvec_row;
  const int vec_per_head = D >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / nvec_row;
    const long long v = i % nvec_row;
    const int h = static_cast<int>(v / vec_per_head);
    const int vv = static_cast<int>(v % vec_per_head);
    const BF8 x = reinterpret_cast<const BF8*>(a + t * Hq * D)[v];
    const BF8 g = reinterpret_cast<const BF8*>(qkv + t * ldqkv + (h / G) * grp_stride +
                                                static_cast<long long>(h % G) * 2 * D + D)[vv];
    BF8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gf = bf2f(g.v[j]);
      const float s = round_bf(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gf))));
      o.v[j] = f2bf(__fmul_rn(bf2f(x.v[j]), s));
    }
    reinterpret_cast<BF8*>(out + t * Hq * D)[v] = o;
  }
}

// ------------------------------------------------------------------ gated out-norm (GDN): per (token, head) over Dv
// out = bf16( bf16(bf16(o*rstd) * g) * bf16(silu(z)) ),  g = w or bf16(1+w)
// HALF: rows of at most 128 elements need 16 lanes, so a warp takes two rows. The 16-lane butterfly has the bits of the
// 32-lane one over a row padded with zero lanes (the skipped first step only ever added +0), so both forms agree with
// each other and with the CPU oracle.
template <bool ZERO_CENTERED, bool HALF>
__global__ void __launch_bounds__(128)
gated_outnorm_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long rows, int D,
                     float eps) {
  constexpr int L = HALF ? 16 : 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = HALF ? (static_cast<long long>(blockIdx.x) * 8 + warp * 2 + (lane >> 4))
                             : (static_cast<long long>(blockIdx.x) * 4 + warp);
  const int sub = lane & (L - 1);
  const bool live = row < rows;
  const int nvec = D >> 3;
  const BF8* orow = reinterpret_cast<const BF8*>(o + (live ? row : 0) * D);
  const BF8* zrow = reinterpret_cast<const BF8*>(z + (live ? row : 0) * D);
  float ss = 0.f;
  BF8 a0;                                   // the common case (D <= 8 * L) keeps the row's vector in registers
  const bool one = nvec <= L;
  if (one) {
    if (sub < nvec && live) {
      a0 = orow[sub];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = bf2f(a0.v[j]);
        ss = __fadd_rn(ss, __fmul_rn(f, f));
      }
    }
  } else {
    for (int v = sub; v < nvec && live; v += L) {
      const BF8 a = orow[v];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = bf2f(a.v[j]);
        ss = __fadd_rn(ss, __fmul_rn(f, f));
      }
    }
  }
#pragma unroll
  for (int off = L / 2; off >= 1; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
  if (!live) return;
  const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(D)), eps)));
  for (int v = sub; v < nvec; v += L) {
    const BF8 a = one ? a0 : orow[v];
    const BF8 zz = zrow[v];
    const BF8 g = reinterpret_cast<const BF8*>(w)[v];
    BF8 r;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float n = round_bf(__fmul_rn(bf2f(a.v[j]), rstd));
      float gg = bf2f(g.v[j]);
      if (ZERO_CENTERED) gg = round_bf(__fadd_rn(1.0f, gg));
      const float yv = round_bf(__fmul_rn(n, gg));
      const float s = round_bf(silu_f32(bf2f(zz.v[j])));
      r.v[j] = f2bf(__fmul_rn(yv, s));
    }
    reinterpret_cast<BF8*>(out + row * D)[v] = r;
  }
}

inline int grid_1d(long long total, int block, int cap = 148 * 16) {
  long long g = (total + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

IX_API int ix_rmsnorm(const void* x, const void* res, const void* w, void* y, void* res_out, void* rstd_out,
                      int rows, int N, float eps, int zero_centered, long long ldx, long long ldy, void* stream) {
  if (rows <= 0) return 0;
  if (N & 7) return ixh::fail(ixh::IX_EARG, "rmsnorm: N=%d must be a multiple of 8", N);
  if ((ldx & 7) || (ldy & 7)) return ixh::fail(ixh::IX_EARG, "rmsnorm: ldx/ldy must be multiples of 8");
  if (res && !res_out) return ixh::fail(ixh::IX_EARG, "rmsnorm: residual input needs res_out");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = (rows + 3) / 4;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(res);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto RO = static_cast<__nv_bfloat16*>(res_out);
  auto RS = static_cast<float*>(rstd_out);
  if (rows <= 1024 && N <= 8192) {
    // few rows: a CTA per row (more threads per row, one memory round trip); same bits as the warp-per-row kernel.
    // At thousands of rows this form measured 2x slower than the warp-per-row kernel (16384 x 4096: 180 us against 94 us)
    if (res) {
      if (zero_centered) IX_CUDA(ixh::launch_pdl(rmsnorm_cta_row_kernel<true, true>, dim3(rows), dim3(128), 0, s, X, R, W, Y, RO, RS, N, eps, ldx, ldy));
      else IX_CUDA(ixh::launch_pdl(rmsnorm_cta_row_kernel<true, false>, dim3(rows), dim3(128), 0, s, X, R, W, Y, RO, RS, N, eps, ldx, ldy));
    } else {
      if (zero_centered) IX_CUDA(ixh::launch_pdl(rmsnorm_cta_row_kernel<false, true>, dim3(rows), dim3(128), 0, s, X, R, W, Y, RO, RS, N, eps, ldx, ldy));
      else IX_CUDA(ixh::launch_pdl(rmsnorm_cta_row_kernel<false, false>, dim3(rows), dim3(128), 0, s, X, R, W, Y, RO, RS, N, eps, ldx, ldy));
    }
    IX_CUDA(cudaGetLastError());
    return 0;
  }
  if (res) {
    if (zero_centered) rmsnorm_kernel<true, true><<<grid, 128, 0, s>>>(X, R, W, Y, RO, RS, rows, N, eps, ldx, ldy);
    else rmsnorm_kernel<true, false><<<grid, 128, 0, s>>>(X, R, W, Y, RO, RS, rows, N, eps, ldx, ldy);
  } else {
    if (zero_centered) rmsnorm_kernel<false, true><<<grid, 128, 0, s>>>(X, R, W, Y, RO, RS, rows, N, eps, ldx, ldy);
    else rmsnorm_kernel<false, false><<<grid, 128, 0, s>>>(X, R, W, Y, RO, RS, rows, N, eps, ldx, ldy);
  }
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_qk_norm_rope(const void* qkv, long long ldqkv, const void* positions, const void* slots,
                           const void* cos_tab, const void* sin_tab, const void* qw, const void* kw, void* q_out,
                           void* k_out, void* v_out, int T, int Hq, int Hkv, int D, int rot_dim, float eps,
                           int qk_norm, int zero_centered, int q_gate, void* stream) {
  if (T <= 0) return 0;
  if (D > 256 || (D & 7)) return ixh::fail(ixh::IX_EARG, "qk_norm_rope: head dim %d unsupported", D);
  if ((rot_dim & 15) || rot_dim > D) return ixh::fail(ixh::IX_EARG, "qk_norm_rope: rot_dim %d unsupported", rot_dim);
  if (ldqkv & 7) return ixh::fail(ixh::IX_EARG, "qk_norm_rope: ldqkv must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // lanes per head, heads per warp (power-of-two lane groups only), width of the row-sum butterfly
  const int Htot = Hq + 2 * Hkv;
  const int nact = D >> 3;
  const bool pow2 = (nact & (nact - 1)) == 0;
  const int hpw = (pow2 && nact <= 16) ? 32 / nact : 1;
  int red_width = 1;
  while (red_width < nact) red_width <<= 1;
  // decode-sized T: every warp makes one pass (hpw heads); otherwise a warp walks several heads of its token and
  // reuses the per-token constants
  int wpt = (Htot + hpw - 1) / hpw;
  if (T > 1024 && wpt > 8) wpt = 8;
  const long long warps = static_cast<long long>(T) * wpt;
  const int grid = static_cast<int>((warps + 3) / 4);
#define IX_QKR(N_, Z_)                                                                                                  \
  IX_CUDA(ixh::launch_pdl(qk_norm_rope_kernel<N_, Z_>, dim3(grid), dim3(128), 0, s, static_cast<const __nv_bfloat16*>(qkv), \
                          ldqkv, static_cast<const int*>(positions), static_cast<const long long*>(slots),              \
                          static_cast<const float*>(cos_tab), static_cast<const float*>(sin_tab),                       \
                          static_cast<const __nv_bfloat16*>(qw), static_cast<const __nv_bfloat16*>(kw),                 \
                          static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_out),                       \
                          static_cast<__nv_bfloat16*>(v_out), T, Hq, Hkv, D, rot_dim, eps, q_gate, wpt, hpw, red_width))
  if (qk_norm) {
    if (zero_centered) IX_QKR(true, true);
    else IX_QKR(true, false);
  } else {
    IX_QKR(false, false);
  }
#undef IX_QKR
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_swiglu(const void* in, void* out, long long T, int F, long long ld_in, void* stream) {
  if (T <= 0) return 0;
  if ((F & 7) || (ld_in & 7)) return ixh::fail(ixh::IX_EARG, "swiglu: F and ld_in must be multiples of 8");
  swiglu_kernel<<<grid_1d(T * (F >> 3), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), T, F, ld_in);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_swiglu_bwd(const void* in, const void* dout, void* din, long long T, int F, long long ld_in,
                         void* stream) {
  if (T <= 0) return 0;
  if ((F & 7) || (ld_in & 7)) return ixh::fail(ixh::IX_EARG, "swiglu_bwd: F and ld_in must be multiples of 8");
  swiglu_bwd_kernel<<<grid_1d(T * (F >> 3), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), static_cast<const __nv_bfloat16*>(dout),
      static_cast<__nv_bfloat16*>(din), T, F, ld_in);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_sigmoid_gate(const void* a, const void* qkv, long long ldqkv, void* out, long long T, int Hq, int Hkv,
                           int D, void* stream) {
  if (T <= 0) return 0;
  if ((D & 7) || (ldqkv & 7)) return ixh::fail(ixh::IX_EARG, "sigmoid_gate: D and ldqkv must be multiples of 8");
  sigmoid_gate_kernel<<<grid_1d(T * (static_cast<long long>(Hq) * D >> 3), 256), 256, 0,
                        reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(qkv), ldqkv,
      static_cast<__nv_bfloat16*>(out), T, Hq, Hkv, D);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_gated_outnorm(const void* o, const void* z, const void* w, void* out, long long rows, int D,
                            float eps, int zero_centered, void* stream) {
  if (rows <= 0) return 0;
  if (D & 7) return ixh::fail(ixh::IX_EARG, "gated_outnorm: D must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto O = static_cast<const __nv_bfloat16*>(o);
  auto Z = static_cast<const __nv_bfloat16*>(z);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(out);
  if (D <= 128) {
    const int grid = static_cast<int>((rows + 7) / 8);
    if (zero_centered) gated_outnorm_kernel<true, true><<<grid, 128, 0, s>>>(O, Z, W, Y, rows, D, eps);
    else gated_outnorm_kernel<false, true><<<grid, 128, 0, s>>>(O, Z, W, Y, rows, D, eps);
  } else {
    const int grid = static_cast<int>((rows + 3) / 4);
    if (zero_centered) gated_outnorm_kernel<true, false><<<grid, 128, 0, s>>>(O, Z, W, Y, rows, D, eps);
    else gated_outnorm_kernel<false, false><<<grid, 128, 0, s>>>(O, Z, W, Y, rows, D, eps);
  }
  IX_CUDA(cudaGetLastError());
  return 0;
}
