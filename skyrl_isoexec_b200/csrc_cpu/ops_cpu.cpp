// CPU restatement of the library's kernels with the SAME reduction orders and rounding
// points as the sm_100a kernels (csrc/*.cu). Two jobs:
//   1. the oracle every CUDA kernel is tested against (bitwise where the chain has no
//      transcendental function, tight tolerance where expf/exp2f/logf implementations differ);
//   2. the compute path of the CPU/gloo configuration (fp32 model, trainer and rollout in
//      separate processes), where batch invariance must hold without any GPU.
// Built with -ffp-contract=off so a*b+c is never fused. dtype codes: 0 = bf16, 1 = fp32.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <vector>

#define IXC_API extern "C" __attribute__((visibility("default")))

namespace {

inline float bf16_to_f(uint16_t v) {
  uint32_t u = static_cast<uint32_t>(v) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline float round_bf(float f) { return bf16_to_f(f_to_bf16(f)); }

// activation accessors: T = uint16_t (bf16) or float
template <typename T> inline float ld(const T* p, long long i);
template <> inline float ld<uint16_t>(const uint16_t* p, long long i) { return bf16_to_f(p[i]); }
template <> inline float ld<float>(const float* p, long long i) { return p[i]; }
template <typename T> inline void st(T* p, long long i, float v);
template <> inline void st<uint16_t>(uint16_t* p, long long i, float v) { p[i] = f_to_bf16(v); }
template <> inline void st<float>(float* p, long long i, float v) { p[i] = v; }
// "round to the activation dtype": bf16 rounds, fp32 is the identity
template <typename T> inline float rnd(float v);
template <> inline float rnd<uint16_t>(float v) { return round_bf(v); }
template <> inline float rnd<float>(float v) { return v; }

// The 32-lane xor butterfly of the CUDA kernels: after the 5 steps every lane holds the same
// association, which for lane 0 is the expression computed here.
inline float butterfly32(float* lane) {
  for (int off = 16; off >= 1; off >>= 1) {
    float nxt[32];
    for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ off];
    memcpy(lane, nxt, sizeof(nxt));
  }
  return lane[0];
}

inline float rstd_of(float ss, int N, float eps) { return 1.0f / sqrtf(ss / static_cast<float>(N) + eps); }

// ------------------------------------------------------------------ GEMM (batch-invariant)
template <typename TI, typename TO>
void gemm_nt(const TI* x, const TI* w, TO* out, int M, int N, int K, long long lda, long long ldb, long long ldc) {
  std::vector<float> wT(static_cast<size_t>(K) * N);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) wT[static_cast<size_t>(k) * N + n] = ld(w, n * ldb + k);
#pragma omp parallel
  {
    std::vector<float> acc(N);
#pragma omp for schedule(static)
    for (int m = 0; m < M; ++m) {
      std::fill(acc.begin(), acc.end(), 0.f);
      for (int k = 0; k < K; ++k) {
        const float xv = ld(x, m * lda + k);
        const float* wr = &wT[static_cast<size_t>(k) * N];
        for (int n = 0; n < N; ++n) acc[n] = acc[n] + xv * wr[n];
      }
      for (int n = 0; n < N; ++n) st(out, m * ldc + n, acc[n]);
    }
  }
}

// Leaf-tree GEMM: K is cut into G equal leaves; leaf j is the sequential fp32 sum over its
// K slice (optionally rounded to bf16 at the leaf boundary); leaves [leaf_lo, leaf_hi) are
// folded by the fixed adjacent-pair tree. With leaf_lo=0, leaf_hi=G this is the whole product;
// a TP rank passes its own contiguous leaf range and x/w already sliced to that range.
template <typename TI>
void leaftree_gemm(const TI* x, const TI* w, float* out, int M, int N, int Kloc, int nleaves, int round_leaf,
                   long long lda, long long ldb, long long ldc) {
  const int LK = Kloc / nleaves;
  std::vector<float> wT(static_cast<size_t>(Kloc) * N);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < Kloc; ++k) wT[static_cast<size_t>(k) * N + n] = ld(w, n * ldb + k);
#pragma omp parallel
  {
    std::vector<float> leaf(static_cast<size_t>(nleaves) * N);
#pragma omp for schedule(static)
    for (int m = 0; m < M; ++m) {
      std::fill(leaf.begin(), leaf.end(), 0.f);
      for (int j = 0; j < nleaves; ++j) {
        float* acc = &leaf[static_cast<size_t>(j) * N];
        for (int k = j * LK; k < (j + 1) * LK; ++k) {
          const float xv = ld(x, m * lda + k);
          const float* wr = &wT[static_cast<size_t>(k) * N];
          for (int n = 0; n < N; ++n) acc[n] = acc[n] + xv * wr[n];
        }
        if (round_leaf)
          for (int n = 0; n < N; ++n) acc[n] = round_bf(acc[n]);
      }
      for (int cnt = nleaves; cnt > 1; cnt >>= 1)
        for (int i = 0; i < cnt / 2; ++i) {
          float* a = &leaf[static_cast<size_t>(i) * N];
          const float* lo = &leaf[static_cast<size_t>(2 * i) * N];
          const float* hi = &leaf[static_cast<size_t>(2 * i + 1) * N];
          for (int n = 0; n < N; ++n) a[n] = lo[n] + hi[n];
        }
      for (int n = 0; n < N; ++n) out[m * ldc + n] = leaf[n];
    }
  }
}

// ------------------------------------------------------------------ RMSNorm
template <typename T>
void rmsnorm(const T* x, const T* res, const T* w, T* y, T* res_out, float* rstd_out, int rows, int N, float eps,
             int zero_centered, long long ldx, long long ldy) {
  const int nvec = N / 8;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    std::vector<float> h(N);
    for (int i = 0; i < N; ++i) {
      float v = ld(x, r * ldx + i);
      if (res) {
        v = rnd<T>(v + ld(res, static_cast<long long>(r) * N + i));
        st(res_out, static_cast<long long>(r) * N + i, v);
      }
      h[i] = v;
    }
    float lane[32];
    for (int l = 0; l < 32; ++l) {
      // four interleaved chains per lane (chain u takes vectors l + 32u, l + 32u + 128, ...), folded as (c0+c1)+(c2+c3)
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      for (int u = 0; u < 4; ++u)
        for (int v = l + 32 * u; v < nvec; v += 128)
          for (int j = 0; j < 8; ++j) {
            const float f = h[v * 8 + j];
            c[u] = c[u] + f * f;
          }
      lane[l] = (c[0] + c[1]) + (c[2] + c[3]);
    }
    const float rstd = rstd_of(butterfly32(lane), N, eps);
    if (rstd_out) rstd_out[r] = rstd;
    for (int i = 0; i < N; ++i) {
      const float n = rnd<T>(h[i] * rstd);
      float g = ld(w, i);
      if (zero_centered) g = rnd<T>(1.0f + g);
      st(y, r * ldy + i, n * g);
    }
  }
}

// ------------------------------------------------------------------ QK-norm + RoPE + KV write
template <typename T>
void qk_norm_rope(const T* qkv, long long ldqkv, const int* positions, const long long* slots, const float* cos_tab,
                  const float* sin_tab, const T* qw, const T* kw, T* q_out, T* k_out, T* v_out, int Tn, int Hq, int Hkv,
                  int D, int rot_dim, float eps, int qk_norm, int zero_centered, int q_gate) {
  const int Htot = Hq + 2 * Hkv;
  const int half = rot_dim / 2;
  const int q_stride = q_gate ? 2 * D : D;
#pragma omp parallel for schedule(static)
  for (long long wid = 0; wid < static_cast<long long>(Tn) * Htot; ++wid) {
    const int t = static_cast<int>(wid / Htot), h = static_cast<int>(wid % Htot);
    const int G = Hq / Hkv;
    const long long grp_stride = static_cast<long long>(G) * q_stride + 2 * D;
    long long src_off;
    if (h < Hq) src_off = (h / G) * grp_stride + static_cast<long long>(h % G) * q_stride;
    else if (h < Hq + Hkv) src_off = (h - Hq) * grp_stride + static_cast<long long>(G) * q_stride;
    else src_off = (h - Hq - Hkv) * grp_stride + static_cast<long long>(G) * q_stride + D;
    const T* src = qkv + t * ldqkv + src_off;
    const long long slot = slots ? slots[t] : t;
    if (h >= Hq + Hkv) {
      if (slot >= 0)
        for (int i = 0; i < D; ++i) v_out[(slot * Hkv + (h - Hq - Hkv)) * D + i] = src[i];
      continue;
    }
    float y[256];
    for (int i = 0; i < D; ++i) y[i] = ld(src, i);
    if (qk_norm) {
      float lane[32];
      for (int l = 0; l < 32; ++l) {
        float ss = 0.f;
        if (l < D / 8)
          for (int j = 0; j < 8; ++j) ss = ss + y[l * 8 + j] * y[l * 8 + j];
        lane[l] = ss;
      }
      const float rstd = rstd_of(butterfly32(lane), D, eps);
      const T* wsrc = h < Hq ? qw : kw;
      for (int i = 0; i < D; ++i) {
        const float n = rnd<T>(y[i] * rstd);
        float g = ld(wsrc, i);
        if (zero_centered) g = rnd<T>(1.0f + g);
        y[i] = rnd<T>(n * g);
      }
    }
    const int pos = positions[t];
    float o[256];
    for (int i = 0; i < D; ++i) {
      if (i < rot_dim) {
        const bool first = i < half;
        const int fi = first ? i : i - half;
        const float c = cos_tab[static_cast<long long>(pos) * half + fi];
        const float s = sin_tab[static_cast<long long>(pos) * half + fi];
        const float other = first ? y[i + half] * -1.0f : y[i - half];
        const float p1 = rnd<T>(y[i] * c);
        const float p2 = rnd<T>(other * s);
        o[i] = p1 + p2;
      } else {
        o[i] = y[i];
      }
    }
    if (h < Hq)
      for (int i = 0; i < D; ++i) st(q_out, (static_cast<long long>(t) * Hq + h) * D + i, o[i]);
    else if (slot >= 0)
      for (int i = 0; i < D; ++i) st(k_out, (slot * Hkv + (h - Hq)) * D + i, o[i]);
  }
}

inline float silu_f32(float g) { return g / (1.0f + expf(-g)); }

template <typename T>
void swiglu(const T* in, T* out, long long Tn, int F, long long ld_in) {
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < Tn; ++t)
    for (int i = 0; i < F; ++i) {
      const float s = rnd<T>(silu_f32(ld(in, t * ld_in + i)));
      st(out, t * F + i, s * ld(in, t * ld_in + F + i));
    }
}

template <typename T>
void sigmoid_gate(const T* a, const T* qkv, long long ldqkv, T* out, long long Tn, int Hq, int Hkv, int D) {
  const int G = Hq / Hkv;
  const long long grp_stride = static_cast<long long>(G) * 2 * D + 2 * D;
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < Tn; ++t)
    for (int h = 0; h < Hq; ++h)
      for (int i = 0; i < D; ++i) {
        const float g = ld(qkv, t * ldqkv + (h / G) * grp_stride + static_cast<long long>(h % G) * 2 * D + D + i);
        const float s = rnd<T>(1.0f / (1.0f + expf(-g)));
        const long long o = (t * Hq + h) * D + i;
        st(out, o, ld(a, o) * s);
      }
}

template <typename T>
void gated_outnorm(const T* o, const T* z, const T* w, T* out, long long rows, int D, float eps, int zero_centered) {
  const int nvec = D / 8;
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < rows; ++r) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
      float ss = 0.f;
      for (int v = l; v < nvec; v += 32)
        for (int j = 0; j < 8; ++j) {
          const float f = ld(o, r * D + v * 8 + j);
          ss = ss + f * f;
        }
      lane[l] = ss;
    }
    const float rstd = rstd_of(butterfly32(lane), D, eps);
    for (int i = 0; i < D; ++i) {
      const float n = rnd<T>(ld(o, r * D + i) * rstd);
      float g = ld(w, i);
      if (zero_centered) g = rnd<T>(1.0f + g);
      const float yv = rnd<T>(n * g);
      const float s = rnd<T>(silu_f32(ld(z, r * D + i)));
      st(out, r * D + i, yv * s);
    }
  }
}

// ------------------------------------------------------------------ rowinv log-probabilities
constexpr int kLpThreads = 256, kLpBlock = 4096;

// fixed CTA sum: per-thread partials -> butterfly per warp -> 8 warp partials left to right
inline float cta_sum_fixed(const float* part) {
  float r = 0.f;
  for (int wp = 0; wp < kLpThreads / 32; ++wp) {
    float lane[32];
    memcpy(lane, part + wp * 32, sizeof(lane));
    const float s = butterfly32(lane);
    r = wp == 0 ? s : r + s;
  }
  return r;
}

template <typename T>
float row_max(const T* row, int n) {
  float m = -INFINITY;
  for (int i = 0; i < n; ++i) m = fmaxf(m, ld(row, i));
  return m;
}

template <typename T>
float leaf_sum(const T* row, int lo, int len, float m, float* px_out) {
  float acc = 0.f, comp = 0.f;
  float pxp[kLpThreads];
  for (int t = 0; t < kLpThreads; ++t) pxp[t] = 0.f;
  for (int off = 0; off < len; off += kLpBlock) {
    float part[kLpThreads];
    for (int t = 0; t < kLpThreads; ++t) {
      float p = 0.f;
      for (int j = 0; j < 16; ++j) {
        const int c = off + t * 16 + j;
        if (c < len) {
          const float x = ld(row, lo + c);
          const float e = expf(x - m);
          p = p + e;
          pxp[t] = pxp[t] + e * x;
        }
      }
      part[t] = p;
    }
    const float bs = cta_sum_fixed(part);
    const float y = bs - comp;
    const float t2 = acc + y;
    comp = (t2 - acc) - y;
    acc = t2;
  }
  if (px_out) *px_out = cta_sum_fixed(pxp);
  return acc;
}

inline float fold_leaves(const float* leaf, int G) {
  float s[64];
  for (int i = 0; i < G; ++i) s[i] = leaf[i];
  for (int n = G; n > 1; n >>= 1)
    for (int i = 0; i < n / 2; ++i) s[i] = s[2 * i] + s[2 * i + 1];
  return s[0];
}

template <typename T>
void logprob_fused(const T* logits, long long ldl, int rows, int V, int G, const long long* targets, float* logprob,
                   float* lse, float* entropy) {
  const int leaf_len = V / G;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const T* x = logits + r * ldl;
    const float m = row_max(x, V);
    float leaf[64], leafpx[64];
    for (int g = 0; g < G; ++g) leaf[g] = leaf_sum(x, g * leaf_len, leaf_len, m, entropy ? &leafpx[g] : nullptr);
    const float S = fold_leaves(leaf, G);
    const float logS = logf(S);
    if (lse) lse[r] = m + logS;
    if (logprob) {
      const long long t = targets ? targets[r] : -1;
      logprob[r] = (t >= 0 && t < V) ? (ld(x, t) - m) - logS : 0.f;
    }
    if (entropy) {
      float px = 0.f;
      for (int i = 0; i < G; ++i) px += leafpx[i];
      entropy[r] = (m + logS) - px / S;
    }
  }
}

template <typename T>
void logprob_rowmax(const T* logits, long long ldl, int rows, int ncols, float* out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) out[r] = row_max(logits + r * ldl, ncols);
}

template <typename T>
void logprob_leafsum(const T* logits, long long ldl, int rows, int ncols, int local_leaves, int G, int leaf_base,
                     const float* rmax, float* leaf_sums, float* leaf_px) {
  const int leaf_len = ncols / local_leaves;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
    for (int lf = 0; lf < local_leaves; ++lf) {
      float px;
      leaf_sums[static_cast<long long>(r) * G + leaf_base + lf] =
          leaf_sum(logits + r * ldl, lf * leaf_len, leaf_len, rmax[r], leaf_px ? &px : nullptr);
      if (leaf_px) leaf_px[static_cast<long long>(r) * G + leaf_base + lf] = px;
    }
}

// ------------------------------------------------------------------ attention (blockwise, same state updates)
struct WorkItem {
  int q_start, q_len, q_pos0, kv_len, bt_row, kv_start, pad0, pad1;
};

template <typename T>
void attention_fwd(const T* q, const T* k, const T* v, const WorkItem* items, const int* block_table, T* out,
                   float* lse_out, int num_items, int Hq, int Hkv, int D, int bt_stride, float scale) {
  const int G = Hq / Hkv, TQ = 128 / G;
  const float scale_log2 = scale * 1.4426950408889634f;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int itx = 0; itx < num_items; ++itx)
    for (int kvh = 0; kvh < Hkv; ++kvh) {
      const WorkItem it = items[itx];
      const int q_valid = std::min(it.q_len, TQ);
      const int kv_hi = std::min(it.q_pos0 + q_valid, it.kv_len);
      const int nb = (kv_hi + 127) / 128;
      std::vector<float> o(D), ob(D), s(128), p(128);
      for (int tok = 0; tok < q_valid; ++tok)
        for (int g = 0; g < G; ++g) {
          const int hq = kvh * G + g;
          const int q_pos = it.q_pos0 + tok;
          const T* qr = q + (static_cast<long long>(it.q_start + tok) * Hq + hq) * D;
          float m = -INFINITY, l = 0.f;
          std::fill(o.begin(), o.end(), 0.f);
          for (int j = 0; j < nb; ++j) {
            const long long row0 = it.bt_row >= 0
                                       ? static_cast<long long>(block_table[static_cast<long long>(it.bt_row) * bt_stride + j]) * 128
                                       : static_cast<long long>(it.kv_start) + j * 128;
            const int lim = std::min(q_pos - j * 128 + 1, it.kv_len - j * 128);
            float mb = -INFINITY;
            for (int c = 0; c < 128 && c < lim; ++c) {
              const T* kr = k + ((row0 + c) * Hkv + kvh) * D;
              float acc = 0.f;
              for (int d = 0; d < D; ++d) acc = acc + ld(qr, d) * ld(kr, d);
              s[c] = acc * scale_log2;
              mb = fmaxf(mb, s[c]);
            }
            const float m_new = fmaxf(m, mb);
            // lazy exponent reference: m only moves when the maximum grew by more than 8 (log2 units)
            float alpha = 1.f;
            if (m_new - m > 8.0f) {
              alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
              m = m_new;
            }
            if (alpha != 1.f) {
              for (int d = 0; d < D; ++d) o[d] = o[d] * alpha;
              l = l * alpha;
            }
            for (int c = 0; c < 128 && c < lim; ++c) {
              const float pv = exp2f(s[c] - m);
              l = l + pv;
              const float pr = rnd<T>(pv);
              const T* vr = v + ((row0 + c) * Hkv + kvh) * D;
              for (int d = 0; d < D; ++d) o[d] = o[d] + pr * ld(vr, d);
            }
          }
          const float inv = 1.0f / l;
          const long long orow = static_cast<long long>(it.q_start + tok) * Hq + hq;
          for (int d = 0; d < D; ++d) st(out, orow * D + d, o[d] * inv);
          if (lse_out) lse_out[orow] = (m + log2f(l)) * 0.6931471805599453f;
        }
    }
}

// ------------------------------------------------------------------ fixed-order sum
template <typename T, bool SQUARE>
float reduce_sum(const T* in, long long n) {
  const long long np = (n + 4095) / 4096;
  std::vector<float> partials(np);
#pragma omp parallel for schedule(static)
  for (long long b = 0; b < np; ++b) {
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float acc = 0.f;
      for (int j = 0; j < 16; ++j) {
        const long long i = b * 4096 + t * 16 + j;
        if (i < n) {
          const float x = ld(in, i);
          acc = acc + (SQUARE ? x * x : x);
        }
      }
      part[t] = acc;
    }
    partials[b] = cta_sum_fixed(part);
  }
  float part[256];
  for (int t = 0; t < 256; ++t) {
    float acc = 0.f;
    for (long long i = t; i < np; i += 256) acc = acc + partials[i];
    part[t] = acc;
  }
  return cta_sum_fixed(part);
}

}  // namespace

#define DISPATCH(dt, ...)        \
  if ((dt) == 0) {               \
    using T = uint16_t;          \
    __VA_ARGS__;                 \
  } else {                       \
    using T = float;             \
    __VA_ARGS__;                 \
  }

IXC_API int ixc_version() { return 1; }

IXC_API void ixc_gemm_nt(const void* x, const void* w, void* out, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int in_dtype, int out_f32) {
  if (in_dtype == 0) {
    if (out_f32) gemm_nt(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(w), static_cast<float*>(out), M, N, K, lda, ldb, ldc);
    else gemm_nt(static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(w), static_cast<uint16_t*>(out), M, N, K, lda, ldb, ldc);
  } else {
    gemm_nt(static_cast<const float*>(x), static_cast<const float*>(w), static_cast<float*>(out), M, N, K, lda, ldb, ldc);
  }
}

IXC_API void ixc_leaftree_gemm(const void* x, const void* w, void* out, int M, int N, int Kloc, int nleaves,
                               int round_leaf, long long lda, long long ldb, long long ldc, int in_dtype) {
  DISPATCH(in_dtype, leaftree_gemm(static_cast<const T*>(x), static_cast<const T*>(w), static_cast<float*>(out), M, N,
                                   Kloc, nleaves, round_leaf, lda, ldb, ldc));
}

IXC_API void ixc_rmsnorm(const void* x, const void* res, const void* w, void* y, void* res_out, void* rstd_out, int rows,
                         int N, float eps, int zero_centered, long long ldx, long long ldy, int dtype) {
  DISPATCH(dtype, rmsnorm(static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(w),
                          static_cast<T*>(y), static_cast<T*>(res_out), static_cast<float*>(rstd_out), rows, N, eps,
                          zero_centered, ldx, ldy));
}

IXC_API void ixc_qk_norm_rope(const void* qkv, long long ldqkv, const void* positions, const void* slots,
                              const void* cos_tab, const void* sin_tab, const void* qw, const void* kw, void* q_out,
                              void* k_out, void* v_out, int Tn, int Hq, int Hkv, int D, int rot_dim, float eps,
                              int qk_norm, int zero_centered, int q_gate, int dtype) {
  DISPATCH(dtype, qk_norm_rope(static_cast<const T*>(qkv), ldqkv, static_cast<const int*>(positions),
                               static_cast<const long long*>(slots), static_cast<const float*>(cos_tab),
                               static_cast<const float*>(sin_tab), static_cast<const T*>(qw),
                               static_cast<const T*>(kw), static_cast<T*>(q_out), static_cast<T*>(k_out),
                               static_cast<T*>(v_out), Tn, Hq, Hkv, D, rot_dim, eps, qk_norm, zero_centered, q_gate));
}

IXC_API void ixc_swiglu(const void* in, void* out, long long Tn, int F, long long ld_in, int dtype) {
  DISPATCH(dtype, swiglu(static_cast<const T*>(in), static_cast<T*>(out), Tn, F, ld_in));
}

IXC_API void ixc_sigmoid_gate(const void* a, const void* qkv, long long ldqkv, void* out, long long Tn, int Hq, int Hkv,
                              int D, int dtype) {
  DISPATCH(dtype, sigmoid_gate(static_cast<const T*>(a), static_cast<const T*>(qkv), ldqkv, static_cast<T*>(out), Tn, Hq, Hkv, D));
}

IXC_API void ixc_gated_outnorm(const void* o, const void* z, const void* w, void* out, long long rows, int D, float eps,
                               int zero_centered, int dtype) {
  DISPATCH(dtype, gated_outnorm(static_cast<const T*>(o), static_cast<const T*>(z), static_cast<const T*>(w),
                                static_cast<T*>(out), rows, D, eps, zero_centered));
}

IXC_API void ixc_logprob_fused(const void* logits, long long ldl, int rows, int V, int G, const void* targets,
                               void* logprob, void* lse, void* entropy, int dtype) {
  DISPATCH(dtype, logprob_fused(static_cast<const T*>(logits), ldl, rows, V, G, static_cast<const long long*>(targets),
                                static_cast<float*>(logprob), static_cast<float*>(lse), static_cast<float*>(entropy)));
}

IXC_API void ixc_logprob_rowmax(const void* logits, long long ldl, int rows, int ncols, void* out, int dtype) {
  DISPATCH(dtype, logprob_rowmax(static_cast<const T*>(logits), ldl, rows, ncols, static_cast<float*>(out)));
}

IXC_API void ixc_logprob_leafsum(const void* logits, long long ldl, int rows, int ncols, int local_leaves, int G,
                                 int leaf_base, const void* rmax, void* leaf_sums, void* leaf_px, int dtype) {
  DISPATCH(dtype, logprob_leafsum(static_cast<const T*>(logits), ldl, rows, ncols, local_leaves, G, leaf_base,
                                  static_cast<const float*>(rmax), static_cast<float*>(leaf_sums),
                                  static_cast<float*>(leaf_px)));
}

IXC_API void ixc_logprob_finalize(const void* leaf_sums, const void* leaf_px, const void* rmax, const void* target_logit,
                                  const void* targets, void* logprob, void* lse, void* entropy, int rows, int G) {
  const float* ls = static_cast<const float*>(leaf_sums);
  const float* lpx = static_cast<const float*>(leaf_px);
  const float* mx = static_cast<const float*>(rmax);
  const float* tl = static_cast<const float*>(target_logit);
  const long long* tg = static_cast<const long long*>(targets);
  for (int r = 0; r < rows; ++r) {
    const float S = fold_leaves(ls + static_cast<long long>(r) * G, G);
    const float logS = logf(S);
    if (lse) static_cast<float*>(lse)[r] = mx[r] + logS;
    const bool valid = tg == nullptr || tg[r] >= 0;
    if (logprob) static_cast<float*>(logprob)[r] = valid ? (tl[r] - mx[r]) - logS : 0.f;
    if (entropy && lpx) {
      float px = 0.f;
      for (int i = 0; i < G; ++i) px += lpx[static_cast<long long>(r) * G + i];
      static_cast<float*>(entropy)[r] = (mx[r] + logS) - px / S;
    }
  }
}

IXC_API void ixc_attention_fwd(const void* q, const void* k, const void* v, const void* items, const void* block_table,
                               void* out, void* lse, int num_items, int Hq, int Hkv, int D, int bt_stride, float scale,
                               int dtype) {
  DISPATCH(dtype, attention_fwd(static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
                                static_cast<const WorkItem*>(items), static_cast<const int*>(block_table),
                                static_cast<T*>(out), static_cast<float*>(lse), num_items, Hq, Hkv, D, bt_stride, scale));
}

IXC_API float ixc_reduce_sum(const void* in, long long n, int dtype, int square) {
  if (dtype == 0) return square ? reduce_sum<uint16_t, true>(static_cast<const uint16_t*>(in), n)
                                : reduce_sum<uint16_t, false>(static_cast<const uint16_t*>(in), n);
  return square ? reduce_sum<float, true>(static_cast<const float*>(in), n)
                : reduce_sum<float, false>(static_cast<const float*>(in), n);
}

// ------------------------------------------------------------------ MoE router (same order as csrc/moe.cu)
IXC_API void ixc_router_topk(const void* logits_, long long ldl, const void* bias_, int Tn, int E, int K, int sigmoid_bias,
                             int norm_topk, void* idx_out_, void* w_out_, void* probs_out_) {
  const float* logits = static_cast<const float*>(logits_);
  const float* bias = static_cast<const float*>(bias_);
  int* idx_out = static_cast<int*>(idx_out_);
  float* w_out = static_cast<float*>(w_out_);
  float* probs_out = static_cast<float*>(probs_out_);
#pragma omp parallel for schedule(static)
  for (int t = 0; t < Tn; ++t) {
    const float* x = logits + t * ldl;
    std::vector<float> score(E), gate(E);
    if (!sigmoid_bias) {
      float m = -INFINITY;
      for (int e = 0; e < E; ++e) m = fmaxf(m, x[e]);
      float lane[32];
      for (int l = 0; l < 32; ++l) {
        float part = 0.f;
        for (int e = l; e < E; e += 32) {
          gate[e] = expf(x[e] - m);
          part = part + gate[e];
        }
        lane[l] = part;
      }
      const float S = butterfly32(lane);
      for (int e = 0; e < E; ++e) {
        gate[e] = gate[e] / S;
        score[e] = gate[e];
      }
    } else {
      for (int e = 0; e < E; ++e) {
        gate[e] = 1.0f / (1.0f + expf(-x[e]));
        score[e] = bias ? gate[e] + bias[e] : gate[e];
      }
    }
    if (probs_out)
      for (int e = 0; e < E; ++e) probs_out[static_cast<long long>(t) * E + e] = gate[e];
    float wsum = 0.f;
    for (int r = 0; r < K; ++r) {
      int bi = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e)
        if (score[e] > bv) {
          bv = score[e];
          bi = e;
        }
      idx_out[static_cast<long long>(t) * K + r] = bi;
      w_out[static_cast<long long>(t) * K + r] = gate[bi];
      wsum = wsum + gate[bi];
      score[bi] = -INFINITY;
    }
    if (norm_topk)
      for (int r = 0; r < K; ++r) w_out[static_cast<long long>(t) * K + r] = w_out[static_cast<long long>(t) * K + r] / wsum;
  }
}

// ------------------------------------------------------------------ GatedDeltaNet (same order as csrc/gdn.cu)
namespace {
struct ScanChunk {
  int tok_start, n_tok, pos0, pad;
  long long row_in, row_out;
};

template <typename T>
void gdn_conv(const T* x, long long ldx, const T* w, const int* tok_back, const long long* state_row, const T* conv_state,
              T* out, long long Tn, int C, int W) {
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < Tn; ++t)
    for (int c = 0; c < C; ++c) {
      const int back = tok_back[t];
      const long long srow = state_row ? state_row[t] : -1;
      float acc = 0.f;
      for (int j = 0; j < W; ++j) {
        const int d = W - 1 - j;
        float xv;
        if (d <= back) xv = ld(x, (t - d) * ldx + c);
        else if (srow >= 0) xv = ld(conv_state, (srow * C + c) * (W - 1) + (W - 1) - (d - back));
        else xv = 0.f;
        acc = fmaf(ld(w, static_cast<long long>(c) * W + j), xv, acc);
      }
      st(out, t * C + c, acc / (1.0f + expf(-acc)));
    }
}

template <typename T>
void gdn_conv_state(const T* x, long long ldx, const ScanChunk* chunks, T* conv_state, int n_chunks, int C, int W) {
  for (int ch = 0; ch < n_chunks; ++ch) {
    const ScanChunk sc = chunks[ch];
    if (sc.row_out < 0) continue;
    for (int c = 0; c < C; ++c) {
      float nv[3];
      for (int j = 0; j < W - 1; ++j) {
        const int d = W - 1 - j;
        if (d <= sc.n_tok) nv[j] = ld(x, static_cast<long long>(sc.tok_start + sc.n_tok - d) * ldx + c);
        else if (sc.row_in >= 0) nv[j] = ld(conv_state, (sc.row_in * C + c) * (W - 1) + j + sc.n_tok);
        else nv[j] = 0.f;
      }
      for (int j = 0; j < W - 1; ++j) st(conv_state, (sc.row_out * C + c) * (W - 1) + j, nv[j]);
    }
  }
}

template <typename T>
void gdn_gate(const T* a, const T* b, long long ldab, const T* A_log, const T* dt_bias, float* g, float* beta, long long Tn, int H) {
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < Tn; ++t)
    for (int h = 0; h < H; ++h) {
      const float x = ld(a, t * ldab + h) + ld(dt_bias, h);
      const float sp = x > 20.f ? x : log1pf(expf(x));
      g[t * H + h] = -expf(ld(A_log, h)) * sp;
      beta[t * H + h] = 1.0f / (1.0f + expf(-ld(b, t * ldab + h)));
    }
}

template <typename T>
void gdn_l2norm(const T* in, long long ldin, T* out_q, T* out_k, long long Tn, int Hk, int D, float eps, float q_scale) {
#pragma omp parallel for schedule(static)
  for (long long wid = 0; wid < Tn * 2 * Hk; ++wid) {
    const long long t = wid / (2 * Hk);
    const int hh = static_cast<int>(wid % (2 * Hk));
    const bool is_k = hh >= Hk;
    const int h = is_k ? hh - Hk : hh;
    const T* src = in + t * ldin + (is_k ? static_cast<long long>(Hk) * D : 0) + static_cast<long long>(h) * D;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
      float ss = 0.f;
      for (int v = l; v < D / 8; v += 32)
        for (int j = 0; j < 8; ++j) {
          const float f = ld(src, v * 8 + j);
          ss = ss + f * f;
        }
      lane[l] = ss;
    }
    const float rstd = 1.0f / sqrtf(butterfly32(lane) + eps);
    T* dst = (is_k ? out_k : out_q) + (t * Hk + h) * D;
    for (int i = 0; i < D; ++i) {
      float n = rnd<T>(ld(src, i) * rstd);
      if (!is_k) n = rnd<T>(n * q_scale);
      st(dst, i, n);
    }
  }
}

template <typename T>
void gdn_scan(const T* q, const T* k, const T* v, const float* g, const float* beta, const ScanChunk* chunks, float* state,
              T* out, int n_chunks, int Hk, int Hv, int DK, int DV, int snapshot_every) {
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int ch = 0; ch < n_chunks; ++ch)
    for (int hv = 0; hv < Hv; ++hv) {
      const ScanChunk sc = chunks[ch];
      const int hk = hv / (Hv / Hk);
      std::vector<float> S(static_cast<size_t>(DV) * DK, 0.f);
      if (sc.row_in >= 0) memcpy(S.data(), state + (sc.row_in * Hv + hv) * DV * DK, sizeof(float) * DV * DK);
      for (int tt = 0; tt < sc.n_tok; ++tt) {
        const long long t = sc.tok_start + tt;
        const float decay = expf(g[t * Hv + hv]), bt = beta[t * Hv + hv];
        const T* kr = k + (t * Hk + hk) * DK;
        const T* qr = q + (t * Hk + hk) * DK;
        for (int j = 0; j < DV; ++j) {
          float* Sj = &S[static_cast<size_t>(j) * DK];
          float kv = 0.f;
          for (int i = 0; i < DK; ++i) {
            Sj[i] = Sj[i] * decay;
            kv = fmaf(Sj[i], ld(kr, i), kv);
          }
          const float d = (ld(v, (t * Hv + hv) * DV + j) - kv) * bt;
          float o = 0.f;
          for (int i = 0; i < DK; ++i) {
            Sj[i] = fmaf(d, ld(kr, i), Sj[i]);
            o = fmaf(Sj[i], ld(qr, i), o);
          }
          st(out, (t * Hv + hv) * DV + j, o);
          if (snapshot_every > 0 && ((sc.pos0 + tt + 1) % snapshot_every) == 0)
            for (int i = 0; i < DK; ++i) Sj[i] = round_bf(Sj[i]);
        }
      }
      if (sc.row_out >= 0) memcpy(state + (sc.row_out * Hv + hv) * DV * DK, S.data(), sizeof(float) * DV * DK);
    }
}
}  // namespace

IXC_API void ixc_gdn_conv(const void* x, long long ldx, const void* w, const void* tok_back, const void* state_row,
                          const void* conv_state, void* out, long long Tn, int C, int W, int dtype) {
  DISPATCH(dtype, gdn_conv(static_cast<const T*>(x), ldx, static_cast<const T*>(w), static_cast<const int*>(tok_back),
                           static_cast<const long long*>(state_row), static_cast<const T*>(conv_state), static_cast<T*>(out), Tn, C, W));
}
IXC_API void ixc_gdn_conv_state(const void* x, long long ldx, const void* chunks, void* conv_state, int n_chunks, int C, int W, int dtype) {
  DISPATCH(dtype, gdn_conv_state(static_cast<const T*>(x), ldx, static_cast<const ScanChunk*>(chunks), static_cast<T*>(conv_state), n_chunks, C, W));
}
IXC_API void ixc_gdn_gate(const void* a, const void* b, long long ldab, const void* A_log, const void* dt_bias, void* g, void* beta,
                          long long Tn, int H, int dtype) {
  DISPATCH(dtype, gdn_gate(static_cast<const T*>(a), static_cast<const T*>(b), ldab, static_cast<const T*>(A_log),
                           static_cast<const T*>(dt_bias), static_cast<float*>(g), static_cast<float*>(beta), Tn, H));
}
IXC_API void ixc_gdn_l2norm(const void* in, long long ldin, void* out_q, void* out_k, long long Tn, int Hk, int D, float eps,
                            float q_scale, int dtype) {
  DISPATCH(dtype, gdn_l2norm(static_cast<const T*>(in), ldin, static_cast<T*>(out_q), static_cast<T*>(out_k), Tn, Hk, D, eps, q_scale));
}
IXC_API void ixc_gdn_scan(const void* q, const void* k, const void* v, const void* g, const void* beta, const void* chunks,
                          void* state, void* out, int n_chunks, int Hk, int Hv, int DK, int DV, int snapshot_every, int dtype) {
  DISPATCH(dtype, gdn_scan(static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<const float*>(g),
                           static_cast<const float*>(beta), static_cast<const ScanChunk*>(chunks), static_cast<float*>(state),
                           static_cast<T*>(out), n_chunks, Hk, Hv, DK, DV, snapshot_every));
}
