// Row-count- and TP-invariant token log-probabilities ("rowinv"), restated for sm_100a.
//
// Arithmetic (same recipe as the reference's ISO/ops/logprobs/rowinv.py:136-245, here as
// one CUDA implementation shared by trainer and engine):
//   m   = max over the full vocabulary row (exact, order-free)
//   the vocabulary is cut into G equal leaves (G a power of two >= the largest TP degree);
//   leaf g is summed in blocks of 4096 columns: block_sum = sum exp(x - m) with a fixed
//   in-block order (256 threads x 16 consecutive-vector elements, xor butterfly, then the 8 warp
//   partials left to right), folded into the leaf by a Kahan update
//       y = block_sum - comp; t = acc + y; comp = (t - acc) - y; acc = t
//   the G leaf sums are folded by log2(G) rounds of adjacent-pair adds (lo + hi)
//   logprob = (x_t - m) - log(S);  lse = m + log(S)
// A TP rank owns G/TP whole leaves, so sharding the vocabulary never changes a bit: the
// three stages below are also exported separately (row max / leaf sums / finalize) and the
// fused single-launch kernel calls the same device functions.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kLpThreads = 256;
constexpr int kLpBlock = 4096;  // columns per Kahan block: 256 threads x 16

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) {
  return p[i];
}

// CTA-wide max; result broadcast to all threads.
__device__ __forceinline__ float cta_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < kLpThreads / 32; ++i) r = fmaxf(r, red[i]);
  return r;
}
// CTA-wide sum in a fixed order: butterfly inside each warp, then warp partials 0..7 left to right.
__device__ __forceinline__ float cta_sum_fixed(float v, float* red) {
  v = warp_sum_butterfly(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < kLpThreads / 32; ++i) r = __fadd_rn(r, red[i]);
  return r;
}

template <typename T>
__device__ __forceinline__ float row_max_dev(const T* row, int n, float* red) {
  float m = -INFINITY;
  for (int i = threadIdx.x; i < n; i += kLpThreads) m = fmaxf(m, ld_logit(row, i));
  return cta_max(m, red);
}

// Kahan-compensated sum of exp(x - m) over columns [lo, lo+len) of `row`.
// Also accumulates sum exp(x-m)*x (plain fp32) for the entropy metric when want_px.
template <typename T>
__device__ __forceinline__ float leaf_sum_dev(const T* row, int lo, int len, float m, float* red, float* px_out) {
  float acc = 0.f, comp = 0.f, px = 0.f;
  for (int off = 0; off < len; off += kLpBlock) {
    float part = 0.f;
    const int base = off + threadIdx.x * 16;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int c = base + j;
      if (c < len) {
        const float x = ld_logit(row, lo + c);
        const float e = expf(__fsub_rn(x, m));
        part = __fadd_rn(part, e);
        px = __fadd_rn(px, __fmul_rn(e, x));
      }
    }
    const float bs = cta_sum_fixed(part, red);
    const float y = __fsub_rn(bs, comp);
    const float t = __fadd_rn(acc, y);
    comp = __fsub_rn(__fsub_rn(t, acc), y);
    acc = t;
  }
  if (px_out) *px_out = cta_sum_fixed(px, red);
  return acc;
}

// Fold G leaf sums by adjacent pairs (round r combines 2i and 2i+1), G power of two <= 64.
__device__ __forceinline__ float fold_leaves(const float* leaf, int G) {
  float s[64];
  for (int i = 0; i < G; ++i) s[i] = leaf[i];
  for (int n = G; n > 1; n >>= 1)
    for (int i = 0; i < n / 2; ++i) s[i] = __fadd_rn(s[2 * i], s[2 * i + 1]);
  return s[0];
}

// ---------------------------------------------------------------- staged kernels (TP path)
template <typename T>
__global__ void __launch_bounds__(kLpThreads)
rowmax_kernel(const T* __restrict__ logits, long long ld, int ncols, float* __restrict__ out) {
  __shared__ float red[kLpThreads / 32];
  const float m = row_max_dev(logits + static_cast<size_t>(blockIdx.x) * ld, ncols, red);
  if (threadIdx.x == 0) out[blockIdx.x] = m;
}

// grid (rows, local_leaves). leaf_sums[row, leaf_base + blockIdx.y] over G total leaves.
template <typename T>
__global__ void __launch_bounds__(kLpThreads)
leafsum_kernel(const T* __restrict__ logits, long long ld, int leaf_len, const float* __restrict__ row_max,
               float* __restrict__ leaf_sums, float* __restrict__ leaf_px, int G, int leaf_base) {
  __shared__ float red[kLpThreads / 32];
  const int row = blockIdx.x, lf = blockIdx.y;
  float px;
  const float s = leaf_sum_dev(logits + static_cast<size_t>(row) * ld, lf * leaf_len, leaf_len, row_max[row], red,
                               leaf_px ? &px : nullptr);
  if (threadIdx.x == 0) {
    leaf_sums[static_cast<size_t>(row) * G + leaf_base + lf] = s;
    if (leaf_px) leaf_px[static_cast<size_t>(row) * G + leaf_base + lf] = px;
  }
}

// target_logit[row] must hold x_t (gathered by the owning rank; others contribute 0 and are summed).
__global__ void finalize_kernel(const float* __restrict__ leaf_sums, const float* __restrict__ leaf_px,
                                const float* __restrict__ row_max, const float* __restrict__ target_logit,
                                const long long* __restrict__ targets, float* __restrict__ logprob,
                                float* __restrict__ lse, float* __restrict__ entropy, int rows, int G) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float S = fold_leaves(leaf_sums + static_cast<size_t>(r) * G, G);
  const float logS = logf(S);
  const float m = row_max[r];
  if (lse) lse[r] = __fadd_rn(m, logS);
  const bool valid = targets == nullptr || targets[r] >= 0;
  if (logprob) logprob[r] = valid ? __fsub_rn(__fsub_rn(target_logit[r], m), logS) : 0.f;
  if (entropy && leaf_px) {
    float px = 0.f;
    for (int i = 0; i < G; ++i) px += leaf_px[static_cast<size_t>(r) * G + i];
    entropy[r] = (m + logS) - px / S;
  }
}

// gather x[row, target - col_base] if the target falls in this shard, else 0
template <typename T>
__global__ void gather_target_kernel(const T* __restrict__ logits, long long ld, int ncols, int col_base,
                                     const long long* __restrict__ targets, float* __restrict__ out, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const long long t = targets[r] - col_base;
  out[r] = (t >= 0 && t < ncols) ? ld_logit(logits + static_cast<size_t>(r) * ld, t) : 0.f;
}

// ---------------------------------------------------------------- fused single-launch kernel (TP = 1)
template <typename T>
__global__ void __launch_bounds__(kLpThreads)
logprob_fused_kernel(const T* __restrict__ logits, long long ld, int V, int G, const long long* __restrict__ targets,
                     float* __restrict__ logprob, float* __restrict__ lse, float* __restrict__ entropy) {
  __shared__ float red[kLpThreads / 32];
  __shared__ float leaf[64];
  __shared__ float leafpx[64];
  const int row = blockIdx.x;
  const T* x = logits + static_cast<size_t>(row) * ld;
  const float m = row_max_dev(x, V, red);
  const int leaf_len = V / G;
  for (int g = 0; g < G; ++g) {
    float px;
    const float s = leaf_sum_dev(x, g * leaf_len, leaf_len, m, red, entropy ? &px : nullptr);
    if (threadIdx.x == 0) {
      leaf[g] = s;
      if (entropy) leafpx[g] = px;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const float S = fold_leaves(leaf, G);
    const float logS = logf(S);
    if (lse) lse[row] = __fadd_rn(m, logS);
    if (logprob) {
      const long long t = targets ? targets[row] : -1;
      logprob[row] = (t >= 0 && t < V) ? __fsub_rn(__fsub_rn(ld_logit(x, t), m), logS) : 0.f;
    }
    if (entropy) {
      float px = 0.f;
      for (int i = 0; i < G; ++i) px += leafpx[i];
      entropy[row] = (m + logS) - px / S;
    }
  }
}

// ---------------------------------------------------------------- backward
// dlogits[r, c] = g_lp[r] * (1[c == t_r] - p) + g_ent[r] * dH/dx, p = exp(x - lse)
// (dH/dx_c = -p_c * (x_c - lse + H)). Written in the logits dtype; may alias the logits buffer.
template <typename T>
__global__ void __launch_bounds__(256)
logprob_bwd_kernel(const T* logits, long long ld, int ncols, int col_base, const long long* __restrict__ targets,
                   const float* __restrict__ lse, const float* __restrict__ g_lp, const float* __restrict__ g_ent,
                   const float* __restrict__ entropy, T* dlogits, long long ld_out) {
  const int row = blockIdx.x;
  const float l = lse[row];
  const float g = g_lp ? g_lp[row] : 0.f;
  const float ge = g_ent ? g_ent[row] : 0.f;
  const float H = (g_ent && entropy) ? entropy[row] : 0.f;
  const long long t = targets[row] - col_base;
  const T* x = logits + static_cast<size_t>(row) * ld;
  T* d = dlogits + static_cast<size_t>(row) * ld_out;
  for (int c = threadIdx.x; c < ncols; c += 256) {
    const float xv = ld_logit(x, c);
    const float p = expf(xv - l);
    float gr = g * ((c == t ? 1.f : 0.f) - p);
    if (g_ent) gr += ge * (-p * (xv - l + H));
    if constexpr (sizeof(T) == 2) d[c] = __float2bfloat16_rn(gr);
    else d[c] = gr;
  }
}

}  // namespace

#define IX_DISPATCH_LOGIT(is_f32, ...)        \
  if (is_f32) {                               \
    using T = float;                          \
    __VA_ARGS__;                              \
  } else {                                    \
    using T = __nv_bfloat16;                  \
    __VA_ARGS__;                              \
  }

IX_API int ix_logprob_fused(const void* logits, long long ld, int rows, int V, int G, const void* targets,
                            void* logprob, void* lse, void* entropy, int is_f32, void* stream) {
  if (rows <= 0) return 0;
  if (G < 1 || G > 64 || (G & (G - 1)) || V % G) return ixh::fail(ixh::IX_EARG, "logprob: G=%d must be a power of two dividing V=%d", G, V);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  IX_DISPATCH_LOGIT(is_f32, (logprob_fused_kernel<T><<<rows, kLpThreads, 0, s>>>(
                                static_cast<const T*>(logits), ld, V, G, static_cast<const long long*>(targets),
                                static_cast<float*>(logprob), static_cast<float*>(lse), static_cast<float*>(entropy))));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_logprob_rowmax(const void* logits, long long ld, int rows, int ncols, void* out, int is_f32,
                             void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  IX_DISPATCH_LOGIT(is_f32, (rowmax_kernel<T><<<rows, kLpThreads, 0, s>>>(static_cast<const T*>(logits), ld, ncols,
                                                                          static_cast<float*>(out))));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_logprob_leafsum(const void* logits, long long ld, int rows, int ncols, int local_leaves, int G,
                              int leaf_base, const void* row_max, void* leaf_sums, void* leaf_px, int is_f32,
                              void* stream) {
  if (rows <= 0) return 0;
  if (local_leaves < 1 || ncols % local_leaves) return ixh::fail(ixh::IX_EARG, "leafsum: %d columns not divisible into %d leaves", ncols, local_leaves);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(rows, local_leaves);
  IX_DISPATCH_LOGIT(is_f32, (leafsum_kernel<T><<<grid, kLpThreads, 0, s>>>(
                                static_cast<const T*>(logits), ld, ncols / local_leaves,
                                static_cast<const float*>(row_max), static_cast<float*>(leaf_sums),
                                static_cast<float*>(leaf_px), G, leaf_base)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_logprob_gather_target(const void* logits, long long ld, int rows, int ncols, int col_base,
                                    const void* targets, void* out, int is_f32, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  IX_DISPATCH_LOGIT(is_f32, (gather_target_kernel<T><<<(rows + 127) / 128, 128, 0, s>>>(
                                static_cast<const T*>(logits), ld, ncols, col_base,
                                static_cast<const long long*>(targets), static_cast<float*>(out), rows)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_logprob_finalize(const void* leaf_sums, const void* leaf_px, const void* row_max,
                               const void* target_logit, const void* targets, void* logprob, void* lse,
                               void* entropy, int rows, int G, void* stream) {
  if (rows <= 0) return 0;
  if (G < 1 || G > 64 || (G & (G - 1))) return ixh::fail(ixh::IX_EARG, "finalize: bad G=%d", G);
  finalize_kernel<<<(rows + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(leaf_sums), static_cast<const float*>(leaf_px), static_cast<const float*>(row_max),
      static_cast<const float*>(target_logit), static_cast<const long long*>(targets),
      static_cast<float*>(logprob), static_cast<float*>(lse), static_cast<float*>(entropy), rows, G);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_logprob_bwd(const void* logits, long long ld, int rows, int ncols, int col_base, const void* targets,
                          const void* lse, const void* g_lp, const void* g_ent, const void* entropy, void* dlogits,
                          long long ld_out, int is_f32, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  IX_DISPATCH_LOGIT(is_f32, (logprob_bwd_kernel<T><<<rows, 256, 0, s>>>(
                                static_cast<const T*>(logits), ld, ncols, col_base,
                                static_cast<const long long*>(targets), static_cast<const float*>(lse),
                                static_cast<const float*>(g_lp), static_cast<const float*>(g_ent),
                                static_cast<const float*>(entropy), static_cast<T*>(dlogits), ld_out)));
  IX_CUDA(cudaGetLastError());
  return 0;
}
