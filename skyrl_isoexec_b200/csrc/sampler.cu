// Fused categorical sampling by the Gumbel-max trick: token = argmax_v (logit_v / T + G_v), G_v ~ Gumbel(0,1).
// One pass over the bf16 logits; the noise comes from a counter-based generator (Philox-4x32-10, a public
// algorithm: Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed by (seed, call counter)
// and indexed by (row, column), so a draw does not depend on how the work is split over threads or on the
// batch composition of other rows' columns. Ties go to the lower index. T == 0 means greedy (no noise).
//
// The reference samples inside vLLM (Sampler patched to raw logprobs, ISO/runtimes/vllm/vllm_patches.py:236-307);
// here the chosen token's log-probability is then computed by the same row-invariant kernel the trainer uses.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

struct alignas(16) BF8 {
  __nv_bfloat16 v[8];
};

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                              uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0, c1 = n1, c2 = n2, c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0, out[1] = c1, out[2] = c2, out[3] = c3;
}

__device__ __forceinline__ float gumbel_from_bits(uint32_t x) {
  const float u = (static_cast<float>(x >> 8) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1), 24 bits
  return -logf(-logf(u));
}

constexpr int kSplits = 8;

// grid (rows, kSplits), 256 threads. partial_val/idx: [rows, kSplits]
__global__ void __launch_bounds__(256)
gumbel_argmax_partial_kernel(const __nv_bfloat16* __restrict__ logits, long long ldl, int V, const float* __restrict__ inv_temp,
                             uint32_t seed_lo, uint32_t seed_hi, uint32_t call, float* __restrict__ partial_val,
                             int* __restrict__ partial_idx) {
  const int row = blockIdx.x, split = blockIdx.y;
  const float it = inv_temp[row];                 // 0: greedy
  const bool noisy = it != 0.f;
  const float scale = noisy ? it : 1.0f;
  const int nvec = V >> 3;
  const int per = (nvec + kSplits - 1) / kSplits;
  const int v0 = split * per, v1 = min(nvec, v0 + per);
  const BF8* src = reinterpret_cast<const BF8*>(logits + static_cast<size_t>(row) * ldl);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int v = v0 + threadIdx.x; v < v1; v += 256) {
    const BF8 a = src[v];
    uint32_t r0[4], r1[4];
    if (noisy) {
      philox4x32_10(static_cast<uint32_t>(2 * v), static_cast<uint32_t>(row), call, 0u, seed_lo, seed_hi, r0);
      philox4x32_10(static_cast<uint32_t>(2 * v + 1), static_cast<uint32_t>(row), call, 0u, seed_lo, seed_hi, r1);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float x = bf2f(a.v[j]) * scale;
      if (noisy) x += gumbel_from_bits(j < 4 ? r0[j] : r1[j - 4]);
      const int i = v * 8 + j;
      if (x > best) best = x, best_i = i;       // ascending i within a thread: strict > keeps the lower index
    }
  }
  // tail columns (V not a multiple of 8) go to the last split's thread 0
  if (split == kSplits - 1 && threadIdx.x == 0) {
    for (int i = nvec * 8; i < V; ++i) {
      float x = bf2f(logits[static_cast<size_t>(row) * ldl + i]) * scale;
      if (noisy) {
        uint32_t r[4];
        philox4x32_10(static_cast<uint32_t>(i >> 2), static_cast<uint32_t>(row), call, 1u, seed_lo, seed_hi, r);
        x += gumbel_from_bits(r[i & 3]);
      }
      if (x > best || (x == best && i < best_i)) best = x, best_i = i;
    }
  }
  // block argmax, lower index on ties
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
  }
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  if ((threadIdx.x & 31) == 0) s_v[threadIdx.x >> 5] = best, s_i[threadIdx.x >> 5] = best_i;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (s_v[w] > best || (s_v[w] == best && s_i[w] < best_i)) best = s_v[w], best_i = s_i[w];
    partial_val[row * kSplits + split] = best;
    partial_idx[row * kSplits + split] = best_i;
  }
}

__global__ void gumbel_argmax_final_kernel(const float* __restrict__ partial_val, const int* __restrict__ partial_idx, int rows,
                                           long long* __restrict__ tokens) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float best = partial_val[row * kSplits];
  int best_i = partial_idx[row * kSplits];
  for (int s = 1; s < kSplits; ++s) {
    const float v = partial_val[row * kSplits + s];
    const int i = partial_idx[row * kSplits + s];
    if (v > best || (v == best && i < best_i)) best = v, best_i = i;
  }
  tokens[row] = best_i;
}

}  // namespace

IX_API int ix_sampler_scratch_elems(int rows) { return rows * kSplits; }

// logits bf16 [rows, ldl]; inv_temp fp32 [rows] (1/T, 0 for greedy); scratch_val fp32 / scratch_idx int32 of
// ix_sampler_scratch_elems(rows) elements; tokens int64 [rows].
IX_API int ix_sample_gumbel(const void* logits, long long ldl, int rows, int V, const void* inv_temp, unsigned long long seed,
                            unsigned call, void* scratch_val, void* scratch_idx, void* tokens, void* stream) {
  if (rows <= 0) return 0;
  if (ldl & 7) return ixh::fail(ixh::IX_EARG, "sampler: ldl must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(rows, kSplits);
  gumbel_argmax_partial_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ldl, V, static_cast<const float*>(inv_temp),
                                                    static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), call,
                                                    static_cast<float*>(scratch_val), static_cast<int*>(scratch_idx));
  IX_CUDA(cudaGetLastError());
  gumbel_argmax_final_kernel<<<(rows + 127) / 128, 128, 0, s>>>(static_cast<const float*>(scratch_val), static_cast<const int*>(scratch_idx),
                                                               rows, static_cast<long long*>(tokens));
  IX_CUDA(cudaGetLastError());
  return 0;
}
