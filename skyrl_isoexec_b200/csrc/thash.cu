// Row digests of a tensor for region tracing, all ladder levels in one pass over the data:
//
//     out[l][r] = sum_i  w(i) * (bits(x[r][i]) & ~((1 << k_l) - 1))   mod 2^64
//
// w(i) is the odd 64-bit splitmix weight of the element's index inside its row (generated in the kernel, no table), so
// the digest of a row does not depend on the order rows are visited in or on how the tensor is tiled; the sum wraps.
// The torch formulation widens every element to int64 and walks the tensor once per level (debug/thash.py); this
// reads the tensor once. (reference scheme: ISO/debug/thash.py:106-307)
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_util.h"

namespace {

constexpr int kLevels = 5;

__device__ __forceinline__ unsigned long long weight_of(unsigned long long i) {
  unsigned long long z = 0x9E3779B97F4A7C15ull * (i + 2ull);      // state of the (i+1)-th splitmix step started at the constant
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return (z ^ (z >> 31)) | 1ull;
}

template <typename T>
__global__ void __launch_bounds__(256)
row_digest_kernel(const T* __restrict__ x, long long rows, long long cols, const int* __restrict__ ks, unsigned long long* __restrict__ out) {
  // one warp per row, 8 rows per CTA
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  unsigned long long mask[kLevels], acc[kLevels];
#pragma unroll
  for (int l = 0; l < kLevels; ++l) {
    mask[l] = ~((1ull << ks[l]) - 1ull);
    acc[l] = 0;
  }
  const T* p = x + row * cols;
  for (long long i = lane; i < cols; i += 32) {
    const unsigned long long b = static_cast<unsigned long long>(p[i]);      // zero-extended bits of the element
    const unsigned long long w = weight_of(static_cast<unsigned long long>(i));
#pragma unroll
    for (int l = 0; l < kLevels; ++l) acc[l] += w * (b & mask[l]);
  }
#pragma unroll
  for (int l = 0; l < kLevels; ++l) {
    unsigned long long v = acc[l];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) out[l * rows + row] = v;
  }
}

}  // namespace

// x: [rows, cols] elements of elem_bytes (2, 4 or 8) each, contiguous; ks: 5 mantissa-bit counts (device ints);
// out: [5, rows] uint64 (device). Integer arithmetic only, so the result is exact and order-free.
IX_API int ix_row_digests(const void* x, long long rows, long long cols, int elem_bytes, const void* ks, void* out, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (rows > (1ll << 31) * 8) return ixh::fail(ixh::IX_EARG, "row_digests: too many rows (%lld)", rows);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  auto* o = static_cast<unsigned long long*>(out);
  const int* k = static_cast<const int*>(ks);
  if (elem_bytes == 2) row_digest_kernel<uint16_t><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), rows, cols, k, o);
  else if (elem_bytes == 4) row_digest_kernel<uint32_t><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(x), rows, cols, k, o);
  else if (elem_bytes == 8) row_digest_kernel<unsigned long long><<<grid, 256, 0, s>>>(static_cast<const unsigned long long*>(x), rows, cols, k, o);
  else return ixh::fail(ixh::IX_EARG, "row_digests: element size %d", elem_bytes);
  IX_CUDA(cudaGetLastError());
  return 0;
}
