// Routing mechanics of a mixture-of-experts layer as integer kernels, with no host round trip and no atomics
// (the reference builds the same tables with Triton kernels: ISO/ops/moe/moe_fused_permute.py:327-593,
// moe_blockmap_kernel.py:37, and orders the backward of the permutation without atomics,
// moe_ordered_dispatch.py:22-75).
//
// Input: idx[T, k] (expert of each (token, slot) pair). Output, all in device memory:
//   offs[E+1]      first dispatch row of each expert; every group is padded to a multiple of `pad` rows so that the
//                  64-row reduction blocks of the weight-gradient GEMM never straddle two experts (pad = 1: dense)
//   row_of[T*k]    dispatch row of each pair: rows are ordered by (expert, token, slot) -- a stable counting sort
//   src_of_row[R]  the pair a row carries, -1 for padding rows
//   pos[T, k]      for each token the rows of its experts in ASCENDING expert index (the fixed combine order)
// and the gather of the activations / gate weights into dispatch order (padding rows are zero).
//
// Stability without atomics: CTA e walks ALL pairs in order and gives the pairs routed to e consecutive ranks with a
// block-wide prefix count, so the rank of a pair is the number of earlier pairs with the same expert.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads)
moe_rank_kernel(const int* __restrict__ idx, int n_pairs, int* __restrict__ rank, int* __restrict__ counts) {
  const int e = blockIdx.x;
  __shared__ int warp_tot[kScanThreads / 32];
  __shared__ int s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n_pairs; i0 += kScanThreads) {
    const int i = i0 + threadIdx.x;
    const bool mine = i < n_pairs && idx[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    const int before = __popc(m & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += warp_tot[w];
    const int base = s_base;
    if (mine) rank[i] = base + wbase + before;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < kScanThreads / 32; ++w) tot += warp_tot[w];
      s_base = base + tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = s_base;
}

__global__ void moe_offsets_kernel(const int* __restrict__ counts, int E, int pad, int* __restrict__ offs) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = acc;
      acc += (counts[e] + pad - 1) / pad * pad;
    }
    offs[E] = acc;
  }
}

// one thread per token: absolute rows of its k pairs, the inverse map, and the token's rows by ascending expert
template <int KMAX>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const int* __restrict__ idx, const int* __restrict__ rank, const int* __restrict__ offs, int T, int k,
                int* __restrict__ row_of, int* __restrict__ src_of_row, long long* __restrict__ pos) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  int ex[KMAX], rw[KMAX];
  for (int s = 0; s < k; ++s) {
    const int p = t * k + s;
    const int e = idx[p];
    const int r = offs[e] + rank[p];
    row_of[p] = r;
    src_of_row[r] = p;
    ex[s] = e, rw[s] = r;
  }
  // insertion sort by expert index (k is small); equal experts cannot occur within a token
  for (int a = 1; a < k; ++a) {
    const int ke = ex[a], kr = rw[a];
    int b = a - 1;
    while (b >= 0 && ex[b] > ke) {
      ex[b + 1] = ex[b], rw[b + 1] = rw[b];
      --b;
    }
    ex[b + 1] = ke, rw[b + 1] = kr;
  }
  for (int s = 0; s < k; ++s) pos[static_cast<size_t>(t) * k + s] = rw[s];
}

// x_rows[r, :] = y[src_of_row[r] / k, :] (zero for padding rows); w_rows[r] = w[src_of_row[r]] (zero for padding).
// Rows at or beyond offs[E] are not touched. One warp per row.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const float* __restrict__ w, const int* __restrict__ src_of_row,
                  const int* __restrict__ offs, int E, int k, int H, __nv_bfloat16* __restrict__ x_rows, float* __restrict__ w_rows) {
  const int total = offs[E];
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total; r += gridDim.x * (blockDim.x >> 5)) {
    const int p = src_of_row[r];
    uint4* dst = reinterpret_cast<uint4*>(x_rows + static_cast<size_t>(r) * H);
    if (p < 0) {
      for (int c = lane; c < H / 8; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
      if (lane == 0 && w_rows) w_rows[r] = 0.f;
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(y + static_cast<size_t>(p / k) * ldy);
      for (int c = lane; c < H / 8; c += 32) dst[c] = src[c];
      if (lane == 0 && w_rows) w_rows[r] = w ? w[p] : 1.f;
    }
  }
}

__device__ __forceinline__ float silu_f32(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))); }

// Backward of  a2 = bf16( bf16( bf16(silu(g)) * u ) * w_row )  with h = [g | u] (bf16, [R, 2F]):
//   d_h = [d_g | d_u] (bf16) and d_w_row (fp32); the roundings are treated as identities. One warp per row.
__global__ void __launch_bounds__(256)
moe_glu_scale_bwd_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ w_rows, const __nv_bfloat16* __restrict__ d_a2,
                         const int* __restrict__ offs, int E, int F, __nv_bfloat16* __restrict__ d_h, float* __restrict__ d_w) {
  const int total = offs[E];
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total; r += gridDim.x * (blockDim.x >> 5)) {
    const __nv_bfloat16* g = h + static_cast<size_t>(r) * 2 * F;
    const __nv_bfloat16* u = g + F;
    const __nv_bfloat16* da2 = d_a2 + static_cast<size_t>(r) * F;
    __nv_bfloat16* dg = d_h + static_cast<size_t>(r) * 2 * F;
    __nv_bfloat16* du = dg + F;
    const float w = w_rows[r];
    float acc = 0.f;
    for (int c = lane * 2; c < F; c += 64) {
      float o_g[2], o_u[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float gv = bf2f(g[c + j]), uv = bf2f(u[c + j]), d = bf2f(da2[c + j]);
        const float sg = round_bf(silu_f32(gv));
        const float a = round_bf(__fmul_rn(sg, uv));
        acc = __fmaf_rn(d, a, acc);
        const float da = __fmul_rn(d, w);
        const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gv)));
        const float dsilu = __fmul_rn(sig, __fmaf_rn(gv, __fsub_rn(1.0f, sig), 1.0f));
        o_u[j] = __fmul_rn(da, sg);
        o_g[j] = __fmul_rn(__fmul_rn(da, uv), dsilu);
      }
      *reinterpret_cast<uint32_t*>(dg + c) = pack_bf2(o_g[0], o_g[1]);
      *reinterpret_cast<uint32_t*>(du + c) = pack_bf2(o_u[0], o_u[1]);
    }
    acc = warp_sum_butterfly(acc);
    if (lane == 0) d_w[r] = acc;
  }
}

// d_rows[r, :] = g[src_of_row[r] / k, :] (bf16), zero for padding rows: backward of the fixed-order combine
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ g, long long ldg, const int* __restrict__ src_of_row, const int* __restrict__ offs,
                        int E, int k, int H, __nv_bfloat16* __restrict__ d_rows) {
  const int total = offs[E];
  const int lane = threadIdx.x & 31;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total; r += gridDim.x * (blockDim.x >> 5)) {
    const int p = src_of_row[r];
    uint4* dst = reinterpret_cast<uint4*>(d_rows + static_cast<size_t>(r) * H);
    if (p < 0) {
      for (int c = lane; c < H / 8; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(g + static_cast<size_t>(p / k) * ldg);
      for (int c = lane; c < H / 8; c += 32) dst[c] = src[c];
    }
  }
}

}  // namespace

// idx int32 [T*k] -> offs int32 [E+1], row_of int32 [T*k], src_of_row int32 [r_cap], pos int64 [T*k].
// scratch: int32 [T*k + E] (ranks, counts). r_cap >= T*k + E*(pad-1) rows. No host synchronisation.
IX_API int ix_moe_dispatch_plan(const void* idx, int T, int k, int E, int pad, void* offs, void* row_of, void* src_of_row, int r_cap,
                                void* pos, void* scratch, void* stream) {
  if (T < 0 || k < 1 || k > 16 || E < 1 || pad < 1) return ixh::fail(ixh::IX_EARG, "moe_dispatch_plan: bad sizes T=%d k=%d E=%d pad=%d", T, k, E, pad);
  const long long need = static_cast<long long>(T) * k + static_cast<long long>(E) * (pad - 1);
  if (r_cap < need) return ixh::fail(ixh::IX_ESIZE, "moe_dispatch_plan: row capacity %d < %lld", r_cap, need);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* rank = static_cast<int*>(scratch);
  int* counts = rank + static_cast<size_t>(T) * k;
  IX_CUDA(cudaMemsetAsync(src_of_row, 0xFF, static_cast<size_t>(r_cap) * sizeof(int), s));
  moe_rank_kernel<<<E, kScanThreads, 0, s>>>(static_cast<const int*>(idx), T * k, rank, counts);
  moe_offsets_kernel<<<1, 32, 0, s>>>(counts, E, pad, static_cast<int*>(offs));
  if (T > 0)
    moe_rows_kernel<16><<<(T + 255) / 256, 256, 0, s>>>(static_cast<const int*>(idx), rank, static_cast<const int*>(offs), T, k,
                                                        static_cast<int*>(row_of), static_cast<int*>(src_of_row), static_cast<long long*>(pos));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_moe_gather_rows(const void* y, long long ldy, const void* w, const void* src_of_row, const void* offs, int E, int k, int H,
                              void* x_rows, void* w_rows, void* stream) {
  if (H & 7) return ixh::fail(ixh::IX_EARG, "moe_gather_rows: H=%d must be a multiple of 8", H);
  moe_gather_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), ldy, static_cast<const float*>(w), static_cast<const int*>(src_of_row),
      static_cast<const int*>(offs), E, k, H, static_cast<__nv_bfloat16*>(x_rows), static_cast<float*>(w_rows));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_moe_scatter_rows(const void* g, long long ldg, const void* src_of_row, const void* offs, int E, int k, int H, void* d_rows,
                               void* stream) {
  if (H & 7) return ixh::fail(ixh::IX_EARG, "moe_scatter_rows: H=%d must be a multiple of 8", H);
  moe_scatter_rows_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(g), ldg, static_cast<const int*>(src_of_row), static_cast<const int*>(offs), E, k, H,
      static_cast<__nv_bfloat16*>(d_rows));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_moe_glu_scale_bwd(const void* h, const void* w_rows, const void* d_a2, const void* offs, int E, int F, void* d_h, void* d_w,
                                void* stream) {
  if (F & 1) return ixh::fail(ixh::IX_EARG, "moe_glu_scale_bwd: F=%d must be even", F);
  moe_glu_scale_bwd_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(h), static_cast<const float*>(w_rows), static_cast<const __nv_bfloat16*>(d_a2),
      static_cast<const int*>(offs), E, F, static_cast<__nv_bfloat16*>(d_h), static_cast<float*>(d_w));
  IX_CUDA(cudaGetLastError());
  return 0;
}
