// MoE routing kernels: top-k router and the fixed-order combine.
//
// Router (one warp per token, E <= 256 experts, lane l holds experts l, l+32, ...):
//   softmax score : m = exact max; e_i = expf(x_i - m); S = lane partials in ascending expert order,
//                   then the 16,8,4,2,1 xor butterfly; p_i = e_i / S (IEEE division)
//   sigmoid+bias  : s_i = 1 / (1 + expf(-x_i)); selection by s_i + bias_i, gate weight s_i
//   top-k         : k rounds of warp arg-max; a tie goes to the LOWER expert index
//                   (the reference pins the same rule, ISO/ops/moe/moe_router_o2_kernel.py:272-443)
//   normalisation : w_r / (w_0 + w_1 + ... in selection order), optional
// Outputs are in selection order (descending score). A token's routing never depends on the
// other tokens of the launch.
//
// Combine (one warp per token): out[t] = round( sum over the token's k expert rows, taken in
// ASCENDING EXPERT INDEX, fp32 ), optionally + shared-expert row after the round.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kMaxPerLane = 8;  // E <= 256

__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias, int T, int E, int K,
                   int sigmoid_bias, int norm_topk, int* __restrict__ idx_out, float* __restrict__ w_out,
                   float* __restrict__ probs_out) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* x = logits + static_cast<size_t>(t) * ld;
  float score[kMaxPerLane], gate[kMaxPerLane];
  const int per = (E + 31) / 32;
  if (!sigmoid_bias) {
    float m = -INFINITY;
    for (int j = 0; j < per; ++j) {
      const int e = lane + 32 * j;
      score[j] = e < E ? x[e] : -INFINITY;
      m = fmaxf(m, score[j]);
    }
    m = warp_max(m);
    float part = 0.f;
    for (int j = 0; j < per; ++j) {
      const int e = lane + 32 * j;
      gate[j] = e < E ? expf(__fsub_rn(score[j], m)) : 0.f;
      part = __fadd_rn(part, gate[j]);
    }
    const float S = warp_sum_butterfly(part);
    for (int j = 0; j < per; ++j) {
      gate[j] = __fdiv_rn(gate[j], S);
      score[j] = (lane + 32 * j) < E ? gate[j] : -INFINITY;
    }
  } else {
    for (int j = 0; j < per; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        gate[j] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x[e])));
        score[j] = bias ? __fadd_rn(gate[j], bias[e]) : gate[j];
      } else {
        gate[j] = 0.f;
        score[j] = -INFINITY;
      }
    }
  }
  if (probs_out)
    for (int j = 0; j < per; ++j)
      if (lane + 32 * j < E) probs_out[static_cast<size_t>(t) * E + lane + 32 * j] = gate[j];
  float wsum = 0.f;
  float my_w = 0.f;   // lane r keeps the weight of selection r (K <= 32)
  int my_i = 0;
  for (int r = 0; r < K; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    float bg = 0.f;
    for (int j = 0; j < per; ++j) {
      const int e = lane + 32 * j;
      if (score[j] > bv || (score[j] == bv && e < bi && score[j] != -INFINITY)) {
        bv = score[j];
        bi = e;
        bg = gate[j];
      }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      const float og = __shfl_xor_sync(0xffffffffu, bg, off);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
        bg = og;
      }
    }
    // every lane now agrees on (bv, bi, bg); the owner retires the expert
    if ((bi & 31) == lane) score[bi >> 5] = -INFINITY;
    wsum = __fadd_rn(wsum, bg);
    if (lane == r) {
      my_w = bg;
      my_i = bi;
    }
  }
  if (lane < K) {
    if (norm_topk) my_w = __fdiv_rn(my_w, wsum);
    idx_out[static_cast<size_t>(t) * K + lane] = my_i;
    w_out[static_cast<size_t>(t) * K + lane] = my_w;
  }
}

// rows: fp32 [R, H] expert outputs in dispatch order; pos[t, j]: row of token t's j-th expert with
// j running over the token's experts in ASCENDING expert index; out: [T, H] activation dtype.
template <bool OUT_BF16>
__global__ void __launch_bounds__(128)
combine_kernel(const float* __restrict__ rows, const long long* __restrict__ pos, const void* __restrict__ shared_rows,
               void* __restrict__ out, int T, int H, int K) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane * 4; c < H; c += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < K; ++j) {
      const long long r = pos[static_cast<size_t>(t) * K + j];
      if (r < 0) continue;
      const float4 v = *reinterpret_cast<const float4*>(rows + static_cast<size_t>(r) * H + c);
      if (j == 0) acc = v;
      else {
        acc.x = __fadd_rn(acc.x, v.x);
        acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z);
        acc.w = __fadd_rn(acc.w, v.w);
      }
    }
    if constexpr (OUT_BF16) {
      float a0 = round_bf(acc.x), a1 = round_bf(acc.y), a2 = round_bf(acc.z), a3 = round_bf(acc.w);
      if (shared_rows) {
        const __nv_bfloat16* sr = static_cast<const __nv_bfloat16*>(shared_rows) + static_cast<size_t>(t) * H + c;
        a0 = __fadd_rn(a0, bf2f(sr[0]));
        a1 = __fadd_rn(a1, bf2f(sr[1]));
        a2 = __fadd_rn(a2, bf2f(sr[2]));
        a3 = __fadd_rn(a3, bf2f(sr[3]));
      }
      uint2 w;
      w.x = pack_bf2(a0, a1);
      w.y = pack_bf2(a2, a3);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(t) * H + c) = w;
    } else {
      if (shared_rows) {
        const float* sr = static_cast<const float*>(shared_rows) + static_cast<size_t>(t) * H + c;
        acc.x = __fadd_rn(acc.x, sr[0]);
        acc.y = __fadd_rn(acc.y, sr[1]);
        acc.z = __fadd_rn(acc.z, sr[2]);
        acc.w = __fadd_rn(acc.w, sr[3]);
      }
      *reinterpret_cast<float4*>(static_cast<float*>(out) + static_cast<size_t>(t) * H + c) = acc;
    }
  }
}

// act[r, :] = round(act[r, :] * w[r]) in place: gate weight applied to the SwiGLU output before fc2
__global__ void __launch_bounds__(256)
scale_rows_kernel(__nv_bfloat16* __restrict__ act, const float* __restrict__ w, long long R, int F) {
  const long long nv = static_cast<long long>(F) >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < R * nv;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / nv;
    uint4* p = reinterpret_cast<uint4*>(act + r * F) + (i % nv);
    uint4 v = *p;
    const float s = w[r];
    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = f2bf(__fmul_rn(bf2f(e[j]), s));
    *p = v;
  }
}

}  // namespace

IX_API int ix_router_topk(const void* logits, long long ld, const void* bias, int T, int E, int K, int sigmoid_bias,
                          int norm_topk, void* idx_out, void* w_out, void* probs_out, void* stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > 32 * kMaxPerLane) return ixh::fail(ixh::IX_EARG, "router: E=%d unsupported (1..256)", E);
  if (K < 1 || K > 32 || K > E) return ixh::fail(ixh::IX_EARG, "router: top-k=%d unsupported", K);
  router_topk_kernel<<<(T + 3) / 4, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(logits), ld, static_cast<const float*>(bias), T, E, K, sigmoid_bias, norm_topk,
      static_cast<int*>(idx_out), static_cast<float*>(w_out), static_cast<float*>(probs_out));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_moe_combine(const void* rows, const void* pos, const void* shared_rows, void* out, int T, int H, int K,
                          int out_bf16, void* stream) {
  if (T <= 0) return 0;
  if (H & 3) return ixh::fail(ixh::IX_EARG, "combine: H=%d must be a multiple of 4", H);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (out_bf16)
    combine_kernel<true><<<(T + 3) / 4, 128, 0, s>>>(static_cast<const float*>(rows), static_cast<const long long*>(pos),
                                                     shared_rows, out, T, H, K);
  else
    combine_kernel<false><<<(T + 3) / 4, 128, 0, s>>>(static_cast<const float*>(rows), static_cast<const long long*>(pos),
                                                      shared_rows, out, T, H, K);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_scale_rows(void* act, const void* w, long long R, int F, void* stream) {
  if (R <= 0) return 0;
  if (F & 7) return ixh::fail(ixh::IX_EARG, "scale_rows: F=%d must be a multiple of 8", F);
  long long g = (R * (F >> 3) + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  scale_rows_kernel<<<static_cast<int>(g), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(act), static_cast<const float*>(w), R, F);
  IX_CUDA(cudaGetLastError());
  return 0;
}
