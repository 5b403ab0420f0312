// PPO/GRPO token loss (forward + gradient in one pass), fixed-order reductions,
// AdamW on flat buffers, and the gradient-norm / clip-coefficient kernels.
//
// Loss semantics follow the reference's policy loss (B/utils/ppo_utils.py:541-571):
//   ratio = exp(clamp(lp - old, -20, 20)); l1 = -A*ratio; l2 = -A*clamp(ratio, 1-lo, 1+hi)
//   loss = max(l1, l2); dual clip (A < 0): loss = min(loss, -A*c)
// plus optional KL-to-reference term (k1 / abs / k2 / k3, ppo_utils.py:88-125).
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

struct PpoArgs {
  const float* lp;
  const float* old_lp;
  const float* adv;
  const float* mask;
  const float* ref_lp;   // may be null
  const float* tis;      // optional per-token importance weights (off-policy correction), may be null
  float* loss_tok;
  float* grad_lp;
  float* clip_tok;       // 1 where the clipped branch was active
  float* kl_tok;         // may be null
  float eps_lo, eps_hi, clip_c, kl_coef;
  int dual_clip, kl_kind;  // kl_kind: 0 k1, 1 abs, 2 k2, 3 k3
  long long n;
};

__global__ void __launch_bounds__(256) ppo_loss_kernel(PpoArgs a) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < a.n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float mk = a.mask[i];
    const float A = a.adv[i];
    const float lp = a.lp[i];
    float d = lp - a.old_lp[i];
    const bool sat = d < -20.f || d > 20.f;
    d = fminf(fmaxf(d, -20.f), 20.f);
    const float ratio = expf(d);
    const float rc = fminf(fmaxf(ratio, 1.f - a.eps_lo), 1.f + a.eps_hi);
    const float l1 = -A * ratio, l2 = -A * rc;
    float loss = fmaxf(l1, l2);
    // gradient wrt lp through the unclipped branch only when it is the active one
    float g = (l1 >= l2 && !sat) ? -A * ratio : 0.f;
    float clipped = (l2 > l1) ? 1.f : 0.f;
    if (a.dual_clip && A < 0.f) {
      const float l3 = -A * a.clip_c;
      if (l3 < loss) {
        loss = l3;
        g = 0.f;
        clipped = 1.f;
      }
    }
    if (a.tis) {
      loss *= a.tis[i];
      g *= a.tis[i];
    }
    float kl = 0.f;
    if (a.ref_lp) {
      const float lr = lp - a.ref_lp[i];
      float gk = 0.f;
      if (a.kl_kind == 0) { kl = lr; gk = 1.f; }
      else if (a.kl_kind == 1) { kl = fabsf(lr); gk = lr > 0.f ? 1.f : (lr < 0.f ? -1.f : 0.f); }
      else if (a.kl_kind == 2) { kl = 0.5f * lr * lr; gk = lr; }
      else {
        // k3: r = ref - lp clamped to +-20, kl = exp(r) - r - 1 clamped to +-10
        float r = fminf(fmaxf(-lr, -20.f), 20.f);
        const float e = expf(r);
        kl = e - r - 1.f;
        const bool inner = (-lr > -20.f && -lr < 20.f);
        gk = (kl < 10.f && kl > -10.f && inner) ? (1.f - e) : 0.f;
        kl = fminf(fmaxf(kl, -10.f), 10.f);
      }
      loss += a.kl_coef * kl;
      g += a.kl_coef * gk;
    }
    a.loss_tok[i] = loss * mk;
    a.grad_lp[i] = g * mk;
    if (a.clip_tok) a.clip_tok[i] = clipped * mk;
    if (a.kl_tok) a.kl_tok[i] = kl * mk;
  }
}

// ---------------------------------------------------------------- fixed-order reductions
// out[0] = sum(in[0..n)) (SQUARE: sum of squares). Stage 1: block b sums elements
// b*4096 .. in a fixed thread order; stage 2: one CTA adds the partials left to right in
// chunks. The order depends only on n, never on the launch grid.
constexpr int kRedChunk = 4096;

template <typename T, bool SQUARE>
__global__ void __launch_bounds__(256)
reduce_stage1_kernel(const T* __restrict__ in, long long n, float* __restrict__ partials) {
  __shared__ float red[8];
  for (long long b = blockIdx.x; b * kRedChunk < n; b += gridDim.x) {
    float acc = 0.f;
    const long long base = b * kRedChunk + threadIdx.x * 16;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const long long i = base + j;
      if (i < n) {
        float x;
        if constexpr (sizeof(T) == 2) x = __bfloat162float(in[i]);
        else x = in[i];
        acc = __fadd_rn(acc, SQUARE ? __fmul_rn(x, x) : x);
      }
    }
    acc = warp_sum_butterfly(acc);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float r = red[0];
      for (int i = 1; i < 8; ++i) r = __fadd_rn(r, red[i]);
      partials[b] = r;
    }
  }
}

// single CTA: thread t sums partials t, t+256, ... ascending; then butterfly + warp order
__global__ void __launch_bounds__(256)
reduce_stage2_kernel(const float* __restrict__ partials, long long np, float* __restrict__ out, int accumulate) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = threadIdx.x; i < np; i += 256) acc = __fadd_rn(acc, partials[i]);
  acc = warp_sum_butterfly(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = red[0];
    for (int i = 1; i < 8; ++i) r = __fadd_rn(r, red[i]);
    out[0] = accumulate ? __fadd_rn(out[0], r) : r;
  }
}

// clip coefficient from a squared norm: coef = min(1, max_norm / (sqrt(sq) + 1e-6)); norm_out = sqrt(sq)
__global__ void clip_coef_kernel(const float* sq, float max_norm, float* coef, float* norm_out) {
  const float nrm = sqrtf(sq[0]);
  norm_out[0] = nrm;
  coef[0] = (max_norm > 0.f) ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
}

// ---------------------------------------------------------------- AdamW (decoupled weight decay), flat buffers
template <typename G>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, const G* __restrict__ grad,
             __nv_bfloat16* __restrict__ param_bf16, long long n, float lr, float beta1, float beta2, float eps,
             float wd, float bc1, float bc2, const float* __restrict__ gscale) {
  const float gs = gscale ? gscale[0] : 1.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g;
    if constexpr (sizeof(G) == 2) g = __bfloat162float(grad[i]);
    else g = grad[i];
    g *= gs;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p -= lr * wd * p;
    p -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = p;
    if (param_bf16) param_bf16[i] = __float2bfloat16_rn(p);
  }
}

// dst_f32[i] (+)= src_bf16[i]: gradient accumulation across micro-batches into an fp32 main-grad buffer
__global__ void __launch_bounds__(256)
accum_bf16_to_f32_kernel(float* __restrict__ dst, const __nv_bfloat16* __restrict__ src, long long n, int accumulate) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float s = __bfloat162float(src[i]);
    dst[i] = accumulate ? dst[i] + s : s;
  }
}

// Same, eight elements per thread and iteration (one 16-byte load of the source, two of the destination)
__global__ void __launch_bounds__(256)
accum_bf16_to_f32_vec8_kernel(float4* __restrict__ dst, const uint4* __restrict__ src, long long n8, int accumulate) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 s = __ldcs(src + i);                       // the bf16 gradient is dead after this read
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&s);
    float4 a = make_float4(__low2float(p[0]), __high2float(p[0]), __low2float(p[1]), __high2float(p[1]));
    float4 b = make_float4(__low2float(p[2]), __high2float(p[2]), __low2float(p[3]), __high2float(p[3]));
    if (accumulate) {
      const float4 x = dst[2 * i], y = dst[2 * i + 1];
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
      b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
    }
    dst[2 * i] = a;
    dst[2 * i + 1] = b;
  }
}

inline int grid_1d(long long total, int block, int cap = 148 * 8) {
  long long g = (total + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

IX_API int ix_ppo_loss(const void* lp, const void* old_lp, const void* adv, const void* mask, const void* ref_lp,
                       const void* tis, void* loss_tok, void* grad_lp, void* clip_tok, void* kl_tok, long long n,
                       float eps_lo, float eps_hi, float clip_c, int dual_clip, float kl_coef, int kl_kind,
                       void* stream) {
  if (n <= 0) return 0;
  PpoArgs a;
  a.lp = static_cast<const float*>(lp);
  a.old_lp = static_cast<const float*>(old_lp);
  a.adv = static_cast<const float*>(adv);
  a.mask = static_cast<const float*>(mask);
  a.ref_lp = static_cast<const float*>(ref_lp);
  a.tis = static_cast<const float*>(tis);
  a.loss_tok = static_cast<float*>(loss_tok);
  a.grad_lp = static_cast<float*>(grad_lp);
  a.clip_tok = static_cast<float*>(clip_tok);
  a.kl_tok = static_cast<float*>(kl_tok);
  a.eps_lo = eps_lo;
  a.eps_hi = eps_hi;
  a.clip_c = clip_c;
  a.kl_coef = kl_coef;
  a.dual_clip = dual_clip;
  a.kl_kind = kl_kind;
  a.n = n;
  ppo_loss_kernel<<<grid_1d(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  IX_CUDA(cudaGetLastError());
  return 0;
}

// Number of fp32 partials `ix_reduce_sum` needs as scratch for n elements.
IX_API long long ix_reduce_scratch_elems(long long n) { return (n + kRedChunk - 1) / kRedChunk; }

// out[0] (+)= sum of in[0..n) (square=1: sum of squares) in an order that depends only on n.
// dtype: 0 = bf16, 1 = fp32. scratch: ix_reduce_scratch_elems(n) floats.
IX_API int ix_reduce_sum(const void* in, long long n, int dtype, int square, void* scratch, void* out,
                         int accumulate, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n <= 0) {
    if (!accumulate) IX_CUDA(cudaMemsetAsync(out, 0, sizeof(float), s));
    return 0;
  }
  const long long np = (n + kRedChunk - 1) / kRedChunk;
  const int grid = static_cast<int>(np < 148 * 8 ? np : 148 * 8);
  float* part = static_cast<float*>(scratch);
  if (dtype == 0) {
    if (square) reduce_stage1_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), n, part);
    else reduce_stage1_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), n, part);
  } else {
    if (square) reduce_stage1_kernel<float, true><<<grid, 256, 0, s>>>(static_cast<const float*>(in), n, part);
    else reduce_stage1_kernel<float, false><<<grid, 256, 0, s>>>(static_cast<const float*>(in), n, part);
  }
  reduce_stage2_kernel<<<1, 256, 0, s>>>(part, np, static_cast<float*>(out), accumulate);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_clip_coef(const void* sq, float max_norm, void* coef, void* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const float*>(sq), max_norm,
                                                                        static_cast<float*>(coef),
                                                                        static_cast<float*>(norm_out));
  IX_CUDA(cudaGetLastError());
  return 0;
}

// grad_dtype: 0 = bf16, 1 = fp32. step >= 1. gscale: optional device scalar multiplied into the gradient.
IX_API int ix_adamw(void* master, void* m, void* v, const void* grad, void* param_bf16, long long n, int grad_dtype,
                    float lr, float beta1, float beta2, float eps, float wd, int step, const void* gscale,
                    void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (grad_dtype == 0)
    adamw_kernel<__nv_bfloat16><<<grid_1d(n, 256, 148 * 16), 256, 0, s>>>(
        static_cast<float*>(master), static_cast<float*>(m), static_cast<float*>(v),
        static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(param_bf16), n, lr, beta1, beta2, eps, wd,
        bc1, bc2, static_cast<const float*>(gscale));
  else
    adamw_kernel<float><<<grid_1d(n, 256, 148 * 16), 256, 0, s>>>(
        static_cast<float*>(master), static_cast<float*>(m), static_cast<float*>(v), static_cast<const float*>(grad),
        static_cast<__nv_bfloat16*>(param_bf16), n, lr, beta1, beta2, eps, wd, bc1, bc2,
        static_cast<const float*>(gscale));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_accum_bf16_to_f32(void* dst, const void* src, long long n, int accumulate, void* stream) {
  if (n <= 0) return 0;
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    accum_bf16_to_f32_vec8_kernel<<<grid_1d(n / 8, 256, 148 * 16), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<float4*>(dst), static_cast<const uint4*>(src), n / 8, accumulate);
    IX_CUDA(cudaGetLastError());
    return 0;
  }
  accum_bf16_to_f32_kernel<<<grid_1d(n, 256, 148 * 16), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(dst), static_cast<const __nv_bfloat16*>(src), n, accumulate);
  IX_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------ allocation-free reduction
// See ix_noalloc.h for who needs this and what the limits are.
#include "ix_noalloc.h"

namespace {

// Partial sums of stage 1 live here instead of in caller-provided memory. One copy of this
// array exists on every GPU whose context loads the library, from load until process exit.
static __device__ __align__(256) float g_noalloc_partials[IX_NOALLOC_MAX_PARTIALS];

// Device address of the array above, per device ordinal. In host code the symbol's name is
// only a handle for the runtime; the address a kernel can dereference comes from
// cudaGetSymbolAddress, taken with that device current.
float* g_noalloc_ptr[64] = {nullptr};

int noalloc_scratch(int dev, float** out) {
  if (dev < 0 || dev >= 64) return ixh::fail(ixh::IX_EARG, "reduce_sum_noalloc: device ordinal %d out of range", dev);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    IX_CUDA(cudaGetSymbolAddress(&p, g_noalloc_partials));
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace

IX_API long long ix_reduce_sum_noalloc_max_elems() {
  return static_cast<long long>(IX_NOALLOC_MAX_PARTIALS) * kRedChunk;
}

IX_API int ix_reduce_sum_noalloc(const void* in, long long n, int dtype, int square, void* out, int accumulate,
                                 void* stream) {
  if (n < 0) return ixh::fail(ixh::IX_EARG, "reduce_sum_noalloc: negative length %lld", n);
  if (n > ix_reduce_sum_noalloc_max_elems())
    return ixh::fail(ixh::IX_ESIZE,
                     "reduce_sum_noalloc: %lld elements exceed the built-in scratch (max %lld); use ix_reduce_sum with "
                     "caller-provided scratch for larger inputs",
                     n, ix_reduce_sum_noalloc_max_elems());
  if (dtype != 0 && dtype != 1) return ixh::fail(ixh::IX_EARG, "reduce_sum_noalloc: dtype must be 0 (bf16) or 1 (fp32)");
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  float* part = nullptr;
  int rc = noalloc_scratch(dev, &part);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n == 0) {
    if (!accumulate) IX_CUDA(cudaMemsetAsync(out, 0, sizeof(float), s));
    return 0;
  }
  // Nothing in the scratch has to start at zero: stage 1 overwrites partials [0, np) and
  // stage 2 reads exactly those, so whatever an earlier call left behind is never read.
  const long long np = (n + kRedChunk - 1) / kRedChunk;
  const int grid = static_cast<int>(np < 148 * 8 ? np : 148 * 8);
  if (dtype == 0) {
    if (square) reduce_stage1_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), n, part);
    else reduce_stage1_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), n, part);
  } else {
    if (square) reduce_stage1_kernel<float, true><<<grid, 256, 0, s>>>(static_cast<const float*>(in), n, part);
    else reduce_stage1_kernel<float, false><<<grid, 256, 0, s>>>(static_cast<const float*>(in), n, part);
  }
  reduce_stage2_kernel<<<1, 256, 0, s>>>(part, np, static_cast<float*>(out), accumulate);
  IX_CUDA(cudaGetLastError());
  return 0;
}
