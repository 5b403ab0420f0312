// GatedDeltaNet kernels: causal conv + SiLU, gating, q/k L2 norm, and the gated delta-rule scan.
//
// One scan kernel serves the trainer (whole packed sequences), the engine's chunked prefill and
// the engine's decode (chunks of one token continuing from the state pool): a (sequence chunk,
// value head) pair is processed by one CTA, token by token, in fp32 with a fixed operation
// order, so "chunked" and "recurrent" execution are the same arithmetic by construction:
//
//   S  <- S * exp(g_t)                        (S is [Dv, Dk] fp32; thread j owns row j)
//   kv <- sum_i S[j][i] * k_t[i]              (fma chain, ascending i)
//   d  <- (v_t[j] - kv) * beta_t
//   S[j][i] <- fma(d, k_t[i], S[j][i])
//   o_t[j] <- sum_i S[j][i] * q_t[i]          (fma chain, ascending i), rounded once
//
// With snapshot_every = C > 0 the state is additionally rounded through bf16 whenever the
// sequence position reaches a multiple of C (the "CPR" variant of the reference, which snapshots
// chunk-boundary states to bf16, ISO/ops/gdn/gdn_cpr.py:104-292); 0 keeps the plain fp32 chain.
// Every fma is written with __fmaf_rn so the C++ oracle (std::fmaf) reproduces the bits wherever
// exp() agrees.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

struct ScanChunk {
  int tok_start;   // first token row of the chunk in the packed tensors
  int n_tok;       // tokens in the chunk
  int pos0;        // sequence position of the first token (for snapshot boundaries)
  int pad;
  long long row_in;   // state-pool row to start from, or -1 for a zero state
  long long row_out;  // state-pool row to store the final state to, or -1
};

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <typename T> __device__ __forceinline__ float rndT(float v);
template <> __device__ __forceinline__ float rndT<__nv_bfloat16>(float v) { return round_bf(v); }
template <> __device__ __forceinline__ float rndT<float>(float v) { return v; }

// ------------------------------------------------------------------ causal depthwise conv (width W <= 4) + SiLU
// x: [T, ldx] (C conv channels starting at column 0). tok_back[t]: how many earlier tokens of the same
// sequence precede t inside this launch (taps reaching further back come from the conv state).
// state_row[t]: row of the conv-state pool of t's sequence (-1: zeros). conv_state: [rows, C, W-1],
// oldest input first.
template <typename T>
__global__ void __launch_bounds__(256)
gdn_conv_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w, const int* __restrict__ tok_back,
                const long long* __restrict__ state_row, const T* __restrict__ conv_state, T* __restrict__ out,
                long long Tn, int C, int W) {
  const long long total = Tn * C;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / C;
    const int c = static_cast<int>(i % C);
    const int back = tok_back[t];
    const long long srow = state_row ? state_row[t] : -1;
    float acc = 0.f;
    for (int j = 0; j < W; ++j) {             // tap j multiplies the input (W-1-j) steps in the past
      const int d = W - 1 - j;
      float xv;
      if (d <= back) xv = ldf(x, (t - d) * ldx + c);
      else if (srow >= 0) xv = ldf(conv_state, (srow * C + c) * (W - 1) + (W - 1) - (d - back));
      else xv = 0.f;
      acc = __fmaf_rn(ldf(w, static_cast<long long>(c) * W + j), xv, acc);
    }
    const float s = __fdiv_rn(acc, __fadd_rn(1.0f, expf(-acc)));
    stf(out, t * C + c, s);
  }
}

// The same function, eight channels per thread (bf16, C and ldx multiples of 8): one 16-byte load per tap instead of
// eight 2-byte ones and 32-bit index arithmetic. Every output element runs the chain of the kernel above (taps in
// ascending j, one fused multiply-add each, then SiLU), so the bits are the same; only the mapping of elements to
// threads differs. Taps that reach behind the launch's first token of a sequence (the conv state) are read element by
// element: they touch at most W-1 tokens per sequence.
template <int W>
__global__ void __launch_bounds__(256)
gdn_conv_vec8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                     const int* __restrict__ tok_back, const long long* __restrict__ state_row,
                     const __nv_bfloat16* __restrict__ conv_state, __nv_bfloat16* __restrict__ out, int Tn, int C) {
  const int c8n = C >> 3;
  const long long total = static_cast<long long>(Tn) * c8n;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / c8n);
    const int c = static_cast<int>(i - static_cast<long long>(t) * c8n) << 3;
    const int back = tok_back[t];
    const long long srow = state_row ? state_row[t] : -1;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // weights of these 8 channels: [c][W] contiguous, 8*W bf16
    __nv_bfloat16 wv[8 * W];
#pragma unroll
    for (int e = 0; e < 8 * W; ++e) wv[e] = w[static_cast<long long>(c) * W + e];
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const int d = W - 1 - j;
      float xv[8];
      if (d <= back) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(t - d) * ldx + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          xv[2 * e] = f.x;
          xv[2 * e + 1] = f.y;
        }
      } else if (srow >= 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          xv[e] = __bfloat162float(conv_state[(srow * C + c + e) * (W - 1) + (W - 1) - (d - back)]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xv[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = __fmaf_rn(__bfloat162float(wv[e * W + j]), xv[e], acc[e]);
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float s0 = __fdiv_rn(acc[2 * e], __fadd_rn(1.0f, expf(-acc[2 * e])));
      const float s1 = __fdiv_rn(acc[2 * e + 1], __fadd_rn(1.0f, expf(-acc[2 * e + 1])));
      oh[e] = __halves2bfloat162(__float2bfloat16_rn(s0), __float2bfloat16_rn(s1));
    }
    *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * C + c) = o;
  }
}

// new conv state of every chunk: the last W-1 pre-conv inputs of the sequence
template <typename T>
__global__ void __launch_bounds__(256)
gdn_conv_state_kernel(const T* __restrict__ x, long long ldx, const ScanChunk* __restrict__ chunks, T* __restrict__ conv_state,
                      int n_chunks, int C, int W) {
  const long long total = static_cast<long long>(n_chunks) * C;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ch = static_cast<int>(i / C);
    const int c = static_cast<int>(i % C);
    const ScanChunk sc = chunks[ch];
    if (sc.row_out < 0) continue;
    float nv[3];
    for (int j = 0; j < W - 1; ++j) {         // slot j holds the input (W-1-j) steps before the next token
      const int d = W - 1 - j;                // steps back from the end of the chunk
      if (d <= sc.n_tok) nv[j] = ldf(x, static_cast<long long>(sc.tok_start + sc.n_tok - d) * ldx + c);
      else if (sc.row_in >= 0) nv[j] = ldf(conv_state, (sc.row_in * C + c) * (W - 1) + j + sc.n_tok);
      else nv[j] = 0.f;
    }
    for (int j = 0; j < W - 1; ++j) stf(conv_state, (sc.row_out * C + c) * (W - 1) + j, nv[j]);
  }
}

// ------------------------------------------------------------------ gating: g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b)
template <typename T>
__global__ void __launch_bounds__(256)
gdn_gate_kernel(const T* __restrict__ a, const T* __restrict__ b, long long ld, const T* __restrict__ A_log,
                const T* __restrict__ dt_bias, float* __restrict__ g, float* __restrict__ beta, long long Tn, int H) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < Tn * H;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / H;
    const int h = static_cast<int>(i % H);
    const float x = __fadd_rn(ldf(a, t * ld + h), ldf(dt_bias, h));
    const float sp = x > 20.f ? x : log1pf(expf(x));
    g[i] = __fmul_rn(-expf(ldf(A_log, h)), sp);
    beta[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-ldf(b, t * ld + h))));
  }
}

// ------------------------------------------------------------------ L2 norm of q and k heads (one warp per (token, head))
// in: [T, ld] with q heads at column 0 and k heads at column Hk*D; out_q, out_k: [T, Hk, D].
// n = round(x * rstd), rstd = 1/sqrt(sum x^2 + eps); q is additionally scaled by D^-0.5 (one more round).
template <typename T>
__global__ void __launch_bounds__(128)
gdn_l2norm_kernel(const T* __restrict__ in, long long ld, T* __restrict__ out_q, T* __restrict__ out_k, long long Tn, int Hk,
                  int D, float eps, float q_scale) {
  const long long wid = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= Tn * 2 * Hk) return;
  const long long t = wid / (2 * Hk);
  const int hh = static_cast<int>(wid % (2 * Hk));
  const bool is_k = hh >= Hk;
  const int h = is_k ? hh - Hk : hh;
  const T* src = in + t * ld + (is_k ? static_cast<long long>(Hk) * D : 0) + static_cast<long long>(h) * D;
  float ss = 0.f;
  for (int v = lane; v < D / 8; v += 32)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = ldf(src, v * 8 + j);
      ss = __fadd_rn(ss, __fmul_rn(f, f));
    }
  ss = warp_sum_butterfly(ss);
  const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, eps)));
  T* dst = (is_k ? out_k : out_q) + (t * Hk + h) * D;
  for (int v = lane; v < D / 8; v += 32)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float n = rndT<T>(__fmul_rn(ldf(src, v * 8 + j), rstd));
      if (!is_k) n = rndT<T>(__fmul_rn(n, q_scale));
      stf(dst, v * 8 + j, n);
    }
}

// ------------------------------------------------------------------ gated delta-rule scan
template <typename T, int DK>
__global__ void __launch_bounds__(128)
gdn_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ g,
                const float* __restrict__ beta, const ScanChunk* __restrict__ chunks, float* __restrict__ state,
                T* __restrict__ out, int Hk, int Hv, int DV, int snapshot_every) {
  __shared__ float sk[2][DK], sq[2][DK];
  __shared__ float sg[2], sb[2];
  const ScanChunk sc = chunks[blockIdx.x];
  const int hv = blockIdx.y;
  const int hk = hv / (Hv / Hk);
  const int j = threadIdx.x;              // value-dim row owned by this thread
  const bool active = j < DV;
  float S[DK];
  if (sc.row_in >= 0 && active) {
    const float* sp = state + ((sc.row_in * Hv + hv) * DV + j) * DK;
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = sp[i];
  } else {
#pragma unroll
    for (int i = 0; i < DK; ++i) S[i] = 0.f;
  }
  auto stage = [&](int tt, int buf) {
    const long long t = sc.tok_start + tt;
    for (int i = threadIdx.x; i < DK; i += 128) {
      sk[buf][i] = ldf(k, (t * Hk + hk) * DK + i);
      sq[buf][i] = ldf(q, (t * Hk + hk) * DK + i);
    }
    if (threadIdx.x == 0) {
      sg[buf] = expf(g[t * Hv + hv]);
      sb[buf] = beta[t * Hv + hv];
    }
  };
  if (sc.n_tok > 0) stage(0, 0);
  __syncthreads();
  for (int tt = 0; tt < sc.n_tok; ++tt) {
    const int buf = tt & 1;
    if (tt + 1 < sc.n_tok) stage(tt + 1, buf ^ 1);
    const long long t = sc.tok_start + tt;
    if (active) {
      const float decay = sg[buf], bt = sb[buf];
      float kv = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        S[i] = __fmul_rn(S[i], decay);
        kv = __fmaf_rn(S[i], sk[buf][i], kv);
      }
      const float d = __fmul_rn(__fsub_rn(ldf(v, (t * Hv + hv) * DV + j), kv), bt);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        S[i] = __fmaf_rn(d, sk[buf][i], S[i]);
        o = __fmaf_rn(S[i], sq[buf][i], o);
      }
      stf(out, (t * Hv + hv) * DV + j, o);
      if (snapshot_every > 0 && ((sc.pos0 + tt + 1) % snapshot_every) == 0) {
#pragma unroll
        for (int i = 0; i < DK; ++i) S[i] = round_bf(S[i]);
      }
    }
    __syncthreads();
  }
  if (sc.row_out >= 0 && active) {
    float* sp = state + ((sc.row_out * Hv + hv) * DV + j) * DK;
#pragma unroll
    for (int i = 0; i < DK; ++i) sp[i] = S[i];
  }
}

inline int grid1d(long long total, int block) {
  long long g = (total + block - 1) / block;
  if (g > 148 * 16) g = 148 * 16;
  return g < 1 ? 1 : static_cast<int>(g);
}

}  // namespace

#define IX_GDN_DT(is_f32, ...)               \
  if (is_f32) {                              \
    using T = float;                         \
    __VA_ARGS__;                             \
  } else {                                   \
    using T = __nv_bfloat16;                 \
    __VA_ARGS__;                             \
  }

IX_API int ix_gdn_conv(const void* x, long long ldx, const void* w, const void* tok_back, const void* state_row,
                       const void* conv_state, void* out, long long Tn, int C, int W, int is_f32, void* stream) {
  if (Tn <= 0) return 0;
  if (W < 1 || W > 4) return ixh::fail(ixh::IX_EARG, "gdn_conv: width %d unsupported (1..4)", W);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!is_f32 && W == 4 && (C & 7) == 0 && (ldx & 7) == 0 && Tn < (1ll << 31) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    gdn_conv_vec8_kernel<4><<<grid1d(Tn * (C >> 3), 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w), static_cast<const int*>(tok_back),
        static_cast<const long long*>(state_row), static_cast<const __nv_bfloat16*>(conv_state), static_cast<__nv_bfloat16*>(out),
        static_cast<int>(Tn), C);
    IX_CUDA(cudaGetLastError());
    return 0;
  }
  IX_GDN_DT(is_f32, (gdn_conv_kernel<T><<<grid1d(Tn * C, 256), 256, 0, s>>>(
                        static_cast<const T*>(x), ldx, static_cast<const T*>(w), static_cast<const int*>(tok_back),
                        static_cast<const long long*>(state_row), static_cast<const T*>(conv_state), static_cast<T*>(out), Tn, C, W)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_gdn_conv_state(const void* x, long long ldx, const void* chunks, void* conv_state, int n_chunks, int C, int W,
                             int is_f32, void* stream) {
  if (n_chunks <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  IX_GDN_DT(is_f32, (gdn_conv_state_kernel<T><<<grid1d(static_cast<long long>(n_chunks) * C, 256), 256, 0, s>>>(
                        static_cast<const T*>(x), ldx, static_cast<const ScanChunk*>(chunks), static_cast<T*>(conv_state), n_chunks, C, W)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_gdn_gate(const void* a, const void* b, long long ld, const void* A_log, const void* dt_bias, void* g, void* beta,
                       long long Tn, int H, int is_f32, void* stream) {
  if (Tn <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  IX_GDN_DT(is_f32, (gdn_gate_kernel<T><<<grid1d(Tn * H, 256), 256, 0, s>>>(
                        static_cast<const T*>(a), static_cast<const T*>(b), ld, static_cast<const T*>(A_log),
                        static_cast<const T*>(dt_bias), static_cast<float*>(g), static_cast<float*>(beta), Tn, H)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_gdn_l2norm(const void* in, long long ld, void* out_q, void* out_k, long long Tn, int Hk, int D, float eps,
                         float q_scale, int is_f32, void* stream) {
  if (Tn <= 0) return 0;
  if (D & 7) return ixh::fail(ixh::IX_EARG, "gdn_l2norm: D=%d must be a multiple of 8", D);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long warps = Tn * 2 * Hk;
  IX_GDN_DT(is_f32, (gdn_l2norm_kernel<T><<<static_cast<int>((warps + 3) / 4), 128, 0, s>>>(
                        static_cast<const T*>(in), ld, static_cast<T*>(out_q), static_cast<T*>(out_k), Tn, Hk, D, eps, q_scale)));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_gdn_scan(const void* q, const void* k, const void* v, const void* g, const void* beta, const void* chunks,
                       void* state, void* out, int n_chunks, int Hk, int Hv, int DK, int DV, int snapshot_every, int is_f32,
                       void* stream) {
  if (n_chunks <= 0) return 0;
  if (DV > 128 || (DK != 64 && DK != 128)) return ixh::fail(ixh::IX_EARG, "gdn_scan: Dk=%d (64|128), Dv=%d (<=128) unsupported", DK, DV);
  if (Hv % Hk) return ixh::fail(ixh::IX_EARG, "gdn_scan: Hv=%d not a multiple of Hk=%d", Hv, Hk);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid(n_chunks, Hv);
#define IX_SCAN(DK_)                                                                                              \
  IX_GDN_DT(is_f32, (gdn_scan_kernel<T, DK_><<<grid, 128, 0, s>>>(                                                \
                        static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),             \
                        static_cast<const float*>(g), static_cast<const float*>(beta),                            \
                        static_cast<const ScanChunk*>(chunks), static_cast<float*>(state), static_cast<T*>(out), Hk, Hv, DV, \
                        snapshot_every)))
  if (DK == 128) { IX_SCAN(128); } else { IX_SCAN(64); }
#undef IX_SCAN
  IX_CUDA(cudaGetLastError());
  return 0;
}
