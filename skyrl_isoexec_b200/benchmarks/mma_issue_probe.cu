// Micro-benchmark of the 5th-generation tensor core's issue rate: clocks per tcgen05.mma (kind::f16, one K=16 step)
// for several (M, N) with 1, 2 or 4 independent accumulators, and the TMEM lane layout of M=64 and M=128
// accumulators. It explains the floor of the decode-sized GEMMs (one CTA must walk K in K/16 such steps).
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue_probe skyrl_isoexec_b200/benchmarks/mma_issue_probe.cu
//   ./mma_issue_probe
// One CTA, a few microseconds per case; every wait is bounded.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "../csrc/bw_common.cuh"
using namespace bw;

struct Res { long long cycles; int status; };

__global__ void __launch_bounds__(192, 1) probe(int M, int N, int chains, int iters, Res* res, float* dump, int do_dump) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                 // 128 rows x 128 B
  uint8_t* sB = smem + 16384;         // 256 rows x 128 B
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 16384 + 32768);
  uint32_t* holder = reinterpret_cast<uint32_t*>(bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(holder + 1);
  __shared__ int status;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // operands: A[r][0] = r + 1, everything else 0; B[n][0] = 1
  for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  __syncthreads();
  if (threadIdx.x < 128) {
    int r = threadIdx.x;
    uint32_t off = (r / 8) * 1024 + (r % 8) * 128 + ((0 ^ (r % 8)) * 16);
    *reinterpret_cast<__nv_bfloat16*>(sA + off) = __float2bfloat16(float(r + 1));
  }
  for (int n = threadIdx.x; n < 256; n += blockDim.x) {
    uint32_t off = (n / 8) * 1024 + (n % 8) * 128 + ((0 ^ (n % 8)) * 16);
    *reinterpret_cast<__nv_bfloat16*>(sB + off) = __float2bfloat16(1.0f);
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    status = 0;
    mbar_init(smem_u32(&bar[0]), 1);
    fence_mbar_init();
  }
  fence_proxy_async();
  if (warp == 1) {
    tmem_alloc<512>(smem_u32(holder));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *holder;
  // zero the first 128 columns of TMEM (all lanes)
  if (warp >= 2) {
    uint32_t z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) z[i] = 0;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    for (int c = 0; c < 4; ++c) tmem_st_32x32(tmem + lane_off + c * 32, z);
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1 && elect_one()) {
    const uint32_t idesc = make_idesc_bf16(M, N);
    const uint64_t da = make_sw128_desc(smem_u32(sA), 16, 1024);
    const uint64_t db = make_sw128_desc(smem_u32(sB), 16, 1024);
    const int ncols = N < 32 ? 32 : N;
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const int c = i % chains;
      umma_f16_ss(tmem + c * ncols, da + 2 * (i & 3), db + 2 * (i & 3), idesc, i >= chains ? 1u : 0u);
    }
    umma_commit(smem_u32(&bar[0]));
    bool ok = mbar_wait(smem_u32(&bar[0]), 0, abort_flag, &status, ST_TIMEOUT_MISC);
    long long t1 = clock64();
    res->cycles = ok ? (t1 - t0) : -1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (do_dump && warp >= 2) {
    const int quad = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t v[32];
    tmem_ld_32x32(tmem + lane_off, v);
    tmem_ld_wait_dep(v);
    // column 0 and column 1 of every lane
    dump[(quad * 32 + lane) * 2 + 0] = __uint_as_float(v[0]);
    dump[(quad * 32 + lane) * 2 + 1] = __uint_as_float(v[1]);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) res->status = status;
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem);
  }
}

int main() {
  Res* res;
  float* dump;
  cudaMalloc(&res, sizeof(Res));
  cudaMalloc(&dump, 128 * 2 * sizeof(float));
  const int smem = 16384 + 32768 + 1024 + 256;
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  const int shapes[][2] = {{128, 32}, {128, 64}, {128, 128}, {128, 256}, {64, 32}, {64, 64}, {64, 128}, {64, 256}, {128, 16}, {64, 16}, {64, 8}};
  for (auto& s : shapes) {
    for (int chains : {1, 2, 4}) {
      const int ncols = s[1] < 32 ? 32 : s[1];
      if (chains * ncols > 512) continue;
      const int iters = 2048;
      Res h;
      for (int rep = 0; rep < 2; ++rep) {
        probe<<<1, 192, smem>>>(s[0], s[1], chains, iters, res, dump, 0);
        cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { printf("cuda error %s\n", cudaGetErrorString(e)); return 1; }
      }
      cudaMemcpy(&h, res, sizeof(Res), cudaMemcpyDeviceToHost);
      printf("M=%d N=%d chains=%d: %.1f clk per mma (status %d)\n", s[0], s[1], chains, double(h.cycles) / iters, h.status);
      fflush(stdout);
    }
  }
  // layout of an M=64 accumulator: one MMA, D[r][n] = r + 1
  for (int M : {64, 128}) {
    cudaMemset(dump, 0, 128 * 2 * sizeof(float));
    probe<<<1, 192, smem>>>(M, 32, 1, 1, res, dump, 1);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("cuda error %s\n", cudaGetErrorString(e)); return 1; }
    std::vector<float> h(256);
    cudaMemcpy(h.data(), dump, 256 * sizeof(float), cudaMemcpyDeviceToHost);
    printf("M=%d accumulator, value at (lane, col0):", M);
    for (int l = 0; l < 128; ++l) printf(" %d:%g", l, h[l * 2]);
    printf("\n");
  }
  return 0;
}
