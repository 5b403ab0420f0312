// Collectives over NVLink peer memory, issued from our own kernels (no NCCL on these paths).
//
// Every rank owns a buffer in symmetric memory (same size on every rank, mapped into every
// rank's address space) and a small flag array that its peers write into. A collective is one
// kernel launch per rank:
//   1. CTA 0 publishes "my data of epoch e is in place" to every peer (fence + st.release.sys into
//      the peer's flag array, slot = my rank);
//   2. every CTA waits until its own flag array shows epoch e from all ranks (ld.acquire.sys on
//      LOCAL memory, bounded by a wall-clock limit: a missing peer yields a status code, not a hang);
//   3. every CTA reads its slice of all peers' buffers with plain loads over NVLink and folds the
//      partials in a FIXED order: the balanced tree over ranks, lower rank on the left, all in fp32.
//      This is the upper part of the same tree the leaf GEMM folds locally, so any tensor-parallel
//      degree dividing the leaf count produces identical bits (ISO/ops/collectives/pik/plan.py:20-36);
//   4. results are stored locally (all-reduce) or pushed to the owner (reduce-scatter phase).
// Buffers are double-buffered by epoch parity. A rank cannot finish the collective of epoch e+1
// before every peer has started it, and a peer starts it only after finishing epoch e, so a buffer
// is never overwritten (by the producer of epoch e+2) while a peer still reads epoch e.
//
// No TMA is used on peer memory: remote data arrives by ld.global.
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kMaxRanks = 16;

struct PeerTable {
  const void* buf[kMaxRanks];     // each rank's data buffer (already offset to the epoch's half)
  uint32_t* flags[kMaxRanks];     // each rank's flag array [kMaxRanks]
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Publish epoch to all peers, then wait for all peers. Returns false if the wait ran out.
__device__ bool handshake(const PeerTable& pt, int rank, int W, uint32_t epoch, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(pt.flags[threadIdx.x] + rank, epoch);
  }
  if (threadIdx.x < W) {
    const uint32_t* mine = pt.flags[rank] + threadIdx.x;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
      if (((++it) & 0x3f) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
        if (status) atomicCAS(status, 0, ST_TIMEOUT_FLAG);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

template <int W>
__device__ __forceinline__ float4 tree_fold(float4 (&v)[W]) {
#pragma unroll
  for (int stride = 1; stride < W; stride <<= 1)
#pragma unroll
    for (int i = 0; i < W; i += 2 * stride) {
      v[i].x = __fadd_rn(v[i].x, v[i + stride].x);
      v[i].y = __fadd_rn(v[i].y, v[i + stride].y);
      v[i].z = __fadd_rn(v[i].z, v[i + stride].z);
      v[i].w = __fadd_rn(v[i].w, v[i + stride].w);
    }
  return v[0];
}

// out[i] = tree over ranks of buf_r[i], i in [lo, hi) (in float4 units). OUT: 0 fp32, 1 bf16.
// dst_rank < 0: store to `out` locally; otherwise store fp32 into rank dst_rank's buffer (reduce-scatter).
template <int W, int OUT>
__global__ void __launch_bounds__(256)
tree_reduce_kernel(PeerTable pt, int rank, uint32_t epoch, long long lo4, long long hi4, void* __restrict__ out,
                   long long out_off4, int* __restrict__ status) {
  if (!handshake(pt, rank, W, epoch, status)) return;
  for (long long i = lo4 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 v[W];
#pragma unroll
    for (int r = 0; r < W; ++r) v[r] = reinterpret_cast<const float4*>(pt.buf[r])[i];
    const float4 s = tree_fold<W>(v);
    if (OUT == 0) {
      reinterpret_cast<float4*>(out)[i - lo4 + out_off4] = s;
    } else {
      uint2 w;
      w.x = pack_bf2(s.x, s.y);
      w.y = pack_bf2(s.z, s.w);
      reinterpret_cast<uint2*>(out)[i - lo4 + out_off4] = w;
    }
  }
}

// all-gather phase of the two-shot all-reduce: out[slice of rank r] = buf_r[slice of rank r]
template <int W>
__global__ void __launch_bounds__(256)
gather_slices_kernel(PeerTable pt, int rank, uint32_t epoch, long long slice4, long long n4, float* __restrict__ out,
                     int* __restrict__ status) {
  if (!handshake(pt, rank, W, epoch, status)) return;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    int r = static_cast<int>(i / slice4);
    if (r >= W) r = W - 1;
    reinterpret_cast<float4*>(out)[i] = reinterpret_cast<const float4*>(pt.buf[r])[i];
  }
}

// Descriptor-driven copy with optional fp32 -> bf16 cast: the trainer -> rollout weight push. One launch
// moves every (source range, destination range) pair; destinations may be peer memory.
struct CopyDesc {
  const void* src;
  void* dst;
  long long n;       // elements
  int src_f32;       // 1: source is fp32 and is rounded to bf16 on the way; 0: bf16 -> bf16
  int pad;
};

__global__ void __launch_bounds__(256) push_copy_kernel(const CopyDesc* __restrict__ descs, int n_desc) {
  for (int d = blockIdx.y; d < n_desc; d += gridDim.y) {
    const CopyDesc c = descs[d];
    const long long n8 = c.n >> 3;
    if (c.src_f32) {
      const float4* s = reinterpret_cast<const float4*>(c.src);
      uint4* o = reinterpret_cast<uint4*>(c.dst);
      for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
           i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float4 a = s[2 * i], b = s[2 * i + 1];
        uint4 w;
        w.x = pack_bf2(a.x, a.y);
        w.y = pack_bf2(a.z, a.w);
        w.z = pack_bf2(b.x, b.y);
        w.w = pack_bf2(b.z, b.w);
        o[i] = w;
      }
      for (long long i = (n8 << 3) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < c.n;
           i += static_cast<long long>(gridDim.x) * blockDim.x)
        reinterpret_cast<__nv_bfloat16*>(c.dst)[i] = f2bf(reinterpret_cast<const float*>(c.src)[i]);
    } else {
      const uint4* s = reinterpret_cast<const uint4*>(c.src);
      uint4* o = reinterpret_cast<uint4*>(c.dst);
      for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
           i += static_cast<long long>(gridDim.x) * blockDim.x)
        o[i] = s[i];
      for (long long i = (n8 << 3) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < c.n;
           i += static_cast<long long>(gridDim.x) * blockDim.x)
        reinterpret_cast<__nv_bfloat16*>(c.dst)[i] = reinterpret_cast<const __nv_bfloat16*>(c.src)[i];
    }
  }
}

// barrier-only kernel: publish + wait (used to order phases and by the bounded-wait test)
__global__ void handshake_kernel(PeerTable pt, int rank, int W, uint32_t epoch, int* status) {
  handshake(pt, rank, W, epoch, status);
}

int fill_table(PeerTable* pt, const long long* bufs, const long long* flags, int W) {
  if (W < 1 || W > kMaxRanks) return ixh::fail(ixh::IX_EARG, "peer collective: world size %d unsupported (1..%d)", W, kMaxRanks);
  for (int r = 0; r < W; ++r) {
    pt->buf[r] = reinterpret_cast<const void*>(bufs[r]);
    pt->flags[r] = reinterpret_cast<uint32_t*>(flags[r]);
  }
  return 0;
}

inline int grid_for(long long n4) {
  long long g = (n4 + 255) / 256;
  if (g > 148 * 4) g = 148 * 4;
  return g < 1 ? 1 : static_cast<int>(g);
}

}  // namespace

// bufs[r], flags[r]: device addresses (as integers) of rank r's data buffer and flag array, as mapped in THIS
// process. n: fp32 elements (multiple of 4). [lo, hi): element range this call reduces (multiple of 4 each).
// out: local destination (fp32 or bf16), written from element out_off.
IX_API int ix_peer_tree_reduce(const long long* bufs, const long long* flags, int rank, int W, unsigned epoch, long long lo,
                               long long hi, void* out, long long out_off, int out_bf16, void* stream) {
  if ((lo & 3) || (hi & 3) || (out_off & 3) || hi < lo) return ixh::fail(ixh::IX_EARG, "peer_tree_reduce: ranges must be multiples of 4");
  PeerTable pt;
  int rc = fill_table(&pt, bufs, flags, W);
  if (rc) return rc;
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long lo4 = lo >> 2, hi4 = hi >> 2, off4 = out_off >> 2;
  const int grid = grid_for(hi4 - lo4);
  int* st = ixh::status_word(dev);
#define IX_TR(W_)                                                                                                   \
  case W_:                                                                                                          \
    if (out_bf16) tree_reduce_kernel<W_, 1><<<grid, 256, 0, s>>>(pt, rank, epoch, lo4, hi4, out, off4, st);          \
    else tree_reduce_kernel<W_, 0><<<grid, 256, 0, s>>>(pt, rank, epoch, lo4, hi4, out, off4, st);                   \
    break;
  switch (W) {
    IX_TR(1) IX_TR(2) IX_TR(4) IX_TR(8) IX_TR(16)
    default:
      return ixh::fail(ixh::IX_EARG, "peer_tree_reduce: world size %d must be a power of two <= 16", W);
  }
#undef IX_TR
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_peer_gather_slices(const long long* bufs, const long long* flags, int rank, int W, unsigned epoch, long long slice,
                                 long long n, void* out, void* stream) {
  if ((slice & 3) || (n & 3)) return ixh::fail(ixh::IX_EARG, "peer_gather_slices: sizes must be multiples of 4");
  PeerTable pt;
  int rc = fill_table(&pt, bufs, flags, W);
  if (rc) return rc;
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int* st = ixh::status_word(dev);
  const int grid = grid_for(n >> 2);
#define IX_GS(W_) case W_: gather_slices_kernel<W_><<<grid, 256, 0, s>>>(pt, rank, epoch, slice >> 2, n >> 2, static_cast<float*>(out), st); break;
  switch (W) {
    IX_GS(1) IX_GS(2) IX_GS(4) IX_GS(8) IX_GS(16)
    default:
      return ixh::fail(ixh::IX_EARG, "peer_gather_slices: world size %d must be a power of two <= 16", W);
  }
#undef IX_GS
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_peer_handshake(const long long* flags, int rank, int W, unsigned epoch, void* stream) {
  PeerTable pt;
  long long dummy[kMaxRanks] = {0};
  int rc = fill_table(&pt, dummy, flags, W);
  if (rc) return rc;
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  handshake_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pt, rank, W, epoch, ixh::status_word(dev));
  IX_CUDA(cudaGetLastError());
  return 0;
}

// descs: device array of {src, dst, n, src_f32} records (see CopyDesc); all ranges 16-byte aligned.
IX_API int ix_push_copy(const void* descs, int n_desc, void* stream) {
  if (n_desc <= 0) return 0;
  dim3 grid(148, n_desc < 64 ? n_desc : 64);
  push_copy_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const CopyDesc*>(descs), n_desc);
  IX_CUDA(cudaGetLastError());
  return 0;
}
