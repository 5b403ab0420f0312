// Trainer -> rollout weight delivery with the layout change done in flight.
//
// The trainer keeps its tensor-parallel shard of every parameter in symmetric (peer-mapped) memory. A rollout rank
// whose engine uses another tensor-parallel degree needs, for each parameter, a few rectangular pieces of a few
// trainer ranks' shards (whole row blocks of column-parallel weights, column blocks of row-parallel ones). This kernel
// executes a list of such pieces in ONE launch: it reads every piece from wherever it lives (this GPU's memory or a
// peer's, plain ld.global over NVLink; no TMA touches peer memory) and writes it to its place in the engine's flat
// parameter buffer, optionally rounding an fp32 source (optimizer master weights) to bf16 on the way. No staging bucket,
// no all-gather of full tensors: the bytes that cross NVLink are exactly the bytes the engine shard is made of.
//
// The kernel waits on nothing: the caller orders it against the trainer's update and the engine's next forward with
// host barriers over the group, so there is no flag to spin on.
//
// Reference behaviour: the TP reshard of ISO/sync/native_weight_sync.py:64-125,237-298 and the CUDA-IPC transfer of
// B/weight_sync/cuda_ipc_strategy.py:242-264, which go through full-tensor gathers and a packed staging buffer.
#include <cuda_bf16.h>

#include "host_util.h"

namespace {

struct ReshardDesc {
  const char* src;      // first byte of the piece in the source shard
  char* dst;            // first byte of the piece in the destination shard
  long long rows;       // number of rows of the piece
  long long row_bytes;  // bytes per row of the piece, counted in DESTINATION bytes
  long long src_pitch;  // bytes between rows in the source
  long long dst_pitch;  // bytes between rows in the destination
  int src_f32;          // 1: the source holds fp32 and is rounded (RNE) to bf16; row_bytes still counts bf16 bytes
  int pad;
};

__device__ __forceinline__ unsigned pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&h);
}

__global__ void __launch_bounds__(256) reshard_pull_kernel(const ReshardDesc* __restrict__ descs, int n_desc) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthr = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int d = 0; d < n_desc; ++d) {
    const ReshardDesc c = descs[d];
    const bool vec = ((reinterpret_cast<unsigned long long>(c.src) | reinterpret_cast<unsigned long long>(c.dst) |
                       static_cast<unsigned long long>(c.row_bytes) | static_cast<unsigned long long>(c.src_pitch) |
                       static_cast<unsigned long long>(c.dst_pitch)) & 15ull) == 0;
    if (vec) {
      const long long rv = c.row_bytes >> 4;            // 16-byte vectors per row (8 bf16)
      const long long total = rv * c.rows;
      for (long long v = tid; v < total; v += nthr) {
        const long long r = v / rv, k = v - r * rv;
        uint4* o = reinterpret_cast<uint4*>(c.dst + r * c.dst_pitch) + k;
        if (c.src_f32) {
          const float4* s = reinterpret_cast<const float4*>(c.src + r * c.src_pitch) + 2 * k;
          const float4 a = s[0], b = s[1];
          uint4 w;
          w.x = pack2(a.x, a.y);
          w.y = pack2(a.z, a.w);
          w.z = pack2(b.x, b.y);
          w.w = pack2(b.z, b.w);
          *o = w;
        } else {
          *o = *(reinterpret_cast<const uint4*>(c.src + r * c.src_pitch) + k);
        }
      }
    } else {
      const long long re = c.row_bytes >> 1;            // bf16 elements per row
      const long long total = re * c.rows;
      for (long long v = tid; v < total; v += nthr) {
        const long long r = v / re, k = v - r * re;
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(c.dst + r * c.dst_pitch) + k;
        if (c.src_f32)
          *o = __float2bfloat16_rn(*(reinterpret_cast<const float*>(c.src + r * c.src_pitch) + k));
        else
          *o = *(reinterpret_cast<const __nv_bfloat16*>(c.src + r * c.src_pitch) + k);
      }
    }
  }
}

}  // namespace

// descs: DEVICE array of n_desc records laid out as ReshardDesc (56 bytes each). Every address is valid in this
// process on the current device (local memory or peer-mapped symmetric memory). Pieces must not overlap in the
// destination. Returns 0 or an error code.
IX_API int ix_reshard_pull(const void* descs, int n_desc, void* stream) {
  if (n_desc < 0) return ixh::fail(ixh::IX_EARG, "reshard_pull: negative descriptor count");
  if (n_desc == 0) return 0;
  if (descs == nullptr) return ixh::fail(ixh::IX_EARG, "reshard_pull: null descriptor table");
  reshard_pull_kernel<<<148 * 4, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const ReshardDesc*>(descs), n_desc);
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_reshard_desc_bytes() { return static_cast<int>(sizeof(ReshardDesc)); }
