// Expert-parallel dispatch over NVLink peer memory (no NCCL, no host round trip).
//
// Every rank holds E/W experts. For one MoE layer a rank
//   1. ep_counts_kernel   publishes its per-expert row counts into every rank's count table, waits for all
//                         ranks' counts (bounded), and derives on the device: where each of its expert groups
//                         starts in the owner's receive buffer, and the row offsets of its OWN experts' groups
//                         (rows ordered by expert, then source rank, then the source's order: the same order a
//                         single-rank run uses, although the order never matters to a row's value);
//   2. ep_dispatch_kernel pushes each dispatch row (activation row, gate weight, and WHERE its result must come back
//                         to: source rank and row) straight into the owner's receive buffers with peer stores;
//   3. (handshake)        then the owner runs the grouped expert GEMMs (moe_grouped_gemm.cu); the second one
//                         scatters its fp32 output rows to the recorded addresses, i.e. the return all-to-all
//                         happens in the GEMM epilogue;
//   4. (handshake)        and each rank sums its tokens' rows in ascending expert order locally.
// The reference moves rows with two NCCL all-to-alls around per-expert library GEMMs
// (ISO/ops/moe/moe_batch_invariant.py:744-887).
#include "bw_common.cuh"
#include "host_util.h"

namespace {
using namespace bw;

constexpr int kMaxRanks = 16;
constexpr int kMaxExperts = 512;

struct EpPeers {
  int* cnt[kMaxRanks];            // rank d's count table [W][E]
  uint32_t* flags[kMaxRanks];     // rank d's flag array (>= W entries at flag_off)
  __nv_bfloat16* xbuf[kMaxRanks]; // rank d's receive buffer for activation rows [cap][K]
  float* wbuf[kMaxRanks];         // gate weights [cap]
  long long* dstbuf[kMaxRanks];   // return addresses [cap]
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// counts: int64 [E] local rows per (global) expert. Outputs (local device memory):
//   send_base [E]      first row of this rank's group for expert e in the owner's buffers
//   local_off [E+1]    prefix of `counts` (where expert e's rows start in this rank's dispatch order)
//   own_offs [E/W + 1] row offsets of this rank's own experts in its receive buffers (all sources)
__global__ void __launch_bounds__(512)
ep_counts_kernel(EpPeers pp, const long long* __restrict__ counts, int rank, int W, int E, uint32_t epoch, int flag_off, int cap,
                 int* __restrict__ send_base, int* __restrict__ local_off, int* __restrict__ own_offs, int* __restrict__ status) {
  __shared__ int s_cnt[kMaxRanks * kMaxExperts / 4];   // W*E <= 2048 entries
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  const int e_loc = E / W;
  if (tid == 0) s_ok = 1;
  for (int e = tid; e < E; e += blockDim.x) {
    const int c = static_cast<int>(counts[e]);
    for (int d = 0; d < W; ++d) pp.cnt[d][rank * E + e] = c;
  }
  __syncthreads();
  if (tid < W) {
    __threadfence_system();
    st_release_sys(pp.flags[tid] + flag_off + rank, epoch);
    const uint32_t* mine = pp.flags[rank] + flag_off + tid;
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
  if (!s_ok) return;
  for (int i = tid; i < W * E; i += blockDim.x) s_cnt[i] = pp.cnt[rank][i];
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    const int o = e / e_loc;
    int base = 0;
    for (int e2 = o * e_loc; e2 < e; ++e2)
      for (int s = 0; s < W; ++s) base += s_cnt[s * E + e2];
    for (int s = 0; s < rank; ++s) base += s_cnt[s * E + e];
    send_base[e] = base;
    int lo = 0;
    for (int e2 = 0; e2 < e; ++e2) lo += s_cnt[rank * E + e2];
    local_off[e] = lo;
    if (e == E - 1) local_off[E] = lo + s_cnt[rank * E + e];
  }
  for (int j = tid; j <= e_loc; j += blockDim.x) {
    int off = 0;
    for (int e2 = rank * e_loc; e2 < rank * e_loc + j; ++e2)
      for (int s = 0; s < W; ++s) off += s_cnt[s * E + e2];
    own_offs[j] = off;
    if (j == e_loc && off > cap && status) atomicCAS(status, 0, ST_BAD_ARG);   // receive buffer too small for this routing
  }
}

// One warp per dispatch row i (this rank's rows sorted by expert): x[tok_of_row[i]] -> owner's xbuf[dest], with its
// gate weight and the address the expert output row has to be written to.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(EpPeers pp, const __nv_bfloat16* __restrict__ x, long long ldx, const long long* __restrict__ tok_of_row,
                   const int* __restrict__ expert_of_row, const float* __restrict__ w_rows, const int* __restrict__ send_base,
                   const int* __restrict__ local_off, int rank, int R, int K, int E, int W, int cap) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int e_loc = E / W;
  for (int i = warp; i < R; i += nwarps) {
    const int e = expert_of_row[i];
    const int o = e / e_loc;
    const int dest = send_base[e] + (i - local_off[e]);
    if (dest >= cap) continue;   // reported by ep_counts_kernel; never write past the buffer
    const uint4* src = reinterpret_cast<const uint4*>(x + tok_of_row[i] * ldx);
    uint4* dst = reinterpret_cast<uint4*>(pp.xbuf[o] + static_cast<size_t>(dest) * K);
    for (int c = lane; c < K / 8; c += 32) dst[c] = src[c];
    if (lane == 0) {
      pp.wbuf[o][dest] = w_rows[i];
      pp.dstbuf[o][dest] = (static_cast<long long>(rank) << 40) | i;   // (source rank, source row); the owner turns it into an address
    }
  }
}

// The owner's view of the return addresses: dst[j] = rows buffer of the source rank (as mapped HERE) + source row * row_bytes.
struct RowsTable {
  long long base[kMaxRanks];
};
__global__ void __launch_bounds__(256)
ep_resolve_dst_kernel(long long* __restrict__ dst, RowsTable rt, const int* __restrict__ own_offs, int e_loc, long long row_bytes) {
  const int total = own_offs[e_loc];
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < total; j += gridDim.x * blockDim.x) {
    const long long v = dst[j];
    dst[j] = rt.base[v >> 40] + (v & ((1ll << 40) - 1)) * row_bytes;
  }
}

int fill(EpPeers* pp, const long long* cnt, const long long* flags, const long long* xbuf, const long long* wbuf,
         const long long* dstbuf, int W) {
  if (W < 1 || W > kMaxRanks) return ixh::fail(ixh::IX_EARG, "ep: world size %d unsupported", W);
  for (int r = 0; r < W; ++r) {
    pp->cnt[r] = reinterpret_cast<int*>(cnt[r]);
    pp->flags[r] = reinterpret_cast<uint32_t*>(flags[r]);
    pp->xbuf[r] = xbuf ? reinterpret_cast<__nv_bfloat16*>(xbuf[r]) : nullptr;
    pp->wbuf[r] = wbuf ? reinterpret_cast<float*>(wbuf[r]) : nullptr;
    pp->dstbuf[r] = dstbuf ? reinterpret_cast<long long*>(dstbuf[r]) : nullptr;
  }
  return 0;
}

}  // namespace

IX_API int ix_ep_counts(const long long* cnt_ptrs, const long long* flag_ptrs, const void* counts, int rank, int W, int E,
                        unsigned epoch, int flag_off, int cap, void* send_base, void* local_off, void* own_offs, void* stream) {
  if (E % W || E > kMaxExperts || W * E > kMaxRanks * kMaxExperts / 4)
    return ixh::fail(ixh::IX_EARG, "ep_counts: E=%d, W=%d unsupported (E %% W == 0, W*E <= 2048)", E, W);
  EpPeers pp;
  int rc = fill(&pp, cnt_ptrs, flag_ptrs, nullptr, nullptr, nullptr, W);
  if (rc) return rc;
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  ep_counts_kernel<<<1, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const long long*>(counts), rank, W, E, epoch, flag_off, cap, static_cast<int*>(send_base),
      static_cast<int*>(local_off), static_cast<int*>(own_offs), ixh::status_word(dev));
  IX_CUDA(cudaGetLastError());
  return 0;
}

IX_API int ix_ep_dispatch(const long long* cnt_ptrs, const long long* flag_ptrs, const long long* xbuf, const long long* wbuf,
                          const long long* dstbuf, const void* x, long long ldx, const void* tok_of_row, const void* expert_of_row,
                          const void* w_rows, const void* send_base, const void* local_off, int rank, int R, int K, int E, int W,
                          int cap, void* stream) {
  if (R <= 0) return 0;
  if ((K & 7) || (ldx & 7)) return ixh::fail(ixh::IX_EARG, "ep_dispatch: K and ldx must be multiples of 8");
  EpPeers pp;
  int rc = fill(&pp, cnt_ptrs, flag_ptrs, xbuf, wbuf, dstbuf, W);
  if (rc) return rc;
  int grid = (R + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  ep_dispatch_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const long long*>(tok_of_row),
      static_cast<const int*>(expert_of_row), static_cast<const float*>(w_rows), static_cast<const int*>(send_base),
      static_cast<const int*>(local_off), rank, R, K, E, W, cap);
  IX_CUDA(cudaGetLastError());
  return 0;
}

// dst: this rank's return-address buffer as filled by the sources; rows_ptrs[r]: rank r's result buffer as mapped in THIS process.
IX_API int ix_ep_resolve_dst(void* dst, const long long* rows_ptrs, const void* own_offs, int e_loc, int W, long long row_bytes,
                             int cap, void* stream) {
  if (W < 1 || W > kMaxRanks) return ixh::fail(ixh::IX_EARG, "ep_resolve_dst: world size %d unsupported", W);
  RowsTable rt;
  for (int r = 0; r < kMaxRanks; ++r) rt.base[r] = r < W ? rows_ptrs[r] : 0;
  int grid = (cap + 255) / 256;
  if (grid > 148 * 4) grid = 148 * 4;
  if (grid < 1) grid = 1;
  ep_resolve_dst_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<long long*>(dst), rt,
                                                                                  static_cast<const int*>(own_offs), e_loc, row_bytes);
  IX_CUDA(cudaGetLastError());
  return 0;
}
