// Host-side helpers shared by the launchers: error strings, per-device status word,
// and TMA tensor-map encoding (driver entry point resolved at run time so the
// library links without libcuda and loads on a CPU-only box).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#define IX_API extern "C" __attribute__((visibility("default")))

namespace ixh {

// Return codes of every exported launcher: 0 ok, >0 cudaError_t, <0 argument error.
enum : int { IX_OK = 0, IX_EARG = -1, IX_EDRV = -2, IX_ESIZE = -3 };

inline char* last_error_buf() {
  static thread_local char buf[512];
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}
inline int cuda_fail(cudaError_t e, const char* what) {
  snprintf(last_error_buf(), 512, "%s: %s", what, cudaGetErrorString(e));
  return static_cast<int>(e) > 0 ? static_cast<int>(e) : IX_EDRV;
}
#define IX_CUDA(call)                                  \
  do {                                                 \
    cudaError_t _e = (call);                           \
    if (_e != cudaSuccess) return ixh::cuda_fail(_e, #call); \
  } while (0)

// Launch with programmatic stream serialization (see pdl_wait / pdl_launch_dependents in bw_common.cuh): the kernel may
// begin while the previous kernel of the stream drains. Only for kernels that call pdl_wait() before touching anything
// a predecessor writes. ix_set_pdl(0) turns the attribute off process-wide (plain stream order).
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tiled map over a row-major tensor of `rank` dims (dims[0] innermost), 128B swizzle.
// strides_bytes[i] is the stride of dim i+1. Returns 0 or an error code.
inline int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(IX_EDRV, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(IX_EARG, "TMA base not 16-byte aligned");
  cuuint64_t d[5], s[5];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      s[i] = strides_bytes[i];
      if (s[i] % 16 != 0) return fail(IX_EARG, "TMA stride %d (%llu B) not a multiple of 16", i, (unsigned long long)s[i]);
    }
  }
  CUresult r = fn(out, dt, rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    // a thread that has made no runtime call yet (an autograd worker's first op) has no context bound: bind the
    // device's primary context and encode again
    cudaFree(nullptr);
    r = fn(out, dt, rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return fail(IX_EDRV, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return IX_OK;
}

// 2D bf16 row-major [rows, cols] with row stride ld (elements); box = [box_rows, 64 cols].
inline int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                             uint32_t box_rows, uint32_t box_cols = 64) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld * 2};
  uint32_t box[2] = {box_cols, box_rows};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box);
}

// Per-device status word (device memory, 64 ints) that kernels write error codes into.
int* status_word(int device);  // defined in runtime.cu

}  // namespace ixh
