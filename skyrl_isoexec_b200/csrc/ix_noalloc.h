// Allocation-free entry point of the native library. It has no counterpart in the reference
// framework; it exists for callers of THIS library that are not allowed to allocate device
// memory at the moment they need a fixed-order sum:
//
//   * code that runs while another component owns the allocator, e.g. between the rollout
//     engine's sleep and the trainer's backload in a colocated run, when every free byte is
//     spoken for and a cudaMalloc could fail or fragment the pool;
//   * hosts that embed the library without PyTorch (a C or ctypes caller has no caching
//     allocator to draw scratch from) and do not want a cudaMalloc/cudaFree pair, which
//     synchronises the device, on their step path;
//   * monitoring hooks (gradient-norm or checksum probes) that must not perturb the memory
//     picture they are observing.
//
// ix_reduce_sum_noalloc computes exactly what ix_reduce_sum computes - out[0] (+)= sum of
// in[0..n), or the sum of squares, in an order that depends only on n - but keeps the stage-1
// partial sums in a fixed array that is part of the library image instead of in memory the
// caller passes in. The caller still provides the input and the one-float output.
//
// Limits and rules:
//   * at most IX_NOALLOC_MAX_PARTIALS * 4096 input elements (268,435,456); a longer input is
//     rejected with a non-zero return code and a message in ix_last_error();
//   * the array costs IX_NOALLOC_MAX_PARTIALS * 4 bytes (256 KiB) of device memory on every GPU
//     that loads the library, held until the process exits;
//   * the first call on a device looks up the array's device address (no allocation); make that
//     first call before starting any stream capture on that device;
//   * all calls on a device share the one array, and it keeps the last call's partials. Calls
//     that may run at the same time on the GPU (different streams without an ordering between
//     them) race on it: order them on one stream or with events. Nothing needs clearing
//     between calls, because a call only reads back the partials it has just written;
//   * the array used is the one of the CURRENT device (cudaGetDevice at the time of the call): make the device that
//     `stream` belongs to current before calling, as for any launch on that stream;
//   * it calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once

#define IX_NOALLOC_MAX_PARTIALS 65536

#ifdef __cplusplus
extern "C" {
#endif

// Largest n the entry point accepts.
long long ix_reduce_sum_noalloc_max_elems(void);

// in: n elements, dtype 0 = bf16, 1 = fp32 (device pointer). square != 0 sums squares.
// out: one float (device pointer); accumulate != 0 adds to it instead of overwriting.
// stream: cudaStream_t. Returns 0 on success.
int ix_reduce_sum_noalloc(const void* in, long long n, int dtype, int square, void* out, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
