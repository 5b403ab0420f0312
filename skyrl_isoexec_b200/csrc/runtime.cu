// Library runtime: per-device status word, last-error string, version.
#include <stdarg.h>

#include "host_util.h"

namespace ixh {

static int* g_status[64] = {nullptr};
static std::mutex g_status_mu;

int* status_word(int device) {
  if (device < 0 || device >= 64) return nullptr;
  if (g_status[device]) return g_status[device];
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status[device]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(int));
    g_status[device] = p;
  }
  return g_status[device];
}

}  // namespace ixh

IX_API const char* ix_last_error() { return ixh::last_error_buf(); }

IX_API int ix_version() { return 1; }

// Allocate the status word of the current device up front (call once per device before
// any stream capture, since the first use would otherwise allocate inside the capture).
IX_API int ix_init() {
  int dev = 0;
  IX_CUDA(cudaGetDevice(&dev));
  return ixh::status_word(dev) ? 0 : ixh::fail(ixh::IX_EDRV, "could not allocate status word");
}

// Read (and clear) the kernel status word of the current device. Synchronises the device.
// 0 = every kernel since the last read finished without a bounded wait running out.
IX_API int ix_read_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  int* p = ixh::status_word(dev);
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// Device pointer of the status word (for kernels launched from other libraries/tests).
IX_API void* ix_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  return ixh::status_word(dev);
}

namespace ixh {
static int g_pdl = 1;
bool pdl_enabled() { return g_pdl != 0; }
}  // namespace ixh

// 1 (default): kernels that support it are launched with programmatic stream serialization; 0: plain stream order.
IX_API int ix_set_pdl(int on) {
  ixh::g_pdl = on ? 1 : 0;
  return 0;
}

// Let kernels of the current device load and store memory that lives on `peer_device` (another GPU of this node, for
// instance a buffer of another process mapped through CUDA IPC, which is opened in the context of the device that owns
// it). A per-process setting of the CUDA context; nothing on the GPU outlasts the process. Returns 0 when access is on
// (or was on already), a negative code when the two devices cannot reach each other.
IX_API int ix_enable_peer_access(int peer_device) {
  int cur = 0;
  IX_CUDA(cudaGetDevice(&cur));
  if (cur == peer_device) return 0;
  int can = 0;
  IX_CUDA(cudaDeviceCanAccessPeer(&can, cur, peer_device));
  if (!can) return ixh::fail(ixh::IX_EARG, "device %d cannot access device %d", cur, peer_device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();   // not an error: clear the sticky code
    return 0;
  }
  if (e != cudaSuccess) return ixh::cuda_fail(e, "cudaDeviceEnablePeerAccess");
  return 0;
}

// Where does `ptr` live? Returns the device ordinal of a device allocation, -1 for anything else (host memory, an
// address CUDA does not know). Never dereferences the pointer.
IX_API int ix_pointer_device(const void* ptr) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return a.type == cudaMemoryTypeDevice ? a.device : -1;
}

// Map a buffer that another process of this node exported with cudaIpcGetMemHandle. The mapping is made with the
// CALLER's current device current, with lazy peer access, so that kernels of this device may store into memory that
// lives on the exporting process's GPU. handle: the 64 bytes of a cudaIpcMemHandle_t. Returns 0 and the mapped base
// address in *out.
IX_API int ix_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  IX_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}
IX_API int ix_ipc_close(void* base) {
  IX_CUDA(cudaIpcCloseMemHandle(base));
  return 0;
}
