// Entry points of the C ABI that are not kernels: version, status text, the
// tuning switches and the read-out of the sticky device status word.
#include <cuda_runtime.h>
#include <string.h>
#include <stdint.h>

#include "../../include/braid_b200.h"
#include "ptx.cuh"

namespace bq {
int quant_set_option(const char* key, long long value);
int gemm_set_option(const char* key, long long value);
}  // namespace bq

extern "C" int bq_version(void) { return 100; }

extern "C" const char* bq_status_string(int status) {
  switch (status) {
    case BQ_OK: return "ok";
    case BQ_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown dtype)";
    case BQ_ERR_UNSUPPORTED: return "unsupported shape, stride or alignment";
    case BQ_ERR_LAUNCH: return "CUDA refused the kernel launch";
    case BQ_ERR_WORKSPACE: return "scratch buffer missing, misaligned or too small";
    case BQ_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
    case BQ_ERR_NO_DRIVER: return "cuTensorMapEncodeTiled is not available from the driver";
    case BQ_ERR_TOO_LARGE: return "size exceeds a fixed capacity";
    default: return "unknown status";
  }
}

extern "C" int bq_set_option(const char* key, int64_t value) {
  if (key == nullptr) return BQ_ERR_BAD_ARG;
  if (bq::quant_set_option(key, value) == BQ_OK) return BQ_OK;
  return bq::gemm_set_option(key, value);
}

extern "C" int bq_read_device_status(void* ws, void* stream, int* status_out) {
  if (ws == nullptr || status_out == nullptr) return BQ_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned int word = 0;
  unsigned int* dev_word = static_cast<unsigned int*>(ws) + 3;
  if (cudaMemcpyAsync(&word, dev_word, sizeof(word), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return BQ_ERR_LAUNCH;
  if (cudaStreamSynchronize(s) != cudaSuccess) return BQ_ERR_LAUNCH;
  if (word != 0) {
    if (cudaMemsetAsync(dev_word, 0, sizeof(word), s) != cudaSuccess) return BQ_ERR_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return BQ_ERR_LAUNCH;
  }
  *status_out = static_cast<int>(word);
  return BQ_OK;
}

extern "C" int bq_enable_peer_access(int peer_device) {
  int dev = -1, can = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return BQ_ERR_LAUNCH; }
  if (peer_device < 0) return BQ_ERR_BAD_ARG;
  if (peer_device == dev) return BQ_OK;
  if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess) {
    (void)cudaGetLastError();
    return BQ_ERR_LAUNCH;
  }
  if (!can) return BQ_ERR_UNSUPPORTED;
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return BQ_ERR_LAUNCH;
  }
  (void)cudaGetLastError();   // "already enabled" is not an error here
  return BQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Buffers that other processes of the node map into their own device's address space
// ---------------------------------------------------------------------------------------------
// The importing side must open the handle with ITS OWN device current: the mapping then belongs
// to that device's context and its kernels may dereference it (peer access is switched on by the
// open).  A mapping opened under the exporting device's context of the importing process is not
// reachable from kernels of another device, whatever peer access says.
extern "C" int bq_peer_alloc(size_t bytes, void** ptr_out, void* handle_out) {
  if (bytes == 0 || ptr_out == nullptr || handle_out == nullptr) return BQ_ERR_BAD_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) { (void)cudaGetLastError(); return BQ_ERR_LAUNCH; }
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    (void)cudaGetLastError();
    (void)cudaFree(p);
    return BQ_ERR_LAUNCH;
  }
  memcpy(handle_out, &h, sizeof(h));
  *ptr_out = p;
  return BQ_OK;
}

extern "C" int bq_peer_free(void* ptr) {
  if (ptr == nullptr) return BQ_ERR_BAD_ARG;
  if (cudaFree(ptr) != cudaSuccess) { (void)cudaGetLastError(); return BQ_ERR_LAUNCH; }
  return BQ_OK;
}

extern "C" int bq_peer_open(const void* handle, void** ptr_out) {
  if (handle == nullptr || ptr_out == nullptr) return BQ_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return BQ_ERR_UNSUPPORTED;
  }
  // a copy through the runtime reports a bad mapping as an error code instead of a kernel fault
  unsigned int probe = 0;
  if (cudaMemcpy(&probe, p, sizeof(probe), cudaMemcpyDeviceToHost) != cudaSuccess) {
    (void)cudaGetLastError();
    (void)cudaIpcCloseMemHandle(p);
    return BQ_ERR_UNSUPPORTED;
  }
  *ptr_out = p;
  return BQ_OK;
}

extern "C" int bq_peer_close(void* ptr) {
  if (ptr == nullptr) return BQ_ERR_BAD_ARG;
  if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) { (void)cudaGetLastError(); return BQ_ERR_LAUNCH; }
  return BQ_OK;
}

#ifdef BQ_PHASES
// ---------------------------------------------------------------------------------------------
// Development build only: the ring the decode-regime kernels stamp their phases into
// ---------------------------------------------------------------------------------------------
static __device__ unsigned long long g_phase_ring[(size_t)bq::kPhaseLaunches * bq::kPhaseCtas * bq::kPhaseWords];
static int g_phase_seq = 0;
static int g_phase_on = 0;

unsigned long long* bq::phase_ring_for_launch(int* seq_out) {
  static unsigned long long* ring = nullptr;
  if (!g_phase_on) return nullptr;
  if (ring == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_phase_ring) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    ring = static_cast<unsigned long long*>(ptr);
  }
  *seq_out = g_phase_seq++;
  return ring;
}

// on = 1 starts numbering launches from 0 again and clears the ring
extern "C" int bq_debug_phases(int on) {
  g_phase_on = on;
  g_phase_seq = 0;
  if (on) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_phase_ring) != cudaSuccess) return BQ_ERR_LAUNCH;
    if (cudaMemset(ptr, 0, sizeof(unsigned long long) * bq::kPhaseLaunches * bq::kPhaseCtas * bq::kPhaseWords) != cudaSuccess)
      return BQ_ERR_LAUNCH;
  }
  return BQ_OK;
}

// copies the whole ring to `out` (kPhaseLaunches * kPhaseCtas * kPhaseWords u64) and returns the
// number of launches numbered so far through *launches_out
extern "C" int bq_debug_read_phases(unsigned long long* out, int* launches_out) {
  if (out == nullptr || launches_out == nullptr) return BQ_ERR_BAD_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) return BQ_ERR_LAUNCH;
  if (cudaMemcpyFromSymbol(out, g_phase_ring, sizeof(unsigned long long) * bq::kPhaseLaunches * bq::kPhaseCtas * bq::kPhaseWords) != cudaSuccess)
    return BQ_ERR_LAUNCH;
  *launches_out = g_phase_seq;
  return BQ_OK;
}
#endif
