// Grid-wide NaN-propagating max of |x| for the quantizer kernels: CTA reduction, one atomicMax
// per CTA on the float's bit pattern, a released arrival counter, and a BOUNDED polled wait.
// All CTAs of the grid must be co-resident (the launchers size grids accordingly).
#pragma once
#include <cuda_runtime.h>

#include "ptx.cuh"
#include "quant_device.cuh"

namespace bq {
namespace qd {

// Scratch words shared by all quantizer kernels (16 bytes, zero between launches).
struct QuantWs {
  unsigned int amax_bits;  // running max of |x| as a float bit pattern
  unsigned int arrive;     // CTAs that published their max
  unsigned int depart;     // CTAs that consumed the global max
  unsigned int status;     // sticky: non-zero once a bounded wait ran out
};

// CTA-wide max, then the grid-wide exchange.  Returns the global amax to every
// thread.  A single-CTA grid never touches global memory here.  Thread 0 of every
// CTA of a multi-CTA grid owes the scratch a grid_depart() call afterwards; that
// part is kept off the critical path on purpose.
__device__ __forceinline__ float grid_amax(float m, QuantWs* ws) {
  __shared__ float s_warp[32];
  __shared__ float s_amax;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, off));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) s_warp[warp] = m;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    float w = (lane < nwarps) ? s_warp[lane] : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) w = nan_max(w, __shfl_xor_sync(0xffffffffu, w, off));
    if (lane == 0) {
      if (gridDim.x == 1) {
        s_amax = w;
      } else {
        // |x| >= 0 or NaN with the sign cleared: the unsigned order of the bit
        // patterns is the order of the values, NaN on top.  The max is published
        // first; the release on the counter orders it before the arrival.
        atomicMax(&ws->amax_bits, __float_as_uint(w));
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&ws->arrive) : "memory");
        // amax word and arrival counter sit in one aligned 8-byte pair: one
        // acquire load sees both
        unsigned int amax_bits = 0, arrived = 0;
        const long long t0 = clock64();
        bool ok = true;
        for (;;) {
          asm volatile("ld.acquire.gpu.global.v2.u32 {%0, %1}, [%2];"
                       : "=r"(amax_bits), "=r"(arrived)
                       : "l"(ws)
                       : "memory");
          if (arrived >= gridDim.x) break;
          if (clock64() - t0 > bq::kSpinLimitCycles) { ok = false; break; }
        }
        if (!ok) atomicExch(&ws->status, (unsigned int)bq::kErrDeviceWait);
        s_amax = __uint_as_float(amax_bits);
      }
    }
  }
  __syncthreads();
  return s_amax;
}

// Column-parallel form: every CTA waits (bounded, thread 0 polls with a system-scope acquire)
// until the arrival counter has advanced by `count` beyond *seen -- i.e. until every rank's push
// launch has stored its share of the buffer this kernel is about to read.  *seen is advanced by
// grid_wait_done() once every CTA has read it.
__device__ __forceinline__ void grid_wait_arrivals(const unsigned int* flag, const unsigned int* seen,
                                                   unsigned int count, QuantWs* ws) {
  if (threadIdx.x == 0) {
    unsigned int base;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(base) : "l"(seen) : "memory");
    const unsigned int target = base + count;
    const long long t0 = clock64();
    for (;;) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (static_cast<int>(v - target) >= 0) break;
      if (clock64() - t0 > bq::kSpinLimitCycles) {
        atomicExch(&ws->status, (unsigned int)bq::kErrDeviceWait);
        break;
      }
    }
  }
  __syncthreads();
}

// Called by thread 0 of every CTA of a multi-CTA grid after it has the global
// amax: the last CTA to check out returns the scratch to zero, so the next
// launch (and a graph replay) starts clean.
__device__ __forceinline__ void grid_depart(QuantWs* ws, unsigned int* wait_seen = nullptr,
                                            unsigned int wait_count = 0u) {
  if (threadIdx.x != 0) return;
  if (gridDim.x == 1) {
    if (wait_seen != nullptr) *wait_seen += wait_count;
    return;
  }
  const unsigned int old = atomicAdd(&ws->depart, 1u);
  if (old == gridDim.x - 1) {
    if (wait_seen != nullptr) *wait_seen += wait_count;   // every CTA has read the old value
    ws->amax_bits = 0u;
    ws->arrive = 0u;
    ws->depart = 0u;
    __threadfence();
  }
}

// Host side: launches a grid-stride kernel with at most as many CTAs as the device holds at
// once (`want` CTAs if that is fewer), so that no partial second wave trails the first -- a grid
// of 8 CTAs per SM where five fit ran 1.6 waves.  Programmatic dependent launch on request.
template <typename Kernel, typename... Args>
inline cudaError_t launch_resident_smem(Kernel kernel, long long want, int threads, int sms, bool pdl,
                                        size_t dynamic_smem, cudaStream_t stream, Args... args) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dynamic_smem) != cudaSuccess ||
      per_sm < 1) {
    (void)cudaGetLastError();
    per_sm = 4;
  }
  const long long cap = static_cast<long long>(per_sm) * sms;
  long long grid = want < cap ? want : cap;
  if (grid < 1) grid = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = dynamic_smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
template <typename Kernel, typename... Args>
inline cudaError_t launch_resident(Kernel kernel, long long want, int threads, int sms, bool pdl,
                                   cudaStream_t stream, Args... args) {
  return launch_resident_smem(kernel, want, threads, sms, pdl, 0, stream, args...);
}

}  // namespace qd
}  // namespace bq
