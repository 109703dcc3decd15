// Dynamic per-tensor FP8 (e4m3fn) activation quantization for sm_100a, one launch.
//
//   scale = max(amax(|x|) * (1/448), 1e-12)        q = e4m3(clamp(x / scale, +-448))
//
// The arithmetic follows, operation for operation, what the reference engine's
// torch spelling evaluates on a CUDA device (braid/model/quant.py:108-115 and
// :228-229; the two-launch kernel braid/kernels/csrc/quant_act.cu:90-131 states
// the same contract): the scale is a reciprocal MULTIPLY, `x / scale` is a true
// IEEE division, clamps are comparisons so NaN survives, and the amax is a
// NaN-propagating max.  max() is exact and order-free, so any grid produces the
// same scale bits.
//
// Shape of the kernel (HBM-bound, 3 bytes moved per bf16 element):
//   * every thread pulls up to kMaxHeld groups of 8 elements with 128-bit loads
//     and KEEPS them in registers;
//   * |x| max: per thread -> warp shuffles -> shared memory -> one atomicMax per
//     CTA on the bit pattern of the non-negative float (exact; NaN patterns sort
//     above +inf, which is the propagation torch.amax has);
//   * a bounded grid barrier (all CTAs co-resident: grid <= #SMs), after which
//     each thread casts what it holds and writes 8 codes with one 64-bit store.
//   Inputs too large to hold (prefill sizes) use the streaming variant: same
//   barrier, second read served mostly by the 126 MB L2.
// Two prologue variants build the activation in registers first and never write
// it to memory: SiLU(gate)*up (braid/model/mlp.py:48) and o*sigmoid(gate)
// (braid/model/attention.py:215), with the double rounding of the two separate
// torch kernels preserved.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/braid_b200.h"
#include "ptx.cuh"
#include "quant_device.cuh"
#include "grid_amax.cuh"

namespace {

using namespace bq::qd;

// Hold variant: each thread keeps `p.held` (<= MAXH) groups in registers across
// the barrier, so the activation is read exactly once.  All loads of a thread
// are issued before the first value is used.
template <typename T, int MODE, int MAXH>
__global__ void __launch_bounds__(512, 1) quant_hold_kernel(const QParams p) {
  if (threadIdx.x == 0) { BQ_STAMP(p, 0); BQ_STAMP_META(p, 1); }
  bq::pdl_launch_dependents();
  const unsigned int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned int nthreads = gridDim.x * blockDim.x;
  Pack8<T> held[MAXH];
  Pack8<T> other[MODE == kPlain ? 1 : MAXH];
  bq::pdl_wait_prior_grids();   // the activation is the previous kernel's output
  if (threadIdx.x == 0) BQ_STAMP(p, 2);
  // a gathered buffer that peers store into while this kernel is resident is read with
  // coherent loads, after the arrival wait
  const bool coherent = p.wait_flag != nullptr;
  if (coherent)
    grid_wait_arrivals(p.wait_flag, p.wait_seen, p.wait_count, static_cast<QuantWs*>(p.ws));
#pragma unroll
  for (int i = 0; i < MAXH; ++i) {
    const unsigned int g = tid + static_cast<unsigned int>(i) * nthreads;
    if (i < p.held && g < p.n_groups) {
      if (coherent) load_raw<T, MODE, true>(p, g, held[i], other[MODE == kPlain ? 0 : i]);
      else load_raw<T, MODE, false>(p, g, held[i], other[MODE == kPlain ? 0 : i]);
    }
  }
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXH; ++i) {
    const unsigned int g = tid + static_cast<unsigned int>(i) * nthreads;
    if (i < p.held && g < p.n_groups) {
      apply_prologue<T, MODE>(held[i], other[MODE == kPlain ? 0 : i]);
      m = absmax8(held[i], m);
    }
  }
  // plain mode: up to 7 trailing elements, owned by the last thread of the grid
  float tail_v[kGroup - 1];
  const bool owns_tail = (MODE == kPlain) && p.tail != 0 && tid == nthreads - 1;
  if (owns_tail) {
    const T* src = reinterpret_cast<const T*>(p.a) + static_cast<size_t>(p.n_groups) * kGroup;
    for (unsigned int i = 0; i < p.tail; ++i) {
      tail_v[i] = widen(coherent ? __ldcg(src + i) : src[i]);
      m = nan_max(m, fabsf(tail_v[i]));
    }
  }
  const float sc = scale_from_amax(grid_amax(m, static_cast<QuantWs*>(p.ws)));
  const ScaleDiv dv(sc);
  if (threadIdx.x == 0) BQ_STAMP(p, 4);
  if (tid == 0) p.scale[0] = sc;
#pragma unroll
  for (int i = 0; i < MAXH; ++i) {
    const unsigned int g = tid + static_cast<unsigned int>(i) * nthreads;
    if (i < p.held && g < p.n_groups) emit8<T, true>(held[i], dv, p.q + static_cast<size_t>(g) * kGroup);
  }
  if (owns_tail) {
    uint8_t* dst = p.q + static_cast<size_t>(p.n_groups) * kGroup;
    for (unsigned int i = 0; i < p.tail; ++i)
      dst[i] = __nv_cvt_float_to_fp8(quant_one(tail_v[i], dv), __NV_SATFINITE, __NV_E4M3);
  }
  grid_depart(static_cast<QuantWs*>(p.ws), p.wait_flag != nullptr ? p.wait_seen : nullptr, p.wait_count);
  if (threadIdx.x == 0) BQ_STAMP(p, 7);
}

// Streaming variant for activations that do not fit in the register file of
// one co-resident grid: pass 1 reduces, pass 2 re-reads (L2) and casts.  Both
// passes keep kUnroll independent groups in flight per thread.
// PHASE selects what runs: kBoth (the quantizer), kScaleOnly (pass 1 and the grid-wide
// exchange; writes the scale, no codes), kCastOnly (pass 2 with the scale read from p.scale;
// no exchange, so the grid need not be co-resident).  The two halves exist for the
// column-parallel MLP: every rank takes the scale of its own shard, the ranks combine the
// scales with a MAX all-reduce (max is exact and order-free, and the scale is a monotone
// function of the amax), and every rank casts its shard with the combined scale.
enum Phase { kBoth = 0, kScaleOnly = 1, kCastOnly = 2 };

template <typename T, int MODE, int PHASE>
__global__ void __launch_bounds__(512, 2) quant_stream_kernel(const QParams p) {
  constexpr int kUnroll = (MODE == kPlain) ? 4 : 2;
  bq::pdl_launch_dependents();
  const unsigned int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned int nthreads = gridDim.x * blockDim.x;
  bq::pdl_wait_prior_grids();
  const bool coherent = p.wait_flag != nullptr;
  if (coherent)
    grid_wait_arrivals(p.wait_flag, p.wait_seen, p.wait_count, static_cast<QuantWs*>(p.ws));
  const bool owns_tail = (MODE == kPlain) && p.tail != 0 && tid == nthreads - 1;
  float sc;
  if constexpr (PHASE == kCastOnly) {
    sc = __ldcg(p.scale);
  } else {
    float m = 0.0f;
    for (unsigned int g0 = tid; g0 < p.n_groups; g0 += nthreads * kUnroll) {
      Pack8<T> a[kUnroll], b[MODE == kPlain ? 1 : kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const unsigned long long g = (unsigned long long)g0 + (unsigned long long)u * nthreads;
        if (g < p.n_groups) {
          if (coherent) load_raw<T, MODE, true>(p, (unsigned int)g, a[u], b[MODE == kPlain ? 0 : u]);
          else load_raw<T, MODE, false>(p, (unsigned int)g, a[u], b[MODE == kPlain ? 0 : u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const unsigned long long g = (unsigned long long)g0 + (unsigned long long)u * nthreads;
        if (g < p.n_groups) {
          apply_prologue<T, MODE>(a[u], b[MODE == kPlain ? 0 : u]);
          m = absmax8(a[u], m);
        }
      }
    }
    if (owns_tail) {
      const T* src = reinterpret_cast<const T*>(p.a) + static_cast<size_t>(p.n_groups) * kGroup;
      for (unsigned int i = 0; i < p.tail; ++i)
        m = nan_max(m, fabsf(widen(coherent ? __ldcg(src + i) : src[i])));
    }
    sc = scale_from_amax(grid_amax(m, static_cast<QuantWs*>(p.ws)));
    if (tid == 0) p.scale[0] = sc;
  }
  if constexpr (PHASE != kScaleOnly) {
    const ScaleDiv dv(sc);
    // Every thread re-reads exactly the groups it read in pass 1 (the L2 keeps a line on
    // the side of the chip whose SM asked for it, so the same SM finds it again), last
    // iteration first: what pass 1 read last is the likeliest to be still there.
    const unsigned int stride = nthreads * kUnroll;
    long long g0 = -1;
    if (tid < p.n_groups) g0 = (long long)tid + (long long)((p.n_groups - 1 - tid) / stride) * stride;
    for (; g0 >= 0; g0 -= stride) {
      Pack8<T> a[kUnroll], b[MODE == kPlain ? 1 : kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long g = g0 + (long long)u * nthreads;
        if (g < (long long)p.n_groups) {
          if (coherent) load_raw<T, MODE, true>(p, (unsigned int)g, a[u], b[MODE == kPlain ? 0 : u]);
          else load_raw<T, MODE, false>(p, (unsigned int)g, a[u], b[MODE == kPlain ? 0 : u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long g = g0 + (long long)u * nthreads;
        if (g < (long long)p.n_groups) {
          apply_prologue<T, MODE>(a[u], b[MODE == kPlain ? 0 : u]);
          emit8<T, PHASE == kBoth>(a[u], dv, p.q + static_cast<size_t>(g) * kGroup);
        }
      }
    }
    if (owns_tail) {
      const T* src = reinterpret_cast<const T*>(p.a) + static_cast<size_t>(p.n_groups) * kGroup;
      uint8_t* dst = p.q + static_cast<size_t>(p.n_groups) * kGroup;
      for (unsigned int i = 0; i < p.tail; ++i)
        dst[i] = __nv_cvt_float_to_fp8(quant_one(widen(coherent ? __ldcg(src + i) : src[i]), dv),
                                       __NV_SATFINITE, __NV_E4M3);
    }
  }
  if constexpr (PHASE != kCastOnly)
    grid_depart(static_cast<QuantWs*>(p.ws), coherent ? p.wait_seen : nullptr, p.wait_count);
}

// Sticky status of the launches that run without scratch from the caller (the cast half alone):
// a bounded wait that ran out there has no status word of the caller's to raise, so it raises
// this one; bq_scratchless_status() reads and clears it.
__device__ unsigned int g_scratchless_status = 0u;

// ---- plain quantizer at prefill sizes: bulk copies into a shared-memory ring --------------
// The register-fed streaming kernel above keeps 64 bytes per thread in flight and computes
// between its loads; at prefill sizes that is half of what HBM needs.  Here one producer lane
// feeds a ring of chunks with untiled bulk copies (bytes in flight cost no registers:
// 2 CTAs x 96 KB per SM), and 512 consumer threads take one, two or four 16-byte units of
// every chunk each.  In the whole quantizer (kBoth) the ring is also a cache: when pass 1 ends, the last
// chunks of every CTA (96 KB) are still in shared memory, and pass 2 walks the CTA's
// chunks backwards, so those are cast without touching memory again and the others are
// re-fetched (from L2 while it still has them) in the order pass 1 read them last.
constexpr int kRingThreads = 512;                  // consumers; one more warp produces
constexpr int kRingSmem = 12 * kRingThreads * 16;  // 96 KB of ring per CTA, two CTAs per SM

template <typename T>
__device__ __forceinline__ float unit_absmax(const uint4& raw, float m) {
  if constexpr (sizeof(T) == 2) {
    return absmax8(*reinterpret_cast<const Pack8<T>*>(&raw), m);
  } else {
    m = nan_max(m, fabsf(__uint_as_float(raw.x)));
    m = nan_max(m, fabsf(__uint_as_float(raw.y)));
    m = nan_max(m, fabsf(__uint_as_float(raw.z)));
    return nan_max(m, fabsf(__uint_as_float(raw.w)));
  }
}

// codes of the 16 bytes `raw` holds: 8 for a 16-bit type, 4 for fp32
template <typename T, bool OWN_SCALE>
__device__ __forceinline__ void unit_emit(const uint4& raw, const ScaleDiv& dv, uint8_t* dst) {
  if constexpr (sizeof(T) == 2) {
    emit8<T, OWN_SCALE>(*reinterpret_cast<const Pack8<T>*>(&raw), dv, dst);
  } else {
    float f[4] = {__uint_as_float(raw.x), __uint_as_float(raw.y), __uint_as_float(raw.z),
                  __uint_as_float(raw.w)};
    divide_group<4, OWN_SCALE>(dv, f);
    const uint32_t a = __nv_cvt_float2_to_fp8x2(make_float2(f[0], f[1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t b = __nv_cvt_float2_to_fp8x2(make_float2(f[2], f[3]), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(dst) = (a & 0xFFFFu) | ((b & 0xFFFFu) << 16);
  }
}

// UNITS = 16-byte units of a chunk per consumer thread (1, 2 or 4): larger chunks spend fewer
// instructions per element on barriers and addresses, smaller ones balance a short input over
// the CTAs; the launcher picks the largest that leaves every CTA about three chunks.
template <typename T, int PHASE, int UNITS>
__global__ void __launch_bounds__(kRingThreads + 32, 2) quant_ring_kernel(const QParams p) {
  constexpr int kRingUnits = UNITS;
  constexpr int kRingChunk = kRingThreads * 16 * UNITS;      // bytes of input per chunk
  constexpr int kRingStages = kRingSmem / kRingChunk;
  extern __shared__ __align__(128) uint8_t ring[];
  // [0] full / [1] empty of the forward pass, [2] full / [3] empty of the backward pass
  __shared__ __align__(8) uint64_t bars[4][12];
  __shared__ unsigned int s_failed;
  bq::pdl_launch_dependents();
  if (threadIdx.x == 0) { BQ_STAMP(p, 0); BQ_STAMP_META(p, 1); }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool producer = warp == kRingThreads / 32;
  if (threadIdx.x == 0) {
    s_failed = 0u;
    for (int s = 0; s < kRingStages; ++s) {
      bq::mbar_init(bq::smem_u32(&bars[0][s]), 1);
      bq::mbar_init(bq::smem_u32(&bars[1][s]), kRingThreads / 32);
      bq::mbar_init(bq::smem_u32(&bars[2][s]), 1);
      bq::mbar_init(bq::smem_u32(&bars[3][s]), kRingThreads / 32);
    }
    bq::fence_mbar_init();
  }
  __syncthreads();
  bq::pdl_wait_prior_grids();
  if (threadIdx.x == 0) BQ_STAMP(p, 2);

  const uint8_t* src = static_cast<const uint8_t*>(p.a);
  const unsigned long long body = (unsigned long long)p.n_groups * kGroup * sizeof(T);   // bytes
  const long long n_chunks = (long long)((body + kRingChunk - 1) / kRingChunk);
  // this CTA's chunks: blockIdx.x, + gridDim.x, ...
  const int count =
      n_chunks > (long long)blockIdx.x ? (int)((n_chunks - 1 - blockIdx.x) / gridDim.x + 1) : 0;
  auto chunk_offset = [&](int k) {
    return ((unsigned long long)blockIdx.x + (unsigned long long)k * gridDim.x) * kRingChunk;
  };
  auto chunk_bytes = [&](int k) {
    const unsigned long long left = body - chunk_offset(k);
    return (uint32_t)(left < (unsigned long long)kRingChunk ? left : (unsigned long long)kRingChunk);
  };
  auto fail = [&]() { atomicExch(&s_failed, 1u); };
  // what a later pass (or the cast launch that follows a scale launch) reads again stays in
  // L2 as long as L2 likes; measured, the hint makes no difference at any size
  const uint64_t policy = (PHASE == kCastOnly) ? bq::policy_evict_first() : bq::policy_evict_last();
  // the elements after the last whole group belong to consumer thread 0 of CTA 0
  const bool owns_tail = p.tail != 0 && blockIdx.x == 0 && threadIdx.x == 0;
  const T* tail_src = reinterpret_cast<const T*>(p.a) + static_cast<size_t>(p.n_groups) * kGroup;
  constexpr int kPerUnit = 16 / (int)sizeof(T);   // elements (and code bytes) per 16 bytes of input

  float sc;
  // ---- forward pass: |x| max (kBoth, kScaleOnly) or the cast itself (kCastOnly) ----
  if constexpr (PHASE == kCastOnly) sc = __ldcg(p.scale);
  {
    const ScaleDiv dv(PHASE == kCastOnly ? sc : 1.0f);
    float m = 0.0f;
    if (producer) {
      if (lane == 0) {
        for (int k = 0; k < count; ++k) {
          const int s = k % kRingStages;
          if (k >= kRingStages &&
              !bq::mbar_wait(bq::smem_u32(&bars[1][s]), (uint32_t)((k / kRingStages - 1) & 1))) {
            fail();
            break;
          }
          const uint32_t bytes = chunk_bytes(k);
          bq::mbar_expect_tx(bq::smem_u32(&bars[0][s]), bytes);
          bq::bulk_load_1d(bq::smem_u32(ring + s * kRingChunk), src + chunk_offset(k), bytes,
                           bq::smem_u32(&bars[0][s]), policy);
        }
      }
    } else {
      for (int k = 0; k < count; ++k) {
        const int s = k % kRingStages;
        if (!bq::mbar_wait(bq::smem_u32(&bars[0][s]), (uint32_t)((k / kRingStages) & 1))) {
          fail();
          break;
        }
        const uint32_t have = chunk_bytes(k);
        uint4 raw[kRingUnits];
#pragma unroll
        for (int u = 0; u < kRingUnits; ++u) {
          const uint32_t unit = threadIdx.x + u * kRingThreads;
          if (unit * 16u < have) raw[u] = *reinterpret_cast<const uint4*>(ring + s * kRingChunk + unit * 16);
        }
#pragma unroll
        for (int u = 0; u < kRingUnits; ++u) {
          const uint32_t unit = threadIdx.x + u * kRingThreads;
          if (unit * 16u < have) {
            if constexpr (PHASE == kCastOnly) {
              unit_emit<T, false>(raw[u], dv, p.q + (chunk_offset(k) / 16 + unit) * kPerUnit);
            } else {
              m = unit_absmax<T>(raw[u], m);
            }
          }
        }
        // hand the stage back when the producer will refill it (kBoth keeps the last ones)
        if (PHASE != kBoth || k + kRingStages < count) {
          __syncwarp();
          if (lane == 0) bq::mbar_arrive(bq::smem_u32(&bars[1][s]));
        }
      }
    }
    if constexpr (PHASE == kCastOnly) {
      if (owns_tail) {
        uint8_t* dst = p.q + static_cast<size_t>(p.n_groups) * kGroup;
        for (unsigned int i = 0; i < p.tail; ++i)
          dst[i] = __nv_cvt_float_to_fp8(quant_one(widen(tail_src[i]), dv), __NV_SATFINITE, __NV_E4M3);
      }
    } else {
      if (owns_tail)
        for (unsigned int i = 0; i < p.tail; ++i) m = nan_max(m, fabsf(widen(tail_src[i])));
      if (threadIdx.x == 0) BQ_STAMP(p, 3);
      sc = scale_from_amax(grid_amax(m, static_cast<QuantWs*>(p.ws)));
      if (threadIdx.x == 0) BQ_STAMP(p, 4);
      if (blockIdx.x == 0 && threadIdx.x == 0) p.scale[0] = sc;
    }
  }
  // ---- backward pass of the whole quantizer: the ring's contents first, then re-fetches ----
  if constexpr (PHASE == kBoth) {
    const ScaleDiv dv(sc);
    const int refetch = count - kRingStages;   // chunks [0, refetch) are no longer in the ring
    if (producer) {
      if (lane == 0 && s_failed == 0u) {
        for (int k = refetch - 1; k >= 0; --k) {
          const int s = k % kRingStages;
          const uint32_t parity = (uint32_t)(((refetch - 1 - k) / kRingStages) & 1);
          if (!bq::mbar_wait(bq::smem_u32(&bars[3][s]), parity)) { fail(); break; }
          const uint32_t bytes = chunk_bytes(k);
          bq::mbar_expect_tx(bq::smem_u32(&bars[2][s]), bytes);
          bq::bulk_load_1d(bq::smem_u32(ring + s * kRingChunk), src + chunk_offset(k), bytes,
                           bq::smem_u32(&bars[2][s]), bq::policy_evict_first());
        }
      }
    } else if (s_failed == 0u) {
      for (int k = count - 1; k >= 0; --k) {
        const int s = k % kRingStages;
        if (k < refetch) {
          const uint32_t parity = (uint32_t)(((refetch - 1 - k) / kRingStages) & 1);
          if (!bq::mbar_wait(bq::smem_u32(&bars[2][s]), parity)) { fail(); break; }
        }
        const uint32_t have = chunk_bytes(k);
        uint4 raw[kRingUnits];
#pragma unroll
        for (int u = 0; u < kRingUnits; ++u) {
          const uint32_t unit = threadIdx.x + u * kRingThreads;
          if (unit * 16u < have) raw[u] = *reinterpret_cast<const uint4*>(ring + s * kRingChunk + unit * 16);
        }
#pragma unroll
        for (int u = 0; u < kRingUnits; ++u) {
          const uint32_t unit = threadIdx.x + u * kRingThreads;
          if (unit * 16u < have)
            unit_emit<T, true>(raw[u], dv, p.q + (chunk_offset(k) / 16 + unit) * kPerUnit);
        }
        if (k >= kRingStages) {   // chunk k - kRingStages comes into this stage next
          __syncwarp();
          if (lane == 0) bq::mbar_arrive(bq::smem_u32(&bars[3][s]));
        }
      }
    }
    if (owns_tail) {
      uint8_t* dst = p.q + static_cast<size_t>(p.n_groups) * kGroup;
      for (unsigned int i = 0; i < p.tail; ++i)
        dst[i] = __nv_cvt_float_to_fp8(quant_one(widen(tail_src[i]), dv), __NV_SATFINITE, __NV_E4M3);
    }
  }
  // no bulk copy is in flight here unless a wait ran out: every issued copy was waited for by
  // the consumers.  After a failed wait, give the copies a bounded time to land before the
  // CTA's shared memory goes away.
  __syncthreads();
  if (s_failed != 0u) {
    if (threadIdx.x == 0) {
      // the cast half alone runs without scratch: it raises the library's own sticky word
      if (p.ws != nullptr)
        atomicExch(&static_cast<QuantWs*>(p.ws)->status, (unsigned int)bq::kErrDeviceWait);
      else
        atomicExch(&g_scratchless_status, (unsigned int)bq::kErrDeviceWait);
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {}
    }
    __syncthreads();
  }
  if constexpr (PHASE != kCastOnly) grid_depart(static_cast<QuantWs*>(p.ws));
  if (threadIdx.x == 0) BQ_STAMP(p, 7);
}

// The prologues alone, unquantized: out[r, c] = the value the quantizer modes quantize
// (`F.silu(gate) * up`, braid/model/mlp.py:48; `o * torch.sigmoid(gate)`,
// braid/model/attention.py:215), contiguous [rows, cols] of T.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) prologue_dense_kernel(const QParams p, T* __restrict__ out) {
  bq::pdl_launch_dependents();
  bq::pdl_wait_prior_grids();
  __shared__ float s_max[8];
  const unsigned int nthreads = gridDim.x * blockDim.x;
  float m = 0.0f;
  for (unsigned long long g = blockIdx.x * blockDim.x + threadIdx.x; g < p.n_groups; g += nthreads) {
    Pack8<T> a, b;
    load_raw<T, MODE, false>(p, (unsigned int)g, a, b);
    apply_prologue<T, MODE>(a, b);
    m = absmax8(a, m);
    if constexpr (sizeof(T) == 4) {
      float4* dst = reinterpret_cast<float4*>(out + g * kGroup);
      dst[0] = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
      dst[1] = make_float4(a.v[4], a.v[5], a.v[6], a.v[7]);
    } else {
      *reinterpret_cast<uint4*>(out + g * kGroup) = *reinterpret_cast<const uint4*>(&a);
    }
  }
  // with a scale asked for: every CTA folds its max into one word and counts itself, the CTA
  // that counts last publishes the scale and returns the scratch to zero; nobody waits
  if (p.scale == nullptr) return;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float w = s_max[0];
    for (unsigned int i = 1; i < blockDim.x / 32; ++i) w = nan_max(w, s_max[i]);
    QuantWs* ws = static_cast<QuantWs*>(p.ws);
    atomicMax(&ws->amax_bits, __float_as_uint(w));
    __threadfence();
    const unsigned int old = atomicAdd(&ws->arrive, 1u);
    if (old == gridDim.x - 1) {
      __threadfence();
      const unsigned int bits = atomicExch(&ws->amax_bits, 0u);
      p.scale[0] = scale_from_amax(__uint_as_float(bits));
      ws->arrive = 0u;
      __threadfence();
    }
  }
}

// ---- column-parallel form: one rank's [rows, cols] block to every rank ----------------------
// Elementwise: every thread takes 8 values of a row of this rank's block and stores them --
// as e4m3 codes under a given scale (CAST) or unchanged -- at the same row and column of every
// rank's gathered buffer (plain stores through peer-mapped pointers, this rank's own buffer
// included; the pointers already carry this rank's column offset).  A warp writes 256 (codes) or
// 512 contiguous bytes of a row per destination, which the links move at their copy rate; the
// 128-byte pieces a GEMM epilogue scatters over rows do not.  The CTAs count themselves on a
// local word and the last one adds 1 to every rank's arrival counter with a system-scope
// release, as the GEMM push epilogues do.
struct RowPush {
  const void* src;
  long long ld_src;               // elements
  int rows, groups_per_row;       // groups of 8 columns
  int wide;                       // CAST: destinations allow 16-byte stores of two groups
  const float* scale;             // CAST: device scalar
  int n;
  void* dst[8];
  long long ld_dst;               // elements of the destination (bytes for codes)
  unsigned int* flag[8];
  unsigned int* done;             // local, zero between launches
};

template <typename T, bool CAST>
__global__ void __launch_bounds__(256) row_push_kernel(const RowPush p) {
  bq::pdl_launch_dependents();
  bq::pdl_wait_prior_grids();
  float sc = 1.0f;
  if constexpr (CAST) sc = __ldcg(p.scale);
  const ScaleDiv dv(sc);
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* src = reinterpret_cast<const T*>(p.src) + (long long)row * p.ld_src;
    if (CAST && p.wide) {
      // two groups per thread, one 16-byte store per destination: a warp writes 512 contiguous
      // bytes of the row on every rank
      for (int g = 2 * threadIdx.x; g < p.groups_per_row; g += 2 * blockDim.x) {
        const Pack8<T> v0 = load8<T, false>(src + g * kGroup);
        const Pack8<T> v1 = load8<T, false>(src + (g + 1) * kGroup);
        const uint2 c0 = codes8<T, false>(v0, dv), c1 = codes8<T, false>(v1, dv);
        const uint4 c = make_uint4(c0.x, c0.y, c1.x, c1.y);
        const long long at = (long long)row * p.ld_dst + g * kGroup;
        for (int d = 0; d < p.n; ++d) *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.dst[d]) + at) = c;
      }
      continue;
    }
    for (int g = threadIdx.x; g < p.groups_per_row; g += blockDim.x) {
      const Pack8<T> v = load8<T, false>(src + g * kGroup);
      const long long at = (long long)row * p.ld_dst + g * kGroup;
      if constexpr (CAST) {
        const uint2 c = codes8<T, false>(v, dv);
        for (int d = 0; d < p.n; ++d) *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.dst[d]) + at) = c;
      } else if constexpr (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(&v);
        for (int d = 0; d < p.n; ++d) *reinterpret_cast<uint4*>(static_cast<T*>(p.dst[d]) + at) = raw;
      } else {
        const float4 lo = make_float4(v.v[0], v.v[1], v.v[2], v.v[3]);
        const float4 hi = make_float4(v.v[4], v.v[5], v.v[6], v.v[7]);
        for (int d = 0; d < p.n; ++d) {
          float4* q = reinterpret_cast<float4*>(static_cast<T*>(p.dst[d]) + at);
          q[0] = lo;
          q[1] = hi;
        }
      }
    }
  }
  // every store of the launch happens before every arrival (see the GEMM push epilogue)
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned int last = 0u;
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int old = atomicAdd(p.done, 1u);
      if (old == gridDim.x - 1u) {
        *p.done = 0u;
        __threadfence_system();
        last = 1u;
      }
    }
    // lane d signals rank d: the round trips run side by side; lane 0's fences come first
    last = __shfl_sync(0xffffffffu, last, 0);
    __syncwarp();
    if (last != 0u && (int)threadIdx.x < p.n) {
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.flag[threadIdx.x]) : "memory");
    }
  }
}

struct DeviceInfo {
  int sms = 0;
};

int device_sms() {
  static DeviceInfo info[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (info[dev].sms == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    info[dev].sms = v;
  }
  return info[dev].sms;
}

long long g_opt_quant_block = 0;   // 0 = heuristic
long long g_opt_quant_held = 0;    // 0 = heuristic
long long g_opt_quant_pdl = 1;     // programmatic dependent launch on by default
long long g_opt_quant_ring = 1;    // plain mode at streaming sizes through the shared-memory ring

template <typename Kernel>
int launch_with_pdl(Kernel kernel, int grid, int block, const QParams& p_in, cudaStream_t stream,
                    size_t dynamic_smem = 0) {
  QParams p = p_in;
  if (dynamic_smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dynamic_smem) !=
          cudaSuccess) {
    (void)cudaGetLastError();
    return bq::kErrLaunch;
  }
#ifdef BQ_PHASES
  p.phase_ring = bq::phase_ring_for_launch(&p.phase_seq);
#endif
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3((unsigned)block, 1, 1);
  cfg.dynamicSmemBytes = dynamic_smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt_quant_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return bq::kErrLaunch; }
  return bq::kOk;
}

// The ring kernel takes the plain mode of an input nobody is still writing (its bulk copies
// are no coherent loads) that starts on a 16-byte boundary.
template <int MODE>
bool ring_applies(const QParams& p) {
  return MODE == kPlain && p.wait_flag == nullptr && (reinterpret_cast<uintptr_t>(p.a) % 16) == 0;
}

template <typename T, int PHASE>
int launch_ring(const QParams& p, int sms, cudaStream_t stream) {
  const unsigned long long body = (unsigned long long)p.n_groups * kGroup * sizeof(T);
  const unsigned long long unit_chunk = (unsigned long long)kRingThreads * 16;
  const unsigned long long ctas = 2ull * sms;
  const int units = body >= 3 * ctas * 4 * unit_chunk ? 4 : (body >= 3 * ctas * 2 * unit_chunk ? 2 : 1);
  unsigned long long chunks = (body + units * unit_chunk - 1) / (units * unit_chunk);
  if (chunks < 1) chunks = 1;
  const int grid = (int)(chunks < ctas ? chunks : ctas);
  const int block = kRingThreads + 32;
  if (units == 4) return launch_with_pdl(quant_ring_kernel<T, PHASE, 4>, grid, block, p, stream, kRingSmem);
  if (units == 2) return launch_with_pdl(quant_ring_kernel<T, PHASE, 2>, grid, block, p, stream, kRingSmem);
  return launch_with_pdl(quant_ring_kernel<T, PHASE, 1>, grid, block, p, stream, kRingSmem);
}

template <typename T, int MODE>
int launch_quant(QParams p, cudaStream_t stream) {
  const int sms = device_sms();
  if (sms <= 0) return bq::kErrLaunch;
  // registers a thread may spend on held values: 8 groups of a 16-bit type in
  // the plain mode; half of that when two operands are staged or T is fp32
  constexpr int kMaxH = (MODE == kPlain ? 8 : 4) / (sizeof(T) == 4 ? 2 : 1);
  const unsigned long long groups = p.n_groups;
  // One group per thread while that covers the input with 256-thread CTAs on
  // every SM; after that 512-thread CTAs, deepening each thread up to kMaxH;
  // beyond that, stream.
  int block = (groups > (unsigned long long)sms * 256ull) ? 512 : 256;
  if (g_opt_quant_block == 256 || g_opt_quant_block == 512) block = (int)g_opt_quant_block;
  const unsigned long long cap = (unsigned long long)sms * block * kMaxH;
  if (groups <= cap) {
    int held = 1;
    while ((unsigned long long)sms * block * held < groups) ++held;
    if (g_opt_quant_held >= held && g_opt_quant_held <= kMaxH) held = (int)g_opt_quant_held;
    unsigned long long per_cta = (unsigned long long)block * held;
    int grid = (int)((groups + per_cta - 1) / per_cta);
    if (grid < 1) grid = 1;
    p.held = held;
    // The smallest instantiation that holds `held` groups: fewer registers per
    // thread, so the next GEMM's CTAs fit on the SM beside a waiting quantizer CTA.
    if (held <= 1) return launch_with_pdl(quant_hold_kernel<T, MODE, 1>, grid, block, p, stream);
    if (held <= 2 && kMaxH >= 2)
      return launch_with_pdl(quant_hold_kernel<T, MODE, (kMaxH >= 2 ? 2 : kMaxH)>, grid, block, p, stream);
    if (held <= 4 && kMaxH >= 4)
      return launch_with_pdl(quant_hold_kernel<T, MODE, (kMaxH >= 4 ? 4 : kMaxH)>, grid, block, p, stream);
    return launch_with_pdl(quant_hold_kernel<T, MODE, kMaxH>, grid, block, p, stream);
  }
  p.held = 0;
  if (ring_applies<MODE>(p) && g_opt_quant_ring) return launch_ring<T, kBoth>(p, sms, stream);
  return launch_with_pdl(quant_stream_kernel<T, MODE, kBoth>, 2 * sms, 512, p, stream);
}

template <int MODE>
int dispatch_dtype(int dtype, const QParams& p, cudaStream_t stream) {
  switch (dtype) {
    case BQ_DTYPE_F32: return launch_quant<float, MODE>(p, stream);
    case BQ_DTYPE_BF16: return launch_quant<__nv_bfloat16, MODE>(p, stream);
    case BQ_DTYPE_F16: return launch_quant<__half, MODE>(p, stream);
    default: return bq::kErrBadArg;
  }
}

// One half of the quantizer (see Phase): always the streaming kernel.
template <int MODE, int PHASE>
int dispatch_phase(int dtype, const QParams& p, cudaStream_t stream) {
  const int sms = device_sms();
  if (sms <= 0) return bq::kErrLaunch;
  // the scale half waits on the whole grid (co-resident: 2 CTAs of 512 threads per SM at most);
  // small inputs get a grid that matches their size
  unsigned long long want = ((unsigned long long)p.n_groups + 511ull) / 512ull;
  if (want < 1) want = 1;
  const int grid = (int)(want < (unsigned long long)(2 * sms) ? want : (unsigned long long)(2 * sms));
  if (ring_applies<MODE>(p) && g_opt_quant_ring && want > (unsigned long long)(2 * sms)) {
    switch (dtype) {
      case BQ_DTYPE_F32: return launch_ring<float, PHASE>(p, sms, stream);
      case BQ_DTYPE_BF16: return launch_ring<__nv_bfloat16, PHASE>(p, sms, stream);
      case BQ_DTYPE_F16: return launch_ring<__half, PHASE>(p, sms, stream);
      default: return bq::kErrBadArg;
    }
  }
  switch (dtype) {
    case BQ_DTYPE_F32:
      return launch_with_pdl(quant_stream_kernel<float, MODE, PHASE>, grid, 512, p, stream);
    case BQ_DTYPE_BF16:
      return launch_with_pdl(quant_stream_kernel<__nv_bfloat16, MODE, PHASE>, grid, 512, p, stream);
    case BQ_DTYPE_F16:
      return launch_with_pdl(quant_stream_kernel<__half, MODE, PHASE>, grid, 512, p, stream);
    default: return bq::kErrBadArg;
  }
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t elem_size(int dtype) { return dtype == BQ_DTYPE_F32 ? 4 : 2; }

int check_ws(void* ws, size_t ws_bytes) {
  if (ws == nullptr || ws_bytes < sizeof(QuantWs) || !aligned_to(ws, 16)) return bq::kErrWorkspace;
  return bq::kOk;
}

}  // namespace

namespace bq {
int quant_set_option(const char* key, long long value);
}
int bq::quant_set_option(const char* key, long long value) {
  auto eq = [](const char* a, const char* b) {
    while (*a && *a == *b) { ++a; ++b; }
    return *a == *b;
  };
  if (eq(key, "quant_block")) { g_opt_quant_block = value; return kOk; }
  if (eq(key, "quant_held")) { g_opt_quant_held = value; return kOk; }
  if (eq(key, "quant_pdl")) { g_opt_quant_pdl = value ? 1 : 0; return kOk; }
  if (eq(key, "quant_ring")) { g_opt_quant_ring = value ? 1 : 0; return kOk; }
  return kErrBadArg;
}

extern "C" int bq_scratchless_status(int* status_out) {
  if (status_out == nullptr) return bq::kErrBadArg;
  unsigned int v = 0u;
  if (cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpyFromSymbol(&v, g_scratchless_status, sizeof(v)) != cudaSuccess)
    return bq::kErrLaunch;
  if (v != 0u) {
    const unsigned int zero = 0u;
    if (cudaMemcpyToSymbol(g_scratchless_status, &zero, sizeof(zero)) != cudaSuccess) return bq::kErrLaunch;
  }
  *status_out = static_cast<int>(v);
  return bq::kOk;
}

extern "C" size_t bq_quant_workspace_bytes(void) { return sizeof(QuantWs); }

extern "C" int bq_quantize_act(const void* x, int dtype, int64_t n, void* q_out, float* scale_out,
                               void* ws, size_t ws_bytes, void* stream) {
  if (x == nullptr || q_out == nullptr || scale_out == nullptr || n <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  if (!aligned_to(x, 16) || !aligned_to(q_out, 8)) return bq::kErrUnsupported;
  if (n / kGroup >= 0x7fffffffLL) return bq::kErrTooLarge;
  QParams p{};
  p.a = x;
  p.q = static_cast<uint8_t*>(q_out);
  p.scale = scale_out;
  p.ws = ws;
  p.n_groups = static_cast<unsigned int>(n / kGroup);
  p.tail = static_cast<unsigned int>(n % kGroup);
  p.groups_per_row = 1;
  return dispatch_dtype<kPlain>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_quantize_act_after(const void* x, int dtype, int64_t n, void* q_out,
                                     float* scale_out, const void* flag, void* seen,
                                     unsigned int count, void* ws, size_t ws_bytes, void* stream) {
  if (x == nullptr || q_out == nullptr || scale_out == nullptr || n <= 0) return bq::kErrBadArg;
  if (flag == nullptr || seen == nullptr || count == 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  if (!aligned_to(x, 16) || !aligned_to(q_out, 8) || !aligned_to(flag, 4) || !aligned_to(seen, 4))
    return bq::kErrUnsupported;
  if (n / kGroup >= 0x7fffffffLL) return bq::kErrTooLarge;
  QParams p{};
  p.a = x;
  p.q = static_cast<uint8_t*>(q_out);
  p.scale = scale_out;
  p.ws = ws;
  p.n_groups = static_cast<unsigned int>(n / kGroup);
  p.tail = static_cast<unsigned int>(n % kGroup);
  p.groups_per_row = 1;
  p.wait_flag = static_cast<const unsigned int*>(flag);
  p.wait_seen = static_cast<unsigned int*>(seen);
  p.wait_count = count;
  return dispatch_dtype<kPlain>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_silu_mul_quant(const void* gate, const void* up, int dtype, int64_t rows,
                                 int64_t cols, int64_t ld_gate, int64_t ld_up, void* q_out,
                                 float* scale_out, void* ws, size_t ws_bytes, void* stream) {
  if (!gate || !up || !q_out || !scale_out || rows <= 0 || cols <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  const size_t es = elem_size(dtype);
  if (cols % kGroup || ld_gate < cols || ld_up < cols || (ld_gate * es) % 16 || (ld_up * es) % 16 ||
      !aligned_to(gate, 16) || !aligned_to(up, 16) || !aligned_to(q_out, 8))
    return bq::kErrUnsupported;
  if (rows * (cols / kGroup) >= 0x7fffffffLL) return bq::kErrTooLarge;
  QParams p{};
  p.a = gate;
  p.b = up;
  p.q = static_cast<uint8_t*>(q_out);
  p.scale = scale_out;
  p.ws = ws;
  p.groups_per_row = static_cast<unsigned int>(cols / kGroup);
  p.n_groups = static_cast<unsigned int>(rows * (cols / kGroup));
  p.ld_a = ld_gate;
  p.ld_b = ld_up;
  return dispatch_dtype<kSiluMul>(dtype, p, static_cast<cudaStream_t>(stream));
}

namespace {
int fill_silu_mul(QParams* p, const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                  int64_t ld_gate, int64_t ld_up) {
  if (!gate || !up || rows <= 0 || cols <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  const size_t es = elem_size(dtype);
  if (cols % kGroup || ld_gate < cols || ld_up < cols || (ld_gate * es) % 16 || (ld_up * es) % 16 ||
      !aligned_to(gate, 16) || !aligned_to(up, 16))
    return bq::kErrUnsupported;
  if (rows * (cols / kGroup) >= 0x7fffffffLL) return bq::kErrTooLarge;
  p->a = gate;
  p->b = up;
  p->groups_per_row = static_cast<unsigned int>(cols / kGroup);
  p->n_groups = static_cast<unsigned int>(rows * (cols / kGroup));
  p->ld_a = ld_gate;
  p->ld_b = ld_up;
  return bq::kOk;
}
}  // namespace

extern "C" int bq_silu_mul_scale(const void* gate, const void* up, int dtype, int64_t rows,
                                 int64_t cols, int64_t ld_gate, int64_t ld_up, float* scale_out,
                                 void* ws, size_t ws_bytes, void* stream) {
  if (!scale_out) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  QParams p{};
  if (int rc = fill_silu_mul(&p, gate, up, dtype, rows, cols, ld_gate, ld_up)) return rc;
  p.scale = scale_out;
  p.ws = ws;
  return dispatch_phase<kSiluMul, kScaleOnly>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_silu_mul_cast(const void* gate, const void* up, int dtype, int64_t rows,
                                int64_t cols, int64_t ld_gate, int64_t ld_up, const float* scale,
                                void* q_out, void* stream) {
  if (!scale || !q_out) return bq::kErrBadArg;
  if (!aligned_to(q_out, 8)) return bq::kErrUnsupported;
  QParams p{};
  if (int rc = fill_silu_mul(&p, gate, up, dtype, rows, cols, ld_gate, ld_up)) return rc;
  p.scale = const_cast<float*>(scale);   // read only in this phase
  p.q = static_cast<uint8_t*>(q_out);
  return dispatch_phase<kSiluMul, kCastOnly>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_cast_act(const void* x, int dtype, int64_t n, const float* scale, void* q_out,
                           void* stream) {
  if (x == nullptr || q_out == nullptr || scale == nullptr || n <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (!aligned_to(x, 16) || !aligned_to(q_out, 8)) return bq::kErrUnsupported;
  if (n / kGroup >= 0x7fffffffLL) return bq::kErrTooLarge;
  QParams p{};
  p.a = x;
  p.q = static_cast<uint8_t*>(q_out);
  p.scale = const_cast<float*>(scale);   // read only in this phase
  p.n_groups = static_cast<unsigned int>(n / kGroup);
  p.tail = static_cast<unsigned int>(n % kGroup);
  p.groups_per_row = 1;
  return dispatch_phase<kPlain, kCastOnly>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_sigmoid_gate_quant(const void* o, const void* gate, int dtype, int64_t rows,
                                     int64_t cols, int64_t ld_o, int64_t ld_gate, int64_t chunk,
                                     int64_t chunk_stride, void* q_out, float* scale_out, void* ws,
                                     size_t ws_bytes, void* stream) {
  if (!o || !gate || !q_out || !scale_out || rows <= 0 || cols <= 0 || chunk <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  const size_t es = elem_size(dtype);
  if (cols % kGroup || chunk % kGroup || cols % chunk || ld_o < cols || (ld_o * es) % 16 ||
      (ld_gate * es) % 16 || (chunk_stride * es) % 16 || !aligned_to(o, 16) ||
      !aligned_to(gate, 16) || !aligned_to(q_out, 8))
    return bq::kErrUnsupported;
  if (rows * (cols / kGroup) >= 0x7fffffffLL) return bq::kErrTooLarge;
  QParams p{};
  p.a = o;
  p.b = gate;
  p.q = static_cast<uint8_t*>(q_out);
  p.scale = scale_out;
  p.ws = ws;
  p.groups_per_row = static_cast<unsigned int>(cols / kGroup);
  p.n_groups = static_cast<unsigned int>(rows * (cols / kGroup));
  p.ld_a = ld_o;
  p.ld_b = ld_gate;
  p.chunk = static_cast<unsigned int>(chunk);
  p.chunk_stride = chunk_stride;
  return dispatch_dtype<kSigmoidGate>(dtype, p, static_cast<cudaStream_t>(stream));
}

namespace {
template <int MODE>
int launch_dense(int dtype, const QParams& p, void* out, cudaStream_t stream) {
  const int sms = device_sms();
  if (sms <= 0) return bq::kErrLaunch;
  const long long want = (long long)(((unsigned long long)p.n_groups + 255ull) / 256ull);
  const bool pdl = g_opt_quant_pdl != 0;
  cudaError_t e;
  switch (dtype) {
    case BQ_DTYPE_F32:
      e = launch_resident(prologue_dense_kernel<float, MODE>, want, 256, sms, pdl, stream, p,
                          static_cast<float*>(out));
      break;
    case BQ_DTYPE_BF16:
      e = launch_resident(prologue_dense_kernel<__nv_bfloat16, MODE>, want, 256, sms, pdl, stream, p,
                          static_cast<__nv_bfloat16*>(out));
      break;
    case BQ_DTYPE_F16:
      e = launch_resident(prologue_dense_kernel<__half, MODE>, want, 256, sms, pdl, stream, p,
                          static_cast<__half*>(out));
      break;
    default: return bq::kErrBadArg;
  }
  if (e != cudaSuccess) { (void)cudaGetLastError(); return bq::kErrLaunch; }
  return bq::kOk;
}
}  // namespace

extern "C" int bq_silu_mul(const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                           int64_t ld_gate, int64_t ld_up, void* h_out, void* stream) {
  if (!h_out) return bq::kErrBadArg;
  if (!aligned_to(h_out, 16)) return bq::kErrUnsupported;
  QParams p{};
  if (int rc = fill_silu_mul(&p, gate, up, dtype, rows, cols, ld_gate, ld_up)) return rc;
  return launch_dense<kSiluMul>(dtype, p, h_out, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_silu_mul_dense_scale(const void* gate, const void* up, int dtype, int64_t rows,
                                       int64_t cols, int64_t ld_gate, int64_t ld_up, void* h_out,
                                       float* scale_out, void* ws, size_t ws_bytes, void* stream) {
  if (!h_out || !scale_out) return bq::kErrBadArg;
  if (!aligned_to(h_out, 16)) return bq::kErrUnsupported;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  QParams p{};
  if (int rc = fill_silu_mul(&p, gate, up, dtype, rows, cols, ld_gate, ld_up)) return rc;
  p.scale = scale_out;
  p.ws = ws;
  return launch_dense<kSiluMul>(dtype, p, h_out, static_cast<cudaStream_t>(stream));
}

namespace {
int sigmoid_mul_common(const void* o, const void* gate, int dtype, int64_t rows, int64_t cols,
                       int64_t ld_o, int64_t ld_gate, int64_t chunk, int64_t chunk_stride, void* out,
                       float* scale_out, void* ws, void* stream);
}

extern "C" int bq_sigmoid_mul_dense_scale(const void* o, const void* gate, int dtype, int64_t rows,
                                          int64_t cols, int64_t ld_o, int64_t ld_gate, int64_t chunk,
                                          int64_t chunk_stride, void* out, float* scale_out, void* ws,
                                          size_t ws_bytes, void* stream) {
  if (!scale_out) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  return sigmoid_mul_common(o, gate, dtype, rows, cols, ld_o, ld_gate, chunk, chunk_stride, out,
                            scale_out, ws, stream);
}

extern "C" int bq_sigmoid_mul(const void* o, const void* gate, int dtype, int64_t rows, int64_t cols,
                              int64_t ld_o, int64_t ld_gate, int64_t chunk, int64_t chunk_stride,
                              void* out, void* stream) {
  return sigmoid_mul_common(o, gate, dtype, rows, cols, ld_o, ld_gate, chunk, chunk_stride, out,
                            nullptr, nullptr, stream);
}

namespace {
int sigmoid_mul_common(const void* o, const void* gate, int dtype, int64_t rows, int64_t cols,
                       int64_t ld_o, int64_t ld_gate, int64_t chunk, int64_t chunk_stride, void* out,
                       float* scale_out, void* ws, void* stream) {
  if (!o || !gate || !out || rows <= 0 || cols <= 0 || chunk <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  const size_t es = elem_size(dtype);
  if (cols % kGroup || chunk % kGroup || cols % chunk || ld_o < cols || (ld_o * es) % 16 ||
      (ld_gate * es) % 16 || (chunk_stride * es) % 16 || !aligned_to(o, 16) ||
      !aligned_to(gate, 16) || !aligned_to(out, 16))
    return bq::kErrUnsupported;
  if (rows * (cols / kGroup) >= 0x7fffffffLL) return bq::kErrTooLarge;
  QParams p{};
  p.a = o;
  p.b = gate;
  p.groups_per_row = static_cast<unsigned int>(cols / kGroup);
  p.n_groups = static_cast<unsigned int>(rows * (cols / kGroup));
  p.ld_a = ld_o;
  p.ld_b = ld_gate;
  p.chunk = static_cast<unsigned int>(chunk);
  p.chunk_stride = chunk_stride;
  p.scale = scale_out;
  p.ws = ws;
  return launch_dense<kSigmoidGate>(dtype, p, out, static_cast<cudaStream_t>(stream));
}
}  // namespace

namespace {
template <bool CAST>
int launch_row_push(int dtype, const RowPush& p, cudaStream_t stream) {
  const int sms = device_sms();
  if (sms <= 0) return bq::kErrLaunch;
  const bool pdl = g_opt_quant_pdl != 0;
  cudaError_t e;
  switch (dtype) {
    case BQ_DTYPE_F32: e = launch_resident(row_push_kernel<float, CAST>, p.rows, 256, sms, pdl, stream, p); break;
    case BQ_DTYPE_BF16:
      e = launch_resident(row_push_kernel<__nv_bfloat16, CAST>, p.rows, 256, sms, pdl, stream, p);
      break;
    case BQ_DTYPE_F16: e = launch_resident(row_push_kernel<__half, CAST>, p.rows, 256, sms, pdl, stream, p); break;
    default: return bq::kErrBadArg;
  }
  if (e != cudaSuccess) { (void)cudaGetLastError(); return bq::kErrLaunch; }
  return bq::kOk;
}

int fill_row_push(RowPush* p, const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                  int n_peers, void* const* dst, int64_t ld_dst, void* const* flags, void* ws,
                  size_t ws_bytes, size_t out_elem) {
  if (!x || !dst || !flags || rows <= 0 || cols <= 0 || n_peers < 1 || n_peers > 8) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (int rc = check_ws(ws, ws_bytes)) return rc;
  const size_t es = elem_size(dtype);
  if (cols % kGroup || ld_x < cols || (ld_x * es) % 16 || !aligned_to(x, 16) || ld_dst < cols ||
      (ld_dst * out_elem) % (8 * out_elem > 16 ? 16 : 8 * out_elem))
    return bq::kErrUnsupported;
  if (rows > 0x7fffffffLL || cols > 0x7fffffffLL) return bq::kErrTooLarge;
  memset(p, 0, sizeof(*p));
  p->src = x;
  p->ld_src = ld_x;
  p->rows = (int)rows;
  p->groups_per_row = (int)(cols / kGroup);
  p->n = n_peers;
  p->ld_dst = ld_dst;
  p->done = static_cast<unsigned int*>(ws);
  for (int i = 0; i < n_peers; ++i) {
    if (!dst[i] || !flags[i]) return bq::kErrBadArg;
    if (!aligned_to(dst[i], 8 * out_elem > 16 ? 16 : 8 * out_elem) || !aligned_to(flags[i], 4))
      return bq::kErrUnsupported;
    p->dst[i] = dst[i];
    p->flag[i] = static_cast<unsigned int*>(flags[i]);
  }
  return bq::kOk;
}
}  // namespace

extern "C" int bq_cast_act_push(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                const float* scale, int n_peers, void* const* q_dst, int64_t ld_q,
                                void* const* flags, void* ws, size_t ws_bytes, void* stream) {
  if (!scale) return bq::kErrBadArg;
  RowPush p;
  if (int rc = fill_row_push(&p, x, dtype, rows, cols, ld_x, n_peers, q_dst, ld_q, flags, ws, ws_bytes, 1))
    return rc;
  p.scale = scale;
  p.wide = (cols % 16 == 0 && ld_q % 16 == 0) ? 1 : 0;
  for (int i = 0; i < n_peers; ++i)
    if (!aligned_to(q_dst[i], 16)) p.wide = 0;
  return launch_row_push<true>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int bq_rows_push(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                            int n_peers, void* const* dst, int64_t ld_dst, void* const* flags,
                            void* ws, size_t ws_bytes, void* stream) {
  RowPush p;
  if (int rc = fill_row_push(&p, x, dtype, rows, cols, ld_x, n_peers, dst, ld_dst, flags, ws, ws_bytes,
                             elem_size(dtype)))
    return rc;
  return launch_row_push<false>(dtype, p, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Quantizer entry point that needs no scratch buffer from the caller
// ---------------------------------------------------------------------------
// Some hosts of this library cannot hand it device memory of their own making:
// a runtime that owns every byte of the GPU through its own arena and forbids
// cudaMalloc after start-up, a plugin called from inside a region where the
// host's allocator is locked or a real-time style loop with a no-allocation
// rule, or a thin FFI shim in a language where creating and zeroing a device
// buffer is more machinery than the call itself.
// For them the 16 bytes of barrier words live in the library's own image.
//
// The array below is device memory reserved when the library is loaded on a
// GPU and kept until the process exits (BQ_STATIC_SCRATCH_BYTES per GPU that
// loads the library).  Inside host code its NAME is only a handle, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, asked
// once per device with that device current, and cached.
static __device__ __align__(256) unsigned int g_static_scratch[BQ_STATIC_SCRATCH_BYTES / 4];

namespace {

// Device address of g_static_scratch on the current device (0 on failure).
QuantWs* static_scratch_for_current_device(int* rc_out) {
  static QuantWs* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc_out = bq::kErrLaunch;
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      *rc_out = bq::kErrLaunch;
      return nullptr;
    }
    cached[dev] = static_cast<QuantWs*>(ptr);
  }
  *rc_out = bq::kOk;
  return cached[dev];
}

}  // namespace

extern "C" int bq_quantize_act_static(const void* x, int dtype, int64_t n, void* q_out,
                                      float* scale_out, void* stream) {
  if (x == nullptr || q_out == nullptr || scale_out == nullptr || n <= 0) return bq::kErrBadArg;
  if (dtype != BQ_DTYPE_F32 && dtype != BQ_DTYPE_BF16 && dtype != BQ_DTYPE_F16) return bq::kErrBadArg;
  if (n > BQ_STATIC_MAX_ELEMENTS) return bq::kErrTooLarge;
  if (!aligned_to(x, 16) || !aligned_to(q_out, 8)) return bq::kErrUnsupported;
  int rc = bq::kOk;
  QuantWs* ws = static_scratch_for_current_device(&rc);
  if (ws == nullptr) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  The kernels return the
  // amax word and the two counters to zero themselves, but a call that was cut
  // short (a wait that ran out) would not have: clear the three words that must
  // start at zero, in stream order, and leave the sticky status word alone.
  if (cudaMemsetAsync(ws, 0, 3 * sizeof(unsigned int), s) != cudaSuccess) {
    (void)cudaGetLastError();
    return bq::kErrLaunch;
  }
  QParams p{};
  p.a = x;
  p.q = static_cast<uint8_t*>(q_out);
  p.scale = scale_out;
  p.ws = ws;
  p.n_groups = static_cast<unsigned int>(n / kGroup);
  p.tail = static_cast<unsigned int>(n % kGroup);
  p.groups_per_row = 1;
  return dispatch_dtype<kPlain>(dtype, p, s);
}
