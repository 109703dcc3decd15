// Device-side building blocks of the FP8 activation quantizer, shared by the stand-alone
// quantizer kernels (quant_act.cu, norm_quant.cu) and the paired gate/up epilogue (gemm_w8a8.cu).
// The arithmetic is the reference's torch spelling as a CUDA device evaluates it
// (braid/model/quant.py:108-115, :228-229): reciprocal-multiply scale, IEEE division,
// comparison clamps (NaN survives), NaN-propagating max, round-to-nearest-even e4m3 cast; the
// prologues keep the per-operation rounding of the separate torch kernels
// (braid/model/mlp.py:48, braid/model/attention.py:215).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bq {
namespace qd {

constexpr float kFp8Max = 448.0f;
// torch divides a tensor by a host scalar as t * (1/scalar) in fp32.
constexpr float kInvFp8Max = 1.0f / 448.0f;
constexpr float kEps = 1e-12f;

constexpr int kGroup = 8;      // elements per group (one 128-bit load of a 16-bit type)

enum Mode { kPlain = 0, kSiluMul = 1, kSigmoidGate = 2 };

struct QParams {
  const void* a;        // x | gate | o
  const void* b;        // - | up   | gate
  uint8_t* q;
  float* scale;
  void* ws;             // kernel-specific scratch words
  unsigned int n_groups;      // full groups of 8
  unsigned int tail;          // plain mode only: leftover elements (< 8)
  unsigned int groups_per_row;
  long long ld_a, ld_b;       // row strides in elements (prologue modes)
  unsigned int chunk;         // sigmoid gate: head width of the strided gate view
  long long chunk_stride;     // sigmoid gate: distance between heads
  int held;                   // groups each thread keeps (hold kernel)
  // column-parallel form: the input is a gathered buffer other ranks store into; wait until the
  // arrival counter has advanced by wait_count beyond *wait_seen before loading (nullptr = no wait)
  const unsigned int* wait_flag;
  unsigned int* wait_seen;
  unsigned int wait_count;
  unsigned long long* phase_ring;   // development builds (BQ_PHASES) only, else nullptr
  int phase_seq;
};

template <typename T> struct alignas(16) Pack8 { T v[8]; };
template <> struct alignas(16) Pack8<float> { float v[8]; };

__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// NaN-propagating max: once either side is NaN the result is NaN.
__device__ __forceinline__ float nan_max(float m, float v) { return (v != v || v > m) ? v : m; }

// COHERENT = false: read-only path (`ld.global.nc`), for inputs nobody writes while the kernel
// is resident.  COHERENT = true: L2-coherent loads (`ld.global.cg`), for a gathered buffer that
// other GPUs (and this GPU's own push launch) are still storing into while this kernel waits
// for their arrival -- the non-coherent path promises nothing for such data.
template <typename T, bool COHERENT = false>
__device__ __forceinline__ Pack8<T> load8(const T* p) {
  Pack8<T> r;
  if constexpr (sizeof(T) == 4) {
    const float4* q = reinterpret_cast<const float4*>(p);
    const float4 lo = COHERENT ? __ldcg(q) : __ldg(q);
    const float4 hi = COHERENT ? __ldcg(q + 1) : __ldg(q + 1);
    r.v[0] = lo.x; r.v[1] = lo.y; r.v[2] = lo.z; r.v[3] = lo.w;
    r.v[4] = hi.x; r.v[5] = hi.y; r.v[6] = hi.z; r.v[7] = hi.w;
  } else {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    const uint4 raw = COHERENT ? __ldcg(q) : __ldg(q);
    *reinterpret_cast<uint4*>(&r) = raw;
  }
  return r;
}

template <typename T>
__device__ __forceinline__ float absmax8(const Pack8<T>& v, float m) {
#pragma unroll
  for (int i = 0; i < 8; ++i) m = nan_max(m, fabsf(widen(v.v[i])));
  return m;
}

__device__ __forceinline__ float quant_one(float x, float sc) {
  float v = __fdiv_rn(x, sc);
  // comparison clamps: both are false for NaN, which therefore falls through
  v = (v < -kFp8Max) ? -kFp8Max : ((v > kFp8Max) ? kFp8Max : v);
  return v;
}

template <typename T>
__device__ __forceinline__ void emit8(const Pack8<T>& v, float sc, uint8_t* dst) {
  uint32_t w[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = half * 4 + j * 2;
      const float2 f = make_float2(quant_one(widen(v.v[i]), sc), quant_one(widen(v.v[i + 1]), sc));
      const uint32_t pair = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
      word |= (pair & 0xFFFFu) << (16 * j);
    }
    w[half] = word;
  }
  *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
}

__device__ __forceinline__ float scale_from_amax(float amax) {
  const float raw = amax * kInvFp8Max;
  return (raw < kEps) ? kEps : raw;   // NaN compares false and stays NaN
}

// Raw operands of one group: one 8-pack for the plain mode, two for the prologues.
template <typename T, int MODE, bool COHERENT = false>
__device__ __forceinline__ void load_raw(const QParams& p, unsigned int g, Pack8<T>& a, Pack8<T>& b) {
  if constexpr (MODE == kPlain) {
    a = load8<T, COHERENT>(reinterpret_cast<const T*>(p.a) + static_cast<size_t>(g) * kGroup);
  } else {
    const unsigned int row = g / p.groups_per_row;
    const unsigned int col = (g - row * p.groups_per_row) * kGroup;
    const T* pa = reinterpret_cast<const T*>(p.a) + static_cast<long long>(row) * p.ld_a + col;
    const T* pb;
    if constexpr (MODE == kSiluMul) {
      pb = reinterpret_cast<const T*>(p.b) + static_cast<long long>(row) * p.ld_b + col;
    } else {
      const unsigned int head = col / p.chunk;
      pb = reinterpret_cast<const T*>(p.b) + static_cast<long long>(row) * p.ld_b +
           static_cast<long long>(head) * p.chunk_stride + (col - head * p.chunk);
    }
    a = load8<T, COHERENT>(pa);
    b = load8<T, COHERENT>(pb);
  }
}

// a <- the activation values (in place); plain mode is the identity.
template <typename T, int MODE>
__device__ __forceinline__ void apply_prologue(Pack8<T>& a, const Pack8<T>& b) {
  if constexpr (MODE != kPlain) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (MODE == kSiluMul) {
        // silu in fp32, rounded to T; product in fp32, rounded to T
        const float x = widen(a.v[i]);
        const T sl = narrow<T>(__fdiv_rn(x, 1.0f + expf(-x)));
        a.v[i] = narrow<T>(widen(sl) * widen(b.v[i]));
      } else {
        const float gt = widen(b.v[i]);
        const T sg = narrow<T>(__fdiv_rn(1.0f, 1.0f + expf(-gt)));
        a.v[i] = narrow<T>(widen(a.v[i]) * widen(sg));
      }
    }
  }
}


}  // namespace qd
}  // namespace bq
