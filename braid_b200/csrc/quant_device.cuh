// Device-side building blocks of the FP8 activation quantizer, shared by the stand-alone
// quantizer kernels (quant_act.cu, norm_quant.cu) and the paired gate/up epilogue (gemm_w8a8.cu).
// The arithmetic is the reference's torch spelling as a CUDA device evaluates it
// (braid/model/quant.py:108-115, :228-229): reciprocal-multiply scale, IEEE division, clamp to
// +-448 (NaN survives), NaN-propagating max, round-to-nearest-even e4m3 cast; the
// prologues keep the per-operation rounding of the separate torch kernels
// (braid/model/mlp.py:48, braid/model/attention.py:215).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <type_traits>

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

// max(m, |v[0..7]|), NaN-propagating.  The 16-bit types take the maximum on packed pairs
// (`abs` and `max.NaN` on two values per instruction; the maximum of 16-bit values is one of
// them, so nothing is rounded) and widen once at the end.
template <typename T>
__device__ __forceinline__ float absmax8(const Pack8<T>& v, float m) {
  if constexpr (sizeof(T) == 2) {
    using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
    const T2* w = reinterpret_cast<const T2*>(&v);
    const T2 m01 = __hmax2_nan(__habs2(w[0]), __habs2(w[1]));
    const T2 m23 = __hmax2_nan(__habs2(w[2]), __habs2(w[3]));
    const T2 mm = __hmax2_nan(m01, m23);
    m = nan_max(m, widen(mm.x));
    m = nan_max(m, widen(mm.y));
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = nan_max(m, fabsf(widen(v.v[i])));
  }
  return m;
}

// x / sc for a divisor every element of the tensor shares, with the bits of the IEEE division
// the reference spells (`x / scale`): the reciprocal is rounded once (`__frcp_rn`), and every
// element takes a product and two residual corrections.  After the first correction the
// quotient is within one unit in the last place, so the second one rounds correctly
// (Markstein's division step: y = RN(1/b), q faithful, r = a - b*q exact, RN(q + r*y) =
// RN(a/b)).  That holds while nothing leaves the normal range: the scale has to lie in
// [2^-60, 2^60], a quotient that overflows or an operand that is not finite shows as a NaN and
// takes the division instruction instead, and quotients too small for the corrections to be
// exact are far below half of the smallest e4m3 step, where only the sign reaches the code
// (hence the copysign, which also keeps -0).
struct ScaleDiv {
  float sc, inv;
  bool fast;
  __device__ __forceinline__ explicit ScaleDiv(float s) {
    sc = s;
    inv = __frcp_rn(s);
    fast = s >= 0x1p-60f && s <= 0x1p60f;
  }
  // The quotient by the corrections alone; NaN where the division instruction has to decide.
  __device__ __forceinline__ float corrected(float x) const {
    float q = __fmul_rn(x, inv);
    float r = __fmaf_rn(-q, sc, x);
    q = __fmaf_rn(r, inv, q);
    r = __fmaf_rn(-q, sc, x);
    return copysignf(__fmaf_rn(r, inv, q), x);
  }
};

// x[i] <- x[i] / sc for the N values of one group: one test for the whole group decides
// between the corrected products and N division instructions.  OWN_SCALE says the scale was
// taken from the very values being divided (sc = max|x| / 448, clamped from below): then a
// scale inside the range means every x is finite and no quotient exceeds 448, and the test
// for NaN among the results is left out.  What goes on to the saturating e4m3 conversion is
// the bare quotient: the reference clamps to +-448 before its (non-saturating) cast,
// `cvt.rn.satfinite` does the same clamp itself (finite values and infinities beyond the
// range become +-448, NaN stays NaN).
template <int N, bool OWN_SCALE = false>
__device__ __forceinline__ void divide_group(const ScaleDiv& d, float (&x)[N]) {
  float q[N];
  bool ok = d.fast;
#pragma unroll
  for (int i = 0; i < N; ++i) {
    q[i] = d.corrected(x[i]);
    if constexpr (!OWN_SCALE) ok = ok && (q[i] == q[i]);
  }
  if (ok) {
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = q[i];
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = __fdiv_rn(x[i], d.sc);
  }
}

__device__ __forceinline__ float quant_one(float x, const ScaleDiv& d) {
  float v[1] = {x};
  divide_group<1>(d, v);
  return v[0];
}

// the 8 e4m3 codes of one group, as two 32-bit words
template <typename T, bool OWN_SCALE = false>
__device__ __forceinline__ uint2 codes8(const Pack8<T>& v, const ScaleDiv& sc) {
  float f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = widen(v.v[i]);
  divide_group<8, OWN_SCALE>(sc, f);
  uint32_t w[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[half * 4], f[half * 4 + 1]), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[half * 4 + 2], f[half * 4 + 3]), __NV_SATFINITE, __NV_E4M3);
    w[half] = (lo & 0xFFFFu) | ((hi & 0xFFFFu) << 16);
  }
  return make_uint2(w[0], w[1]);
}

template <typename T, bool OWN_SCALE = false>
__device__ __forceinline__ void emit8(const Pack8<T>& v, const ScaleDiv& sc, uint8_t* dst) {
  *reinterpret_cast<uint2*>(dst) = codes8<T, OWN_SCALE>(v, sc);
}

__device__ __forceinline__ float scale_from_amax(float amax) {
  const float raw = amax * kInvFp8Max;
  return (raw < kEps) ? kEps : raw;   // NaN compares false and stays NaN
}

// x / (1 + exp(-x)) and 1 / (1 + exp(-x)) rounded to T as torch evaluates F.silu and
// torch.sigmoid of a T tensor on a CUDA device: fp32, expf, an IEEE division, one rounding.
// (Taking ex2/rcp approximations wherever the rounding to a 16-bit T hides them, with the exact
// instructions for values near a rounding tie, passed the exhaustive test but measured slower:
// the guard and the divergent exact path cost what the approximations saved.)
template <typename T> __device__ __forceinline__ T silu_to(float x) {
  return narrow<T>(__fdiv_rn(x, 1.0f + expf(-x)));
}
template <typename T> __device__ __forceinline__ T sigmoid_to(float x) {
  return narrow<T>(__fdiv_rn(1.0f, 1.0f + expf(-x)));
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
        const T sl = silu_to<T>(x);
        a.v[i] = narrow<T>(widen(sl) * widen(b.v[i]));
      } else {
        const float gt = widen(b.v[i]);
        const T sg = sigmoid_to<T>(gt);
        a.v[i] = narrow<T>(widen(a.v[i]) * widen(sg));
      }
    }
  }
}


}  // namespace qd
}  // namespace bq
