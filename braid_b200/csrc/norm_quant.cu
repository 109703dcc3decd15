// RMSNorm fused into the FP8 activation quantizer, one launch each:
//
//   bq_rmsnorm_quant        h = rms_norm(x, gamma, eps)            -> (h), e4m3 codes, scale
//                           braid/model/norm.py:31-45 feeding `project` / the MLP
//                           (braid/model/layer.py:49,59 -> gdn.py:254, attention.py:173, mlp.py:45)
//   bq_gated_rmsnorm_quant  core = rms_norm_gated(y, z, gamma, eps) -> e4m3 codes, scale
//                           braid/model/norm.py:48-71 feeding out_proj (braid/model/gdn.py:373-387)
//
// The result has to be bit-identical to the reference's torch spelling on a CUDA device, and a
// sum of squares is not order-free, so the reduction restates the arithmetic of the kernel torch
// runs for `F.rms_norm` on an fp32 row (its vectorized layer-norm kernel in the rms_norm mode,
// one CTA of 32 x 4 threads per row): thread t accumulates the 4-element vectors t, t+128, ...
// in order as s = fma(v, v, s); lanes combine by shuffle-down (16, 8, 4, 2, 1); the four warps
// combine as (w0 + w2) + (w1 + w3); sigma2 = s / float(N) (IEEE division);
// rstd = rsqrtf(sigma2 + eps); y = gamma * (rstd * x) in fp32, then ONE rounding to the
// activation type.  The gated form normalises without gamma, rounds to the activation type,
// multiplies by gamma in fp32, multiplies by silu(z) evaluated in fp32 (x / (1 + expf(-x))) and
// rounds once more.  tests/test_norm_quant_gpu.py pins all of this against torch on the device.
//
// After the norm the values stay in registers; amax, grid-wide exchange and cast are the
// activation quantizer's (quant_act.cu).  One CTA per token row, so grids are <= 2048 rows
// (all CTAs must be co-resident for the exchange); larger inputs are refused and the caller runs
// the norm and the quantizer separately.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/braid_b200.h"
#include "ptx.cuh"
#include "quant_device.cuh"
#include "grid_amax.cuh"

namespace {

using namespace bq::qd;

constexpr int kNormThreads = 128;   // 32 x 4, the block shape whose reduction order is restated
constexpr int kVec = 4;

struct NormParams {
  const void* x;
  const float* gamma;
  void* h_out;        // optional normalised activation in the activation type
  uint8_t* q;
  float* scale;
  void* ws;
  int rows, cols;
  long long ld_x, ld_h;
  float eps;
};

template <typename T> struct Vec4 { T v[kVec]; };

template <typename T>
__device__ __forceinline__ Vec4<T> load4(const T* p) {
  Vec4<T> r;
  if constexpr (sizeof(T) == 4) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(p));
    r.v[0] = f.x; r.v[1] = f.y; r.v[2] = f.z; r.v[3] = f.w;
  } else {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    *reinterpret_cast<uint2*>(&r) = raw;
  }
  return r;
}

template <typename T>
__device__ __forceinline__ void store4(T* p, const Vec4<T>& v) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v.v[0], v.v[1], v.v[2], v.v[3]);
  } else {
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(&v);
  }
}

template <typename T>
__device__ __forceinline__ void emit4(const Vec4<T>& v, const ScaleDiv& sc, uint8_t* dst) {
  float f[4] = {widen(v.v[0]), widen(v.v[1]), widen(v.v[2]), widen(v.v[3])};
  divide_group<4, true>(sc, f);   // the scale is that of these very values
  const uint32_t a = __nv_cvt_float2_to_fp8x2(make_float2(f[0], f[1]), __NV_SATFINITE, __NV_E4M3);
  const uint32_t b = __nv_cvt_float2_to_fp8x2(make_float2(f[2], f[3]), __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(dst) = (a & 0xFFFFu) | ((b & 0xFFFFu) << 16);
}

// Lane 0 of the warp ends up with the shuffle-down tree sum (the other lanes hold partial
// garbage, as in the kernel this restates).
__device__ __forceinline__ float warp_tree_sum(float s) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xffffffffu, s, off));
  return s;
}

// ---------------------------------------------------------------------------------------------
// plain RMSNorm -> quantize.  One CTA of 128 threads per row; VPT = vectors held per thread.
// ---------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_quant_kernel(const NormParams p) {
  bq::pdl_launch_dependents();
  __shared__ float s_red[4];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int row = blockIdx.x;
  const int n_vec = p.cols / kVec;
  const T* xr = reinterpret_cast<const T*>(p.x) + static_cast<long long>(row) * p.ld_x;
  // gamma is a weight, not the previous kernel's output: fetch it before the dependency wait
  float g[VPT][kVec];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * kNormThreads;
    if (v < n_vec) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(p.gamma) + v);
      g[i][0] = f.x; g[i][1] = f.y; g[i][2] = f.z; g[i][3] = f.w;
    }
  }
  bq::pdl_wait_prior_grids();
  Vec4<T> x[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * kNormThreads;
    if (v < n_vec) x[i] = load4(xr + v * kVec);
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * kNormThreads;
    if (v < n_vec) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const float f = widen(x[i].v[j]);
        s = __fmaf_rn(f, f, s);
      }
    }
  }
  s = warp_tree_sum(s);
  if (lane == 0 && warp >= 2) s_red[warp - 2] = s;
  __syncthreads();
  if (lane == 0 && warp < 2) s = __fadd_rn(s, s_red[warp]);
  __syncthreads();
  if (lane == 0 && warp == 1) s_red[0] = s;
  __syncthreads();
  if (t == 0) s_red[1] = __fdiv_rn(__fadd_rn(s, s_red[0]), static_cast<float>(p.cols));
  __syncthreads();
  const float rstd = rsqrtf(__fadd_rn(s_red[1], p.eps));

  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * kNormThreads;
    if (v < n_vec) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const float y = __fmul_rn(g[i][j], __fmul_rn(rstd, widen(x[i].v[j])));
        x[i].v[j] = narrow<T>(y);
        m = nan_max(m, fabsf(widen(x[i].v[j])));
      }
    }
  }
  if (p.h_out != nullptr) {
    T* hr = reinterpret_cast<T*>(p.h_out) + static_cast<long long>(row) * p.ld_h;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * kNormThreads;
      if (v < n_vec) store4(hr + v * kVec, x[i]);
    }
  }
  const float sc = scale_from_amax(grid_amax(m, static_cast<QuantWs*>(p.ws)));
  const ScaleDiv dv(sc);
  if (blockIdx.x == 0 && t == 0) p.scale[0] = sc;
  uint8_t* qr = p.q + static_cast<long long>(row) * p.cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t + i * kNormThreads;
    if (v < n_vec) emit4(x[i], dv, qr + v * kVec);
  }
  grid_depart(static_cast<QuantWs*>(p.ws));
}

// ---------------------------------------------------------------------------------------------
// plain RMSNorm at prefill sizes: more rows than one co-resident grid has CTAs.  Every CTA loops
// over rows (row arithmetic exactly as above), writes the normalised activation h, and keeps the
// running max |h|; nobody waits for anybody: each CTA folds its max into one word with an
// atomicMax and counts itself, and the CTA that counts last turns the word into the scale and
// returns the scratch to zero.  The codes are then one cast pass over h under that scale
// (bq_cast_act), in stream order.
// ---------------------------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_scale_kernel(const NormParams p) {
  bq::pdl_launch_dependents();
  __shared__ float s_red[4];
  __shared__ float s_max[4];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int n_vec = p.cols / kVec;
  // gamma lives in shared memory here, not in registers: a CTA normalises many rows, and 32
  // registers less per thread are three more CTAs per SM to hide the loads behind
  extern __shared__ float4 s_gamma[];
  for (int v = t; v < n_vec; v += kNormThreads) s_gamma[v] = __ldg(reinterpret_cast<const float4*>(p.gamma) + v);
  __syncthreads();
  bq::pdl_wait_prior_grids();
  float m = 0.0f;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* xr = reinterpret_cast<const T*>(p.x) + static_cast<long long>(row) * p.ld_x;
    Vec4<T> x[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * kNormThreads;
      if (v < n_vec) x[i] = load4(xr + v * kVec);
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * kNormThreads;
      if (v < n_vec) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float f = widen(x[i].v[j]);
          s = __fmaf_rn(f, f, s);
        }
      }
    }
    s = warp_tree_sum(s);
    if (lane == 0 && warp >= 2) s_red[warp - 2] = s;
    __syncthreads();
    if (lane == 0 && warp < 2) s = __fadd_rn(s, s_red[warp]);
    __syncthreads();
    if (lane == 0 && warp == 1) s_red[0] = s;
    __syncthreads();
    if (t == 0) s_red[1] = __fdiv_rn(__fadd_rn(s, s_red[0]), static_cast<float>(p.cols));
    __syncthreads();
    const float rstd = rsqrtf(__fadd_rn(s_red[1], p.eps));
    T* hr = reinterpret_cast<T*>(p.h_out) + static_cast<long long>(row) * p.ld_h;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * kNormThreads;
      if (v < n_vec) {
        const float4 gv = s_gamma[v];
        const float g[kVec] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float y = __fmul_rn(g[j], __fmul_rn(rstd, widen(x[i].v[j])));
          x[i].v[j] = narrow<T>(y);
          m = nan_max(m, fabsf(widen(x[i].v[j])));
        }
        store4(hr + v * kVec, x[i]);
      }
    }
    __syncthreads();   // s_red is written again by the next row
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, off));
  if (lane == 0) s_max[warp] = m;
  __syncthreads();
  if (t == 0) {
    float w = s_max[0];
    for (int i = 1; i < kNormThreads / 32; ++i) w = nan_max(w, s_max[i]);
    QuantWs* ws = static_cast<QuantWs*>(p.ws);
    // |h| >= 0 or NaN with the sign cleared: bit patterns order like the values, NaN on top
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

// ---------------------------------------------------------------------------------------------
// gated RMSNorm (per 128-wide head) -> quantize.  One CTA per token row, one warp per head
// (warps loop when there are more heads than warps); a lane owns one 4-element vector of a head.
// ---------------------------------------------------------------------------------------------
struct GatedParams {
  const void* y;       // scan output, fp32 or the activation type
  const void* z;       // gate, the activation type
  const float* gamma;  // [128]
  void* h_out;         // looped form: the gated, normalised activation [rows, heads * 128]
  long long ld_h;
  uint8_t* q;
  float* scale;
  void* ws;
  int rows, heads;
  long long ld_y, ld_z;
  float eps;
};

constexpr int kHeadDim = 128;
constexpr int kGatedWarps = 8;
constexpr int kMaxHeadsPerWarp = 8;    // up to 64 heads

template <typename T, bool Y_F32, int HPW>
__global__ void __launch_bounds__(kGatedWarps * 32) gated_rmsnorm_quant_kernel(const GatedParams p) {
  bq::pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x;
  const float4 gm = __ldg(reinterpret_cast<const float4*>(p.gamma) + lane);
  const float gmv[kVec] = {gm.x, gm.y, gm.z, gm.w};
  bq::pdl_wait_prior_grids();
  Vec4<T> core[HPW];
  Vec4<T> gate[HPW];
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int head = warp + i * kGatedWarps;
    if (head < p.heads) {
      const long long off = static_cast<long long>(head) * kHeadDim + lane * kVec;
      if constexpr (Y_F32) {
        // the reference rounds the scan output to the activation type first (gdn.py:383)
        const float4 f = __ldg(reinterpret_cast<const float4*>(
            reinterpret_cast<const float*>(p.y) + static_cast<long long>(row) * p.ld_y + off));
        core[i].v[0] = narrow<T>(f.x); core[i].v[1] = narrow<T>(f.y);
        core[i].v[2] = narrow<T>(f.z); core[i].v[3] = narrow<T>(f.w);
      } else {
        core[i] = load4(reinterpret_cast<const T*>(p.y) + static_cast<long long>(row) * p.ld_y + off);
      }
      gate[i] = load4(reinterpret_cast<const T*>(p.z) + static_cast<long long>(row) * p.ld_z + off);
    }
  }
  float m = 0.0f;
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int head = warp + i * kGatedWarps;   // warp-uniform
    if (head < p.heads) {
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const float f = widen(core[i].v[j]);
        s = __fmaf_rn(f, f, s);
      }
      s = warp_tree_sum(s);
      s = __shfl_sync(0xffffffffu, s, 0);
      // the three idle warps of the restated kernel contribute exact zeros
      const float sigma2 = __fdiv_rn(s, static_cast<float>(kHeadDim));
      const float rstd = rsqrtf(__fadd_rn(sigma2, p.eps));
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const T xn = narrow<T>(__fmul_rn(rstd, widen(core[i].v[j])));
        const float zf = widen(gate[i].v[j]);
        const float silu = __fdiv_rn(zf, 1.0f + expf(-zf));
        const float h = __fmul_rn(__fmul_rn(gmv[j], widen(xn)), silu);
        core[i].v[j] = narrow<T>(h);
        m = nan_max(m, fabsf(widen(core[i].v[j])));
      }
    }
  }
  const float sc = scale_from_amax(grid_amax(m, static_cast<QuantWs*>(p.ws)));
  const ScaleDiv dv(sc);
  if (blockIdx.x == 0 && threadIdx.x == 0) p.scale[0] = sc;
  uint8_t* qr = p.q + static_cast<long long>(row) * p.heads * kHeadDim;
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int head = warp + i * kGatedWarps;
    if (head < p.heads) emit4(core[i], dv, qr + head * kHeadDim + lane * kVec);
  }
  grid_depart(static_cast<QuantWs*>(p.ws));
}

// ---------------------------------------------------------------------------------------------
template <typename Kernel, typename Params>
int launch_rows(Kernel kernel, int rows, int threads, const Params& p, cudaStream_t stream) {
  // every CTA waits for every other: the whole grid must fit on the device at once
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess) {
    (void)cudaGetLastError();
    return bq::kErrLaunch;
  }
  if (static_cast<long long>(rows) > static_cast<long long>(sms) * per_sm) return bq::kErrTooLarge;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return bq::kErrLaunch; }
  return bq::kOk;
}

template <typename T>
int launch_rmsnorm(const NormParams& p, cudaStream_t stream) {
  const int per_thread = (p.cols / kVec + kNormThreads - 1) / kNormThreads;
  if (per_thread <= 2) return launch_rows(rmsnorm_quant_kernel<T, 2>, p.rows, kNormThreads, p, stream);
  if (per_thread <= 4) return launch_rows(rmsnorm_quant_kernel<T, 4>, p.rows, kNormThreads, p, stream);
  if (per_thread <= 8) return launch_rows(rmsnorm_quant_kernel<T, 8>, p.rows, kNormThreads, p, stream);
  if (per_thread <= 16) return launch_rows(rmsnorm_quant_kernel<T, 16>, p.rows, kNormThreads, p, stream);
  return bq::kErrUnsupported;
}

template <typename T, bool Y_F32>
int launch_gated(const GatedParams& p, cudaStream_t stream) {
  const int hpw = (p.heads + kGatedWarps - 1) / kGatedWarps;
  const int threads = kGatedWarps * 32;
  if (hpw <= 1) return launch_rows(gated_rmsnorm_quant_kernel<T, Y_F32, 1>, p.rows, threads, p, stream);
  if (hpw <= 2) return launch_rows(gated_rmsnorm_quant_kernel<T, Y_F32, 2>, p.rows, threads, p, stream);
  if (hpw <= 4) return launch_rows(gated_rmsnorm_quant_kernel<T, Y_F32, 4>, p.rows, threads, p, stream);
  if (hpw <= kMaxHeadsPerWarp)
    return launch_rows(gated_rmsnorm_quant_kernel<T, Y_F32, kMaxHeadsPerWarp>, p.rows, threads, p, stream);
  return bq::kErrUnsupported;
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t elem_size(int dtype) { return dtype == BQ_DTYPE_F32 ? 4 : 2; }
inline bool known_dtype(int d) { return d == BQ_DTYPE_F32 || d == BQ_DTYPE_BF16 || d == BQ_DTYPE_F16; }

}  // namespace

// The gated norm for more rows than one co-resident grid has CTAs (prefill): a warp owns one
// head of one row at a time (head arithmetic exactly as above; no CTA-wide step in it), the
// warps of the grid stride over all (row, head) pairs, write the gated activation and fold
// max |h| into one word as rmsnorm_scale_kernel does; the cast pass follows in stream order.
template <typename T, bool Y_F32>
__global__ void __launch_bounds__(kGatedWarps * 32) gated_rmsnorm_scale_kernel(const GatedParams p) {
  bq::pdl_launch_dependents();
  __shared__ float s_max[kGatedWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float4 gm = __ldg(reinterpret_cast<const float4*>(p.gamma) + lane);
  const float gmv[kVec] = {gm.x, gm.y, gm.z, gm.w};
  bq::pdl_wait_prior_grids();
  const long long units = static_cast<long long>(p.rows) * p.heads;
  const long long stride = static_cast<long long>(gridDim.x) * kGatedWarps;
  float m = 0.0f;
  for (long long u = static_cast<long long>(blockIdx.x) * kGatedWarps + warp; u < units; u += stride) {
    const long long row = u / p.heads;
    const int head = static_cast<int>(u - row * p.heads);
    const long long off = static_cast<long long>(head) * kHeadDim + lane * kVec;
    Vec4<T> core;
    if constexpr (Y_F32) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(
          reinterpret_cast<const float*>(p.y) + row * p.ld_y + off));
      core.v[0] = narrow<T>(f.x); core.v[1] = narrow<T>(f.y);
      core.v[2] = narrow<T>(f.z); core.v[3] = narrow<T>(f.w);
    } else {
      core = load4(reinterpret_cast<const T*>(p.y) + row * p.ld_y + off);
    }
    const Vec4<T> gate = load4(reinterpret_cast<const T*>(p.z) + row * p.ld_z + off);
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      const float f = widen(core.v[j]);
      s = __fmaf_rn(f, f, s);
    }
    s = warp_tree_sum(s);
    s = __shfl_sync(0xffffffffu, s, 0);
    const float sigma2 = __fdiv_rn(s, static_cast<float>(kHeadDim));
    const float rstd = rsqrtf(__fadd_rn(sigma2, p.eps));
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      const T xn = narrow<T>(__fmul_rn(rstd, widen(core.v[j])));
      const float zf = widen(gate.v[j]);
      const float silu = __fdiv_rn(zf, 1.0f + expf(-zf));
      const float h = __fmul_rn(__fmul_rn(gmv[j], widen(xn)), silu);
      core.v[j] = narrow<T>(h);
      m = nan_max(m, fabsf(widen(core.v[j])));
    }
    store4(reinterpret_cast<T*>(p.h_out) + row * p.ld_h + off, core);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, off));
  if (lane == 0) s_max[warp] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float w = s_max[0];
    for (int i = 1; i < kGatedWarps; ++i) w = nan_max(w, s_max[i]);
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

namespace {
template <typename T>
int launch_rmsnorm_scale(const NormParams& p, cudaStream_t stream) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return bq::kErrLaunch;
  }
  const int per_thread = (p.cols / kVec + kNormThreads - 1) / kNormThreads;
  const size_t smem = static_cast<size_t>(p.cols) * sizeof(float);     // gamma
  if (smem > 48 * 1024) return bq::kErrUnsupported;
  cudaError_t e;
  if (per_thread <= 2) e = launch_resident_smem(rmsnorm_scale_kernel<T, 2>, p.rows, kNormThreads, sms, true, smem, stream, p);
  else if (per_thread <= 4) e = launch_resident_smem(rmsnorm_scale_kernel<T, 4>, p.rows, kNormThreads, sms, true, smem, stream, p);
  else if (per_thread <= 8) e = launch_resident_smem(rmsnorm_scale_kernel<T, 8>, p.rows, kNormThreads, sms, true, smem, stream, p);
  else if (per_thread <= 16) e = launch_resident_smem(rmsnorm_scale_kernel<T, 16>, p.rows, kNormThreads, sms, true, smem, stream, p);
  else return bq::kErrUnsupported;
  if (e != cudaSuccess) { (void)cudaGetLastError(); return bq::kErrLaunch; }
  return bq::kOk;
}
}  // namespace

extern "C" int bq_rmsnorm_scale(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                const float* gamma, float eps, void* h_out, int64_t ld_h,
                                float* scale_out, void* ws, size_t ws_bytes, void* stream) {
  if (!x || !gamma || !h_out || !scale_out || rows <= 0 || cols <= 0) return bq::kErrBadArg;
  if (!known_dtype(dtype)) return bq::kErrBadArg;
  if (ws == nullptr || ws_bytes < sizeof(QuantWs) || !aligned_to(ws, 16)) return bq::kErrWorkspace;
  const size_t es = elem_size(dtype);
  const size_t vec_bytes = kVec * es;
  if (cols % kVec || ld_x < cols || (ld_x * es) % vec_bytes || !aligned_to(x, vec_bytes) ||
      !aligned_to(gamma, 16) || ld_h < cols || (ld_h * es) % vec_bytes || !aligned_to(h_out, vec_bytes))
    return bq::kErrUnsupported;
  if (rows > 0x7fffffffLL || cols > 0x7fffffffLL) return bq::kErrTooLarge;
  NormParams p{};
  p.x = x; p.gamma = gamma; p.h_out = h_out;
  p.scale = scale_out; p.ws = ws;
  p.rows = static_cast<int>(rows); p.cols = static_cast<int>(cols);
  p.ld_x = ld_x; p.ld_h = ld_h; p.eps = eps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BQ_DTYPE_F32: return launch_rmsnorm_scale<float>(p, s);
    case BQ_DTYPE_BF16: return launch_rmsnorm_scale<__nv_bfloat16>(p, s);
    default: return launch_rmsnorm_scale<__half>(p, s);
  }
}

extern "C" int bq_rmsnorm_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                const float* gamma, float eps, void* h_out, int64_t ld_h, void* q_out,
                                float* scale_out, void* ws, size_t ws_bytes, void* stream) {
  if (!x || !gamma || !q_out || !scale_out || rows <= 0 || cols <= 0) return bq::kErrBadArg;
  if (!known_dtype(dtype)) return bq::kErrBadArg;
  if (ws == nullptr || ws_bytes < sizeof(QuantWs) || !aligned_to(ws, 16)) return bq::kErrWorkspace;
  const size_t es = elem_size(dtype);
  const size_t vec_bytes = kVec * es;
  if (cols % kVec || ld_x < cols || (ld_x * es) % vec_bytes || !aligned_to(x, vec_bytes) ||
      !aligned_to(gamma, 16) || !aligned_to(q_out, 4))
    return bq::kErrUnsupported;
  if (h_out != nullptr && (ld_h < cols || (ld_h * es) % vec_bytes || !aligned_to(h_out, vec_bytes)))
    return bq::kErrUnsupported;
  if (rows > 0x7fffffffLL || cols > 0x7fffffffLL) return bq::kErrTooLarge;
  NormParams p{};
  p.x = x; p.gamma = gamma; p.h_out = h_out;
  p.q = static_cast<uint8_t*>(q_out); p.scale = scale_out; p.ws = ws;
  p.rows = static_cast<int>(rows); p.cols = static_cast<int>(cols);
  p.ld_x = ld_x; p.ld_h = ld_h; p.eps = eps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case BQ_DTYPE_F32: return launch_rmsnorm<float>(p, s);
    case BQ_DTYPE_BF16: return launch_rmsnorm<__nv_bfloat16>(p, s);
    default: return launch_rmsnorm<__half>(p, s);
  }
}

extern "C" int bq_gated_rmsnorm_quant(const void* y, int y_dtype, int64_t ld_y, const void* z, int dtype,
                                      int64_t ld_z, const float* gamma, float eps, int64_t rows,
                                      int64_t heads, int64_t head_dim, void* q_out, float* scale_out,
                                      void* ws, size_t ws_bytes, void* stream) {
  if (!y || !z || !gamma || !q_out || !scale_out || rows <= 0 || heads <= 0) return bq::kErrBadArg;
  if (!known_dtype(dtype) || (y_dtype != dtype && y_dtype != BQ_DTYPE_F32)) return bq::kErrBadArg;
  if (ws == nullptr || ws_bytes < sizeof(QuantWs) || !aligned_to(ws, 16)) return bq::kErrWorkspace;
  if (head_dim != kHeadDim || heads > kGatedWarps * kMaxHeadsPerWarp) return bq::kErrUnsupported;
  const size_t es = elem_size(dtype), ys = elem_size(y_dtype);
  const int64_t width = heads * head_dim;
  if (ld_y < width || ld_z < width || (ld_y * ys) % (kVec * ys) || (ld_z * es) % (kVec * es) ||
      !aligned_to(y, kVec * ys) || !aligned_to(z, kVec * es) || !aligned_to(gamma, 16) ||
      !aligned_to(q_out, 4))
    return bq::kErrUnsupported;
  if (rows > 0x7fffffffLL) return bq::kErrTooLarge;
  GatedParams p{};
  p.y = y; p.z = z; p.gamma = gamma;
  p.q = static_cast<uint8_t*>(q_out); p.scale = scale_out; p.ws = ws;
  p.rows = static_cast<int>(rows); p.heads = static_cast<int>(heads);
  p.ld_y = ld_y; p.ld_z = ld_z; p.eps = eps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool yf32 = (y_dtype == BQ_DTYPE_F32) && (dtype != BQ_DTYPE_F32);
  switch (dtype) {
    case BQ_DTYPE_F32: return launch_gated<float, false>(p, s);
    case BQ_DTYPE_BF16:
      return yf32 ? launch_gated<__nv_bfloat16, true>(p, s) : launch_gated<__nv_bfloat16, false>(p, s);
    default:
      return yf32 ? launch_gated<__half, true>(p, s) : launch_gated<__half, false>(p, s);
  }
}

extern "C" int bq_gated_rmsnorm_scale(const void* y, int y_dtype, int64_t ld_y, const void* z, int dtype,
                                      int64_t ld_z, const float* gamma, float eps, int64_t rows,
                                      int64_t heads, int64_t head_dim, void* h_out, int64_t ld_h,
                                      float* scale_out, void* ws, size_t ws_bytes, void* stream) {
  if (!y || !z || !gamma || !h_out || !scale_out || rows <= 0 || heads <= 0) return bq::kErrBadArg;
  if (!known_dtype(dtype) || (y_dtype != dtype && y_dtype != BQ_DTYPE_F32)) return bq::kErrBadArg;
  if (ws == nullptr || ws_bytes < sizeof(QuantWs) || !aligned_to(ws, 16)) return bq::kErrWorkspace;
  if (head_dim != kHeadDim) return bq::kErrUnsupported;
  const size_t es = elem_size(dtype), ys = elem_size(y_dtype);
  const int64_t width = heads * head_dim;
  if (ld_y < width || ld_z < width || ld_h < width || (ld_y * ys) % (kVec * ys) ||
      (ld_z * es) % (kVec * es) || (ld_h * es) % (kVec * es) || !aligned_to(y, kVec * ys) ||
      !aligned_to(z, kVec * es) || !aligned_to(h_out, kVec * es) || !aligned_to(gamma, 16))
    return bq::kErrUnsupported;
  if (rows > 0x7fffffffLL || heads > 0x7fffLL) return bq::kErrTooLarge;
  GatedParams p{};
  p.y = y; p.z = z; p.gamma = gamma; p.h_out = h_out; p.ld_h = ld_h;
  p.scale = scale_out; p.ws = ws;
  p.rows = static_cast<int>(rows); p.heads = static_cast<int>(heads);
  p.ld_y = ld_y; p.ld_z = ld_z; p.eps = eps;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return bq::kErrLaunch;
  }
  const long long want = (rows * heads + kGatedWarps - 1) / kGatedWarps;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int threads = kGatedWarps * 32;
  const bool yf32 = (y_dtype == BQ_DTYPE_F32) && (dtype != BQ_DTYPE_F32);
  cudaError_t e;
  switch (dtype) {
    case BQ_DTYPE_F32:
      e = launch_resident(gated_rmsnorm_scale_kernel<float, false>, want, threads, sms, true, st, p);
      break;
    case BQ_DTYPE_BF16:
      e = yf32 ? launch_resident(gated_rmsnorm_scale_kernel<__nv_bfloat16, true>, want, threads, sms, true, st, p)
               : launch_resident(gated_rmsnorm_scale_kernel<__nv_bfloat16, false>, want, threads, sms, true, st, p);
      break;
    default:
      e = yf32 ? launch_resident(gated_rmsnorm_scale_kernel<__half, true>, want, threads, sms, true, st, p)
               : launch_resident(gated_rmsnorm_scale_kernel<__half, false>, want, threads, sms, true, st, p);
  }
  if (e != cudaSuccess) { (void)cudaGetLastError(); return bq::kErrLaunch; }
  return bq::kOk;
}
