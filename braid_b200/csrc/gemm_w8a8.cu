// Per-tensor FP8 W8A8 GEMM for sm_100a:  Y[M,N] = (Xq[M,K] . Wq[N,K]^T) * sx * sw.
//
// Stands in for the `torch._scaled_mm(xq, w.data.t(), scale_a=sx, scale_b=w.scale)`
// call of the reference engine (braid/model/quant.py:232-241).  Both operands are
// K-major, so 128-byte-swizzled TMA tiles feed tcgen05 shared-memory descriptors
// directly; accumulation is fp32 in tensor memory; the dequant scales and the
// output cast are applied in the epilogue.
//
// Two kernels, chosen by M:
//
//  * gemm_stream_kernel (M <= 256, the decode regime; HBM-bound, measured in GB/s).
//    Operands are swapped: 128 WEIGHT rows sit on the MMA M side and the (padded)
//    batch on the MMA N side, so a tile streams 128 x K weight bytes whatever the
//    batch is.  One CTA per (row tile, K slice); the K slices of a tile form a
//    thread-block cluster and are summed through distributed shared memory in a
//    fixed order -- no float atomics, so results are run-to-run identical and a
//    graph replay equals the eager run bit for bit.  Several weights that share
//    one activation (q/k/v, qkv/z, gate/up) go in one launch, each segment with
//    its own scale.
//
//  * gemm_pair_kernel (M > 256, the prefill regime; tensor-bound, measured in
//    TFLOP/s).  Persistent, warp-specialised CTA pairs (cta_group::2): one TMA
//    producer warp, one MMA issuer warp, four epilogue warps; 256x256 output
//    tiles; two 256-column accumulators in tensor memory so a tile's epilogue
//    overlaps the next tile's main loop; the epilogue stages 128-byte row
//    pieces in shared memory and hands them to TMA stores.
//
// Every mbarrier wait is bounded (ptx.cuh); a wait that runs out sets the sticky
// status word and the CTA unwinds through the normal teardown.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/braid_b200.h"
#include "ptx.cuh"
#include "quant_device.cuh"

namespace {

using namespace bq;

constexpr int kBK = 128;         // K bytes per pipeline stage: one swizzle span
constexpr int kUmmaK = 32;       // K elements one f8 MMA consumes
constexpr int kRowTile = 128;    // MMA M
constexpr int kATileBytes = kRowTile * kBK;   // 16 KiB
constexpr int kMaxSmem = 232448;              // 227 KiB opt-in limit per CTA
#ifndef BQ_STREAM_THREADS
#define BQ_STREAM_THREADS 384
#endif
constexpr int kStreamThreads = BQ_STREAM_THREADS;   // weight-streaming kernel: warps 0 / 1 load and
constexpr int kStreamWarps = kStreamThreads / 32;   // issue MMAs, ALL warps run the epilogue
constexpr int kBarrierBytes = 1024;           // mbarriers + tmem slot + flags

struct Segment {
  const float* sw;     // device: weight dequant scale
  void* y;             // device: output base of this segment
  long long ldy;       // row stride of y, elements
  const void* res;     // stream kernel: optional residual [M, n] of the output type, added after
                       // the output has been rounded to that type (two roundings, as the separate
                       // GEMM and add kernels give)
  long long ld_res;
  int dense;           // stream kernel: 1 = a 16-bit (bf16 / fp16) weight multiplied with the
                       // unquantized activation (kind::f16 MMA, no scales), 0 = e4m3 weight
  int y_tma;           // pair kernel: the output can be described to TMA (16-byte aligned base and pitch)
  int n;               // weight rows (output columns) of this segment
  int tile_begin;      // tile kernel: index of the segment's first tile
  int split;           // stream kernel: K slices of this weight (1, 2, 4 or 8)
  int split_forced;    // stream kernel: non-zero = use this split instead of the shape rule
  int cluster_begin;   // stream kernel: index of the segment's first cluster
};

// SiLU(gate)*up and the quantization of the product, done in the epilogue of ONE GEMM whose
// 128-row MMA tiles are put together from 64 gate rows and the 64 up rows of the same output
// columns -- two TMA boxes per pipeline stage, read from the two weights where they lie (the
// reference keeps gate_proj and up_proj as two tensors, braid/model/mlp.py:27-29; nothing is
// repacked or copied).
struct PairSilu {
  int on;
  int prefill;             // M > 256: the CTA-pair kernel writes h itself ([M, I], activation type)
                           // and the scale of h; the codes are a separate cast pass
  const void* wq_up;       // device: the up weight [I, K] (segment 0's weight pointer is the gate weight)
  const float* sw_up;      // device: dequant scale of the up half (seg.sw is the gate half's)
  uint8_t* hq;             // device: e4m3 codes of h, [M, ld_hq]
  long long ld_hq;
  float* sh;               // device: the scale of h
  unsigned int* words;     // [0] amax bits [1] arrivals [2] departures ([3] is the sticky status)
  unsigned int expected;   // CTAs that take part in the exchange (the active ones)
};

// Greedy pick fused into the lm_head GEMM: every CTA (one 128-row tile of the vocabulary, K not
// split) reduces, per batch row, the largest of ITS 128 logits -- taken after the rounding to the
// output type the logits tensor would have had, lowest index winning ties, NaN winning over
// everything, which is `logits.argmax(-1)` as torch evaluates it -- and writes one (value,
// index) pair per row; a second, tiny kernel reduces the pairs of all tiles.
struct ArgmaxOut {
  int on;
  int store_logits;          // 0 = the logits themselves are not written at all
  uint2* partial;            // device: [tiles][M] pairs {value as fp32 bits, vocabulary index}
};

// a beats b: NaN first, then the larger value, then the lower index
__device__ __forceinline__ bool argmax_beats(float av, int ai, float bv, int bi) {
  const bool an = av != av, bn = bv != bv;
  if (an || bn) return an && (!bn || ai < bi);
  return av > bv || (av == bv && ai < bi);
}

// Column-parallel form: the output tile (or, in the paired form, h) is stored straight into the
// gathered buffer of every rank of the node -- plain stores through peer-mapped pointers, this
// rank's own buffer included.  The CTAs of the launch count themselves on a local word; the last
// one to finish adds 1 to a counter on each rank with a system-scope release (one arrival per
// rank and exchange).  No collective call, no multicast.  The pointers already carry this rank's
// column offset.
constexpr int kMaxPeers = 8;
struct PushParams {
  int n;                          // destinations (0 = not a push launch)
  void* dst[kMaxPeers];
  long long ld;                   // row stride of every destination, elements
  unsigned int* flag[kMaxPeers];  // one arrival counter per destination rank
  unsigned int* done;             // local: CTAs of this launch that have stored their share
  unsigned int expected;          // CTAs that store (the active ones)
  // prefill SiLU form: where this rank's max |h| (float bits) goes on every rank, written by
  // the last CTA before the arrivals; nullptr = not wanted
  unsigned int* amax_dst[kMaxPeers];
  unsigned int* amax_local;       // local running max of the launch (zero between launches)
};

struct GemmParams {
  Segment seg[BQ_MAX_SEGMENTS];
  int n_seg;
  const float* sx;     // device: activation dequant scale
  int M;               // activation rows
  int mma_n;           // stream kernel: padded batch = MMA N (multiple of 16)
  int k_blocks;        // ceil(K / 128)
  int k_blocks_dense;  // stream kernel: 128-byte K blocks of a 16-bit row, ceil(2K / 128)
  int dense_fmt;       // stream kernel: tcgen05 operand format of the 16-bit segments (0 f16, 1 bf16)
  int cluster;         // stream kernel: CTAs per cluster = largest split of the launch
  int stages;          // stream kernel: depth of the weight ring; pair kernel: pipeline depth
  int b_stages;        // stream kernel: depth of the activation ring
  int out_dtype;
  int m_tiles;         // tile kernel: ceil(M / 128)
  int pair_n;          // pair kernel, plain form: output columns per tile, 256 or 128
  int total_tiles;     // tile kernel
  unsigned int* status;
  ArgmaxOut argmax;
  unsigned long long* phase_ring;   // development builds (BQ_PHASES) only, else nullptr
  int phase_seq;
  PairSilu pair;
  PushParams push;
};

struct alignas(64) WeightMaps {
  CUtensorMap w[BQ_MAX_SEGMENTS];
};

__device__ __forceinline__ int find_segment(const GemmParams& p, int tile) {
  int s = 0;
#pragma unroll
  for (int i = 1; i < BQ_MAX_SEGMENTS; ++i)
    if (i < p.n_seg && tile >= p.seg[i].tile_begin) s = i;
  return s;
}

__device__ __forceinline__ void store_out4(void* y, long long idx, int out_dtype, float4 v) {
  if (out_dtype == BQ_DTYPE_BF16) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t*>(&lo);
    w.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(y) + idx) = w;
  } else if (out_dtype == BQ_DTYPE_F16) {
    const __half2 lo = __floats2half2_rn(v.x, v.y);
    const __half2 hi = __floats2half2_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t*>(&lo);
    w.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(static_cast<__half*>(y) + idx) = w;
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(y) + idx) = v;
  }
}

struct EpilogueArgs {
  const float* part;       // this CTA's staging buffer [mma_n][128] fp32
  uint32_t part_addr;      // its shared-memory address
  int peer0;               // cluster rank of K slice 0 of this tile
  int m_begin, m_end;      // output rows this CTA reduces and writes
  int warp, lane;
  int row0;                // first weight row (output column) of the tile
  float scale;
  bool col_ok;
  void* y;
  long long ldy;
  int out_dtype;
  const void* res;
  long long ld_res;
  const PushParams* push;
};

// Four residual values of the output type, as raw bits (16 bytes cover the widest case).
__device__ __forceinline__ uint4 load_res4(const void* res, long long idx, int out_dtype) {
  uint4 r = make_uint4(0u, 0u, 0u, 0u);
  if (out_dtype == BQ_DTYPE_F32) {
    r = __ldg(reinterpret_cast<const uint4*>(static_cast<const float*>(res) + idx));
  } else {
    const uint2 h = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(res) + idx));
    r.x = h.x; r.y = h.y;
  }
  return r;
}

// out = T(float(T(v)) + float(res)): the GEMM's own rounding, then the add's.
__device__ __forceinline__ float4 add_res4(float4 v, uint4 raw, int out_dtype) {
  if (out_dtype == BQ_DTYPE_BF16) {
    const __nv_bfloat162 r0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 r1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    v.x = __bfloat162float(__float2bfloat16_rn(v.x)) + __bfloat162float(r0.x);
    v.y = __bfloat162float(__float2bfloat16_rn(v.y)) + __bfloat162float(r0.y);
    v.z = __bfloat162float(__float2bfloat16_rn(v.z)) + __bfloat162float(r1.x);
    v.w = __bfloat162float(__float2bfloat16_rn(v.w)) + __bfloat162float(r1.y);
  } else if (out_dtype == BQ_DTYPE_F16) {
    const __half2 r0 = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 r1 = *reinterpret_cast<const __half2*>(&raw.y);
    v.x = __half2float(__float2half_rn(v.x)) + __half2float(r0.x);
    v.y = __half2float(__float2half_rn(v.y)) + __half2float(r0.y);
    v.z = __half2float(__float2half_rn(v.z)) + __half2float(r1.x);
    v.w = __half2float(__float2half_rn(v.w)) + __half2float(r1.y);
  } else {
    // intrinsics: a plain + would be contracted with the scaling multiply into one fma
    v.x = __fadd_rn(v.x, __uint_as_float(raw.x)); v.y = __fadd_rn(v.y, __uint_as_float(raw.y));
    v.z = __fadd_rn(v.z, __uint_as_float(raw.z)); v.w = __fadd_rn(v.w, __uint_as_float(raw.w));
  }
  return v;
}

// Sums the SPLIT partial tiles of this CTA's rows in rank order (fixed order:
// the result does not depend on timing) and stores them.  Every thread asks
// for all the partials of a batch of rows before it uses any of them, so the
// remote shared-memory latency is paid once per batch, not once per load.
template <int SPLIT, bool RES>
__device__ __forceinline__ void reduce_store(const EpilogueArgs& e) {
  // rows in flight per thread (half as many when residual values are held as well)
  constexpr int kRows = ((RES && SPLIT < 8) ? 8 / SPLIT : 16 / SPLIT) > (kStreamWarps > 8 ? 2 : 1)
                            ? ((RES && SPLIT < 8) ? 8 / SPLIT : 16 / SPLIT) / (kStreamWarps > 8 ? 2 : 1)
                            : 1;
  constexpr int kWarps = kStreamWarps;
  const int n4 = e.lane * 4;                 // 4 consecutive output columns
  for (int m0 = e.m_begin + e.warp; m0 < e.m_end; m0 += kWarps * kRows) {
    float4 v[kRows][SPLIT];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const int m = m0 + i * kWarps;
      if (m < e.m_end) {
        const uint32_t off = e.part_addr + static_cast<uint32_t>(m * kRowTile + n4) * 4u;
#pragma unroll
        for (int r = 0; r < SPLIT; ++r) {
          if constexpr (SPLIT == 1)
            v[i][0] = *reinterpret_cast<const float4*>(e.part + m * kRowTile + n4);
          else
            v[i][r] = ld_cluster_f4(map_to_cta(off, e.peer0 + r));
        }
      }
    }
    uint4 rraw[RES ? kRows : 1];
    if constexpr (RES) {
#pragma unroll
      for (int i = 0; i < kRows; ++i) {
        const int m = m0 + i * kWarps;
        if (m < e.m_end && e.col_ok)
          rraw[i] = load_res4(e.res, (long long)m * e.ld_res + e.row0 + n4, e.out_dtype);
      }
    }
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const int m = m0 + i * kWarps;
      if (m < e.m_end) {
        float4 acc = v[i][0];
#pragma unroll
        for (int r = 1; r < SPLIT; ++r) {
          acc.x += v[i][r].x; acc.y += v[i][r].y; acc.z += v[i][r].z; acc.w += v[i][r].w;
        }
        acc.x *= e.scale; acc.y *= e.scale; acc.z *= e.scale; acc.w *= e.scale;
        if constexpr (RES) {
          if (e.col_ok) acc = add_res4(acc, rraw[i], e.out_dtype);
        }
        if (e.col_ok) {
          if (e.push->n == 0) {
            store_out4(e.y, (long long)m * e.ldy + e.row0 + n4, e.out_dtype, acc);
          } else {
            for (int d = 0; d < e.push->n; ++d)
              store_out4(e.push->dst[d], (long long)m * e.push->ld + e.row0 + n4, e.out_dtype, acc);
          }
        }
      }
    }
  }
}

// Per batch row of this CTA's share: the best of the tile's 128 logits (see ArgmaxOut).  K is
// not split in an argmax launch, so the staged tile is final.
template <typename T>
__device__ __forceinline__ void argmax_rows(const EpilogueArgs& e, int n_total, uint2* partial_tile) {
  using namespace bq::qd;
  const int n4 = e.lane * 4;
  for (int m = e.m_begin + e.warp; m < e.m_end; m += kStreamWarps) {
    const float4 v = *reinterpret_cast<const float4*>(e.part + m * kRowTile + n4);
    const float r[4] = {widen(narrow<T>(v.x * e.scale)), widen(narrow<T>(v.y * e.scale)),
                        widen(narrow<T>(v.z * e.scale)), widen(narrow<T>(v.w * e.scale))};
    float bv = 0.0f;
    int bi = 0x7fffffff;                      // "nothing yet": loses against any real column
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = e.row0 + n4 + j;
      if (idx < n_total && (bi == 0x7fffffff || argmax_beats(r[j], idx, bv, bi))) { bv = r[j]; bi = idx; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || argmax_beats(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    if (e.lane == 0) partial_tile[m] = make_uint2(__float_as_uint(bv), static_cast<unsigned int>(bi));
  }
}

// Second stage of the greedy pick: one CTA per batch row reduces the pairs of all tiles.
__global__ void __launch_bounds__(128) argmax_finish_kernel(const uint2* partial, int tiles, int M,
                                                            long long* idx_out) {
  pdl_wait_prior_grids();
  const int m = blockIdx.x;
  float bv = 0.0f;
  int bi = 0x7fffffff;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const uint2 pr = __ldcg(partial + static_cast<size_t>(t) * M + m);
    const float ov = __uint_as_float(pr.x);
    const int oi = static_cast<int>(pr.y);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || argmax_beats(ov, oi, bv, bi))) { bv = ov; bi = oi; }
  }
  __shared__ float s_v[4];
  __shared__ int s_i[4];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || argmax_beats(ov, oi, bv, bi))) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = bv; s_i[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 4; ++w)
      if (s_i[w] != 0x7fffffff && (bi == 0x7fffffff || argmax_beats(s_v[w], s_i[w], bv, bi))) {
        bv = s_v[w];
        bi = s_i[w];
      }
    idx_out[m] = bi;
  }
}

// Interleaved gate/up tile: columns 0..63 of the tile are gate rows, 64..127 the up rows of the
// same 64 output columns.  Sums the K slices like reduce_store, rounds both halves to the
// activation type T exactly as the plain GEMM would have stored them, forms
// h = T(T(silu(gate)) * up) (the two roundings of the separate torch kernels,
// braid/model/mlp.py:48), and parks h (64 values of T per row) at the start of the row's
// staging slot in THIS CTA's buffer -- rows of this CTA's share are read by no peer.
// Lane L < 16 ends up with columns 4L, 4L+1; lane L+16 with 4L+2, 4L+3.  Returns max |h|.
template <int SPLIT, typename T>
__device__ __forceinline__ float silu_pair_rows(const EpilogueArgs& e, float scale_up, float* part_rw) {
  using namespace bq::qd;
  constexpr int kRows = ((SPLIT < 8) ? 8 / SPLIT : 1) > (kStreamWarps > 8 ? 2 : 1)
                            ? ((SPLIT < 8) ? 8 / SPLIT : 1) / (kStreamWarps > 8 ? 2 : 1)
                            : 1;
  constexpr int kWarps = kStreamWarps;
  const int n4 = e.lane * 4;
  const bool up_half = e.lane >= 16;
  const float sc = up_half ? scale_up : e.scale;
  const int hcol = (e.lane & 15) * 4 + (up_half ? 2 : 0);
  float mx = 0.0f;
  for (int m0 = e.m_begin + e.warp; m0 < e.m_end; m0 += kWarps * kRows) {
    float4 v[kRows][SPLIT];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const int m = m0 + i * kWarps;
      if (m < e.m_end) {
        const uint32_t off = e.part_addr + static_cast<uint32_t>(m * kRowTile + n4) * 4u;
#pragma unroll
        for (int r = 0; r < SPLIT; ++r) {
          if constexpr (SPLIT == 1)
            v[i][0] = *reinterpret_cast<const float4*>(e.part + m * kRowTile + n4);
          else
            v[i][r] = ld_cluster_f4(map_to_cta(off, e.peer0 + r));
        }
      }
    }
    __syncwarp();   // every lane has its slice of the rows before any lane overwrites them
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const int m = m0 + i * kWarps;    // warp-uniform
      if (m < e.m_end) {
        float4 acc = v[i][0];
#pragma unroll
        for (int r = 1; r < SPLIT; ++r) {
          acc.x += v[i][r].x; acc.y += v[i][r].y; acc.z += v[i][r].z; acc.w += v[i][r].w;
        }
        // the value the plain GEMM would have stored: one rounding to T
        const float r0 = widen(narrow<T>(acc.x * sc)), r1 = widen(narrow<T>(acc.y * sc));
        const float r2 = widen(narrow<T>(acc.z * sc)), r3 = widen(narrow<T>(acc.w * sc));
        const float got0 = __shfl_xor_sync(0xffffffffu, up_half ? r0 : r2, 16);
        const float got1 = __shfl_xor_sync(0xffffffffu, up_half ? r1 : r3, 16);
        const float g0 = up_half ? got0 : r0, g1 = up_half ? got1 : r1;
        const float u0 = up_half ? r2 : got0, u1 = up_half ? r3 : got1;
        const T s0 = silu_to<T>(g0);
        const T s1 = silu_to<T>(g1);
        const T h0 = narrow<T>(widen(s0) * u0);
        const T h1 = narrow<T>(widen(s1) * u1);
        mx = nan_max(mx, fabsf(widen(h0)));
        mx = nan_max(mx, fabsf(widen(h1)));
        T* hrow = reinterpret_cast<T*>(part_rw + m * kRowTile);
        hrow[hcol] = h0;
        hrow[hcol + 1] = h1;
      }
    }
  }
  return mx;
}

// After the grid-wide scale is known: cast the parked h of this CTA's rows and write the codes.
template <typename T>
__device__ __forceinline__ void silu_pair_emit(const EpilogueArgs& e, const float* part, float scale,
                                               uint8_t* hq, long long ld_hq, int col0) {
  using namespace bq::qd;
  const ScaleDiv sc(scale);
  const int hcol = (e.lane & 15) * 4 + (e.lane >= 16 ? 2 : 0);
  for (int m = e.m_begin + e.warp; m < e.m_end; m += kStreamWarps) {
    const T* hrow = reinterpret_cast<const T*>(part + m * kRowTile);
    float f[2] = {widen(hrow[hcol]), widen(hrow[hcol + 1])};
    divide_group<2, true>(sc, f);   // the scale is that of these very values
    const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(f[0], f[1]), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint16_t*>(hq + static_cast<long long>(m) * ld_hq + col0 + hcol) =
        static_cast<uint16_t>(pair & 0xFFFFu);
  }
}

// ---------------------------------------------------------------------------
// Weight-streaming kernel (swap-AB, cluster split-K)
// ---------------------------------------------------------------------------
// Shared memory, after aligning the dynamic base to 1024 bytes:
//   [stages x 16 KiB weight tiles][b_stages x (mma_n*128) activation tiles] ... [barrier block]
// Two rings with their own barriers and their own producer thread.  The weight ring is as deep
// as the shared memory allows: its tiles come from HBM, and the bytes in flight per SM are what
// sets the streaming rate.  The activation ring is shallow (2 to 4 tiles at wide batches): its
// tiles are L2 hits shared by every row tile, and a wide batch tile is as large as a weight
// tile, so every activation slot given up is a weight tile more in flight.
// The tile area is reused after the main loop as the fp32 staging buffer
// part[m][128] that the cluster reduction reads.
#ifndef BQ_STREAM_MIN_CTAS
#define BQ_STREAM_MIN_CTAS 2
#endif
__global__ void __launch_bounds__(kStreamThreads, BQ_STREAM_MIN_CTAS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_xd,
                   const __grid_constant__ WeightMaps tm_w, const __grid_constant__ GemmParams p,
                   const int smem_tile_bytes) {
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_dyn + (base - smem_u32(smem_dyn));
  const int b_tile_bytes = p.mma_n * kBK;
  const uint32_t a_base = base;
  const uint32_t b_base = base + p.stages * kATileBytes;
  const uint32_t bar_base = base + smem_tile_bytes;          // 8-byte aligned
  // barrier block: weight ring full / empty, activation ring full, accumulator.  One
  // tcgen05.commit per K block: it arrives on the weight slot's "empty" barrier, and the
  // activation producer watches the same barrier for the block whose activation slot it wants
  // to refill.
  const int n_bars = 2 * p.stages + p.b_stages;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (p.stages + s); };
  auto full_bar_b = [&](int s) { return bar_base + 8u * (2 * p.stages + s); };
  const uint32_t accum_bar = bar_base + 8u * n_bars;
  volatile uint32_t* const tmem_slot =
      reinterpret_cast<volatile uint32_t*>(base_ptr + smem_tile_bytes + 8 * (n_bars + 1));
  volatile uint32_t* const abort_flag = tmem_slot + 1;
  float* const s_quant = reinterpret_cast<float*>(const_cast<uint32_t*>(tmem_slot) + 2);   // one float per warp

  if (threadIdx.x == 0) { BQ_STAMP(p, 0); BQ_STAMP_META(p, 0); }
  pdl_launch_dependents();   // the next kernel may start its own set-up right away
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A cluster of p.cluster CTAs works on p.cluster / split row tiles of one weight
  // at a time: CTAs [g*split, (g+1)*split) of the cluster hold the K slices of
  // tile g and reduce among themselves.
  const int crank = (p.cluster > 1) ? static_cast<int>(cluster_ctarank()) : 0;
  const int cluster_id = blockIdx.x / p.cluster;
  int sg = 0;
#pragma unroll
  for (int i = 1; i < BQ_MAX_SEGMENTS; ++i)
    if (i < p.n_seg && cluster_id >= p.seg[i].cluster_begin) sg = i;
  const Segment seg = p.seg[sg];
  const int split = seg.split;
  const int group = crank / split;              // which tile of the cluster
  const int krank = crank - group * split;      // which K slice of that tile
  const int tile_in_seg = (cluster_id - seg.cluster_begin) * (p.cluster / split) + group;
  const int row0 = tile_in_seg * kRowTile;
  const bool active = row0 < seg.n;             // padding CTAs only keep the cluster barriers

  // this CTA's K slice, balanced to within one block
  // a 16-bit segment (a weight the reference keeps unquantized) walks 128-byte K blocks of
  // 64 elements over the dense activation; everything else about the pipeline is the same
  const bool dense = seg.dense != 0;
  const int seg_k_blocks = dense ? p.k_blocks_dense : p.k_blocks;
  const CUtensorMap* const x_map = dense ? &tm_xd : &tm_x;
  const int kb_base = seg_k_blocks / split, kb_rem = seg_k_blocks % split;
  const int kb_count = active ? kb_base + (krank < kb_rem ? 1 : 0) : 0;
  const int kb_begin = krank * kb_base + (krank < kb_rem ? krank : kb_rem);

  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.mma_n)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(x_map);
    tma_prefetch_desc(&tm_w.w[sg]);
    if (p.pair.on) tma_prefetch_desc(&tm_w.w[1]);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < p.b_stages; ++s) mbar_init(full_bar_b(s), 1);
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1 && active) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) BQ_STAMP(p, 1);

  if (!active) {
    // nothing to multiply: it only matches the two cluster barriers of the working CTAs
    if (p.cluster > 1) { cluster_sync_all(); cluster_sync_all(); }
    return;
  }

  if (warp == 0) {
    if (elect_one()) {
      // Weights do not depend on any earlier kernel: this thread never waits for the kernel
      // that produces the activation, it only follows the MMAs through the weight ring.
      // weights are read once: evict first
      const uint64_t pol_w = policy_evict_first();
      // one 128-row box, or (paired gate/up) two 64-row boxes from the two weights
      const bool paired = p.pair.on != 0;
      const int half_row0 = tile_in_seg * (kRowTile / 2);
      // slot and phase are carried along: an integer division by a run-time depth costs a
      // single issuing thread more than the loads it issues
      int s = 0;
      uint32_t phase = 1;                      // parity of the completion that frees slot s
      for (int i = 0; i < kb_count; ++i) {
        if (i >= p.stages && !mbar_wait(empty_bar(s), phase)) {
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(full_bar(s), kATileBytes);
        const int kx = (kb_begin + i) * kBK;
        const uint32_t dst = a_base + s * kATileBytes;
        if (paired) {
          tma_load_2d(dst, &tm_w.w[0], full_bar(s), kx, half_row0, pol_w);
          tma_load_2d(dst + kATileBytes / 2, &tm_w.w[1], full_bar(s), kx, half_row0, pol_w);
        } else {
          tma_load_2d(dst, &tm_w.w[sg], full_bar(s), kx, row0, pol_w);
        }
        if (++s == p.stages) { s = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    if (elect_one()) {
      // the activation tile is shared by every row tile: keep it in L2
      const uint64_t pol_x = policy_evict_last();
      pdl_wait_prior_grids();   // the kernel that produces the activation has completed
      BQ_STAMP(p, 2);
      // Activation slot s was last read by the MMAs of block j = i - b_stages, whose completion
      // is completion number j / stages of weight slot j % stages.  That barrier cannot complete
      // a second time before this thread has looked: block j + stages >= i needs THIS load first
      // (the host keeps b_stages <= stages).
      int s = 0, js = 0;                       // activation slot of block i, weight slot of block j
      uint32_t jphase = 0;                     // parity of completion j / stages
      for (int i = 0; i < kb_count; ++i) {
        if (i >= p.b_stages) {
          if (!mbar_wait(empty_bar(js), jphase)) {
            *abort_flag = 1;
            break;
          }
          if (++js == p.stages) { js = 0; jphase ^= 1u; }
        }
        mbar_expect_tx(full_bar_b(s), b_tile_bytes);
        tma_load_2d(b_base + s * b_tile_bytes, x_map, full_bar_b(s), (kb_begin + i) * kBK, 0, pol_x);
        if (++s == p.b_stages) s = 0;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = dense ? idesc_f16(kRowTile, p.mma_n, p.dense_fmt)
                                   : idesc_e4m3(kRowTile, p.mma_n);
      int s = 0, sb = 0;
      uint32_t phase = 0, phase_b = 0;
      for (int i = 0; i < kb_count; ++i) {
        if (!mbar_wait(full_bar(s), phase) || !mbar_wait(full_bar_b(sb), phase_b)) {
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        if (i == 0) BQ_STAMP(p, 3);
        const uint64_t da = smem_desc_sw128(a_base + s * kATileBytes);
        const uint64_t db = smem_desc_sw128(b_base + sb * b_tile_bytes);
#pragma unroll
        for (int j = 0; j < kBK / kUmmaK; ++j) {
          // +32 bytes along K inside the swizzle span = +2 in descriptor units (32 e4m3 or 16
          // 16-bit elements: one MMA's K either way)
          if (dense) mma_f16(tmem_base, da + 2u * j, db + 2u * j, idesc, (i | j) != 0 ? 1u : 0u);
          else mma_f8(tmem_base, da + 2u * j, db + 2u * j, idesc, (i | j) != 0 ? 1u : 0u);
        }
        mma_commit(empty_bar(s));   // both slots are free once these MMAs retire
        if (++s == p.stages) { s = 0; phase ^= 1u; }
        if (++sb == p.b_stages) { sb = 0; phase_b ^= 1u; }
      }
      mma_commit(accum_bar);        // accumulator complete
    }
    __syncwarp();
  }

  // ---- epilogue: TMEM -> fp32 staging in shared memory ----------------------
  pdl_wait_prior_grids();   // scales are read and outputs written only after this
  // the epilogue warps get here at once and have the scale ready long before
  // the accumulator is
  const float sw = dense ? 1.0f : __ldg(seg.sw);
  const float sx_ready = dense ? 1.0f : __ldg(p.sx);
  bool ok = mbar_wait(accum_bar, 0);
  tc_fence_after();
  if (threadIdx.x == 0) BQ_STAMP(p, 4);
  if (!ok) *abort_flag = 1;
  __syncthreads();
  ok = (*abort_flag == 0);
  const float scale = sx_ready * sw;
  float* const part = reinterpret_cast<float*>(base_ptr);   // [mma_n][128]
  if (ok) {
    // 8 warps: warp w reads TMEM lanes 32*(w%4).. (the only ones it may touch)
    // and every other 16-column chunk, starting at chunk w/4
    const int quad = warp & 3;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int n_local = quad * 32 + lane;
    for (int c = (warp >> 2) * 16; c < p.mma_n; c += 4 * kStreamWarps) {
      uint32_t r[16];
      tmem_ld16(lane_addr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) part[(c + j) * kRowTile + n_local] = __uint_as_float(r[j]);
    }
  } else if (threadIdx.x == 0) {
    atomicExch(p.status, (unsigned int)kErrDeviceWait);
  }
  tc_fence_before();
  if (p.cluster > 1) cluster_sync_all(); else __syncthreads();
  if (threadIdx.x == 0) BQ_STAMP(p, 5);

  // ---- reduce the K slices in rank order and write this CTA's share of rows --
  float pair_max = 0.0f;
  const int per = (p.M + split - 1) / split;
  const int m_begin = krank * per;
  const int m_end = (m_begin + per < p.M) ? (m_begin + per) : p.M;
  if (ok) {
    const bool col_ok = (row0 + lane * 4) < seg.n;      // n is a multiple of 16
    const uint32_t part_addr = smem_u32(part);
    const int peer0 = group * split;
    const EpilogueArgs ea{part, part_addr, peer0, m_begin, m_end, warp, lane, row0, scale, col_ok,
                          seg.y, seg.ldy, p.out_dtype, seg.res, seg.ld_res, &p.push};
    if (p.pair.on) {
      const float scale_up = sx_ready * __ldg(p.pair.sw_up);
      float mx;
#define BQ_PAIR_ROWS(TT)                                                          \
      switch (split) {                                                             \
        case 1: mx = silu_pair_rows<1, TT>(ea, scale_up, part); break;             \
        case 2: mx = silu_pair_rows<2, TT>(ea, scale_up, part); break;             \
        case 4: mx = silu_pair_rows<4, TT>(ea, scale_up, part); break;             \
        default: mx = silu_pair_rows<8, TT>(ea, scale_up, part); break;            \
      }
      if (p.out_dtype == BQ_DTYPE_BF16) { BQ_PAIR_ROWS(__nv_bfloat16) }
      else if (p.out_dtype == BQ_DTYPE_F16) { BQ_PAIR_ROWS(__half) }
      else { BQ_PAIR_ROWS(float) }
#undef BQ_PAIR_ROWS
      pair_max = mx;
    } else if (p.argmax.on) {
      uint2* const mine = p.argmax.partial + static_cast<size_t>(tile_in_seg) * p.M;
      if (p.out_dtype == BQ_DTYPE_BF16) argmax_rows<__nv_bfloat16>(ea, seg.n, mine);
      else if (p.out_dtype == BQ_DTYPE_F16) argmax_rows<__half>(ea, seg.n, mine);
      else argmax_rows<float>(ea, seg.n, mine);
      if (p.argmax.store_logits) reduce_store<1, false>(ea);
    } else if (seg.res == nullptr) {
      switch (split) {
        case 1: reduce_store<1, false>(ea); break;
        case 2: reduce_store<2, false>(ea); break;
        case 4: reduce_store<4, false>(ea); break;
        default: reduce_store<8, false>(ea); break;
      }
    } else {
      switch (split) {
        case 1: reduce_store<1, true>(ea); break;
        case 2: reduce_store<2, true>(ea); break;
        case 4: reduce_store<4, true>(ea); break;
        default: reduce_store<8, true>(ea); break;
      }
    }
  }
  if (threadIdx.x == 0) BQ_STAMP(p, 6);
  // nobody leaves while a peer may still read its staging buffer
  if (p.cluster > 1) cluster_sync_all(); else __syncthreads();
  if (p.pair.on && p.push.n > 0) {
    // ---- column-parallel form: h itself goes to every rank's gathered buffer; the amax needs
    // all ranks' shards and is taken by the quantizer that follows the exchange ----
    __syncthreads();   // parked rows are complete
    if (ok) {
      const int col0 = tile_in_seg * (kRowTile / 2);
      const int hcol = (lane & 15) * 4 + (lane >= 16 ? 2 : 0);
      for (int m = m_begin + warp; m < m_end; m += kStreamWarps) {
        const long long at = static_cast<long long>(m) * p.push.ld + col0 + hcol;
        if (p.out_dtype == BQ_DTYPE_F32) {
          const float2 v = *reinterpret_cast<const float2*>(part + m * kRowTile + hcol);
          for (int d = 0; d < p.push.n; ++d)
            *reinterpret_cast<float2*>(static_cast<float*>(p.push.dst[d]) + at) = v;
        } else {
          const uint32_t v = *reinterpret_cast<const uint32_t*>(
              reinterpret_cast<const uint16_t*>(part + m * kRowTile) + hcol);
          for (int d = 0; d < p.push.n; ++d)
            *reinterpret_cast<uint32_t*>(static_cast<uint16_t*>(p.push.dst[d]) + at) = v;
        }
      }
    }
  } else if (p.pair.on) {
    // ---- grid-wide max |h| -> scale -> codes of this CTA's rows (h is parked in `part`) ----
    using namespace bq::qd;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
      pair_max = nan_max(pair_max, __shfl_xor_sync(0xffffffffu, pair_max, off));
    if (lane == 0) s_quant[warp] = pair_max;
    __syncthreads();
    if (threadIdx.x == 0) {
      float w = s_quant[0];
#pragma unroll
      for (int i = 1; i < kStreamWarps; ++i) w = nan_max(w, s_quant[i]);
      unsigned int* const words = p.pair.words;
      if (p.pair.expected > 1) {
        // an aborted CTA still arrives (with 0), so the others are not left waiting
        atomicMax(&words[0], __float_as_uint(w));
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&words[1]) : "memory");
        unsigned int amax_bits = 0, arrived = 0;
        const long long t0 = clock64();
        for (;;) {
          asm volatile("ld.acquire.gpu.global.v2.u32 {%0, %1}, [%2];"
                       : "=r"(amax_bits), "=r"(arrived)
                       : "l"(words)
                       : "memory");
          if (arrived >= p.pair.expected) break;
          if (clock64() - t0 > kSpinLimitCycles) {
            atomicExch(p.status, (unsigned int)kErrDeviceWait);
            break;
          }
        }
        w = __uint_as_float(amax_bits);
      }
      const float sc = scale_from_amax(w);
      if (blockIdx.x == 0) p.pair.sh[0] = sc;
      s_quant[0] = sc;
    }
    __syncthreads();
    const float sc = s_quant[0];
    if (ok) {
      const EpilogueArgs ea{part, smem_u32(part), 0, m_begin, m_end, warp, lane, row0, 0.0f, true,
                            nullptr, 0, p.out_dtype, nullptr, 0, &p.push};
      const int col0 = tile_in_seg * (kRowTile / 2);
      if (p.out_dtype == BQ_DTYPE_BF16)
        silu_pair_emit<__nv_bfloat16>(ea, part, sc, p.pair.hq, p.pair.ld_hq, col0);
      else if (p.out_dtype == BQ_DTYPE_F16)
        silu_pair_emit<__half>(ea, part, sc, p.pair.hq, p.pair.ld_hq, col0);
      else
        silu_pair_emit<float>(ea, part, sc, p.pair.hq, p.pair.ld_hq, col0);
    }
    if (threadIdx.x == 0 && p.pair.expected > 1) {
      unsigned int* const words = p.pair.words;
      const unsigned int old = atomicAdd(&words[2], 1u);
      if (old == p.pair.expected - 1) {
        words[0] = 0u; words[1] = 0u; words[2] = 0u;
        __threadfence();
      }
    }
  }
  if (p.push.n > 0) {
    // The stores of all threads of this CTA are ordered before thread 0's fence by the barrier
    // (fences are cumulative); the fence orders them before this CTA's count; the last CTA sees
    // every count, fences again and only then signals the ranks: every store of the launch
    // happens before every arrival.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int old = atomicAdd(p.push.done, 1u);
      if (old == p.push.expected - 1u) {
        *p.push.done = 0u;                       // ready for the next launch on this scratch
        __threadfence_system();
        for (int d = 0; d < p.push.n; ++d)
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.push.flag[d]) : "memory");
      }
    }
  }
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
  if (threadIdx.x == 0) BQ_STAMP(p, 7);
}

// Waits (bounded) until `flag` has counted `count` more arrivals than at the end of the
// previous wait, i.e. until every CTA of every rank's push launch has stored its share into
// this rank's gathered buffer.  One thread; the arrival total is kept in `seen`.
__global__ void wait_flag_kernel(const unsigned int* flag, unsigned int* seen, unsigned int count,
                                 unsigned int* status) {
  const unsigned int target = *seen + count;
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - target) >= 0) break;
    if (clock64() - t0 > kSpinLimitCycles) {
      atomicExch(status, (unsigned int)kErrDeviceWait);
      break;
    }
  }
  *seen = target;
  __threadfence();
}

// The same wait, then the quantization scale of the gathered h from the ranks' max |h| words
// (each written by its rank ahead of that rank's arrival): scale = max over ranks, turned into
// the scale as the quantizer does it.  The maximum of the shards' maxima is the maximum of the
// whole tensor, so this is the scale the unsharded quantizer computes, bit for bit.
__global__ void wait_flag_scale_kernel(const unsigned int* flag, unsigned int* seen, unsigned int count,
                                       unsigned int* status, const unsigned int* amax_slots, int n,
                                       int slots_hold_scales, float* scale_out) {
  const unsigned int target = *seen + count;
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - target) >= 0) break;
    if (clock64() - t0 > kSpinLimitCycles) {
      atomicExch(status, (unsigned int)kErrDeviceWait);
      break;
    }
  }
  unsigned int best = 0u;
  for (int i = 0; i < n; ++i) {
    unsigned int b;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(b) : "l"(amax_slots + i) : "memory");
    best = b > best ? b : best;      // |h| bit patterns order like the values, NaN on top
  }
  // the scale is a monotone function of the amax (and its lower clamp commutes with max), so
  // the maximum of the ranks' scales is the scale of the maximum
  *scale_out = slots_hold_scales ? __uint_as_float(best) : bq::qd::scale_from_amax(__uint_as_float(best));
  *seen = target;
  __threadfence();
}

// ---------------------------------------------------------------------------
// Persistent tile kernel on CTA pairs (prefill regime, cta_group::2)
// ---------------------------------------------------------------------------
// Two CTAs on neighbouring SMs share one 256 x 256 output tile: each loads 128
// activation rows and 128 weight rows per K block (32 KB instead of the 48 KB a
// lone CTA needs for 128 x 256), the leader issues one MMA that spans both SMs,
// and each CTA keeps the accumulator of its own 128 rows in its tensor memory.
// Shared-memory traffic per flop drops by a third, which is what limits the
// a lone CTA with a 128 x 256 tile.  Warp roles per CTA: 0 = TMA producer, 1 = MMA issuer
// (leader CTA only), 2..5 = epilogue.
//
// Epilogue: eight warps; a warp owns 32 rows (its TMEM lane quarter) and one half of the
// columns of the CTA's 128 x 256 accumulator.  It walks them in pieces of 128 bytes of output
// per row (64 columns of a 16-bit type, 32 of fp32): tcgen05.ld -> scale -> cast -> one 32-row x
// 128-byte box in shared memory, written in the 128-byte swizzle pattern so that neither the
// lane-per-row writes nor the reader meet bank conflicts -> one TMA store of the box (clipped
// at M and N by the tensor map); the next piece waits until the store has read the box.  Outputs whose base or row pitch is not 16-byte aligned
// cannot be described to TMA: the same staged box is then written with coalesced 128-byte
// row segments by the warp itself.
constexpr int kPairStageBytes = 2 * kATileBytes;    // 16 KB activation rows + 16 KB weight rows
constexpr int kPairStages = 6;
constexpr int kPairTile = 256;
constexpr int kPairEpiWarps = 8;                    // two per TMEM lane quarter
constexpr int kTileThreads = 64 + 32 * kPairEpiWarps;
constexpr int kStoreBoxBytes = 32 * 128;            // 32 rows x 128 bytes
constexpr int kPairStagingBytes = kPairEpiWarps * kStoreBoxBytes;   // one box per epilogue warp

// Order in which a weight's 256 x 256 tiles are visited: bands of kRasterM tile rows, inside a
// band the row index runs fastest.  The ~74 tiles in flight at a time then cover about
// 8 x 9 tiles -- (8 + 9) x 256 x K operand bytes, which stay in L2 for every K of the model --
// instead of all tile rows of two or three tile columns (M x K activation bytes per wave:
// 100 MB at M = 8192, K = 12288, more than L2 holds).
constexpr int kRasterM = 8;
__device__ __forceinline__ void pair_tile_coords(int local, int m_tiles, int n_tiles, int& m_idx,
                                                 int& n_idx) {
  const int band_tiles = kRasterM * n_tiles;      // every band but the last is full
  const int band = local / band_tiles;
  const int r = local - band * band_tiles;
  const int m_begin = band * kRasterM;
  const int height = (m_tiles - m_begin) < kRasterM ? (m_tiles - m_begin) : kRasterM;
  n_idx = r / height;
  m_idx = m_begin + (r - n_idx * height);
}

struct alignas(64) OutMaps {
  CUtensorMap y[BQ_MAX_SEGMENTS];
};

// 16 accumulator values -> scaled, cast to the output type, as 16-byte pieces.
template <int ES>
__device__ __forceinline__ void cast16(const uint32_t (&r)[16], float scale, int out_dtype,
                                       uint4 (&out)[ES == 4 ? 4 : 2]) {
  if constexpr (ES == 4) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      out[q] = make_uint4(__float_as_uint(__uint_as_float(r[4 * q]) * scale),
                          __float_as_uint(__uint_as_float(r[4 * q + 1]) * scale),
                          __float_as_uint(__uint_as_float(r[4 * q + 2]) * scale),
                          __float_as_uint(__uint_as_float(r[4 * q + 3]) * scale));
  } else {
    uint32_t w[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float a = __uint_as_float(r[2 * q]) * scale, b = __uint_as_float(r[2 * q + 1]) * scale;
      if (out_dtype == BQ_DTYPE_BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        w[q] = *reinterpret_cast<const uint32_t*>(&v);
      } else {
        const __half2 v = __floats2half2_rn(a, b);
        w[q] = *reinterpret_cast<const uint32_t*>(&v);
      }
    }
    out[0] = make_uint4(w[0], w[1], w[2], w[3]);
    out[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// h = T(T(silu(gate)) * up) of 16 columns from the 16 gate and the 16 up accumulator values of
// the same columns, each first rounded to T as the plain GEMM would have stored it
// (braid/model/mlp.py:46-48), as 16-byte pieces; returns max |h| folded into `mx`.
template <typename T>
__device__ __forceinline__ void silu16(const uint32_t (&g)[16], const uint32_t (&u)[16], float sg,
                                       float su, uint4 (&out)[sizeof(T) == 4 ? 4 : 2], float& mx) {
  using namespace bq::qd;
  T h[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float gg = widen(narrow<T>(__uint_as_float(g[i]) * sg));
    const float uu = widen(narrow<T>(__uint_as_float(u[i]) * su));
    const T sl = silu_to<T>(gg);
    h[i] = narrow<T>(widen(sl) * uu);
    mx = nan_max(mx, fabsf(widen(h[i])));
  }
  const uint4* raw = reinterpret_cast<const uint4*>(h);
#pragma unroll
  for (int q = 0; q < (sizeof(T) == 4 ? 4 : 2); ++q) out[q] = raw[q];
}

// The epilogue of one warp for one tile: 32 rows x 256 accumulator columns.  SILU: the tile's
// columns [0,128) are gate and [128,256) up of the same 128 output columns, and the output is
// h = silu(gate) * up (128 columns); max |h| is folded into `mx`.
template <int ES, bool SILU>
__device__ __forceinline__ void pair_epilogue_rows(const GemmParams& p, const Segment& seg,
                                                   const CUtensorMap* ymap, bool use_tma,
                                                   uint32_t taddr, float scale, float scale_up,
                                                   int m_row0, int n0, uint8_t* box,
                                                   uint32_t box_addr, int lane, int col_half,
                                                   float& mx) {
  constexpr int kCols = 128 / ES;              // output columns per 128-byte piece
  constexpr int kPieces = ES == 4 ? 4 : 2;     // 16-byte pieces per 16 accumulator columns
  const int out_cols = SILU ? kPairTile / 2 : p.pair_n;
  const int c_end = (col_half + 1) * (out_cols / 2);
  for (int c = col_half * (out_cols / 2); c < c_end; c += kCols) {
    // pieces beyond this weight's rows are never stored (warp-uniform)
    if ((n0 + c) >= seg.n) break;
    // the TMA store of the previous piece must have finished reading the box
    if (use_tma && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
#pragma unroll
    for (int j = 0; j < kCols; j += 16) {
      uint32_t r[16];
      tmem_ld16(taddr + c + j, r);          // warp-collective: no divergence before it
      uint4 v[kPieces];
      if constexpr (SILU) {
        uint32_t up[16];
        tmem_ld16(taddr + kPairTile / 2 + c + j, up);
        tmem_ld_wait();
        if constexpr (ES == 4) silu16<float>(r, up, scale, scale_up, v, mx);
        else if (p.out_dtype == BQ_DTYPE_BF16) silu16<__nv_bfloat16>(r, up, scale, scale_up, v, mx);
        else silu16<__half>(r, up, scale, scale_up, v, mx);
      } else {
        tmem_ld_wait();
        cast16<ES>(r, scale, p.out_dtype, v);
      }
#pragma unroll
      for (int q = 0; q < kPieces; ++q) {
        const int piece = (j * ES) / 16 + q;                  // 0..7 along the 128-byte row
        *reinterpret_cast<uint4*>(box + lane * 128 + ((piece ^ (lane & 7)) << 4)) = v[q];
      }
    }
    if (use_tma) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        // column-parallel form: the same box into every rank's gathered buffer (ymap[d] then
        // describes rank d's buffer at this rank's columns; peers' buffers are reached through
        // peer-mapped addresses by plain, non-multicast bulk stores)
        const int n_dst = p.push.n > 0 ? p.push.n : 1;
        for (int d = 0; d < n_dst; ++d) tma_store_2d(ymap + d, box_addr, n0 + c, m_row0);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    } else {
      __syncwarp();
      // 8 lanes cover one 128-byte row segment, 4 rows per pass
      const int piece = lane & 7;
      const int col = n0 + c + piece * (16 / ES);
#pragma unroll
      for (int pass = 0; pass < 8; ++pass) {
        const int row = pass * 4 + (lane >> 3);
        const int m = m_row0 + row;
        const uint4 v = *reinterpret_cast<const uint4*>(box + row * 128 + ((piece ^ (row & 7)) << 4));
        if (m < p.M && col < seg.n) {         // n is a multiple of 16: a piece is in or out as a whole
          // rows are 8-byte aligned at least (checked by the host)
          if (p.push.n == 0) {
            uint8_t* dst = static_cast<uint8_t*>(seg.y) + ((long long)m * seg.ldy + col) * ES;
            *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
            *reinterpret_cast<uint2*>(dst + 8) = make_uint2(v.z, v.w);
          } else {
            // column-parallel form: the same piece into every rank's gathered buffer (plain
            // stores through peer-mapped pointers, this rank's own buffer included)
            // 16-byte stores (destinations and row pitch are 16-byte aligned, checked by the
            // host): 8 lanes write one whole 128-byte line, which is what the link moves well --
            // halves of 32-byte sectors, as the 8-byte stores above produce, reached 0.3 TB/s
            const long long at = ((long long)m * p.push.ld + col) * ES;
            for (int d = 0; d < p.push.n; ++d)
              *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.push.dst[d]) + at) = v;
          }
        }
      }
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(kTileThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_x,
                 const __grid_constant__ WeightMaps tm_w, const __grid_constant__ OutMaps tm_y,
                 const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t bar_base = base + kPairStages * kPairStageBytes;
  auto a_tile = [&](int s) { return base + s * kPairStageBytes; };
  auto b_tile = [&](int s) { return base + s * kPairStageBytes + kATileBytes; };
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * kPairStages + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * kPairStages + 2 + b); };
  volatile uint32_t* const tmem_slot = reinterpret_cast<volatile uint32_t*>(
      base_ptr + kPairStages * kPairStageBytes + 8 * (2 * kPairStages + 4));
  volatile uint32_t* const abort_flag = tmem_slot + 1;
  // store boxes of the epilogue warps, after the barrier block (1024-byte aligned: the swizzle
  // pattern of a box is a function of its address bits)
  uint8_t* const staging = base_ptr + kPairStages * kPairStageBytes + kBarrierBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());     // 0 = leader of the pair
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + kPairTile - 1) / kPairTile;
  const bool silu = p.pair.on != 0;                       // gate/up tiles, h = silu(gate) * up out
  // output columns per tile: 128 of h in the SiLU form; 256 in the plain form, or 128 for a weight
  // so narrow that 256-wide tiles would leave CTA pairs without work (same sums, more tiles)
  const int n_step = silu ? kPairTile / 2 : p.pair_n;
  const int b_rows = silu ? kRowTile : p.pair_n / 2;       // weight rows this CTA loads per K block
  float* const s_amax = reinterpret_cast<float*>(base_ptr + kPairStages * kPairStageBytes + 512);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_x);
    for (int i = 0; i < p.n_seg; ++i) tma_prefetch_desc(&tm_w.w[i]);
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full_bar(s), 1);     // the leader's producer arrives, bytes of both CTAs expected
      mbar_init(empty_bar(s), 1);    // one MMA commit per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 2 * kPairEpiWarps);    // the epilogue warps of both CTAs of the pair
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();     // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait_prior_grids();

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol = policy_evict_last();
      int it = 0;
      bool ok = true;
      for (int t = pair; t < p.total_tiles && ok; t += n_pairs) {
        const int sg = find_segment(p, t);
        const int local = t - p.seg[sg].tile_begin;
        int m_idx, n_idx;
        pair_tile_coords(local, m_tiles, (p.seg[sg].n + n_step - 1) / n_step, m_idx, n_idx);
        const int m0 = m_idx * kPairTile + rank * kRowTile;
        // plain: this CTA's half of the tile's 256 weight rows; SiLU form: the leader loads 128
        // gate rows, its peer the 128 up rows of the same output columns
        const int n0 = silu ? n_idx * kRowTile : n_idx * n_step + rank * b_rows;
        const CUtensorMap* const w_map = silu ? &tm_w.w[rank] : &tm_w.w[sg];
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kPairStages, use = it / kPairStages;
          if (use > 0 && !mbar_wait(empty_bar(s), (use - 1) & 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(s), 2u * (kATileBytes + (uint32_t)b_rows * kBK));
          tma_load_2d_pair(a_tile(s), &tm_x, full_bar(s), kb * kBK, m0, pol);
          tma_load_2d_pair(b_tile(s), w_map, full_bar(s), kb * kBK, n0, pol);
        }
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = (silu || p.pair_n == kPairTile) ? idesc_e4m3(kPairTile, kPairTile)
                                                             : idesc_e4m3(kPairTile, kPairTile / 2);
      int it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = pair; t < p.total_tiles && ok; t += n_pairs, ++tile_iter) {
        const int b = tile_iter & 1, use_b = tile_iter >> 1;
        if (use_b > 0 && !mbar_wait(acc_empty(b), (use_b - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + b * kPairTile;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kPairStages, use = it / kPairStages;
          if (!mbar_wait(full_bar(s), use & 1)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = smem_desc_sw128(a_tile(s));
          const uint64_t db = smem_desc_sw128(b_tile(s));
#pragma unroll
          for (int j = 0; j < kBK / kUmmaK; ++j)
            mma_f8_pair(tmem_d, da + 2u * j, db + 2u * j, idesc, (kb | j) != 0 ? 1u : 0u);
          // the stage is free in BOTH CTAs once these MMAs retire
          mma_commit_pair(empty_bar(s));
          mma_commit_pair(map_to_cta(empty_bar(s), 1));
        }
        if (ok) {
          mma_commit_pair(acc_full(b));
          mma_commit_pair(map_to_cta(acc_full(b), 1));
        }
      }
      if (!ok) *abort_flag = 1;
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;                   // TMEM lanes [32 * quad, +32): rows of the tile
    const int col_half = (warp - 2) >> 2;        // which half of the columns this warp stores
    int tile_iter = 0;
    bool ok = true;
    float h_max = 0.0f;                          // SiLU form: max |h| over everything this thread wrote
    uint8_t* const stage = staging + (warp - 2) * kStoreBoxBytes;
    const uint32_t stage_addr = smem_u32(stage);
    const uint32_t leader_acc_empty0 = map_to_cta(acc_empty(0), 0);
    const uint32_t leader_acc_empty1 = map_to_cta(acc_empty(1), 0);
    for (int t = pair; t < p.total_tiles && ok; t += n_pairs, ++tile_iter) {
      const int b = tile_iter & 1, use_b = tile_iter >> 1;
      const int sg = find_segment(p, t);
      const Segment seg = p.seg[sg];
      const int local = t - seg.tile_begin;
      int m_idx, n_idx;
      pair_tile_coords(local, m_tiles, (seg.n + n_step - 1) / n_step, m_idx, n_idx);
      const int m0 = m_idx * kPairTile + rank * kRowTile;
      const int n0 = n_idx * n_step;
      if (!mbar_wait(acc_full(b), use_b & 1)) { ok = false; break; }
      tc_fence_after();
      const float sx = __ldg(p.sx);
      const float scale = sx * __ldg(seg.sw);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + b * kPairTile;
      const bool use_tma = seg.y_tma != 0;
      if (silu) {
        const float scale_up = sx * __ldg(p.pair.sw_up);
        if (p.out_dtype == BQ_DTYPE_F32)
          pair_epilogue_rows<4, true>(p, seg, &tm_y.y[p.push.n > 0 ? 0 : sg], use_tma, taddr, scale, scale_up,
                                      m0 + quad * 32, n0, stage, stage_addr, lane, col_half, h_max);
        else
          pair_epilogue_rows<2, true>(p, seg, &tm_y.y[p.push.n > 0 ? 0 : sg], use_tma, taddr, scale, scale_up,
                                      m0 + quad * 32, n0, stage, stage_addr, lane, col_half, h_max);
      } else if (p.out_dtype == BQ_DTYPE_F32) {
        pair_epilogue_rows<4, false>(p, seg, &tm_y.y[p.push.n > 0 ? 0 : sg], use_tma, taddr, scale, 0.0f, m0 + quad * 32,
                                     n0, stage, stage_addr, lane, col_half, h_max);
      } else {
        pair_epilogue_rows<2, false>(p, seg, &tm_y.y[p.push.n > 0 ? 0 : sg], use_tma, taddr, scale, 0.0f, m0 + quad * 32,
                                     n0, stage, stage_addr, lane, col_half, h_max);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(b == 0 ? leader_acc_empty0 : leader_acc_empty1);
    }
    // the boxes must stay valid until the last stores have read them; for the column-parallel
    // form the wait also means the stores have been written, before anybody is told to look
    if (lane == 0) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (p.push.n > 0) asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncwarp();
    if (!ok) *abort_flag = 1;
    if (p.push.n > 0) {
      // The stores of all epilogue threads are ordered before the elected thread's fence by the
      // barrier (fences are cumulative); the fence orders them before this CTA's count; the
      // last CTA sees every count, fences again and only then signals the ranks: every store of
      // the launch happens before every arrival.
      const bool want_amax = silu && p.push.amax_local != nullptr;
      if (want_amax) {
        using namespace bq::qd;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
          h_max = nan_max(h_max, __shfl_xor_sync(0xffffffffu, h_max, off));
        if (lane == 0) s_amax[warp - 2] = h_max;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kPairEpiWarps) : "memory");
      if (warp == 2 && lane == 0) {
        if (want_amax) {
          using namespace bq::qd;
          float w = s_amax[0];
#pragma unroll
          for (int i = 1; i < kPairEpiWarps; ++i) w = nan_max(w, s_amax[i]);
          // bit patterns of |h| order like the values, NaN on top: exact and order-free
          atomicMax(p.push.amax_local, __float_as_uint(w));
        }
        __threadfence_system();
        const unsigned int old = atomicAdd(p.push.done, 1u);
        if (old == p.push.expected - 1u) {
          *p.push.done = 0u;                     // ready for the next launch on this scratch
          if (want_amax) {
            // every CTA's max is in (its atomicMax precedes its count): hand this rank's
            // max |h| to every rank, ahead of the arrival that tells them to look
            const unsigned int bits = atomicExch(p.push.amax_local, 0u);
            for (int d = 0; d < p.push.n; ++d)
              if (p.push.amax_dst[d] != nullptr)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.push.amax_dst[d]), "r"(bits) : "memory");
          }
          __threadfence_system();
          for (int d = 0; d < p.push.n; ++d)
            asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.push.flag[d]) : "memory");
        }
      }
    } else if (silu) {
      // max |h| of the launch: warps -> CTA -> one atomicMax per CTA on the bit pattern (exact
      // and order-free; NaN patterns sort on top); the CTA that arrives last turns the result into
      // the scale of h and returns the scratch words to zero
      using namespace bq::qd;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
        h_max = nan_max(h_max, __shfl_xor_sync(0xffffffffu, h_max, off));
      if (lane == 0) s_amax[warp - 2] = h_max;
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kPairEpiWarps) : "memory");      // the epilogue warps
      if (warp == 2 && lane == 0) {
        float w = s_amax[0];
#pragma unroll
        for (int i = 1; i < kPairEpiWarps; ++i) w = nan_max(w, s_amax[i]);
        unsigned int* const words = p.pair.words;
        atomicMax(&words[0], __float_as_uint(w));
        __threadfence();
        const unsigned int old = atomicAdd(&words[1], 1u);
        if (old == gridDim.x - 1) {
          __threadfence();
          const unsigned int bits = atomicMax(&words[0], 0u);
          p.pair.sh[0] = scale_from_amax(__uint_as_float(bits));
          words[0] = 0u;
          words[1] = 0u;
          __threadfence();
        }
      }
    }
  }

  tc_fence_before();
  cluster_sync_all();     // nobody frees tensor memory while the peer may still use the pair
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, (unsigned int)kErrDeviceWait);
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// [rows, K] uint8 row-major tensor, box = 128 K-bytes x box_rows, 128-byte swizzle,
// out-of-range rows/columns read as zero.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return kErrNoDriver;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? kOk : kErrUnsupported;
}

// [M, N] output of the prefill kernel, row pitch ldy elements: boxes of 32 rows x 128 bytes,
// 128-byte swizzle; rows beyond M and columns beyond N are clipped by the store.
int make_out_map(CUtensorMap* out, void* ptr, long long M, long long N, long long ldy, int out_dtype) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return kErrNoDriver;
  const cuuint64_t es = out_dtype == BQ_DTYPE_F32 ? 4 : 2;
  const CUtensorMapDataType dt = out_dtype == BQ_DTYPE_F32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : out_dtype == BQ_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)ldy * es};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / es), 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(out, dt, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? kOk : kErrUnsupported;
}

int device_sms() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (sms[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    sms[dev] = v;
  }
  return sms[dev];
}

long long g_opt_split = 0, g_opt_stages = 0, g_opt_stream_max_m = 256, g_opt_cta_target = 160;
long long g_opt_push_tma = 1;   // prefill push epilogue: bulk tensor stores (0: 16-byte plain stores)
long long g_opt_pair_narrow = -1;   // prefill: 128-column tiles for a lone narrow weight (-1 auto, 0 never, 1 always)
long long g_opt_pdl = 1;   // programmatic dependent launch on by default
long long g_opt_b_stages = 0;   // activation ring depth: 0 = heuristic, -1 = as deep as the weight ring
long long g_opt_smem_cap = 0;   // 0 = no cap on pipeline bytes per CTA
thread_local long long g_last_launch[6] = {0, 0, 0, 0, 0, 0};

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int configure_once() {
  static int rc = -1;
  if (rc < 0) {
    cudaError_t e1 = cudaFuncSetAttribute(gemm_stream_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    cudaError_t e3 = cudaFuncSetAttribute(gemm_pair_kernel,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    rc = (e1 == cudaSuccess && e3 == cudaSuccess) ? kOk : kErrLaunch;
    if (rc != kOk) (void)cudaGetLastError();
  }
  return rc;
}

// Largest grid of the stream kernel that is resident at once with this cluster
// size and shared-memory footprint (the paired gate/up epilogue has a grid-wide wait).
int max_resident_ctas(int cluster, int smem) {
  struct Entry { int cluster, smem, cap; };
  static Entry cache[64];
  static int n_cached = 0;
  for (int i = 0; i < n_cached; ++i)
    if (cache[i].cluster == cluster && cache[i].smem == smem) return cache[i].cap;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(cluster * 64), 1, 1);
  cfg.blockDim = dim3(kStreamThreads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_stream_kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    clusters = 0;
  }
  // The occupancy calculator reports one CTA per SM for this kernel even where two
  // demonstrably run side by side (all 256 CTAs of a 100 KB launch start within 1.3 us of
  // each other), so the per-SM count is derived from the resources themselves: shared
  // memory (1 KB reserved per CTA), registers, and the two-CTA cap of the launch bounds.
  cudaFuncAttributes fa;
  memset(&fa, 0, sizeof(fa));
  int regs = 128;
  if (cudaFuncGetAttributes(&fa, gemm_stream_kernel) == cudaSuccess && fa.numRegs > 0)
    regs = fa.numRegs;
  else
    (void)cudaGetLastError();
  int per_sm = 233472 / (smem + 1024);
  const int by_regs = 65536 / (((regs + 7) / 8) * 8 * kStreamThreads);
  if (per_sm > by_regs) per_sm = by_regs;
  if (per_sm > 2) per_sm = 2;
  if (per_sm < 1) per_sm = 1;
  int cap = clusters * cluster * per_sm > 0 ? clusters * cluster * per_sm : -1;
  if (getenv("BQ_DEBUG"))
    fprintf(stderr, "[bq] residency: cluster %d smem %d regs %d -> %d clusters x %d per SM = %d CTAs\n",
            cluster, smem, regs, clusters, per_sm, cap);
  if (n_cached < 64) cache[n_cached++] = Entry{cluster, smem, cap};
  return cap;
}

// K slices of one weight.  A function of the weight's own shape only -- never of
// what else shares the launch or of the batch -- so an output element is summed
// in the same order whether its weight is multiplied alone or grouped with
// others (`project` stays bit-identical to per-weight calls).  Small weights
// are sliced so that their tiles x slices cover most of the SMs.
int split_for_weight(long long n_rows, int k_blocks) {
  const long long tiles = (n_rows + kRowTile - 1) / kRowTile;
  // at most 4: clusters of 8 leave a fifth of the SMs unusable (15 clusters of 8 fit on the
  // 148 SMs, against 33 clusters of 4)
  int s = 1;
  while (s < 4 && tiles * (s * 2) <= g_opt_cta_target && (s * 2) * 2 <= k_blocks) s *= 2;
  if (g_opt_split > 0) {
    s = 1;
    while (s * 2 <= g_opt_split && s < 8) s *= 2;
    while (s > 1 && s > k_blocks) s /= 2;
  }
  return s;
}

int launch_stream(const CUtensorMap& tm_x, const CUtensorMap& tm_xd, const WeightMaps& maps,
                  GemmParams& p, cudaStream_t stream) {
  const int sms = device_sms();
  if (sms <= 0) return kErrLaunch;
  p.mma_n = ((p.M + 15) / 16) * 16;
  const int b_tile = p.mma_n * kBK;
  const int stage_bytes = kATileBytes + b_tile;
  int cluster = 1, min_split = 8;
  for (int i = 0; i < p.n_seg; ++i) {
    p.seg[i].split = p.seg[i].split_forced > 0 ? p.seg[i].split_forced
                                               : split_for_weight(p.seg[i].n, p.seg[i].dense ? p.k_blocks_dense
                                                                                             : p.k_blocks);
    if (p.seg[i].split > cluster) cluster = p.seg[i].split;
    if (p.seg[i].split < min_split) min_split = p.seg[i].split;
  }
  p.cluster = cluster;
  int clusters = 0;
  for (int i = 0; i < p.n_seg; ++i) {
    const int tiles = (p.seg[i].n + kRowTile - 1) / kRowTile;
    const int per_cluster = cluster / p.seg[i].split;
    p.seg[i].cluster_begin = clusters;
    clusters += (tiles + per_cluster - 1) / per_cluster;
  }
  const long long grid = (long long)clusters * cluster;
  if (grid > 0x7fffffffLL) return kErrTooLarge;
  int kb_max = (p.k_blocks + min_split - 1) / min_split;
  for (int i = 0; i < p.n_seg; ++i)
    if (p.seg[i].dense) {
      const int kb = (p.k_blocks_dense + p.seg[i].split - 1) / p.seg[i].split;
      if (kb > kb_max) kb_max = kb;
    }
  const int staging = p.mma_n * kRowTile * 4;
  // Shared memory per CTA: small enough that the whole grid is resident at once
  // (up to 2 CTAs per SM: 256 threads x ~128 registers each), so one CTA's
  // epilogue overlaps its neighbour's loads.
  int per_sm = (int)((grid + sms - 1) / sms);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2) per_sm = 2;
  int budget = kMaxSmem / per_sm - 1024 - kBarrierBytes - 1024;
  // Leave room for the NEXT kernel's CTAs: with programmatic dependent launch they
  // become resident while this kernel still runs and pre-load their weights.
  if (g_opt_smem_cap > 0 && budget > g_opt_smem_cap) budget = (int)g_opt_smem_cap;
  int stages = budget / stage_bytes;            // both rings equally deep: the starting point
  if (stages > kb_max) stages = kb_max;
  if (stages > 24) stages = 24;
  if (stages < 2) stages = kb_max < 2 ? kb_max : 2;
  if (g_opt_stages > 0 && g_opt_stages < stages) stages = (int)g_opt_stages;
  int b_stages = stages;
  // Wide batch tiles: a shallow activation ring (its tiles are L2 hits), the rest goes to
  // weight tiles in flight.  Two slots cover the L2 latency at the rate one CTA of a two-per-SM
  // launch consumes tiles; a CTA that has the SM to itself consumes twice as fast.
  long long want_b = g_opt_b_stages;
  if (want_b == 0) want_b = b_tile >= 8192 ? (per_sm == 2 ? 2 : 4) : -1;
  if (want_b > 0 && want_b < b_stages && !(g_opt_stages > 0)) {
    b_stages = (int)want_b;
    stages = (budget - b_stages * b_tile) / kATileBytes;
    if (stages > kb_max) stages = kb_max;
    if (stages > 24) stages = 24;
    if (b_stages > stages) b_stages = stages;
  }
  p.stages = stages;
  p.b_stages = b_stages;
  int tile_bytes = stages * kATileBytes + b_stages * b_tile;
  if (tile_bytes < staging) tile_bytes = staging;
  const int smem = tile_bytes + kBarrierBytes + 1024;
  if (smem > kMaxSmem) return kErrUnsupported;
  if (p.pair.on) p.pair.expected = (unsigned)((p.seg[0].n / kRowTile) * p.seg[0].split);
  if (p.push.n > 0)
    p.push.expected = (unsigned)(((p.seg[0].n + kRowTile - 1) / kRowTile) * p.seg[0].split);
  if (p.pair.on && p.push.n == 0) {
    // the epilogue's amax exchange waits on the whole grid: every CTA must be resident
    const int cap = max_resident_ctas(cluster, smem);
    if (getenv("BQ_DEBUG"))
      fprintf(stderr, "[bq] paired launch: grid %lld cluster %d smem %d resident cap %d\n", grid,
              cluster, smem, cap);
    if (cap <= 0 || grid > cap) return kErrUnsupported;
  }

  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(kStreamThreads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt_pdl ? 2 : 1;
  g_last_launch[0] = 0; g_last_launch[1] = grid; g_last_launch[2] = cluster;
  g_last_launch[3] = stages; g_last_launch[4] = smem; g_last_launch[5] = p.mma_n;
#ifdef BQ_PHASES
  p.phase_ring = bq::phase_ring_for_launch(&p.phase_seq);
#endif
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel, tm_x, tm_xd, maps, p, tile_bytes);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return kErrLaunch; }
  return kOk;
}

int launch_pair(const CUtensorMap& tm_x, const WeightMaps& maps, const OutMaps& ymaps, GemmParams& p,
                cudaStream_t stream) {
  const int sms = device_sms();
  if (sms <= 0) return kErrLaunch;
  const int smem = kPairStages * kPairStageBytes + kBarrierBytes + kPairStagingBytes + 1024;
  static_assert(kPairStages * kPairStageBytes + kBarrierBytes + kPairStagingBytes + 1024 <= kMaxSmem,
                "pair kernel: pipeline + store boxes exceed the shared memory of an SM");
  int pairs = p.total_tiles < sms / 2 ? p.total_tiles : sms / 2;
  if (pairs < 1) pairs = 1;
  if (p.push.n > 0) p.push.expected = (unsigned)(2 * pairs);   // every CTA has a tile and stores
  g_last_launch[0] = 2; g_last_launch[1] = 2 * pairs; g_last_launch[2] = 2;
  g_last_launch[3] = kPairStages; g_last_launch[4] = smem; g_last_launch[5] = p.pair_n;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(kTileThreads, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt_pdl ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel, tm_x, maps, ymaps, p);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return kErrLaunch; }
  return kOk;
}

}  // namespace

namespace bq {
int gemm_set_option(const char* key, long long value);
}
int bq::gemm_set_option(const char* key, long long value) {
  if (strcmp(key, "decode_split_k") == 0) { g_opt_split = value; return kOk; }
  if (strcmp(key, "decode_stages") == 0) { g_opt_stages = value; return kOk; }
  if (strcmp(key, "decode_b_stages") == 0) { g_opt_b_stages = value; return kOk; }
  if (strcmp(key, "gemm_pdl") == 0) { g_opt_pdl = value ? 1 : 0; return kOk; }
  if (strcmp(key, "push_tma") == 0) { g_opt_push_tma = value ? 1 : 0; return kOk; }
  if (strcmp(key, "pair_narrow") == 0) { g_opt_pair_narrow = value < 0 ? -1 : (value ? 1 : 0); return kOk; }
  if (strcmp(key, "decode_smem_cap") == 0) { g_opt_smem_cap = value; return kOk; }
  if (strcmp(key, "decode_cta_target") == 0) {
    if (value < 1) return kErrBadArg;
    g_opt_cta_target = value;
    return kOk;
  }
  if (strcmp(key, "stream_max_m") == 0) {
    if (value < 1 || value > 256) return kErrBadArg;
    g_opt_stream_max_m = value;
    return kOk;
  }
  return kErrBadArg;
}

extern "C" size_t bq_gemm_workspace_bytes(int64_t, int64_t, int64_t) {
  // the status word and the counters of the paired / push epilogues; partial sums never leave the chip
  return 16;
}

namespace {

// Weights of a mixed launch that are NOT quantized: kind[i] != 0 marks segment i as a 16-bit
// weight [N_i, K] of type `dtype`, multiplied with the unquantized activation `x` [M, K].
struct DenseArgs {
  const void* x;
  int dtype;
  const int* kind;
};

int run_grouped(const void* xq, const float* sx, int64_t M, int64_t K, int n_seg,
                const void* const* wq, const float* const* sw, void* const* y, const int64_t* N,
                const int64_t* ldy, int out_dtype, void* ws, size_t ws_bytes, void* stream_v,
                const void* const* res = nullptr,
                const int64_t* ld_res = nullptr, const PairSilu* pair = nullptr,
                int split_forced = 0, const PushParams* push = nullptr,
                const DenseArgs* dn = nullptr, const ArgmaxOut* am = nullptr) {
  if (!xq || !sx || !wq || !sw || !y || !N || !ldy || M <= 0 || K <= 0) return kErrBadArg;
  if (n_seg < 1 || n_seg > BQ_MAX_SEGMENTS) return kErrBadArg;
  if (out_dtype != BQ_DTYPE_F32 && out_dtype != BQ_DTYPE_BF16 && out_dtype != BQ_DTYPE_F16)
    return kErrBadArg;
  if (ws == nullptr || ws_bytes < 16u || !aligned_to(ws, 16)) return kErrWorkspace;
  if (K % 16 || !aligned_to(xq, 16)) return kErrUnsupported;
  if (M > 0x7fffff00LL || K > 0x7fffff00LL) return kErrTooLarge;
  const int out_align = out_dtype == BQ_DTYPE_F32 ? 16 : 8;
  for (int i = 0; i < n_seg; ++i) {   // argument checks first: no CUDA call before they pass
    const bool is_dense = dn != nullptr && dn->kind[i] != 0;
    if (!wq[i] || (!sw[i] && !is_dense) || N[i] <= 0) return kErrBadArg;
    if (N[i] % 16 || !aligned_to(wq[i], 16)) return kErrUnsupported;
    if ((pair == nullptr || pair->prefill) && push == nullptr &&
        !(am != nullptr && !am->store_logits)) {   // forms that write y
      if (!y[i]) return kErrBadArg;
      if (ldy[i] < N[i] || ldy[i] % 4 || !aligned_to(y[i], out_align)) return kErrUnsupported;
    }
    if (N[i] > 0x7fffff00LL) return kErrTooLarge;
  }
  const bool stream_path = M <= g_opt_stream_max_m;
  if (dn != nullptr) {    // 16-bit segments exist in the weight-streaming kernel only
    if (!stream_path || pair || push || res) return kErrUnsupported;
    if (!dn->x || (dn->dtype != BQ_DTYPE_BF16 && dn->dtype != BQ_DTYPE_F16)) return kErrBadArg;
    if (!aligned_to(dn->x, 16)) return kErrUnsupported;
  }
  if (pair && stream_path == (pair->prefill != 0)) return kErrUnsupported;   // each form has its regime
  if (pair && (res || n_seg != 1)) return kErrBadArg;
  if (push) {
    if (res || n_seg != 1) return kErrBadArg;
    // the prefill kernel stores 16-byte pieces
    if (!stream_path) {
      const long long es = out_dtype == BQ_DTYPE_F32 ? 4 : 2;
      if ((push->ld * es) % 16) return kErrUnsupported;
      for (int d = 0; d < push->n; ++d)
        if (!aligned_to(push->dst[d], 16)) return kErrUnsupported;
    }
  }
  if (res != nullptr) {   // the residual epilogue exists in the weight-streaming kernel only
    if (!stream_path || ld_res == nullptr) return kErrUnsupported;
    for (int i = 0; i < n_seg; ++i)
      if (res[i] && (ld_res[i] < N[i] || ld_res[i] % 4 || !aligned_to(res[i], out_align)))
        return kErrUnsupported;
  }
  if (int rc = configure_once()) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  GemmParams p;
  memset(&p, 0, sizeof(p));
  WeightMaps maps;
  memset(&maps, 0, sizeof(maps));
  p.n_seg = n_seg;
  p.sx = sx;
  p.M = (int)M;
  p.k_blocks = (int)((K + kBK - 1) / kBK);
  p.k_blocks_dense = (int)((2 * K + kBK - 1) / kBK);
  p.dense_fmt = (dn != nullptr && dn->dtype == BQ_DTYPE_BF16) ? 1 : 0;
  p.out_dtype = out_dtype;
  // the sticky status word is the 4th word of the scratch, as in the quantizer
  p.status = static_cast<unsigned int*>(ws) + 3;
  if (pair) {
    p.pair = *pair;
    p.pair.on = 1;
    p.pair.words = static_cast<unsigned int*>(ws);
  }
  if (am) {
    if (!stream_path || pair || push || res || dn || n_seg != 1) return kErrUnsupported;
    p.argmax = *am;
    p.argmax.on = 1;
  }
  if (push) {
    p.push = *push;
    p.push.done = static_cast<unsigned int*>(ws);   // first scratch word: zero between launches
    // second scratch word: the launch's running max |h| where the ranks want it
    p.push.amax_local = (push->amax_dst[0] != nullptr) ? static_cast<unsigned int*>(ws) + 1 : nullptr;
  }

  const bool pair_path = !stream_path;
  p.m_tiles = pair_path ? (int)((M + kPairTile - 1) / kPairTile) : (int)((M + kRowTile - 1) / kRowTile);
  // plain prefill form of ONE narrow weight: 128-column tiles when all of them still run at once,
  // i.e. when 256-column ones would leave half of the CTA pairs without a tile (the sums are the
  // same, tile by tile; a 128-column tile takes 0.6-0.75 of a 256-column one, so a second round
  // of them costs more than the idle pairs do)
  p.pair_n = kPairTile;
  if (pair_path && pair == nullptr && n_seg == 1) {
    const long long wide_tiles = ((N[0] + kPairTile - 1) / kPairTile) * p.m_tiles;
    const long long pairs = device_sms() / 2;
    const bool narrow = g_opt_pair_narrow > 0 || (g_opt_pair_narrow < 0 && wide_tiles * 2 <= pairs);
    if (narrow) p.pair_n = kPairTile / 2;
  }
  const int w_box_rows = (pair_path && pair == nullptr) ? p.pair_n / 2 : kRowTile;
  const int tile_n = pair_path ? ((pair && pair->prefill) ? kPairTile / 2 : p.pair_n) : kRowTile;
  OutMaps ymaps;
  memset(&ymaps, 0, sizeof(ymaps));
  int tiles = 0;
  for (int i = 0; i < n_seg; ++i) {
    p.seg[i].sw = sw[i];
    const bool no_y = (pair && !pair->prefill) || push || (am != nullptr && !am->store_logits);
    p.seg[i].y = no_y ? nullptr : y[i];
    p.seg[i].ldy = no_y ? 0 : ldy[i];
    p.seg[i].split_forced = split_forced;
    p.seg[i].res = res ? res[i] : nullptr;
    p.seg[i].ld_res = res ? ld_res[i] : 0;
    p.seg[i].n = (int)N[i];
    p.seg[i].dense = (dn != nullptr && dn->kind[i] != 0) ? 1 : 0;
    p.seg[i].tile_begin = tiles;
    const long long nt = (N[i] + tile_n - 1) / tile_n;
    const long long add = stream_path ? nt : nt * p.m_tiles;
    if (tiles + add > 0x3fffffffLL) return kErrTooLarge;
    tiles += (int)add;
    if (pair_path && !no_y) {
      const size_t es = out_dtype == BQ_DTYPE_F32 ? 4 : 2;
      p.seg[i].y_tma = aligned_to(y[i], 16) && (ldy[i] * es) % 16 == 0 &&
                       make_out_map(&ymaps.y[i], y[i], M, N[i], ldy[i], out_dtype) == kOk;
    }
    if (pair_path && push && g_opt_push_tma) {
      // one map per destination rank over its [M, N shard] window (n_seg is 1 for a push)
      bool ok = true;
      for (int d = 0; d < push->n && ok; ++d)
        ok = make_out_map(&ymaps.y[d], push->dst[d], M, N[i], push->ld, out_dtype) == kOk;
      p.seg[i].y_tma = ok ? 1 : 0;
    }
    if (pair && pair->prefill) {
      // two maps over the two weights, 128-row boxes: one CTA of a pair loads gate rows, the other
      // the up rows of the same output columns
      if (int rc = make_map(&maps.w[0], wq[0], N[0], K, kRowTile)) return rc;
      if (int rc = make_map(&maps.w[1], pair->wq_up, N[0], K, kRowTile)) return rc;
    } else if (pair) {
      // two maps over the two weights, 64-row boxes: the kernel puts a tile together from both
      if (int rc = make_map(&maps.w[0], wq[0], N[0] / 2, K, kRowTile / 2)) return rc;
      if (int rc = make_map(&maps.w[1], pair->wq_up, N[0] / 2, K, kRowTile / 2)) return rc;
    } else if (int rc = make_map(&maps.w[i], wq[i], N[i], p.seg[i].dense ? 2 * K : K, w_box_rows)) {
      return rc;     // a 16-bit weight is described by its bytes: [N, 2K]
    }
  }
  p.total_tiles = tiles;
  CUtensorMap tm_x;
  if (stream_path) {
    const int mma_n = (int)(((M + 15) / 16) * 16);
    if (int rc = make_map(&tm_x, xq, M, K, mma_n)) return rc;
    CUtensorMap tm_xd = tm_x;
    if (dn != nullptr)
      if (int rc = make_map(&tm_xd, dn->x, M, 2 * K, mma_n)) return rc;
    return launch_stream(tm_x, tm_xd, maps, p, stream);
  }
  if (int rc = make_map(&tm_x, xq, M, K, kRowTile)) return rc;
  return launch_pair(tm_x, maps, ymaps, p, stream);
}

}  // namespace

extern "C" int bq_gemm_w8a8_grouped(const void* xq, const float* sx, int64_t M, int64_t K, int n_seg,
                                    const void* const* wq, const float* const* sw, void* const* y,
                                    const int64_t* N, const int64_t* ldy, int out_dtype, void* ws,
                                    size_t ws_bytes, void* stream_v) {
  return run_grouped(xq, sx, M, K, n_seg, wq, sw, y, N, ldy, out_dtype, ws, ws_bytes, stream_v);
}

extern "C" int bq_project_mixed(const void* xq, const float* sx, const void* x_dense, int dense_dtype,
                                int64_t M, int64_t K, int n_seg, const void* const* w,
                                const float* const* sw, const int* kind, void* const* y,
                                const int64_t* N, const int64_t* ldy, int out_dtype, void* ws,
                                size_t ws_bytes, void* stream_v) {
  if (kind == nullptr) return kErrBadArg;
  bool any_dense = false;
  for (int i = 0; i < n_seg && i < BQ_MAX_SEGMENTS; ++i) any_dense = any_dense || kind[i] != 0;
  if (!any_dense)
    return run_grouped(xq, sx, M, K, n_seg, w, sw, y, N, ldy, out_dtype, ws, ws_bytes, stream_v);
  if (out_dtype != dense_dtype) return kErrUnsupported;   // F.linear returns the activation's type
  const DenseArgs dn{x_dense, dense_dtype, kind};
  return run_grouped(xq, sx, M, K, n_seg, w, sw, y, N, ldy, out_dtype, ws, ws_bytes, stream_v,
                     nullptr, nullptr, nullptr, 0, nullptr, &dn);
}

extern "C" int bq_gemm_w8a8(const void* xq, const void* wq, const float* sx, const float* sw,
                            void* y, int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldy,
                            void* ws, size_t ws_bytes, void* stream) {
  const void* wqs[1] = {wq};
  const float* sws[1] = {sw};
  void* ys[1] = {y};
  const int64_t Ns[1] = {N};
  const int64_t ldys[1] = {ldy};
  return bq_gemm_w8a8_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, out_dtype, ws, ws_bytes,
                              stream);
}

extern "C" size_t bq_lm_head_argmax_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  return static_cast<size_t>((N + kRowTile - 1) / kRowTile) * static_cast<size_t>(M) * sizeof(uint2);
}

extern "C" int bq_lm_head_argmax(const void* xq, const void* wq, const float* sx, const float* sw,
                                 int out_dtype, int64_t M, int64_t N, int64_t K, void* logits_or_null,
                                 int64_t ldy, int64_t* idx_out, void* partial, size_t partial_bytes,
                                 void* ws, size_t ws_bytes, void* stream) {
  if (!idx_out || !partial || M <= 0 || N <= 0) return kErrBadArg;
  if (M > g_opt_stream_max_m) return kErrUnsupported;
  if (partial_bytes < bq_lm_head_argmax_workspace_bytes(M, N) || !aligned_to(partial, 8) ||
      !aligned_to(idx_out, 8))
    return kErrWorkspace;
  ArgmaxOut am;
  memset(&am, 0, sizeof(am));
  am.store_logits = logits_or_null != nullptr ? 1 : 0;
  am.partial = static_cast<uint2*>(partial);
  const void* wqs[1] = {wq};
  const float* sws[1] = {sw};
  void* ys[1] = {logits_or_null};
  const int64_t Ns[1] = {N};
  const int64_t ldys[1] = {ldy};
  // K is not split: every tile's logits are final inside one CTA
  if (int rc = run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, out_dtype, ws, ws_bytes, stream,
                           nullptr, nullptr, nullptr, 1, nullptr, nullptr, &am))
    return rc;
  const int tiles = (int)((N + kRowTile - 1) / kRowTile);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)M, 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_finish_kernel, am.partial, tiles, (int)M,
                                           reinterpret_cast<long long*>(idx_out));
  if (e != cudaSuccess) { (void)cudaGetLastError(); return kErrLaunch; }
  return kOk;
}

extern "C" int bq_gate_up_silu_quant_w8a8(const void* xq, const float* sx, const void* wq_gate,
                                          const void* wq_up, const float* sw_gate,
                                          const float* sw_up, int64_t M,
                                          int64_t I, int64_t K, int act_dtype, void* hq_out,
                                          float* sh_out, void* ws, size_t ws_bytes, void* stream) {
  if (!wq_gate || !wq_up || !sw_gate || !sw_up || !hq_out || !sh_out || I <= 0) return kErrBadArg;
  if (I % (kRowTile / 2) || !aligned_to(hq_out, 2) || !aligned_to(wq_up, 16)) return kErrUnsupported;
  PairSilu pair;
  memset(&pair, 0, sizeof(pair));
  pair.wq_up = wq_up;
  pair.sw_up = sw_up;
  pair.hq = static_cast<uint8_t*>(hq_out);
  pair.ld_hq = I;
  pair.sh = sh_out;
  const void* wqs[1] = {wq_gate};
  const float* sws[1] = {sw_gate};
  void* ys[1] = {nullptr};
  const int64_t Ns[1] = {2 * I};
  const int64_t ldys[1] = {0};
  // K slices as the gate weight alone would get them: every dot product is then summed in the
  // order of the separate gate and up GEMMs
  const int k_blocks = (int)((K + kBK - 1) / kBK);
  const int split = (K > 0 && K <= 0x7fffff00LL) ? split_for_weight((int)I, k_blocks) : 1;
  return run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, act_dtype, ws, ws_bytes, stream,
                     nullptr, nullptr, &pair, split);
}

extern "C" int bq_gate_up_silu_w8a8(const void* xq, const float* sx, const void* wq_gate,
                                    const void* wq_up, const float* sw_gate, const float* sw_up,
                                    int64_t M, int64_t I, int64_t K, int act_dtype, void* h_out,
                                    int64_t ld_h, float* sh_out, void* ws, size_t ws_bytes,
                                    void* stream) {
  if (!wq_gate || !wq_up || !sw_gate || !sw_up || !h_out || !sh_out || I <= 0) return kErrBadArg;
  if (I % 16 || !aligned_to(wq_up, 16)) return kErrUnsupported;
  PairSilu pair;
  memset(&pair, 0, sizeof(pair));
  pair.prefill = 1;
  pair.wq_up = wq_up;
  pair.sw_up = sw_up;
  pair.sh = sh_out;
  const void* wqs[1] = {wq_gate};
  const float* sws[1] = {sw_gate};
  void* ys[1] = {h_out};
  const int64_t Ns[1] = {I};
  const int64_t ldys[1] = {ld_h};
  return run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, act_dtype, ws, ws_bytes, stream,
                     nullptr, nullptr, &pair);
}

namespace {
int fill_push(PushParams* pp, int n_peers, void* const* dst, int64_t ld, void* const* flags,
              int64_t width, size_t align, void* const* amax_slots = nullptr) {
  if (n_peers < 1 || n_peers > kMaxPeers || !dst || !flags) return kErrBadArg;
  if (ld < width || ld % 4) return kErrUnsupported;
  memset(pp, 0, sizeof(*pp));
  pp->n = n_peers;
  pp->ld = ld;
  for (int i = 0; i < n_peers; ++i) {
    if (!dst[i] || !flags[i]) return kErrBadArg;
    if (!aligned_to(dst[i], align) || !aligned_to(flags[i], 4)) return kErrUnsupported;
    pp->dst[i] = dst[i];
    pp->flag[i] = static_cast<unsigned int*>(flags[i]);
    if (amax_slots != nullptr) {
      if (!amax_slots[i]) return kErrBadArg;
      if (!aligned_to(amax_slots[i], 4)) return kErrUnsupported;
      pp->amax_dst[i] = static_cast<unsigned int*>(amax_slots[i]);
    }
  }
  return kOk;
}
}  // namespace

extern "C" int bq_gemm_w8a8_push(const void* xq, const void* wq, const float* sx, const float* sw,
                                 int out_dtype, int64_t M, int64_t N, int64_t K, int n_peers,
                                 void* const* y_dst, int64_t ldy, void* const* flags, void* ws,
                                 size_t ws_bytes, void* stream) {
  PushParams push;
  if (int rc = fill_push(&push, n_peers, y_dst, ldy, flags, N, out_dtype == BQ_DTYPE_F32 ? 16 : 8))
    return rc;
  const void* wqs[1] = {wq};
  const float* sws[1] = {sw};
  void* ys[1] = {nullptr};
  const int64_t Ns[1] = {N};
  const int64_t ldys[1] = {0};
  return run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, out_dtype, ws, ws_bytes, stream,
                     nullptr, nullptr, nullptr, 0, &push);
}

extern "C" int bq_gate_up_silu_push_w8a8(const void* xq, const float* sx, const void* wq_gate,
                                         const void* wq_up, const float* sw_gate,
                                         const float* sw_up, int64_t M,
                                         int64_t I, int64_t K, int act_dtype, int n_peers,
                                         void* const* h_dst, int64_t ld_h, void* const* flags,
                                         void* const* amax_slots, void* ws, size_t ws_bytes,
                                         void* stream) {
  if (!wq_gate || !wq_up || !sw_gate || !sw_up || I <= 0) return kErrBadArg;
  if (I % (kRowTile / 2) || !aligned_to(wq_up, 16)) return kErrUnsupported;
  // the max |h| of the shard travels with the prefill form only (decode sizes re-quantize the
  // gathered h in the kernel that waits for it)
  if (amax_slots != nullptr && M <= g_opt_stream_max_m) amax_slots = nullptr;
  PushParams push;
  if (int rc = fill_push(&push, n_peers, h_dst, ld_h, flags, I, act_dtype == BQ_DTYPE_F32 ? 8 : 4,
                         amax_slots))
    return rc;
  PairSilu pair;
  memset(&pair, 0, sizeof(pair));
  pair.wq_up = wq_up;
  pair.sw_up = sw_up;
  const void* wqs[1] = {wq_gate};
  const float* sws[1] = {sw_gate};
  void* ys[1] = {nullptr};
  const int64_t ldys[1] = {0};
  if (M > g_opt_stream_max_m) {
    // prefill sizes: the CTA-pair kernel, SiLU*mul in its epilogue, h pieces to every rank
    pair.prefill = 1;
    const int64_t Ns[1] = {I};
    return run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, act_dtype, ws, ws_bytes, stream,
                       nullptr, nullptr, &pair, 0, &push);
  }
  const int64_t Ns[1] = {2 * I};
  const int k_blocks = (int)((K + kBK - 1) / kBK);
  const int split = (K > 0 && K <= 0x7fffff00LL) ? split_for_weight(I, k_blocks) : 1;
  return run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, act_dtype, ws, ws_bytes, stream,
                     nullptr, nullptr, &pair, split, &push);
}

extern "C" int bq_wait_flag(const void* flag, void* seen, unsigned int count, void* status_word,
                            void* stream) {
  if (!flag || !seen || !status_word || count == 0) return kErrBadArg;
  if (!aligned_to(flag, 4) || !aligned_to(seen, 4) || !aligned_to(status_word, 4)) return kErrUnsupported;
  wait_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned int*>(flag), static_cast<unsigned int*>(seen), count,
      static_cast<unsigned int*>(status_word));
  if (cudaGetLastError() != cudaSuccess) return kErrLaunch;
  return kOk;
}

// One warp, lane d for rank d: the 4-byte word at `word` (a scale, a max) into `dst_words[d]`,
// then one arrival on that rank's counter, the word first (system-scope release on the
// counter).  One lane per rank so that the round trips to the ranks run side by side (a single
// thread walking four ranks took 12 us).
__global__ void word_push_kernel(const unsigned int* word, int n, PushParams dst) {
  const int d = threadIdx.x;
  if (d >= n) return;
  const unsigned int v = __ldcg(word);
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst.amax_dst[d]), "r"(v) : "memory");
  __threadfence_system();
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(dst.flag[d]) : "memory");
}

extern "C" int bq_word_push(const void* word, int n_peers, void* const* dst_words, void* const* flags,
                            void* stream) {
  if (!word || !dst_words || !flags || n_peers < 1 || n_peers > kMaxPeers) return kErrBadArg;
  if (!aligned_to(word, 4)) return kErrUnsupported;
  PushParams pp;
  memset(&pp, 0, sizeof(pp));
  for (int i = 0; i < n_peers; ++i) {
    if (!dst_words[i] || !flags[i]) return kErrBadArg;
    if (!aligned_to(dst_words[i], 4) || !aligned_to(flags[i], 4)) return kErrUnsupported;
    pp.amax_dst[i] = static_cast<unsigned int*>(dst_words[i]);
    pp.flag[i] = static_cast<unsigned int*>(flags[i]);
  }
  word_push_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned int*>(word),
                                                                   n_peers, pp);
  if (cudaGetLastError() != cudaSuccess) return kErrLaunch;
  return kOk;
}

extern "C" int bq_wait_flag_scale(const void* flag, void* seen, unsigned int count, void* status_word,
                                  const void* amax_slots, int n_slots, int slots_hold_scales,
                                  float* scale_out, void* stream) {
  if (!flag || !seen || !status_word || !amax_slots || !scale_out || count == 0) return kErrBadArg;
  if (n_slots < 1 || n_slots > kMaxPeers) return kErrBadArg;
  if (!aligned_to(flag, 4) || !aligned_to(seen, 4) || !aligned_to(status_word, 4) ||
      !aligned_to(amax_slots, 4) || !aligned_to(scale_out, 4))
    return kErrUnsupported;
  wait_flag_scale_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned int*>(flag), static_cast<unsigned int*>(seen), count,
      static_cast<unsigned int*>(status_word), static_cast<const unsigned int*>(amax_slots), n_slots,
      slots_hold_scales, scale_out);
  if (cudaGetLastError() != cudaSuccess) return kErrLaunch;
  return kOk;
}

extern "C" int bq_gemm_w8a8_residual(const void* xq, const void* wq, const float* sx, const float* sw,
                                     const void* residual, int64_t ld_res, void* y, int out_dtype,
                                     int64_t M, int64_t N, int64_t K, int64_t ldy, void* ws,
                                     size_t ws_bytes, void* stream) {
  if (residual == nullptr) return kErrBadArg;
  const void* wqs[1] = {wq};
  const float* sws[1] = {sw};
  void* ys[1] = {y};
  const int64_t Ns[1] = {N};
  const int64_t ldys[1] = {ldy};
  const void* rs[1] = {residual};
  const int64_t ldrs[1] = {ld_res};
  return run_grouped(xq, sx, M, K, 1, wqs, sws, ys, Ns, ldys, out_dtype, ws, ws_bytes, stream,
                     rs, ldrs);
}


extern "C" int bq_last_gemm_launch(int64_t out[6]) {
  if (!out) return kErrBadArg;
  for (int i = 0; i < 6; ++i) out[i] = g_last_launch[i];
  return kOk;
}
