/*
 * braid_b200 — C ABI of the B200 (sm_100a) FP8 W8A8 projection path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void* so the header needs no CUDA include) and returns an int
 * status (BQ_OK == 0).  Nothing here allocates device memory unless it says
 * so: outputs and scratch are owned by the caller.  All launches go to the
 * stream given; none of the calls synchronises the device, so they are legal
 * inside a CUDA stream capture.  Scales are always read and written ON THE
 * DEVICE through pointers — never passed by value — which is what keeps a
 * captured graph valid when the activation changes between replays.
 *
 * Each declaration cites the interface of the reference engine
 * (plind-junior/braid) that it stands in for, as path:line inside that project.
 */
#ifndef BRAID_B200_H_
#define BRAID_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define BQ_OK 0
#define BQ_ERR_BAD_ARG 1        /* null pointer, n <= 0, unknown dtype code           */
#define BQ_ERR_UNSUPPORTED 2    /* shape/alignment the kernels do not take            */
#define BQ_ERR_LAUNCH 3         /* the CUDA runtime refused the launch                */
#define BQ_ERR_WORKSPACE 4      /* scratch pointer null, misaligned or too small      */
#define BQ_ERR_DEVICE_WAIT 5    /* a bounded device-side wait ran out (see bq_read_device_status) */
#define BQ_ERR_NO_DRIVER 6      /* cuTensorMapEncodeTiled could not be resolved       */
#define BQ_ERR_TOO_LARGE 7      /* request exceeds a fixed capacity                   */

/* ---- element type codes for activations / outputs ----------------------- */
#define BQ_DTYPE_F32 0
#define BQ_DTYPE_BF16 1
#define BQ_DTYPE_F16 2

/* Largest number of weights one grouped GEMM launch takes. */
#define BQ_MAX_SEGMENTS 8

/* Library version (major*100 + minor). */
int bq_version(void);

/*
 * Synchronises the current device and returns, through *status_out, the sticky status of the
 * launches that take no scratch from the caller (bq_cast_act): 0, or BQ_ERR_DEVICE_WAIT when a
 * bounded wait of such a launch ran out since the last call; clears it.  Never during capture.
 */
int bq_scratchless_status(int* status_out);

/* Human-readable text for a status code; never NULL. */
const char* bq_status_string(int status);

/*
 * Bytes of zero-initialised scratch the quantizer entry points need.  The
 * scratch holds the grid-level amax word, the two barrier counters and a
 * sticky device status word.  It must be 16-byte aligned and zeroed ONCE by
 * the caller (cudaMemset); the kernels return it to zero themselves, so one
 * buffer serves any number of calls that are ordered on a stream.  Calls that
 * may overlap on the GPU (different streams) need separate buffers.
 */
size_t bq_quant_workspace_bytes(void);

/*
 * Per-tensor dynamic FP8 (e4m3fn) quantization of a contiguous activation:
 *     scale = max(amax(|x|) * (1/448), 1e-12)   (fp32; NaN propagates)
 *     q     = e4m3_rne(clamp(x / scale, -448, 448))
 * bit-identical to the reference's torch spelling run on a CUDA device.
 * One launch: 128-bit loads, warp-shuffle + grid-level amax, single-pass cast.
 *
 * Replaces: braid/model/quant.py:209-229 (`quantize_act`), whose fused arm is
 * `quantize_act_cuda` in braid/kernels/csrc/quant_act.cu:140-176 bound at
 * braid/kernels/csrc/bindings.cpp:33.
 *
 *   x         device, `n` elements of `dtype` (BQ_DTYPE_*), contiguous
 *   q_out     device, n bytes (e4m3fn codes)
 *   scale_out device, one float (the dequant scale, shape [1,1] upstream)
 *   ws        scratch, see bq_quant_workspace_bytes()
 */
int bq_quantize_act(const void* x, int dtype, int64_t n, void* q_out, float* scale_out,
                    void* ws, size_t ws_bytes, void* stream);

/*
 * The same quantizer for callers that cannot give the library a scratch buffer.
 * It has no counterpart in the reference; it exists for hosts that may not
 * allocate device memory at the point of the call: runtimes that pre-carve the
 * whole GPU into their own arena and forbid cudaMalloc afterwards, code that
 * runs while the host's allocator is locked, control loops with a no-allocation
 * rule, and FFI shims for which creating and zeroing a device buffer is the
 * hard part.  The barrier words live in a fixed array of
 * BQ_STATIC_SCRATCH_BYTES inside the library image (held by every GPU that
 * loads the library, until the process exits).  The call allocates nothing and
 * calls no allocating routine; inputs and outputs are still the caller's.
 *
 *  - Limit: n <= BQ_STATIC_MAX_ELEMENTS, otherwise BQ_ERR_TOO_LARGE and nothing
 *    is launched.  Alignment rules as for bq_quantize_act.
 *  - The first call on each device looks up the array's device address (once,
 *    with that device current).  Make that first call before any stream capture,
 *    and from one thread: the lookup is cached without a lock, so two threads
 *    must not make a device's first call at the same time.
 *  - All calls on a device share the one array: calls that may overlap on the
 *    GPU (different streams without ordering) race on it and give wrong scales.
 *    Each call clears the words that must start at zero, in stream order.
 *  - A bounded wait that runs out is recorded inside the array only; use
 *    bq_quantize_act with your own scratch if you need to read that status.
 */
#define BQ_STATIC_SCRATCH_BYTES 256
#define BQ_STATIC_MAX_ELEMENTS (INT64_C(1) << 28)
int bq_quantize_act_static(const void* x, int dtype, int64_t n, void* q_out, float* scale_out,
                           void* stream);

/*
 * SiLU(gate)*up fused into the quantizer: h = bf16(bf16(silu(gate)) * up) is
 * formed in registers (double rounding exactly as the two torch kernels do),
 * its amax reduced grid-wide, and only the e4m3 codes of h and the scale are
 * written — h itself never touches memory.
 *
 * Replaces: braid/model/mlp.py:48-49 (`h = F.silu(gate) * up` followed by the
 * `quantize_act` inside `linear(h, down_proj)`).
 *
 *   gate, up   device, [rows, cols] of `dtype` with row strides ld_gate / ld_up
 *              (elements); cols must be a multiple of 8, rows 16-byte aligned
 *   q_out      device, rows*cols bytes, contiguous [rows, cols]
 */
int bq_silu_mul_quant(const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                      int64_t ld_gate, int64_t ld_up, void* q_out, float* scale_out,
                      void* ws, size_t ws_bytes, void* stream);

/*
 * The two halves of bq_silu_mul_quant, for a column-parallel MLP whose ranks each
 * hold a column shard of gate and up: bq_silu_mul_scale writes only the scale of
 * the shard (pass 1 and the grid-wide exchange), the ranks combine their scales
 * with a MAX all-reduce (the scale is a monotone function of the amax and max is
 * exact, so the result is the scale of the whole intermediate), and
 * bq_silu_mul_cast writes the shard's codes under that scale.  The codes equal,
 * byte for byte, those a quantizer of the gathered intermediate would write.
 *
 * Replaces: the `quantize_act` inside `linear(h, down_proj)` of
 * braid/model/mlp.py:48-49 when h is sharded over GPUs (the reference itself is
 * single-GPU).  Arguments as bq_silu_mul_quant; `scale` is a device float that
 * bq_silu_mul_cast only reads.  bq_silu_mul_cast needs no scratch.
 */
int bq_silu_mul_scale(const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                      int64_t ld_gate, int64_t ld_up, float* scale_out, void* ws, size_t ws_bytes,
                      void* stream);
int bq_silu_mul_cast(const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                     int64_t ld_gate, int64_t ld_up, const float* scale, void* q_out, void* stream);

/*
 * o * sigmoid(gate) fused into the quantizer, h = bf16(o * bf16(sigmoid(gate))).
 * `gate` may be the strided per-head view the attention layer produces: element
 * (r, c) lives at gate[r*ld_gate + (c / chunk)*chunk_stride + (c % chunk)], so
 * the [q | gate] interleave of the q projection is read in place, no copy.
 *
 * Replaces: braid/model/attention.py:215-216 (`o = o * torch.sigmoid(gate)`
 * followed by the `quantize_act` inside `linear(o, o_proj)`); the strided gate
 * is the `chunk(2, dim=-1)` view of braid/model/attention.py:177-178.
 *
 *   o            device, [rows, cols], row stride ld_o (elements)
 *   chunk        head_dim of the gate view (multiple of 8); pass cols for a dense gate
 *   chunk_stride distance between consecutive heads of the gate (elements)
 */
int bq_sigmoid_gate_quant(const void* o, const void* gate, int dtype, int64_t rows, int64_t cols,
                          int64_t ld_o, int64_t ld_gate, int64_t chunk, int64_t chunk_stride,
                          void* q_out, float* scale_out, void* ws, size_t ws_bytes, void* stream);

/*
 * The two prologues alone, unquantized, with the rounding the quantizer modes apply:
 * bq_silu_mul writes h = T(T(silu(gate)) * up), bq_sigmoid_mul writes T(o * T(sigmoid(gate))),
 * contiguous [rows, cols] of the input type, 16-byte aligned.  Arguments as in
 * bq_silu_mul_quant / bq_sigmoid_gate_quant; no scratch.
 *
 * Replaces: the elementwise torch kernels of braid/model/mlp.py:48 (`F.silu(gate) * up`) and
 * braid/model/attention.py:215 (`o * torch.sigmoid(gate)`) where the product is wanted dense
 * (an unquantized down / o projection), bit for bit.
 */
int bq_silu_mul(const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                int64_t ld_gate, int64_t ld_up, void* h_out, void* stream);
int bq_sigmoid_mul(const void* o, const void* gate, int dtype, int64_t rows, int64_t cols,
                   int64_t ld_o, int64_t ld_gate, int64_t chunk, int64_t chunk_stride, void* out,
                   void* stream);

/*
 * The same two products together with the quantization scale of the result (one atomicMax and
 * one count per CTA on `ws`, 16 bytes as for bq_quantize_act; the CTA that counts last writes
 * *scale_out; no grid-wide wait): the first of two launches that replace bq_silu_mul_quant /
 * bq_sigmoid_gate_quant at prefill sizes, where their two passes would evaluate the prologue
 * twice -- bq_cast_act(out, scale_out) is the second.  Same bits as the one-launch forms.
 */
int bq_silu_mul_dense_scale(const void* gate, const void* up, int dtype, int64_t rows, int64_t cols,
                            int64_t ld_gate, int64_t ld_up, void* h_out, float* scale_out, void* ws,
                            size_t ws_bytes, void* stream);
int bq_sigmoid_mul_dense_scale(const void* o, const void* gate, int dtype, int64_t rows, int64_t cols,
                               int64_t ld_o, int64_t ld_gate, int64_t chunk, int64_t chunk_stride,
                               void* out, float* scale_out, void* ws, size_t ws_bytes, void* stream);

/*
 * RMSNorm fused into the quantizer: h = T(gamma * (rstd * x)), rstd = rsqrt(mean(x^2) + eps),
 * computed in fp32 from the fp32-widened input with ONE rounding to the activation type T,
 * then amax / scale / e4m3 codes of h as bq_quantize_act produces them.  The sum of squares
 * follows the reduction order of the kernel torch runs for `F.rms_norm` on a CUDA device, so h,
 * the scale and the codes are bit-identical to the reference's two steps.
 *
 * Replaces: braid/model/norm.py:31-45 (`rms_norm`) at braid/model/layer.py:49 and :59,
 * together with the `quantize_act` of the consumer (`project` at braid/model/gdn.py:254 and
 * braid/model/attention.py:173; braid/model/mlp.py:45).
 *
 *   x        device, [rows, cols] of `dtype`, row stride ld_x (elements); cols % 4 == 0,
 *            cols <= 8192; rows are limited to what is co-resident on the device
 *            (one 128-thread CTA per row, BQ_ERR_TOO_LARGE beyond that)
 *   gamma    device, cols floats: the EFFECTIVE gamma (1 + W already folded, loader.py:196-199)
 *   h_out    device or NULL: the normalised activation in `dtype`, row stride ld_h — needed
 *            only when a consumer reads it unquantized (the bf16 a/b gates of the GDN layer)
 *   q_out    device, rows*cols bytes, contiguous
 */
int bq_rmsnorm_quant(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                     const float* gamma, float eps, void* h_out, int64_t ld_h, void* q_out,
                     float* scale_out, void* ws, size_t ws_bytes, void* stream);

/*
 * The same norm for more rows than one co-resident grid has CTAs (prefill): every CTA loops
 * over rows, writes the normalised activation h_out (required here) and the grid leaves the
 * quantization scale of h in *scale_out without anybody waiting for anybody (one atomicMax and
 * one count per CTA; the CTA that counts last publishes).  bq_cast_act(h_out, scale_out) in
 * stream order then gives the codes: the two calls equal bq_rmsnorm_quant bit for bit.
 */
int bq_rmsnorm_scale(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                     const float* gamma, float eps, void* h_out, int64_t ld_h, float* scale_out,
                     void* ws, size_t ws_bytes, void* stream);

/*
 * Gated RMSNorm of the GDN readout fused into the quantizer of out_proj's input:
 *   core = T(y);  xn = T(rstd * core) per 128-wide head;  h = T((gamma * xn) * silu(float(z)))
 * with the fp32 arithmetic and the three roundings of the reference's spelling, then amax /
 * scale / codes of h.  `y` may be the fp32 scan output (rounded to T first, as the reference
 * does) or already of type T.
 *
 * Replaces: braid/model/gdn.py:383-387 (`_readout`: `y.to(dtype)`, `rms_norm_gated`
 * braid/model/norm.py:48-71, and the `quantize_act` inside `linear(core, out_proj)`).
 *
 *   y        device, [rows, heads*head_dim] of y_dtype (BQ_DTYPE_F32 or `dtype`), stride ld_y
 *   z        device, [rows, heads*head_dim] of `dtype`, stride ld_z
 *   gamma    device, head_dim floats (stored directly: no 1 + W for the gated norm)
 *   head_dim must be 128; heads <= 64
 *   q_out    device, rows*heads*head_dim bytes, contiguous [rows, heads*head_dim]
 */
int bq_gated_rmsnorm_quant(const void* y, int y_dtype, int64_t ld_y, const void* z, int dtype,
                           int64_t ld_z, const float* gamma, float eps, int64_t rows, int64_t heads,
                           int64_t head_dim, void* q_out, float* scale_out, void* ws,
                           size_t ws_bytes, void* stream);

/*
 * The gated norm for more rows than one co-resident grid has CTAs (prefill): writes the gated,
 * normalised activation h_out [rows, heads*head_dim] and leaves its quantization scale in
 * *scale_out with no grid-wide wait; bq_cast_act(h_out, scale_out) then gives the codes.  The
 * two calls equal bq_gated_rmsnorm_quant bit for bit.  Any number of heads.
 */
int bq_gated_rmsnorm_scale(const void* y, int y_dtype, int64_t ld_y, const void* z, int dtype,
                           int64_t ld_z, const float* gamma, float eps, int64_t rows, int64_t heads,
                           int64_t head_dim, void* h_out, int64_t ld_h, float* scale_out, void* ws,
                           size_t ws_bytes, void* stream);

/*
 * Bytes of scratch the GEMM entry points need: 16 (the sticky status word and
 * the counters of the paired / push epilogues).  Split-K partial sums travel
 * through distributed shared memory and never reach global memory.  Zero the
 * scratch once (cudaMemset); the kernels leave it zeroed where it matters.
 * Launches that share a scratch slot must be ordered on one stream.
 */
size_t bq_gemm_workspace_bytes(int64_t M, int64_t N_total, int64_t K);

/*
 * Per-tensor W8A8 GEMM:  Y[M,N] = (Xq[M,K] . Wq[N,K]^T) * sx * sw, fp32
 * accumulation in tensor memory, scales applied in the epilogue, output cast
 * to `out_dtype`.  Both operands are K-major, exactly the layout the reference
 * keeps (`FP8Weight.data` is [N,K] row-major).  M <= 256 takes the
 * weight-streaming kernel (weight rows on the MMA M side, batch on the N side,
 * deterministic split-K over a thread-block cluster); larger M takes the
 * persistent compute-bound kernel.
 *
 * Replaces: braid/model/quant.py:232-241 (`fp8_matmul`), i.e. the call
 * `torch._scaled_mm(xq, w.data.t(), scale_a=sx, scale_b=w.scale, out_dtype=...)`.
 *
 *   xq   device, [M,K] e4m3fn codes, contiguous, 16-byte aligned, K % 16 == 0
 *   wq   device, [N,K] e4m3fn codes, contiguous, 16-byte aligned, N % 16 == 0
 *   sx   device, one float (activation dequant scale)
 *   sw   device, one float (weight dequant scale)
 *   y    device, [M,N] of out_dtype, row stride ldy elements (ldy >= N)
 */
int bq_gemm_w8a8(const void* xq, const void* wq, const float* sx, const float* sw, void* y,
                 int out_dtype, int64_t M, int64_t N, int64_t K, int64_t ldy,
                 void* ws, size_t ws_bytes, void* stream);

/*
 * bq_gemm_w8a8 with the residual add of the decoder layer in the epilogue:
 *   y = T(float(T(acc * sx * sw)) + float(residual))
 * i.e. the GEMM's own rounding to the output type T followed by the add's rounding, which is
 * what the reference's separate kernels produce.  Decode regime only (M <= 256): larger M
 * returns BQ_ERR_UNSUPPORTED and the caller adds separately.
 *
 * Replaces: `x = x + h` after the mixer's output projection and `x + self.mlp(h)`
 * (braid/model/layer.py:57,60), fused into `linear(core, out_proj)` (braid/model/gdn.py:387),
 * `linear(o, o_proj)` (braid/model/attention.py:216) and `linear(h, down_proj)`
 * (braid/model/mlp.py:49).
 *
 *   residual  device, [M,N] of out_dtype, row stride ld_res elements (ld_res >= N, % 4 == 0);
 *             may not overlap y
 */
int bq_gemm_w8a8_residual(const void* xq, const void* wq, const float* sx, const float* sw,
                          const void* residual, int64_t ld_res, void* y, int out_dtype,
                          int64_t M, int64_t N, int64_t K, int64_t ldy,
                          void* ws, size_t ws_bytes, void* stream);

/*
 * lm_head with the greedy pick in its epilogue (decode regime, M <= 256):
 *   logits = (Xq . Wq^T) * sx * sw rounded to out_dtype, idx_out[m] = argmax_n logits[m, n]
 * with torch's conventions (lowest index among equal maxima, NaN beats everything).  Every CTA
 * reduces its 128 vocabulary rows per batch row and writes one (value, index) pair into
 * `partial`; a second small kernel reduces the pairs.  The logits themselves are written only
 * when `logits_or_null` is given ([M, N], row pitch ldy); without them the 2*M*N output bytes
 * never reach memory.  The index equals `logits.argmax(-1)` of bq_gemm_w8a8's output exactly.
 *
 * Replaces: `linear(h, self.lm_head)[:, 0]` of braid/model/engine.py:349 followed by
 * `logits.argmax(-1)` of braid/serve/scheduler.py:346 (the greedy rows of `_sample_rows`).
 *
 *   idx_out   device, M int64
 *   partial   device scratch, bq_lm_head_argmax_workspace_bytes(M, N) bytes, 8-byte aligned;
 *             need not be zeroed; calls that overlap on the GPU must not share it
 *   ws        16 bytes as for bq_gemm_w8a8
 */
size_t bq_lm_head_argmax_workspace_bytes(int64_t M, int64_t N);
int bq_lm_head_argmax(const void* xq, const void* wq, const float* sx, const float* sw,
                      int out_dtype, int64_t M, int64_t N, int64_t K, void* logits_or_null,
                      int64_t ldy, int64_t* idx_out, void* partial, size_t partial_bytes,
                      void* ws, size_t ws_bytes, void* stream);

/*
 * The first half of the quantized MLP at prefill sizes (M > 256), on the CTA-pair kernel: every
 * 256-column MMA tile holds 128 gate rows and the 128 up rows of the same output columns (one
 * CTA of the pair loads each, from the two weights where they lie), and the epilogue writes
 *   h = T(T(silu(T(gate))) * T(up))      [M, I] of the activation type, row pitch ld_h
 * instead of gate and up, together with the scale of h (max |h| over the launch, taken with
 * one atomicMax per CTA; the CTA that finishes last publishes max(amax/448, 1e-12) to sh_out).
 * bq_cast_act then turns h into codes under that scale.  h, scale and codes are bit-identical
 * to bq_gemm_w8a8_grouped(gate, up) + bq_silu_mul_quant, with a third of their memory traffic
 * and the SiLU arithmetic done once, inside the GEMM's otherwise idle epilogue warps.
 *
 * Replaces: braid/model/mlp.py:46-48 and the scale half of the `quantize_act` of :49.
 *   ws   16 bytes, zero before the first call, self-resetting
 * Returns BQ_ERR_UNSUPPORTED for M <= 256 (use bq_gate_up_silu_quant_w8a8).
 */
int bq_gate_up_silu_w8a8(const void* xq, const float* sx, const void* wq_gate, const void* wq_up,
                         const float* sw_gate, const float* sw_up, int64_t M, int64_t I, int64_t K,
                         int act_dtype, void* h_out, int64_t ld_h, float* sh_out, void* ws,
                         size_t ws_bytes, void* stream);

/*
 * e4m3 codes of x under a scale decided elsewhere: q = e4m3(clamp(x / *scale, +-448)), the cast
 * half of bq_quantize_act (braid/model/quant.py:229).  No scratch, no grid-wide wait.
 */
int bq_cast_act(const void* x, int dtype, int64_t n, const float* scale, void* q_out, void* stream);

/*
 * The first half of the quantized MLP in ONE launch (decode regime, M <= 256):
 *   gate = Xq.Wg^T, up = Xq.Wu^T (each rounded to the activation type as bq_gemm_w8a8 would),
 *   h = T(T(silu(gate)) * up), then amax / scale / e4m3 codes of h
 * -- neither gate, up nor h is written; only the codes and the scale are.  Bit-identical to
 * bq_gemm_w8a8_grouped(gate, up) followed by bq_silu_mul_quant.
 *
 * The kernel needs gate and up of the same columns in one MMA tile: every 128-row tile is put
 * together in shared memory from 64 rows of the gate weight and the 64 rows of the up weight
 * with the same indices (two TMA boxes per pipeline stage).  The two weights stay where and
 * as the reference keeps them -- two [I, K] tensors with two scales; nothing is repacked.
 * I must be a multiple of 64.
 *
 * Replaces: braid/model/mlp.py:46-48 (`gate = fp8_matmul(..)`, `up = fp8_matmul(..)`,
 * `h = F.silu(gate) * up`) and the `quantize_act` inside `linear(h, down_proj)` (:49).
 *
 *   wq_gate, wq_up  device, [I, K] e4m3 codes each, contiguous, 16-byte aligned
 *   hq_out   device, M*I bytes, contiguous [M, I];  sh_out  device, one float
 *   ws       16 bytes, zero before the first call, self-resetting (as for bq_quantize_act)
 * Returns BQ_ERR_UNSUPPORTED when the launch cannot be resident at once or M > 256.
 */
int bq_gate_up_silu_quant_w8a8(const void* xq, const float* sx, const void* wq_gate,
                               const void* wq_up, const float* sw_gate, const float* sw_up,
                               int64_t M, int64_t I,
                               int64_t K, int act_dtype, void* hq_out, float* sh_out,
                               void* ws, size_t ws_bytes, void* stream);

/*
 * Column-parallel forms for one NVLink/NVSwitch node (no counterpart in the reference, which is
 * single-GPU; the benchmark configuration defines an N-split MLP with gathered outputs).  The
 * GEMM of a rank's weight shard stores its output tile straight into the gathered buffer of
 * EVERY rank -- `dst[i]` are device pointers valid in this process (this rank's own buffer and
 * the peers' buffers mapped through CUDA IPC), already offset to this rank's first column --
 * and the last CTA of the launch to finish then adds 1 to the arrival counter `flags[i]` of each
 * rank with a system-scope release (the CTAs count themselves on the first word of `ws`, which
 * must be zero before the first call and is returned to zero).  A rank's buffer is complete when
 * its counter has advanced by the number of ranks; bq_wait_flag waits for exactly that (bounded)
 * in stream order.  Plain stores and counters only: no collective call, no multicast.  Up to
 * 8 destinations; M <= 256 runs the weight-streaming kernel, larger M the CTA-pair kernel
 * (destinations and their row pitch then 16-byte aligned).
 */

/*
 * Lets kernels launched on the CURRENT device dereference memory of `peer_device` that this
 * process has mapped (cudaDeviceEnablePeerAccess; already-enabled is success).  A peer buffer
 * opened through CUDA IPC is mapped for the peer device's context: without this call a kernel
 * on the current device faults on it.  BQ_ERR_UNSUPPORTED when the two devices have no peer path.
 */
int bq_enable_peer_access(int peer_device);

/*
 * Set-up calls of the column-parallel form (never on the hot path).  bq_peer_alloc makes a
 * zeroed device buffer on the current device and a 64-byte handle other PROCESSES of the node
 * can open; bq_peer_open maps such a buffer for the CURRENT device of the calling process (peer
 * access included) and verifies the mapping with a copy through the runtime, so a bad mapping is
 * an error code, never a kernel fault.  A handle may be opened once per process and device.
 */
#define BQ_PEER_HANDLE_BYTES 64
int bq_peer_alloc(size_t bytes, void** ptr_out, void* handle_out /* BQ_PEER_HANDLE_BYTES */);
int bq_peer_free(void* ptr);
int bq_peer_open(const void* handle /* BQ_PEER_HANDLE_BYTES */, void** ptr_out);
int bq_peer_close(void* ptr);

/* y shard = Xq . Wq^T * sx * sw pushed to every rank; rows = N of this rank's shard. */
int bq_gemm_w8a8_push(const void* xq, const void* wq, const float* sx, const float* sw,
                      int out_dtype, int64_t M, int64_t N, int64_t K, int n_peers,
                      void* const* y_dst, int64_t ldy, void* const* flags,
                      void* ws, size_t ws_bytes, void* stream);

/*
 * h shard = T(T(silu(gate)) * up) of this rank's gate and up shards (two [I, K] tensors as for
 * bq_gate_up_silu_quant_w8a8, I = columns of this rank) pushed to every rank.  The amax of h
 * spans all ranks' shards: at decode sizes quantization is left to bq_quantize_act_after on the
 * gathered buffer; at prefill sizes (M > 256) the launch also hands this rank's max |h| (the
 * bits of the float) to every rank -- `amax_slots[i]` = the word for THIS rank on rank i, or
 * NULL for none -- written before the arrivals, so that bq_wait_flag_scale + bq_cast_act
 * replace the two-pass quantizer of the gathered tensor.  `ws`: 16 bytes as for the other GEMMs
 * (the first two words are used and returned to zero).
 */
int bq_gate_up_silu_push_w8a8(const void* xq, const float* sx, const void* wq_gate,
                              const void* wq_up, const float* sw_gate, const float* sw_up,
                              int64_t M, int64_t I,
                              int64_t K, int act_dtype, int n_peers, void* const* h_dst,
                              int64_t ld_h, void* const* flags, void* const* amax_slots,
                              void* ws, size_t ws_bytes, void* stream);

/*
 * One-thread kernel: waits until *flag has advanced by `count` beyond *seen (bounded; a wait
 * that runs out sets *status_word to BQ_ERR_DEVICE_WAIT and returns), then adds `count` to
 * *seen.  `flag` is this rank's arrival counter, `seen` a device word owned by this rank.
 */
int bq_wait_flag(const void* flag, void* seen, unsigned int count, void* status_word, void* stream);

/*
 * bq_wait_flag, then *scale_out = the quantization scale of the gathered h from the `n_slots`
 * words the ranks wrote on this rank (`amax_slots`): either max |h| of each rank's shard
 * (bq_gate_up_silu_push_w8a8; slots_hold_scales = 0: the maximum is turned into a scale as
 * bq_quantize_act does) or each shard's scale (bq_word_push of the scale bq_gate_up_silu_w8a8
 * returned; slots_hold_scales = 1: the maximum IS the scale, the scale being a monotone function
 * of the amax).  The maximum over the shards is the maximum over the tensor: the scale of the
 * unsharded quantizer, bit for bit.
 */
int bq_wait_flag_scale(const void* flag, void* seen, unsigned int count, void* status_word,
                       const void* amax_slots, int n_slots, int slots_hold_scales, float* scale_out,
                       void* stream);

/*
 * One-warp kernel (a lane per rank): the 4-byte word at `word` into `dst_words[i]` on every rank
 * (peer-mapped pointers, this rank's own included), then one arrival on that rank's counter
 * `flags[i]`.
 */
int bq_word_push(const void* word, int n_peers, void* const* dst_words, void* const* flags,
                 void* stream);

/*
 * One rank's [rows, cols] block to every rank of the node, elementwise, by plain stores through
 * peer-mapped pointers (`dst[i]` already offset to this rank's first column in rank i's
 * gathered buffer, row pitch ld_dst), then one arrival per rank (`flags[i]`), counted as in the
 * GEMM push forms on the first word of `ws` (16 bytes, zero between launches).
 * bq_cast_act_push stores the e4m3 codes of the block under `*scale` (bq_cast_act's
 * arithmetic): a warp writes 256 contiguous bytes of a row per destination, which NVLink moves
 * at its copy rate -- the way a column-parallel MLP exchanges h as codes once the shards'
 * scales have been combined (bq_word_push + bq_wait_flag_scale).  bq_rows_push stores the
 * block unchanged.  cols a multiple of 8; x and its pitch 16-byte aligned.
 */
int bq_cast_act_push(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x,
                     const float* scale, int n_peers, void* const* q_dst, int64_t ld_q,
                     void* const* flags, void* ws, size_t ws_bytes, void* stream);
int bq_rows_push(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ld_x, int n_peers,
                 void* const* dst, int64_t ld_dst, void* const* flags, void* ws, size_t ws_bytes,
                 void* stream);

/*
 * bq_quantize_act on a gathered buffer, with the wait of bq_wait_flag folded into the kernel:
 * every CTA waits (bounded; a wait that runs out raises the status word of `ws`) until *flag has
 * advanced by `count` beyond *seen before it loads, and *seen is advanced once all have.  One
 * launch fewer per exchange and the dependent-launch chain stays intact.
 */
int bq_quantize_act_after(const void* x, int dtype, int64_t n, void* q_out, float* scale_out,
                          const void* flag, void* seen, unsigned int count,
                          void* ws, size_t ws_bytes, void* stream);

/*
 * Several projections of ONE quantized activation in a single launch: segment
 * i computes Y_i[M,N_i] = (Xq . Wq_i^T) * sx * sw_i with its own weight scale,
 * so results are bit-identical to n_seg separate bq_gemm_w8a8 calls.  The
 * pointer arrays are HOST arrays of device pointers.
 *
 * Replaces: the per-weight loop of braid/model/quant.py:260-286 (`project`)
 * and the gate/up pair of braid/model/mlp.py:44-47.
 */
int bq_gemm_w8a8_grouped(const void* xq, const float* sx, int64_t M, int64_t K, int n_seg,
                         const void* const* wq, const float* const* sw, void* const* y,
                         const int64_t* N, const int64_t* ldy, int out_dtype,
                         void* ws, size_t ws_bytes, void* stream);

/*
 * `project` with a mixed set of weights in ONE launch (decode regime, M <= 256): segments
 * with kind[i] == 0 are e4m3 weights multiplied with the quantized activation exactly as in
 * bq_gemm_w8a8_grouped; segments with kind[i] != 0 are weights the reference leaves
 * unquantized (bf16 / fp16, [N_i, K] row-major) and are multiplied with the UNQUANTIZED
 * activation `x_dense` [M, K] of the same 16-bit type on the tensor cores (kind::f16, fp32
 * accumulation, no scales; sw[i] is ignored and may be null).  The FP8 segments are
 * bit-identical to separate calls; a 16-bit segment is `F.linear(x, w)` up to the summation
 * order of a tensor-core GEMM (it is not bit-identical to the cuBLAS kernel torch would pick).
 *
 * Replaces: braid/model/quant.py:260-286 (`project`) including its `F.linear(x, w)` arm for
 * weights left in bf16 -- the GDN gates in_proj_a / in_proj_b of braid/model/gdn.py:254-255.
 *
 *   x_dense      device, [M, K] of dense_dtype (BQ_DTYPE_BF16 or BQ_DTYPE_F16), contiguous,
 *                16-byte aligned; out_dtype must equal dense_dtype when a 16-bit segment exists
 *   w[i]         device, e4m3 codes (kind 0) or 16-bit values (kind != 0), contiguous [N_i, K]
 * Returns BQ_ERR_UNSUPPORTED for M > 256: call bq_gemm_w8a8_grouped and a dense GEMM instead.
 */
int bq_project_mixed(const void* xq, const float* sx, const void* x_dense, int dense_dtype, int64_t M,
                     int64_t K, int n_seg, const void* const* w, const float* const* sw,
                     const int* kind, void* const* y, const int64_t* N, const int64_t* ldy,
                     int out_dtype, void* ws, size_t ws_bytes, void* stream);

/*
 * Copies the sticky device status word of a scratch buffer to the host
 * (synchronises `stream`; never call during capture).  0 means every bounded
 * device wait so far completed; otherwise BQ_ERR_DEVICE_WAIT.  The word is
 * cleared by the call.
 */
int bq_read_device_status(void* ws, void* stream, int* status_out);

/*
 * Tuning hooks used by the benchmark and tests; not needed for normal use.
 * bq_set_option("decode_split_k", v)    0 = heuristic, else force the K slices per tile
 * bq_set_option("decode_stages", v)     0 = heuristic, else cap the pipeline depth
 * bq_set_option("decode_b_stages", v)   activation ring depth: 0 = heuristic, -1 = as the weight ring
 * bq_set_option("decode_cta_target", v) CTAs a small weight is sliced to reach (default 160)
 * bq_set_option("decode_smem_cap", v)   0 = none, else cap pipeline bytes per CTA
 * bq_set_option("stream_max_m", v)      largest M the weight-streaming kernel takes (<= 256)
 * bq_set_option("gemm_pdl" | "quant_pdl", 0/1)  programmatic dependent launch
 * bq_set_option("quant_block" | "quant_held", v) quantizer launch shape overrides
 * bq_set_option("quant_ring", 0/1)      plain quantizer at prefill sizes through the shared-memory ring (default 1)
 * bq_set_option("push_tma", 0/1)        prefill push epilogue by bulk tensor stores (default 1) or 16-byte plain stores
 * bq_set_option("pair_narrow", -1/0/1) prefill kernel: 128-column tiles for a lone narrow weight (-1 = when 256-column
 *                                       tiles would leave half of the CTA pairs idle; same results either way)
 * Returns BQ_ERR_BAD_ARG for an unknown key.
 */
int bq_set_option(const char* key, int64_t value);

/*
 * Describes the launch the last GEMM call on this thread chose:
 * out[0]=kernel (0 weight-streaming cluster kernel, 2 CTA-pair tile kernel) out[1]=grid out[2]=cluster/split
 * out[3]=stages out[4]=dynamic smem bytes out[5]=batch tile (MMA N)
 */
int bq_last_gemm_launch(int64_t out[6]);

#ifdef __cplusplus
}
#endif
#endif /* BRAID_B200_H_ */
