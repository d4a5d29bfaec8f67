/*
 * vxb200_w8a8.h - C ABI of the B200 (sm_100a) W8A8 linear route.
 *
 * The op: fp32 activations -> per-token symmetric int8 (scale = absmax/127)
 * -> int8 x int8 -> int32 GEMM against pre-packed per-output-channel int8
 * weights -> fused epilogue: dequant (act-scale x weight-scale) + bias to fp32,
 * or bit-exact requantization to int8 for a following W8A8 layer.
 *
 * Two layers of entry points:
 *   1. device-pointer entries (vxb_linear_*, vxb_quantize_rows): inputs and
 *      outputs already live in GPU memory; the caller owns them.
 *   2. reference-facing entries (vxb_qlinear_i8u8, vxb_cuda_graph_llm_f32,
 *      vxb_cuda_graph_packed_linear_decode_f32): HOST pointers in, HOST results
 *      out, signatures and return convention of the reference's own CUDA
 *      backend hooks so that its C host code can bind them unchanged.
 *
 * Return convention of every int-returning entry (the reference's tri-state,
 * native/src/backends/cuda_engine.h:13-19):
 *      1  handled - result is in the output buffer
 *      0  declined before touching the output (unsupported dtype/shape/...);
 *         the caller may use another route
 *     -1  failed after work was submitted; do not fall back
 * vxb_last_error() describes the most recent 0 / -1 on the calling thread.
 * There is no CPU fallback anywhere in this library.
 *
 * Plain C types only; all pointers are raw addresses.
 */
#ifndef VXB200_W8A8_H
#define VXB200_W8A8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VXB_ABI_VERSION 1u

#if defined(__GNUC__)
#define VXB_API __attribute__((visibility("default")))
#else
#define VXB_API
#endif

/* Byte dtypes, numerically equal to the reference's VX_DTYPE_U8 / VX_DTYPE_I8
 * (native/include/volvoxai_enums.h:479-480). */
#define VXB_DTYPE_U8 5u
#define VXB_DTYPE_I8 6u
/* Operator id of PackedLinear (native/src/generated/operator_vocabulary.h:127). */
#define VXB_OP_PACKED_LINEAR 1036

typedef struct VxbContext VxbContext; /* device + stream + reusable scratch */
typedef struct VxbWeight VxbWeight;   /* one linear's weights, repacked once */

/* Kernel route selection for vxb_linear_* (VXB_ROUTE_AUTO in production). */
enum {
    VXB_ROUTE_AUTO = 0,
    VXB_ROUTE_GEMV = 1,     /* dp4a + warp-shuffle GEMV (rows <= 32) */
    VXB_ROUTE_TCGEN05 = 2,  /* TMA-fed tcgen05 kind::i8 GEMM, TMEM accumulators */
    VXB_ROUTE_SIMT = 3,     /* one-thread-per-output dp4a kernel (verification) */
    VXB_ROUTE_DECODE = 4,   /* weight-streaming tcgen05 kernel, whole channels per CTA (rows <= 128) */
    VXB_ROUTE_DECODE_STREAMK = 5, /* weight-streaming stream-K tcgen05 kernel (rows <= 128) */
    VXB_ROUTE_TCGEN05_PAIR = 6, /* the tcgen05 GEMM by pairs of CTAs (cta_group::2) on 256 x 256 tiles */
    VXB_ROUTE_DECODE_FUSED = 7, /* the decode kernel quantizing the fp32 rows itself: one launch (rows <= 8, fp32 input) */
    VXB_ROUTE_TCGEN05_WIDE = 8  /* the GEMM for 32-bit outputs: sixteen epilogue warps, TMA tile stores (aligned output) */
};

VXB_API uint32_t vxb_abi_version(void);
VXB_API const char* vxb_last_error(void);
/* Name of the kernel route the calling thread's last handled call took,
 * e.g. "k1+tcgen05-i8+e1"; the counterpart of the reference's per-node route
 * labels (native/src/runtime/engine_runtime_dispatch.inc:2118). */
VXB_API const char* vxb_last_route(void);
/* Number of kernels this library launched since load (all threads). */
VXB_API uint64_t vxb_launch_count(void);

/* ---- context ---------------------------------------------------------- */
/* `stream` is a cudaStream_t (NULL = the legacy default stream). Scratch
 * (quantized activations, row scales, split-K partials) grows on demand and is
 * reused; one context must not be used from two threads at once.  Mirrors the
 * reference's rule that contexts never share mutable scratch
 * (docs/backend-sdk.md:75-95). */
VXB_API int vxb_context_create(int device, void* stream, VxbContext** out);
VXB_API void vxb_context_destroy(VxbContext* ctx);
VXB_API int vxb_context_set_stream(VxbContext* ctx, void* stream);
VXB_API int vxb_context_synchronize(VxbContext* ctx);

/* ---- weight loader ("repack once at compile time") -------------------- */
/* Replaces the reference's per-model one-time packing of QLinear weights,
 * qlinear_metadata_build -> vx_pack_q8_weight
 * (native/src/runtime/engine_runtime_model.inc:2125-2218,
 *  native/src/kernels/packed_quant_gemm.c:237-392).
 * Source layout = the canonical W8A8 SafeTensors tensors
 * (docs/w8a8-safetensors.md:13-121): int8 weight [d_out,d_in] row-major,
 * fp32 per-output-channel scale [d_out] (all > 0, finite).  bias_f32 (E1) and
 * bias_i32 (E2, accumulator domain) are optional.  HOST pointers; the data is
 * copied, laid out for TMA (rows padded to a multiple of 128 bytes with zeros)
 * and the per-channel code sums needed for activation zero points are
 * computed on the device. */
VXB_API int vxb_weight_create_i8(VxbContext* ctx, const int8_t* weight, const float* weight_scales,
                         const float* bias_f32, const int32_t* bias_i32,
                         uint32_t d_out, uint32_t d_in, VxbWeight** out);
/* Same, from PackedLinear W8 storage (docs/packed-linear-design.md:24-41;
 * native/src/kernels/llm_ops.h:22-32): I32 words [d_out, ceil(d_in/4)] in
 * offset-binary (int8 = byte ^ 0x80, padding bytes 0x80) and fp32 group scales
 * [d_out, ceil(d_in/group_size)], group_size 32/64/128/256, all scales positive and
 * finite (else declined, 0).  When every group scale of a row is identical the weight is
 * a per-channel weight like the above.  Otherwise it keeps its group scales and is served
 * by the grouped-scale kernel, which follows the reference's arithmetic group by group
 * (an exact integer dot per group, fp32 accumulation in ascending group order,
 * native/src/kernels/packed_linear_ops.inc:1493-1531): such a weight gives fp32 output
 * (vxb_linear_f32 and the PackedLinear host entries) on the automatic route only; the
 * int8, int32 and explicit-route entries decline it. */
VXB_API int vxb_weight_create_w8_words(VxbContext* ctx, const int32_t* words, const float* group_scales,
                               const float* bias_f32, uint32_t d_out, uint32_t d_in,
                               uint32_t group_size, VxbWeight** out);
/* Same, from PackedLinear W4 storage with A8 arithmetic (the reference's W4/A8 mode,
 * docs/quantization-benchmark-20261023.md:17): eight 4-bit codes per word, earlier K in lower bits,
 * w = code - 8, padding codes 8 (tools/exporter/packed_linear.py:39-87).  The codes are unpacked to
 * int8 once at load time and served by the same kernels as a W8 weight (the grouped-scale kernel
 * when the group scales differ, which is the exporter's normal output). */
VXB_API int vxb_weight_create_w4_words(VxbContext* ctx, const int32_t* words, const float* group_scales,
                               const float* bias_f32, uint32_t d_out, uint32_t d_in,
                               uint32_t group_size, VxbWeight** out);
VXB_API void vxb_weight_destroy(VxbWeight* w);
VXB_API uint32_t vxb_weight_d_in(const VxbWeight* w);
VXB_API uint32_t vxb_weight_d_out(const VxbWeight* w);
/* Bytes of device memory the repacked weight occupies. */
VXB_API uint64_t vxb_weight_device_bytes(const VxbWeight* w);

/* ---- device-pointer entries ------------------------------------------- */
/* Per-token quantizer alone. Device twin of vx_packed_prepare_i8_*
 * (native/src/kernels/packed_linear_ops.inc:97-217) and of the scalar branch
 * at :1574-1597.  x: fp32 [rows,k] (device).  q: int8 [rows,ldq], ldq >= k,
 * bytes k..ldq-1 of every row are zeroed.  row_scales: fp32 [rows]; a row that
 * holds NaN/Inf gets scale NaN, all-zero codes and valid 0.  valid may be NULL. */
VXB_API int vxb_quantize_rows(VxbContext* ctx, const float* x, uint32_t rows, uint32_t k,
                      int8_t* q, uint32_t ldq, float* row_scales, int32_t* valid);

/* Whole op, fp32 out (epilogue E1): y[m,n] = f32(f32(acc)*f32(as[m]*ws[n])) + bias[n].
 * Device twin of vx_packed_linear_forward in dynamic-I8 mode with one scale
 * group per channel (native/src/kernels/packed_linear_ops.inc:1545-1621).
 * x: fp32 [rows,d_in]; y: fp32, row stride ldy elements (>= d_out). */
VXB_API int vxb_linear_f32(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                   float* y, uint32_t ldy, int route);

/* Whole op, int8 out (epilogue E2), bit-exact:
 *   mult = f32(f32(as[m]*ws[n]) / out_scale)
 *   q    = sat_i8(rte(f32(f32(f32(acc + bias_i32[n]) * mult) + out_zero)))
 * The arithmetic of vx_w8a8_requantize_accumulator / vx_w8a8_multiplier
 * (native/src/kernels/w8a8_affine.h:125-181) with the dynamic per-token
 * activation scale in place of the static input scale. Rows holding NaN/Inf
 * produce out_zero. y: int8, row stride ldy bytes. */
VXB_API int vxb_linear_i8(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                  float out_scale, int32_t out_zero, int8_t* y, uint32_t ldy, int route);

/* Whole op up to the exact accumulator (no epilogue), for parity checks:
 * acc int32 [rows,d_out]; q_out (int8 [rows,d_in]) and scales_out (fp32 [rows])
 * may be NULL. Exposes what vx_packed_dot_i8 returns per (row, channel)
 * (native/src/kernels/packed_linear_ops.inc:483-493). */
VXB_API int vxb_linear_acc_i32(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                       int32_t* acc, int8_t* q_out, float* scales_out, int route);

/* ---- N-sharded multi-GPU form (no counterpart in the reference, which is single-GPU:
 * docs/cuda.md:26,45-52) -------------------------------------------------------------
 * Each GPU holds a contiguous range of the output channels (one VxbWeight per shard) and a
 * full-width replicated output buffer [rows, ldy]. vxb_linear_i8_gather computes this GPU's
 * channel slab and stores every finished tile both at y (this GPU's buffer, already offset to
 * the shard's first channel) and at the same position of up to 7 peers' buffers, with plain
 * stores over NVLink from the GEMM epilogue: the all-gather is fused into the kernel and
 * overlaps the MMAs. peer_y[p] must be peer-mapped addresses (vxb_peer_open) offset like y.
 * The call only orders this GPU's work; callers synchronise the GPUs (any barrier) before
 * reading a buffer that peers write, and before the next call overwrites it.
 *
 * vxb_peer_alloc allocates such a buffer (cudaMalloc) and returns its 64-byte inter-process
 * handle; the other ranks (one process per GPU) map it with vxb_peer_open and unmap it with
 * vxb_peer_close before the owner calls vxb_peer_free. */
VXB_API int vxb_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
VXB_API int vxb_peer_open(const unsigned char handle[64], void** ptr);
VXB_API int vxb_peer_close(void* ptr);
VXB_API int vxb_peer_free(void* ptr);
VXB_API int vxb_linear_i8_gather(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                         float out_scale, int32_t out_zero, int8_t* y, uint32_t ldy,
                         void* const* peer_y, uint32_t n_peers);
/* Barrier between the GPUs of the N-sharded linear, enqueued on the context's stream like a kernel:
 * when it has completed on a rank, every rank has reached the same point of its stream, and the
 * peer stores each of them issued before that point are visible here.  my_flags is this GPU's flag
 * array (uint32[8], zero at start, from vxb_peer_alloc), peer_flags[p] the peer-mapped address of
 * peer p's array, peer_ranks[p] its rank; epoch counts the barriers (1, 2, 3, ... the same on every
 * rank).  A few microseconds instead of a collective's tens; every wait in it is bounded: a rank
 * that never arrives turns the next vxb_context_synchronize() into -1 instead of a hang. */
VXB_API int vxb_peer_barrier(VxbContext* ctx, uint32_t* my_flags, void* const* peer_flags, const uint32_t* peer_ranks,
                     uint32_t n_peers, uint32_t my_rank, uint32_t epoch);

/* ---- boundary of a static W8A8 island (device pointers) --------------------------------
 * QuantizeLinear, DequantizeLinear and RequantizeLinear with scalar (per-tensor) metadata,
 * the arithmetic of the reference's CPU authority:
 *   quantize    NaN -> zero point; f32(x / scale) + f32(zero), saturated, ties to even
 *               (native/src/kernels/quantize_linear_ops.inc:155-170,230-254)
 *   dequantize  f32((x - zero) * scale), rounded once (:9-16,95-122)
 *   requantize  f32(f32(x - in_zero) * f32(in_scale / out_scale)) + f32(out_zero), NaN -> out_zero,
 *               saturated, ties to even (portable_inference_kernels.inc:2437-2463)
 * Dtypes are VXB_DTYPE_I8 / VXB_DTYPE_U8; scales must be positive and finite (the reference's
 * dequantizer also takes other scales: those are declined here), zero points inside their
 * dtype.  Declined (0) before anything is launched otherwise. */
VXB_API int vxb_quantize_linear_device(VxbContext* ctx, const float* x, uint64_t elements, float scale,
                               int32_t zero_point, uint32_t output_dtype, void* out);
VXB_API int vxb_dequantize_linear_device(VxbContext* ctx, const void* x, uint64_t elements, float scale,
                                 int32_t zero_point, uint32_t input_dtype, float* out);
VXB_API int vxb_requantize_linear_device(VxbContext* ctx, const void* x, uint64_t elements, float input_scale,
                                 int32_t input_zero_point, float output_scale, int32_t output_zero_point,
                                 uint32_t input_dtype, uint32_t output_dtype, void* out);

/* ---- fused decode patterns on the fp32 epilogue --------------------------------------------
 * What the reference's fused GEMV kernels append to a PackedLinear
 * (native/src/backends/cuda/kernels/cuda_forward_gemv_pair_kernels.inc:406-459 gate/up +
 * SiLU * Mul, :670-713 projection + residual Add; recognised by
 * native/src/runtime/incremental_runtime.c:1178-1232):
 *   residual != NULL           y[m, n] = linear(x)[m, n] + residual[m, n]        (fp32 add, rounded once)
 *   activation SILU_MUL        the weight's channels are interleaved (gate_0, up_0, gate_1, up_1, ...):
 *                              y[m, j] = g * sigmoid(g) * u with g, u = linear(x)[m, 2j], [m, 2j+1];
 *                              y is d_out / 2 wide; no residual in this form
 * Automatic route only (decode kernel up to 128 rows, tensor-core GEMM above). q/k/v, or gate/up,
 * share one activation quantization by concatenating their weights along the output channels. */
enum { VXB_ACT_NONE = 0, VXB_ACT_SILU_MUL = 1 };
VXB_API int vxb_linear_f32_fused(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows, float* y,
                         uint32_t ldy, const float* residual, uint32_t ld_residual, int activation);

/* RMSNorm folded into the quantizer: the head of the reference's fused decode patterns
 * RMSNorm + {q,k,v} and RMSNorm + gate/up + SiLU*Mul
 * (native/src/backends/cuda/kernels/cuda_forward_gemv_pair_kernels.inc:1133-1711, recognised at
 * native/src/runtime/incremental_runtime.c:1178-1232), for any number of rows.  The residual
 * stream x is read once; norm_out (fp32 [rows,k], may be NULL) receives the normalized rows for
 * other consumers, as the reference's kernels persist them; q / row_scales / valid as
 * vxb_quantize_rows.  Normalization arithmetic of the reference's CPU operator
 * (native/src/kernels/softmax_rmsnorm.inc:3-16): mean of squares and 1/sqrt(mean + epsilon) in
 * double, y = float((double(x) * inv) * double(norm_weight)); the double additions run as a tree, so
 * a normalized value can differ from the sequential loop's by one fp32 unit in the last place in
 * rare cases; the quantization of the normalized row is bit-exact.  epsilon > 0 and finite
 * (native/src/runtime/engine_runtime_dispatch.inc:2912-2915). */
VXB_API int vxb_rmsnorm_quantize_rows(VxbContext* ctx, const float* x, const float* norm_weight, float epsilon,
                              uint32_t rows, uint32_t k, float* norm_out, int8_t* q, uint32_t ldq,
                              float* row_scales, int32_t* valid);

/* RMSNorm -> per-token quantization -> linear -> fp32 epilogue with the optional SiLU*Mul tail of
 * vxb_linear_f32_fused: ONE launch for one and two rows (the decode kernel normalizes and quantizes the
 * rows itself; the counterpart of the reference's fused decode kernels,
 * native/src/backends/cuda/kernels/cuda_forward_gemv_pair_kernels.inc:1136-1424), two launches
 * otherwise, with the same bits either way.  q/k/v (or gate/up, interleaved for SILU_MUL) are one
 * weight concatenated along the output channels, so the three (two) projections share the
 * normalization and the quantization.  norm_out may be NULL. */
VXB_API int vxb_rmsnorm_linear_f32_fused(VxbContext* ctx, const VxbWeight* w, const float* x, const float* norm_weight,
                                 float epsilon, float* norm_out, uint32_t rows, float* y, uint32_t ldy,
                                 int activation);

/* Prepared-activation form, the counterpart of the reference's prepared path
 * (x[4] prepared words / x[5] row scales, native/src/backends/cuda/host/
 * cuda_graph_llm_host.inc:15-107): the caller quantized the rows itself with
 * vxb_quantize_rows into q with row stride vxb_weight_row_bytes(w) (bytes past
 * d_in zero) and passes the row scales.  mode 0: int32 accumulators, 1: fp32
 * (E1), 2: int8 (E2, uses out_scale / out_zero).  ldy in elements of `out`. */
VXB_API uint32_t vxb_weight_row_bytes(const VxbWeight* w);
VXB_API int vxb_linear_prepared(VxbContext* ctx, const VxbWeight* w, const int8_t* q,
                        const float* row_scales, uint32_t rows, int mode, float out_scale,
                        int32_t out_zero, void* out, uint32_t ldy, int route);

/* Static-activation QLinear on device buffers: int8/uint8 input with one
 * per-tensor scale and zero point, int8/uint8 output.  Device twin of
 * vx_qlinear_i8u8_packed (native/src/kernels/packed_quant_gemm.c:2633-2763);
 * uses the weight's bias_i32.  input: [rows,d_in] bytes; output [rows,ldy]. */
VXB_API int vxb_qlinear_device(VxbContext* ctx, const VxbWeight* w, const void* input, uint32_t rows,
                       float input_scale, int32_t input_zero_point, float output_scale,
                       int32_t output_zero_point, uint32_t input_dtype, uint32_t output_dtype,
                       void* output, uint32_t ldy, int route);

/* Whole op with HOST buffers (what an application holding host tensors calls):
 * copies x (fp32 [rows,d_in]) to the device, runs vxb_linear_i8 (requant != 0;
 * y_host int8 [rows,d_out]) or vxb_linear_f32 (requant == 0; y_host fp32
 * [rows,d_out]), copies the result back and waits for it.  The host-pointer
 * convention of the reference's backend hooks
 * (native/src/backends/cuda/host/cuda_graph_llm_host.inc:714-783) applied to the
 * new op.  Batches of 1024 rows or more are cut into row chunks whose upload, kernels and
 * download overlap on three streams (with pinned host memory the copies are asynchronous DMA
 * in both directions at once); the call returns when the whole result is in y_host. */
VXB_API int vxb_linear_host(VxbContext* ctx, const VxbWeight* w, const float* x_host, uint32_t rows,
                    int requant, float out_scale, int32_t out_zero, void* y_host);

/* Per-kernel device timing, the counterpart of the reference's instrumented
 * replay plan (docs/cuda.md:537-556): while enabled, every quantizer launch and
 * every GEMM/GEMV launch of this context is bracketed by CUDA events on the
 * context's stream (at most 8192 launches of each kind are recorded).
 * vxb_context_profile(ctx, 1) clears and starts, (ctx, 0) clears and stops; (ctx, n) with n > 1
 * brackets only every n-th launch of each kind (an event between two launches keeps the later one
 * from starting as a programmatic dependent of the earlier, so dense sampling perturbs a chain).
 * _read waits for the stream and returns summed milliseconds and counts of the RECORDED launches. */
VXB_API int vxb_context_profile(VxbContext* ctx, int enable);
VXB_API int vxb_context_profile_read(VxbContext* ctx, double* quantize_ms, uint64_t* quantize_launches,
                             double* gemm_ms, uint64_t* gemm_launches);

/* Measurement utility (no counterpart in the reference): every SM issues
 * `iters` x 256 back-to-back M128xN256xK32 kind::i8 MMAs on operands resident
 * in shared memory; *tops receives the dense int8 rate in tera-ops/s (2 ops per
 * multiply-accumulate), timed with CUDA events.  The measured denominator for
 * the tensor-bound roofline. */
VXB_API int vxb_measure_i8_tensor_peak(VxbContext* ctx, uint32_t iters, double* tops);

/* Decode linear that allocates nothing.  It has no counterpart in the reference.
 *
 * Who needs it: a host that must not allocate device memory at run time - for
 * example one that reports a fixed memory inventory for a compiled model and
 * is held to it, or code that runs while its stream is being captured, where
 * cudaMalloc is not permitted.  The ordinary entries above grow scratch inside
 * a VxbContext with cudaMalloc; this one takes the split-K scratch of the decode
 * kernel (partial sums, tile counters, status word) from a fixed array that is
 * part of the library image.  Every GPU that loads the library holds that array
 * (about 2 MiB) until the process exits.
 *
 * It runs y = dequant(q * W^T) + bias for rows <= VXB_NOALLOC_MAX_ROWS and
 * d_out <= VXB_NOALLOC_MAX_CHANNELS, fp32 out, on DEVICE buffers that the caller
 * owns: q int8 [rows,row_bytes] and row_scales fp32 [rows] as vxb_quantize_rows
 * writes them (ldq = row_bytes, a multiple of 128, padding zero), weight int8
 * [d_out,row_bytes] row-major with zero padding, weight_scales fp32 [d_out], bias
 * fp32 [d_out] or NULL, y fp32 with row stride ldy.  Larger sizes are refused
 * (return 0) with the limit named in `error`; nothing has been written then.
 *
 * The call makes no cudaMalloc / cudaFree and calls no allocating routine.  The
 * first call on each device looks up the array's address on that device and sets
 * a kernel attribute; make that first call before any stream capture begins.
 * All calls share the one array: each call clears the part it uses, so results
 * do not depend on earlier calls, but two calls whose GPU work overlaps (different
 * streams, or graphs replayed concurrently) race on it - keep them ordered.
 * The work is enqueued on `stream` (a cudaStream_t); with wait != 0 the call also
 * waits for it and returns -1 if a bounded device wait expired.  A call with
 * wait == 0 (the form to use under stream capture) only enqueues and so reports
 * nothing by itself: if one of the kernel's bounded waits expires, the status
 * word in the array stays raised - later calls do not clear it - and the next
 * call made with wait != 0 returns -1 for it, whichever call raised it.  After a
 * sequence of wait == 0 calls or graph replays, make one waited call (or check
 * the outputs) before trusting the results.  error/error_bytes name an optional
 * buffer for a message. */
#define VXB_NOALLOC_MAX_ROWS 32u
#define VXB_NOALLOC_MAX_CHANNELS 16384u
VXB_API int vxb_decode_linear_f32_noalloc(const int8_t* q, const float* row_scales, uint32_t rows,
                                  const int8_t* weight, const float* weight_scales,
                                  const float* bias, uint32_t d_out, uint32_t row_bytes,
                                  float* y, uint32_t ldy, void* stream, int wait,
                                  char* error, size_t error_bytes);

/* ---- reference-facing entries (HOST pointers) ------------------------- */
/* Drop-in for the VxW8A8Ops.qlinear_i8u8 slot
 * (native/src/backends/w8a8_device_ops.h:15-17,89-124; CUDA implementation
 * cuda_graph_qlinear_i8u8, native/src/backends/cuda/host/
 * cuda_graph_quantized_linear_conv_host.inc:19-106).  Same argument order.
 * Weights are keyed by host address and repacked on first use (immutable, as
 * the reference marks them is_weight). Declines non-zero weight zero points,
 * U8 weights, overlapping output, non-finite or non-positive scales. */
VXB_API int vxb_qlinear_i8u8(const void* input, const void* weight, const float* weight_scales,
                     const int32_t* weight_zero_points, const int32_t* bias, void* output,
                     uint32_t rows, uint32_t d_in, uint32_t d_out, float input_scale,
                     int32_t input_zero_point, float output_scale, int32_t output_zero_point,
                     uint32_t input_dtype, uint32_t weight_dtype, uint32_t output_dtype);

/* Layout-compatible with the reference's VxLLMOpArgs
 * (native/src/kernels/llm_ops.h:38-53); only the PackedLinear fields are read:
 * x[0]=input fp32 [rows,K], x[1]=W8 words, x[2]=group scales, x[3]=bias or NULL,
 * y[0]=out fp32 [rows,N]; key_dim=K, value_dim=N, rate=group size,
 * groups=weight bits, normalize=activation bits, batch*sequence=rows,
 * first_unit/unit_count = flat output window (0 = everything). */
typedef struct VxbLLMOpArgs {
    int32_t kind, batch, sequence, keys, heads, kv_heads, key_dim, value_dim;
    int32_t streams, groups, rate, window, top_k, iterations;
    int32_t index_heads, index_dim, rotary_dim, rotary_offset;
    int32_t normalize, causal, interleaved, mask_mode;
    float eps, hc_eps, scale;
    const float* x[8];
    float* y[3];
    const int32_t* mask;
    const int32_t* positions;
    uint64_t x_elements[8], y_elements[3], mask_elements, position_elements;
    int32_t query_offset;
    uint64_t first_unit, unit_count;
} VxbLLMOpArgs;

/* The three boundary operators with HOST pointers: the slots quantize_typed_f32_i8u8,
 * dequantize_typed_i8u8_f32 and requantize_linear_i8u8 of VxW8A8Ops
 * (native/src/backends/w8a8_device_ops.h:28-31,111-113), signatures of
 * cuda_graph_quantize_typed_f32_i8u8 / cuda_graph_dequantize_typed_i8u8_f32 /
 * cuda_graph_requantize_linear_i8u8 (native/src/backends/cuda_engine.h:627-644).
 * 1 = handled, 0 = declined before the output was touched, -1 = failed after submission. */
VXB_API int vxb_quantize_typed_f32_i8u8(const float* input, uint32_t elements, void* output, float output_scale,
                                int32_t output_zero_point, uint32_t output_dtype);
VXB_API int vxb_dequantize_typed_i8u8_f32(const void* input, uint32_t elements, float input_scale,
                                  int32_t input_zero_point, uint32_t input_dtype, float* output);
VXB_API int vxb_requantize_linear_i8u8(const void* input, uint32_t input_elements, void* output,
                               uint32_t output_elements, float input_scale, int32_t input_zero_point,
                               float output_scale, int32_t output_zero_point, uint32_t input_dtype,
                               uint32_t output_dtype);

/* Drop-in for cuda_graph_llm_f32 with kind == PackedLinear
 * (native/src/backends/cuda_engine.h:13-15; native/src/backends/cuda/host/
 * cuda_graph_llm_host.inc:714-783).  Admits weight bits 8 or 4 with activation
 * bits 8 and group size 32/64/128/256, with group scales that repeat the channel
 * scale (served as a per-channel weight) or differ within a channel (served by the
 * grouped-scale kernels, exact per-group arithmetic).  Declines (0) everything
 * else - weight bits 2/3, activation bits 16/32, ragged windows, an output window
 * that overlaps a source - before anything is touched, so that the reference's own
 * routes keep serving those.  A window must cover whole rows.  Weights are keyed
 * by their host addresses, shape, bit width and group size and repacked on first
 * use. */
VXB_API int vxb_cuda_graph_llm_f32(const VxbLLMOpArgs* args);

/* Drop-in for the scalar decode entry cuda_graph_packed_linear_decode_f32
 * (native/src/backends/cuda_engine.h:16-19; impl cuda_graph_llm_host.inc:111-186):
 * one row, group size 128. */
VXB_API int vxb_cuda_graph_packed_linear_decode_f32(const float* input, const int32_t* packed_weights,
                                            const float* weight_scales, const float* bias,
                                            float* output, uint32_t input_width,
                                            uint32_t output_width, uint32_t weight_bits,
                                            uint32_t activation_bits);

/* Device residency behind the reference-facing entries, the counterpart of the reference backend's
 * host-pointer -> device-slot table with dirty marking (graph_ensure_input_view / graph_mark_device,
 * native/src/backends/cuda/host/cuda_graph_memory_host.inc:1302-1310).  Off (the default), every entry
 * uploads its input, downloads its output and returns when the host buffer holds the result.  On, an
 * entry's output stays in a device buffer keyed by its host address - the host copy is STALE until
 * vxb_host_download(ptr) (NULL: every tensor) - and a later entry whose input is that tensor, or a row
 * window inside it, reads it where it lies: a chain of nodes bound through these entries crosses PCIe
 * once in and once out instead of twice per node.  Ownership rule: while residency is on, the host
 * calls vxb_host_download before it reads such an output and vxb_host_invalidate(ptr) (NULL: all)
 * after it writes into one by itself; inputs the library did not produce are uploaded on every call, so
 * plain host inputs need no announcement.  Partial output windows are written to the host at once.
 * Turning residency off downloads everything that is still device-dirty. */
VXB_API int vxb_host_residency(int enable);
VXB_API int vxb_host_download(const void* host_ptr);
VXB_API int vxb_host_invalidate(const void* host_ptr);

/* Drops every cached weight / context / resident tensor the reference-facing entries created
 * (the counterpart of freeing a compiled model). */
VXB_API void vxb_host_cache_clear(void);

#ifdef __cplusplus
}
#endif
#endif /* VXB200_W8A8_H */
