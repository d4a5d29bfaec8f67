/*
 * Thin export layer over the reference's OWN CPU sources, compiled from where
 * they lie in the reference checkout (nothing is copied into this repository;
 * see oracle/Makefile).  The resulting oracle/_ref/libvxref.so is test
 * infrastructure: it validates the restatement in w8a8_oracle.c and serves as
 * the timed CPU baseline.  The CUDA library never loads it.
 *
 * This translation unit includes packed_linear_ops.inc directly to reach the
 * file-local quantizer / integer dot; everything with external linkage
 * (vx_llm_forward_f32, qlinear_i8u8, vx_qlinear_i8u8_packed, the thread pool)
 * comes from the reference's kernels.c amalgamation linked beside it.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "llm_ops.h"
#include "packed_linear_ops.inc"   /* static: vx_packed_prepare_i8_simd, vx_packed_dot_i8 */
#include "packed_quant_gemm.h"
#include "thread_pool.h"
#include "kernel_platform.h"
#include "w8a8_affine.h"

#define REF_API __attribute__((visibility("default")))

int qlinear_i8u8(const void*, const void*, const int32_t*, const float*, const int32_t*,
                 void*, uint32_t, uint32_t, uint32_t, float, int32_t, float, int32_t,
                 uint32_t, uint32_t, uint32_t);

REF_API int32_t ref_round_i8(float v) { return vx_packed_round_i8(v); }

/* Narrow (int8) per-row preparation exactly as the forward pass runs it. */
REF_API int ref_prepare_i8(const float* x, uint32_t k, int8_t* q, float* scale) {
#if VX_PACKED_HAS_SIMD_QUANT
    return vx_packed_prepare_i8_simd(x, k, (unsigned char*)q, 0, scale);
#else
    (void)x; (void)k; (void)q; (void)scale; return -1;
#endif
}

/* All rows, spread over the reference's thread pool when a scope is entered. */
typedef struct { const float* x; uint32_t k; int8_t* q; float* scales; } RefPrepareJob;
static void ref_prepare_range(void* opaque, int begin, int end) {
    RefPrepareJob* job = (RefPrepareJob*)opaque;
    for (int r = begin; r < end; r++)
        ref_prepare_i8(job->x + (size_t)r * job->k, job->k, job->q + (size_t)r * job->k,
                       job->scales + r);
}
REF_API void ref_prepare_rows(const float* x, uint32_t rows, uint32_t k, int8_t* q, float* scales) {
    RefPrepareJob job = {x, k, q, scales};
    vx_kernels_parallel_for((int)rows, 8, ref_prepare_range, &job);
}

REF_API int32_t ref_dot_i8(const int8_t* q, const uint32_t* words, uint32_t count, uint32_t bits) {
    return vx_packed_dot_i8(q, words, count, bits);
}

/* R1 through the public CPU entry (allocates its own scratch). */
REF_API int ref_packed_linear(const float* x, uint32_t rows, uint32_t k, uint32_t n,
                              const uint32_t* words, const float* scales, uint32_t group,
                              uint32_t bits, const float* bias, float* y,
                              uint64_t first_unit, uint64_t unit_count) {
    VxLLMOpArgs a; memset(&a, 0, sizeof a);
    a.kind = VX_OP_PACKED_LINEAR; a.batch = 1; a.sequence = (int32_t)rows;
    a.key_dim = (int32_t)k; a.value_dim = (int32_t)n; a.groups = (int32_t)bits;
    a.rate = (int32_t)group; a.normalize = 8;
    a.x[0] = x; a.x[1] = (const float*)words; a.x[2] = scales; a.x[3] = bias; a.y[0] = y;
    a.first_unit = first_unit; a.unit_count = unit_count;
    return vx_llm_forward_f32(&a);
}

REF_API int ref_qlinear_portable(const void* in, const void* w, const int32_t* bias,
        const float* ws, const int32_t* wz, void* out, uint32_t rows, uint32_t d_in,
        uint32_t d_out, float is, int32_t iz, float os, int32_t oz,
        uint32_t in_dt, uint32_t w_dt, uint32_t out_dt) {
    return qlinear_i8u8(in, w, bias, ws, wz, out, rows, d_in, d_out, is, iz, os, oz,
                        in_dt, w_dt, out_dt);
}

REF_API uint32_t ref_packed_q8_size(uint32_t d_in, uint32_t d_out) {
    return vx_packed_q8_weight_size(d_in, d_out);
}
REF_API int ref_pack_q8(void* packed, uint32_t bytes, const void* w, uint32_t d_in,
                        uint32_t d_out, uint32_t w_dt) {
    return vx_pack_q8_weight(packed, bytes, w, d_in, d_out, w_dt, 1u);
}
REF_API int ref_qlinear_packed(const void* in, const void* packed, const int32_t* bias,
        const float* ws, const int32_t* wz, void* out, uint32_t rows, uint32_t d_in,
        uint32_t d_out, float is, int32_t iz, float os, int32_t oz,
        uint32_t in_dt, uint32_t w_dt, uint32_t out_dt) {
    return vx_qlinear_i8u8_packed(in, packed, bias, ws, wz, out, rows, d_in, d_out,
                                  is, iz, os, oz, in_dt, w_dt, out_dt);
}

REF_API int ref_multiplier(float is, float ws, float os, float* out) {
    return vx_w8a8_multiplier(is, ws, os, out);
}
REF_API int32_t ref_round_ties_even(float v) { return vx_w8a8_round_ties_even(v); }
REF_API int32_t ref_requantize_accumulator(int64_t acc, float mult, int32_t oz,
                                           int32_t lo, int32_t hi) {
    return vx_w8a8_requantize_accumulator(acc, mult, oz, lo, hi);
}

/* Thread-pool scope for the calling thread: T<=1 leaves execution serial. */
static VxKernelThreadPool* g_pool;
static VxKernelThreadPoolScope g_scope;
REF_API int ref_threads_enter(int threads) {
    if (g_pool) return -1;
    if (threads <= 1) return 1;
    g_pool = vx_kernel_thread_pool_create(threads);
    if (!g_pool) return -1;
    g_scope = vx_kernel_thread_pool_scope_enter(g_pool);
    return vx_kernels_thread_count();
}
REF_API void ref_threads_leave(void) {
    if (!g_pool) return;
    vx_kernel_thread_pool_scope_leave(g_scope);
    vx_kernel_thread_pool_destroy(g_pool);
    g_pool = NULL;
}
REF_API const char* ref_isa_name(void) {
    return vx_kernel_isa_name(vx_kernel_platform()->isa);
}

/* The F32 <-> integer boundary and the byte-to-byte bridge, as the reference computes them
 * (kernels.c amalgamation: quantize_linear_ops.inc, portable_inference_kernels.inc). */
int quantize_linear_typed(const float*, const float*, const void*, uint32_t, void*, uint32_t, uint32_t);
int dequantize_linear_typed(const void*, int, const float*, const void*, int, float*, int);
int requantize_linear_i8u8(const void*, void*, uint32_t, float, int32_t, float, int32_t, uint32_t, uint32_t);

void rmsnorm_f32(const float*, const float*, float*, int, int, double);
REF_API void ref_rmsnorm_rows(const float* x, const float* weight, float* y, uint32_t rows, uint32_t k, double eps) {
    rmsnorm_f32(x, weight, y, (int)rows, (int)k, eps);
}

REF_API int ref_quantize_linear(const float* x, uint32_t elements, float scale, int32_t zero,
                                uint32_t out_dtype, void* out) {
    int8_t z8 = (int8_t)zero; uint8_t zu = (uint8_t)zero;
    return quantize_linear_typed(x, &scale, out_dtype == VX_DTYPE_I8 ? (const void*)&z8 : (const void*)&zu,
                                 out_dtype, out, out_dtype, elements);
}
REF_API int ref_dequantize_linear(const void* x, uint32_t elements, float scale, int32_t zero,
                                  uint32_t in_dtype, float* out) {
    int8_t z8 = (int8_t)zero; uint8_t zu = (uint8_t)zero;
    return dequantize_linear_typed(x, (int)in_dtype, &scale,
                                   in_dtype == VX_DTYPE_I8 ? (const void*)&z8 : (const void*)&zu,
                                   (int)in_dtype, out, (int)elements);
}
REF_API int ref_requantize_linear(const void* x, void* out, uint32_t elements, float in_scale, int32_t in_zero,
                                  float out_scale, int32_t out_zero, uint32_t in_dtype, uint32_t out_dtype) {
    return requantize_linear_i8u8(x, out, elements, in_scale, in_zero, out_scale, out_zero, in_dtype, out_dtype);
}
