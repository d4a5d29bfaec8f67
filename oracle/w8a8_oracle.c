/*
 * CPU oracle for the W8A8 linear: a plain-C restatement of the reference's
 * arithmetic, used ONLY as a checker by the tests, the smoke run and the
 * benchmark's cpu_baseline leg.  It is test infrastructure, never a product
 * path: the CUDA library does not link, load or call anything in here.
 *
 * Parity is pinned: tests/test_oracle_pins.py checks every function below
 * against (a) the known-answer vectors of the reference's own tests, (b) the
 * reference's CPU sources compiled unmodified into oracle/_ref (when present)
 * and (c) committed fixtures generated from the reference's NumPy packer.
 *
 * Each function cites the reference file:line it follows (paths relative to
 * the reference project root).  Build with -O2 -ffp-contract=off so no
 * multiply-add is fused.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#if defined(__GNUC__)
#define VXO_API __attribute__((visibility("default")))
#else
#define VXO_API
#endif

static int vxo_finite(float v) {
    /* native/src/kernels/packed_linear.h:82-85: exponent not all ones. */
    union { float f; uint32_t u; } b; b.f = v;
    return (b.u & 0x7f800000u) != 0x7f800000u;
}

/* native/src/kernels/packed_linear.h:108-116 (vx_packed_round_i8):
 * saturate at +-127 first, truncate, then fix up with the remainder so that
 * ties go to even. */
VXO_API int32_t vxo_round_i8(float value) {
    if (value >= 127.0f) return 127;
    if (value <= -127.0f) return -127;
    int32_t whole = (int32_t)value;
    float rest = value - (float)whole;
    if (rest > 0.5f || (rest == 0.5f && (whole & 1))) whole++;
    if (rest < -0.5f || (rest == -0.5f && (whole & 1))) whole--;
    return whole;
}

/* Per-row dynamic int8 preparation.
 * native/src/kernels/packed_linear_ops.inc:1574-1597 (scalar branch) and
 * :97-153 (AVX2 twin): a row holding NaN/Inf is invalid (all-zero codes);
 * scale = max==0 ? 1 : max/127 with a true fp32 divide, floored at 2^-126;
 * q = round_i8(x / scale).
 * q is written with row stride ldq (bytes beyond K are left untouched). */
VXO_API void vxo_quantize_rows(const float* x, uint64_t rows, uint32_t k,
                               int8_t* q, uint64_t ldq, float* scales,
                               int32_t* valid) {
    for (uint64_t r = 0; r < rows; r++) {
        const float* in = x + r * (uint64_t)k;
        float maximum = 0.0f; int finite = 1;
        for (uint32_t j = 0; j < k; j++) {
            float v = in[j];
            if (!vxo_finite(v)) { finite = 0; break; }
            float a = v < 0.0f ? -v : v;
            if (a > maximum) maximum = a;
        }
        volatile float scale = maximum == 0.0f ? 1.0f : maximum / 127.0f;
        if (scale < 0x1p-126f) scale = 0x1p-126f;
        /* The AVX2 twin computes the scale from the maximum seen before the
         * first non-finite lane; only validity is observable for such rows,
         * so the oracle reports scale 1 for them. */
        if (!finite) scale = 1.0f;
        scales[r] = scale;
        if (valid) valid[r] = finite;
        for (uint32_t j = 0; j < k; j++) {
            volatile float ratio = finite ? in[j] / scale : 0.0f;
            q[r * ldq + j] = (int8_t)(finite ? vxo_round_i8(ratio) : 0);
        }
    }
}

/* Exact integer accumulator: acc[m,n] = sum_k q[m,k] * w[n,k].
 * native/src/kernels/portable_inference_kernels.inc:1006-1020 (int64 running
 * sum, int32 range check) with zero points 0; equals vx_packed_dot_i8 over
 * the whole row (native/src/kernels/packed_linear_ops.inc:483-493).
 * Returns 0 if any accumulator leaves int32 range, 1 otherwise. */
VXO_API int vxo_gemm_i32(const int8_t* q, uint64_t ldq, const int8_t* w,
                         uint64_t ldw, uint64_t rows, uint32_t k, uint32_t n,
                         int32_t* acc) {
    for (uint64_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < n; c++) {
            int64_t sum = 0;
            const int8_t* a = q + r * ldq; const int8_t* b = w + (uint64_t)c * ldw;
            for (uint32_t j = 0; j < k; j++) sum += (int64_t)a[j] * (int64_t)b[j];
            if (sum < INT32_MIN || sum > INT32_MAX) return 0;
            acc[r * n + c] = (int32_t)sum;
        }
    return 1;
}

/* E1, per-channel form: y = f32(f32(acc) * f32(as*ws[n])) + bias[n]; an
 * invalid row yields NaN.  This is the one-group case of
 * native/src/kernels/packed_linear_ops.inc:1500-1531
 * (sum += (float)dot * (activation_scale * scale[group]); + bias). */
VXO_API void vxo_dequant_bias_f32(const int32_t* acc, uint64_t rows, uint32_t n,
                                  const float* row_scales, const int32_t* valid,
                                  const float* ws, const float* bias, float* y) {
    for (uint64_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < n; c++) {
            if (valid && !valid[r]) { y[r * n + c] = __builtin_nanf(""); continue; }
            volatile float combined = row_scales[r] * ws[c];
            volatile float product = (float)acc[r * n + c] * combined;
            volatile float sum = 0.0f + product;
            y[r * n + c] = sum + (bias ? bias[c] : 0.0f);
        }
}

/* R1 in full, W8 words with grouped scales, dynamic-I8 arithmetic.
 * native/src/kernels/packed_linear_ops.inc:1545-1621 (driver) and :1493-1531
 * (column loop): per storage group an exact integer dot, then
 * sum += (float)dot * (as * scale[n,g]) in ascending group order, + bias.
 * words: uint32 [N, ceil(K/4)], byte j of a row holds code = w + 128
 * (docs/packed-linear-design.md:24-41). scales: [N, ceil(K/G)]. */
VXO_API int vxo_packed_linear_w8_grouped(const float* x, uint64_t rows, uint32_t k,
                                         uint32_t n, const uint32_t* words,
                                         const float* scales, uint32_t group,
                                         const float* bias, float* y) {
    if (group != 32 && group != 64 && group != 128 && group != 256) return -1;
    if (!k || !n) return -1;
    const uint32_t row_words = (k + 3u) / 4u, groups = (k + group - 1u) / group;
    int8_t q[k];
    for (uint64_t r = 0; r < rows; r++) {
        float as; int32_t ok;
        vxo_quantize_rows(x + r * (uint64_t)k, 1, k, q, k, &as, &ok);
        for (uint32_t c = 0; c < n; c++) {
            if (!ok) { y[r * n + c] = __builtin_nanf(""); continue; }
            const uint8_t* code = (const uint8_t*)(words + (uint64_t)c * row_words);
            volatile float sum = 0.0f;
            for (uint32_t g = 0; g < groups; g++) {
                uint32_t begin = g * group, end = begin + group < k ? begin + group : k;
                int32_t dot = 0;
                for (uint32_t j = begin; j < end; j++)
                    dot += (int32_t)q[j] * ((int32_t)code[j] - 128);
                volatile float combined = as * scales[(uint64_t)c * groups + g];
                volatile float product = (float)dot * combined;
                sum = sum + product;
            }
            y[r * n + c] = sum + (bias ? bias[c] : 0.0f);
        }
    }
    return 0;
}

/* The same forward for W4 storage (A8 arithmetic): eight codes per word, earlier K in lower
 * bits, w = code - 8 (docs/packed-linear-design.md:24-41; tools/exporter/packed_linear.py:39-87;
 * dot over nibbles native/src/kernels/packed_linear_ops.inc:285-493 with bits = 4). */
VXO_API int vxo_packed_linear_w4_grouped(const float* x, uint64_t rows, uint32_t k,
                                         uint32_t n, const uint32_t* words,
                                         const float* scales, uint32_t group,
                                         const float* bias, float* y) {
    if (group != 32 && group != 64 && group != 128 && group != 256) return -1;
    if (!k || !n) return -1;
    const uint32_t row_words = (k + 7u) / 8u, groups = (k + group - 1u) / group;
    int8_t q[k];
    for (uint64_t r = 0; r < rows; r++) {
        float as; int32_t ok;
        vxo_quantize_rows(x + r * (uint64_t)k, 1, k, q, k, &as, &ok);
        for (uint32_t c = 0; c < n; c++) {
            if (!ok) { y[r * n + c] = __builtin_nanf(""); continue; }
            const uint32_t* wr = words + (uint64_t)c * row_words;
            volatile float sum = 0.0f;
            for (uint32_t g = 0; g < groups; g++) {
                uint32_t begin = g * group, end = begin + group < k ? begin + group : k;
                int32_t dot = 0;
                for (uint32_t j = begin; j < end; j++)
                    dot += (int32_t)q[j] * ((int32_t)((wr[j >> 3] >> (4u * (j & 7u))) & 0xFu) - 8);
                volatile float combined = as * scales[(uint64_t)c * groups + g];
                volatile float product = (float)dot * combined;
                sum = sum + product;
            }
            y[r * n + c] = sum + (bias ? bias[c] : 0.0f);
        }
    }
    return 0;
}

/* native/src/kernels/w8a8_affine.h:114-120 (ties to even through floor). */
VXO_API int32_t vxo_round_ties_even(float value) {
    const int32_t lower = (int32_t)__builtin_floorf(value);
    const float fraction = value - (float)lower;
    if (fraction < 0.5f) return lower;
    if (fraction > 0.5f) return lower + 1;
    return lower % 2 == 0 ? lower : lower + 1;
}

/* native/src/kernels/w8a8_affine.h:125-131: NaN -> zero point, saturate. */
static int32_t vxo_requantize(float t, int32_t lo, int32_t hi, int32_t nan_value) {
    if (t != t) return nan_value;
    if (t <= (float)lo) return lo;
    if (t >= (float)hi) return hi;
    return vxo_round_ties_even(t);
}

/* native/src/kernels/w8a8_affine.h:155-181: multiplier =
 * f32(f32(input_scale*weight_scale)/output_scale); 0 when any operand or the
 * result is not a positive finite fp32. */
VXO_API int vxo_multiplier(float is, float ws, float os, float* out) {
    volatile float product, multiplier;
    if (!(vxo_finite(is) && is > 0.0f) || !(vxo_finite(ws) && ws > 0.0f) ||
        !(vxo_finite(os) && os > 0.0f)) return 0;
    product = is * ws;
    multiplier = product / os;
    if (!(vxo_finite(multiplier) && multiplier > 0.0f)) return 0;
    *out = multiplier;
    return 1;
}

/* E2 on an exact accumulator, one activation scale per ROW (the dynamic
 * per-token extension of R2).  Per element, with acc' = acc + bias_i32[n]:
 *   t = f32(f32(acc') * mult(as[m], ws[n], os));  t = f32(t + oz);
 *   q = NaN->oz, saturate to [lo,hi], else ties-to-even
 * native/src/kernels/w8a8_affine.h:140-153 and
 * native/src/kernels/portable_inference_kernels.inc:1021-1028.
 * out_unsigned selects U8 [0,255] instead of I8 [-128,127].  Invalid rows
 * store the zero point.  Returns 0 (nothing promised about out) when a
 * multiplier is not representable, as the reference refuses such calls. */
VXO_API int vxo_requant_rows(const int32_t* acc, uint64_t rows, uint32_t n,
                             const float* row_scales, const int32_t* valid,
                             const float* ws, const int32_t* bias_i32,
                             float out_scale, int32_t out_zero, int out_unsigned,
                             uint8_t* out) {
    const int32_t lo = out_unsigned ? 0 : -128, hi = out_unsigned ? 255 : 127;
    for (uint64_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < n; c++) {
            if (valid && !valid[r]) { out[r * n + c] = (uint8_t)out_zero; continue; }
            float mult;
            if (!vxo_multiplier(row_scales[r], ws[c], out_scale, &mult)) return 0;
            int64_t a = (int64_t)acc[r * n + c] + (bias_i32 ? bias_i32[c] : 0);
            if (a < INT32_MIN || a > INT32_MAX) return 0;
            volatile float scaled = (float)a * mult;
            volatile float moved = scaled + (float)out_zero;
            out[r * n + c] = (uint8_t)vxo_requantize(moved, lo, hi, out_zero);
        }
    return 1;
}

/* R2 in full: static per-tensor activations, raw [d_out,d_in] weights.
 * native/src/kernels/portable_inference_kernels.inc:968-1032 (qlinear_i8u8).
 * dtype flags: 0 = I8, 1 = U8.  Returns 1 handled / 0 refused. */
VXO_API int vxo_qlinear_i8u8(const void* input, const void* weight,
                             const int32_t* bias, const float* ws,
                             const int32_t* wz, void* output, uint32_t rows,
                             uint32_t d_in, uint32_t d_out, float in_scale,
                             int32_t in_zero, float out_scale, int32_t out_zero,
                             int in_unsigned, int w_unsigned, int out_unsigned) {
    if (!input || !weight || !bias || !ws || !wz || !output || !rows || !d_in || !d_out)
        return 0;
    const int32_t lo = out_unsigned ? 0 : -128, hi = out_unsigned ? 255 : 127;
    if (in_zero < (in_unsigned ? 0 : -128) || in_zero > (in_unsigned ? 255 : 127)) return 0;
    if (out_zero < lo || out_zero > hi) return 0;
    for (uint32_t c = 0; c < d_out; c++) {
        float mult;
        if (wz[c] < (w_unsigned ? 0 : -128) || wz[c] > (w_unsigned ? 255 : 127)) return 0;
        if (!vxo_multiplier(in_scale, ws[c], out_scale, &mult)) return 0;
    }
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < d_out; c++) {
            int64_t acc = bias[c];
            float mult; vxo_multiplier(in_scale, ws[c], out_scale, &mult);
            for (uint32_t j = 0; j < d_in; j++) {
                size_t xi = (size_t)r * d_in + j, wi = (size_t)c * d_in + j;
                int32_t xv = in_unsigned ? ((const uint8_t*)input)[xi] : ((const int8_t*)input)[xi];
                int32_t wv = w_unsigned ? ((const uint8_t*)weight)[wi] : ((const int8_t*)weight)[wi];
                acc += (int64_t)(xv - in_zero) * (int64_t)(wv - wz[c]);
                if (acc < INT32_MIN || acc > INT32_MAX) return 0;
            }
            volatile float scaled = (float)acc * mult;
            volatile float moved = scaled + (float)out_zero;
            int32_t qv = vxo_requantize(moved, lo, hi, out_zero);
            if (out_unsigned) ((uint8_t*)output)[(size_t)r * d_out + c] = (uint8_t)qv;
            else ((int8_t*)output)[(size_t)r * d_out + c] = (int8_t)qv;
        }
    return 1;
}

/* The whole new op on the CPU in one call, for the benchmark's "port" leg:
 * quantize rows -> int32 GEMM -> E1 (fp32) or E2 (int8). scratch_q holds
 * rows*k int8, scratch_acc rows*n int32. */
VXO_API int vxo_w8a8_linear(const float* x, uint64_t rows, uint32_t k, uint32_t n,
                            const int8_t* w, const float* ws, const float* bias,
                            const int32_t* bias_i32, float out_scale, int32_t out_zero,
                            int requant, int8_t* scratch_q, int32_t* scratch_acc,
                            float* row_scales, int32_t* valid, void* out) {
    vxo_quantize_rows(x, rows, k, scratch_q, k, row_scales, valid);
    if (!vxo_gemm_i32(scratch_q, k, w, k, rows, k, n, scratch_acc)) return 0;
    if (!requant) {
        vxo_dequant_bias_f32(scratch_acc, rows, n, row_scales, valid, ws, bias, (float*)out);
        return 1;
    }
    return vxo_requant_rows(scratch_acc, rows, n, row_scales, valid, ws, bias_i32,
                            out_scale, out_zero, 0, (uint8_t*)out);
}

/* Checker for the constant-divisor division the CUDA epilogues use (no
 * counterpart in the reference, which divides with the IEEE operator): computes
 * a/d through rcp = RN(1/d) and two FMA corrections and counts disagreements
 * with the correctly rounded quotient over `count` pseudo-random positive a
 * whose exponents are uniform in [lo_exp, hi_exp]. */
#include <math.h>
VXO_API uint64_t vxo_div_const_mismatches(float d, uint64_t count, uint64_t seed,
                                          int lo_exp, int hi_exp) {
    const float rcp = (float)(1.0 / (double)d);
    uint64_t bad = 0, state = seed * 6364136223846793005ull + 1442695040888963407ull;
    for (uint64_t i = 0; i < count; i++) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        const uint32_t mant = (uint32_t)(state >> 41);                 /* 23 bits */
        const int span = hi_exp - lo_exp + 1;
        const int e = lo_exp + (int)((state >> 20) % (uint64_t)span);
        union { uint32_t u; float f; } a;
        a.u = ((uint32_t)(e + 127) << 23) | mant;
        volatile float want = a.f / d;
        const float q0 = a.f * rcp;
        const float r0 = fmaf(-d, q0, a.f);
        const float q1 = fmaf(r0, rcp, q0);
        const float r1 = fmaf(-d, q1, a.f);
        const float q2 = fmaf(r1, rcp, q1);
        union { float f; uint32_t u; } x, y; x.f = q2; y.f = want;
        bad += x.u != y.u;
    }
    return bad;
}

/* ---- the F32 <-> byte boundary and the byte-to-byte bridge ---------------------------------
 * dtype: 0 = int8, 1 = uint8 (the callers translate the reference's VX_DTYPE codes). */
static void vxo_byte_range(int is_unsigned, int32_t* lo, int32_t* hi) {
    *lo = is_unsigned ? 0 : -128; *hi = is_unsigned ? 255 : 127;
}


/* RMSNorm over the last axis (native/src/kernels/softmax_rmsnorm.inc:3-16): squares and their
 * mean accumulated left to right in double, inv = 1/sqrt(mean + eps) in double,
 * y = float((double(x) * inv) * weight) with weight promoted to double. */
VXO_API void vxo_rmsnorm_rows(const float* x, const float* weight, float* y, uint32_t rows, uint32_t k, double eps) {
    for (uint32_t r = 0; r < rows; r++) {
        const float* in = x + (size_t)r * k;
        double var = 0.0;
        for (uint32_t j = 0; j < k; j++) { const double v = in[j]; var += v * v; }
        var /= (double)k;
        const double inv = 1.0 / sqrt(var + eps);
        for (uint32_t j = 0; j < k; j++) y[(size_t)r * k + j] = (float)((double)in[j] * inv * weight[j]);
    }
}

/* native/src/kernels/quantize_linear_ops.inc:155-170,230-254 (quantize_linear_typed):
 * NaN -> zero point; t = x / scale + (float)zero; saturate, ties to even. */
VXO_API int vxo_quantize_linear(const float* x, uint64_t elements, float scale, int32_t zero,
                                int out_unsigned, void* out) {
    int32_t lo, hi;
    vxo_byte_range(out_unsigned, &lo, &hi);
    if (!vxo_finite(scale) || scale <= 0.0f || zero < lo || zero > hi) return 0;
    for (uint64_t i = 0; i < elements; i++) {
        int32_t q;
        float v = x[i];
        if (v != v) q = zero;
        else {
            volatile float quotient = v / scale;
            volatile float t = quotient + (float)zero;
            if (t <= (float)lo) q = lo;
            else if (t >= (float)hi) q = hi;
            else if (!vxo_finite(t)) q = t < 0.0f ? lo : hi;
            else q = vxo_round_ties_even(t);
        }
        if (out_unsigned) ((uint8_t*)out)[i] = (uint8_t)q; else ((int8_t*)out)[i] = (int8_t)q;
    }
    return 1;
}

/* native/src/kernels/quantize_linear_ops.inc:9-16,95-122 (dequantize_linear_typed):
 * (float)(((double)x - zero) * (double)scale). */
VXO_API int vxo_dequantize_linear(const void* x, uint64_t elements, float scale, int32_t zero,
                                  int in_unsigned, float* out) {
    for (uint64_t i = 0; i < elements; i++) {
        const double v = in_unsigned ? (double)((const uint8_t*)x)[i] : (double)((const int8_t*)x)[i];
        out[i] = (float)((v - (double)zero) * (double)scale);
    }
    return 1;
}

/* native/src/kernels/portable_inference_kernels.inc:2437-2463 (requantize_linear_i8u8):
 * multiplier = in_scale / out_scale (f32); f32(f32(x - in_zero) * multiplier) + f32(out_zero),
 * then the canonical requantization (NaN -> out_zero, saturate, ties to even). */
VXO_API int vxo_requantize_linear(const void* x, void* out, uint64_t elements, float in_scale, int32_t in_zero,
                                  float out_scale, int32_t out_zero, int in_unsigned, int out_unsigned) {
    int32_t ilo, ihi, lo, hi;
    vxo_byte_range(in_unsigned, &ilo, &ihi);
    vxo_byte_range(out_unsigned, &lo, &hi);
    if (!elements || !vxo_finite(in_scale) || in_scale <= 0.0f || !vxo_finite(out_scale) || out_scale <= 0.0f ||
        in_zero < ilo || in_zero > ihi || out_zero < lo || out_zero > hi) return 0;
    volatile float multiplier = in_scale / out_scale;
    if (!vxo_finite(multiplier) || multiplier <= 0.0f) return 0;
    for (uint64_t i = 0; i < elements; i++) {
        const int32_t v = in_unsigned ? (int32_t)((const uint8_t*)x)[i] : (int32_t)((const int8_t*)x)[i];
        volatile float centered = (float)(v - in_zero);
        volatile float scaled = centered * multiplier;
        volatile float t = scaled + (float)out_zero;
        const int32_t q = vxo_requantize(t, lo, hi, out_zero);
        if (out_unsigned) ((uint8_t*)out)[i] = (uint8_t)q; else ((int8_t*)out)[i] = (int8_t)q;
    }
    return 1;
}
