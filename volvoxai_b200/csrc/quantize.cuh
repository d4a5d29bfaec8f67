// Arithmetic of the per-token quantizer shared by the K1 kernels (quantize.cu) and by the decode
// kernel's fused prologue (decode_rows.cu).  Contract (reference:
// native/src/kernels/packed_linear_ops.inc:97-153,1574-1597):
//   scale = amax == 0 ? 1 : amax / 127 (IEEE divide), floored at 2^-126
//   q     = ties-to-even(clamp(x / scale, -127, 127)) with the IEEE quotient
#pragma once

#include "common.cuh"

namespace vxb {

__device__ __forceinline__ bool nonfinite_bits(float v) {
    return (__float_as_uint(v) & 0x7f800000u) == 0x7f800000u;
}

// The row's scale is a constant divisor for the whole row: when it is well inside the
// exponent range and its significand is not all ones, x / scale is computed through the
// correctly rounded reciprocal and two FMA corrections (div_const), which yields the IEEE
// quotient bit for bit wherever the quotient can round to a non-zero code; otherwise
// the IEEE divide is used.
struct RowDivisor {
    float scale, rcp;
    bool fast;
    __device__ __forceinline__ explicit RowDivisor(float s) {
        scale = s;
        rcp = __frcp_rn(s);
        const uint32_t bits = __float_as_uint(s);
        fast = s >= 8.67361737988403547206e-19f && s <= 1152921504606846976.0f &&  // 2^-60 .. 2^60
               (bits & 0x007fffffu) != 0x007fffffu;
    }
};

template <bool FAST>
__device__ __forceinline__ int32_t quant1(float v, const RowDivisor& d) {
    float r = FAST ? div_const(v, d.scale, d.rcp) : __fdiv_rn(v, d.scale);
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    return __float2int_rn(r);
}

// x / scale for two elements with the packed fp32 instructions (div_const, each half rounded like
// the scalar instruction), then round-to-nearest-even by adding 1.5 * 2^23: the sum's low mantissa
// bits are the two's-complement integer, rounded by the addition itself (ties to even), so no
// conversion instruction is needed.  |x| <= amax = 127 * scale up to rounding, so the quotient
// never reaches +-127.5 and the code stays within +-127, the clamp of the contract.  The low
// byte of each returned word is the int8 code.
__device__ __forceinline__ void quant2_fast(float x0, float x1, uint64_t rcp2, uint64_t neg_d2, int32_t& q0, int32_t& q1) {
    const uint64_t a = f32x2(x0, x1);
    const uint64_t d0 = mul_f32x2(a, rcp2);
    const uint64_t r0 = fma_f32x2(neg_d2, d0, a);
    const uint64_t d1 = fma_f32x2(r0, rcp2, d0);
    const uint64_t r1 = fma_f32x2(neg_d2, d1, a);
    const uint64_t q = fma_f32x2(r1, rcp2, d1);
    uint64_t m;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(m) : "l"(q), "l"(f32x2(12582912.0f, 12582912.0f)));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(q0), "=r"(q1) : "l"(m));
}

template <bool FAST>
__device__ __forceinline__ uint32_t pack4t(float4 v, const RowDivisor& d) {
    int32_t a, b, c, e;
    if (FAST) {
        const uint64_t rcp2 = f32x2(d.rcp, d.rcp), neg_d2 = f32x2(-d.scale, -d.scale);
        quant2_fast(v.x, v.y, rcp2, neg_d2, a, b);
        quant2_fast(v.z, v.w, rcp2, neg_d2, c, e);
    } else {
        a = quant1<false>(v.x, d); b = quant1<false>(v.y, d);
        c = quant1<false>(v.z, d); e = quant1<false>(v.w, d);
    }
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, e, 0x0040), 0x5410);
}
__device__ __forceinline__ uint32_t pack4(float4 v, const RowDivisor& d) {
    return d.fast ? pack4t<true>(v, d) : pack4t<false>(v, d);
}

// Scale of a row from its absolute maximum.
__device__ __forceinline__ float row_scale_from_amax(float amax) {
    const float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    return fmaxf(scale, 1.1754943508222875e-38f);
}

// RMSNorm in front of the quantizer (the reference's CPU operator, native/src/kernels/softmax_rmsnorm.inc:3-16):
// squares and their mean in double, inv = 1 / sqrt(mean + eps) in double, y = float((double(x) * inv) * double(gamma)).
__device__ __forceinline__ float norm1(float x, double inv, float g) {
    return __double2float_rn(__dmul_rn(__dmul_rn((double)x, inv), (double)g));
}
__device__ __forceinline__ float4 norm4(float4 c, double inv, float4 g) {
    return make_float4(norm1(c.x, inv, g.x), norm1(c.y, inv, g.y), norm1(c.z, inv, g.z), norm1(c.w, inv, g.w));
}
__device__ __forceinline__ double square_sum4(float4 c, double acc) {
    acc = __fma_rn((double)c.x, (double)c.x, acc);
    acc = __fma_rn((double)c.y, (double)c.y, acc);
    acc = __fma_rn((double)c.z, (double)c.z, acc);
    return __fma_rn((double)c.w, (double)c.w, acc);
}

}  // namespace vxb
