// The F32 <-> byte boundary of a static W8A8 island and the byte-to-byte bridge between two
// quantized domains: QuantizeLinear, DequantizeLinear, RequantizeLinear. HBM-bound elementwise
// work: 16 elements per thread, 128-bit accesses where the pointers allow.
//
// Arithmetic (CPU authority of the reference, restated in oracle/w8a8_oracle.c):
//   quantize    NaN -> zero point; t = f32(x / scale) + f32(zero); saturate; ties to even
//               (native/src/kernels/quantize_linear_ops.inc:155-170, 230-254)
//   dequantize  f32((x - zero) * scale), one rounding (:9-16, 95-122)
//   requantize  t = f32(f32(x - in_zero) * f32(in_scale / out_scale)) + f32(out_zero); NaN -> out
//               zero point; saturate; ties to even (portable_inference_kernels.inc:2437-2463)
// CUDA twins in the reference: vx_cuda_quantize_i8u8, vx_cuda_dequantize_i8u8,
// vx_cuda_requantize_i8u8 (native/src/backends/cuda/kernels/
// cuda_forward_quantized_basic_kernels.inc:163-193), one element per thread.
#include "common.cuh"

namespace vxb {

namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 16;

__device__ __forceinline__ int32_t load_byte(const uint8_t* p, bool is_unsigned) {
    return is_unsigned ? (int32_t)*p : (int32_t)*reinterpret_cast<const int8_t*>(p);
}
__device__ __forceinline__ int32_t byte_of(uint32_t word, int i, bool is_unsigned) {
    const uint32_t b = (word >> (8 * i)) & 0xffu;
    return is_unsigned ? (int32_t)b : (int32_t)(int8_t)b;
}

__device__ __forceinline__ int32_t quantize1(float v, float scale, float zero_f, int32_t zero, float lo_f,
                                             float hi_f, int32_t lo, int32_t hi) {
    if (v != v) return zero;
    const float t = __fadd_rn(__fdiv_rn(v, scale), zero_f);
    if (t <= lo_f) return lo;
    if (t >= hi_f) return hi;
    return __float2int_rn(t);   // finite and inside the range here: round to nearest even
}
__device__ __forceinline__ int32_t requantize1(int32_t x, int32_t in_zero, float multiplier, float zero_f,
                                               int32_t zero, float lo_f, float hi_f, int32_t lo, int32_t hi) {
    const float t = __fadd_rn(__fmul_rn(__int2float_rn(x - in_zero), multiplier), zero_f);
    if (t != t) return zero;
    if (t <= lo_f) return lo;
    if (t >= hi_f) return hi;
    return __float2int_rn(t);
}

__global__ void __launch_bounds__(kThreads)
quantize_linear_kernel(const float* __restrict__ x, unsigned long long n, float scale, int32_t zero, int32_t lo,
                       int32_t hi, uint8_t* __restrict__ out, int vec) {
    const float zero_f = __int2float_rn(zero), lo_f = __int2float_rn(lo), hi_f = __int2float_rn(hi);
    const unsigned long long base = ((unsigned long long)blockIdx.x * kThreads + threadIdx.x) * kPerThread;
    if (base >= n) return;
    if (vec && base + kPerThread <= n) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(x + base) + j);
            const int32_t a = quantize1(v.x, scale, zero_f, zero, lo_f, hi_f, lo, hi);
            const int32_t b = quantize1(v.y, scale, zero_f, zero, lo_f, hi_f, lo, hi);
            const int32_t c = quantize1(v.z, scale, zero_f, zero, lo_f, hi_f, lo, hi);
            const int32_t d = quantize1(v.w, scale, zero_f, zero, lo_f, hi_f, lo, hi);
            w[j] = __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
        }
        *reinterpret_cast<uint4*>(out + base) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        for (unsigned long long i = base; i < n && i < base + kPerThread; i++)
            out[i] = (uint8_t)quantize1(x[i], scale, zero_f, zero, lo_f, hi_f, lo, hi);
    }
}

__global__ void __launch_bounds__(kThreads)
dequantize_linear_kernel(const uint8_t* __restrict__ x, unsigned long long n, float scale, int32_t zero,
                         int is_unsigned, float* __restrict__ out, int vec) {
    const unsigned long long base = ((unsigned long long)blockIdx.x * kThreads + threadIdx.x) * kPerThread;
    if (base >= n) return;
    if (vec && base + kPerThread <= n) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + base));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float4 o;
            o.x = __fmul_rn(__int2float_rn(byte_of(w[j], 0, is_unsigned) - zero), scale);
            o.y = __fmul_rn(__int2float_rn(byte_of(w[j], 1, is_unsigned) - zero), scale);
            o.z = __fmul_rn(__int2float_rn(byte_of(w[j], 2, is_unsigned) - zero), scale);
            o.w = __fmul_rn(__int2float_rn(byte_of(w[j], 3, is_unsigned) - zero), scale);
            reinterpret_cast<float4*>(out + base)[j] = o;
        }
    } else {
        for (unsigned long long i = base; i < n && i < base + kPerThread; i++)
            out[i] = __fmul_rn(__int2float_rn(load_byte(x + i, is_unsigned) - zero), scale);
    }
}

__global__ void __launch_bounds__(kThreads)
requantize_linear_kernel(const uint8_t* __restrict__ x, unsigned long long n, float multiplier, int32_t in_zero,
                         int in_unsigned, int32_t zero, int32_t lo, int32_t hi, uint8_t* __restrict__ out, int vec) {
    const float zero_f = __int2float_rn(zero), lo_f = __int2float_rn(lo), hi_f = __int2float_rn(hi);
    const unsigned long long base = ((unsigned long long)blockIdx.x * kThreads + threadIdx.x) * kPerThread;
    if (base >= n) return;
    if (vec && base + kPerThread <= n) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + base));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int32_t a = requantize1(byte_of(w[j], 0, in_unsigned), in_zero, multiplier, zero_f, zero, lo_f, hi_f, lo, hi);
            const int32_t b = requantize1(byte_of(w[j], 1, in_unsigned), in_zero, multiplier, zero_f, zero, lo_f, hi_f, lo, hi);
            const int32_t c = requantize1(byte_of(w[j], 2, in_unsigned), in_zero, multiplier, zero_f, zero, lo_f, hi_f, lo, hi);
            const int32_t d = requantize1(byte_of(w[j], 3, in_unsigned), in_zero, multiplier, zero_f, zero, lo_f, hi_f, lo, hi);
            o[j] = __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
        }
        *reinterpret_cast<uint4*>(out + base) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        for (unsigned long long i = base; i < n && i < base + kPerThread; i++)
            out[i] = (uint8_t)requantize1(load_byte(x + i, in_unsigned), in_zero, multiplier, zero_f, zero, lo_f, hi_f, lo, hi);
    }
}

inline unsigned int grid_for(unsigned long long n) {
    return (unsigned int)((n + (unsigned long long)kThreads * kPerThread - 1) / ((unsigned long long)kThreads * kPerThread));
}
inline int aligned16(const void* a, const void* b) { return (((uintptr_t)a | (uintptr_t)b) & 15u) == 0 ? 1 : 0; }

}  // namespace

cudaError_t launch_quantize_linear(const float* x, unsigned long long n, float scale, int32_t zero, bool out_unsigned,
                                   void* out, cudaStream_t stream) {
    if (!n) return cudaSuccess;
    quantize_linear_kernel<<<grid_for(n), kThreads, 0, stream>>>(x, n, scale, zero, out_unsigned ? 0 : -128,
                                                                out_unsigned ? 255 : 127, (uint8_t*)out, aligned16(x, out));
    return cudaGetLastError();
}

cudaError_t launch_dequantize_linear(const void* x, unsigned long long n, float scale, int32_t zero, bool in_unsigned,
                                     float* out, cudaStream_t stream) {
    if (!n) return cudaSuccess;
    dequantize_linear_kernel<<<grid_for(n), kThreads, 0, stream>>>((const uint8_t*)x, n, scale, zero, in_unsigned ? 1 : 0,
                                                                  out, aligned16(x, out));
    return cudaGetLastError();
}

cudaError_t launch_requantize_linear(const void* x, unsigned long long n, float multiplier, int32_t in_zero,
                                     bool in_unsigned, int32_t out_zero, bool out_unsigned, void* out,
                                     cudaStream_t stream) {
    if (!n) return cudaSuccess;
    requantize_linear_kernel<<<grid_for(n), kThreads, 0, stream>>>((const uint8_t*)x, n, multiplier, in_zero,
                                                                  in_unsigned ? 1 : 0, out_zero, out_unsigned ? 0 : -128,
                                                                  out_unsigned ? 255 : 127, (uint8_t*)out, aligned16(x, out));
    return cudaGetLastError();
}

}  // namespace vxb
