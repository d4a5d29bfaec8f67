// K1: per-token symmetric int8 quantizer, plus the small layout helpers
// (weight repack, zero-point folding, byte copies).  HBM-bound byte work:
// 128-bit loads, 128-bit stores, one pass over the fp32 activations.
//
// Arithmetic contract (reference: native/src/kernels/packed_linear_ops.inc
// :97-153 AVX2, :1574-1597 scalar; CUDA twin cuda_forward_llm_kernels.inc
// :195-247):
//   row invalid if any element has an all-ones exponent (NaN/Inf)
//   amax  = max |x|;  scale = amax == 0 ? 1 : amax / 127  (IEEE divide)
//   scale = max(scale, 2^-126)
//   q     = cvt.rni(clamp(x / scale, -127, 127))            (IEEE divide, ties to even)
// A reciprocal-multiply would move half-way values across a rounding
// boundary, so the divide is __fdiv_rn on every element.
#include "quantize.cuh"
#include <cooperative_groups.h>

namespace vxb {

namespace {

constexpr int kThreads = 256;
constexpr int kMaxVecPerThread = 8;   // float4 per thread kept in registers (K <= 8192)
constexpr uint32_t kClusterMaxRows = 32;   // up to this many rows a cluster of CTAs shares each row

// Reduce (max, or-flag) over THREADS_PER_ROW consecutive threads (power of two).
template <int THREADS_PER_ROW>
__device__ __forceinline__ void row_reduce(float& amax, int& bad, float* smem_max, int* smem_bad) {
    constexpr int kWarpSpan = THREADS_PER_ROW < 32 ? THREADS_PER_ROW : 32;
#pragma unroll
    for (int off = kWarpSpan / 2; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        bad |= __shfl_xor_sync(0xffffffffu, bad, off);
    }
    if constexpr (THREADS_PER_ROW > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) { smem_max[warp] = amax; smem_bad[warp] = bad; }
        __syncthreads();
        constexpr int kWarps = THREADS_PER_ROW / 32;
        const int first = (threadIdx.x / THREADS_PER_ROW) * kWarps;  // this row's first warp
        float m = 0.0f; int b = 0;
#pragma unroll
        for (int i = 0; i < kWarps; i++) { m = fmaxf(m, smem_max[first + i]); b |= smem_bad[first + i]; }
        amax = m; bad = b;
    }
}

// THREADS_PER_ROW threads cooperate on one row; kThreads/THREADS_PER_ROW rows per CTA.
// VEC: row addressed as float4 (k % 4 == 0, 16-byte aligned base and ldq % 16 == 0).
// CACHE: the row's float4s stay in registers between the two passes.
template <int THREADS_PER_ROW, bool CACHE>
__global__ void __launch_bounds__(kThreads)
quantize_rows_vec(const float* __restrict__ x, uint32_t rows, uint32_t k, int8_t* __restrict__ q,
                  uint32_t ldq, float* __restrict__ row_scales, int32_t* __restrict__ valid) {
    __shared__ float smem_max[kThreads / 32];
    __shared__ int smem_bad[kThreads / 32];
    // let the consumer kernel start its prologue and weight prefetch now; then wait until the
    // kernel before this one has finished with the activations and the q scratch
    pdl_release();
    pdl_wait();
    constexpr int kRowsPerCta = kThreads / THREADS_PER_ROW;
    const uint32_t row = blockIdx.x * kRowsPerCta + threadIdx.x / THREADS_PER_ROW;
    const int t = threadIdx.x % THREADS_PER_ROW;
    const bool active = row < rows;
    const uint32_t nvec = k / 4;
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(active ? row : 0) * k);

    float4 cache[CACHE ? kMaxVecPerThread : 1];
    float amax = 0.0f; int bad = 0;
    if (active) {
        if constexpr (CACHE) {
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) {
                const uint32_t v = t + i * THREADS_PER_ROW;
                cache[i] = v < nvec ? __ldg(in + v) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) {
                const float4 c = cache[i];
                bad |= nonfinite_bits(c.x) | nonfinite_bits(c.y) | nonfinite_bits(c.z) | nonfinite_bits(c.w);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))));
            }
        } else {
            for (uint32_t v = t; v < nvec; v += THREADS_PER_ROW) {
                const float4 c = __ldg(in + v);
                bad |= nonfinite_bits(c.x) | nonfinite_bits(c.y) | nonfinite_bits(c.z) | nonfinite_bits(c.w);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))));
            }
        }
    }
    row_reduce<THREADS_PER_ROW>(amax, bad, smem_max, smem_bad);
    if (!active) return;

    float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    scale = fmaxf(scale, 1.1754943508222875e-38f);
    if (t == 0) {
        row_scales[row] = bad ? __int_as_float(0x7fc00000) : scale;
        if (valid) valid[row] = bad ? 0 : 1;
    }
    uint32_t* out = reinterpret_cast<uint32_t*>(q + (size_t)row * ldq);
    const uint32_t nwords = ldq / 4;
    const RowDivisor div(scale);
    if constexpr (CACHE) {
        if (div.fast && !bad) {
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) {
                const uint32_t v = t + i * THREADS_PER_ROW;
                if (v < nwords) out[v] = v < nvec ? pack4t<true>(cache[i], div) : 0u;
            }
        } else {
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) {
                const uint32_t v = t + i * THREADS_PER_ROW;
                if (v < nwords) out[v] = (v < nvec && !bad) ? pack4t<false>(cache[i], div) : 0u;
            }
        }
        for (uint32_t v = t + kMaxVecPerThread * THREADS_PER_ROW; v < nwords; v += THREADS_PER_ROW) out[v] = 0u;
    } else {
        for (uint32_t v = t; v < nwords; v += THREADS_PER_ROW)
            out[v] = (v < nvec && !bad) ? pack4(__ldg(in + v), div) : 0u;
    }
}

// Few rows (decode): one row per CTA leaves most of the GPU idle and makes the kernel a chain of
// dependent loads. Here a thread-block cluster of S CTAs shares a row: each CTA keeps its K/S
// slice in registers (at most 8 float4 per thread), the S partial (absmax, non-finite) pairs
// are exchanged through distributed shared memory, and every CTA quantizes its own slice.
// grid = (S, rows), cluster = (S, 1, 1). max and OR are exact in any order, so the result is
// bit-identical to the one-CTA kernel.
template <int S>
__global__ void __launch_bounds__(kThreads)
quantize_rows_cluster(const float* __restrict__ x, uint32_t rows, uint32_t k, int8_t* __restrict__ q,
                      uint32_t ldq, float* __restrict__ row_scales, int32_t* __restrict__ valid) {
    namespace cg = cooperative_groups;
    __shared__ float smem_max[kThreads / 32];
    __shared__ int smem_bad[kThreads / 32];
    __shared__ float peer_max[S];
    __shared__ int peer_bad[S];
    pdl_release();
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank();
    const uint32_t row = blockIdx.y;
    const uint32_t nvec = k / 4, nwords = ldq / 4;
    const uint32_t seg = (nwords + S - 1) / S;                 // words (= float4s) of this CTA's slice
    const uint32_t w0 = rank * seg;
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)row * k);

    float4 cache[kMaxVecPerThread];
    float amax = 0.0f; int bad = 0;
#pragma unroll
    for (int i = 0; i < kMaxVecPerThread; i++) {
        const uint32_t o = threadIdx.x + i * kThreads, v = w0 + o;
        cache[i] = (o < seg && v < nvec) ? __ldg(in + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < kMaxVecPerThread; i++) {
        const float4 c = cache[i];
        bad |= nonfinite_bits(c.x) | nonfinite_bits(c.y) | nonfinite_bits(c.z) | nonfinite_bits(c.w);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))));
    }
    row_reduce<kThreads>(amax, bad, smem_max, smem_bad);
    if (threadIdx.x < S) {
        // thread p publishes this CTA's pair in CTA p's table
        *cluster.map_shared_rank(&peer_max[rank], threadIdx.x) = amax;
        *cluster.map_shared_rank(&peer_bad[rank], threadIdx.x) = bad;
    }
    cluster.sync();
    amax = 0.0f; bad = 0;
#pragma unroll
    for (int p = 0; p < S; p++) { amax = fmaxf(amax, peer_max[p]); bad |= peer_bad[p]; }

    float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    scale = fmaxf(scale, 1.1754943508222875e-38f);
    if (rank == 0 && threadIdx.x == 0) {
        row_scales[row] = bad ? __int_as_float(0x7fc00000) : scale;
        if (valid) valid[row] = bad ? 0 : 1;
    }
    uint32_t* out = reinterpret_cast<uint32_t*>(q + (size_t)row * ldq);
    const RowDivisor div(scale);
    const bool fast = div.fast && !bad;
#pragma unroll
    for (int i = 0; i < kMaxVecPerThread; i++) {
        const uint32_t o = threadIdx.x + i * kThreads, v = w0 + o;
        if (o < seg && v < nwords)
            out[v] = (v < nvec && !bad) ? (fast ? pack4t<true>(cache[i], div) : pack4t<false>(cache[i], div)) : 0u;
    }
}

template <int S>
cudaError_t launch_cluster(const float* x, uint32_t rows, uint32_t k, int8_t* q, uint32_t ldq,
                           float* row_scales, int32_t* valid, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, rows); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, quantize_rows_cluster<S>, x, rows, k, q, ldq, row_scales, valid);
}

// Any k / alignment: one warp per row, scalar accesses.
__global__ void __launch_bounds__(kThreads)
quantize_rows_scalar(const float* __restrict__ x, uint32_t rows, uint32_t k, int8_t* __restrict__ q,
                     uint32_t ldq, float* __restrict__ row_scales, int32_t* __restrict__ valid) {
    pdl_release();
    pdl_wait();
    const uint32_t row = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* in = x + (size_t)row * k;
    float amax = 0.0f; int bad = 0;
    for (uint32_t j = lane; j < k; j += 32) {
        const float v = in[j];
        bad |= nonfinite_bits(v);
        amax = fmaxf(amax, fabsf(v));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        bad |= __shfl_xor_sync(0xffffffffu, bad, off);
    }
    float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    scale = fmaxf(scale, 1.1754943508222875e-38f);
    if (lane == 0) {
        row_scales[row] = bad ? __int_as_float(0x7fc00000) : scale;
        if (valid) valid[row] = bad ? 0 : 1;
    }
    int8_t* out = q + (size_t)row * ldq;
    const RowDivisor div(scale);
    for (uint32_t j = lane; j < ldq; j += 32)
        out[j] = (j < k && !bad) ? (int8_t)quant1<false>(in[j], div) : (int8_t)0;
}

__global__ void fill_f32_kernel(float* dst, uint32_t count, float value) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) dst[i] = value;
}

__global__ void fold_zero_point_kernel(const int32_t* bias, const int32_t* wsum, int32_t zero,
                                       int32_t* out, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (bias ? bias[i] : 0) - zero * wsum[i];
}

__global__ void copy_bytes_padded_kernel(const uint8_t* __restrict__ src, uint32_t rows, uint32_t k,
                                         uint8_t* __restrict__ dst, uint32_t ld, uint32_t xor_mask) {
    const uint32_t row = blockIdx.y;
    for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < ld; j += gridDim.x * blockDim.x)
        dst[(size_t)row * ld + j] = j < k ? (uint8_t)(src[(size_t)row * k + j] ^ xor_mask) : (uint8_t)0;
}

// One warp per weight row: copy (with optional ^0x80), zero the padding, sum the codes.
__global__ void __launch_bounds__(kThreads)
repack_weight_kernel(const uint8_t* __restrict__ src, uint32_t src_ld, uint32_t n, uint32_t k,
                     uint32_t xor_mask, int8_t* __restrict__ dst, uint32_t kpad,
                     int32_t* __restrict__ wsum) {
    const uint32_t row = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n) return;
    const uint8_t* in = src + (size_t)row * src_ld;
    int8_t* out = dst + (size_t)row * kpad;
    int32_t sum = 0;
    for (uint32_t j = lane; j < kpad; j += 32) {
        const int8_t v = j < k ? (int8_t)(in[j] ^ xor_mask) : (int8_t)0;
        out[j] = v;
        sum += v;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) wsum[row] = sum;
}

template <int TPR>
cudaError_t launch_vec(const float* x, uint32_t rows, uint32_t k, int8_t* q, uint32_t ldq,
                       float* row_scales, int32_t* valid, cudaStream_t stream) {
    constexpr int kRowsPerCta = kThreads / TPR;
    const uint32_t grid = (rows + kRowsPerCta - 1) / kRowsPerCta;
    if (k / 4 <= (uint32_t)TPR * kMaxVecPerThread)
        return launch_pdl(quantize_rows_vec<TPR, true>, dim3(grid), dim3(kThreads), 0, stream,
                          x, rows, k, q, ldq, row_scales, valid);
    return launch_pdl(quantize_rows_vec<TPR, false>, dim3(grid), dim3(kThreads), 0, stream,
                      x, rows, k, q, ldq, row_scales, valid);
}


// ---- RMSNorm folded into the quantizer --------------------------------------------------------
// The decode and prefill patterns RMSNorm -> {q,k,v} and RMSNorm -> {gate,up} read the residual
// stream once: normalize, (optionally) persist the normalized row for other consumers, quantize.
// Arithmetic of the normalization follows the reference's CPU operator
// (native/src/kernels/softmax_rmsnorm.inc:3-16): squares and their mean in double,
// inv = 1 / sqrt(mean + eps) in double, y = float((double(x) * inv) * double(gamma)).  The squares
// are exact in double; only the order of the double additions differs from the sequential loop
// (tree instead of left to right), which moves the mean by at most a few units of 2^-53.

template <int THREADS_PER_ROW>
__device__ __forceinline__ double row_sum(double v, double* smem_sum) {
    constexpr int kWarpSpan = THREADS_PER_ROW < 32 ? THREADS_PER_ROW : 32;
#pragma unroll
    for (int off = kWarpSpan / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if constexpr (THREADS_PER_ROW > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) smem_sum[warp] = v;
        __syncthreads();
        constexpr int kWarps = THREADS_PER_ROW / 32;
        const int first = (threadIdx.x / THREADS_PER_ROW) * kWarps;
        double s = 0.0;
#pragma unroll
        for (int i = 0; i < kWarps; i++) s += smem_sum[first + i];
        v = s;
    }
    return v;
}

template <int THREADS_PER_ROW, bool CACHE>
__global__ void __launch_bounds__(kThreads)
rmsnorm_quantize_rows_vec(const float* __restrict__ x, const float* __restrict__ gamma, double eps,
                          uint32_t rows, uint32_t k, float* __restrict__ norm_out, int8_t* __restrict__ q,
                          uint32_t ldq, float* __restrict__ row_scales, int32_t* __restrict__ valid) {
    __shared__ float smem_max[kThreads / 32];
    __shared__ int smem_bad[kThreads / 32];
    __shared__ double smem_sum[kThreads / 32];
    pdl_release();
    pdl_wait();
    constexpr int kRowsPerCta = kThreads / THREADS_PER_ROW;
    const uint32_t row = blockIdx.x * kRowsPerCta + threadIdx.x / THREADS_PER_ROW;
    const int t = threadIdx.x % THREADS_PER_ROW;
    const bool active = row < rows;
    const uint32_t nvec = k / 4;
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(active ? row : 0) * k);
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    float4* nout = norm_out ? reinterpret_cast<float4*>(norm_out + (size_t)(active ? row : 0) * k) : nullptr;

    float4 cache[CACHE ? kMaxVecPerThread : 1];
    double ss = 0.0;
    if (active) {
        if constexpr (CACHE) {
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) {
                const uint32_t v = t + i * THREADS_PER_ROW;
                cache[i] = v < nvec ? __ldg(in + v) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) ss = square_sum4(cache[i], ss);
        } else {
            for (uint32_t v = t; v < nvec; v += THREADS_PER_ROW) ss = square_sum4(__ldg(in + v), ss);
        }
    }
    ss = row_sum<THREADS_PER_ROW>(ss, smem_sum);
    // one thread per row does the double-precision division and square root (slow, shared units); the others
    // take the result from shared memory
    __shared__ double smem_inv[kThreads / 8];
    if (t == 0) smem_inv[threadIdx.x / THREADS_PER_ROW] = 1.0 / sqrt(ss / (double)k + eps);
    if constexpr (THREADS_PER_ROW > 32) __syncthreads(); else __syncwarp();
    const double inv = smem_inv[threadIdx.x / THREADS_PER_ROW];

    float amax = 0.0f; int bad = 0;
    if (active) {
        if constexpr (CACHE) {
#pragma unroll
            for (int i = 0; i < kMaxVecPerThread; i++) {
                const uint32_t v = t + i * THREADS_PER_ROW;
                if (v < nvec) {
                    const float4 c = norm4(cache[i], inv, __ldg(g4 + v));
                    cache[i] = c;
                    if (nout) nout[v] = c;
                    bad |= nonfinite_bits(c.x) | nonfinite_bits(c.y) | nonfinite_bits(c.z) | nonfinite_bits(c.w);
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))));
                }
            }
        } else {
            for (uint32_t v = t; v < nvec; v += THREADS_PER_ROW) {
                const float4 c = norm4(__ldg(in + v), inv, __ldg(g4 + v));
                if (nout) nout[v] = c;
                bad |= nonfinite_bits(c.x) | nonfinite_bits(c.y) | nonfinite_bits(c.z) | nonfinite_bits(c.w);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w))));
            }
        }
    }
    row_reduce<THREADS_PER_ROW>(amax, bad, smem_max, smem_bad);
    if (!active) return;

    float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    scale = fmaxf(scale, 1.1754943508222875e-38f);
    if (t == 0) {
        row_scales[row] = bad ? __int_as_float(0x7fc00000) : scale;
        if (valid) valid[row] = bad ? 0 : 1;
    }
    uint32_t* out = reinterpret_cast<uint32_t*>(q + (size_t)row * ldq);
    const uint32_t nwords = ldq / 4;
    const RowDivisor div(scale);
    if constexpr (CACHE) {
        const bool fast = div.fast && !bad;
#pragma unroll
        for (int i = 0; i < kMaxVecPerThread; i++) {
            const uint32_t v = t + i * THREADS_PER_ROW;
            if (v < nwords)
                out[v] = (v < nvec && !bad) ? (fast ? pack4t<true>(cache[i], div) : pack4t<false>(cache[i], div)) : 0u;
        }
        for (uint32_t v = t + kMaxVecPerThread * THREADS_PER_ROW; v < nwords; v += THREADS_PER_ROW) out[v] = 0u;
    } else {
        for (uint32_t v = t; v < nwords; v += THREADS_PER_ROW)
            out[v] = (v < nvec && !bad) ? pack4(norm4(__ldg(in + v), inv, __ldg(g4 + v)), div) : 0u;
    }
}

// Any k / alignment: one warp per row, scalar accesses, the row is read three times.
__global__ void __launch_bounds__(kThreads)
rmsnorm_quantize_rows_scalar(const float* __restrict__ x, const float* __restrict__ gamma, double eps,
                             uint32_t rows, uint32_t k, float* __restrict__ norm_out, int8_t* __restrict__ q,
                             uint32_t ldq, float* __restrict__ row_scales, int32_t* __restrict__ valid) {
    pdl_release();
    pdl_wait();
    const uint32_t row = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* in = x + (size_t)row * k;
    double ss = 0.0;
    for (uint32_t j = lane; j < k; j += 32) ss = __fma_rn((double)in[j], (double)in[j], ss);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const double inv = 1.0 / sqrt(ss / (double)k + eps);
    float amax = 0.0f; int bad = 0;
    for (uint32_t j = lane; j < k; j += 32) {
        const float v = norm1(in[j], inv, gamma[j]);
        if (norm_out) norm_out[(size_t)row * k + j] = v;
        bad |= nonfinite_bits(v);
        amax = fmaxf(amax, fabsf(v));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        bad |= __shfl_xor_sync(0xffffffffu, bad, off);
    }
    float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 127.0f);
    scale = fmaxf(scale, 1.1754943508222875e-38f);
    if (lane == 0) {
        row_scales[row] = bad ? __int_as_float(0x7fc00000) : scale;
        if (valid) valid[row] = bad ? 0 : 1;
    }
    int8_t* out = q + (size_t)row * ldq;
    const RowDivisor div(scale);
    for (uint32_t j = lane; j < ldq; j += 32)
        out[j] = (j < k && !bad) ? (int8_t)quant1<false>(norm1(in[j], inv, gamma[j]), div) : (int8_t)0;
}

template <int TPR>
cudaError_t launch_norm_vec(const float* x, const float* gamma, double eps, uint32_t rows, uint32_t k,
                            float* norm_out, int8_t* q, uint32_t ldq, float* row_scales, int32_t* valid,
                            cudaStream_t stream) {
    constexpr int kRowsPerCta = kThreads / TPR;
    const uint32_t grid = (rows + kRowsPerCta - 1) / kRowsPerCta;
    if (k / 4 <= (uint32_t)TPR * kMaxVecPerThread)
        return launch_pdl(rmsnorm_quantize_rows_vec<TPR, true>, dim3(grid), dim3(kThreads), 0, stream,
                          x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid);
    return launch_pdl(rmsnorm_quantize_rows_vec<TPR, false>, dim3(grid), dim3(kThreads), 0, stream,
                      x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid);
}

}  // namespace

cudaError_t launch_quantize_rows(const float* x, uint32_t rows, uint32_t k, int8_t* q, uint32_t ldq,
                                 float* row_scales, int32_t* valid, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const bool vec = (k % 4 == 0) && (ldq % 4 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)q % 4 == 0);
    if (!vec) {
        const uint32_t grid = (rows + kThreads / 32 - 1) / (kThreads / 32);
        return launch_pdl(quantize_rows_scalar, dim3(grid), dim3(kThreads), 0, stream,
                          x, rows, k, q, ldq, row_scales, valid);
    }
    // Few long rows: a cluster of 2..8 CTAs per row (each thread then holds one or two float4)
    if (rows <= kClusterMaxRows && ldq / 4 >= 2u * kThreads && ldq / 4 <= 8u * kThreads * kMaxVecPerThread) {
        const uint32_t per = (ldq / 4 + kThreads - 1) / kThreads;   // float4 per thread with one CTA
        if (per >= 8) return launch_cluster<8>(x, rows, k, q, ldq, row_scales, valid, stream);
        if (per >= 4) return launch_cluster<4>(x, rows, k, q, ldq, row_scales, valid, stream);
        return launch_cluster<2>(x, rows, k, q, ldq, row_scales, valid, stream);
    }
    // Threads per row grow with K so each thread keeps at most 8 float4 in registers.
    if (k <= 256) return launch_vec<8>(x, rows, k, q, ldq, row_scales, valid, stream);
    if (k <= 1024) return launch_vec<32>(x, rows, k, q, ldq, row_scales, valid, stream);
    if (k <= 2048) return launch_vec<64>(x, rows, k, q, ldq, row_scales, valid, stream);
    if (k <= 4096) return launch_vec<128>(x, rows, k, q, ldq, row_scales, valid, stream);
    return launch_vec<256>(x, rows, k, q, ldq, row_scales, valid, stream);
}

cudaError_t launch_rmsnorm_quantize_rows(const float* x, const float* gamma, float epsilon, uint32_t rows,
                                         uint32_t k, float* norm_out, int8_t* q, uint32_t ldq,
                                         float* row_scales, int32_t* valid, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const double eps = (double)epsilon;
    const bool vec = (k % 4 == 0) && (ldq % 4 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)gamma % 16 == 0) &&
                     ((uintptr_t)norm_out % 16 == 0) && ((uintptr_t)q % 4 == 0);
    if (!vec) {
        const uint32_t grid = (rows + kThreads / 32 - 1) / (kThreads / 32);
        return launch_pdl(rmsnorm_quantize_rows_scalar, dim3(grid), dim3(kThreads), 0, stream,
                          x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid);
    }
    if (k <= 256) return launch_norm_vec<8>(x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid, stream);
    if (k <= 1024) return launch_norm_vec<32>(x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid, stream);
    if (k <= 2048) return launch_norm_vec<64>(x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid, stream);
    if (k <= 4096) return launch_norm_vec<128>(x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid, stream);
    return launch_norm_vec<256>(x, gamma, eps, rows, k, norm_out, q, ldq, row_scales, valid, stream);
}

cudaError_t launch_fill_f32(float* dst, uint32_t count, float value, cudaStream_t stream) {
    if (!count) return cudaSuccess;
    fill_f32_kernel<<<(count + 255) / 256, 256, 0, stream>>>(dst, count, value);
    return cudaGetLastError();
}

cudaError_t launch_fold_zero_point(const int32_t* bias, const int32_t* wsum, int32_t input_zero,
                                   int32_t* out, uint32_t n, cudaStream_t stream) {
    if (!n) return cudaSuccess;
    fold_zero_point_kernel<<<(n + 255) / 256, 256, 0, stream>>>(bias, wsum, input_zero, out, n);
    return cudaGetLastError();
}

cudaError_t launch_copy_bytes_padded(const uint8_t* src, uint32_t rows, uint32_t k, uint8_t* dst,
                                     uint32_t ld, uint32_t xor_mask, cudaStream_t stream) {
    if (!rows) return cudaSuccess;
    dim3 grid((ld + 1023) / 1024 < 8 ? (ld + 1023) / 1024 : 8, rows);
    // grid.y is limited to 65535: larger row counts go in slabs
    for (uint32_t r0 = 0; r0 < rows; r0 += 65535u) {
        const uint32_t cnt = rows - r0 < 65535u ? rows - r0 : 65535u;
        grid.y = cnt;
        copy_bytes_padded_kernel<<<grid, 256, 0, stream>>>(src + (size_t)r0 * k, cnt, k,
                                                            dst + (size_t)r0 * ld, ld, xor_mask);
    }
    return cudaGetLastError();
}

cudaError_t launch_repack_weight(const uint8_t* src, uint32_t src_ld, uint32_t n, uint32_t k,
                                 uint32_t xor_mask, int8_t* dst, uint32_t kpad, int32_t* wsum,
                                 cudaStream_t stream) {
    if (!n) return cudaSuccess;
    const uint32_t grid = (n + kThreads / 32 - 1) / (kThreads / 32);
    repack_weight_kernel<<<grid, kThreads, 0, stream>>>(src, src_ld, n, k, xor_mask, dst, kpad, wsum);
    return cudaGetLastError();
}

}  // namespace vxb
