// K3: decode GEMV for rows <= 32 (HBM-bound: the int8 weights are streamed
// exactly once), and the one-thread-per-output verification kernel.
//
// Reference counterparts: the single-row route of vx_packed_linear_forward
// (native/src/kernels/packed_linear_ops.inc:1471-1535) and the CUDA decode
// kernels vx_packed_cuda_a8_columns / vx_cuda_qlinear_warp_dp4a_i8u8
// (native/src/backends/cuda/kernels/cuda_forward_llm_kernels.inc:254-459,
//  cuda_forward_quantized_basic_kernels.inc:49-104), which assign one warp (or
// eight lanes) per output and re-quantize the activation row per column tile.
// Here the activations are quantized once (K1), staged in shared memory, and
// every warp streams CH weight rows with 128-bit loads, reusing each
// activation register across the CH rows; integer partials are reduced with
// warp shuffles (integer addition is associative, so any order is bit-exact).
#include "common.cuh"

namespace vxb {

namespace {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr uint32_t kGemvSmemBytes = 96 * 1024;  // activation chunk budget

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
    return __dp4a((int)a, (int)b, c);
}

// MR activation rows (compile time), CH weight rows (output channels) per warp.
template <int MR, int CH>
__global__ void __launch_bounds__(kGemvThreads)
gemv_dp4a_kernel(const int8_t* __restrict__ q, uint32_t rows, const int8_t* __restrict__ w,
                 uint32_t n, uint32_t kpad, uint32_t kchunk, EpilogueParams epi) {
    extern __shared__ __align__(16) uint8_t smem[];  // [MR][kchunk] activations
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kChannelsPerCta = kGemvWarps * CH;
    const uint32_t blocks = (n + kChannelsPerCta - 1) / kChannelsPerCta;
    const bool single_chunk = kchunk >= kpad;

    for (uint32_t blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const uint32_t c0 = blk * kChannelsPerCta + warp * CH;
        int acc[MR][CH];
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) acc[m][c] = 0;

        for (uint32_t kb = 0; kb < kpad; kb += kchunk) {
            const uint32_t klen = kpad - kb < kchunk ? kpad - kb : kchunk;
            if (!(single_chunk && blk != blockIdx.x)) {
                // stage the activation chunk (zero rows beyond `rows`)
                __syncthreads();
                const uint32_t vec_per_row = klen / 16;
                for (uint32_t i = threadIdx.x; i < MR * vec_per_row; i += kGemvThreads) {
                    const uint32_t m = i / vec_per_row, v = i % vec_per_row;
                    uint4 val = make_uint4(0, 0, 0, 0);
                    if (m < rows) val = *reinterpret_cast<const uint4*>(q + (size_t)m * kpad + kb + v * 16);
                    *reinterpret_cast<uint4*>(smem + (size_t)m * kchunk + v * 16) = val;
                }
                __syncthreads();
            }
            // each lane owns 16 bytes of every 512-byte step
            for (uint32_t k0 = lane * 16; k0 < klen; k0 += 512) {
                uint4 wv[CH];
#pragma unroll
                for (int c = 0; c < CH; c++) {
                    const uint32_t ch = c0 + c;
                    wv[c] = ch < n ? __ldcs(reinterpret_cast<const uint4*>(w + (size_t)ch * kpad + kb + k0))
                                   : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    const uint4 a = *reinterpret_cast<const uint4*>(smem + (size_t)m * kchunk + k0);
#pragma unroll
                    for (int c = 0; c < CH; c++) {
                        int s = acc[m][c];
                        s = dp4a_s8(a.x, wv[c].x, s);
                        s = dp4a_s8(a.y, wv[c].y, s);
                        s = dp4a_s8(a.z, wv[c].z, s);
                        s = dp4a_s8(a.w, wv[c].w, s);
                        acc[m][c] = s;
                    }
                }
            }
        }
        // warp-shuffle reduction of the integer partials, then the fused epilogue
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) {
                int s = acc[m][c];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                acc[m][c] = s;
            }
        // lane (m*CH + c) % 32 writes element (m, c)
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) {
                if (lane == ((m * CH + c) & 31) && (uint32_t)m < rows && c0 + c < n)
                    epi_store(epi, m, c0 + c, acc[m][c]);
            }
    }
}

template <int MR, int CH>
cudaError_t launch_gemv_t(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n,
                          uint32_t kpad, const EpilogueParams& epi, int sm_count,
                          cudaStream_t stream) {
    const GemvShape shape = gemv_shape(0, rows, n, kpad, sm_count);
    if (shape.mr != (uint32_t)MR || shape.ch != (uint32_t)CH) return cudaErrorInvalidValue;
    cudaError_t e = ensure_dynamic_smem<gemv_dp4a_kernel<MR, CH>>(kGemvSmemBytes);
    if (e != cudaSuccess) return e;
    gemv_dp4a_kernel<MR, CH><<<shape.grid, kGemvThreads, shape.smem, stream>>>(q, rows, w, n, kpad, shape.kchunk, epi);
    return cudaGetLastError();
}

// ---- verification kernel: one thread per output element -------------------
__global__ void gemm_simt_kernel(const int8_t* __restrict__ q, uint32_t rows,
                                 const int8_t* __restrict__ w, uint32_t n, uint32_t kpad,
                                 EpilogueParams epi) {
    const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t row = blockIdx.y;
    if (col >= n || row >= rows) return;
    const uint32_t* a = reinterpret_cast<const uint32_t*>(q + (size_t)row * kpad);
    const uint32_t* b = reinterpret_cast<const uint32_t*>(w + (size_t)col * kpad);
    int acc = 0;
    for (uint32_t j = 0; j < kpad / 4; j++) acc = dp4a_s8(a[j], b[j], acc);
    epi_store(epi, row, col, acc);
}

// ---- grouped weight scales ---------------------------------------------------------------
// y[m,n] = (sum over groups g, ascending, of f32(dot_g) * f32(as[m] * ws[n,g])) + bias[n], every
// product and sum rounded on its own: the arithmetic of the reference's packed-linear column
// loop (native/src/kernels/packed_linear_ops.inc:1493-1531), which the tensor-core kernels
// cannot reproduce from one int32 accumulator per output. One thread per channel and MR
// token rows (each weight word is loaded once for the MR rows).
template <int MR>
__global__ void __launch_bounds__(128)
gemm_grouped_kernel(const int8_t* __restrict__ q, uint32_t rows, const int8_t* __restrict__ w,
                    uint32_t n, uint32_t kpad, EpilogueParams epi) {
    const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t row0 = blockIdx.y * MR;
    if (col >= n) return;
    const uint4* b = reinterpret_cast<const uint4*>(w + (size_t)col * kpad);
    const uint4* a[MR];
    float as[MR], sum[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) {
        const uint32_t r = row0 + m < rows ? row0 + m : rows - 1;
        a[m] = reinterpret_cast<const uint4*>(q + (size_t)r * kpad);
        as[m] = epi.row_scales[r];
        sum[m] = 0.0f;
    }
    const uint32_t gvec = epi.group / 16, kvec = kpad / 16;
    for (uint32_t g = 0, v0 = 0; g < epi.groups; g++, v0 += gvec) {
        const uint32_t v1 = v0 + gvec < kvec ? v0 + gvec : kvec;
        int dot[MR];
#pragma unroll
        for (int m = 0; m < MR; m++) dot[m] = 0;
        for (uint32_t v = v0; v < v1; v++) {
            const uint4 wv = __ldg(b + v);
#pragma unroll
            for (int m = 0; m < MR; m++) {
                const uint4 av = __ldg(a[m] + v);
                int s = dot[m];
                s = dp4a_s8(av.x, wv.x, s); s = dp4a_s8(av.y, wv.y, s);
                s = dp4a_s8(av.z, wv.z, s); s = dp4a_s8(av.w, wv.w, s);
                dot[m] = s;
            }
        }
        const float gs = __ldg(epi.gscales + (size_t)col * epi.groups + g);
#pragma unroll
        for (int m = 0; m < MR; m++)
            sum[m] = __fadd_rn(sum[m], __fmul_rn(__int2float_rn(dot[m]), __fmul_rn(as[m], gs)));
    }
    const float bias = epi.bias_f32 ? __ldg(epi.bias_f32 + col) : 0.0f;
#pragma unroll
    for (int m = 0; m < MR; m++)
        if (row0 + m < rows) ((float*)epi.out)[(size_t)(row0 + m) * epi.ld + col] = __fadd_rn(sum[m], bias);
}


// ---- grouped weight scales, few rows (decode) -------------------------------------------------
// The reference's own decode mode: one row against PackedLinear storage with a scale per
// G-element group.  Same streaming as gemv_dp4a_kernel (every warp reads CH weight rows with
// 128-bit loads, each lane 16 bytes of every 512-byte step, activations staged in shared memory),
// but the integer partials are reduced only within the G/16 lanes that share a group, and after
// every step the 512/G group dots go through the reference's arithmetic in ascending order:
//   sum = sum + f32(dot_g) * f32(as * ws[n,g])        (every operation rounded on its own)
// All lanes carry the same chain, so no lane diverges; int -> fp32 by the exact 1.5 * 2^23 trick.
template <int MR, int CH, int G>
__global__ void __launch_bounds__(kGemvThreads)
gemv_grouped_kernel(const int8_t* __restrict__ q, uint32_t rows, const int8_t* __restrict__ w,
                    uint32_t n, uint32_t kpad, uint32_t kchunk, EpilogueParams epi) {
    extern __shared__ __align__(16) uint8_t smem[];  // [MR][kchunk] activations
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kChannelsPerCta = kGemvWarps * CH;
    constexpr int kLanesPerGroup = G / 16, kGroupsPerStep = 512 / G;
    const uint32_t blocks = (n + kChannelsPerCta - 1) / kChannelsPerCta;
    const bool single_chunk = kchunk >= kpad;
    float as[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) as[m] = (uint32_t)m < rows ? __ldg(epi.row_scales + m) : 0.0f;

    for (uint32_t blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const uint32_t c0 = blk * kChannelsPerCta + warp * CH;
        float sum[MR][CH];
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) sum[m][c] = 0.0f;

        for (uint32_t kb = 0; kb < kpad; kb += kchunk) {
            const uint32_t klen = kpad - kb < kchunk ? kpad - kb : kchunk;
            if (!(single_chunk && blk != blockIdx.x)) {
                __syncthreads();
                const uint32_t vec_per_row = klen / 16;
                for (uint32_t i = threadIdx.x; i < MR * vec_per_row; i += kGemvThreads) {
                    const uint32_t m = i / vec_per_row, v = i % vec_per_row;
                    uint4 val = make_uint4(0, 0, 0, 0);
                    if (m < rows) val = *reinterpret_cast<const uint4*>(q + (size_t)m * kpad + kb + v * 16);
                    *reinterpret_cast<uint4*>(smem + (size_t)m * kchunk + v * 16) = val;
                }
                __syncthreads();
            }
            // the next step's weights are requested before this step's arithmetic: a warp's K loop is
            // otherwise a chain of load -> use round trips of a microsecond each
            uint4 wv[CH];
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const uint32_t ch = c0 + c;
                wv[c] = (lane * 16u < klen && ch < n) ? __ldcs(reinterpret_cast<const uint4*>(w + (size_t)ch * kpad + kb + lane * 16))
                                                      : make_uint4(0, 0, 0, 0);
            }
            for (uint32_t ks = 0; ks < klen; ks += 512) {
                const uint32_t k0 = ks + lane * 16;
                const bool in = k0 < klen;
                int part[MR][CH];
                uint4 wn[CH];
#pragma unroll
                for (int c = 0; c < CH; c++) {
                    const uint32_t ch = c0 + c;
                    wn[c] = (k0 + 512u < klen && ch < n) ? __ldcs(reinterpret_cast<const uint4*>(w + (size_t)ch * kpad + kb + k0 + 512u))
                                                         : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    const uint4 a = in ? *reinterpret_cast<const uint4*>(smem + (size_t)m * kchunk + k0) : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int c = 0; c < CH; c++) {
                        int s = dp4a_s8(a.x, wv[c].x, 0);
                        s = dp4a_s8(a.y, wv[c].y, s);
                        s = dp4a_s8(a.z, wv[c].z, s);
                        s = dp4a_s8(a.w, wv[c].w, s);
#pragma unroll
                        for (int off = kLanesPerGroup / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                        part[m][c] = s;
                    }
                }
                const uint32_t g0 = (kb + ks) / G;
#pragma unroll
                for (int j = 0; j < kGroupsPerStep; j++) {
                    if (g0 + j >= epi.groups) break;                       // uniform over the warp
#pragma unroll
                    for (int c = 0; c < CH; c++) {
                        const uint32_t ch = c0 + c < n ? c0 + c : n - 1;
                        const float gs = __ldg(epi.gscales + (size_t)ch * epi.groups + g0 + j);
#pragma unroll
                        for (int m = 0; m < MR; m++) {
                            const int d = __shfl_sync(0xffffffffu, part[m][c], j * kLanesPerGroup);
                            const float f = __fadd_rn(__int_as_float(d + 0x4B400000), -12582912.0f);
                            sum[m][c] = __fadd_rn(sum[m][c], __fmul_rn(f, __fmul_rn(as[m], gs)));
                        }
                    }
                }
#pragma unroll
                for (int c = 0; c < CH; c++) wv[c] = wn[c];
            }
        }
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) {
                if (lane == ((m * CH + c) & 31) && (uint32_t)m < rows && c0 + c < n) {
                    const float bias = epi.bias_f32 ? __ldg(epi.bias_f32 + c0 + c) : 0.0f;
                    ((float*)epi.out)[(size_t)m * epi.ld + c0 + c] = __fadd_rn(sum[m][c], bias);
                }
            }
    }
}

template <int MR, int CH, int G>
cudaError_t launch_gemv_grouped_t(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                                  const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    const GemvShape shape = gemv_shape(1, rows, n, kpad, sm_count);
    if (shape.mr != (uint32_t)MR || shape.ch != (uint32_t)CH) return cudaErrorInvalidValue;
    cudaError_t e = ensure_dynamic_smem<gemv_grouped_kernel<MR, CH, G>>(kGemvSmemBytes);
    if (e != cudaSuccess) return e;
    gemv_grouped_kernel<MR, CH, G><<<shape.grid, kGemvThreads, shape.smem, stream>>>(q, rows, w, n, kpad, shape.kchunk, epi);
    return cudaGetLastError();
}

template <int G>
cudaError_t launch_gemv_grouped_g(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                                  const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    if (rows <= 1) return launch_gemv_grouped_t<1, 4, G>(q, rows, w, n, kpad, epi, sm_count, stream);
    if (rows <= 2) return launch_gemv_grouped_t<2, 4, G>(q, rows, w, n, kpad, epi, sm_count, stream);
    return launch_gemv_grouped_t<4, 2, G>(q, rows, w, n, kpad, epi, sm_count, stream);
}


// ---- W4 storage, grouped scales, one or two rows ----------------------------------------------
// The same decode kernel over the 4-bit words themselves (half the weight bytes of the int8
// copy): eight codes per word, earlier K in lower bits, w = code - 8 (the reference's
// vx_packed_cuda_unpack_w4_low/high, cuda_forward_llm_kernels.inc:152-165).  A word's low nibbles
// are codes 0,2,4,6 and its high nibbles codes 1,3,5,7, so the activations are staged in shared
// memory de-interleaved per 8 (even four, odd four) and a word costs two masks, a shift and two
// dp4a; sum a * (c - 8) = sum a * c - 8 * sum a, with sum a taken once per row and step.
// Each lane owns 16 bytes = 32 codes of every 1024-code step; G / 32 lanes share a group.
template <int MR, int CH, int G>
__global__ void __launch_bounds__(kGemvThreads)
gemv_w4_grouped_kernel(const int8_t* __restrict__ q, uint32_t rows, const uint32_t* __restrict__ w4,
                       uint32_t row_words, uint32_t n, uint32_t kpad, uint32_t kchunk, EpilogueParams epi) {
    extern __shared__ __align__(16) uint8_t smem[];  // [MR][kchunk] de-interleaved activations
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr uint32_t kChannelsPerCta = kGemvWarps * CH;
    constexpr int kLanesPerGroup = G / 32, kGroupsPerStep = 1024 / G;
    const uint32_t blocks = (n + kChannelsPerCta - 1) / kChannelsPerCta;
    const bool single_chunk = kchunk >= kpad;
    float as[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) as[m] = (uint32_t)m < rows ? __ldg(epi.row_scales + m) : 0.0f;

    for (uint32_t blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
        const uint32_t c0 = blk * kChannelsPerCta + warp * CH;
        float sum[MR][CH];
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) sum[m][c] = 0.0f;

        for (uint32_t kb = 0; kb < kpad; kb += kchunk) {
            const uint32_t klen = kpad - kb < kchunk ? kpad - kb : kchunk;
            if (!(single_chunk && blk != blockIdx.x)) {
                __syncthreads();
                const uint32_t vec_per_row = klen / 16;
                for (uint32_t i = threadIdx.x; i < MR * vec_per_row; i += kGemvThreads) {
                    const uint32_t m = i / vec_per_row, v = i % vec_per_row;
                    uint4 val = make_uint4(0, 0, 0, 0);
                    if (m < rows) val = *reinterpret_cast<const uint4*>(q + (size_t)m * kpad + kb + v * 16);
                    const uint4 perm = make_uint4(__byte_perm(val.x, val.y, 0x6420), __byte_perm(val.x, val.y, 0x7531),
                                                  __byte_perm(val.z, val.w, 0x6420), __byte_perm(val.z, val.w, 0x7531));
                    *reinterpret_cast<uint4*>(smem + (size_t)m * kchunk + v * 16) = perm;
                }
                __syncthreads();
            }
            const uint4 kZero4 = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
            uint4 wv[CH];
#pragma unroll
            for (int c = 0; c < CH; c++) {
                const uint32_t ch = c0 + c;
                wv[c] = (lane * 32u < klen && ch < n) ? __ldcs(reinterpret_cast<const uint4*>(w4 + (size_t)ch * row_words + (kb + lane * 32u) / 8))
                                                      : kZero4;
            }
            for (uint32_t ks = 0; ks < klen; ks += 1024) {
                const uint32_t k0 = ks + lane * 32;                  // this lane's first code of the step
                const bool in = k0 < klen;
                uint4 wn[CH];
#pragma unroll
                for (int c = 0; c < CH; c++) {
                    const uint32_t ch = c0 + c;
                    wn[c] = (k0 + 1024u < klen && ch < n) ? __ldcs(reinterpret_cast<const uint4*>(w4 + (size_t)ch * row_words + (kb + k0 + 1024u) / 8))
                                                          : kZero4;
                }
                int part[MR][CH];
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                    if (in) {
                        a0 = *reinterpret_cast<const uint4*>(smem + (size_t)m * kchunk + k0);
                        a1 = *reinterpret_cast<const uint4*>(smem + (size_t)m * kchunk + k0 + 16);
                    }
                    const uint32_t av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};   // (even, odd) per word
                    int asum = 0;
#pragma unroll
                    for (int i = 0; i < 8; i++) asum = dp4a_s8(av[i], 0x01010101u, asum);
#pragma unroll
                    for (int c = 0; c < CH; c++) {
                        const uint32_t wd[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
                        int s = 0;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            s = dp4a_s8(av[2 * i], wd[i] & 0x0F0F0F0Fu, s);
                            s = dp4a_s8(av[2 * i + 1], (wd[i] >> 4) & 0x0F0F0F0Fu, s);
                        }
                        s -= 8 * asum;
#pragma unroll
                        for (int off = kLanesPerGroup / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                        part[m][c] = s;
                    }
                }
                const uint32_t g0 = (kb + ks) / G;
#pragma unroll
                for (int j = 0; j < kGroupsPerStep; j++) {
                    if (g0 + j >= epi.groups) break;                       // uniform over the warp
#pragma unroll
                    for (int c = 0; c < CH; c++) {
                        const uint32_t ch = c0 + c < n ? c0 + c : n - 1;
                        const float gs = __ldg(epi.gscales + (size_t)ch * epi.groups + g0 + j);
#pragma unroll
                        for (int m = 0; m < MR; m++) {
                            const int d = __shfl_sync(0xffffffffu, part[m][c], j * kLanesPerGroup);
                            const float f = __fadd_rn(__int_as_float(d + 0x4B400000), -12582912.0f);
                            sum[m][c] = __fadd_rn(sum[m][c], __fmul_rn(f, __fmul_rn(as[m], gs)));
                        }
                    }
                }
#pragma unroll
                for (int c = 0; c < CH; c++) wv[c] = wn[c];
            }
        }
#pragma unroll
        for (int m = 0; m < MR; m++)
#pragma unroll
            for (int c = 0; c < CH; c++) {
                if (lane == ((m * CH + c) & 31) && (uint32_t)m < rows && c0 + c < n) {
                    const float bias = epi.bias_f32 ? __ldg(epi.bias_f32 + c0 + c) : 0.0f;
                    ((float*)epi.out)[(size_t)m * epi.ld + c0 + c] = __fadd_rn(sum[m][c], bias);
                }
            }
    }
}

template <int MR, int CH, int G>
cudaError_t launch_gemv_w4_t(const int8_t* q, uint32_t rows, const uint32_t* w4, uint32_t row_words, uint32_t n,
                             uint32_t kpad, const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    const GemvShape shape = gemv_shape(2, rows, n, kpad, sm_count);
    if (shape.mr != (uint32_t)MR || shape.ch != (uint32_t)CH) return cudaErrorInvalidValue;
    cudaError_t e = ensure_dynamic_smem<gemv_w4_grouped_kernel<MR, CH, G>>(kGemvSmemBytes);
    if (e != cudaSuccess) return e;
    gemv_w4_grouped_kernel<MR, CH, G><<<shape.grid, kGemvThreads, shape.smem, stream>>>(q, rows, w4, row_words, n, kpad, shape.kchunk, epi);
    return cudaGetLastError();
}

template <int G>
cudaError_t launch_gemv_w4_g(const int8_t* q, uint32_t rows, const uint32_t* w4, uint32_t row_words, uint32_t n,
                             uint32_t kpad, const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    if (rows <= 1) return launch_gemv_w4_t<1, 4, G>(q, rows, w4, row_words, n, kpad, epi, sm_count, stream);
    return launch_gemv_w4_t<2, 4, G>(q, rows, w4, row_words, n, kpad, epi, sm_count, stream);
}

}  // namespace

GemvShape gemv_shape(int kind, uint32_t rows, uint32_t n, uint32_t kpad, int sm_count) {
    GemvShape s{};
    // rows per CTA pass (compile-time MR) and channels per warp (CH)
    if (kind == 0) {
        s.mr = rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : rows <= 8 ? 8 : rows <= 16 ? 16 : 32;
        s.ch = s.mr <= 4 ? 4 : s.mr <= 16 ? 2 : 1;
    } else if (kind == 1) {
        s.mr = rows <= 1 ? 1 : rows <= 2 ? 2 : 4;
        s.ch = s.mr <= 2 ? 4 : 2;
    } else {
        s.mr = rows <= 1 ? 1 : 2;
        s.ch = 4;
    }
    // K chunk staged in shared memory: whole (rounded) K when mr * K fits the budget, else the
    // largest multiple of the kernel's step that does
    const uint32_t step = kind == 2 ? 1024u : 512u;
    s.kchunk = kind == 0 ? kpad : (kpad + step - 1) / step * step;
    if ((uint64_t)s.mr * s.kchunk > kGemvSmemBytes) s.kchunk = (kGemvSmemBytes / s.mr) / step * step;
    s.smem = s.mr * s.kchunk;
    const uint32_t per_cta = (uint32_t)kGemvWarps * s.ch;
    const uint32_t blocks = (n + per_cta - 1) / per_cta;
    uint32_t per_sm = s.smem ? (200u * 1024u) / (s.smem + 1024u) : 8u;
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    s.grid = (uint32_t)sm_count * per_sm;
    if (s.grid > blocks) s.grid = blocks;
    return s;
}

cudaError_t launch_gemm_grouped(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                                const EpilogueParams& epi, cudaStream_t stream) {
    if (rows == 0 || n == 0) return cudaSuccess;
    if (epi.mode != kEpiF32 || !epi.gscales || epi.group % 16 != 0 || !epi.groups) return cudaErrorInvalidValue;
    constexpr int kMR = 4;
    for (uint32_t r0 = 0; r0 < rows; r0 += 65535u * kMR) {
        const uint32_t cnt = rows - r0 < 65535u * kMR ? rows - r0 : 65535u * kMR;
        EpilogueParams e = epi;
        e.row_scales = epi.row_scales + r0;
        e.out = (uint8_t*)epi.out + (size_t)r0 * epi.ld * 4;
        dim3 grid((n + 127) / 128, (cnt + kMR - 1) / kMR);
        if (cnt == 1) gemm_grouped_kernel<1><<<dim3(grid.x, 1), 128, 0, stream>>>(q + (size_t)r0 * kpad, cnt, w, n, kpad, e);
        else gemm_grouped_kernel<kMR><<<grid, 128, 0, stream>>>(q + (size_t)r0 * kpad, cnt, w, n, kpad, e);
    }
    return cudaGetLastError();
}

cudaError_t launch_gemv_grouped(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                                const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    if (rows == 0 || n == 0) return cudaSuccess;
    if (rows > 4 || epi.mode != kEpiF32 || !epi.gscales || !epi.groups) return cudaErrorInvalidValue;
    switch (epi.group) {
        case 32: return launch_gemv_grouped_g<32>(q, rows, w, n, kpad, epi, sm_count, stream);
        case 64: return launch_gemv_grouped_g<64>(q, rows, w, n, kpad, epi, sm_count, stream);
        case 128: return launch_gemv_grouped_g<128>(q, rows, w, n, kpad, epi, sm_count, stream);
        case 256: return launch_gemv_grouped_g<256>(q, rows, w, n, kpad, epi, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemv_w4_grouped(const int8_t* q, uint32_t rows, const uint32_t* w4, uint32_t row_words, uint32_t n,
                                   uint32_t kpad, const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    if (rows == 0 || n == 0) return cudaSuccess;
    if (rows > 2 || epi.mode != kEpiF32 || !epi.gscales || !epi.groups || row_words % 4 != 0 || row_words * 8 < kpad)
        return cudaErrorInvalidValue;
    switch (epi.group) {
        case 32: return launch_gemv_w4_g<32>(q, rows, w4, row_words, n, kpad, epi, sm_count, stream);
        case 64: return launch_gemv_w4_g<64>(q, rows, w4, row_words, n, kpad, epi, sm_count, stream);
        case 128: return launch_gemv_w4_g<128>(q, rows, w4, row_words, n, kpad, epi, sm_count, stream);
        case 256: return launch_gemv_w4_g<256>(q, rows, w4, row_words, n, kpad, epi, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemv(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                        const EpilogueParams& epi, int sm_count, cudaStream_t stream) {
    if (rows == 0 || n == 0) return cudaSuccess;
    if (rows > 32) return cudaErrorInvalidValue;
    if (rows <= 1) return launch_gemv_t<1, 4>(q, rows, w, n, kpad, epi, sm_count, stream);
    if (rows <= 2) return launch_gemv_t<2, 4>(q, rows, w, n, kpad, epi, sm_count, stream);
    if (rows <= 4) return launch_gemv_t<4, 4>(q, rows, w, n, kpad, epi, sm_count, stream);
    if (rows <= 8) return launch_gemv_t<8, 2>(q, rows, w, n, kpad, epi, sm_count, stream);
    if (rows <= 16) return launch_gemv_t<16, 2>(q, rows, w, n, kpad, epi, sm_count, stream);
    return launch_gemv_t<32, 1>(q, rows, w, n, kpad, epi, sm_count, stream);
}

cudaError_t launch_gemm_simt(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n,
                             uint32_t kpad, const EpilogueParams& epi, cudaStream_t stream) {
    if (rows == 0 || n == 0) return cudaSuccess;
    for (uint32_t r0 = 0; r0 < rows; r0 += 65535u) {
        const uint32_t cnt = rows - r0 < 65535u ? rows - r0 : 65535u;
        EpilogueParams e = epi;
        // shift row-indexed pointers for the slab
        e.row_scales = epi.row_scales ? epi.row_scales + r0 : nullptr;
        const size_t elem = epi.mode == kEpiI8 ? 1 : 4;
        e.out = (uint8_t*)epi.out + (size_t)r0 * epi.ld * elem;
        dim3 grid((n + 127) / 128, cnt);
        gemm_simt_kernel<<<grid, 128, 0, stream>>>(q + (size_t)r0 * kpad, cnt, w, n, kpad, e);
    }
    return cudaGetLastError();
}

}  // namespace vxb
