// K2g: the int8 GEMM for weights whose scales differ between the K groups of a channel
// (PackedLinear storage with G = 32 / 64 / 128 / 256), on the tensor cores.
//
//   y[m,n] = (sum over groups g, ascending, of f32(dot_g[m,n]) * f32(as[m] * ws[n,g])) + bias[n]
//
// every product and every sum rounded on its own: the arithmetic of the reference's column loop
// (native/src/kernels/packed_linear_ops.inc:1493-1531; CUDA twin vx_packed_cuda_a8_tile,
// native/src/backends/cuda/kernels/cuda_forward_llm_kernels.inc:693-883).  One int32 accumulator
// per output cannot reproduce the per-group rounding, so the accumulator is drained once per
// group: the MMA-issuing thread gives every group a fresh 128-column TMEM accumulator (four of
// them rotate), and the epilogue warps read it, convert, scale and add into fp32 running sums
// that stay in registers for the whole K loop.
//
//   warp 0      TMA producers: lane 0 the activation tile (128 rows x 128 B per stage), lane 1
//               the weight tile (128 channels x 128 B)
//   warp 1      allocates TMEM; one lane issues tcgen05.mma.cta_group::1.kind::i8
//               (M128 x N128 x K32), G/32 instructions per group
//   warps 2-9   drain: two warps per TMEM lane quarter, 64 columns each (sixteen warps of 32
//               columns were 1.6x slower: barrier, fence and bias-store overhead is per warp)
//
// int32 -> fp32 without a conversion instruction: |dot_g| <= 256 * 127 * 128 < 2^22, so
// as_float(dot + 0x4B400000) - 1.5 * 2^23 is the exact value, and the addition of 0x4B400000 is
// done by the tensor core (the accumulators start from that bit pattern instead of zero).
// Every wait on an mbarrier is bounded; on expiry the kernel raises a status word, drains,
// frees its TMEM and returns.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kBM = 128, kBN = 128, kBK = 128;
constexpr uint32_t kStages = 6;
constexpr uint32_t kABytes = kBM * kBK, kBBytes = kBN * kBK, kStageBytes = kABytes + kBBytes;
constexpr uint32_t kAccBufs = 4, kAccCols = kBN, kTmemCols = 512;
constexpr uint32_t kEpiWarps = 8, kEpiCols = kBN * 4 / kEpiWarps;   // two warps per TMEM lane quarter (sixteen were 1.6x slower: the per-group barrier and store overhead is per warp)
constexpr uint32_t kChunks = kEpiCols / 32, kGsLanes = kEpiCols / 4;
constexpr uint32_t kThreads = 64 + 32 * kEpiWarps;
constexpr uint32_t kEndWarp = 2 + kEpiWarps;

constexpr uint32_t kOffStages = 0;
constexpr uint32_t kOffGs = kStages * kStageBytes;                  // float[8 warps][64] group scales
constexpr uint32_t kOffBias = kOffGs + kEpiWarps * kEpiCols * 4;    // float[8 warps][64]
constexpr uint32_t kOffStore = kOffBias + kEpiWarps * kEpiCols * 4; // [8 warps][16 rows x 128 B]
constexpr uint32_t kStoreBytes = 16 * 128;
constexpr uint32_t kOffBars = kOffStore + kEpiWarps * kStoreBytes;
constexpr uint32_t kNumBars = 2 * kStages + 2 * kAccBufs;
constexpr uint32_t kOffTmemPtr = kOffBars + kNumBars * 8;
constexpr uint32_t kOffAbort = kOffTmemPtr + 4;
constexpr uint32_t kSmemBytes = kOffAbort + 8 + 1024;

struct Smem {
    uint8_t* base;
    __device__ uint32_t a(uint32_t s) const { return smem_u32(base + kOffStages + s * kStageBytes); }
    __device__ uint32_t b(uint32_t s) const { return a(s) + kABytes; }
    __device__ uint32_t full(uint32_t s) const { return smem_u32(base + kOffBars + s * 8); }
    __device__ uint32_t empty(uint32_t s) const { return smem_u32(base + kOffBars + (kStages + s) * 8); }
    __device__ uint32_t tmem_full(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + b) * 8); }
    __device__ uint32_t tmem_empty(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + kAccBufs + b) * 8); }
    __device__ uint32_t* tmem_ptr() const { return reinterpret_cast<uint32_t*>(base + kOffTmemPtr); }
    __device__ volatile int* abort_flag() const { return reinterpret_cast<volatile int*>(base + kOffAbort); }
};

// The accumulators are never zeroed: before every use the drain warps store the bit pattern of
// 1.5 * 2^23 into them and the MMAs accumulate on top, so what comes back is 0x4B400000 + dot,
// which read as fp32 is 12582912 + dot exactly (|dot| < 2^22).  One fp32 subtraction finishes the
// int -> float conversion; no conversion instruction and no integer addition per element.
constexpr uint32_t kBiasBits = 0x4B400000u;
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&c)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4]), "r"(c[5]), "r"(c[6]), "r"(c[7]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// eight registers holding the bias serve all stores of a warp's column slice
__device__ __forceinline__ void bias_slice(uint32_t taddr, const uint32_t (&c)[8]) {
#pragma unroll
    for (uint32_t i = 0; i < kEpiCols / 8u; i++) tmem_st8(taddr + 8u * i, c);
}

// sum += f32(dot) * (as * gs), every operation rounded on its own: four fp32-pipe instructions
// per element (packed f32x2 forms of the same arithmetic were no faster here)
__device__ __forceinline__ void drain1(uint32_t biased, float as, float g, float& s) {
    const float f = __fadd_rn(__uint_as_float(biased), -12582912.0f);
    s = __fadd_rn(s, __fmul_rn(f, __fmul_rn(as, g)));
}

template <uint32_t MPG>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_grouped_tcgen05_kernel(const __grid_constant__ GemmGroupedArgs args) {
    extern __shared__ uint8_t smem_raw[];
    Smem sm;
    sm.base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t tiles_m = (args.rows + kBM - 1) / kBM;
    const uint32_t tiles_n = (args.n + kBN - 1) / kBN;
    const uint32_t total_tiles = tiles_m * tiles_n;
    constexpr uint32_t mpg = MPG;                                // MMAs per group (group size / 32)
    const uint32_t all_ks = args.kpad / 32u;
    const uint32_t total_ks = all_ks < args.groups * mpg ? all_ks : args.groups * mpg;
    const uint32_t num_kb = (total_ks + 3u) / 4u;                // stages per tile
    volatile int* abort_flag = sm.abort_flag();

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) { mbar_init(sm.full(s), 1); mbar_init(sm.empty(s), 1); }
        for (uint32_t b = 0; b < kAccBufs; b++) { mbar_init(sm.tmem_full(b), 1); mbar_init(sm.tmem_empty(b), kEpiWarps); }
        arm_abort(abort_flag, args.status);
        fence_barrier_init();
        prefetch_tmap(&args.tmap_a);
        prefetch_tmap(&args.tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(sm.tmem_ptr()), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_ptr();

    if (warp == 0) {
        // ---------------- TMA producers: lane 0 the activation tile, lane 1 the weight tile ----------------
        if (lane < 2) {
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int32_t m0 = (int32_t)((t % tiles_m) * kBM), n0 = (int32_t)((t / tiles_m) * kBN);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    if (lane == 0) {
                        mbar_expect_tx(sm.full(stage), kStageBytes);
                        tma_load_2d(sm.a(stage), &args.tmap_a, sm.full(stage), (int32_t)(kb * kBK), m0);
                    } else {
                        tma_load_2d(sm.b(stage), &args.tmap_b, sm.full(stage), (int32_t)(kb * kBK), n0);
                    }
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && lane == 0) {
                // drain: give this CTA's own copies in flight a bounded time to land
                for (uint32_t s = 0; s < kStages; s++) {
                    if (!(armed & (1u << s))) continue;
                    for (uint32_t i = 0; i < 2000; i++) {
                        if (mbar_try_wait(sm.full(s), (armed_parity >> s) & 1u)) break;
                        __nanosleep(500);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kBM, kBN);
            uint32_t stage = 0, phase = 0, buf = 0, buf_phase = 0;
            bool ok = true;
            // everything the thread does between two MMAs is idle time of the tensor pipe, and it
            // shares its scheduler with two drain warps that never pause: where a group starts
            // and ends is a compile-time fact (MPG = MMAs per group), barrier addresses and
            // descriptor low words advance by constants
            const uint32_t a_lo0 = smem_desc_lo(sm.a(0));
            uint32_t full_s = sm.full(0), empty_s = sm.empty(0), a_lo = a_lo0;
            uint32_t tfull = sm.tmem_full(0), tempty = sm.tmem_empty(0), d_tmem = tmem_base;
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                for (uint32_t kb = 0; ok && kb < num_kb; kb++) {
                    if (!mbar_try_wait(full_s, phase) && !mbar_wait(full_s, phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (uint32_t j = 0; j < 4; j++) {
                        if (MPG < 4 && kb * 4u + j >= total_ks) break;
                        const bool first = MPG >= 8 ? (j == 0 && !(kb & 1u)) : (j % MPG == 0);
                        const bool last = MPG >= 8 ? (j == 3 && ((kb & 1u) || kb + 1 == num_kb)) : (j % MPG == MPG - 1);
                        if (first) {
                            // the next accumulator, once the drain warps have read its previous contents
                            // and stored the conversion bias into it (phase 0: the fill at kernel start)
                            if (!mbar_try_wait(tempty, buf_phase) && !mbar_wait(tempty, buf_phase, abort_flag)) { ok = false; break; }
                            tc_fence_after();
                        }
                        umma_i8_lo(d_tmem, a_lo + 2u * j, a_lo + (kABytes >> 4) + 2u * j, idesc);
                        if (last) {
                            umma_commit(tfull);
                            tfull += 8; tempty += 8; d_tmem += kAccCols;
                            if (++buf == kAccBufs) { buf = 0; buf_phase ^= 1u; tfull = sm.tmem_full(0); tempty = sm.tmem_empty(0); d_tmem = tmem_base; }
                        }
                    }
                    if (!ok) break;
                    umma_commit(empty_s);
                    full_s += 8; empty_s += 8; a_lo += kStageBytes >> 4;
                    if (++stage == kStages) { stage = 0; phase ^= 1u; full_s = sm.full(0); empty_s = sm.empty(0); a_lo = a_lo0; }
                }
            }
        }
    } else if (warp < kEndWarp) {
        // ---------------- drain and epilogue (warps 2..9) ----------------
        const uint32_t quarter = warp & 3u;              // TMEM lanes [32*quarter, +32)
        const uint32_t cbase = ((warp - 2u) >> 2) * kEpiCols;   // columns [cbase, +64) of the tile
        float* s_gs = reinterpret_cast<float*>(sm.base + kOffGs) + (warp - 2u) * kEpiCols;
        float* s_bias = reinterpret_cast<float*>(sm.base + kOffBias) + (warp - 2u) * kEpiCols;
        uint8_t* stage_store = sm.base + kOffStore + (warp - 2u) * kStoreBytes;
        uint32_t buf = 0, buf_phase = 0;
        bool ok = true;
        // fill this warp's part of all four accumulators with the conversion bias
        uint32_t bias_regs[8];
#pragma unroll
        for (int i = 0; i < 8; i++) asm volatile("mov.u32 %0, %1;" : "=r"(bias_regs[i]) : "n"(kBiasBits));   // opaque: one block of registers, not one per store
        for (uint32_t b = 0; b < kAccBufs; b++) bias_slice(tmem_base + ((quarter * 32u) << 16) + b * kAccCols + cbase, bias_regs);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
            for (uint32_t b = 0; b < kAccBufs; b++) mbar_arrive(sm.tmem_empty(b));
        for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
            const uint32_t m0 = (t % tiles_m) * kBM, n0 = (t / tiles_m) * kBN + cbase;
            const uint32_t row = m0 + quarter * 32 + lane;
            const bool row_ok = row < args.rows;
            const float as = row_ok ? __ldg(args.row_scales + row) : 0.0f;
            __syncwarp();
            for (uint32_t i = lane; i < kEpiCols; i += 32) {
                const uint32_t n = n0 + i;
                s_bias[i] = (n < args.n && args.bias) ? __ldg(args.bias + n) : 0.0f;
            }
            float sum[kEpiCols];
#pragma unroll
            for (uint32_t i = 0; i < kEpiCols; i++) sum[i] = 0.0f;
            // this warp's 64 scales of a group are 256 contiguous bytes of the transposed table
            const float4* gs4 = reinterpret_cast<const float4*>(args.gscales_t + n0) + lane;
            const uint32_t gstride4 = args.n_pad / 4u;
            const bool live = m0 + quarter * 32u < args.rows && n0 < args.n;
            float4 pre = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live && lane < kGsLanes) pre = __ldg(gs4);
#pragma unroll 1
            for (uint32_t g = 0; g < args.groups; g++) {
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + buf * kAccCols + cbase;
                if (!live) {
                    // none of this warp's 32 rows or 64 columns exists (few rows: decode): keep the
                    // barrier protocol and the bias of its accumulator slice, skip the arithmetic
                    ok = __all_sync(0xffffffffu, mbar_wait(sm.tmem_full(buf), buf_phase, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    bias_slice(taddr, bias_regs);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sm.tmem_empty(buf));
                    if (++buf == kAccBufs) { buf = 0; buf_phase ^= 1u; }
                    continue;
                }
                __syncwarp();
                if (lane < kGsLanes) reinterpret_cast<float4*>(s_gs)[lane] = pre;
                __syncwarp();
                if (lane < kGsLanes && g + 1 < args.groups) pre = __ldg(gs4 + (size_t)(g + 1) * gstride4);
                ok = __all_sync(0xffffffffu, mbar_wait(sm.tmem_full(buf), buf_phase, abort_flag));
                if (!ok) break;
                tc_fence_after();
                const float4* g4 = reinterpret_cast<const float4*>(s_gs);
                uint32_t r[32];
#pragma unroll
                for (uint32_t ch = 0; ch < kChunks; ch++) {
                    tmem_ld32(taddr + 32u * ch, r);
                    tmem_ld_wait();
                    if (ch == kChunks - 1) {
                        // the accumulator is free again as soon as it is in registers and holds the bias
                        bias_slice(taddr, bias_regs);
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(sm.tmem_empty(buf));
                        if (++buf == kAccBufs) { buf = 0; buf_phase ^= 1u; }
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float4 gv = g4[8 * ch + j];
                        drain1(r[4 * j + 0], as, gv.x, sum[32 * ch + 4 * j + 0]);
                        drain1(r[4 * j + 1], as, gv.y, sum[32 * ch + 4 * j + 1]);
                        drain1(r[4 * j + 2], as, gv.z, sum[32 * ch + 4 * j + 2]);
                        drain1(r[4 * j + 3], as, gv.w, sum[32 * ch + 4 * j + 3]);
                    }
                }
            }
            if (!ok) break;
            // + bias, then whole 128-byte row segments through shared memory (16 rows at a time,
            // 16-byte pieces XOR-swizzled by row)
#pragma unroll
            for (uint32_t c = 0; c < kEpiCols; c += 32) {
                const uint32_t col = n0 + c;
                if (col >= args.n) continue;
                uint32_t o[32];
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__fadd_rn(sum[c + i], s_bias[c + i]));
#pragma unroll
                for (uint32_t half16 = 0; half16 < 2; half16++) {
                    __syncwarp();
                    if ((lane >> 4) == half16) {
                        uint8_t* mine = stage_store + (lane & 15u) * 128u;
#pragma unroll
                        for (uint32_t j = 0; j < 8; j++)
                            *reinterpret_cast<uint4*>(mine + ((j ^ (lane & 7u)) << 4)) =
                                make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    }
                    __syncwarp();
                    const uint32_t piece = lane & 7u;
#pragma unroll
                    for (uint32_t i = 0; i < 4; i++) {
                        const uint32_t rl = 4u * i + (lane >> 3);
                        const uint4 v = *reinterpret_cast<const uint4*>(stage_store + rl * 128u + ((piece ^ (rl & 7u)) << 4));
                        const uint32_t grow = m0 + quarter * 32u + half16 * 16u + rl, gcol = col + piece * 4u;
                        if (grow >= args.rows || gcol >= args.n) continue;
                        uint32_t* dst = (uint32_t*)args.out + (size_t)grow * args.ld + gcol;
                        if (gcol + 4u <= args.n && (((uintptr_t)dst) & 15u) == 0) {
                            *reinterpret_cast<uint4*>(dst) = v;
                        } else {
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (uint32_t e = 0; e < 4; e++)
                                if (gcol + e < args.n) dst[e] = w[e];
                        }
                    }
                }
            }
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        nap(200);
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 1);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

cudaError_t gemm_grouped_tcgen05_prepare() {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_grouped_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_grouped_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_grouped_tcgen05_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_grouped_tcgen05_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    return e;
}

cudaError_t launch_gemm_grouped_tcgen05(const GemmGroupedArgs& args, int sm_count, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    if (!args.groups || args.n_pad % kBN != 0 || args.n_pad < args.n || args.kpad % kBK != 0) return cudaErrorInvalidValue;
    const uint32_t tiles = ((args.rows + kBM - 1) / kBM) * ((args.n + kBN - 1) / kBN);
    const uint32_t grid = tiles < (uint32_t)sm_count ? tiles : (uint32_t)sm_count;
    switch (args.group) {
        case 32: gemm_i8_grouped_tcgen05_kernel<1><<<grid, kThreads, kSmemBytes, stream>>>(args); break;
        case 64: gemm_i8_grouped_tcgen05_kernel<2><<<grid, kThreads, kSmemBytes, stream>>>(args); break;
        case 128: gemm_i8_grouped_tcgen05_kernel<4><<<grid, kThreads, kSmemBytes, stream>>>(args); break;
        case 256: gemm_i8_grouped_tcgen05_kernel<8><<<grid, kThreads, kSmemBytes, stream>>>(args); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace vxb
