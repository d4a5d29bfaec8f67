// K2w: the int8 GEMM for 32-BIT OUTPUTS (fp32 after dequantization + bias (+ residual), or the raw
// int32 accumulators), built for the shapes where the output, not the tensor pipe, bounds the launch:
// prefill of small models (K of a few hundred to a few thousand) writes 4 bytes per output against
// K / 2048 microseconds-per-tile of MMA work.
//
//   y[m,n] = f32(f32(acc[m,n]) * f32(as[m] * ws[n])) + bias[n] (+ residual[m,n]),   acc = sum_k q[m,k] * w[n,k]
//
// What differs from the general kernel (gemm_tcgen05.cu), and why (B200 time stamps of that kernel at
// M 4096, K 576, N 3072: 1.8 us of operand loading per 128 x 256 tile against a 4.6 us epilogue):
//   * SIXTEEN epilogue warps, four per TMEM lane quarter, 64 columns each: four warps per scheduler
//     instead of two hide the TMEM-load, conversion (one int32 -> fp32 conversion per output on the XU
//     pipe, 16 per clock and SM: ~1 us per tile by itself) and shared-memory latencies that eight warps
//     left exposed, and a CTA with a single tile finishes it in half the time.
//   * The finished 32 x 32 chunk goes to global memory as ONE TMA tile store per warp: each lane writes
//     its 128-byte row into a 128B-swizzled [32 rows x 128 B] staging tile, one lane issues
//     cp.async.bulk.tensor (shared -> global, clipped by the tensor map at the matrix edges, no
//     multicast), and the warp goes on with the next chunk while the store drains.
//   * Three 48 KB pipeline stages instead of four: the fourth stage's room is the sixteen staging tiles.
//   * 96 registers per thread (608 threads), which only this epilogue fits in; the requantizing
//     epilogues stay in the general kernel.
// Launched with programmatic dependent launch: barriers, TMEM and the first weight tiles are set up
// while the launch before it drains; the activation producer and the epilogue warps wait for it.
//
// Every wait on an mbarrier is bounded; on expiry the kernel raises the status word, drains, frees its
// TMEM and returns.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kBM = 128, kBN = 256, kBK = 128;
constexpr uint32_t kStages = 3;
constexpr uint32_t kABytes = kBM * kBK, kBBytes = kBN * kBK, kStageBytes = kABytes + kBBytes;
constexpr uint32_t kAccCols = kBN, kTmemCols = 512;
constexpr uint32_t kEpiWarps = 16;
constexpr uint32_t kBWarp = 2 + kEpiWarps;
constexpr uint32_t kThreads = 32 * (kBWarp + 1);
constexpr uint32_t kEpiCols = kBN / 4;          // columns per epilogue warp
constexpr uint32_t kTileBytes = 32 * 128;       // one staging tile: 32 rows x 32 32-bit columns

constexpr uint32_t kOffStages = 0;
constexpr uint32_t kOffTiles = kStages * kStageBytes;                 // [16 warps][4 KB], 1024-byte aligned
constexpr uint32_t kOffWs = kOffTiles + kEpiWarps * kTileBytes;       // float[16 warps][64]
constexpr uint32_t kOffBias = kOffWs + kEpiWarps * kEpiCols * 4;
constexpr uint32_t kOffBars = kOffBias + kEpiWarps * kEpiCols * 4;
constexpr uint32_t kNumBars = 2 * kStages + 4;
constexpr uint32_t kOffTmemPtr = kOffBars + kNumBars * 8;
constexpr uint32_t kOffAbort = kOffTmemPtr + 4;
constexpr uint32_t kSmemBytes = kOffAbort + 8 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert(kOffTiles % 1024 == 0, "staging tiles must keep the swizzle atom alignment");

struct Smem {
    uint8_t* base;
    __device__ uint32_t a(uint32_t s) const { return smem_u32(base + kOffStages + s * kStageBytes); }
    __device__ uint32_t full(uint32_t s) const { return smem_u32(base + kOffBars + s * 8); }
    __device__ uint32_t empty(uint32_t s) const { return smem_u32(base + kOffBars + (kStages + s) * 8); }
    __device__ uint32_t tmem_full(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + b) * 8); }
    __device__ uint32_t tmem_empty(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + 2 + b) * 8); }
    __device__ uint32_t* tmem_ptr() const { return reinterpret_cast<uint32_t*>(base + kOffTmemPtr); }
    __device__ volatile int* abort_flag() const { return reinterpret_cast<volatile int*>(base + kOffAbort); }
};

// time stamps for the launch timeline (diagnostic; args.trace is null in ordinary runs)
__device__ __forceinline__ void stamp(unsigned long long* trace, uint32_t slot) {
    if (trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        trace[(size_t)blockIdx.x * 8 + slot] = t;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_wide_kernel(const __grid_constant__ GemmTcgen05Args args) {
    extern __shared__ uint8_t smem_raw[];
    Smem sm;
    sm.base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) stamp(args.trace, 0);

    const uint32_t tiles_m = (args.rows + kBM - 1) / kBM;
    const uint32_t tiles_n = (args.n + kBN - 1) / kBN;
    const uint32_t total_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = args.kpad / kBK;
    volatile int* abort_flag = sm.abort_flag();

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) { mbar_init(sm.full(s), 1); mbar_init(sm.empty(s), 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(sm.tmem_full(b), 1); mbar_init(sm.tmem_empty(b), kEpiWarps); }
        arm_abort(abort_flag, args.status);
        fence_barrier_init();
        prefetch_tmap(&args.tmap_a);
        prefetch_tmap(&args.tmap_b);
        prefetch_tmap(&args.tmap_out);
        pdl_release();   // the next launch in the stream may begin its own prologue
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(sm.tmem_ptr()), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_ptr();
    if (threadIdx.x == 0) stamp(args.trace, 1);

    if (warp == 0) {
        // ---------------- TMA producer, activation tiles ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            pdl_wait();   // the activations come from the launch before this one
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int32_t m0 = (int32_t)((t % tiles_m) * kBM);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(sm.full(stage), kStageBytes);
                    tma_load_2d(sm.a(stage), &args.tmap_a, sm.full(stage), (int32_t)(kb * kBK), m0);
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
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
    } else if (warp == kBWarp) {
        // ---------------- TMA producer, weight tiles (constant data: no wait for the predecessor) ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int32_t n0 = (int32_t)((t / tiles_m) * kBN);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    tma_load_2d(sm.a(stage) + kABytes, &args.tmap_b, sm.full(stage), (int32_t)(kb * kBK), n0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kBM, kBN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                if (!mbar_wait(sm.tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccCols;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_try_wait(sm.full(stage), phase) && !mbar_wait(sm.full(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    if (t == blockIdx.x && kb == 0) stamp(args.trace, 2);
                    const uint32_t a_lo = smem_desc_lo(sm.a(stage)), b_lo = a_lo + (kABytes >> 4);
                    umma_i8_lo_first(d_tmem, a_lo, b_lo, idesc, kb);
                    umma_i8_lo(d_tmem, a_lo + 2u, b_lo + 2u, idesc);   // +32 bytes of K = +2
                    umma_i8_lo(d_tmem, a_lo + 4u, b_lo + 4u, idesc);
                    umma_i8_lo(d_tmem, a_lo + 6u, b_lo + 6u, idesc);
                    umma_commit(sm.empty(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(sm.tmem_full(acc));
                if (t == blockIdx.x) stamp(args.trace, 3);
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..17) ----------------
        const uint32_t ew = warp - 2u;
        const uint32_t quarter = warp & 3u;                  // TMEM lanes [32*quarter, +32): fixed by the warp's index
        const uint32_t cbase = (ew >> 2) * kEpiCols;         // columns [64*(ew/4), +64) of the tile
        const EpilogueParams& ep = args.epi;
        float* s_ws = reinterpret_cast<float*>(sm.base + kOffWs) + ew * kEpiCols;
        float* s_bias = reinterpret_cast<float*>(sm.base + kOffBias) + ew * kEpiCols;
        const uint32_t out_tile = smem_u32(sm.base + kOffTiles + ew * kTileBytes);
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        pdl_wait();   // row scales and residual come from earlier launches, and one may still read the output
        for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
            const uint32_t m0 = (t % tiles_m) * kBM, n0 = (t / tiles_m) * kBN + cbase;
            // this warp's own copy of the tile's per-channel vectors: no warp waits for another
            __syncwarp();
            for (uint32_t i = lane; i < kEpiCols; i += 32) {
                const uint32_t n = n0 + i;
                float wsv = 0.0f, bv = 0.0f;
                if (n < args.n && ep.mode == kEpiF32) {
                    wsv = __ldg(ep.ws + n);
                    bv = ep.bias_f32 ? __ldg(ep.bias_f32 + n) : 0.0f;
                }
                s_ws[i] = wsv; s_bias[i] = bv;
            }
            __syncwarp();
            ok = __all_sync(0xffffffffu, mbar_wait(sm.tmem_full(acc), acc_phase, abort_flag));
            if (!ok) break;
            tc_fence_after();
            if (t == blockIdx.x && ew == 0) stamp(args.trace, 4);

            const uint32_t row = m0 + quarter * 32 + lane;
            const bool row_ok = row < args.rows;
            const float as = (row_ok && ep.mode == kEpiF32) ? __ldg(ep.row_scales + row) : 0.0f;
            const uint64_t as2 = f32x2(as, as);
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * kAccCols + cbase;
#pragma unroll 1
            for (uint32_t c = 0; c < kEpiCols; c += 32) {
                const uint32_t col = n0 + c;
                if (col >= args.n) break;                      // uniform over the warp
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                if (ep.mode == kEpiF32) {
                    const float4* w4 = reinterpret_cast<const float4*>(s_ws + c);
                    const float4* b4 = reinterpret_cast<const float4*>(s_bias + c);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float4 wv = w4[j], bv = b4[j];
                        epi_f32_2((int32_t)r[4 * j + 0], (int32_t)r[4 * j + 1], as2, f32x2(wv.x, wv.y), bv.x, bv.y, r[4 * j + 0], r[4 * j + 1]);
                        epi_f32_2((int32_t)r[4 * j + 2], (int32_t)r[4 * j + 3], as2, f32x2(wv.z, wv.w), bv.z, bv.w, r[4 * j + 2], r[4 * j + 3]);
                    }
                    if (ep.residual && row_ok) {
                        // fused residual addition: y += residual[row, col ...]
                        const float* res = ep.residual + (size_t)row * ep.ld_res + col;
                        if (col + 32 <= args.n && (((uintptr_t)res) & 15u) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const float4 rv = __ldg(reinterpret_cast<const float4*>(res) + j);
                                r[4 * j + 0] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * j + 0]), rv.x));
                                r[4 * j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * j + 1]), rv.y));
                                r[4 * j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * j + 2]), rv.z));
                                r[4 * j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(r[4 * j + 3]), rv.w));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (col + i < args.n) r[i] = __float_as_uint(__fadd_rn(__uint_as_float(r[i]), __ldg(res + i)));
                        }
                    }
                }
                if (lane == 0) tma_store_wait_read();          // the previous chunk's store has left the tile
                __syncwarp();
#pragma unroll
                for (uint32_t j = 0; j < 8; j++)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(out_tile + lane * 128u + ((j ^ (lane & 7u)) << 4)),
                                   "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&args.tmap_out, out_tile, (int32_t)col, (int32_t)(m0 + quarter * 32u));
                    tma_store_commit();
                }
            }
            // every lane's TMEM reads are complete (the wait after each load): hand the accumulator back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sm.tmem_empty(acc));
            if (lane == 0 && ew == 0) stamp(args.trace, t == blockIdx.x ? 5 : 6);
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (lane == 0) tma_store_wait_all();   // shared memory is released and the kernel ends after this
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a bounded wait expired somewhere: let asynchronous work in flight settle
        nap(200);
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 1);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
    if (threadIdx.x == 0) stamp(args.trace, 7);
}

}  // namespace

cudaError_t gemm_wide_prepare() { return ensure_dynamic_smem<gemm_i8_wide_kernel>(kSmemBytes); }

cudaError_t launch_gemm_wide(const GemmTcgen05Args& args, int sm_count, cudaStream_t stream) {
    const uint32_t tiles = ((args.rows + kBM - 1) / kBM) * ((args.n + kBN - 1) / kBN);
    if (!tiles) return cudaSuccess;
    if (args.kpad % kBK != 0 || !args.tma_out) return cudaErrorInvalidValue;
    cudaError_t e = gemm_wide_prepare();
    if (e != cudaSuccess) return e;
    const uint32_t grid = tiles < (uint32_t)sm_count ? tiles : (uint32_t)sm_count;
    return launch_pdl(gemm_i8_wide_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, args);
}

}  // namespace vxb
