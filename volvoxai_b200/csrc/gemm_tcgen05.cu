// K2: int8 x int8 -> int32 GEMM on the 5th-generation tensor cores.
//
//   acc[m,n] = sum_k q[m,k] * w[n,k]      q: [rows,kpad] int8, w: [n,kpad] int8
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer of the 128x128B activation tile of each stage (128B-swizzled
//               shared memory, 4-stage ring, mbarrier transaction counts)
//   warp 10     TMA producer of the 256x128B weight tile of each stage (starting a TMA copy
//               costs the issuing thread ~200 ns, more than half of the time the tensor pipe
//               needs for a stage, so the two copies of a stage come from two threads)
//   warp 1      allocates TMEM; one lane issues tcgen05.mma.cta_group::1
//               .kind::i8 (M128 x N256 x K32 per instruction, 4 per stage);
//               tcgen05.commit releases smem stages and publishes accumulators
//   warps 2-9   epilogue: tcgen05.ld the int32 accumulators (two warps per 32-lane
//               TMEM quarter, one per 128-column half), apply the fused epilogue
//               (raw int32 / dequant+bias fp32 / requant int8) and store.
// Two 256-column accumulators fill the 512-column TMEM, so the epilogue of
// tile i overlaps the MMAs of tile i+1.
//
// It replaces the reference's mma.sync tile kernels for the same arithmetic
// (vx_packed_cuda_a8_tile, vx_cuda_packed_a8_m16/_m64:
//  native/src/backends/cuda/kernels/cuda_forward_llm_kernels.inc:693-883,
//  :1249-1511) and its thread/warp dp4a QLinear kernels
// (cuda_forward_quantized_basic_kernels.inc:1-104).
//
// Every wait on an mbarrier is bounded (~2 s of SM clocks); on expiry the
// kernel raises a status word, drains, frees its TMEM and returns.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kBM = 128;           // activation rows per tile (UMMA M)
constexpr uint32_t kBN = 256;           // output channels per tile (UMMA N)
constexpr uint32_t kBK = 128;           // K bytes per stage (one swizzle span)
constexpr uint32_t kStages = 4;
constexpr uint32_t kABytes = kBM * kBK;            // 16 KiB
constexpr uint32_t kBBytes = kBN * kBK;            // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kAccCols = kBN;                 // int32 columns per accumulator
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kEpiWarps = 8;
constexpr uint32_t kThreads = 64 + 32 * kEpiWarps + 32;  // A producer + MMA warp + epilogue warps + B producer
constexpr uint32_t kBWarp = 2 + kEpiWarps;
constexpr uint32_t kEpiThreads = 32 * kEpiWarps;
constexpr uint32_t kEpiCols = kBN / 2;              // columns per epilogue warp

// dynamic shared memory layout (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffStages = 0;
constexpr uint32_t kOffWs = kStages * kStageBytes;                   // float[8 warps][128]
constexpr uint32_t kOffBias = kOffWs + kEpiWarps * kEpiCols * 4;     // float/int32[8 warps][128]
constexpr uint32_t kOffStore = kOffBias + kEpiWarps * kEpiCols * 4;  // [8 warps][16 rows x 128 B] store staging
constexpr uint32_t kStoreBytes = 16 * 128;
constexpr uint32_t kOffBars = kOffStore + kEpiWarps * kStoreBytes;   // 8-byte barriers
constexpr uint32_t kNumBars = 2 * kStages + 4 + 8;   // ... + (staged, flushed) per pair of epilogue warps sharing a TMEM lane quarter
constexpr uint32_t kOffTmemPtr = kOffBars + kNumBars * 8;
constexpr uint32_t kOffAbort = kOffTmemPtr + 4;
constexpr uint32_t kSmemBytes = kOffAbort + 8 + 1024;        // + alignment slack

struct Smem {
    uint8_t* base;
    __device__ uint32_t a(uint32_t s) const { return smem_u32(base + kOffStages + s * kStageBytes); }
    __device__ uint32_t b(uint32_t s) const { return a(s) + kABytes; }
    __device__ uint32_t full(uint32_t s) const { return smem_u32(base + kOffBars + s * 8); }
    __device__ uint32_t empty(uint32_t s) const { return smem_u32(base + kOffBars + (kStages + s) * 8); }
    __device__ uint32_t tmem_full(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + b) * 8); }
    __device__ uint32_t tmem_empty(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + 2 + b) * 8); }
    __device__ uint32_t pair_staged(uint32_t q) const { return smem_u32(base + kOffBars + (2 * kStages + 4 + q) * 8); }
    __device__ uint32_t pair_flushed(uint32_t q) const { return smem_u32(base + kOffBars + (2 * kStages + 8 + q) * 8); }
    __device__ uint32_t* tmem_ptr() const { return reinterpret_cast<uint32_t*>(base + kOffTmemPtr); }
    __device__ volatile int* abort_flag() const { return reinterpret_cast<volatile int*>(base + kOffAbort); }
    __device__ float* ws() const { return reinterpret_cast<float*>(base + kOffWs); }
    __device__ float* bias() const { return reinterpret_cast<float*>(base + kOffBias); }
};

// time stamps for the launch timeline (diagnostic; args.trace is null in ordinary runs)
__device__ __forceinline__ void stamp(unsigned long long* trace, uint32_t slot) {
    if (trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        trace[(size_t)blockIdx.x * 8 + slot] = t;
    }
}

__device__ __forceinline__ void gemm_i8_tcgen05_body(const GemmTcgen05Args& args) {
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
    // with peer destinations the last pipeline stage becomes the epilogue warps' staging area
    // for coalesced stores (the exchange, not the MMA pipeline, bounds that launch)
    const bool gather = args.epi.n_peers != 0;
    // the flush of the fused all-gather as TMA tile stores (one per destination and warp) instead of lane stores
    const bool gather_tma = gather && args.gather_tma != 0;
    const uint32_t nstages = gather ? kStages - 1 : kStages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) { mbar_init(sm.full(s), 1); mbar_init(sm.empty(s), 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(sm.tmem_full(b), 1); mbar_init(sm.tmem_empty(b), kEpiThreads); }
        for (uint32_t q = 0; q < 4; q++) { mbar_init(sm.pair_staged(q), 2); mbar_init(sm.pair_flushed(q), 2); }
        arm_abort(abort_flag, args.status);
        fence_barrier_init();
        prefetch_tmap(&args.tmap_a);
        prefetch_tmap(&args.tmap_b);
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
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            pdl_wait();   // the activations come from the launch before this one; the weight producer does not wait
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int32_t m0 = (int32_t)((t % tiles_m) * kBM);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(sm.full(stage), kStageBytes);
                    tma_load_2d(sm.a(stage), &args.tmap_a, sm.full(stage), (int32_t)(kb * kBK), m0);
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == nstages) { stage = 0; phase ^= 1u; }
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
        // ---------------- TMA producer, weight tiles ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                const int32_t n0 = (int32_t)((t / tiles_m) * kBN);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    tma_load_2d(sm.b(stage), &args.tmap_b, sm.full(stage), (int32_t)(kb * kBK), n0);
                    if (++stage == nstages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kBM, kBN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            // barrier addresses and descriptor low words advance by constants from stage to stage
            const uint32_t a_lo0 = smem_desc_lo(sm.a(0));
            uint32_t full_s = sm.full(0), empty_s = sm.empty(0), a_lo = a_lo0;
            for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
                if (!mbar_wait(sm.tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccCols;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_try_wait(full_s, phase) && !mbar_wait(full_s, phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    if (t == blockIdx.x && kb == 0) stamp(args.trace, 2);
                    umma_i8_lo_first(d_tmem, a_lo, a_lo + (kABytes >> 4), idesc, kb);
                    umma_i8_lo(d_tmem, a_lo + 2u, a_lo + (kABytes >> 4) + 2u, idesc);   // +32 bytes of K = +2
                    umma_i8_lo(d_tmem, a_lo + 4u, a_lo + (kABytes >> 4) + 4u, idesc);
                    umma_i8_lo(d_tmem, a_lo + 6u, a_lo + (kABytes >> 4) + 6u, idesc);
                    umma_commit(empty_s);
                    full_s += 8; empty_s += 8; a_lo += kStageBytes >> 4;
                    if (++stage == nstages) { stage = 0; phase ^= 1u; full_s = sm.full(0); empty_s = sm.empty(0); a_lo = a_lo0; }
                }
                if (!ok) break;
                umma_commit(sm.tmem_full(acc));
                if (t == blockIdx.x) stamp(args.trace, 3);
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else if (warp < kBWarp) {
        // ---------------- epilogue (warps 2..9) ----------------
        // Two warps per TMEM lane quarter (one per SM sub-partition pair), each owning one
        // half of the tile's 256 columns, so every scheduler has two epilogue warps to
        // interleave.
        const uint32_t quarter = warp & 3u;              // TMEM lanes [32*quarter, +32)
        const uint32_t half = (warp - 2u) >> 2;          // columns [128*half, +128) of the tile
        const uint32_t cbase = half * kEpiCols;
        const EpilogueParams& ep = args.epi;
        // each epilogue warp stages its own slice of the per-channel vectors, so the warps
        // never wait on one another
        float* s_ws = sm.ws() + (warp - 2u) * kEpiCols;
        float* s_bias = sm.bias() + (warp - 2u) * kEpiCols;
        // fused all-gather: the two warps of a lane quarter (left and right half of the tile's columns)
        // stage into ONE [32 rows x 256 B] tile, so that the flush can store whole 256-byte row
        // segments - NVLink moves long contiguous runs far better than 128-byte ones; the pair meets on
        // two mbarriers (bounded waits, like every wait here) instead of a bar.sync
        // TMA form: every warp has a [32 rows x 128 B] tile of its own (128B-swizzled), no partner
        uint8_t* stage_tile = sm.base + kOffStages + (kStages - 1) * kStageBytes +
                              (gather_tma ? (warp - 2u) * (32u * kEpiCols) : quarter * (32u * 2u * kEpiCols));
        uint32_t pair_phase = 0;
        bool first_gather_tile = true;
        const float zero_f = __int2float_rn(ep.out_zero);
        const float lo_f = __int2float_rn(ep.out_lo), hi_f = __int2float_rn(ep.out_hi);
        const bool sat_s8 = ep.out_lo == -128 && ep.out_hi == 127, sat_u8 = ep.out_lo == 0 && ep.out_hi == 255;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        pdl_wait();   // row scales and residual come from earlier launches, and the output may still be read by one
        for (uint32_t t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
            const uint32_t m0 = (t % tiles_m) * kBM, n0 = (t / tiles_m) * kBN + cbase;
            // stage this warp's per-channel vectors for the tile
            __syncwarp();
            for (uint32_t i = lane; i < kEpiCols; i += 32) {
                const uint32_t n = n0 + i;
                float wsv = 0.0f, bv = 0.0f;
                if (n < args.n && ep.mode != kEpiAcc) {
                    wsv = __ldg(ep.ws + n);
                    if (ep.mode == kEpiF32) bv = ep.bias_f32 ? __ldg(ep.bias_f32 + n) : 0.0f;
                    else bv = __int_as_float(ep.bias_i32 ? __ldg(ep.bias_i32 + n) : 0);
                }
                s_ws[i] = wsv; s_bias[i] = bv;
            }
            __syncwarp();
            ok = __all_sync(0xffffffffu, mbar_wait(sm.tmem_full(acc), acc_phase, abort_flag));
            if (!ok) break;
            tc_fence_after();
            if (t == blockIdx.x && threadIdx.x == 64) stamp(args.trace, 4);
            if (gather_tma) {
                if (lane == 0) tma_store_wait_read();   // the previous tile's stores have left the staging tile
                __syncwarp();
            } else if (gather && !first_gather_tile) {
                // the partner must have finished flushing the previous tile out of the shared staging tile
                ok = __all_sync(0xffffffffu, mbar_wait(sm.pair_flushed(quarter), pair_phase ^ 1u, abort_flag));
                if (!ok) break;
            }

            const uint32_t row = m0 + quarter * 32 + lane;
            const bool row_ok = row < args.rows;
            const float as = (row_ok && ep.mode != kEpiAcc) ? __ldg(ep.row_scales + row) : 0.0f;
            const bool fast = ep.fast_div != 0 && div_const_row_ok(as);
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * kAccCols + cbase;
#pragma unroll 1
            for (uint32_t c = 0; c < kEpiCols; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                const uint32_t col = n0 + c;
                if (col >= args.n) continue;                       // uniform over the warp
                const bool wide = ep.mode != kEpiI8;                // 32-bit outputs go through the staging below
                if (!row_ok && !wide) continue;
                const bool full = col + 32 <= args.n;
                const float4* w4 = reinterpret_cast<const float4*>(s_ws + c);
                const float4* b4 = reinterpret_cast<const float4*>(s_bias + c);
                if (ep.mode == kEpiI8) {
                    int8_t* dst = (int8_t*)ep.out + (size_t)row * ep.ld + col;
                    uint32_t packed[8];
                    if (fast && sat_s8 && !ep.bias_i32 && ep.out_zero == 0) {
                        // no bias, zero point 0: fewest instructions per element, and the epilogue's length
                        // is what the MMA-issuing thread pays for while both run
                        const RequantPair rq(as, ep.out_scale, ep.out_rcp, zero_f);
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 wv = w4[j];
                            int32_t q0, q1, q2, q3;
                            epi_i8_sat2<false, false>((int32_t)r[4 * j + 0], (int32_t)r[4 * j + 1], f32x2(wv.x, wv.y), rq, q0, q1);
                            epi_i8_sat2<false, false>((int32_t)r[4 * j + 2], (int32_t)r[4 * j + 3], f32x2(wv.z, wv.w), rq, q2, q3);
                            packed[j] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
                        }
                    } else if (fast && sat_s8) {
                        const RequantPair rq(as, ep.out_scale, ep.out_rcp, zero_f);
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 wv = w4[j], bv = b4[j];
                            int32_t q0, q1, q2, q3;
                            epi_i8_sat2<false, true>((int32_t)r[4 * j + 0] + __float_as_int(bv.x), (int32_t)r[4 * j + 1] + __float_as_int(bv.y),
                                                     f32x2(wv.x, wv.y), rq, q0, q1);
                            epi_i8_sat2<false, true>((int32_t)r[4 * j + 2] + __float_as_int(bv.z), (int32_t)r[4 * j + 3] + __float_as_int(bv.w),
                                                     f32x2(wv.z, wv.w), rq, q2, q3);
                            packed[j] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
                        }
                    } else if (fast && sat_u8) {
                        const RequantPair rq(as, ep.out_scale, ep.out_rcp, zero_f);
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 wv = w4[j], bv = b4[j];
                            int32_t q0, q1, q2, q3;
                            epi_i8_sat2<true, true>((int32_t)r[4 * j + 0] + __float_as_int(bv.x), (int32_t)r[4 * j + 1] + __float_as_int(bv.y),
                                                    f32x2(wv.x, wv.y), rq, q0, q1);
                            epi_i8_sat2<true, true>((int32_t)r[4 * j + 2] + __float_as_int(bv.z), (int32_t)r[4 * j + 3] + __float_as_int(bv.w),
                                                    f32x2(wv.z, wv.w), rq, q2, q3);
                            packed[j] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
                        }
                    } else if (fast) {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 wv = w4[j], bv = b4[j];
                            const int32_t q0 = epi_i8_v2<true>((int32_t)r[4 * j + 0] + __float_as_int(bv.x), as, wv.x, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            const int32_t q1 = epi_i8_v2<true>((int32_t)r[4 * j + 1] + __float_as_int(bv.y), as, wv.y, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            const int32_t q2 = epi_i8_v2<true>((int32_t)r[4 * j + 2] + __float_as_int(bv.z), as, wv.z, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            const int32_t q3 = epi_i8_v2<true>((int32_t)r[4 * j + 3] + __float_as_int(bv.w), as, wv.w, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            packed[j] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 wv = w4[j], bv = b4[j];
                            const int32_t q0 = epi_i8_v2<false>((int32_t)r[4 * j + 0] + __float_as_int(bv.x), as, wv.x, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            const int32_t q1 = epi_i8_v2<false>((int32_t)r[4 * j + 1] + __float_as_int(bv.y), as, wv.y, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            const int32_t q2 = epi_i8_v2<false>((int32_t)r[4 * j + 2] + __float_as_int(bv.z), as, wv.z, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            const int32_t q3 = epi_i8_v2<false>((int32_t)r[4 * j + 3] + __float_as_int(bv.w), as, wv.w, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            packed[j] = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
                        }
                    }
                    if (gather) {
                        // this warp's half of row `lane` of the pair's [32 rows x 256 B] staging tile; 16-byte
                        // pieces XOR-swizzled by row within the half so that both the row-wise writes here and
                        // the piece-wise reads of the flush are free of bank conflicts
                        uint8_t* st = gather_tma ? stage_tile + lane * kEpiCols
                                                 : stage_tile + lane * (2u * kEpiCols) + half * kEpiCols;
                        const uint32_t p0 = c >> 4;
                        *reinterpret_cast<uint4*>(st + (((p0) ^ (lane & 7u)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        *reinterpret_cast<uint4*>(st + (((p0 + 1u) ^ (lane & 7u)) << 4)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else if (full && (((uintptr_t)dst) & 15u) == 0) {
                        reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (col + i < args.n) dst[i] = (int8_t)((packed[i >> 2] >> (8 * (i & 3))) & 0xffu);
                    }
                } else {
                    uint32_t o[32];
                    if (ep.mode == kEpiF32) {
                        const uint64_t as2 = f32x2(as, as);
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float4 wv = w4[j], bv = b4[j];
                            epi_f32_2((int32_t)r[4 * j + 0], (int32_t)r[4 * j + 1], as2, f32x2(wv.x, wv.y), bv.x, bv.y, o[4 * j + 0], o[4 * j + 1]);
                            epi_f32_2((int32_t)r[4 * j + 2], (int32_t)r[4 * j + 3], as2, f32x2(wv.z, wv.w), bv.z, bv.w, o[4 * j + 2], o[4 * j + 3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = r[i];
                    }
                    if (ep.mode == kEpiF32 && ep.residual && row_ok) {
                        // fused residual addition: y += residual[row, col ...]
                        const float* res = ep.residual + (size_t)row * ep.ld_res + col;
                        if (full && (((uintptr_t)res) & 15u) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const float4 rv = __ldg(reinterpret_cast<const float4*>(res) + j);
                                o[4 * j + 0] = __float_as_uint(__fadd_rn(__uint_as_float(o[4 * j + 0]), rv.x));
                                o[4 * j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(o[4 * j + 1]), rv.y));
                                o[4 * j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(o[4 * j + 2]), rv.z));
                                o[4 * j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(o[4 * j + 3]), rv.w));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (col + i < args.n) o[i] = __float_as_uint(__fadd_rn(__uint_as_float(o[i]), __ldg(res + i)));
                        }
                    }
                    if (ep.mode == kEpiF32 && ep.act == 1u) {
                        // channel pairs (gate, up) -> silu(gate) * up, one output column per pair
                        if (row_ok) {
                            float* dst = (float*)ep.out + (size_t)row * ep.ld + (col >> 1);
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (col + 2 * j + 1 < args.n)
                                    dst[j] = epi_silu_mul(__uint_as_float(o[2 * j]), __uint_as_float(o[2 * j + 1]));
                        }
                        continue;
                    }
                    // Each thread holds 128 contiguous bytes of its own row; stored directly, one store
                    // instruction touches 32 different rows. Instead the warp passes 16 rows at a time
                    // through shared memory (16-byte pieces XOR-swizzled by row: no bank conflicts either
                    // way) and stores whole 128-byte row segments, four rows per instruction.
                    uint8_t* stage = sm.base + kOffStore + (warp - 2u) * kStoreBytes;
#pragma unroll
                    for (uint32_t half16 = 0; half16 < 2; half16++) {
                        __syncwarp();
                        if ((lane >> 4) == half16) {
                            uint8_t* mine = stage + (lane & 15u) * 128u;
#pragma unroll
                            for (uint32_t j = 0; j < 8; j++)
                                *reinterpret_cast<uint4*>(mine + ((j ^ (lane & 7u)) << 4)) =
                                    make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                        }
                        __syncwarp();
                        const uint32_t piece = lane & 7u;
#pragma unroll
                        for (uint32_t i = 0; i < 4; i++) {
                            const uint32_t rl = 4u * i + (lane >> 3);                 // row within the 16
                            const uint4 v = *reinterpret_cast<const uint4*>(stage + rl * 128u + ((piece ^ (rl & 7u)) << 4));
                            const uint32_t grow = m0 + quarter * 32u + half16 * 16u + rl, gcol = col + piece * 4u;
                            if (grow >= args.rows || gcol >= args.n) continue;
                            uint32_t* dst = (uint32_t*)ep.out + (size_t)grow * ep.ld + gcol;
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
            tc_fence_before();
            mbar_arrive(sm.tmem_empty(acc));
            if (threadIdx.x == 64) stamp(args.trace, t == blockIdx.x ? 5 : 6);
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
            if (!ok) break;
            if (gather_tma) {
                // this warp's 32 rows x 128 columns leave as one TMA tile store per destination: this GPU's
                // buffer (0) and every peer's, each map covering this rank's channel range of that buffer, so
                // the tensor map clips the shard's ragged last tile and the rows beyond the batch.  Plain
                // tile stores over NVLink: no multicast, nothing is loaded from a peer.
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && n0 < args.n) {
                    for (uint32_t d = 0; d <= ep.n_peers; d++)
                        tma_store_2d(&args.tmap_gather[d], smem_u32(stage_tile), (int32_t)n0, (int32_t)(m0 + quarter * 32u));
                    tma_store_commit();
                }
            } else if (gather) {
                // both halves staged -> this warp flushes 16 of the 32 rows: 16 lanes cover the 256 bytes of
                // one row, 2 rows per pass, the same 16 bytes going to this GPU's buffer (destination 0) and
                // to the same rows and columns of every peer's buffer - plain stores over NVLink, so the
                // all-gather of the output is part of the epilogue and overlaps the next tile's MMAs
                __syncwarp();
                if (lane == 0) mbar_arrive(sm.pair_staged(quarter));
                ok = __all_sync(0xffffffffu, mbar_wait(sm.pair_staged(quarter), pair_phase, abort_flag));
                if (!ok) break;
                const uint32_t piece = lane & 15u, phalf = piece >> 3, p = piece & 7u;
                const uint32_t tile_n0 = n0 - cbase;
#pragma unroll 1
                for (uint32_t i = 0; i < 8; i++) {
                    const uint32_t rl = half * 16u + 2u * i + (lane >> 4);
                    const uint4 v = *reinterpret_cast<const uint4*>(stage_tile + rl * (2u * kEpiCols) + phalf * kEpiCols + ((p ^ (rl & 7u)) << 4));
                    const uint32_t grow = m0 + quarter * 32 + rl, gcol = tile_n0 + piece * 16;
                    if (grow >= args.rows || gcol >= args.n) continue;
                    const bool whole = gcol + 16 <= args.n;
                    const size_t off = (size_t)grow * ep.ld + gcol;
                    for (uint32_t d = 0; d <= ep.n_peers; d++) {
                        int8_t* dst = (int8_t*)(d ? ep.peer_out[d - 1] : ep.out) + off;
                        if (whole && (((uintptr_t)dst) & 15u) == 0) {
                            *reinterpret_cast<uint4*>(dst) = v;
                        } else {
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int b = 0; b < 16; b++)
                                if (gcol + b < args.n) dst[b] = (int8_t)((w[b >> 2] >> (8 * (b & 3))) & 0xffu);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sm.pair_flushed(quarter));
                pair_phase ^= 1u;
                first_gather_tile = false;
            }
        }
        if (gather_tma && lane == 0) tma_store_wait_all();   // the stores are complete before the kernel ends
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

__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_tcgen05_kernel(const __grid_constant__ GemmTcgen05Args args) { gemm_i8_tcgen05_body(args); }

// The same kernel held to 128 registers per thread (45 K of the SM's 64 K registers), which leaves
// room for one CTA of the row quantizer beside it.  Launched for a link-bound fused all-gather when the
// tunable "gemm.overlap_gather" is set (the quantizer of the later rows then runs underneath it).  Off
// by default: measured on four GPUs the pair of launches took 207 us against 173 us for the single
// launch of the full-register build after the whole-batch quantizer.
__global__ void __maxnreg__(128)
gemm_i8_tcgen05_gather_kernel(const __grid_constant__ GemmTcgen05Args args) { gemm_i8_tcgen05_body(args); }

// ---- tensor-pipe peak probe --------------------------------------------------
// Every CTA issues back-to-back M128xN256xK32 kind::i8 MMAs on operands that
// stay resident in shared memory (no TMA, no epilogue): the dense int8 rate the
// tensor pipe sustains, used as the measured roofline denominator for K2.
__global__ void __launch_bounds__(128, 1)
i8_peak_probe_kernel(uint32_t iters, long long* cycles, int* status, uint32_t idesc, uint32_t accs,
                     uint32_t acc_stride, uint32_t per_commit) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_ptr;
    __shared__ int abort_flag[2];
    const uint32_t warp = threadIdx.x >> 5;
    for (uint32_t i = threadIdx.x; i < kStageBytes / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(base)[i] = 0x01010101u;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); arm_abort(abort_flag, status); fence_barrier_init(); }
    fence_proxy_async();
    if (warp == 0) { tmem_alloc(smem_u32(&tmem_ptr), kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_ptr;
    // `issuers` (high 16 bits of accs) warps issue concurrently, each with its own barrier and
    // accumulator set; issuer 0 reports its clocks
    const uint32_t issuers = (accs >> 16) ? (accs >> 16) : 1u;
    accs &= 0xffffu;
    __shared__ uint64_t bars[4];
    if (threadIdx.x == 0) { for (int i = 0; i < 4; i++) mbar_init(smem_u32(&bars[i]), 1); fence_barrier_init(); }
    __syncthreads();
    if ((threadIdx.x & 31) == 0 && warp < issuers) {
        const uint32_t a_addr = smem_u32(base), b_addr = a_addr + kABytes;
        const uint32_t my_bar = smem_u32(&bars[warp]);
        const uint32_t my_tmem = tmem_base + warp * accs * acc_stride;
        const long long t0 = clock64();
        uint32_t parity = 0;
        bool ok = true;
        for (uint32_t it = 0; ok && it < iters; it++) {
            for (uint32_t j = 0; j < per_commit; j++)
                umma_i8(my_tmem + (j & (accs - 1u)) * acc_stride, make_smem_desc(a_addr + (j & 3u) * kUmmaK),
                        make_smem_desc(b_addr + (j & 3u) * kUmmaK), idesc, 1u);
            umma_commit(my_bar);
            ok = mbar_wait(my_bar, parity, abort_flag);
            parity ^= 1u;
        }
        if (warp == 0) cycles[blockIdx.x] = clock64() - t0;
        if (!ok && status) atomicExch(status, 2);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

cudaError_t gemm_tcgen05_prepare() {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_tcgen05_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gemm_i8_tcgen05_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(i8_peak_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)(kStageBytes + 1024));
}

cudaError_t launch_gemm_tcgen05(const GemmTcgen05Args& args, int sm_count, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    const uint32_t tiles = ((args.rows + kBM - 1) / kBM) * ((args.n + kBN - 1) / kBN);
    const uint32_t grid = tiles < (uint32_t)sm_count ? tiles : (uint32_t)sm_count;
    if (gather_is_link_bound(args.epi.n_peers, args.kpad) && tunables().overlap_gather)
        return launch_pdl(gemm_i8_tcgen05_gather_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, args);
    return launch_pdl(gemm_i8_tcgen05_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, args);
}

cudaError_t launch_i8_peak_probe(uint32_t iters, long long* cycles, int* status, int sm_count,
                                 cudaStream_t stream) {
    i8_peak_probe_kernel<<<sm_count, 128, kStageBytes + 1024, stream>>>(
        iters, cycles, status, make_idesc(kBM, kBN), 2u, kAccCols, 256u);
    return cudaGetLastError();
}

cudaError_t launch_mma_probe(uint32_t m, uint32_t n, uint32_t accs, uint32_t per_commit, uint32_t iters,
                             long long* cycles, int* status, cudaStream_t stream) {
    uint32_t stride = n < 32 ? 32 : n;
    const uint32_t issuers = (accs >> 16) ? (accs >> 16) : 1u;
    if ((accs & 0xffffu) * stride * issuers > kTmemCols || issuers > 4) return cudaErrorInvalidValue;
    i8_peak_probe_kernel<<<1, 128, kStageBytes + 1024, stream>>>(iters, cycles, status, make_idesc(m, n), accs,
                                                                 stride, per_commit);
    return cudaGetLastError();
}

}  // namespace vxb
