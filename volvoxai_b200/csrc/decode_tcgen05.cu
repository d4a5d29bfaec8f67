// K3b: skinny (decode-shaped) W8A8 GEMM for rows <= 128: HBM-bound, the int8 weights are
// streamed exactly once and every SM streams the same number of bytes.
//
//   acc[m,n] = sum_k q[m,k] * w[n,k]
//
// The operands are swapped relative to the large-M kernel: the WEIGHT tile is the UMMA
// M operand (128 output channels x 128 K bytes per stage) and the few activation rows are
// the UMMA N operand (MT = 32/64/128 token slots, zero-filled by TMA beyond `rows`), so the
// tensor pipe only does the work the tokens need while TMA keeps ~160 KB of weight bytes in
// flight per SM.  Work is split stream-K style: the (channel tile, K block) units are dealt
// out in equal contiguous ranges to one persistent CTA per SM, so a CTA may finish one tile,
// compute whole tiles, and start another.  A CTA that holds only part of a tile's K range
// adds its int32 partials into a zero-initialised workspace with red.global.add and bumps the
// tile's counter; the CTA that completes the count applies the epilogue and clears workspace
// and counter again (a contiguous range has at most two partial segments; their counting and
// finishing is batched after the main loop).  Integer addition is associative, so the result
// is bit-identical for every split.
//
// Reference counterparts: the decode kernels vx_packed_cuda_a8_columns and the fused
// GEMV family (native/src/backends/cuda/kernels/cuda_forward_llm_kernels.inc:254-459,
// cuda_forward_gemv_pair_kernels.inc:155-1711), which give each CTA one row x 32 columns and
// re-quantize the activation row per column tile; and the CPU single-row route
// (native/src/kernels/packed_linear_ops.inc:1471-1535).
//
// All mbarrier waits are bounded; on expiry the kernel raises the status word, drains and
// frees its TMEM.  No CTA ever waits for another CTA.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kDM = 128;            // output channels per tile (UMMA M)
constexpr uint32_t kDK = 128;            // K bytes per stage
constexpr uint32_t kWBytes = kDM * kDK;  // 16 KiB weight tile
constexpr uint32_t kThreads = 192;       // producer warp, MMA warp, 4 epilogue warps

template <uint32_t MT> struct DecodeCfg {
    static constexpr uint32_t kXBytes = MT * kDK;
    static constexpr uint32_t kStageBytes = kWBytes + kXBytes;
    // about 100 KB of stages per CTA: two CTAs fit one SM, so the next launch's CTA can move
    // in (and prefetch its weights) while the previous launch's CTA is still finishing
    static constexpr uint32_t kStages = MT <= 32 ? 5 : MT <= 64 ? 4 : 3;
    static constexpr uint32_t kTmemCols = 2 * MT < 32 ? 32 : 2 * MT;
    static constexpr uint32_t kOffBars = kStages * kStageBytes;
    static constexpr uint32_t kNumBars = 2 * kStages + 4;
    static constexpr uint32_t kOffTmemPtr = kOffBars + kNumBars * 8;
    static constexpr uint32_t kOffAbort = kOffTmemPtr + 4;
    static constexpr uint32_t kOffFlag = kOffAbort + 8;       // epilogue-uniform decisions (4 ints)
    static constexpr uint32_t kOffScales = kOffFlag + 16;     // float[MT] activation scales
    static constexpr uint32_t kSmemBytes = kOffScales + MT * 4 + 1024;
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Segment { uint32_t tile, kb_begin, kb_end; };

// Next segment of this CTA's unit range [u, u1): consecutive K blocks of one tile.
__device__ __forceinline__ bool next_segment(uint64_t& u, uint64_t u1, uint32_t num_kb, Segment& seg) {
    if (u >= u1) return false;
    seg.tile = (uint32_t)(u / num_kb);
    seg.kb_begin = (uint32_t)(u % num_kb);
    const uint64_t left = u1 - u;
    const uint32_t room = num_kb - seg.kb_begin;
    const uint32_t take = left < room ? (uint32_t)left : room;
    seg.kb_end = seg.kb_begin + take;
    u += take;
    return true;
}

template <uint32_t MT>
__global__ void __launch_bounds__(kThreads, 2)
decode_i8_tcgen05_kernel(const __grid_constant__ DecodeTcgen05Args args) {
    using Cfg = DecodeCfg<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto w_addr = [&](uint32_t s) { return smem_u32(base + s * Cfg::kStageBytes); };
    auto x_addr = [&](uint32_t s) { return smem_u32(base + s * Cfg::kStageBytes + kWBytes); };
    auto full = [&](uint32_t s) { return smem_u32(base + Cfg::kOffBars + s * 8); };
    auto empty = [&](uint32_t s) { return smem_u32(base + Cfg::kOffBars + (Cfg::kStages + s) * 8); };
    auto tmem_full = [&](uint32_t b) { return smem_u32(base + Cfg::kOffBars + (2 * Cfg::kStages + b) * 8); };
    auto tmem_empty = [&](uint32_t b) { return smem_u32(base + Cfg::kOffBars + (2 * Cfg::kStages + 2 + b) * 8); };
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(base + Cfg::kOffTmemPtr);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + Cfg::kOffAbort);
    volatile int* epi_flag = reinterpret_cast<volatile int*>(base + Cfg::kOffFlag);
    float* s_as = reinterpret_cast<float*>(base + Cfg::kOffScales);

    const uint32_t tiles_n = (args.n + kDM - 1) / kDM;
    const uint32_t num_kb = args.kpad / kDK;
    const uint64_t units = (uint64_t)tiles_n * num_kb;
    const uint64_t u0 = units * blockIdx.x / gridDim.x;
    const uint64_t u1 = units * (blockIdx.x + 1) / gridDim.x;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < Cfg::kStages; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(tmem_full(b), 1); mbar_init(tmem_empty(b), 128); }
        arm_abort(abort_flag, args.status);
        fence_barrier_init();
        prefetch_tmap(&args.tmap_w);
        prefetch_tmap(&args.tmap_x);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_ptr), Cfg::kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    if (threadIdx.x == 0) pdl_release();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            // Weights never depend on the preceding kernel: fill the ring with weight tiles
            // first, then wait for the dependency and add the activation tiles.
            {
                uint64_t u = u0; Segment seg; uint32_t s = 0;
                while (s < Cfg::kStages && next_segment(u, u1, num_kb, seg))
                    for (uint32_t kb = seg.kb_begin; kb < seg.kb_end && s < Cfg::kStages; kb++, s++) {
                        mbar_expect_tx(full(s), Cfg::kStageBytes);
                        tma_load_2d(w_addr(s), &args.tmap_w, full(s), (int32_t)(kb * kDK), (int32_t)(seg.tile * kDM));
                        armed |= 1u << s;
                    }
            }
            pdl_wait();
            uint64_t u = u0; Segment seg; uint32_t issued = 0;
            while (ok && next_segment(u, u1, num_kb, seg)) {
                for (uint32_t kb = seg.kb_begin; kb < seg.kb_end; kb++, issued++) {
                    if (issued >= Cfg::kStages) {
                        if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                        mbar_expect_tx(full(stage), Cfg::kStageBytes);
                        tma_load_2d(w_addr(stage), &args.tmap_w, full(stage), (int32_t)(kb * kDK), (int32_t)(seg.tile * kDM));
                    }
                    tma_load_2d(x_addr(stage), &args.tmap_x, full(stage), (int32_t)(kb * kDK), 0);
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                for (uint32_t s = 0; s < Cfg::kStages; s++) {
                    if (!(armed & (1u << s))) continue;
                    for (uint32_t i = 0; i < 2000; i++) {
                        if (mbar_try_wait(full(s), (armed_parity >> s) & 1u)) break;
                        __nanosleep(500);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(kDM, MT);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            uint64_t u = u0; Segment seg;
            while (ok && next_segment(u, u1, num_kb, seg)) {
                if (!mbar_wait(tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * MT;
                for (uint32_t kb = seg.kb_begin; kb < seg.kb_end; kb++) {
                    if (!mbar_wait(full(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t wa = w_addr(stage), xa = x_addr(stage);
#pragma unroll
                    for (uint32_t k = 0; k < kDK / kUmmaK; k++)
                        umma_i8(d_tmem, make_smem_desc(wa + k * kUmmaK), make_smem_desc(xa + k * kUmmaK),
                                idesc, (kb != seg.kb_begin || k != 0u) ? 1u : 0u);
                    umma_commit(empty(stage));
                    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(tmem_full(acc));
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5): thread = one output channel ----------------
        const uint32_t quarter = warp & 3u;
        const uint32_t e = threadIdx.x - 64;
        const EpilogueParams& ep = args.epi;
        const float zero_f = __int2float_rn(ep.out_zero);
        const float lo_f = __int2float_rn(ep.out_lo), hi_f = __int2float_rn(ep.out_hi);
        // everything below reads what the preceding kernel wrote, or writes what it may read
        pdl_wait();
        if (e < MT) s_as[e] = (e < args.rows && ep.mode != kEpiAcc) ? __ldg(ep.row_scales + e) : 0.0f;
        epi_bar();

        // One 32-token chunk of channel n through the selected epilogue.
        auto finish_chunk = [&](uint32_t n, uint32_t c, const int32_t (&v)[32], float wsv, float bias_f,
                                int32_t bias_i) {
#pragma unroll
            for (uint32_t i = 0; i < 32; i++) {
                const uint32_t m = c + i;
                if (m >= args.rows) continue;
                const size_t at = (size_t)m * ep.ld + n;
                if (ep.mode == kEpiAcc) {
                    ((int32_t*)ep.out)[at] = v[i];
                } else if (ep.mode == kEpiF32) {
                    ((float*)ep.out)[at] = epi_f32(v[i], s_as[m], wsv, bias_f);
                } else {
                    const float as = s_as[m];
                    const int32_t qv = (ep.fast_div != 0 && div_const_row_ok(as))
                        ? epi_i8_v2<true>(v[i] + bias_i, as, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero)
                        : epi_i8_v2<false>(v[i] + bias_i, as, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                    ((int8_t*)ep.out)[at] = (int8_t)qv;
                }
            }
        };
        auto channel_consts = [&](uint32_t n, float& wsv, float& bias_f, int32_t& bias_i) {
            const bool n_ok = n < args.n;
            wsv = (n_ok && ep.mode != kEpiAcc) ? __ldg(ep.ws + n) : 0.0f;
            bias_f = (n_ok && ep.mode == kEpiF32 && ep.bias_f32) ? __ldg(ep.bias_f32 + n) : 0.0f;
            bias_i = (n_ok && ep.mode == kEpiI8 && ep.bias_i32) ? __ldg(ep.bias_i32 + n) : 0;
        };

        // A contiguous unit range holds at most two partial segments (its first and its last);
        // their counting and finishing is deferred and done together after the loop.
        uint32_t part_tile[2] = {0, 0}, part_blocks[2] = {0, 0}, parts = 0;
        uint32_t acc = 0, acc_phase = 0;
        bool gave_up = false;
        uint64_t u = u0; Segment seg;
        while (next_segment(u, u1, num_kb, seg)) {
            const uint32_t n = seg.tile * kDM + quarter * 32 + lane;
            const bool n_ok = n < args.n;
            const bool whole = seg.kb_begin == 0 && seg.kb_end == num_kb;
            float wsv, bias_f; int32_t bias_i;
            channel_consts(n, wsv, bias_f, bias_i);   // in flight while the MMAs run

            const bool waited = mbar_wait(tmem_full(acc), acc_phase, abort_flag);
            // make the give-up decision uniform across the four epilogue warps
            epi_bar();
            if (threadIdx.x == 64) epi_flag[0] = (*abort_flag != 0 || !waited) ? 1 : 0;
            epi_bar();
            if (epi_flag[0]) { gave_up = true; break; }
            tc_fence_after();

            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * MT;
#pragma unroll 1
            for (uint32_t c = 0; c < MT; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                if (c >= args.rows || !n_ok) continue;
                int32_t v[32];
#pragma unroll
                for (int i = 0; i < 32; i++) v[i] = (int32_t)r[i];
                if (whole) {
                    finish_chunk(n, c, v, wsv, bias_f, bias_i);
                } else {
                    // partial K range: add into the zero-initialised workspace
#pragma unroll
                    for (uint32_t i = 0; i < 32; i++)
                        if (c + i < args.rows) atomicAdd(args.workspace + (size_t)(c + i) * args.n + n, v[i]);
                }
            }
            // the accumulator has been consumed: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            mbar_arrive(tmem_empty(acc));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
            if (!whole && parts < 2) {
                part_tile[parts] = seg.tile;
                part_blocks[parts] = seg.kb_end - seg.kb_begin;
                parts++;
            }
        }

        if (!gave_up && parts > 0) {
            // count the K blocks delivered to each partial tile; whoever completes a tile finishes it
            __threadfence();
            epi_bar();
            if (threadIdx.x == 64) {
                uint32_t before[2] = {0, 0};
                for (uint32_t p = 0; p < parts; p++) before[p] = atomicAdd(args.counters + part_tile[p], part_blocks[p]);
                for (uint32_t p = 0; p < parts; p++) epi_flag[1 + p] = (before[p] + part_blocks[p] == num_kb) ? 1 : 0;
            }
            epi_bar();
            bool any = false;
            for (uint32_t p = 0; p < parts; p++) any |= epi_flag[1 + p] != 0;
            if (any) __threadfence();
            for (uint32_t p = 0; p < parts; p++) {
                if (epi_flag[1 + p] == 0) continue;
                const uint32_t tile = part_tile[p];
                const uint32_t n = tile * kDM + quarter * 32 + lane;
                if (n < args.n) {
                    float wsv, bias_f; int32_t bias_i;
                    channel_consts(n, wsv, bias_f, bias_i);
#pragma unroll 1
                    for (uint32_t c = 0; c < MT && c < args.rows; c += 32) {
                        int32_t v[32];
#pragma unroll
                        for (uint32_t i = 0; i < 32; i++) {
                            v[i] = 0;
                            if (c + i < args.rows) {
                                int32_t* slot = args.workspace + (size_t)(c + i) * args.n + n;
                                v[i] = __ldcg(slot);
                                __stcg(slot, 0);   // leave the workspace clean for the next call
                            }
                        }
                        finish_chunk(n, c, v, wsv, bias_f, bias_i);
                    }
                }
                if (threadIdx.x == 64) args.counters[tile] = 0u;
            }
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        nap(200);
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 3);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <uint32_t MT>
cudaError_t launch_t(const DecodeTcgen05Args& args, int sm_count, cudaStream_t stream) {
    using Cfg = DecodeCfg<MT>;
    cudaError_t e = ensure_dynamic_smem<decode_i8_tcgen05_kernel<MT>>(Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    const uint64_t units = (uint64_t)((args.n + kDM - 1) / kDM) * (args.kpad / kDK);
    const uint32_t grid = units < (uint64_t)sm_count ? (uint32_t)units : (uint32_t)sm_count;
    // This launch may begin (prologue, weight prefetch) while the kernel before it in the
    // stream is still finishing; the kernel waits before it touches the predecessor's data.
    return launch_pdl(decode_i8_tcgen05_kernel<MT>, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, args);
}

}  // namespace

uint32_t decode_token_slots(uint32_t rows) { return rows <= 32 ? 32u : rows <= 64 ? 64u : 128u; }

cudaError_t launch_decode_tcgen05(const DecodeTcgen05Args& args, int sm_count, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    if (args.rows > 128) return cudaErrorInvalidValue;
    if (args.rows <= 32) return launch_t<32>(args, sm_count, stream);
    if (args.rows <= 64) return launch_t<64>(args, sm_count, stream);
    return launch_t<128>(args, sm_count, stream);
}

}  // namespace vxb

// ---------------------------------------------------------------------------------------
// Allocation-free entry point (declared in include/vxb200_w8a8.h).
//
// The stream-K decode kernel needs scratch in global memory: an int32 [rows, d_out]
// workspace where CTAs that hold part of a tile's K range meet, one counter per 128-channel
// tile and a status word.  The library's ordinary entries take that scratch from buffers a
// VxbContext allocates with cudaMalloc.  This variant instead keeps it in a fixed array that
// is part of the loaded module, so a caller that is not allowed to allocate (a host with a
// sealed device-memory inventory, or code running while its stream is being captured) can
// still run the decode linear.  Every GPU that loads the library holds the array until exit.
// ---------------------------------------------------------------------------------------
#include "../../include/vxb200_w8a8.h"

#include <cstdio>
#include <mutex>

namespace {

constexpr uint32_t kNoAllocMaxRows = VXB_NOALLOC_MAX_ROWS;
constexpr uint32_t kNoAllocMaxChannels = VXB_NOALLOC_MAX_CHANNELS;
constexpr size_t kNoAllocStatusBytes = 256;
constexpr size_t kNoAllocCounterBytes = (size_t)(kNoAllocMaxChannels / 128) * 4;
constexpr size_t kNoAllocWorkspaceBytes = (size_t)kNoAllocMaxRows * kNoAllocMaxChannels * 4;
constexpr size_t kNoAllocBytes = kNoAllocStatusBytes + kNoAllocCounterBytes + kNoAllocWorkspaceBytes;

// In host code this name is only a stand-in for the symbol, not a device address: the
// address a kernel can use comes from cudaGetSymbolAddress on the device in question.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_ptr[kMaxDevices] = {};   // per device: address of its copy of the array
int g_noalloc_sms[kMaxDevices] = {};

typedef CUresult (*NoAllocEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Writes the reason into the caller's buffer (if any) and returns `code`.
struct NoAllocError {
    char* text; size_t bytes;
    int operator()(int code, const char* what, cudaError_t e = cudaSuccess) const {
        if (text && bytes) {
            if (e != cudaSuccess) snprintf(text, bytes, "%s: %s", what, cudaGetErrorString(e));
            else snprintf(text, bytes, "%s", what);
        }
        return code;
    }
};

bool noalloc_encode(CUtensorMap* map, const void* base, uint32_t rows, uint32_t row_bytes, uint32_t box_rows) {
    static NoAllocEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) return false;
        fn = (NoAllocEncodeFn)p;
    }
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int vxb_decode_linear_f32_noalloc(const int8_t* q, const float* row_scales, uint32_t rows,
                                             const int8_t* weight, const float* weight_scales,
                                             const float* bias, uint32_t d_out, uint32_t row_bytes,
                                             float* y, uint32_t ldy, void* stream, int wait,
                                             char* error, size_t error_bytes) {
    const NoAllocError noalloc_fail{error, error_bytes};
    if (error && error_bytes) error[0] = 0;
    if (!q || !row_scales || !weight || !weight_scales || !y)
        return noalloc_fail(0, "null argument");
    if (rows == 0 || d_out == 0) return 1;
    if (rows > kNoAllocMaxRows) {
        if (error && error_bytes)
            snprintf(error, error_bytes, "rows %u exceeds the fixed scratch (at most %u rows)", rows, kNoAllocMaxRows);
        return 0;
    }
    if (d_out > kNoAllocMaxChannels) {
        if (error && error_bytes)
            snprintf(error, error_bytes, "d_out %u exceeds the fixed scratch (at most %u output channels)",
                     d_out, kNoAllocMaxChannels);
        return 0;
    }
    if (row_bytes == 0 || row_bytes % 128 != 0) return noalloc_fail(0, "row_bytes must be a positive multiple of 128");
    if (ldy < d_out) return noalloc_fail(0, "output row stride smaller than d_out");
    if (((uintptr_t)q | (uintptr_t)weight) & 15u) return noalloc_fail(0, "q and weight must be 16-byte aligned");

    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return noalloc_fail(0, "cudaGetDevice", e);
    if (device < 0 || device >= kMaxDevices) return noalloc_fail(0, "device index out of range");
    {
        // One-time set-up for this device, with this device current: find where ITS copy of the
        // array lives and let the kernel use its shared-memory budget. Nothing is allocated.
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_ptr[device]) {
            unsigned char* ptr = nullptr;
            e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
            if (e != cudaSuccess || !ptr) return noalloc_fail(0, "cudaGetSymbolAddress(scratch)", e);
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess || sms <= 0) return noalloc_fail(0, "cudaDeviceGetAttribute", e);
            e = cudaFuncSetAttribute(vxb::decode_i8_tcgen05_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)vxb::DecodeCfg<32>::kSmemBytes);
            if (e != cudaSuccess) return noalloc_fail(0, "cudaFuncSetAttribute", e);
            g_noalloc_sms[device] = sms;
            g_noalloc_ptr[device] = ptr;
        }
    }
    unsigned char* scratch = g_noalloc_ptr[device];
    int* status = reinterpret_cast<int*>(scratch);
    uint32_t* counters = reinterpret_cast<uint32_t*>(scratch + kNoAllocStatusBytes);
    int32_t* workspace = reinterpret_cast<int32_t*>(scratch + kNoAllocStatusBytes + kNoAllocCounterBytes);
    cudaStream_t s = (cudaStream_t)stream;

    // The array keeps whatever the previous call left: counters and the part of the workspace
    // this call will use must start at zero (a memset node, not an allocation). The status block
    // in front of them is NOT cleared here: a word raised by an expired wait stays up until a
    // call with wait != 0 has reported it, so that a call enqueued with wait == 0 (or a graph
    // replay) cannot wipe the evidence of its predecessor's failure.
    const size_t used = kNoAllocCounterBytes + (size_t)rows * d_out * 4;
    e = cudaMemsetAsync(scratch + kNoAllocStatusBytes, 0, used, s);
    if (e != cudaSuccess) return noalloc_fail(-1, "cudaMemsetAsync(scratch)", e);

    vxb::DecodeTcgen05Args a;
    if (!noalloc_encode(&a.tmap_w, weight, d_out, row_bytes, 128) ||
        !noalloc_encode(&a.tmap_x, q, rows, row_bytes, 32))
        return noalloc_fail(0, "cuTensorMapEncodeTiled failed");
    a.rows = rows; a.n = d_out; a.kpad = row_bytes;
    a.epi = vxb::EpilogueParams{};
    a.epi.mode = vxb::kEpiF32; a.epi.row_scales = row_scales; a.epi.ws = weight_scales;
    a.epi.bias_f32 = bias; a.epi.out = y; a.epi.ld = ldy;
    a.workspace = workspace; a.counters = counters; a.status = status;
    const uint64_t units = (uint64_t)((d_out + 127) / 128) * (row_bytes / 128);
    const uint32_t grid = units < (uint64_t)g_noalloc_sms[device] ? (uint32_t)units : (uint32_t)g_noalloc_sms[device];
    vxb::decode_i8_tcgen05_kernel<32><<<grid, vxb::kThreads, vxb::DecodeCfg<32>::kSmemBytes, s>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return noalloc_fail(-1, "kernel launch", e);
    if (wait) {
        int host_status = 0;
        e = cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return noalloc_fail(-1, "waiting for the result", e);
        if (host_status != 0) {
            // reported once: lower the word and clear everything an aborted launch may have left
            cudaMemsetAsync(scratch, 0, sizeof(int), s);
            cudaMemsetAsync(scratch + kNoAllocStatusBytes, 0, kNoAllocBytes - kNoAllocStatusBytes, s);
            cudaStreamSynchronize(s);
            return noalloc_fail(-1, "a bounded device wait expired in this call or in an earlier call made with "
                                    "wait == 0; outputs since the last waited call are invalid");
        }
    }
    return 1;
}
