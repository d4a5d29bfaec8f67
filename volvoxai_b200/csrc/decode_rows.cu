// K3: decode-shaped W8A8 linear (rows <= 128) in which every CTA owns whole output
// channels.  HBM-bound: the int8 weights are streamed exactly once, every SM streams the
// same number of bytes, and no partial sum ever leaves the CTA (no workspace, no atomics).
//
//   acc[m,n] = sum_k q[m,k] * w[n,k]
//
// The N output channels are dealt out in equal contiguous ranges, one per SM: C =
// ceil(N / #SMs) channels per CTA, processed as ceil(C/128) tiles of T <= 128 channels.  A
// tile's weights arrive through TMA boxes of exactly T rows x 128 K-bytes (so no byte of
// another CTA's channels is fetched) into a deep ring of small stages; the tile is the UMMA
// M operand (the instruction always spans 128 rows: rows >= T read stale shared memory and
// produce accumulator lanes nobody reads) and the few activation rows are the UMMA N operand
// (MT = 8..128 token slots, zero-filled by TMA beyond `rows`).  Accumulators are int32 in
// TMEM, double buffered (and, for few token slots, split four ways over the K-slices of a
// stage so that consecutive MMAs do not wait on one another); four epilogue warps add them
// up and apply the fused epilogue, one thread per channel.
//
// Launched with programmatic stream serialization: the prologue and the first ring-full of
// weight tiles (which depend on nothing) are issued before griddepcontrol.wait, i.e. while
// the kernel that produces the activations is still running.
//
// Reference counterparts: the decode kernels vx_packed_cuda_a8_columns and the fused GEMV
// family (native/src/backends/cuda/kernels/cuda_forward_llm_kernels.inc:254-459,
// cuda_forward_gemv_pair_kernels.inc:155-1711), one row x 32 columns per CTA with the
// activation row re-quantized per column tile; and the CPU single-row route
// (native/src/kernels/packed_linear_ops.inc:1471-1535).
//
// All mbarrier waits are bounded; on expiry the kernel raises the status word, drains and
// frees its TMEM.  No CTA waits for another CTA.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kRK = 128;              // K bytes per stage
constexpr uint32_t kThreads = 192;         // producer warp, MMA warp, 4 epilogue warps
constexpr uint32_t kMaxStages = 24;
constexpr uint32_t kUmmaRows = 128;        // rows the MMA reads from a weight stage
constexpr uint32_t kRingBudget = 96 * 1024;

template <uint32_t MT> struct RowsCfg {
    static constexpr uint32_t kXBytes = MT * kRK < 1024 ? 1024 : MT * kRK;
    static constexpr uint32_t kAccStride = MT < 32 ? 32 : MT;          // TMEM columns per accumulator
    // With few token slots an MMA is short but its latency is not, and MMAs into one
    // accumulator serialise. The four K-slices of a stage therefore go to kAccs independent
    // accumulators, which the epilogue adds up (integers: exact).
    static constexpr uint32_t kAccs = MT <= 32 ? 4 : MT <= 64 ? 2 : 1;
    static constexpr uint32_t kBufCols = kAccs * kAccStride;           // one of the two buffers
    static constexpr uint32_t kTmemCols = 2 * kBufCols;                // 256 for every MT
};

struct RowsLayout {       // dynamic shared memory, offsets from a 1024-byte aligned base
    uint32_t stages, w_bytes, x_bytes;
    __host__ __device__ uint32_t w_off(uint32_t s) const { return s * w_bytes; }
    __host__ __device__ uint32_t x_off(uint32_t s) const { return stages * w_bytes + s * x_bytes; }
    // the MMA of the last stage reads kUmmaRows x 128 bytes from its weight buffer
    __host__ __device__ uint32_t data_end() const {
        const uint32_t ring = stages * (w_bytes + x_bytes);
        const uint32_t reach = (stages - 1) * w_bytes + kUmmaRows * kRK;
        return ring > reach ? ring : reach;
    }
    __host__ __device__ uint32_t bars_off() const { return data_end(); }
    __host__ __device__ uint32_t misc_off() const { return bars_off() + (2 * kMaxStages + 4) * 8; }
    __host__ __device__ uint32_t total(uint32_t mt) const { return misc_off() + 32 + mt * 4 + 1024; }
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <uint32_t MT>
__global__ void __launch_bounds__(kThreads, 2)
decode_rows_kernel(const __grid_constant__ DecodeRowsArgs args) {
    using Cfg = RowsCfg<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const RowsLayout lay{args.stages, args.w_stage_bytes, Cfg::kXBytes};
    const uint32_t stages = args.stages;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto w_addr = [&](uint32_t s) { return smem_u32(base + lay.w_off(s)); };
    auto x_addr = [&](uint32_t s) { return smem_u32(base + lay.x_off(s)); };
    auto full = [&](uint32_t s) { return smem_u32(base + lay.bars_off() + s * 8); };
    auto empty = [&](uint32_t s) { return smem_u32(base + lay.bars_off() + (kMaxStages + s) * 8); };
    auto tmem_full = [&](uint32_t b) { return smem_u32(base + lay.bars_off() + (2 * kMaxStages + b) * 8); };
    auto tmem_empty = [&](uint32_t b) { return smem_u32(base + lay.bars_off() + (2 * kMaxStages + 2 + b) * 8); };
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(base + lay.misc_off());
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + lay.misc_off() + 4);
    volatile int* epi_flag = reinterpret_cast<volatile int*>(base + lay.misc_off() + 8);
    float* s_as = reinterpret_cast<float*>(base + lay.misc_off() + 32);

    const uint32_t num_kb = args.kpad / kRK;
    const uint32_t tiles = args.tiles_per_cta;
    const uint32_t first_channel = blockIdx.x * tiles * args.tile_rows;
    const uint32_t stage_tx = args.tile_rows * kRK + MT * kRK;   // bytes one stage receives

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (uint32_t b = 0; b < 2; b++) { mbar_init(tmem_full(b), 1); mbar_init(tmem_empty(b), 128); }
        *abort_flag = 0;
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
            const uint32_t total = tiles * num_kb;
            // Every CTA walks K from a different starting block (integer sums do not care about
            // the order): otherwise all CTAs ask L2 for the same activation line at the same time.
            const uint32_t rot = (blockIdx.x * 5u) % num_kb;
            // Weights depend on nothing that runs before this kernel: fill the ring with weight
            // tiles first, then wait for the activations' producer and add the activation tiles.
            const uint32_t ahead = total < stages ? total : stages;
            for (uint32_t i = 0; i < ahead; i++) {
                const uint32_t t = i / num_kb, kb = (i % num_kb + rot) % num_kb;
                mbar_expect_tx(full(i), stage_tx);
                tma_load_2d(w_addr(i), &args.tmap_w, full(i), (int32_t)(kb * kRK),
                            (int32_t)(first_channel + t * args.tile_rows));
            }
            pdl_wait();
            uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
            bool ok = true;
            for (uint32_t i = 0; ok && i < total; i++) {
                const uint32_t t = i / num_kb, kb = (i % num_kb + rot) % num_kb;
                if (i >= ahead) {
                    if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(full(stage), stage_tx);
                    tma_load_2d(w_addr(stage), &args.tmap_w, full(stage), (int32_t)(kb * kRK),
                                (int32_t)(first_channel + t * args.tile_rows));
                }
                tma_load_2d(x_addr(stage), &args.tmap_x, full(stage), (int32_t)(kb * kRK), 0);
                armed |= 1u << stage;
                armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                if (++stage == stages) { stage = 0; phase ^= 1u; }
            }
            if (!ok) {
                for (uint32_t s = 0; s < stages; s++) {
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
            constexpr uint32_t idesc = make_idesc(kUmmaRows, MT);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t t = 0; ok && t < tiles; t++) {
                if (!mbar_wait(tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::kBufCols;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(full(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t wa = w_addr(stage), xa = x_addr(stage);
#pragma unroll
                    for (uint32_t k = 0; k < kRK / kUmmaK; k++)
                        umma_i8(d_tmem + (k % Cfg::kAccs) * Cfg::kAccStride,
                                make_smem_desc(wa + k * kUmmaK), make_smem_desc(xa + k * kUmmaK),
                                idesc, (kb != 0u || k >= Cfg::kAccs) ? 1u : 0u);
                    umma_commit(empty(stage));
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
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

        uint32_t acc = 0, acc_phase = 0;
        for (uint32_t t = 0; t < tiles; t++) {
            const uint32_t in_tile = quarter * 32 + lane;
            const uint32_t n = first_channel + t * args.tile_rows + in_tile;
            const bool n_ok = in_tile < args.tile_rows && n < args.n;
            // per-channel constants are in flight while the MMAs run
            const float wsv = (n_ok && ep.mode != kEpiAcc) ? __ldg(ep.ws + n) : 0.0f;
            const float bias_f = (n_ok && ep.mode == kEpiF32 && ep.bias_f32) ? __ldg(ep.bias_f32 + n) : 0.0f;
            const int32_t bias_i = (n_ok && ep.mode == kEpiI8 && ep.bias_i32) ? __ldg(ep.bias_i32 + n) : 0;

            const bool waited = mbar_wait(tmem_full(acc), acc_phase, abort_flag);
            // make the give-up decision uniform across the four epilogue warps
            epi_bar();
            if (threadIdx.x == 64) epi_flag[0] = (*abort_flag != 0 || !waited) ? 1 : 0;
            epi_bar();
            if (epi_flag[0]) break;
            tc_fence_after();

            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * Cfg::kBufCols;
#pragma unroll 1
            for (uint32_t c = 0; c < MT; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t a = 1; a < Cfg::kAccs; a++) {
                    uint32_t more[32];
                    tmem_ld32(taddr + a * Cfg::kAccStride + c, more);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) r[i] += more[i];
                }
                if (c >= args.rows || !n_ok) continue;
#pragma unroll
                for (uint32_t i = 0; i < 32; i++) {
                    const uint32_t m = c + i;
                    if (i >= MT || m >= args.rows) continue;
                    const size_t at = (size_t)m * ep.ld + n;
                    const int32_t v = (int32_t)r[i];
                    if (ep.mode == kEpiAcc) {
                        ((int32_t*)ep.out)[at] = v;
                    } else if (ep.mode == kEpiF32) {
                        ((float*)ep.out)[at] = epi_f32(v, s_as[m], wsv, bias_f);
                    } else {
                        const float as = s_as[m];
                        const int32_t qv = (ep.fast_div != 0 && div_const_row_ok(as))
                            ? epi_i8_v2<true>(v + bias_i, as, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero)
                            : epi_i8_v2<false>(v + bias_i, as, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                        ((int8_t*)ep.out)[at] = (int8_t)qv;
                    }
                }
            }
            // the accumulator has been consumed: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            mbar_arrive(tmem_empty(acc));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    // ---------------- teardown ----------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        nap(200);
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 4);
        __syncthreads();
    }
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <uint32_t MT>
cudaError_t launch_t(DecodeRowsArgs args, cudaStream_t stream) {
    using Cfg = RowsCfg<MT>;
    // ring depth: as many stages as fit the budget (two CTAs of consecutive launches share an SM)
    const uint32_t per_stage = args.w_stage_bytes + Cfg::kXBytes;
    uint32_t stages = kRingBudget / per_stage;
    if (stages < 2) stages = 2;
    if (stages > kMaxStages) stages = kMaxStages;
    args.stages = stages;
    const RowsLayout lay{stages, args.w_stage_bytes, Cfg::kXBytes};
    const uint32_t smem = lay.total(MT);
    static uint32_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_rows_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    const uint32_t per_cta = args.tiles_per_cta * args.tile_rows;
    const uint32_t grid = (args.n + per_cta - 1) / per_cta;
    return launch_pdl(decode_rows_kernel<MT>, dim3(grid), dim3(kThreads), smem, stream, args);
}

}  // namespace

uint32_t decode_rows_token_slots(uint32_t rows) {
    return rows <= 8 ? 8u : rows <= 16 ? 16u : rows <= 32 ? 32u : rows <= 64 ? 64u : 128u;
}

void decode_rows_plan(uint32_t n, int sm_count, uint32_t* tile_rows, uint32_t* tiles_per_cta) {
    uint32_t per_cta = (n + (uint32_t)sm_count - 1) / (uint32_t)sm_count;
    if (per_cta < 8) per_cta = n < 8 ? n : 8;
    const uint32_t tiles = (per_cta + 127) / 128;
    *tiles_per_cta = tiles;
    *tile_rows = (per_cta + tiles - 1) / tiles;
}

cudaError_t launch_decode_rows(const DecodeRowsArgs& args, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    if (args.rows > 128 || args.tile_rows == 0 || args.tile_rows > 128) return cudaErrorInvalidValue;
    const uint32_t mt = decode_rows_token_slots(args.rows);
    if (mt == 8) return launch_t<8>(args, stream);
    if (mt == 16) return launch_t<16>(args, stream);
    if (mt == 32) return launch_t<32>(args, stream);
    if (mt == 64) return launch_t<64>(args, stream);
    return launch_t<128>(args, stream);
}

}  // namespace vxb
