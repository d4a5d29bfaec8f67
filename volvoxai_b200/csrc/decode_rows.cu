// K3: decode-shaped W8A8 linear (rows <= 128) in which every CTA owns whole output
// channels.  HBM-bound: the int8 weights are streamed exactly once, every SM streams the
// same number of bytes, and no partial sum ever leaves the CTA (no workspace, no atomics).
//
//   acc[m,n] = sum_k q[m,k] * w[n,k]
//
// The N output channels are dealt out in equal contiguous ranges, one per SM: C =
// ceil(N / #SMs) channels per CTA, processed as ceil(C/256) tiles of T <= 256 channels.  A
// tile's weights arrive through TMA boxes of exactly T rows x 128 K-bytes (no byte of another
// CTA's channels is fetched) into a deep ring of small stages and are the UMMA N operand;
// the few activation rows (TMA box of MT = 8..128 token slots, zero-filled beyond `rows`) are
// the UMMA M operand.  A tcgen05.mma takes about one cycle per M row whatever N is, so this
// orientation (M = 64 for up to 64 tokens) keeps the tensor pipe far ahead of the weight
// stream.  The instruction always spans 64/128 M rows and a multiple of 16 N rows: the rows
// beyond the boxes read stale shared memory and produce accumulator entries nobody reads.
// Accumulators are int32 in TMEM; four epilogue warps apply the fused epilogue, one thread
// per token row.
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
constexpr uint32_t kIssuerWarps = 4;        // warps 1..4 may issue MMAs
constexpr uint32_t kXWarp = 1 + kIssuerWarps + 4;             // first activation-producer warp
constexpr uint32_t kThreads = 32 * (kXWarp + kIssuerWarps);   // weight producer, issuers, 4 epilogue warps, activation producers
constexpr uint32_t kEpiBase = 32 * (1 + kIssuerWarps);
constexpr uint32_t kMaxStages = 32;
constexpr uint32_t kMaxTile = 256;         // channels per tile (UMMA N limit)
constexpr uint32_t kRingBudgetDeep = 150 * 1024;  // one CTA per SM; the ring takes most of its shared memory
constexpr uint32_t kXposePitch = 33;       // ints per row of the epilogue transpose buffer

template <uint32_t MT> struct RowsCfg {
    static constexpr uint32_t kXBytes = MT * kRK < 1024 ? 1024 : MT * kRK;  // activation stage
    static constexpr uint32_t kUmmaM = MT <= 64 ? 64 : 128;                  // rows the MMA spans
};

struct RowsLayout {       // dynamic shared memory, offsets from a 1024-byte aligned base
    uint32_t stages, w_bytes, x_bytes, umma_m, umma_n;
    __host__ __device__ uint32_t w_off(uint32_t s) const { return s * w_bytes; }
    __host__ __device__ uint32_t w_end() const {
        // the MMA reads umma_n x 128 bytes from a weight stage
        const uint32_t reach = (stages - 1) * w_bytes + umma_n * kRK;
        return stages * w_bytes > reach ? stages * w_bytes : reach;
    }
    __host__ __device__ uint32_t x_off(uint32_t s) const { return round_up(w_end(), 1024u) + s * x_bytes; }
    __host__ __device__ uint32_t x_end() const {
        // ... and umma_m x 128 bytes from an activation stage
        const uint32_t ring = x_off(0) + stages * x_bytes;
        const uint32_t reach = x_off(stages - 1) + umma_m * kRK;
        return ring > reach ? ring : reach;
    }
    __host__ __device__ uint32_t consts_off() const { return x_end(); }   // float ws[256], bias[256]
    __host__ __device__ uint32_t xpose_off() const { return consts_off() + 2 * kMaxTile * 4; }  // int32 [128][33]
    __host__ __device__ uint32_t bars_off() const { return xpose_off() + 128 * kXposePitch * 4; }
    __host__ __device__ uint32_t misc_off() const { return bars_off() + (2 * kMaxStages + 4) * 8; }
    __host__ __device__ uint32_t total() const { return misc_off() + 32 + 128 * 4 + 1024; }
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <uint32_t MT>
__global__ void __launch_bounds__(kThreads, 1)
decode_rows_kernel(const __grid_constant__ DecodeRowsArgs args) {
    using Cfg = RowsCfg<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const RowsLayout lay{args.stages, args.w_stage_bytes, Cfg::kXBytes, Cfg::kUmmaM, args.umma_n};
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
    float* s_ws = reinterpret_cast<float*>(base + lay.consts_off());
    float* s_bias = s_ws + kMaxTile;
    int32_t* s_xpose = reinterpret_cast<int32_t*>(base + lay.xpose_off());

    const uint32_t num_kb = args.kpad / kRK;
    const uint32_t tiles = args.tiles_per_cta;
    const uint32_t first_channel = blockIdx.x * tiles * args.tile_rows;
    const uint32_t stage_tx = args.tile_rows * kRK + MT * kRK;   // bytes one stage receives
    const bool double_buffered = tiles > 1;                       // else one accumulator, reused
    const uint32_t acc_stride = args.tmem_cols / 2;              // columns between the two accumulators

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        mbar_init(tmem_full(0), args.issuers); mbar_init(tmem_full(1), 1);
        for (uint32_t b = 0; b < 2; b++) mbar_init(tmem_empty(b), 128);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&args.tmap_w);
        prefetch_tmap(&args.tmap_x);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_ptr), args.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    if (threadIdx.x == 0) pdl_release();

    if (warp == 0) {
        // ---------------- weight producer ----------------
        // One thread, and every clock of it counts: with few channels per CTA a K block is only
        // a few KB, so the loop below is kept to address increments (no divisions, no layout
        // arithmetic). Weights depend on nothing that runs before this kernel, so this thread
        // never waits for the preceding kernel; the activation tiles come from their own thread.
        if (lane == 0 && args.issuers == 1) {   // with several issuers, each loads its own weight tiles
            const uint32_t total = tiles * num_kb;
            const uint32_t w0 = w_addr(0), f0 = full(0), e0 = empty(0), wstep = lay.w_bytes;
            uint32_t w_sm = w0, fb = f0, eb = e0, stage = 0, phase = 0, kb = 0, armed = 0;
            int32_t kcoord = 0, channel = (int32_t)first_channel;
            bool ok = true;
            for (uint32_t i = 0; i < total; i++) {
                if (i >= stages && !mbar_wait(eb, phase ^ 1u, abort_flag)) { ok = false; break; }
                mbar_expect_tx(fb, stage_tx);
                tma_load_2d(w_sm, &args.tmap_w, fb, kcoord, channel);
                armed |= 1u << stage;
                kcoord += (int32_t)kRK;
                if (++kb == num_kb) { kb = 0; kcoord = 0; channel += (int32_t)args.tile_rows; }
                w_sm += wstep; fb += 8; eb += 8;
                if (++stage == stages) { stage = 0; phase ^= 1u; w_sm = w0; fb = f0; eb = e0; }
            }
            if (!ok) {
                // drain: give this CTA's own copies in flight a bounded time to land
                for (uint32_t s = 0; s < stages; s++) {
                    if (!(armed & (1u << s))) continue;
                    for (uint32_t n = 0; n < 2000; n++) {
                        if (mbar_try_wait(full(s), 0u) || mbar_try_wait(full(s), 1u)) break;
                        __nanosleep(500);
                    }
                }
            }
        }
    } else if (warp >= kXWarp) {
        // ---------------- activation producers ----------------
        // Starting a TMA copy costs the issuing thread some 200 ns whatever the box size, so one
        // thread cannot feed small K blocks fast enough: producer p of P (= the issuer count)
        // loads the activation tiles of the K blocks p, p+P, ... into its own stages p, p+P, ...
        const uint32_t p = warp - kXWarp, P = args.issuers;
        if (lane == 0 && p < P) {
            const uint32_t total = tiles * num_kb, own = stages / P;
            const uint32_t x0 = x_addr(p), f0 = full(p), e0 = empty(p), xstep = lay.x_bytes * P;
            uint32_t x_sm = x0, fb = f0, eb = e0, stage = 0, phase = 0, kb = p % num_kb, uses = 0;
            pdl_wait();   // the activations are the preceding kernel's output
            for (uint32_t i = p; i < total; i += P, uses++) {
                if (uses >= own && !mbar_wait(eb, phase ^ 1u, abort_flag)) break;
                tma_load_2d(x_sm, &args.tmap_x, fb, (int32_t)(kb * kRK), 0);
                kb += P; while (kb >= num_kb) kb -= num_kb;
                x_sm += xstep; fb += 8 * P; eb += 8 * P;
                if (++stage == own) { stage = 0; phase ^= 1u; x_sm = x0; fb = f0; eb = e0; }
            }
        }
    } else if (warp <= kIssuerWarps && args.issuers > 1) {
        // ---------------- MMA issuers, several: issuer ii takes K blocks ii, ii+I, ... into its own
        // accumulator (one thread can start an MMA only every ~70 clocks, far slower than the tensor
        // pipe finishes a narrow one; the epilogue adds the accumulators up, integers: exact) ------
        const uint32_t ii = warp - 1u;
        if (lane == 0 && ii < args.issuers) {
            const uint32_t idesc = make_idesc(Cfg::kUmmaM, args.umma_n);
            const uint32_t d_tmem = tmem_base + ii * args.acc_cols;
            bool ok = true;
            // Stage index = kb mod stages and stages is a multiple of the issuer count, so this
            // issuer owns the stages ii, ii+I, ... (its j-th own stage is ii + I*j). It also loads
            // the WEIGHT tiles of its own K blocks (weights depend on nothing before this kernel, so
            // there is no wait for the preceding kernel here): first it fills its stages, then after
            // each K block it re-arms the stage it consumed `lag` blocks earlier, whose MMAs have
            // finished by then. Increments only, no divisions.
            const uint32_t I = args.issuers, own = stages / I, lag = own > 2 ? 2u : own - 1u;
            const uint32_t wstep = lay.w_bytes * I, xstep = lay.x_bytes * I;
            const uint32_t w0 = w_addr(ii), x0 = x_addr(ii), f0 = full(ii), e0 = empty(ii);
            const int32_t channel = (int32_t)first_channel;
            uint32_t load_kb = ii, lw = w0, lf = f0;               // next K block to load and its stage
            for (uint32_t j = 0; j < own && load_kb < num_kb; j++) {
                mbar_expect_tx(lf, stage_tx);
                tma_load_2d(lw, &args.tmap_w, lf, (int32_t)(load_kb * kRK), channel);
                load_kb += I; lw += wstep; lf += 8 * I;
            }
            // refill cursor: the stage consumed `lag` blocks ago
            uint32_t rw = w0, rf = f0, re = e0, rstage = 0, rphase = 0;
            uint32_t wa = w0, xa = x0, fb = f0, eb = e0, cstage = 0, cphase = 0, first = 1, done = 0;
            for (uint32_t i = ii; i < num_kb; i += I, done++) {
                if (!mbar_wait(fb, cphase, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t da = make_smem_desc(xa), db = make_smem_desc(wa);
#pragma unroll
                for (uint32_t k = 0; k < kRK / kUmmaK; k++)   // +32 bytes of K = +2 in the descriptor's address field
                    umma_i8(d_tmem, da + 2u * k, db + 2u * k, idesc, (first && k == 0u) ? 0u : 1u);
                first = 0;
                umma_commit(eb);
                wa += wstep; xa += xstep; fb += 8 * I; eb += 8 * I;
                if (++cstage == own) { cstage = 0; cphase ^= 1u; wa = w0; xa = x0; fb = f0; eb = e0; }
                if (done >= lag && load_kb < num_kb) {
                    if (!mbar_wait(re, rphase, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(rf, stage_tx);
                    tma_load_2d(rw, &args.tmap_w, rf, (int32_t)(load_kb * kRK), channel);
                    load_kb += I;
                    rw += wstep; rf += 8 * I; re += 8 * I;
                    if (++rstage == own) { rstage = 0; rphase ^= 1u; rw = w0; rf = f0; re = e0; }
                }
            }
            if (ok) umma_commit(tmem_full(0));
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer, single ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(Cfg::kUmmaM, args.umma_n);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t t = 0; ok && t < tiles; t++) {
                if (!mbar_wait(tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_stride;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(full(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t wa = w_addr(stage), xa = x_addr(stage);
#pragma unroll
                    for (uint32_t k = 0; k < kRK / kUmmaK; k++)   // A = activations, B = weights
                        umma_i8(d_tmem, make_smem_desc(xa + k * kUmmaK), make_smem_desc(wa + k * kUmmaK),
                                idesc, (kb | k) != 0u ? 1u : 0u);
                    umma_commit(empty(stage));
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(tmem_full(acc));
                if (double_buffered) { acc ^= 1u; if (acc == 0) acc_phase ^= 1u; }
                else acc_phase ^= 1u;
            }
        }
    } else if (warp > kIssuerWarps && warp < kXWarp) {
        // ---------------- epilogue (last four warps): thread = one token row ----------------
        const uint32_t quarter = warp & 3u;
        const uint32_t e = threadIdx.x - kEpiBase;
        const EpilogueParams& ep = args.epi;
        const float zero_f = __int2float_rn(ep.out_zero);
        const float lo_f = __int2float_rn(ep.out_lo), hi_f = __int2float_rn(ep.out_hi);
        // accumulator row r sits in TMEM lane r (M = 128) or in lane 32*(r/16) + r%16 (M = 64)
        const uint32_t m = Cfg::kUmmaM == 128 ? quarter * 32 + lane : quarter * 16 + lane;
        const bool m_ok = (Cfg::kUmmaM == 128 || lane < 16) && m < args.rows;

        uint32_t acc = 0, acc_phase = 0;
        for (uint32_t t = 0; t < tiles; t++) {
            const uint32_t c0 = first_channel + t * args.tile_rows;
            // per-channel constants of this tile: weight metadata, independent of the preceding
            // kernel, staged while the MMAs run
            epi_bar();
            for (uint32_t i = e; i < args.tile_rows; i += 128) {
                const uint32_t n = c0 + i;
                float wsv = 0.0f, bv = 0.0f;
                if (n < args.n && ep.mode != kEpiAcc) {
                    wsv = __ldg(ep.ws + n);
                    if (ep.mode == kEpiF32) bv = ep.bias_f32 ? __ldg(ep.bias_f32 + n) : 0.0f;
                    else bv = __int_as_float(ep.bias_i32 ? __ldg(ep.bias_i32 + n) : 0);
                }
                s_ws[i] = wsv; s_bias[i] = bv;
            }
            if (t == 0) {
                // from here on: reads of what the preceding kernel wrote, writes of what it may read
                pdl_wait();
                if (e < 128) s_as[e] = (e < args.rows && ep.mode != kEpiAcc) ? __ldg(ep.row_scales + e) : 0.0f;
            }
            const bool waited = mbar_wait(tmem_full(acc), acc_phase, abort_flag);
            // make the give-up decision uniform across the four epilogue warps (the first
            // barrier also publishes the staged constants)
            epi_bar();
            if (e == 0) epi_flag[0] = (*abort_flag != 0 || !waited) ? 1 : 0;
            epi_bar();
            if (epi_flag[0]) break;
            tc_fence_after();

            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * acc_stride;
            const uint32_t left = args.n > c0 ? args.n - c0 : 0u;
            const uint32_t valid = left < args.tile_rows ? left : args.tile_rows;
            // TMEM hands each thread one token row; the stores want one channel per lane. Each
            // 32-channel chunk is therefore transposed through shared memory: row threads park
            // their 32 values, then thread (lane = channel, warp = row group) finishes rows
            // warp, warp+4, ... so that every store instruction covers 32 consecutive channels.
            const uint32_t row_group = e >> 5;
#pragma unroll 1
            for (uint32_t c = 0; c < args.umma_n; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                for (uint32_t a = 1; a < args.issuers; a++) {   // add the other issuers' accumulators
                    uint32_t more[32];
                    tmem_ld32(taddr + a * args.acc_cols + c, more);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) r[i] += more[i];
                }
                if (c >= valid) continue;          // uniform: nothing of this chunk is stored
                epi_bar();                           // the previous chunk has been read
                if (m_ok) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; i++) s_xpose[m * kXposePitch + i] = (int32_t)r[i];
                }
                epi_bar();
                const uint32_t col = c + lane;
                if (col < valid) {
                    const float wsv = s_ws[col];
                    const float bf = s_bias[col];
                    const int32_t bi = __float_as_int(bf);
                    const size_t at = (size_t)c0 + col;
                    for (uint32_t mm = row_group; mm < args.rows; mm += 4) {
                        const int32_t v = s_xpose[mm * kXposePitch + lane];
                        const float asv = s_as[mm];
                        if (ep.mode == kEpiF32) {
                            ((float*)ep.out)[(size_t)mm * ep.ld + at] = epi_f32(v, asv, wsv, bf);
                        } else if (ep.mode == kEpiI8) {
                            const int32_t qv = (ep.fast_div != 0 && div_const_row_ok(asv))
                                ? epi_i8_v2<true>(v + bi, asv, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero)
                                : epi_i8_v2<false>(v + bi, asv, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
                            ((int8_t*)ep.out)[(size_t)mm * ep.ld + at] = (int8_t)qv;
                        } else {
                            ((int32_t*)ep.out)[(size_t)mm * ep.ld + at] = v;
                        }
                    }
                }
            }
            // the accumulator has been consumed: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            mbar_arrive(tmem_empty(acc));
            if (double_buffered) { acc ^= 1u; if (acc == 0) acc_phase ^= 1u; }
            else acc_phase ^= 1u;
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
    if (warp == 1) tmem_dealloc(tmem_base, args.tmem_cols);
}

template <uint32_t MT>
cudaError_t launch_t(DecodeRowsArgs args, cudaStream_t stream) {
    using Cfg = RowsCfg<MT>;
    args.umma_n = round_up(args.tile_rows, 16u);
    // TMEM: a power-of-two number of columns >= umma_n per accumulator; a CTA with one tile
    // allocates twice that too (the second half stays unused) so acc_stride is uniform, except
    // that 256-column tiles with a single tile allocate exactly 256 so two CTAs still fit an SM.
    uint32_t cols = 32;
    while (cols < args.umma_n) cols *= 2;
    args.acc_cols = cols;
    // ring depth: as many stages as fit the budget
    const uint32_t per_stage = args.w_stage_bytes + Cfg::kXBytes;
    uint32_t stages = kRingBudgetDeep / per_stage;
    if (stages < 2) stages = 2;
    if (stages > kMaxStages) stages = kMaxStages;
    // several issuers (each with its own accumulator) while they fit the 512 TMEM columns.
    // Issuer ii takes the K blocks
    // kb = ii (mod issuers); the ring depth is made a multiple of the issuer count so that each
    // stage (kb mod stages) is only ever waited on by one issuer, in order - a parity wait on an
    // mbarrier is only meaningful for a waiter that saw the previous phase complete.
    uint32_t issuers = 1;
    if (args.tiles_per_cta == 1) {
        issuers = 512 / cols;
        if (issuers > kIssuerWarps) issuers = kIssuerWarps;
        const uint32_t num_kb = args.kpad / kRK;
        while (issuers > 1 && (issuers > num_kb || issuers > stages)) issuers /= 2;
    }
    stages -= stages % issuers;
    args.stages = stages;
    args.issuers = issuers;
    args.tmem_cols = issuers > 1 ? issuers * cols : ((args.tiles_per_cta == 1 && cols == 256) ? 256u : 2 * cols);
    if (args.tmem_cols < 32) args.tmem_cols = 32;
    const RowsLayout lay{stages, args.w_stage_bytes, Cfg::kXBytes, Cfg::kUmmaM, args.umma_n};
    const uint32_t smem = lay.total();
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
    const uint32_t tiles = (per_cta + kMaxTile - 1) / kMaxTile;
    *tiles_per_cta = tiles;
    *tile_rows = (per_cta + tiles - 1) / tiles;
}

cudaError_t launch_decode_rows(const DecodeRowsArgs& args, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    if (args.rows > 128 || args.tile_rows == 0 || args.tile_rows > kMaxTile) return cudaErrorInvalidValue;
    const uint32_t mt = decode_rows_token_slots(args.rows);
    if (mt == 8) return launch_t<8>(args, stream);
    if (mt == 16) return launch_t<16>(args, stream);
    if (mt == 32) return launch_t<32>(args, stream);
    if (mt == 64) return launch_t<64>(args, stream);
    return launch_t<128>(args, stream);
}

}  // namespace vxb
