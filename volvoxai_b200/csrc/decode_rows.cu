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
#include "quantize.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kRK = 128;              // K bytes per stage
constexpr uint32_t kMaxStages = 48;
constexpr uint32_t kMaxTile = 256;         // channels per tile (UMMA N limit)
// Two CTAs fit an SM (shared memory, registers and TMEM columns are all held to half of it), so
// that the CTAs of the NEXT launch in the stream become resident while this launch still runs:
// their prologue and the first ring-full of their weights overlap this launch's tail, and the
// weight stream from HBM does not stop between back-to-back decode kernels.
//
// That only pays while a CTA's whole weight share is not much larger than the ring it can hold
// in half an SM: then most of it is already in shared memory when the preceding kernel ends.
// CTAs with more to stream run alone on their SM (kPair = false) with a ring twice as deep -
// the stream rate follows the bytes in flight - and with up to eight MMA issuers.
constexpr uint32_t kPairSmemBytes = (233472 - 2 * 1024) / 2;   // 228 KB per SM, 1 KB reserved per CTA
constexpr uint32_t kSoloSmemBytes = 200 * 1024;
constexpr uint32_t kPairShareBytes = 160 * 1024;               // largest weight share per CTA run in pairs

template <bool PAIR> struct ModeCfg {
    static constexpr uint32_t kIssuerWarps = PAIR ? 4 : 8;     // warps 0.. may issue MMAs
    static constexpr uint32_t kProducerWarps = PAIR ? 4 : 5;   // TMA warps: weight producers, then one for the activations
    static constexpr uint32_t kXWarp = kIssuerWarps + 4;       // first producer warp (4 epilogue warps before it)
    static constexpr uint32_t kThreads = 32 * (kXWarp + kProducerWarps);
    static constexpr uint32_t kEpiBase = 32 * kIssuerWarps;
    static constexpr uint32_t kSmemBytes = PAIR ? kPairSmemBytes : kSoloSmemBytes;
    static constexpr uint32_t kTmemCols = PAIR ? 256 : 512;
    static constexpr uint32_t kCtasPerSm = PAIR ? 2 : 1;
};
constexpr uint32_t kXposePitch = 33;       // ints per row of the epilogue transpose buffer

template <uint32_t MT> struct RowsCfg {
    static constexpr uint32_t kXAtom = MT * kRK;   // one [MT x 128 B] activation tile (MT >= 8: whole swizzle atoms)
    static constexpr uint32_t kUmmaM = MT <= 64 ? 64 : 128;                  // rows the MMA spans
    static constexpr bool kParkAll = MT <= 64;   // up to 64 token rows (M = 64 layout): the epilogue parks the whole tile at once
    // parking area of the epilogue: the whole [rows, umma_n] tile (pitch umma_n + 4 ints) for few
    // token rows, else two [MT][33] buffers for 32-channel chunks
    // whole 32-channel chunks per row, + 4 ints (pitch = 4 mod 32: 16-byte row stores hit distinct banks)
    static __host__ __device__ uint32_t park_pitch(uint32_t umma_n) { return round_up(umma_n, 32u) + 4u; }
    static __host__ __device__ uint32_t xpose_bytes(uint32_t rows, uint32_t umma_n) {
        return kParkAll ? round_up(rows, 8u) * park_pitch(umma_n) * 4u : 2u * MT * kXposePitch * 4u;
    }
};

constexpr uint32_t kMaxXSlots = 8;
constexpr uint32_t kFusedMaxKpad = 8192;   // single-launch form: 8 rows x padded K of int8 stay in shared memory (64 KB at most)

struct RowsLayout {       // dynamic shared memory, offsets from a 1024-byte aligned base
    uint32_t stages, w_bytes;           // weight ring: one [tile_rows x 128 B] tile per stage
    uint32_t x_slots, x_chunk_bytes;    // activation ring: x_chunk_blocks atoms of [MT x 128 B] per slot
    uint32_t umma_m, umma_n, xpose_bytes;
    __host__ __device__ uint32_t w_off(uint32_t s) const { return s * w_bytes; }
    __host__ __device__ uint32_t w_end() const {
        // the MMA reads umma_n x 128 bytes from a weight stage
        const uint32_t reach = (stages - 1) * w_bytes + umma_n * kRK;
        return stages * w_bytes > reach ? stages * w_bytes : reach;
    }
    __host__ __device__ uint32_t x_off(uint32_t slot) const { return round_up(w_end(), 1024u) + slot * x_chunk_bytes; }
    // ... and umma_m x 128 bytes from an activation atom (the last atom's reach goes past the ring)
    __host__ __device__ uint32_t x_end() const { return x_off(x_slots) + umma_m * kRK; }
    __host__ __device__ uint32_t consts_off() const { return x_end(); }   // float ws[256], bias[256]
    __host__ __device__ uint32_t xpose_off() const { return consts_off() + 2 * kMaxTile * 4; }  // the epilogue's parking area
    __host__ __device__ uint32_t bars_off() const { return xpose_off() + xpose_bytes; }
    __host__ __device__ uint32_t misc_off() const { return bars_off() + (2 * kMaxStages + 2 * kMaxXSlots + 4) * 8; }
    __host__ __device__ uint32_t total() const { return misc_off() + 32 + 128 * 4 + 1024; }
};

__device__ __forceinline__ void stamp(unsigned long long* trace, uint32_t slot) {
    if (trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        trace[(size_t)blockIdx.x * kTraceSlots + slot] = t;
    }
}

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Finishes a tile parked in shared memory as int32 [rows][pitch].  The (row, channel) pairs of the
// tile are dealt out flat over the `workers` participating threads (worker index `me`): consecutive
// threads take consecutive channels of one row, so a store instruction covers a contiguous run of
// a row whatever the tile's width, and narrow tiles still keep every thread busy.
__device__ __forceinline__ void finish_parked(const DecodeRowsArgs& args, const int32_t* parked, uint32_t pitch,
                                              const float* s_ws, const float* s_bias, const float* s_as,
                                              uint32_t c0, uint32_t valid, uint32_t me, uint32_t workers) {
    const EpilogueParams& ep = args.epi;
    const float zero_f = __int2float_rn(ep.out_zero);
    const float lo_f = __int2float_rn(ep.out_lo), hi_f = __int2float_rn(ep.out_hi);
    if (ep.mode == kEpiF32 && ep.act == 1u) {
        // channel pairs (gate, up) -> one output column each
        const uint32_t pairs = valid >> 1, total = pairs * args.rows;
        for (uint32_t idx = me; idx < total; idx += workers) {
            const uint32_t mm = idx / pairs, o = idx - mm * pairs;
            const float asv = s_as[mm];
            const float g = epi_f32(parked[mm * pitch + 2 * o], asv, s_ws[2 * o], s_bias[2 * o]);
            const float u = epi_f32(parked[mm * pitch + 2 * o + 1], asv, s_ws[2 * o + 1], s_bias[2 * o + 1]);
            ((float*)ep.out)[(size_t)mm * ep.ld + (c0 >> 1) + o] = epi_silu_mul(g, u);
        }
        return;
    }
    const uint32_t total = valid * args.rows;
    for (uint32_t idx = me; idx < total; idx += workers) {
        const uint32_t mm = idx / valid, col = idx - mm * valid;
        const int32_t v = parked[mm * pitch + col];
        const float asv = s_as[mm], wsv = s_ws[col], bf = s_bias[col];
        const size_t at = (size_t)c0 + col;
        if (ep.mode == kEpiF32) {
            float y = epi_f32(v, asv, wsv, bf);
            if (ep.residual) y = __fadd_rn(y, __ldg(ep.residual + (size_t)mm * ep.ld_res + at));
            ((float*)ep.out)[(size_t)mm * ep.ld + at] = y;
        } else if (ep.mode == kEpiI8) {
            const int32_t bi = __float_as_int(bf);
            const int32_t qv = (ep.fast_div != 0 && div_const_row_ok(asv))
                ? epi_i8_v2<true>(v + bi, asv, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero)
                : epi_i8_v2<false>(v + bi, asv, wsv, ep.out_scale, ep.out_rcp, zero_f, lo_f, hi_f, ep.out_zero);
            ((int8_t*)ep.out)[(size_t)mm * ep.ld + at] = (int8_t)qv;
        } else {
            ((int32_t*)ep.out)[(size_t)mm * ep.ld + at] = v;
        }
    }
}

// Single-launch form: every CTA quantizes the (at most 8) fp32 rows itself, with K1's arithmetic bit
// for bit, straight into the shared-memory layout the MMA reads (one [8 x 128 B] swizzled atom per
// 128-byte K block: the 16-byte piece c of row r sits at piece c ^ r).  The rows are read from L2 once
// per pass (absmax, then quantize); rows * k * 4 bytes per CTA is far below what the weight stream
// brings in meanwhile, so the work hides behind the filling weight ring.  The row scales go to s_as.
// Warps are dealt out to rows, `wpr` warps per row, each over a contiguous part of the row.
// With `gamma` the rows pass through an RMSNorm first (the arithmetic of the stand-alone fused quantizer,
// quantize.cuh): one more pass for the sum of squares, the normalized values are recomputed in the absmax
// and in the quantizing pass, and the first CTA persists them in `norm_out` when other consumers need them.
__device__ __forceinline__ void fused_quantize_rows(const float* __restrict__ x, uint32_t rows, uint32_t k, uint8_t* x_smem,
                                                    float* s_as, float* part_max, int* part_bad, uint32_t warps,
                                                    const float* __restrict__ gamma, double eps, float* __restrict__ norm_out,
                                                    double* part_ss) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t wpr = warps / rows;                      // >= 1: rows <= 8 <= warps
    const uint32_t row = warp / wpr, part = warp - row * wpr;
    const bool active = row < rows;
    const uint32_t nvec = k >> 2, seg = (nvec + wpr - 1) / wpr;
    const uint32_t v0 = part * seg, v1 = v0 + seg < nvec ? v0 + seg : nvec;
    const float4* in = reinterpret_cast<const float4*>(x + (size_t)(active ? row : 0) * k);
    // loads go out in batches of kBatch per lane before any of them is used: the loop is a chain of
    // L2 round trips otherwise (one outstanding load per lane).  Keeping a warp's part of the row in
    // registers across the passes instead of reading it again was slower (the kernel's 96-register
    // budget spilled: 15.8 against 14.2 us per launch for one row at K 4096, N 14336).
    constexpr uint32_t kBatch = 8;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    double inv = 0.0;
    if (gamma) {
        // the row's sum of squares: exact products, double additions; the partial sums of a row's warps are
        // added in a fixed order, so every CTA arrives at the same bits
        double ss = 0.0;
        if (active)
            for (uint32_t vb = v0 + lane; vb < v1; vb += 32 * kBatch) {
                float4 c[kBatch];
#pragma unroll
                for (uint32_t j = 0; j < kBatch; j++) c[j] = vb + 32 * j < v1 ? __ldg(in + vb + 32 * j) : zero4;
#pragma unroll
                for (uint32_t j = 0; j < kBatch; j++) ss = square_sum4(c[j], ss);
            }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if (lane == 0) part_ss[warp] = ss;
        __syncthreads();
        // one thread per row does the double-precision division and square root
        if (threadIdx.x < rows) {
            double t = 0.0;
            for (uint32_t i = 0; i < wpr; i++) t += part_ss[threadIdx.x * wpr + i];
            part_ss[32 + threadIdx.x] = 1.0 / sqrt(t / (double)k + eps);
        }
        __syncthreads();
        if (active) inv = part_ss[32 + row];
    }
    float4* nout = (gamma && norm_out && blockIdx.x == 0 && active) ? reinterpret_cast<float4*>(norm_out + (size_t)row * k) : nullptr;
    float amax = 0.0f; int bad = 0;
    if (active)
        for (uint32_t vb = v0 + lane; vb < v1; vb += 32 * kBatch) {
            float4 c[kBatch];
#pragma unroll
            for (uint32_t j = 0; j < kBatch; j++) c[j] = vb + 32 * j < v1 ? __ldg(in + vb + 32 * j) : zero4;
#pragma unroll
            for (uint32_t j = 0; j < kBatch; j++) {
                if (gamma && vb + 32 * j < v1) {
                    c[j] = norm4(c[j], inv, __ldg(g4 + vb + 32 * j));
                    if (nout) nout[vb + 32 * j] = c[j];
                }
                bad |= nonfinite_bits(c[j].x) | nonfinite_bits(c[j].y) | nonfinite_bits(c[j].z) | nonfinite_bits(c[j].w);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(c[j].x), fabsf(c[j].y)), fmaxf(fabsf(c[j].z), fabsf(c[j].w))));
            }
        }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        bad |= __shfl_xor_sync(0xffffffffu, bad, off);
    }
    if (lane == 0) { part_max[warp] = amax; part_bad[warp] = bad; }
    __syncthreads();
    if (!active) return;
    amax = 0.0f; bad = 0;
    for (uint32_t i = 0; i < wpr; i++) { amax = fmaxf(amax, part_max[row * wpr + i]); bad |= part_bad[row * wpr + i]; }
    const float scale = row_scale_from_amax(amax);
    if (part == 0 && lane == 0) s_as[row] = bad ? __int_as_float(0x7fc00000) : scale;
    const RowDivisor div(scale);
    const bool fast = div.fast && !bad;
    uint8_t* row_base = x_smem + row * kRK;
    for (uint32_t vb = v0 + lane; vb < v1; vb += 32 * kBatch) {
        float4 c[kBatch];
#pragma unroll
        for (uint32_t j = 0; j < kBatch; j++) c[j] = vb + 32 * j < v1 ? __ldg(in + vb + 32 * j) : zero4;
#pragma unroll
        for (uint32_t j = 0; j < kBatch; j++) {
            const uint32_t v = vb + 32 * j;
            if (v >= v1) break;
            if (gamma) c[j] = norm4(c[j], inv, __ldg(g4 + v));
            const uint32_t word = bad ? 0u : (fast ? pack4t<true>(c[j], div) : pack4t<false>(c[j], div));
            const uint32_t kbyte = v << 2, kb = kbyte >> 7, off = kbyte & 127u;
            *reinterpret_cast<uint32_t*>(row_base + (size_t)kb * (8u * kRK) + (((off >> 4) ^ row) << 4) + (off & 15u)) = word;
        }
    }
}

template <uint32_t MT, bool PAIR>
__global__ void __launch_bounds__(ModeCfg<PAIR>::kThreads, ModeCfg<PAIR>::kCtasPerSm)
decode_rows_kernel(const __grid_constant__ DecodeRowsArgs args) {
    using Cfg = RowsCfg<MT>;
    constexpr uint32_t kIssuerWarps = ModeCfg<PAIR>::kIssuerWarps, kXWarp = ModeCfg<PAIR>::kXWarp;
    constexpr uint32_t kEpiBase = ModeCfg<PAIR>::kEpiBase, kProducerWarps = ModeCfg<PAIR>::kProducerWarps;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const RowsLayout lay{args.stages, args.w_stage_bytes, args.x_slots, args.x_chunk_blocks * Cfg::kXAtom,
                         Cfg::kUmmaM, args.umma_n, Cfg::xpose_bytes(args.rows, args.umma_n)};
    const uint32_t stages = args.stages;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto w_addr = [&](uint32_t s) { return smem_u32(base + lay.w_off(s)); };
    auto x_addr = [&](uint32_t s) { return smem_u32(base + lay.x_off(s)); };
    auto full = [&](uint32_t s) { return smem_u32(base + lay.bars_off() + s * 8); };
    auto empty = [&](uint32_t s) { return smem_u32(base + lay.bars_off() + (kMaxStages + s) * 8); };
    auto xfull = [&](uint32_t s) { return smem_u32(base + lay.bars_off() + (2 * kMaxStages + s) * 8); };
    auto xempty = [&](uint32_t s) { return smem_u32(base + lay.bars_off() + (2 * kMaxStages + kMaxXSlots + s) * 8); };
    auto tmem_full = [&](uint32_t b) { return smem_u32(base + lay.bars_off() + (2 * kMaxStages + 2 * kMaxXSlots + b) * 8); };
    auto tmem_empty = [&](uint32_t b) { return smem_u32(base + lay.bars_off() + (2 * kMaxStages + 2 * kMaxXSlots + 2 + b) * 8); };
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(base + lay.misc_off());
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + lay.misc_off() + 4);
    volatile int* epi_flag = reinterpret_cast<volatile int*>(base + lay.misc_off() + 12);
    float* s_as = reinterpret_cast<float*>(base + lay.misc_off() + 32);
    float* s_ws = reinterpret_cast<float*>(base + lay.consts_off());
    float* s_bias = s_ws + kMaxTile;
    int32_t* s_xpose = reinterpret_cast<int32_t*>(base + lay.xpose_off());

    // let the next launch in the stream become resident as early as possible (see kPairSmemBytes)
    if (threadIdx.x == 0) { pdl_release(); stamp(args.trace, 0); }

    const uint32_t num_kb = args.kpad / kRK;
    const uint32_t tiles = args.tiles_per_cta;
    const uint32_t first_channel = blockIdx.x * tiles * args.tile_rows;
    const uint32_t stage_tx = args.tile_rows * kRK;              // bytes one weight stage receives
    const uint32_t KC = args.x_chunk_blocks, x_slots = args.x_slots;
    const bool double_buffered = tiles > 1;                       // else one accumulator, reused
    const uint32_t acc_stride = args.tmem_cols / 2;              // columns between the two accumulators

    // Weight producer p owns the stages p, p+P, ... (the ring depth is a multiple of P): it initialises
    // their barriers itself and requests its first ring-full of weights at once, before the CTA-wide
    // set-up below (TMEM allocation, the other barriers) has finished - the weight stream is the
    // critical path of the kernel and depends on nothing else.
    struct ProducerState { uint32_t kb; int32_t channel; uint32_t w_sm, fb, eb, stage, phase, i, u; };
    ProducerState prod{};
    const bool is_producer = warp >= kXWarp && warp < kXWarp + kProducerWarps - 1 && lane == 0 && warp - kXWarp < args.producers;
    if (is_producer) {
        const uint32_t p = warp - kXWarp, P = args.producers;
        const uint32_t total = tiles * num_kb, own = stages / P;
        for (uint32_t st = p; st < stages; st += P) { mbar_init(full(st), 1); mbar_init(empty(st), 1); }
        fence_barrier_init();
        prod.kb = p; prod.channel = (int32_t)first_channel;
        while (prod.kb >= num_kb) { prod.kb -= num_kb; prod.channel += (int32_t)args.tile_rows; }
        prod.w_sm = w_addr(p); prod.fb = full(p); prod.eb = empty(p);
        prod.i = p;
        for (; prod.i < total && prod.u < own; prod.i += P, prod.u++) {
            mbar_expect_tx(prod.fb, stage_tx);
            tma_load_2d(prod.w_sm, &args.tmap_w, prod.fb, (int32_t)(prod.kb * kRK), prod.channel);
            prod.kb += P; while (prod.kb >= num_kb) { prod.kb -= num_kb; prod.channel += (int32_t)args.tile_rows; }
            prod.w_sm += lay.w_bytes * P; prod.fb += 8 * P; prod.eb += 8 * P;
            if (++prod.stage == own) { prod.stage = 0; prod.phase ^= 1u; prod.w_sm = w_addr(p); prod.fb = full(p); prod.eb = empty(p); }
        }
    }
    if (warp == 1) {
        if (lane < x_slots) { mbar_init(xfull(lane), 1); mbar_init(xempty(lane), args.issuers); }
        if (lane == 0) {
            mbar_init(tmem_full(0), args.issuers); mbar_init(tmem_full(1), 1);
            for (uint32_t b = 0; b < 2; b++) mbar_init(tmem_empty(b), 128);
            arm_abort(abort_flag, args.status);
            prefetch_tmap(&args.tmap_w);
            if (!args.x_f32) prefetch_tmap(&args.tmap_x);
        }
        fence_barrier_init();
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_ptr), args.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    if (threadIdx.x == 0) stamp(args.trace, 1);

    const bool fused = args.x_f32 != nullptr;
    if constexpr (MT == 8) {
        if (fused) {
            // the weight producers have their first ring-full in flight; the whole CTA now turns the fp32
            // rows (the preceding kernel's output) into the MMA's activation operand
            pdl_wait();
            if (threadIdx.x == 0) stamp(args.trace, 6);
            float* part_max = reinterpret_cast<float*>(s_xpose);          // the parking area is free until the epilogue
            int* part_bad = reinterpret_cast<int*>(s_xpose) + 32;
            double* part_ss = reinterpret_cast<double*>(s_xpose) + 32;    // bytes 256.. of the same area
            fused_quantize_rows(args.x_f32, args.rows, args.k, base + lay.x_off(0), s_as, part_max, part_bad,
                                ModeCfg<PAIR>::kThreads / 32, args.norm_weight, args.norm_eps, args.norm_out, part_ss);
            fence_proxy_async();   // generic-proxy writes to shared memory -> visible to the tensor core's reads
            __syncthreads();
        }
    }

    if (warp == kXWarp + kProducerWarps - 1) {
        // ---------------- activation producer ----------------
        // The activations are shared by every K block's MMAs and small: one copy brings KC
        // consecutive K blocks ([KC][MT x 128 B] atoms, a 3-D box) into one slot of a short ring of
        // their own, so a TMA start (some 200 ns of the issuing thread whatever the box size) is
        // paid once per KC blocks. Every issuer owns the same number of blocks in each chunk and
        // hands the slot back (tcgen05.commit -> xempty) after its last one.
        if (lane == 0 && !fused) {
            const uint32_t nch = (num_kb + KC - 1) / KC, total = tiles * nch;
            const uint32_t chunk_tx = KC * Cfg::kXAtom;    // the whole box, zero-filled past the edges
            pdl_wait();   // the activations are the preceding kernel's output
            stamp(args.trace, 6);
            uint32_t slot = 0, phase = 0, kc = 0;
            for (uint32_t c = 0; c < total; c++) {
                if (c >= x_slots && !mbar_wait(xempty(slot), phase ^ 1u, abort_flag)) break;
                mbar_expect_tx(xfull(slot), chunk_tx);
                tma_load_3d(x_addr(slot), &args.tmap_x, xfull(slot), 0, 0, (int32_t)(kc * KC));
                if (++kc == nch) kc = 0;
                if (++slot == x_slots) { slot = 0; phase ^= 1u; }
            }
        }
    } else if (warp >= kXWarp) {
        // ---------------- weight producers ----------------
        // Producer p of P loads the weight tiles of the blocks p, p+P, ... (block = tile * num_kb +
        // kb) into its own stages p, p+P, ... (the ring depth is a multiple of P), re-arming a
        // stage as soon as the MMAs that read it have completed. Only increments in the loop.
        // Weights depend on nothing that runs before this kernel, so these threads never wait
        // for the preceding kernel: the ring is full before the activations may be read.
        const uint32_t p = warp - kXWarp, P = args.producers;
        if (is_producer) {
            // the first ring-full was requested in the prologue; from here on a stage is re-armed as soon
            // as the MMAs that read it have completed
            const uint32_t total = tiles * num_kb, own = stages / P;
            const uint32_t w0 = w_addr(p), f0 = full(p), e0 = empty(p), wstep = lay.w_bytes * P;
            // block one ring-depth ahead of the one being copied (stages is a multiple of P, so this
            // producer owns it too): optionally requested from L2 early
            uint32_t pkb = prod.kb + stages; int32_t pchannel = prod.channel;
            while (pkb >= num_kb) { pkb -= num_kb; pchannel += (int32_t)args.tile_rows; }
            bool ok = true;
            for (; prod.i < total; prod.i += P, prod.u++) {
                if (args.l2_prefetch && prod.i + stages < total) tma_prefetch_l2_2d(&args.tmap_w, (int32_t)(pkb * kRK), pchannel);
                pkb += P; while (pkb >= num_kb) { pkb -= num_kb; pchannel += (int32_t)args.tile_rows; }
                if (!mbar_wait(prod.eb, prod.phase ^ 1u, abort_flag)) { ok = false; break; }
                mbar_expect_tx(prod.fb, stage_tx);
                tma_load_2d(prod.w_sm, &args.tmap_w, prod.fb, (int32_t)(prod.kb * kRK), prod.channel);
                prod.kb += P; while (prod.kb >= num_kb) { prod.kb -= num_kb; prod.channel += (int32_t)args.tile_rows; }
                prod.w_sm += wstep; prod.fb += 8 * P; prod.eb += 8 * P;
                if (++prod.stage == own) { prod.stage = 0; prod.phase ^= 1u; prod.w_sm = w0; prod.fb = f0; prod.eb = e0; }
            }
            if (!ok) {
                // drain: give this thread's own copies in flight a bounded time to land
                for (uint32_t st = p; st < stages; st += P) {
                    for (uint32_t n = 0; n < 2000; n++) {
                        if (mbar_try_wait(full(st), 0u) || mbar_try_wait(full(st), 1u)) break;
                        __nanosleep(500);
                    }
                }
            }
        }
    } else if (warp < kIssuerWarps) {
        // ---------------- MMA issuers ----------------
        // One thread can start an MMA only every ~100 clocks, far slower than the tensor pipe
        // finishes a narrow one, so up to eight threads issue: issuer ii of I takes the K blocks
        // ii, ii+I, ... into an accumulator of its own (the epilogue adds them up; integers:
        // exact). Block b lives in weight stage b mod stages and stages is a multiple of I, so
        // this thread owns the stages ii, ii+I, ... and sees each of their phases in order; of
        // every activation chunk (KC = I * m blocks) it owns the atoms ii, ii+I, ...
        // A CTA with several tiles has one issuer, which alternates between two accumulators.
        const uint32_t ii = warp, I = args.issuers;
        if (lane == 0 && ii < I) {
            const uint32_t idesc = make_idesc(Cfg::kUmmaM, args.umma_n);
            const uint32_t own = stages / I, per_chunk = KC / I;
            const uint32_t wstep = lay.w_bytes * I, xstep = Cfg::kXAtom * I;
            const uint32_t w0 = w_addr(ii), f0 = full(ii), e0 = empty(ii);
            uint32_t wa = w0, fb = f0, eb = e0, cstage = 0, cphase = 0;
            uint32_t xslot = 0, xphase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            for (uint32_t t = 0; ok && t < tiles; t++) {
                uint32_t d_tmem = tmem_base + ii * args.acc_cols;
                if (I == 1) {
                    if (!mbar_wait(tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    d_tmem = tmem_base + acc * acc_stride;
                }
                uint32_t first = 1, in_chunk = 0, xa = 0;
                for (uint32_t kb = ii; kb < num_kb; kb += I) {
                    if (in_chunk == 0) {
                        if (!fused && !mbar_wait(xfull(xslot), xphase, abort_flag)) { ok = false; break; }
                        xa = x_addr(xslot) + ii * Cfg::kXAtom;
                    }
                    if (!mbar_wait(fb, cphase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    if ((t | kb) == 0) stamp(args.trace, 2);
                    // descriptors by their low words: the time this thread spends between two MMAs is
                    // tensor-pipe idle time
                    const uint32_t da = smem_desc_lo(xa), db = smem_desc_lo(wa);
                    umma_i8_lo_first(d_tmem, da, db, idesc, first ? 0u : 1u);   // +32 bytes of K = +2
                    umma_i8_lo(d_tmem, da + 2u, db + 2u, idesc);
                    umma_i8_lo(d_tmem, da + 4u, db + 4u, idesc);
                    umma_i8_lo(d_tmem, da + 6u, db + 6u, idesc);
                    first = 0;
                    umma_commit(eb);
                    wa += wstep; fb += 8 * I; eb += 8 * I; xa += xstep;
                    if (++cstage == own) { cstage = 0; cphase ^= 1u; wa = w0; fb = f0; eb = e0; }
                    if (++in_chunk == per_chunk || kb + I >= num_kb) {
                        umma_commit(xempty(xslot));
                        in_chunk = 0;
                        if (++xslot == x_slots) { xslot = 0; xphase ^= 1u; }
                    }
                }
                if (!ok) break;
                if (I == 1) {
                    umma_commit(tmem_full(acc));
                    if (double_buffered) { acc ^= 1u; if (acc == 0) acc_phase ^= 1u; }
                    else acc_phase ^= 1u;
                } else {
                    umma_commit(tmem_full(0));
                }
            }
            if (ii == 0) stamp(args.trace, 3);
        }
    } else if (warp >= kIssuerWarps && warp < kXWarp) {
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
                if (e < 128 && !fused) s_as[e] = (e < args.rows && ep.mode != kEpiAcc) ? __ldg(ep.row_scales + e) : 0.0f;
            }
            if constexpr (Cfg::kParkAll) {
                if (tiles == 1) break;   // the single tile is drained by every warp of the CTA, below
            }
            const bool waited = mbar_wait(tmem_full(acc), acc_phase, abort_flag);
            // make the give-up decision uniform across the four epilogue warps (the first
            // barrier also publishes the staged constants)
            epi_bar();
            if (e == 0) epi_flag[0] = (*abort_flag != 0 || !waited) ? 1 : 0;
            epi_bar();
            if (epi_flag[0]) break;
            tc_fence_after();
            if (e == 0 && t + 1 == tiles) stamp(args.trace, 4);

            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * acc_stride;
            const uint32_t left = args.n > c0 ? args.n - c0 : 0u;
            const uint32_t valid = left < args.tile_rows ? left : args.tile_rows;
            if constexpr (Cfg::kParkAll) {
                // Few token rows (M = 64: row r sits in lane r % 16 of warp r / 16). The warps that
                // hold rows move the whole tile into shared memory, one barrier, then thread =
                // channel finishes every row of its channel: each store instruction covers
                // consecutive channels of one row.
                const uint32_t pitch = Cfg::park_pitch(args.umma_n);
                if (quarter * 16u < args.rows) {
                    const uint32_t nchunks = (valid + 31u) >> 5;
#pragma unroll 1
                    for (uint32_t ci = 0; ci < nchunks; ci++) {
                        const uint32_t c = ci << 5;
                        uint32_t r[32];
                        tmem_ld32(taddr + c, r);
                        if (args.issuers > 1) {
                            uint32_t more[32];
                            tmem_ld32(taddr + args.acc_cols + c, more);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; i++) r[i] += more[i];
                            for (uint32_t a = 2; a < args.issuers; a++) {
                                tmem_ld32(taddr + a * args.acc_cols + c, more);
                                tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < 32; i++) r[i] += more[i];
                            }
                        } else {
                            tmem_ld_wait();
                        }
                        if (m_ok) {
                            uint4* dst = reinterpret_cast<uint4*>(s_xpose + m * pitch + c);
#pragma unroll
                            for (int j = 0; j < 8; j++) dst[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        }
                    }
                }
                epi_bar();
                finish_parked(args, s_xpose, pitch, s_ws, s_bias, s_as, c0, valid, e, 128u);
            } else {
            // TMEM hands each thread one token row; the stores want one channel per lane. Each
            // 32-channel chunk is therefore transposed through shared memory: row threads park
            // their 32 values, then thread (lane = channel, warp = row group) finishes rows
            // warp, warp+4, ... so that every store instruction covers 32 consecutive channels.
            // Two parking buffers alternate, so one barrier per chunk is enough, and the TMEM
            // load of the next chunk is in flight while this one is finished.
            const uint32_t row_group = e >> 5;
            const uint32_t nchunks = (valid + 31u) >> 5;
            uint32_t r[32];
            if (nchunks) tmem_ld32(taddr, r);
#pragma unroll 1
            for (uint32_t ci = 0; ci < nchunks; ci++) {
                const uint32_t c = ci << 5;
                tmem_ld_wait();
                for (uint32_t a = 1; a < args.issuers; a++) {   // add the other issuers' accumulators
                    uint32_t more[32];
                    tmem_ld32(taddr + a * args.acc_cols + c, more);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) r[i] += more[i];
                }
                int32_t* park = s_xpose + (ci & 1u) * (MT * kXposePitch);
                if (m_ok) {
#pragma unroll
                    for (uint32_t i = 0; i < 32; i++) park[m * kXposePitch + i] = (int32_t)r[i];
                }
                if (ci + 1 < nchunks) tmem_ld32(taddr + c + 32, r);
                epi_bar();
                const uint32_t col = c + lane;
                if (col < valid) {
                    const float wsv = s_ws[col];
                    const float bf = s_bias[col];
                    const int32_t bi = __float_as_int(bf);
                    const size_t at = (size_t)c0 + col;
                    for (uint32_t mm = row_group; mm < args.rows; mm += 4) {
                        const int32_t v = park[mm * kXposePitch + lane];
                        const float asv = s_as[mm];
                        if (ep.mode == kEpiF32 && ep.act == 1u) {
                            // channel pairs (gate, up): the even lane finishes both and writes one column
                            if ((lane & 1u) == 0u && col + 1u < valid) {
                                const float g = epi_f32(v, asv, wsv, bf);
                                const float u = epi_f32(park[mm * kXposePitch + lane + 1], asv, s_ws[col + 1], s_bias[col + 1]);
                                ((float*)ep.out)[(size_t)mm * ep.ld + (at >> 1)] = epi_silu_mul(g, u);
                            }
                        } else if (ep.mode == kEpiF32) {
                            float y = epi_f32(v, asv, wsv, bf);
                            if (ep.residual) y = __fadd_rn(y, __ldg(ep.residual + (size_t)mm * ep.ld_res + at));
                            ((float*)ep.out)[(size_t)mm * ep.ld + at] = y;
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
            }
            // the accumulator has been consumed: hand the TMEM buffer back to the MMA warp
            if (e == 0 && t + 1 == tiles) stamp(args.trace, 5);
            tc_fence_before();
            mbar_arrive(tmem_empty(acc));
            if (double_buffered) { acc ^= 1u; if (acc == 0) acc_phase ^= 1u; }
            else acc_phase ^= 1u;
        }
    }

    if constexpr (Cfg::kParkAll) {
        if (tiles == 1) {
            // Every role's loop is over.  The accumulators of few token rows sit in one or two TMEM lane
            // quarters, which only warps with the matching index (warp % 4) can read; a single warp
            // reading all 32-channel chunks one after the other was a chain of dependent TMEM loads
            // (over a microsecond at 97 channels).  All warps of the CTA that can read a quarter
            // therefore share its chunks, park them in shared memory, and then the whole CTA finishes
            // the tile: pure latency at the end of the kernel, spread over every thread.
            __syncwarp();
            uint32_t ready = 1;
            if (lane == 0) ready = mbar_wait(tmem_full(0), 0u, abort_flag) ? 1u : 0u;
            ready = __shfl_sync(0xffffffffu, ready, 0);
            tc_fence_after();
            const uint32_t left = args.n > first_channel ? args.n - first_channel : 0u;
            const uint32_t valid = left < args.tile_rows ? left : args.tile_rows;
            const uint32_t pitch = Cfg::park_pitch(args.umma_n);
            const uint32_t quarter = warp & 3u;
            if (ready && quarter * 16u < args.rows) {
                constexpr uint32_t kWarps = ModeCfg<PAIR>::kThreads / 32;
                const uint32_t sharers = (kWarps - quarter + 3u) / 4u, mine = warp >> 2;
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16);
                const uint32_t m = quarter * 16u + lane;
                const bool m_ok = lane < 16 && m < args.rows;
                const uint32_t nchunks = (valid + 31u) >> 5;
#pragma unroll 1
                for (uint32_t ci = mine; ci < nchunks; ci += sharers) {
                    const uint32_t c = ci << 5;
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
                    if (m_ok) {
                        uint4* dst = reinterpret_cast<uint4*>(s_xpose + m * pitch + c);
#pragma unroll
                        for (int j = 0; j < 8; j++) dst[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    }
                }
            }
            if (threadIdx.x == kEpiBase) stamp(args.trace, 4);
            tc_fence_before();
            __syncthreads();
            if (!*abort_flag) {
                pdl_wait();
                finish_parked(args, s_xpose, pitch, s_ws, s_bias, s_as, first_channel, valid, threadIdx.x, ModeCfg<PAIR>::kThreads);
                if (threadIdx.x == kEpiBase) stamp(args.trace, 5);
            }
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
    if (warp == 0) tmem_dealloc(tmem_base, args.tmem_cols);
    if (threadIdx.x == 0) stamp(args.trace, 7);
}

// Fills in the launch shape: issuers, producers, ring depths, TMEM columns.
template <uint32_t MT, bool PAIR>
bool configure_t(DecodeRowsArgs& args) {
    using Cfg = RowsCfg<MT>;
    using Mode = ModeCfg<PAIR>;
    args.pair = PAIR ? 1u : 0u;
    args.umma_n = round_up(args.tile_rows, 16u);
    // TMEM: a power-of-two number of columns >= umma_n per accumulator
    uint32_t cols = 32;
    while (cols < args.umma_n) cols *= 2;
    args.acc_cols = cols;
    const uint32_t num_kb = args.kpad / kRK;
    uint32_t max_issuers = 1;
    if (args.tiles_per_cta == 1) {
        max_issuers = Mode::kTmemCols / cols;
        if (max_issuers > Mode::kIssuerWarps) max_issuers = Mode::kIssuerWarps;
        if (max_issuers > num_kb) max_issuers = num_kb;
        if (max_issuers < 1) max_issuers = 1;
    }
    uint32_t max_producers = Mode::kProducerWarps - 1;   // the last producer warp loads the activations
    if (max_producers > num_kb) max_producers = num_kb;
    auto divisor = [](uint32_t st, uint32_t cap) { uint32_t d = cap; while (st % d) d--; return d; };
    // Issuers: a power of two (one accumulator each; TMEM is allocated in powers of two), as many
    // as leave every issuer two weight stages of its own. Block b lives in stage b mod stages:
    // the ring depth is a multiple of the issuer and of the producer count, so that each stage's
    // barriers are only ever waited on by one issuer and one producer, in order - a parity wait
    // on an mbarrier is only meaningful for a waiter that saw the previous phase complete.
    // How many are wanted: a thread starts the four MMAs of a K block in some 0.4 us, and the block
    // (tile_rows x 128 B) is due every tile_rows x 2.9 ns at this SM's share of the HBM stream; more
    // issuers than that only lengthen the epilogue, which adds their accumulators up.
    const uint32_t wanted = (190u + args.tile_rows - 1) / args.tile_rows;
    uint32_t issuers = 1;
    while (issuers < wanted && 2 * issuers <= max_issuers) issuers *= 2;
    for (;; issuers /= 2) {
        // activation chunk: a multiple of the issuer count, about 8 KB, at most the row's blocks
        uint32_t per = 8192u / (issuers * Cfg::kXAtom);
        if (per < 1) per = 1;
        const uint32_t most = (num_kb + issuers - 1) / issuers;
        if (per > most) per = most;
        if (args.x_f32) per = most;   // single-launch form: every K block of the rows stays resident
        const uint32_t kc = issuers * per;
        const uint32_t nch = ((num_kb + kc - 1) / kc) * args.tiles_per_cta;
        uint32_t slots = kc * Cfg::kXAtom > 8192u ? 2u : 4u;
        if (slots > nch) slots = nch;
        if (args.x_f32) slots = 1;
        auto fits = [&](uint32_t st) {
            const RowsLayout f{st, args.w_stage_bytes, slots, kc * Cfg::kXAtom, Cfg::kUmmaM, args.umma_n,
                               Cfg::xpose_bytes(args.rows, args.umma_n)};
            return f.total() <= Mode::kSmemBytes;
        };
        uint32_t deepest = kMaxStages;
        while (deepest > 1 && !fits(deepest)) deepest--;
        // among the deepest few depths that the issuers divide: most producers first, then depth
        uint32_t best = 0, best_p = 0;
        for (uint32_t st = deepest; st >= 1 && st + 8 > deepest; st--) {
            if (st % issuers) continue;
            const uint32_t pp = divisor(st, max_producers);
            if (pp > best_p) { best = st; best_p = pp; }
        }
        if (best >= 2 * issuers || (issuers == 1 && best >= 1)) {
            if (!fits(best)) return false;   // not even the shallowest ring fits
            args.stages = best; args.producers = best_p; args.issuers = issuers;
            args.x_chunk_blocks = kc; args.x_slots = slots;
            break;
        }
        if (issuers == 1) return false;
    }
    // one accumulator per issuer; a CTA with several tiles double-buffers one issuer's accumulator
    args.tmem_cols = args.issuers > 1 ? args.issuers * cols : (args.tiles_per_cta == 1 ? cols : 2 * cols);
    if (args.tmem_cols < 32) args.tmem_cols = 32;
    return (args.tmem_cols & (args.tmem_cols - 1)) == 0 && args.tmem_cols <= 512;   // tcgen05.alloc: powers of two
}

template <uint32_t MT, bool PAIR>
cudaError_t launch_t(const DecodeRowsArgs& args, cudaStream_t stream) {
    using Cfg = RowsCfg<MT>;
    using Mode = ModeCfg<PAIR>;
    const RowsLayout lay{args.stages, args.w_stage_bytes, args.x_slots, args.x_chunk_blocks * Cfg::kXAtom,
                         Cfg::kUmmaM, args.umma_n, Cfg::xpose_bytes(args.rows, args.umma_n)};
    const uint32_t smem = lay.total();
    cudaError_t e = ensure_dynamic_smem<decode_rows_kernel<MT, PAIR>>(smem);
    if (e != cudaSuccess) return e;
    const uint32_t per_cta = args.tiles_per_cta * args.tile_rows;
    const uint32_t grid = (args.n + per_cta - 1) / per_cta;
    return launch_pdl(decode_rows_kernel<MT, PAIR>, dim3(grid), dim3(Mode::kThreads), smem, stream, args);
}

}  // namespace

Tunables& tunables() {
    static Tunables t{kPairShareBytes, false, false, false, 1755u, 2u, true};
    return t;
}

uint32_t decode_rows_threads(bool pair) { return pair ? ModeCfg<true>::kThreads : ModeCfg<false>::kThreads; }

uint32_t decode_rows_token_slots(uint32_t rows) {
    return rows <= 8 ? 8u : rows <= 16 ? 16u : rows <= 32 ? 32u : rows <= 64 ? 64u : 128u;
}

void decode_rows_plan(uint32_t n, int sm_count, uint32_t* tile_rows, uint32_t* tiles_per_cta) {
    uint32_t per_cta = (n + (uint32_t)sm_count - 1) / (uint32_t)sm_count;
    if (per_cta < 8) per_cta = n < 8 ? n : 8;
    if ((per_cta & 1u) && per_cta < n) per_cta++;   // even, so that (gate, up) channel pairs never straddle CTAs
    const uint32_t tiles = (per_cta + kMaxTile - 1) / kMaxTile;
    *tiles_per_cta = tiles;
    *tile_rows = (per_cta + tiles - 1) / tiles;
    if ((*tile_rows & 1u) && tiles > 1) (*tile_rows)++;   // ... nor tiles
}

#define VXB_DECODE_DISPATCH(fn, ...)                                                          \
    do {                                                                                      \
        const uint32_t mt = decode_rows_token_slots(args.rows);                               \
        if (pair) {                                                                           \
            if (mt == 8) return fn<8, true>(__VA_ARGS__);                                     \
            if (mt == 16) return fn<16, true>(__VA_ARGS__);                                   \
            if (mt == 32) return fn<32, true>(__VA_ARGS__);                                   \
            if (mt == 64) return fn<64, true>(__VA_ARGS__);                                   \
            return fn<128, true>(__VA_ARGS__);                                                \
        }                                                                                     \
        if (mt == 8) return fn<8, false>(__VA_ARGS__);                                        \
        if (mt == 16) return fn<16, false>(__VA_ARGS__);                                      \
        if (mt == 32) return fn<32, false>(__VA_ARGS__);                                      \
        if (mt == 64) return fn<64, false>(__VA_ARGS__);                                      \
        return fn<128, false>(__VA_ARGS__);                                                   \
    } while (0)

bool decode_rows_configure(DecodeRowsArgs& args) {
    if (args.rows == 0 || args.rows > 128 || args.n == 0 || args.tile_rows == 0 || args.tile_rows > kMaxTile) return false;
    // the single-launch form holds the quantized rows of every K block in shared memory: 8 rows, one tile per CTA
    if (args.x_f32 && (args.rows > 8 || args.tiles_per_cta != 1 || args.kpad > kFusedMaxKpad || (args.k & 3u) || args.k > args.kpad)) return false;
    // small weight shares: two CTAs per SM, so that successive launches overlap (see kPairSmemBytes)
    const bool pair = (size_t)args.tiles_per_cta * args.tile_rows * args.kpad <= tunables().decode_pair_share_bytes;
    args.l2_prefetch = tunables().decode_l2_prefetch ? 1u : 0u;
    VXB_DECODE_DISPATCH(configure_t, args);
}

cudaError_t launch_decode_rows(const DecodeRowsArgs& args, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    if (args.rows > 128 || args.stages == 0 || args.x_chunk_blocks == 0) return cudaErrorInvalidValue;
    if (args.x_f32 && (args.rows > 8 || args.x_slots != 1 || ((uintptr_t)args.x_f32 & 15u))) return cudaErrorInvalidValue;
    const bool pair = args.pair != 0;
    VXB_DECODE_DISPATCH(launch_t, args, stream);
}

}  // namespace vxb
