// K2, paired form: the int8 GEMM with two CTAs (a cluster of 2, on the two SMs of a pair)
// working on one 256 x 256 output tile through tcgen05.mma.cta_group::2.
//
//   acc[m,n] = sum_k q[m,k] * w[n,k]      q: [rows,kpad] int8, w: [n,kpad] int8
//
// Why: with one CTA per 128 x 256 tile every SM pulls 48 KB (16 KB of activations + 32 KB of
// weights) from L2 for every 128 bytes of K, 94 bytes per tensor-pipe clock, and four such
// stages are all the shared memory holds - barely one L2 round trip of cover. In a pair, CTA r
// loads its own 128 activation rows and only HALF of the tile's 256 weight rows (channels
// n0 + 128 r ...); the pair's MMA reads the other half from the partner's shared memory. Each SM
// now pulls 32 KB per 128 bytes of K for the same MMA time; the ring holds 3 stages of 256 K bytes.
//
// Per CTA (same warp roles as the single-CTA kernel):
//   warp 0      TMA producer, activation tiles (two of 128 rows x 128 B) of each stage
//   warp 10     TMA producer, weight half-tiles (two of 128 channels x 128 B) of each stage
//               both complete on the LEADER's (cluster rank 0) full barrier of the stage
//   warp 1      allocates TMEM (cta_group::2); in the leader one lane issues
//               tcgen05.mma.cta_group::2.kind::i8 (M256 x N256 x K32, 8 per stage) and commits
//               to the stage's empty barrier and the accumulator's full barrier of BOTH CTAs
//   warps 2-9   epilogue of this CTA's 128 rows x 256 columns (its own TMEM), then one arrive
//               per warp on the leader's accumulator-empty barrier
// Two 256-column accumulators per CTA: the epilogue of tile i overlaps the MMAs of tile i+1.
//
// Every copy lands in the shared memory of the CTA that issued it (plain tile loads, one
// destination each). All mbarrier waits are bounded; a CTA that gives up raises
// the status word and tells its partner, and both drain, free their TMEM and return.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

constexpr uint32_t kBM = 128;           // activation rows per CTA (256 per pair)
constexpr uint32_t kBNHalf = 128;       // weight rows loaded per CTA
constexpr uint32_t kBN = 256;           // output channels per tile
constexpr uint32_t kAtomK = 128;        // K bytes of one swizzle span (one TMA box, four MMAs)
constexpr uint32_t kAtoms = 2;
constexpr uint32_t kBK = kAtoms * kAtomK;           // K bytes per stage: two spans, so that the issuing thread's
                                        // per-stage work (barrier wait, commits) is paid once per 8 MMAs
constexpr uint32_t kStages = 3;
constexpr uint32_t kAAtomBytes = kBM * kAtomK;     // 16 KiB
constexpr uint32_t kBAtomBytes = kBNHalf * kAtomK; // 16 KiB
constexpr uint32_t kABytes = kAtoms * kAAtomBytes;
constexpr uint32_t kBBytes = kAtoms * kBAtomBytes;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kAccCols = kBN;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kEpiWarps = 8;
constexpr uint32_t kThreads = 64 + 32 * kEpiWarps + 32;
constexpr uint32_t kBWarp = 2 + kEpiWarps;
constexpr uint32_t kEpiCols = kBN / 2;              // columns per epilogue warp

constexpr uint32_t kOffStages = 0;
constexpr uint32_t kOffWs = kStages * kStageBytes;                   // float[8 warps][128]
constexpr uint32_t kOffBias = kOffWs + kEpiWarps * kEpiCols * 4;
constexpr uint32_t kOffStore = kOffBias + kEpiWarps * kEpiCols * 4;   // [8 warps][16 rows x 128 B] store staging
constexpr uint32_t kStoreBytes = 16 * 128;
constexpr uint32_t kOffBars = kOffStore + kEpiWarps * kStoreBytes;
constexpr uint32_t kNumBars = 2 * kStages + 4;
constexpr uint32_t kOffTmemPtr = kOffBars + kNumBars * 8;
constexpr uint32_t kOffAbort = kOffTmemPtr + 4;
constexpr uint32_t kSmemBytes = kOffAbort + 8 + 1024;

// ---- cluster-scope PTX ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared::cluster address of `local` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t in_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void store_flag_cluster(uint32_t cluster_addr, int v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA tile load into this CTA's shared memory that completes on a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster,
                                                 int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the descriptors given by their low words (start address >> 4 | leading offset): the
// high word (stride, version, swizzle) is one constant for every tile of this kernel. Fewer
// instructions in the issuing thread, whose time between two MMAs is exposed tensor-pipe idle time.
__device__ __forceinline__ void umma_i8_pair_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "mov.b64 da, {%1, %4};\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kSmemDescHi) : "memory");
}
__device__ __forceinline__ void umma_i8_pair_lo_first(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                      uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %4};\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kSmemDescHi), "r"(accumulate) : "memory");
}
// the barrier (any CTA of the cluster) gets one arrival once all MMAs issued so far have finished
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar_cluster) : "memory");
}

struct Smem {
    uint8_t* base;
    __device__ uint32_t a(uint32_t s) const { return smem_u32(base + kOffStages + s * kStageBytes); }
    __device__ uint32_t b(uint32_t s) const { return a(s) + kABytes; }
    __device__ uint32_t full(uint32_t s) const { return smem_u32(base + kOffBars + s * 8); }
    __device__ uint32_t empty(uint32_t s) const { return smem_u32(base + kOffBars + (kStages + s) * 8); }
    __device__ uint32_t tmem_full(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + b) * 8); }
    __device__ uint32_t tmem_empty(uint32_t b) const { return smem_u32(base + kOffBars + (2 * kStages + 2 + b) * 8); }
    __device__ uint32_t* tmem_ptr() const { return reinterpret_cast<uint32_t*>(base + kOffTmemPtr); }
    __device__ volatile int* abort_flag() const { return reinterpret_cast<volatile int*>(base + kOffAbort); }
    __device__ float* ws() const { return reinterpret_cast<float*>(base + kOffWs); }
    __device__ float* bias() const { return reinterpret_cast<float*>(base + kOffBias); }
};

__device__ __forceinline__ void gemm_i8_pair_body(const GemmTcgen05Args& args) {
    extern __shared__ uint8_t smem_raw[];
    Smem sm;
    sm.base = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();            // 0 = leader (issues the pair's MMAs)
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    const uint32_t tiles_m = (args.rows + 2 * kBM - 1) / (2 * kBM);
    const uint32_t tiles_n = (args.n + kBN - 1) / kBN;
    const uint32_t total_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (args.kpad + kBK - 1) / kBK;   // a last half-empty stage is zero-filled by TMA
    volatile int* abort_flag = sm.abort_flag();

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) { mbar_init(sm.full(s), 1); mbar_init(sm.empty(s), 1); }
        // accumulator-empty: one arrival per epilogue warp of both CTAs (only the leader's is waited on)
        for (uint32_t b = 0; b < 2; b++) { mbar_init(sm.tmem_full(b), 1); mbar_init(sm.tmem_empty(b), 2 * kEpiWarps); }
        arm_abort(abort_flag, args.status);
        fence_barrier_init();
        prefetch_tmap(&args.tmap_a);
        prefetch_tmap(&args.tmap_b);
        pdl_release();   // the next launch in the stream may begin its own prologue
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(sm.tmem_ptr()), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the partner's barriers exist before anything is signalled across
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_ptr();

    if (warp == 0) {
        // ---------------- TMA producer, activation rows of this CTA ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            pdl_wait();   // the activations come from the launch before this one; the weight producer does not wait
            for (uint32_t t = pair; ok && t < total_tiles; t += pairs) {
                const int32_t m0 = (int32_t)((t % tiles_m) * 2 * kBM + rank * kBM);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
                    // the leader's barrier collects the bytes of both CTAs' copies of the stage
                    if (rank == 0) mbar_expect_tx(sm.full(stage), 2 * kStageBytes);
#pragma unroll
                    for (uint32_t a = 0; a < kAtoms; a++)
                        tma_load_2d_pair(sm.a(stage) + a * kAAtomBytes, &args.tmap_a, in_cta(sm.full(stage), 0), (int32_t)(kb * kBK + a * kAtomK), m0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == kBWarp) {
        // ---------------- TMA producer, this CTA's half of the weight tile ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < total_tiles; t += pairs) {
                const int32_t n0 = (int32_t)((t / tiles_m) * kBN + rank * kBNHalf);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(sm.empty(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (uint32_t a = 0; a < kAtoms; a++)
                        tma_load_2d_pair(sm.b(stage) + a * kBAtomBytes, &args.tmap_b, in_cta(sm.full(stage), 0), (int32_t)(kb * kBK + a * kAtomK), n0);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(2 * kBM, kBN);
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t a_lo0 = smem_desc_lo(sm.a(0));
            const uint32_t peer_delta = in_cta(sm.empty(0), 1) - sm.empty(0);   // the same offset for every barrier
            uint32_t full_s = sm.full(0), empty_s = sm.empty(0), a_lo = a_lo0;
            for (uint32_t t = pair; ok && t < total_tiles; t += pairs) {
                if (!mbar_wait(sm.tmem_empty(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kAccCols;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    if (!mbar_try_wait(full_s, phase) && !mbar_wait(full_s, phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t b_lo = a_lo + (kABytes >> 4);
                    umma_i8_pair_lo_first(d_tmem, a_lo, b_lo, idesc, kb);       // +32 bytes of K = +2
                    umma_i8_pair_lo(d_tmem, a_lo + 2u, b_lo + 2u, idesc);
                    umma_i8_pair_lo(d_tmem, a_lo + 4u, b_lo + 4u, idesc);
                    umma_i8_pair_lo(d_tmem, a_lo + 6u, b_lo + 6u, idesc);
#pragma unroll
                    for (uint32_t a = 1; a < kAtoms; a++) {   // the other spans' tiles
                        const uint32_t a2 = a_lo + a * (kAAtomBytes >> 4), b2 = b_lo + a * (kBAtomBytes >> 4);
                        umma_i8_pair_lo(d_tmem, a2, b2, idesc);
                        umma_i8_pair_lo(d_tmem, a2 + 2u, b2 + 2u, idesc);
                        umma_i8_pair_lo(d_tmem, a2 + 4u, b2 + 4u, idesc);
                        umma_i8_pair_lo(d_tmem, a2 + 6u, b2 + 6u, idesc);
                    }
                    // the stage is free again in both CTAs once these MMAs have read it
                    umma_commit_pair(empty_s);
                    umma_commit_pair(empty_s + peer_delta);
                    full_s += 8; empty_s += 8; a_lo += kStageBytes >> 4;
                    if (++stage == kStages) { stage = 0; phase ^= 1u; full_s = sm.full(0); empty_s = sm.empty(0); a_lo = a_lo0; }
                }
                if (!ok) break;
                umma_commit_pair(sm.tmem_full(acc));
                umma_commit_pair(sm.tmem_full(acc) + peer_delta);
                acc ^= 1u;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9): this CTA's 128 rows x 256 columns ----------------
        const uint32_t quarter = warp & 3u;              // TMEM lanes [32*quarter, +32)
        const uint32_t half = (warp - 2u) >> 2;          // columns [128*half, +128) of the tile
        const uint32_t cbase = half * kEpiCols;
        const EpilogueParams& ep = args.epi;
        float* s_ws = sm.ws() + (warp - 2u) * kEpiCols;
        float* s_bias = sm.bias() + (warp - 2u) * kEpiCols;
        const float zero_f = __int2float_rn(ep.out_zero);
        const float lo_f = __int2float_rn(ep.out_lo), hi_f = __int2float_rn(ep.out_hi);
        const bool sat_s8 = ep.out_lo == -128 && ep.out_hi == 127, sat_u8 = ep.out_lo == 0 && ep.out_hi == 255;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        // fused all-gather (int8 output, aligned buffers): 64 columns at a time leave through this warp's
        // 2 KB staging tile ([32 rows x 64 B], 64B-swizzled) as one TMA tile store per destination
        const bool gather = ep.n_peers != 0;
        const uint32_t gbuf = smem_u32(sm.base + kOffStore + (warp - 2u) * kStoreBytes);
        pdl_wait();   // row scales and residual come from earlier launches, and one may still read the output
        for (uint32_t t = pair; ok && t < total_tiles; t += pairs) {
            const uint32_t m0 = (t % tiles_m) * 2 * kBM + rank * kBM, n0 = (t / tiles_m) * kBN + cbase;
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
                const bool wide = ep.mode != kEpiI8;                // 32-bit outputs go through the staging below
                if (gather) {
                    // no early exit: the destination's tensor map clips rows beyond the batch and columns beyond
                    // the shard.  A new group of 64 columns starts once the previous group's stores have left the tile.
                    if ((c & 32u) == 0) {
                        if (lane == 0) tma_store_wait_read();
                        __syncwarp();
                    }
                } else {
                    if (col >= args.n) continue;                   // uniform over the warp
                    if (!row_ok && !wide) continue;
                }
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
                        // this lane's 32 bytes of its row: 16-byte pieces 0,1 or 2,3 of the 64-byte row, XORed with
                        // bits 1-2 of the row number (the 64B swizzle of the tensor map)
                        const uint32_t piece = (c & 32u) >> 4, sw = (lane >> 1) & 3u, base = gbuf + lane * 64u;
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + ((piece ^ sw) << 4)),
                                     "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + (((piece + 1u) ^ sw) << 4)),
                                     "r"(packed[4]), "r"(packed[5]), "r"(packed[6]), "r"(packed[7]) : "memory");
                        if (c & 32u) {
                            fence_proxy_async();
                            __syncwarp();
                            const uint32_t g0 = col - 32u;
                            if (lane == 0 && g0 < args.n) {
                                for (uint32_t d = 0; d <= ep.n_peers; d++)
                                    tma_store_2d(&args.tmap_gather[d], gbuf, (int32_t)g0, (int32_t)(m0 + quarter * 32u));
                                tma_store_commit();
                            }
                        }
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
            // this warp has read its part of the accumulator: one arrival on the leader's barrier
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(in_cta(sm.tmem_empty(acc), 0));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (gather && lane == 0) tma_store_wait_all();   // the stores are complete before the kernel ends
    }

    // ---------------- teardown ----------------
    __syncwarp();
    // a CTA that gave up tells its partner, whose waits then end at their next look at the flag
    if (lane == 0 && *abort_flag) store_flag_cluster(in_cta(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u), 1);
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        nap(200);   // let asynchronous work in flight settle
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, 5);
    }
    // neither CTA may free its TMEM or leave while the partner's MMAs, copies or arrivals can
    // still target it
    cluster_sync_all();
    tc_fence_after();
    if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_pair_kernel(const __grid_constant__ GemmTcgen05Args args) { gemm_i8_pair_body(args); }

int g_pair_clusters = 0;   // co-resident clusters of two, queried once

}  // namespace

cudaError_t gemm_pair_prepare() {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, gemm_i8_pair_kernel, &cfg);
    if (e != cudaSuccess) return e;
    g_pair_clusters = clusters;
    return cudaSuccess;
}

int gemm_pair_clusters() { return g_pair_clusters; }

cudaError_t launch_gemm_pair(const GemmTcgen05Args& args, cudaStream_t stream) {
    if (args.rows == 0 || args.n == 0) return cudaSuccess;
    if (g_pair_clusters <= 0 || (args.epi.n_peers != 0 && (!args.gather_tma || args.epi.mode != kEpiI8))) return cudaErrorInvalidValue;
    const uint32_t tiles = ((args.rows + 2 * kBM - 1) / (2 * kBM)) * ((args.n + kBN - 1) / kBN);
    const uint32_t pairs = tiles < (uint32_t)g_pair_clusters ? tiles : (uint32_t)g_pair_clusters;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kSmemBytes; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // set-up and weight loads under the predecessor's tail
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, gemm_i8_pair_kernel, args);
}

}  // namespace vxb
