// Shared declarations for the W8A8 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <mutex>

namespace vxb {

// Weight rows and quantized activation rows are padded to this many bytes
// (one 128-byte TMA swizzle span) and zero-filled, so every kernel walks K in
// whole 128-byte steps without a tail.
constexpr uint32_t kKAlign = 128;

__host__ __device__ inline uint32_t round_up(uint32_t v, uint32_t m) { return (v + m - 1) / m * m; }

// Epilogue selection shared by all GEMM-shaped kernels.
enum Epilogue : int { kEpiAcc = 0, kEpiF32 = 1, kEpiI8 = 2 };

struct EpilogueParams {
    int mode;                 // Epilogue
    const float* row_scales;  // [rows]   activation scale per token (NaN = invalid row)
    const float* ws;          // [N]      weight scale per output channel
    const float* bias_f32;    // [N] or nullptr (E1)
    const int32_t* bias_i32;  // [N] or nullptr (E2, accumulator domain, zero-point folded)
    float out_scale;          // E2
    float out_rcp;            // E2: RN(1/out_scale), used when fast_div != 0
    int32_t fast_div;         // E2: host verified that division by out_scale may use div_const()
    int32_t out_zero;         // E2
    int32_t out_lo, out_hi;   // E2 saturation range (I8: -128..127, U8: 0..255)
    void* out;                // int32 / float / int8 [rows, ld]
    uint32_t ld;              // output row stride in elements
    // fused all-gather (large-M kernel only): the same [rows, ld] window in up to 7 peer GPUs'
    // buffers (peer-mapped addresses); every output tile is also stored there
    const float* gscales;   // grouped weight scales [n, groups] (R1 storage groups), or null
    uint32_t group, groups;  // K bytes per group (32/64/128/256), groups per channel; 0 = per-channel scales
    uint32_t n_peers;
    void* peer_out[7];
    // fused decode patterns on the fp32 epilogue (E1): y += residual[m, n], or, with the weight's
    // channels interleaved as (gate_0, up_0, gate_1, up_1, ...), y[m, j] = silu(gate_j) * up_j
    const float* residual;   // [rows, ld_res] or null
    uint32_t ld_res;
    uint32_t act;            // 0 none, 1 SiLU(gate) * up over channel pairs (output d_out / 2 wide)
};

// ---- programmatic dependent launch ------------------------------------------------------
// A kernel launched with launch_pdl() may start while the kernel before it in the stream is
// still running. pdl_wait() returns once every kernel this launch depends on has completed
// and its writes are visible (at once when the launch carries no such dependency);
// pdl_release() lets the NEXT launch in the stream begin. Only kernels that call pdl_wait()
// before touching a predecessor's data may be launched this way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Raises a kernel's dynamic shared-memory limit to `bytes`, once per device and size: the
// attribute belongs to the (function, device) pair, and contexts may live on several devices and
// threads of one process.
template <auto Kernel>
inline cudaError_t ensure_dynamic_smem(uint32_t bytes) {
    static std::mutex guard;
    static uint32_t configured[64] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(guard);
    if (bytes > configured[device]) {
        e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
        configured[device] = bytes;
    }
    return cudaSuccess;
}

// ---- epilogue arithmetic (every operation separately rounded; no FMA) ----

// E1: y = f32(f32(acc) * f32(as*ws)) + bias
__device__ __forceinline__ float epi_f32(int32_t acc, float as, float ws, float bias) {
    const float combined = __fmul_rn(as, ws);
    const float product = __fmul_rn(__int2float_rn(acc), combined);
    return __fadd_rn(product, bias);
}

// E2: multiplier association f32(f32(as*ws)/os) is part of the contract.
__device__ __forceinline__ int32_t epi_i8(int32_t acc, float as, float ws, float out_scale,
                                          int32_t out_zero, int32_t lo, int32_t hi) {
    const float product = __fmul_rn(as, ws);
    const float mult = __fdiv_rn(product, out_scale);
    const float scaled = __fmul_rn(__int2float_rn(acc), mult);
    const float moved = __fadd_rn(scaled, __int2float_rn(out_zero));
    if (moved != moved) return out_zero;
    if (moved <= (float)lo) return lo;
    if (moved >= (float)hi) return hi;
    return __float2int_rn(moved);
}

// Correctly rounded a / d for a constant divisor whose reciprocal rcp = RN(1/d) was
// computed once: two Newton corrections with exact FMA residuals (the tail of the
// IEEE division sequence, without the per-element reciprocal approximation and range
// check). Valid - bit-identical to __fdiv_rn - when d's significand is not all ones and
// a, d and a/d stay far from the fp32 exponent limits; the caller guards both.
__device__ __forceinline__ float div_const(float a, float d, float rcp) {
    const float q0 = __fmul_rn(a, rcp);
    const float r0 = __fmaf_rn(-d, q0, a);
    const float q1 = __fmaf_rn(r0, rcp, q0);
    const float r1 = __fmaf_rn(-d, q1, a);
    return __fmaf_rn(r1, rcp, q1);
}
// Range guard for div_const on the activation scale of one row (the host checked the
// weight scales and out_scale): 2^-30 <= as <= 2^30. NaN fails the guard.
__device__ __forceinline__ bool div_const_row_ok(float as) {
    return as >= 9.31322574615478515625e-10f && as <= 1073741824.0f;
}

// E2 with the saturation done by min/max and the division by div_const (FAST) or
// __fdiv_rn; same result as epi_i8 bit for bit.
template <bool FAST>
__device__ __forceinline__ int32_t epi_i8_v2(int32_t acc, float as, float ws, float out_scale,
                                             float out_rcp, float zero_f, float lo_f, float hi_f,
                                             int32_t out_zero) {
    const float product = __fmul_rn(as, ws);
    const float mult = FAST ? div_const(product, out_scale, out_rcp) : __fdiv_rn(product, out_scale);
    const float scaled = __fmul_rn(__int2float_rn(acc), mult);
    const float moved = __fadd_rn(scaled, zero_f);
    const int32_t q = __float2int_rn(fminf(fmaxf(moved, lo_f), hi_f));
    return moved != moved ? out_zero : q;
}

// E2 inside the fast-division guard with the byte range of the output type as the clamp: as,
// ws and out_scale within 2^+-30 keep every intermediate finite (|acc| < 2^31, multiplier < 2^90),
// so no NaN can appear, and round + saturate is one conversion instruction. Same result as
// epi_i8 bit for bit there.
template <bool UNSIGNED, bool ADD_ZERO = true>
__device__ __forceinline__ int32_t epi_i8_sat(int32_t acc, float as, float ws, float out_scale,
                                              float out_rcp, float zero_f) {
    const float mult = div_const(__fmul_rn(as, ws), out_scale, out_rcp);
    // a zero point of 0 needs no addition (ADD_ZERO = false): x + 0 = x except -0 + 0 = +0, and
    // both convert to 0
    const float scaled = __fmul_rn(__int2float_rn(acc), mult);
    const float moved = ADD_ZERO ? __fadd_rn(scaled, zero_f) : scaled;
    int32_t q;
    if (UNSIGNED) asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(moved));
    else asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q) : "f"(moved));
    return q;
}

// The same two elements at a time with the packed fp32 instructions of sm_100 (mul/fma.rn.f32x2:
// each half rounded to nearest like the scalar instruction, subnormals kept), which halves the
// floating-point instruction count of the requantization. A pair lives in a 64-bit register.
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// Constants of one thread's requantization, each duplicated into both halves.
struct RequantPair {
    uint64_t as2, rcp2, neg_d2;
    float zero;
    __device__ __forceinline__ RequantPair(float as, float out_scale, float out_rcp, float zero_f)
        : as2(f32x2(as, as)), rcp2(f32x2(out_rcp, out_rcp)), neg_d2(f32x2(-out_scale, -out_scale)),
          zero(zero_f) {}
};
// epi_i8_sat for the accumulators (acc0, acc1) of two neighbouring channels with scales ws2.
template <bool UNSIGNED, bool ADD_ZERO>
__device__ __forceinline__ void epi_i8_sat2(int32_t acc0, int32_t acc1, uint64_t ws2, const RequantPair& c,
                                            int32_t& q0, int32_t& q1) {
    const uint64_t p = mul_f32x2(c.as2, ws2);
    // div_const, both halves: a * rcp, then two corrections with exact residuals
    const uint64_t d0 = mul_f32x2(p, c.rcp2);
    const uint64_t r0 = fma_f32x2(c.neg_d2, d0, p);
    const uint64_t d1 = fma_f32x2(r0, c.rcp2, d0);
    const uint64_t r1 = fma_f32x2(c.neg_d2, d1, p);
    const uint64_t mult = fma_f32x2(r1, c.rcp2, d1);
    const uint64_t scaled = mul_f32x2(f32x2(__int2float_rn(acc0), __int2float_rn(acc1)), mult);
    float m0, m1;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(m0), "=f"(m1) : "l"(scaled));
    // the zero point is added with scalar instructions: a packed add right after the packed
    // multiply came out as one fused multiply-add (33.4999962 instead of 33.5 in a tie case)
    if (ADD_ZERO) { m0 = __fadd_rn(m0, c.zero); m1 = __fadd_rn(m1, c.zero); }
    if (UNSIGNED) {
        asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q0) : "f"(m0));
        asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q1) : "f"(m1));
    } else {
        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(m0));
        asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(m1));
    }
}

// E1 for two neighbouring channels: (f32(acc) * (as * ws)) + bias, each step rounded; the two
// multiplications packed, the additions scalar (see epi_i8_sat2).
__device__ __forceinline__ void epi_f32_2(int32_t acc0, int32_t acc1, uint64_t as2, uint64_t ws2, float bias0, float bias1,
                                          uint32_t& y0, uint32_t& y1) {
    const uint64_t combined = mul_f32x2(as2, ws2);
    const uint64_t product = mul_f32x2(f32x2(__int2float_rn(acc0), __int2float_rn(acc1)), combined);
    float p0, p1;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(p0), "=f"(p1) : "l"(product));
    y0 = __float_as_uint(__fadd_rn(p0, bias0));
    y1 = __float_as_uint(__fadd_rn(p1, bias1));
}

// silu(g) * u as the reference's fused gate/up decode kernel computes it (g * sigmoid(g), then * u;
// native/src/backends/cuda/kernels/cuda_forward_gemv_pair_kernels.inc:457-459), with an accurate exp.
__device__ __forceinline__ float epi_silu_mul(float gate, float up) {
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gate)));
    return __fmul_rn(__fmul_rn(gate, sig), up);
}

// One output element through the selected epilogue (scalar path).
__device__ __forceinline__ void epi_store(const EpilogueParams& p, uint32_t row, uint32_t col,
                                          int32_t acc) {
    const size_t at = (size_t)row * p.ld + col;
    if (p.mode == kEpiAcc) {
        ((int32_t*)p.out)[at] = acc;
    } else if (p.mode == kEpiF32) {
        ((float*)p.out)[at] = epi_f32(acc, p.row_scales[row], p.ws[col],
                                      p.bias_f32 ? p.bias_f32[col] : 0.0f);
    } else {
        const int32_t a = acc + (p.bias_i32 ? p.bias_i32[col] : 0);
        ((int8_t*)p.out)[at] = (int8_t)epi_i8(a, p.row_scales[row], p.ws[col], p.out_scale,
                                              p.out_zero, p.out_lo, p.out_hi);
    }
}

// Thread-local error / route text of the C ABI (defined beside vxb_last_error); returns `code`.
int set_error(int code, const char* fmt, ...);
void set_route(const char* text);
}  // namespace vxb
struct VxbContext;
namespace vxb {
cudaStream_t context_stream(const VxbContext* ctx);   // the stream a context queues its work on

// ---- launchers implemented in the .cu files -------------------------------

// Boundary ops of a static W8A8 island (boundary_ops.cu): byte outputs are int8 or uint8.
cudaError_t launch_quantize_linear(const float* x, unsigned long long n, float scale, int32_t zero, bool out_unsigned,
                                   void* out, cudaStream_t stream);
cudaError_t launch_dequantize_linear(const void* x, unsigned long long n, float scale, int32_t zero, bool in_unsigned,
                                     float* out, cudaStream_t stream);
cudaError_t launch_requantize_linear(const void* x, unsigned long long n, float multiplier, int32_t in_zero,
                                     bool in_unsigned, int32_t out_zero, bool out_unsigned, void* out,
                                     cudaStream_t stream);

// Grouped weight scales (the reference's PackedLinear storage groups): one thread per output,
// an exact integer dot per group, fp32 accumulation in ascending group order. fp32 output only.
// Grouped scales, rows <= 4 (decode): warp-per-channel streaming kernel, fp32 output.
cudaError_t launch_gemv_grouped(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                                const EpilogueParams& epi, int sm_count, cudaStream_t stream);
// The same over the 4-bit words themselves (rows <= 2): w4 is [n][row_words] uint32, row_words a
// multiple of 4 with row_words * 8 >= kpad, codes past the logical width 8 (= weight 0).
cudaError_t launch_gemv_w4_grouped(const int8_t* q, uint32_t rows, const uint32_t* w4, uint32_t row_words, uint32_t n,
                                   uint32_t kpad, const EpilogueParams& epi, int sm_count, cudaStream_t stream);
cudaError_t launch_gemm_grouped(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n, uint32_t kpad,
                                const EpilogueParams& epi, cudaStream_t stream);

// K1: per-token absmax + quantize. q rows have stride ldq (multiple of 16 when
// the vector path is to be used); bytes [k, ldq) are zeroed.
cudaError_t launch_rmsnorm_quantize_rows(const float* x, const float* gamma, float epsilon, uint32_t rows,
                                         uint32_t k, float* norm_out, int8_t* q, uint32_t ldq,
                                         float* row_scales, int32_t* valid, cudaStream_t stream);
cudaError_t launch_quantize_rows(const float* x, uint32_t rows, uint32_t k, int8_t* q,
                                 uint32_t ldq, float* row_scales, int32_t* valid,
                                 cudaStream_t stream);

// Fill a float array with one value (static-activation QLinear row scales).
cudaError_t launch_fill_f32(float* dst, uint32_t count, float value, cudaStream_t stream);

// bias_eff[n] = bias[n] - input_zero * wsum[n]  (activation zero-point folding)
cudaError_t launch_fold_zero_point(const int32_t* bias, const int32_t* wsum, int32_t input_zero,
                                   int32_t* out, uint32_t n, cudaStream_t stream);

// Convert U8 activations to the signed domain (x ^ 0x80) with row padding.
cudaError_t launch_copy_bytes_padded(const uint8_t* src, uint32_t rows, uint32_t k, uint8_t* dst,
                                     uint32_t ld, uint32_t xor_mask, cudaStream_t stream);

// Weight repack: int8 [N,K] (or W8 offset-binary bytes with xor 0x80, source row
// stride src_ld bytes) -> [N, kpad] zero padded + per-channel code sums.
cudaError_t launch_repack_weight(const uint8_t* src, uint32_t src_ld, uint32_t n, uint32_t k,
                                 uint32_t xor_mask, int8_t* dst, uint32_t kpad, int32_t* wsum,
                                 cudaStream_t stream);

// Launch geometry of the three streaming GEMV kernels (256 threads, one warp per `ch` channels,
// activations staged in a shared-memory chunk): kind 0 = per-channel scales (rows <= 32),
// 1 = grouped scales (rows <= 4), 2 = grouped scales over 4-bit words (rows <= 2).
struct GemvShape { uint32_t mr, ch, kchunk, smem, grid; };
GemvShape gemv_shape(int kind, uint32_t rows, uint32_t n, uint32_t kpad, int sm_count);

// K3: small-M (rows <= 32) bandwidth-bound GEMV, dp4a + warp-shuffle reduction.
cudaError_t launch_gemv(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n,
                        uint32_t kpad, const EpilogueParams& epi, int sm_count,
                        cudaStream_t stream);

// Verification kernel: one thread per output, dp4a over K.
cudaError_t launch_gemm_simt(const int8_t* q, uint32_t rows, const int8_t* w, uint32_t n,
                             uint32_t kpad, const EpilogueParams& epi, cudaStream_t stream);

// K2: TMA-fed tcgen05 kind::i8 GEMM. `status` is a device int the kernel sets
// non-zero when a bounded wait expired; tmap_* are encoded by the caller.
struct GemmTcgen05Args {
    CUtensorMap tmap_a;  // activations int8 [rows, kpad], box 128 x 128B, swizzle 128B
    CUtensorMap tmap_b;  // weights     int8 [n, kpad],    box 256 x 128B, swizzle 128B
    uint32_t rows, n, kpad;
    EpilogueParams epi;
    int* status;
    unsigned long long* trace;   // optional [grid][8] of %globaltimer stamps (single-CTA kernel), or null
    // 32-bit outputs [rows, ld] as a tensor map with a (32 columns x 32 rows) box, 128B swizzle: the
    // wide-output kernel's epilogue stores through it (16-byte aligned base and row pitch)
    CUtensorMap tmap_out;
    uint32_t tma_out;
    // fused all-gather through TMA tile stores: this rank's channel range of its own output buffer
    // (index 0) and of every peer's buffer, int8 [rows, n] with the buffers' row pitch, box 128 columns x
    // 32 rows, 128B swizzle; used when gather_tma != 0 (16-byte aligned bases and pitch)
    CUtensorMap tmap_gather[8];
    uint32_t gather_tma;
};
cudaError_t launch_gemm_tcgen05(const GemmTcgen05Args& args, int sm_count, cudaStream_t stream);
// Fused all-gather: the launch is bound by its NVLink stores rather than by the MMAs when every row sends
// n_local * peers bytes at ~770 GB/s for longer than its 2 * K * n_local operations take at ~3.3 POPS,
// i.e. when peers * 2140 > K (three GPUs and more at K = 4096; two GPUs stay MMA-bound).
inline bool gather_is_link_bound(uint32_t n_peers, uint32_t kpad) { return n_peers != 0 && (uint64_t)n_peers * 2140u > kpad; }
cudaError_t gemm_tcgen05_prepare();  // one-time func attribute set-up
// K2w: the GEMM for 32-bit outputs (fp32 / raw int32) with sixteen epilogue warps and TMA tile stores through
// args.tmap_out (args.tma_out must be set)
cudaError_t launch_gemm_wide(const GemmTcgen05Args& args, int sm_count, cudaStream_t stream);
// The same GEMM by pairs of CTAs (cta_group::2) on 256 x 256 tiles; tmap_b has a box of 128 rows.
cudaError_t gemm_pair_prepare();    // func attribute + how many pairs can be resident
int gemm_pair_clusters();           // 0: pairs cannot run on this device
cudaError_t launch_gemm_pair(const GemmTcgen05Args& args, cudaStream_t stream);

// K2g: the GEMM for weights with grouped scales on the tensor cores (fp32 output).  tmap_a and
// tmap_b have boxes of 128 rows; gscales_t is the group-scale table transposed to
// [groups][n_pad] (n_pad a multiple of 128, padding zero).
struct GemmGroupedArgs {
    CUtensorMap tmap_a, tmap_b;
    uint32_t rows, n, kpad;
    uint32_t group, groups, n_pad;
    const float* gscales_t;
    const float* row_scales;
    const float* bias;
    float* out;
    uint32_t ld;
    int* status;
};
cudaError_t gemm_grouped_tcgen05_prepare();
cudaError_t launch_gemm_grouped_tcgen05(const GemmGroupedArgs& args, int sm_count, cudaStream_t stream);

// K3: decode kernel in which every CTA owns whole output channels (rows <= 128).
// tile_rows / tiles_per_cta come from decode_rows_plan(); tmap_w has a box of tile_rows rows,
// tmap_x a box of decode_rows_token_slots(rows) rows.
struct DecodeRowsArgs {
    CUtensorMap tmap_w;       // weights [n, kpad], box tile_rows x 128 B
    CUtensorMap tmap_x;       // activations [rows, kpad] seen as {128 B, rows, kpad/128}, box 128 B x token slots x x_chunk_blocks
    uint32_t rows, n, kpad;
    uint32_t tile_rows, tiles_per_cta;
    // filled in by decode_rows_configure
    uint32_t stages, umma_n, tmem_cols, acc_cols, issuers, producers, x_chunk_blocks, x_slots, pair;
    uint32_t w_stage_bytes;   // round_up(tile_rows * 128, 1024)
    uint32_t l2_prefetch;     // 1: producers prefetch the tile one ring-depth ahead into L2
    // single-launch form (rows <= 8): the CTA quantizes the fp32 rows itself into shared memory, in
    // the UMMA operand layout, while its weight ring fills; tmap_x and epi.row_scales are unused then
    const float* x_f32;       // [rows, k] fp32 activations, or null (activations come prepared through tmap_x)
    uint32_t k;               // logical width of x_f32 (a multiple of 4)
    const float* norm_weight; // single-launch form only: RMSNorm weight [k] applied to the rows before they are quantized, or null
    double norm_eps;
    float* norm_out;          // optional [rows, k]: the normalized rows, written by the first CTA
    EpilogueParams epi;
    int* status;
    unsigned long long* trace;   // optional [grid][kTraceSlots] of %globaltimer stamps, or null
};
constexpr uint32_t kTraceSlots = 8;   // 0 entry, 1 prologue done, 2 first weights landed, 3 last MMA issued,
                                      // 4 accumulator ready, 5 last store, 6 predecessor finished, 7 exit
uint32_t decode_rows_token_slots(uint32_t rows);  // 8 / 16 / 32 / 64 / 128
void decode_rows_plan(uint32_t n, int sm_count, uint32_t* tile_rows, uint32_t* tiles_per_cta);
bool decode_rows_configure(DecodeRowsArgs& args);   // before the activation tensor map is encoded
uint32_t decode_rows_threads(bool pair);             // threads per CTA of the two residency modes
cudaError_t launch_decode_rows(const DecodeRowsArgs& args, cudaStream_t stream);

// K3b: skinny stream-K tcgen05 kernel for rows <= 128 (weights are the UMMA M operand).
// workspace: int32 [rows, n] zero on entry and zero again on exit; counters: uint32
// [ceil(n/128)] likewise.
struct DecodeTcgen05Args {
    CUtensorMap tmap_w;  // weights     int8 [n, kpad],    box 128 x 128B, swizzle 128B
    CUtensorMap tmap_x;  // activations int8 [rows, kpad], box MT x 128B (MT = token slots)
    uint32_t rows, n, kpad;
    EpilogueParams epi;
    int32_t* workspace;
    uint32_t* counters;
    int* status;
};
uint32_t decode_token_slots(uint32_t rows);  // 32 / 64 / 128
cudaError_t launch_decode_tcgen05(const DecodeTcgen05Args& args, int sm_count, cudaStream_t stream);

// Cross-GPU barrier (selftest.cu): flag arrays of uint32, one slot per rank, in peer-mapped memory.
struct PeerBarrierArgs {
    uint32_t* peer_flags[7];   // the peers' flag arrays (peer-mapped addresses)
    uint32_t peer_ranks[7];    // rank of peer t (its slot in this GPU's own array)
    uint32_t n_peers, my_rank, epoch;
};
cudaError_t launch_peer_barrier(uint32_t* my_flags, const PeerBarrierArgs& args, int* status, cudaStream_t stream);

// Device self-tests (selftest.cu): a wait that expires by design, and div_const against the IEEE divide.
cudaError_t launch_wait_expiry(int* status, cudaStream_t stream);
cudaError_t launch_div_const_check(int exponent, uint32_t neighbours, uint32_t samples, unsigned long long* mismatches,
                                   unsigned long long* checked, int sm_count, cudaStream_t stream);

// Internal tunables (defaults are what ships; changed through the diagnostic entry vxb_tune()).
struct Tunables {
    uint32_t decode_pair_share_bytes;   // largest per-CTA weight share the decode kernel runs as two CTAs per SM
    bool decode_l2_prefetch;            // weight producers ask L2 for the tile one ring-depth ahead
    bool overlap_k1;                    // large batches: quantize the later rows under the GEMM of the first ones (off: measured slower)
    bool overlap_gather;                // the same for a link-bound fused all-gather launch, with its 128-register build (off: measured slower)
    uint32_t overlap_ratio;             // rows_first / rows_rest >= overlap_ratio / d_out when a batch is cut in two
    uint32_t decode_fused_max_rows;     // fp32 rows up to which the automatic route takes the decode kernel's single-launch form
    bool gather_tma;                    // fused all-gather: TMA tile stores to the peers instead of per-lane stores
};
Tunables& tunables();

// tensor-pipe peak probe: issues `iters` rounds of kind::i8 MMAs on resident
// shared-memory operands in every CTA; returns through `cycles` the SM clocks
// spent per CTA.
cudaError_t launch_i8_peak_probe(uint32_t iters, long long* cycles, int* status, int sm_count,
                                 cudaStream_t stream);

// Issue-pattern probe on one SM: `iters` rounds of `per_commit` MMAs of shape m x n x 32 cycling
// through `accs` accumulators, one commit + wait per round; cycles[0] = SM clocks spent.
cudaError_t launch_mma_probe(uint32_t m, uint32_t n, uint32_t accs, uint32_t per_commit, uint32_t iters,
                             long long* cycles, int* status, cudaStream_t stream);

}  // namespace vxb
