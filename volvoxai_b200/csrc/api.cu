// C ABI of the W8A8 linear route (declarations and contracts: include/vxb200_w8a8.h).
// Host-side orchestration only: validation, scratch, route choice, tensor maps.
#include "../../include/vxb200_w8a8.h"
#include "../../include/vxb200_plan.h"
#include "diag.h"
#include "common.cuh"

#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

using namespace vxb;

namespace {

thread_local char g_error[512] = "";
thread_local char g_route[96] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace

// Sets the calling thread's error text from another translation unit of the library.
int vxb::set_error(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}
void vxb::set_route(const char* text) { snprintf(g_route, sizeof g_route, "%s", text); }

namespace {
#define CUDA_TRY(expr, code)                                                              \
    do { cudaError_t e__ = (expr);                                                        \
         if (e__ != cudaSuccess) return fail((code), "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = (EncodeTiledFn)fn;
    });
    return g_encode;
}

// int8 matrix [rows, kpad] row-major -> 2-D tensor map with a (128 B x box_rows) box, 128B swizzle
bool encode_i8_rows(CUtensorMap* map, const void* base, uint32_t rows, uint32_t kpad, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {kpad, rows};
    cuuint64_t strides[1] = {kpad};
    cuuint32_t box[2] = {kKAlign, box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same matrix seen as {128 B, rows, kpad / 128}: a box of (128 B x box_rows x box_blocks) lands as
// box_blocks consecutive [box_rows x 128 B] swizzled tiles, one per 128-byte K block.
// 32-bit matrix [rows, n] with row pitch ld (elements) -> 2-D tensor map with a (32 columns x 32 rows) box,
// 128B swizzle: the wide-output GEMM's TMA tile stores
bool encode_out32(CUtensorMap* map, const void* base, uint32_t rows, uint32_t n, uint32_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || ((uintptr_t)base & 15u) || (ld & 3u)) return false;
    cuuint64_t dims[2] = {n, rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4u};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// int8 matrix [rows, n] with row pitch ld bytes -> 2-D tensor map with a (128 columns x 32 rows) box, 128B
// swizzle: the destination of the fused all-gather's TMA tile stores
bool encode_gather_i8(CUtensorMap* map, const void* base, uint32_t rows, uint32_t n, uint32_t ld, uint32_t box_columns = 128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || ((uintptr_t)base & 15u) || (ld & 15u)) return false;
    cuuint64_t dims[2] = {n, rows};
    cuuint64_t strides[1] = {ld};
    cuuint32_t box[2] = {box_columns, 32};   // 128 columns with the 128B swizzle, 64 with the 64B one
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, box_columns == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_i8_kblocks(CUtensorMap* map, const void* base, uint32_t rows, uint32_t kpad, uint32_t box_rows,
                       uint32_t box_blocks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {kKAlign, rows, kpad / kKAlign};
    cuuint64_t strides[2] = {kpad, kKAlign};
    cuuint32_t box[3] = {kKAlign, box_rows, box_blocks};
    cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Host-side failure injection (diag.h): countdowns to the launch / allocation that is refused.
std::atomic<uint32_t> g_fail_launch{0}, g_fail_alloc{0};
bool injected(std::atomic<uint32_t>& countdown) {
    uint32_t c = countdown.load(std::memory_order_relaxed);
    while (c != 0) {
        if (countdown.compare_exchange_weak(c, c - 1, std::memory_order_relaxed)) return c == 1;
    }
    return false;
}

struct Buffer {
    void* ptr = nullptr; size_t bytes = 0;
    cudaError_t reserve(size_t need) {
        if (need <= bytes) return cudaSuccess;
        if (injected(g_fail_alloc)) return cudaErrorMemoryAllocation;
        if (ptr) cudaFree(ptr);
        ptr = nullptr; bytes = 0;
        size_t grow = need + need / 4;
        cudaError_t e = cudaMalloc(&ptr, grow);
        if (e == cudaSuccess) bytes = grow;
        return e;
    }
    void release() { if (ptr) cudaFree(ptr); ptr = nullptr; bytes = 0; }
};

}  // namespace

struct VxbContext {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    Buffer q, row_scales, bias_eff, stage_in, stage_out;
    Buffer splitk_ws, splitk_counters;   // zero between calls (the decode kernel cleans up)
    int* status = nullptr;        // device block: [0] raised by bounded waits, [1] wait limit in 1024-clock units (0 = default)
    unsigned long long* trace = nullptr;   // caller's device buffer for decode-kernel time stamps, or null
    int* status_host = nullptr;   // pinned mirror
    bool tcgen05_ready = false;
    bool pair_ready = false;
    bool grouped_ready = false;
    // optional per-kernel timing (event pairs on the launching stream)
    // vxb_linear_host: upload / download streams and their events
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[2] = {}, ev_done[2] = {}, ev_out[2] = {}, ev_start = nullptr;
    cudaEvent_t ev_switch = nullptr;   // orders the context's scratch across a stream change
    // K1 / K2 overlap: the quantizer of the later rows runs on `side` under the GEMM of the first rows
    cudaStream_t side = nullptr;
    cudaEvent_t ev_first = nullptr, ev_rest = nullptr;
    int profiling = 0;          // 0 off, n: every n-th launch of a kind is bracketed by events
    uint32_t prof_seen[2] = {0, 0};
    std::vector<cudaEvent_t> prof_events[2];   // [0] = K1 quantizer, [1] = GEMM / GEMV
};

struct VxbWeight {
    int device = 0;
    uint32_t d_in = 0, d_out = 0, kpad = 0;
    int8_t* w = nullptr;       // [d_out, kpad]
    float* ws = nullptr;       // [d_out]
    float* bias_f32 = nullptr; // [d_out] or null
    int32_t* bias_i32 = nullptr;
    int32_t* wsum = nullptr;   // [d_out] sum of codes per channel
    CUtensorMap tmap_b;        // box 256 rows (large-M kernel)
    CUtensorMap tmap_w128;     // box 128 rows (stream-K decode kernel)
    CUtensorMap tmap_rows;     // box tile_rows rows (channel-owning decode kernel)
    uint32_t tile_rows = 0, tiles_per_cta = 0;
    bool has_tmap = false;
    uint64_t bytes = 0;
    float ws_min = 0.0f, ws_max = 0.0f;  // range of the per-channel scales
    // grouped scales (storage groups of the reference's PackedLinear): 0 = per-channel
    uint32_t group = 0, groups = 0;
    float* gscales = nullptr;  // [d_out, groups]
    float* gscales_t = nullptr;  // [groups, n_pad], n_pad = round_up(d_out, 128), padding zero (tensor-core grouped kernel)
    uint32_t n_pad = 0;
    uint32_t* w4 = nullptr;      // W4 storage kept as words [d_out, w4_row_words] for the one/two-row decode kernel
    uint32_t w4_row_words = 0;   // multiple of 4, * 8 >= kpad; codes past d_in are 8 (weight 0)
};

cudaStream_t vxb::context_stream(const VxbContext* ctx) { return ctx->stream; }

namespace {

int ensure_device(const VxbContext* ctx) {
    int cur = -1;
    CUDA_TRY(cudaGetDevice(&cur), -1);
    if (cur != ctx->device) CUDA_TRY(cudaSetDevice(ctx->device), -1);
    return 1;
}

void count_launch(int n = 1) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

constexpr size_t kMaxProfiledLaunches = 8192;
struct ProfileScope {
    VxbContext* ctx; int kind; bool on;
    ProfileScope(VxbContext* c, int k) : ctx(c), kind(k), on(false) {
        on = c->profiling && (c->prof_seen[k]++ % (uint32_t)c->profiling) == 0 && c->prof_events[k].size() < 2 * kMaxProfiledLaunches;
        if (on) { cudaEvent_t e; cudaEventCreate(&e); cudaEventRecord(e, ctx->stream); ctx->prof_events[kind].push_back(e); }
    }
    ~ProfileScope() {
        if (on) { cudaEvent_t e; cudaEventCreate(&e); cudaEventRecord(e, ctx->stream); ctx->prof_events[kind].push_back(e); }
    }
};

bool valid_scale(float v) { return std::isfinite(v) && v > 0.0f; }

// The requantizing epilogue may divide by out_scale through its precomputed reciprocal
// (div_const) when every operand stays far from the exponent limits and out_scale's
// significand is not all ones; otherwise the kernels use the IEEE divide.
void set_requant_divisor(EpilogueParams& epi, const VxbWeight* w, float out_scale);

// Finish building a weight whose int8 rows already sit (unpadded) in `staging` on the device.
int finish_weight(VxbContext* ctx, VxbWeight* w, const uint8_t* staging, uint32_t src_ld,
                  uint32_t xor_mask, const float* ws_host, const float* bias_f32,
                  const int32_t* bias_i32) {
    const uint32_t n = w->d_out, k = w->d_in;
    w->kpad = round_up(k, kKAlign);
    w->ws_min = w->ws_max = ws_host[0];
    for (uint32_t i = 1; i < n; i++) {
        w->ws_min = ws_host[i] < w->ws_min ? ws_host[i] : w->ws_min;
        w->ws_max = ws_host[i] > w->ws_max ? ws_host[i] : w->ws_max;
    }
    CUDA_TRY(cudaMalloc(&w->w, (size_t)n * w->kpad), 0);
    CUDA_TRY(cudaMalloc(&w->ws, (size_t)n * 4), 0);
    CUDA_TRY(cudaMalloc(&w->wsum, (size_t)n * 4), 0);
    w->bytes = (uint64_t)n * w->kpad + 8ull * n;
    CUDA_TRY(launch_repack_weight(staging, src_ld, n, k, xor_mask, w->w, w->kpad, w->wsum, ctx->stream), -1);
    count_launch();
    CUDA_TRY(cudaMemcpyAsync(w->ws, ws_host, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), -1);
    if (bias_f32) {
        CUDA_TRY(cudaMalloc(&w->bias_f32, (size_t)n * 4), 0);
        CUDA_TRY(cudaMemcpyAsync(w->bias_f32, bias_f32, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), -1);
        w->bytes += 4ull * n;
    }
    if (bias_i32) {
        CUDA_TRY(cudaMalloc(&w->bias_i32, (size_t)n * 4), 0);
        CUDA_TRY(cudaMemcpyAsync(w->bias_i32, bias_i32, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream), -1);
        w->bytes += 4ull * n;
    }
    w->has_tmap = encode_i8_rows(&w->tmap_b, w->w, n, w->kpad, 256) &&
                  encode_i8_rows(&w->tmap_w128, w->w, n, w->kpad, 128);
    decode_rows_plan(n, ctx->sm_count, &w->tile_rows, &w->tiles_per_cta);
    w->has_tmap = w->has_tmap && encode_i8_rows(&w->tmap_rows, w->w, n, w->kpad, w->tile_rows);
    CUDA_TRY(cudaStreamSynchronize(ctx->stream), -1);
    return 1;
}

void set_requant_divisor(EpilogueParams& epi, const VxbWeight* w, float out_scale) {
    uint32_t bits; memcpy(&bits, &out_scale, 4);
    const bool all_ones = (bits & 0x007fffffu) == 0x007fffffu;
    const float lo = 9.31322574615478515625e-10f, hi = 1073741824.0f;  // 2^-30 .. 2^30
    epi.out_scale = out_scale;
    epi.out_rcp = (float)(1.0 / (double)out_scale);
    epi.fast_div = (!all_ones && out_scale >= lo && out_scale <= hi && w->ws_min >= lo && w->ws_max <= hi) ? 1 : 0;
}

// Group scales that differ within a channel: keep them as given ([d_out, groups], CUDA-core
// kernel) and transposed and padded ([groups, n_pad], tensor-core kernel).
int upload_group_scales(VxbContext* ctx, VxbWeight* w, const float* group_scales, uint32_t d_out,
                        uint32_t groups, uint32_t group_size) {
    const size_t gbytes = (size_t)d_out * groups * 4;
    const uint32_t n_pad = (d_out + 127u) / 128u * 128u;
    std::vector<float> t((size_t)groups * n_pad, 0.0f);
    for (uint32_t n = 0; n < d_out; n++)
        for (uint32_t g = 0; g < groups; g++) t[(size_t)g * n_pad + n] = group_scales[(size_t)n * groups + g];
    if (cudaMalloc(&w->gscales, gbytes) != cudaSuccess || cudaMalloc(&w->gscales_t, t.size() * 4) != cudaSuccess)
        return fail(0, "group scale allocation failed");
    if (cudaMemcpyAsync(w->gscales, group_scales, gbytes, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(w->gscales_t, t.data(), t.size() * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
        return fail(-1, "group scale upload failed");
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return fail(-1, "group scale upload failed");
    w->group = group_size; w->groups = groups; w->n_pad = n_pad; w->bytes += gbytes + t.size() * 4;
    return 1;
}

// A refused launch (diag.h, vxb_inject_failure) looks like a launch the driver rejected.
#define LAUNCH_TRY(expr)                                                                                  \
    do { if (injected(g_fail_launch)) return fail(-1, "%s: launch refused (injected)", #expr);            \
         CUDA_TRY((expr), -1); } while (0)

uint32_t weight_kind(const VxbWeight* w) {
    return !w->group ? VXB_WEIGHT_PER_CHANNEL : w->w4 ? VXB_WEIGHT_W4_WORDS : VXB_WEIGHT_GROUPED;
}

VxbPlanQuery plan_query(const VxbContext* ctx, const VxbWeight* w, uint32_t rows, const EpilogueParams& epi, int requested, bool fp32_input) {
    VxbPlanQuery query{};
    query.rows = rows; query.k = w->d_in; query.n = w->d_out;
    query.weight_kind = weight_kind(w); query.group_size = w->group;
    query.epilogue = epi.mode == kEpiAcc ? VXB_EPI_ACC : epi.mode == kEpiF32 ? VXB_EPI_F32 : VXB_EPI_I8;
    query.requested_route = requested; query.n_peers = epi.n_peers;
    query.fused_tail = (epi.residual ? 1u : 0u) | (epi.act ? 2u : 0u);
    // TMA tile stores clip at the matrix edge in units of 16 bytes: the width must be a multiple of four 32-bit columns too
    query.out_store_aligned = (epi.mode != kEpiI8 && !((uintptr_t)epi.out & 15u) && !(epi.ld & 3u) && !(w->d_out & 3u)) ? 1u : 0u;
    if (epi.mode == kEpiI8 && epi.n_peers) {
        bool aligned = !((uintptr_t)epi.out & 15u) && !(epi.ld & 15u) && !(w->d_out & 15u) && tunables().gather_tma;
        for (uint32_t p = 0; p < epi.n_peers; p++) aligned = aligned && !((uintptr_t)epi.peer_out[p] & 15u);
        query.out_store_aligned = aligned ? 1u : 0u;
    }
    query.fp32_input = fp32_input ? 1u : 0u;
    query.sm_count = (uint32_t)ctx->sm_count;
    query.pair_clusters = (uint32_t)(gemm_pair_clusters() > 0 ? gemm_pair_clusters() : 0);
    return query;
}

// The decode kernel's single-launch form: the CTAs quantize the fp32 rows themselves.
int launch_decode_fused(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows, const EpilogueParams& epi,
                        const float* norm_weight = nullptr, float epsilon = 0.0f, float* norm_out = nullptr) {
    if (!w->has_tmap) return fail(0, "no tensor map for this weight (driver entry point missing)");
    if ((uintptr_t)x & 15u) return fail(0, "the single-launch decode form needs 16-byte aligned activations");
    DecodeRowsArgs a{};
    a.tmap_w = w->tmap_rows;
    a.rows = rows; a.n = w->d_out; a.kpad = w->kpad;
    a.tile_rows = w->tile_rows; a.tiles_per_cta = w->tiles_per_cta;
    a.w_stage_bytes = round_up(w->tile_rows * kKAlign, 1024u);
    a.x_f32 = x; a.k = w->d_in;
    a.norm_weight = norm_weight; a.norm_eps = (double)epsilon; a.norm_out = norm_out;
    a.epi = epi; a.status = ctx->status; a.trace = ctx->trace;
    if (!decode_rows_configure(a)) return fail(0, "no launch shape for the single-launch decode form (rows %u, d_out %u)", rows, w->d_out);
    ProfileScope scope(ctx, 1);
    LAUNCH_TRY(launch_decode_rows(a, ctx->stream));
    count_launch();
    const char* tail = epi.mode == kEpiAcc ? "acc" : epi.mode == kEpiF32 ? "e1" : "e2";
    snprintf(g_route, sizeof g_route, "%s%s+%s", norm_weight ? "norm+" : "", vxb_variant_info(VXB_VARIANT_DECODE_FUSED)->route_label, tail);
    return 1;
}

// int32 GEMM + epilogue over already-quantized activations q [rows, kpad].  The kernel is the one
// vxb_plan() names for this call: the same function tests call without a GPU.
int run_gemm(VxbContext* ctx, const VxbWeight* w, const int8_t* q, uint32_t rows,
             const EpilogueParams& epi, int requested, const char* prefix) {
    if (!ctx->tcgen05_ready) {
        CUDA_TRY(gemm_tcgen05_prepare(), 0);
        ctx->tcgen05_ready = true;
    }
    if (!ctx->pair_ready) {
        CUDA_TRY(gemm_pair_prepare(), 0);
        ctx->pair_ready = true;
    }
    if (requested == VXB_ROUTE_DECODE_FUSED) return fail(0, "the single-launch decode form starts from fp32 rows");
    const VxbPlanQuery query = plan_query(ctx, w, rows, epi, requested, false);
    VxbLaunchPlan plan;
    char why[160];
    if (vxb_plan(&query, &plan, why, sizeof why) != 1) return fail(0, "%s", why);
    const VxbVariant* variant = vxb_variant_info((uint32_t)plan.variant);
    const bool tensor_map_route = plan.variant == VXB_VARIANT_DECODE_ROWS || plan.variant == VXB_VARIANT_DECODE_STREAMK ||
                                  plan.variant == VXB_VARIANT_TCGEN05 || plan.variant == VXB_VARIANT_TCGEN05_PAIR ||
                                  plan.variant == VXB_VARIANT_GROUPED_TCGEN05;
    if (tensor_map_route && !w->has_tmap) return fail(0, "no tensor map for this weight (driver entry point missing)");
    EpilogueParams ge = epi;
    if (w->group) { ge.gscales = w->gscales; ge.group = w->group; ge.groups = w->groups; }
    ProfileScope scope(ctx, 1);
    switch (plan.variant) {
        case VXB_VARIANT_GEMV_W4_GROUPED:
            // W4 storage: the decode kernel over the 4-bit words themselves (half the bytes)
            LAUNCH_TRY(launch_gemv_w4_grouped(q, rows, w->w4, w->w4_row_words, w->d_out, w->kpad, ge, ctx->sm_count, ctx->stream));
            break;
        case VXB_VARIANT_GEMV_GROUPED:
            LAUNCH_TRY(launch_gemv_grouped(q, rows, w->w, w->d_out, w->kpad, ge, ctx->sm_count, ctx->stream));
            break;
        case VXB_VARIANT_GROUPED_TCGEN05: {
            if (!w->gscales_t) return fail(0, "no transposed group-scale table for this weight");
            if (!ctx->grouped_ready) {
                CUDA_TRY(gemm_grouped_tcgen05_prepare(), 0);
                ctx->grouped_ready = true;
            }
            GemmGroupedArgs a;
            if (!encode_i8_rows(&a.tmap_a, q, rows, w->kpad, 128)) return fail(0, "cuTensorMapEncodeTiled failed for activations");
            a.tmap_b = w->tmap_w128;
            a.rows = rows; a.n = w->d_out; a.kpad = w->kpad;
            a.group = w->group; a.groups = w->groups; a.n_pad = w->n_pad; a.gscales_t = w->gscales_t;
            a.row_scales = epi.row_scales; a.bias = epi.bias_f32; a.out = (float*)epi.out; a.ld = epi.ld;
            a.status = ctx->status;
            LAUNCH_TRY(launch_gemm_grouped_tcgen05(a, ctx->sm_count, ctx->stream));
            break;
        }
        case VXB_VARIANT_DP4A_GROUPED:
            LAUNCH_TRY(launch_gemm_grouped(q, rows, w->w, w->d_out, w->kpad, ge, ctx->stream));
            break;
        case VXB_VARIANT_GEMV_DP4A:
            LAUNCH_TRY(launch_gemv(q, rows, w->w, w->d_out, w->kpad, epi, ctx->sm_count, ctx->stream));
            break;
        case VXB_VARIANT_SIMT_DP4A:
            LAUNCH_TRY(launch_gemm_simt(q, rows, w->w, w->d_out, w->kpad, epi, ctx->stream));
            break;
        case VXB_VARIANT_DECODE_ROWS: {
            DecodeRowsArgs a{};
            a.tmap_w = w->tmap_rows;
            a.rows = rows; a.n = w->d_out; a.kpad = w->kpad;
            a.tile_rows = w->tile_rows; a.tiles_per_cta = w->tiles_per_cta;
            a.w_stage_bytes = round_up(w->tile_rows * kKAlign, 1024u);
            a.epi = epi; a.status = ctx->status; a.trace = ctx->trace;
            if (!decode_rows_configure(a)) return fail(0, "no launch shape for the decode kernel (rows %u, d_out %u)", rows, w->d_out);
            if (!encode_i8_kblocks(&a.tmap_x, q, rows, w->kpad, decode_rows_token_slots(rows), a.x_chunk_blocks))
                return fail(0, "cuTensorMapEncodeTiled failed for activations");
            LAUNCH_TRY(launch_decode_rows(a, ctx->stream));
            break;
        }
        case VXB_VARIANT_DECODE_STREAMK: {
            // split-K scratch: int32 [rows, d_out] + one counter per 128-channel tile, kept zero
            const size_t ws_bytes = (size_t)128 * w->d_out * 4, cnt_bytes = (size_t)((w->d_out + 127) / 128) * 4;
            if (ctx->splitk_ws.bytes < ws_bytes) {
                CUDA_TRY(ctx->splitk_ws.reserve(ws_bytes), 0);
                CUDA_TRY(cudaMemsetAsync(ctx->splitk_ws.ptr, 0, ctx->splitk_ws.bytes, ctx->stream), -1);
            }
            if (ctx->splitk_counters.bytes < cnt_bytes) {
                CUDA_TRY(ctx->splitk_counters.reserve(cnt_bytes), 0);
                CUDA_TRY(cudaMemsetAsync(ctx->splitk_counters.ptr, 0, ctx->splitk_counters.bytes, ctx->stream), -1);
            }
            DecodeTcgen05Args a;
            if (!encode_i8_rows(&a.tmap_x, q, rows, w->kpad, decode_token_slots(rows)))
                return fail(0, "cuTensorMapEncodeTiled failed for activations");
            a.tmap_w = w->tmap_w128;
            a.rows = rows; a.n = w->d_out; a.kpad = w->kpad; a.epi = epi;
            a.workspace = (int32_t*)ctx->splitk_ws.ptr; a.counters = (uint32_t*)ctx->splitk_counters.ptr;
            a.status = ctx->status;
            LAUNCH_TRY(launch_decode_tcgen05(a, ctx->sm_count, ctx->stream));
            break;
        }
        case VXB_VARIANT_TCGEN05: case VXB_VARIANT_TCGEN05_PAIR: case VXB_VARIANT_TCGEN05_WIDE: {
            GemmTcgen05Args a;
            if (!encode_i8_rows(&a.tmap_a, q, rows, w->kpad, 128)) return fail(0, "cuTensorMapEncodeTiled failed for activations");
            a.rows = rows; a.n = w->d_out; a.kpad = w->kpad; a.epi = epi; a.status = ctx->status; a.trace = ctx->trace; a.tma_out = 0;
            if (plan.variant == VXB_VARIANT_TCGEN05_PAIR) {
                a.tmap_b = w->tmap_w128;   // each CTA of a pair loads half of the tile's weight rows
                a.gather_tma = 0;
                if (epi.n_peers) {
                    bool ok = encode_gather_i8(&a.tmap_gather[0], epi.out, rows, w->d_out, epi.ld, 64);
                    for (uint32_t p = 0; ok && p < epi.n_peers; p++)
                        ok = encode_gather_i8(&a.tmap_gather[p + 1], epi.peer_out[p], rows, w->d_out, epi.ld, 64);
                    if (!ok) return fail(0, "cuTensorMapEncodeTiled failed for a gather destination");
                    a.gather_tma = 1;
                }
                LAUNCH_TRY(launch_gemm_pair(a, ctx->stream));
            } else if (plan.variant == VXB_VARIANT_TCGEN05_WIDE) {
                a.tmap_b = w->tmap_b;
                if (!encode_out32(&a.tmap_out, epi.out, rows, w->d_out, epi.ld)) return fail(0, "cuTensorMapEncodeTiled failed for the output");
                a.tma_out = 1;
                LAUNCH_TRY(launch_gemm_wide(a, ctx->sm_count, ctx->stream));
            } else {
                a.tmap_b = w->tmap_b;
                a.gather_tma = 0;
                // (a tile store clips at the shard's edge in units of 16 bytes: whole 16-channel groups only)
                if (epi.n_peers && epi.mode == kEpiI8 && tunables().gather_tma && !(w->d_out & 15u)) {
                    bool ok = encode_gather_i8(&a.tmap_gather[0], epi.out, rows, w->d_out, epi.ld);
                    for (uint32_t p = 0; ok && p < epi.n_peers; p++)
                        ok = encode_gather_i8(&a.tmap_gather[p + 1], epi.peer_out[p], rows, w->d_out, epi.ld);
                    a.gather_tma = ok ? 1u : 0u;   // otherwise the per-lane stores serve (unaligned buffers)
                }
                LAUNCH_TRY(launch_gemm_tcgen05(a, ctx->sm_count, ctx->stream));
            }
            break;
        }
        default:
            return fail(0, "variant %d has no launcher", plan.variant);
    }
    count_launch();
    const char* tail = epi.mode == kEpiAcc ? "acc" : epi.mode == kEpiF32 ? "e1" : "e2";
    snprintf(g_route, sizeof g_route, "%s%s+%s", prefix, variant->route_label, tail);
    return 1;
}

int check_common(const VxbContext* ctx, const VxbWeight* w, const void* x, const void* y, uint32_t ldy) {
    if (!ctx || !w || !x || !y) return fail(0, "null argument");
    if (w->device != ctx->device) return fail(0, "weight lives on device %d, context on %d", w->device, ctx->device);
    if (ldy < w->d_out) return fail(0, "output row stride %u < d_out %u", ldy, w->d_out);
    return 1;
}

int quantize_into_scratch(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                          const float* norm_weight = nullptr, float epsilon = 0.0f, float* norm_out = nullptr) {
    CUDA_TRY(ctx->q.reserve((size_t)rows * w->kpad), 0);
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    {
        ProfileScope scope(ctx, 0);
        if (norm_weight)
            LAUNCH_TRY(launch_rmsnorm_quantize_rows(x, norm_weight, epsilon, rows, w->d_in, norm_out, (int8_t*)ctx->q.ptr,
                                                    w->kpad, (float*)ctx->row_scales.ptr, nullptr, ctx->stream));
        else
            LAUNCH_TRY(launch_quantize_rows(x, rows, w->d_in, (int8_t*)ctx->q.ptr, w->kpad,
                                            (float*)ctx->row_scales.ptr, nullptr, ctx->stream));
    }
    count_launch();
    return 1;
}

// Rows of the first chunk when a large batch is cut in two so that the quantizer of the later rows
// runs under the GEMM of the first ones (K1 is HBM-bound, K2 tensor-bound or link-bound): 0 = do
// not split.  Off unless the tunable "gemm.overlap_k1" is set: on the B200 the GEMM kernels hold 168
// registers per thread, so no quantizer CTA fits beside them and the second quantizer simply queues
// behind the first GEMM (325 -> 381 us per step at M 8192, K 4096, N 14336); with 128-register
// builds of the GEMM kernels the quantizer did run underneath, and slowed the GEMM by as much as
// it saved (361 -> 364 us).  The first chunk is the smallest number of row tiles whose GEMM lasts at least as
// long as the quantizer of the rest and that adds no wave of tiles to the launch pair.
uint32_t overlap_first_rows(const VxbContext* ctx, const VxbWeight* w, uint32_t rows, const EpilogueParams& epi, int route) {
    const bool gather = epi.n_peers != 0;
    // only when a tunable asks for it (see overlap_first_rows' note and the gather kernel's)
    const bool link_bound = gather_is_link_bound(epi.n_peers, w->kpad);
    if (!(link_bound ? tunables().overlap_gather : tunables().overlap_k1) || w->group || rows < 2048) return 0;
    if (route != VXB_ROUTE_AUTO && route != VXB_ROUTE_TCGEN05 && route != VXB_ROUTE_TCGEN05_PAIR) return 0;
    const uint32_t tiles128 = ((rows + 127) / 128) * ((w->d_out + 255) / 256);
    const bool pair = !gather && route != VXB_ROUTE_TCGEN05 && gemm_pair_clusters() > 0 &&
                      (route == VXB_ROUTE_TCGEN05_PAIR || tiles128 >= 2u * (uint32_t)ctx->sm_count);
    const uint32_t tile_rows = pair ? 256u : 128u;
    const uint32_t slots = pair ? (uint32_t)gemm_pair_clusters() : (uint32_t)ctx->sm_count;
    const uint32_t cols = (w->d_out + 255) / 256, row_tiles = (rows + tile_rows - 1) / tile_rows;
    if (row_tiles < 4) return 0;
    auto waves = [&](uint32_t r) { return (r * cols + slots - 1) / slots; };
    // GEMM seconds per row ~ 2 K N / 3.3e15 (link-bound with peers: slower still), quantizer seconds per
    // row ~ 5 K / 4.7e12: the first chunk needs rows_first / rows_rest >= 1755 / N
    const double ratio = (double)tunables().overlap_ratio / (double)w->d_out;
    uint32_t r_min = gather ? 1u : (uint32_t)((double)row_tiles * ratio / (1.0 + ratio)) + 1;
    if (r_min >= row_tiles) return 0;
    uint32_t best = 0;
    if (!gather) {
        for (uint32_t r = r_min; r < row_tiles && r <= 2 * r_min + 4; r++)
            if (waves(r) + waves(row_tiles - r) == waves(row_tiles)) { best = r; break; }
        if (!best) return 0;   // every cut here would idle part of a wave: keep the single launch
    } else best = r_min < row_tiles / 4 ? row_tiles / 4 : r_min;   // link-bound launch: a quarter of the rows is plenty
    return best * tile_rows;
}

// Quantizer + GEMM of one call; a large batch takes the overlapped form when the side stream exists
// (it is created on first use outside stream capture).
int quantize_then_gemm(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows, const EpilogueParams& epi,
                       int route, const char* prefix, const float* norm_weight = nullptr, float epsilon = 0.0f,
                       float* norm_out = nullptr) {
    if ((route == VXB_ROUTE_AUTO || route == VXB_ROUTE_DECODE_FUSED) && rows <= 8) {
        // up to 8 rows: one launch, the decode kernel normalizes (when asked to) and quantizes the rows itself
        // (when the plan admits it)
        const VxbPlanQuery query = plan_query(ctx, w, rows, epi, route, true);
        VxbLaunchPlan plan;
        char why[160];
        const int planned = vxb_plan(&query, &plan, why, sizeof why);
        const bool aligned = (((uintptr_t)x | (uintptr_t)norm_weight | (uintptr_t)norm_out) & 15u) == 0;
        if (planned == 1 && plan.variant == VXB_VARIANT_DECODE_FUSED && aligned)
            return launch_decode_fused(ctx, w, x, rows, epi, norm_weight, epsilon, norm_out);
        if (route == VXB_ROUTE_DECODE_FUSED) return fail(0, "%s", planned == 1 ? "activations are not 16-byte aligned" : why);
    } else if (route == VXB_ROUTE_DECODE_FUSED) {
        return fail(0, "the single-launch decode form serves up to 8 rows");
    }
    uint32_t first = norm_weight ? 0u : overlap_first_rows(ctx, w, rows, epi, route);
    if (first) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->stream, &capturing) != cudaSuccess) { cudaGetLastError(); capturing = cudaStreamCaptureStatusActive; }
        if (!ctx->side && capturing == cudaStreamCaptureStatusNone) {
            if (cudaStreamCreateWithFlags(&ctx->side, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&ctx->ev_first, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&ctx->ev_rest, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError(); ctx->side = nullptr;
            }
        }
        if (!ctx->side) first = 0;
    }
    if (!first) {
        int rc = quantize_into_scratch(ctx, w, x, rows, norm_weight, epsilon, norm_out);
        if (rc != 1) return rc;
        return run_gemm(ctx, w, (const int8_t*)ctx->q.ptr, rows, epi, route, prefix);
    }
    CUDA_TRY(ctx->q.reserve((size_t)rows * w->kpad), 0);
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    int8_t* q = (int8_t*)ctx->q.ptr; float* scales = (float*)ctx->row_scales.ptr;
    const uint32_t rest = rows - first;
    {
        ProfileScope scope(ctx, 0);
        LAUNCH_TRY(launch_quantize_rows(x, first, w->d_in, q, w->kpad, scales, nullptr, ctx->stream));
    }
    // the quantizer of the rest starts when the first chunk's has finished (two at once would only share
    // the HBM bandwidth) and runs under the first chunk's GEMM
    CUDA_TRY(cudaEventRecord(ctx->ev_first, ctx->stream), -1);
    CUDA_TRY(cudaStreamWaitEvent(ctx->side, ctx->ev_first, 0), -1);
    LAUNCH_TRY(launch_quantize_rows(x + (size_t)first * w->d_in, rest, w->d_in, q + (size_t)first * w->kpad, w->kpad,
                                    scales + first, nullptr, ctx->side));
    CUDA_TRY(cudaEventRecord(ctx->ev_rest, ctx->side), -1);
    count_launch(2);
    int rc = run_gemm(ctx, w, q, first, epi, route, prefix);
    if (rc != 1) { cudaStreamWaitEvent(ctx->stream, ctx->ev_rest, 0); return rc; }   // 0: no output was touched
    CUDA_TRY(cudaStreamWaitEvent(ctx->stream, ctx->ev_rest, 0), -1);
    EpilogueParams tail = epi;
    const size_t elem = epi.mode == kEpiI8 ? 1 : 4;
    tail.row_scales = epi.row_scales + first;
    tail.out = (uint8_t*)epi.out + (size_t)first * epi.ld * elem;
    if (epi.residual) tail.residual = epi.residual + (size_t)first * epi.ld_res;
    for (uint32_t p = 0; p < epi.n_peers; p++) tail.peer_out[p] = (uint8_t*)epi.peer_out[p] + (size_t)first * epi.ld * elem;
    char overlapped[32];
    snprintf(overlapped, sizeof overlapped, "%s", prefix);
    rc = run_gemm(ctx, w, q + (size_t)first * w->kpad, rest, tail, route, overlapped);
    if (rc == 1) {
        char route_text[96];
        snprintf(route_text, sizeof route_text, "%s", g_route);
        snprintf(g_route, sizeof g_route, "%s|2-chunk-overlap", route_text);
    }
    return rc == 0 ? -1 : rc;
}

}  // namespace

extern "C" {

uint32_t vxb_abi_version(void) { return VXB_ABI_VERSION; }
const char* vxb_last_error(void) { return g_error; }
const char* vxb_last_route(void) { return g_route; }
uint64_t vxb_launch_count(void) { return g_launches.load(); }

int vxb_context_create(int device, void* stream, VxbContext** out) {
    if (!out) return fail(0, "null out");
    *out = nullptr;
    int count = 0;
    CUDA_TRY(cudaGetDeviceCount(&count), 0);
    if (device < 0 || device >= count) return fail(0, "device %d out of range (%d present)", device, count);
    CUDA_TRY(cudaSetDevice(device), 0);
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device), 0);
    if (prop.major != 10) return fail(0, "device %d is sm_%d%d; this library is sm_100a only", device, prop.major, prop.minor);
    VxbContext* ctx = new VxbContext();
    ctx->device = device; ctx->stream = (cudaStream_t)stream; ctx->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&ctx->status, 2 * sizeof(int)) != cudaSuccess ||
        cudaMemset(ctx->status, 0, 2 * sizeof(int)) != cudaSuccess ||
        cudaMallocHost(&ctx->status_host, sizeof(int)) != cudaSuccess) {
        delete ctx;
        return fail(0, "context allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    *out = ctx;
    return 1;
}

void vxb_context_destroy(VxbContext* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& v : ctx->prof_events) { for (cudaEvent_t e : v) cudaEventDestroy(e); v.clear(); }
    ctx->q.release(); ctx->row_scales.release(); ctx->bias_eff.release();
    ctx->stage_in.release(); ctx->stage_out.release();
    ctx->splitk_ws.release(); ctx->splitk_counters.release();
    if (ctx->copy_in) {
        cudaStreamDestroy(ctx->copy_in); cudaStreamDestroy(ctx->copy_out);
        for (int b = 0; b < 2; b++) { cudaEventDestroy(ctx->ev_in[b]); cudaEventDestroy(ctx->ev_done[b]); cudaEventDestroy(ctx->ev_out[b]); }
        cudaEventDestroy(ctx->ev_start);
    }
    if (ctx->ev_switch) cudaEventDestroy(ctx->ev_switch);
    if (ctx->side) { cudaStreamDestroy(ctx->side); cudaEventDestroy(ctx->ev_first); cudaEventDestroy(ctx->ev_rest); }
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    delete ctx;
}

int vxb_context_set_stream(VxbContext* ctx, void* stream) {
    if (!ctx) return fail(0, "null context");
    cudaStream_t next = (cudaStream_t)stream;
    if (next == ctx->stream) return 1;
    // The context's scratch (quantized rows, row scales, split-K workspace, status block) is shared
    // by everything queued through it: work on the new stream must not overtake what is still
    // queued on the old one.  Under stream capture the recording is skipped (an event of a stream
    // that is not part of the capture cannot be waited on there); the caller orders the streams.
    if (ensure_device(ctx) != 1) return -1;
    cudaStreamCaptureStatus cap_old = cudaStreamCaptureStatusNone, cap_new = cudaStreamCaptureStatusNone;
    const bool plain = cudaStreamIsCapturing(ctx->stream, &cap_old) == cudaSuccess && cap_old == cudaStreamCaptureStatusNone &&
                       cudaStreamIsCapturing(next, &cap_new) == cudaSuccess && cap_new == cudaStreamCaptureStatusNone;
    cudaGetLastError();
    if (plain) {
        if (!ctx->ev_switch) CUDA_TRY(cudaEventCreateWithFlags(&ctx->ev_switch, cudaEventDisableTiming), 0);
        CUDA_TRY(cudaEventRecord(ctx->ev_switch, ctx->stream), -1);
        CUDA_TRY(cudaStreamWaitEvent(next, ctx->ev_switch, 0), -1);
    }
    ctx->stream = next;
    return 1;
}

int vxb_context_synchronize(VxbContext* ctx) {
    if (!ctx) return fail(0, "null context");
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(cudaMemcpyAsync(ctx->status_host, ctx->status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream), -1);
    CUDA_TRY(cudaStreamSynchronize(ctx->stream), -1);
    if (*ctx->status_host != 0) {
        const int code = *ctx->status_host;
        cudaMemsetAsync(ctx->status, 0, sizeof(int), ctx->stream);
        if (ctx->splitk_ws.ptr) cudaMemsetAsync(ctx->splitk_ws.ptr, 0, ctx->splitk_ws.bytes, ctx->stream);
        if (ctx->splitk_counters.ptr) cudaMemsetAsync(ctx->splitk_counters.ptr, 0, ctx->splitk_counters.bytes, ctx->stream);
        return fail(-1, "a bounded device wait expired (status %d); results of this batch are invalid", code);
    }
    return 1;
}

int vxb_weight_create_i8(VxbContext* ctx, const int8_t* weight, const float* weight_scales,
                         const float* bias_f32, const int32_t* bias_i32, uint32_t d_out,
                         uint32_t d_in, VxbWeight** out) {
    if (!ctx || !weight || !weight_scales || !out) return fail(0, "null argument");
    *out = nullptr;
    if (!d_out || !d_in) return fail(0, "empty weight");
    // K*127*128 must stay inside int32 (the reference's overflow proof,
    // native/src/kernels/packed_quant_gemm.c:741-755)
    if ((uint64_t)d_in * 127u * 128u > 2147483647ull) return fail(0, "d_in %u can overflow the int32 accumulator", d_in);
    for (uint32_t i = 0; i < d_out; i++)
        if (!valid_scale(weight_scales[i])) return fail(0, "weight scale %u is not positive and finite", i);
    if (ensure_device(ctx) != 1) return -1;
    VxbWeight* w = new VxbWeight();
    w->device = ctx->device; w->d_in = d_in; w->d_out = d_out;
    Buffer staging;
    int rc;
    if (staging.reserve((size_t)d_out * d_in) != cudaSuccess) { rc = fail(0, "staging allocation failed"); }
    else if (cudaMemcpyAsync(staging.ptr, weight, (size_t)d_out * d_in, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) {
        rc = fail(-1, "weight upload failed");
    } else {
        rc = finish_weight(ctx, w, (const uint8_t*)staging.ptr, d_in, 0u, weight_scales, bias_f32, bias_i32);
    }
    cudaStreamSynchronize(ctx->stream);
    staging.release();
    if (rc != 1) { vxb_weight_destroy(w); return rc; }
    *out = w;
    return 1;
}

int vxb_weight_create_w8_words(VxbContext* ctx, const int32_t* words, const float* group_scales,
                               const float* bias_f32, uint32_t d_out, uint32_t d_in,
                               uint32_t group_size, VxbWeight** out) {
    if (!ctx || !words || !group_scales || !out) return fail(0, "null argument");
    *out = nullptr;
    if (!d_out || !d_in) return fail(0, "empty weight");
    if (group_size != 32 && group_size != 64 && group_size != 128 && group_size != 256)
        return fail(0, "group size %u is not 32/64/128/256", group_size);
    if ((uint64_t)d_in * 127u * 128u > 2147483647ull) return fail(0, "d_in %u can overflow the int32 accumulator", d_in);
    const uint32_t groups = (d_in + group_size - 1) / group_size, row_words = (d_in + 3) / 4;
    std::vector<float> ws(d_out);
    bool grouped = false;   // some channel's groups differ: the grouped-scale kernel serves this weight
    for (uint32_t n = 0; n < d_out; n++) {
        const float s = group_scales[(size_t)n * groups];
        for (uint32_t g = 0; g < groups; g++) {
            const float sg = group_scales[(size_t)n * groups + g];
            if (!valid_scale(sg)) return fail(0, "scale of channel %u, group %u is not positive and finite", n, g);
            if (memcmp(&sg, &s, 4) != 0) grouped = true;
        }
        ws[n] = s;
        // canonical padding: unused bytes of the final word hold the encoded zero 0x80
        const uint8_t* bytes = (const uint8_t*)(words + (size_t)n * row_words);
        for (uint32_t j = d_in; j < row_words * 4; j++)
            if (bytes[j] != 0x80u) return fail(0, "channel %u: padding byte %u is not the encoded zero", n, j);
    }
    if (ensure_device(ctx) != 1) return -1;
    VxbWeight* w = new VxbWeight();
    w->device = ctx->device; w->d_in = d_in; w->d_out = d_out;
    Buffer staging;
    int rc;
    const size_t src_bytes = (size_t)d_out * row_words * 4;
    if (staging.reserve(src_bytes) != cudaSuccess) rc = fail(0, "staging allocation failed");
    else if (cudaMemcpyAsync(staging.ptr, words, src_bytes, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
        rc = fail(-1, "weight upload failed");
    else rc = finish_weight(ctx, w, (const uint8_t*)staging.ptr, row_words * 4, 0x80u, ws.data(), bias_f32, nullptr);
    if (rc == 1 && grouped) rc = upload_group_scales(ctx, w, group_scales, d_out, groups, group_size);
    cudaStreamSynchronize(ctx->stream);
    staging.release();
    if (rc != 1) { vxb_weight_destroy(w); return rc; }
    *out = w;
    return 1;
}

int vxb_weight_create_w4_words(VxbContext* ctx, const int32_t* words, const float* group_scales,
                               const float* bias_f32, uint32_t d_out, uint32_t d_in,
                               uint32_t group_size, VxbWeight** out) {
    if (!ctx || !words || !group_scales || !out) return fail(0, "null argument");
    *out = nullptr;
    if (!d_out || !d_in) return fail(0, "empty weight");
    if (group_size != 32 && group_size != 64 && group_size != 128 && group_size != 256)
        return fail(0, "group size %u is not 32/64/128/256", group_size);
    const uint32_t groups = (d_in + group_size - 1) / group_size, row_words = (d_in + 7) / 8;
    std::vector<float> ws(d_out);
    bool grouped = false;
    for (uint32_t n = 0; n < d_out; n++) {
        const float s = group_scales[(size_t)n * groups];
        for (uint32_t g = 0; g < groups; g++) {
            const float sg = group_scales[(size_t)n * groups + g];
            if (!valid_scale(sg)) return fail(0, "scale of channel %u, group %u is not positive and finite", n, g);
            if (memcmp(&sg, &s, 4) != 0) grouped = true;
        }
        ws[n] = s;
    }
    // unpack once: eight codes per word, earlier K in lower bits, w = code - 8; padding codes must be 8
    std::vector<int8_t> dense((size_t)d_out * d_in);
    for (uint32_t n = 0; n < d_out; n++) {
        const uint32_t* wr = (const uint32_t*)words + (size_t)n * row_words;
        for (uint32_t j = 0; j < row_words * 8; j++) {
            const int32_t code = (int32_t)((wr[j >> 3] >> (4u * (j & 7u))) & 0xFu);
            if (j < d_in) dense[(size_t)n * d_in + j] = (int8_t)(code - 8);
            else if (code != 8) return fail(0, "channel %u: padding code %u is not the encoded zero", n, j);
        }
    }
    if (ensure_device(ctx) != 1) return -1;
    VxbWeight* w = new VxbWeight();
    w->device = ctx->device; w->d_in = d_in; w->d_out = d_out;
    Buffer staging;
    int rc;
    if (staging.reserve(dense.size()) != cudaSuccess) rc = fail(0, "staging allocation failed");
    else if (cudaMemcpyAsync(staging.ptr, dense.data(), dense.size(), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
        rc = fail(-1, "weight upload failed");
    else rc = finish_weight(ctx, w, (const uint8_t*)staging.ptr, d_in, 0u, ws.data(), bias_f32, nullptr);
    if (rc == 1 && grouped) rc = upload_group_scales(ctx, w, group_scales, d_out, groups, group_size);
    if (rc == 1 && grouped) {
        // the words themselves, rows padded with the encoded zero to the padded K of the int8 copy
        const uint32_t padded_words = w->kpad / 8u;
        std::vector<uint32_t> padded((size_t)d_out * padded_words, 0x88888888u);
        for (uint32_t n = 0; n < d_out; n++)
            memcpy(&padded[(size_t)n * padded_words], (const uint32_t*)words + (size_t)n * row_words, (size_t)row_words * 4);
        if (cudaMalloc(&w->w4, padded.size() * 4) != cudaSuccess) rc = fail(0, "W4 word allocation failed");
        else if (cudaMemcpyAsync(w->w4, padded.data(), padded.size() * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
                 cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = fail(-1, "W4 word upload failed");
        else { w->w4_row_words = padded_words; w->bytes += padded.size() * 4; }
    }
    cudaStreamSynchronize(ctx->stream);
    staging.release();
    if (rc != 1) { vxb_weight_destroy(w); return rc; }
    *out = w;
    return 1;
}

void vxb_weight_destroy(VxbWeight* w) {
    if (!w) return;
    cudaSetDevice(w->device);
    if (w->w) cudaFree(w->w);
    if (w->ws) cudaFree(w->ws);
    if (w->bias_f32) cudaFree(w->bias_f32);
    if (w->bias_i32) cudaFree(w->bias_i32);
    if (w->wsum) cudaFree(w->wsum);
    if (w->gscales) cudaFree(w->gscales);
    if (w->gscales_t) cudaFree(w->gscales_t);
    if (w->w4) cudaFree(w->w4);
    delete w;
}
uint32_t vxb_weight_d_in(const VxbWeight* w) { return w ? w->d_in : 0; }
uint32_t vxb_weight_d_out(const VxbWeight* w) { return w ? w->d_out : 0; }
uint64_t vxb_weight_device_bytes(const VxbWeight* w) { return w ? w->bytes : 0; }

int vxb_quantize_rows(VxbContext* ctx, const float* x, uint32_t rows, uint32_t k, int8_t* q,
                      uint32_t ldq, float* row_scales, int32_t* valid) {
    if (!ctx || !x || !q || !row_scales) return fail(0, "null argument");
    if (!k || ldq < k) return fail(0, "bad widths k=%u ldq=%u", k, ldq);
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(launch_quantize_rows(x, rows, k, q, ldq, row_scales, valid, ctx->stream), -1);
    count_launch();
    snprintf(g_route, sizeof g_route, "k1");
    return 1;
}

int vxb_linear_f32(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows, float* y,
                   uint32_t ldy, int route) {
    int rc = check_common(ctx, w, x, y, ldy);
    if (rc != 1) return rc;
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    EpilogueParams epi{};
    epi.mode = kEpiF32; epi.row_scales = (const float*)ctx->row_scales.ptr; epi.ws = w->ws;
    epi.bias_f32 = w->bias_f32; epi.out = y; epi.ld = ldy;
    return quantize_then_gemm(ctx, w, x, rows, epi, route, "k1+");
}

static int fused_linear(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows, float* y,
                        uint32_t ldy, const float* residual, uint32_t ld_residual, int activation,
                        const float* norm_weight, float epsilon, float* norm_out) {
    if (!ctx || !w || !x || !y) return fail(0, "null argument");
    if (w->device != ctx->device) return fail(0, "weight lives on device %d, context on %d", w->device, ctx->device);
    if (activation != VXB_ACT_NONE && activation != VXB_ACT_SILU_MUL) return fail(0, "unknown activation %d", activation);
    if (w->group) return fail(0, "weights with grouped scales have no fused epilogue");
    const uint32_t width = activation == VXB_ACT_SILU_MUL ? w->d_out / 2 : w->d_out;
    if (activation == VXB_ACT_SILU_MUL && ((w->d_out & 1u) || residual))
        return fail(0, "SiLU * up needs an even channel count and takes no residual");
    if (ldy < width) return fail(0, "output row stride %u < output width %u", ldy, width);
    if (residual && ld_residual < width) return fail(0, "residual row stride %u < output width %u", ld_residual, width);
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    EpilogueParams epi{};
    epi.mode = kEpiF32; epi.row_scales = (const float*)ctx->row_scales.ptr; epi.ws = w->ws;
    epi.bias_f32 = w->bias_f32; epi.out = y; epi.ld = ldy;
    epi.residual = residual; epi.ld_res = ld_residual; epi.act = activation == VXB_ACT_SILU_MUL ? 1u : 0u;
    // the decode kernel up to 128 rows, the tensor-core GEMM above: both carry the fused forms
    return quantize_then_gemm(ctx, w, x, rows, epi, VXB_ROUTE_AUTO, norm_weight ? "norm+k1+" : "k1+", norm_weight, epsilon, norm_out);
}

int vxb_linear_f32_fused(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows, float* y,
                         uint32_t ldy, const float* residual, uint32_t ld_residual, int activation) {
    return fused_linear(ctx, w, x, rows, y, ldy, residual, ld_residual, activation, nullptr, 0.0f, nullptr);
}

int vxb_rmsnorm_linear_f32_fused(VxbContext* ctx, const VxbWeight* w, const float* x, const float* norm_weight,
                                 float epsilon, float* norm_out, uint32_t rows, float* y, uint32_t ldy,
                                 int activation) {
    if (!norm_weight) return fail(0, "null norm weight");
    if (!(epsilon > 0.0f) || !std::isfinite(epsilon)) return fail(0, "epsilon is not positive and finite");
    if (norm_out && x == norm_out) return fail(0, "the normalized rows cannot overwrite the input");
    return fused_linear(ctx, w, x, rows, y, ldy, nullptr, 0, activation, norm_weight, epsilon, norm_out);
}

int vxb_rmsnorm_quantize_rows(VxbContext* ctx, const float* x, const float* norm_weight, float epsilon,
                              uint32_t rows, uint32_t k, float* norm_out, int8_t* q, uint32_t ldq,
                              float* row_scales, int32_t* valid) {
    if (!ctx || !x || !norm_weight || !q || !row_scales) return fail(0, "null argument");
    if (!k || ldq < k) return fail(0, "bad widths k=%u ldq=%u", k, ldq);
    if (!(epsilon > 0.0f) || !std::isfinite(epsilon)) return fail(0, "epsilon is not positive and finite");
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(launch_rmsnorm_quantize_rows(x, norm_weight, epsilon, rows, k, norm_out, q, ldq, row_scales, valid,
                                          ctx->stream), -1);
    count_launch();
    snprintf(g_route, sizeof g_route, "norm+k1");
    return 1;
}

int vxb_linear_i8(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                  float out_scale, int32_t out_zero, int8_t* y, uint32_t ldy, int route) {
    int rc = check_common(ctx, w, x, y, ldy);
    if (rc != 1) return rc;
    if (!valid_scale(out_scale)) return fail(0, "output scale is not positive and finite");
    if (out_zero < -128 || out_zero > 127) return fail(0, "output zero point %d outside int8", out_zero);
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    EpilogueParams epi{};
    epi.mode = kEpiI8; epi.row_scales = (const float*)ctx->row_scales.ptr; epi.ws = w->ws;
    epi.bias_i32 = w->bias_i32; set_requant_divisor(epi, w, out_scale); epi.out_zero = out_zero;
    epi.out_lo = -128; epi.out_hi = 127; epi.out = y; epi.ld = ldy;
    return quantize_then_gemm(ctx, w, x, rows, epi, route, "k1+");
}

int vxb_linear_acc_i32(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                       int32_t* acc, int8_t* q_out, float* scales_out, int route) {
    int rc = check_common(ctx, w, x, acc, w ? w->d_out : 0);
    if (rc != 1) return rc;
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    if ((rc = quantize_into_scratch(ctx, w, x, rows)) != 1) return rc;
    if (q_out)
        CUDA_TRY(cudaMemcpy2DAsync(q_out, w->d_in, ctx->q.ptr, w->kpad, w->d_in, rows,
                                   cudaMemcpyDeviceToDevice, ctx->stream), -1);
    if (scales_out)
        CUDA_TRY(cudaMemcpyAsync(scales_out, ctx->row_scales.ptr, (size_t)rows * 4,
                                 cudaMemcpyDeviceToDevice, ctx->stream), -1);
    EpilogueParams epi{};
    epi.mode = kEpiAcc; epi.out = acc; epi.ld = w->d_out;
    if (route == VXB_ROUTE_DECODE_FUSED) {
        // q_out / scales_out came from the stand-alone quantizer above; the accumulators from the kernel's own quantization
        const VxbPlanQuery query = plan_query(ctx, w, rows, epi, route, true);
        VxbLaunchPlan plan;
        char why[160];
        if (vxb_plan(&query, &plan, why, sizeof why) != 1) return fail(0, "%s", why);
        return launch_decode_fused(ctx, w, x, rows, epi);
    }
    return run_gemm(ctx, w, (const int8_t*)ctx->q.ptr, rows, epi, route, "k1+");
}

int vxb_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
    if (!bytes || !ptr || !handle) return fail(0, "bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    CUDA_TRY(cudaMalloc(&p, bytes), 0);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) { cudaFree(p); return fail(0, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e)); }
    memcpy(handle, &h, 64);
    *ptr = p;
    return 1;
}

int vxb_peer_open(const unsigned char handle[64], void** ptr) {
    if (!handle || !ptr) return fail(0, "bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), 0);
    return 1;
}

int vxb_peer_close(void* ptr) {
    if (!ptr) return 1;
    CUDA_TRY(cudaIpcCloseMemHandle(ptr), -1);
    return 1;
}

int vxb_peer_free(void* ptr) {
    if (!ptr) return 1;
    CUDA_TRY(cudaFree(ptr), -1);
    return 1;
}

int vxb_linear_i8_gather(VxbContext* ctx, const VxbWeight* w, const float* x, uint32_t rows,
                         float out_scale, int32_t out_zero, int8_t* y, uint32_t ldy,
                         void* const* peer_y, uint32_t n_peers) {
    int rc = check_common(ctx, w, x, y, ldy);
    if (rc != 1) return rc;
    if (n_peers > 7 || (n_peers && !peer_y)) return fail(0, "at most 7 peers");
    for (uint32_t p = 0; p < n_peers; p++)
        if (!peer_y[p]) return fail(0, "null peer pointer");
    if (!valid_scale(out_scale)) return fail(0, "output scale is not positive and finite");
    if (out_zero < -128 || out_zero > 127) return fail(0, "output zero point %d outside int8", out_zero);
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    EpilogueParams epi{};
    epi.mode = kEpiI8; epi.row_scales = (const float*)ctx->row_scales.ptr; epi.ws = w->ws;
    epi.bias_i32 = w->bias_i32; set_requant_divisor(epi, w, out_scale); epi.out_zero = out_zero;
    epi.out_lo = -128; epi.out_hi = 127; epi.out = y; epi.ld = ldy;
    epi.n_peers = n_peers;
    for (uint32_t p = 0; p < n_peers; p++) epi.peer_out[p] = peer_y[p];
    // with peers the plan picks between the two GEMM kernels that carry the peer stores
    return quantize_then_gemm(ctx, w, x, rows, epi, n_peers ? VXB_ROUTE_AUTO : VXB_ROUTE_TCGEN05, "k1+");
}

int vxb_peer_barrier(VxbContext* ctx, uint32_t* my_flags, void* const* peer_flags, const uint32_t* peer_ranks,
                     uint32_t n_peers, uint32_t my_rank, uint32_t epoch) {
    if (!ctx || !my_flags || (n_peers && (!peer_flags || !peer_ranks))) return fail(0, "null argument");
    if (n_peers > 7 || my_rank > 7) return fail(0, "at most 8 ranks");
    if (!n_peers) return 1;
    PeerBarrierArgs a{};
    for (uint32_t p = 0; p < n_peers; p++) {
        if (!peer_flags[p] || peer_ranks[p] > 7 || peer_ranks[p] == my_rank) return fail(0, "bad peer %u", p);
        a.peer_flags[p] = (uint32_t*)peer_flags[p]; a.peer_ranks[p] = peer_ranks[p];
    }
    a.n_peers = n_peers; a.my_rank = my_rank; a.epoch = epoch;
    if (ensure_device(ctx) != 1) return -1;
    LAUNCH_TRY(launch_peer_barrier(my_flags, a, ctx->status, ctx->stream));
    count_launch();
    return 1;
}

namespace {
bool byte_dtype(uint32_t dt) { return dt == VXB_DTYPE_I8 || dt == VXB_DTYPE_U8; }
bool zero_in_range(int32_t z, uint32_t dt) { return dt == VXB_DTYPE_I8 ? (z >= -128 && z <= 127) : (z >= 0 && z <= 255); }
}

int vxb_quantize_linear_device(VxbContext* ctx, const float* x, uint64_t elements, float scale, int32_t zero_point,
                               uint32_t output_dtype, void* out) {
    if (!ctx || !x || !out) return fail(0, "null argument");
    if (!byte_dtype(output_dtype)) return fail(0, "output dtype %u is not I8/U8", output_dtype);
    if (!valid_scale(scale)) return fail(0, "scale is not positive and finite");
    if (!zero_in_range(zero_point, output_dtype)) return fail(0, "zero point %d outside the output dtype", zero_point);
    if (!elements) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(launch_quantize_linear(x, elements, scale, zero_point, output_dtype == VXB_DTYPE_U8, out, ctx->stream), -1);
    count_launch();
    return 1;
}

int vxb_dequantize_linear_device(VxbContext* ctx, const void* x, uint64_t elements, float scale, int32_t zero_point,
                                 uint32_t input_dtype, float* out) {
    if (!ctx || !x || !out) return fail(0, "null argument");
    if (!byte_dtype(input_dtype)) return fail(0, "input dtype %u is not I8/U8", input_dtype);
    if (!valid_scale(scale)) return fail(0, "scale is not positive and finite");
    if (!zero_in_range(zero_point, input_dtype)) return fail(0, "zero point %d outside the input dtype", zero_point);
    if (!elements) return 1;
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(launch_dequantize_linear(x, elements, scale, zero_point, input_dtype == VXB_DTYPE_U8, out, ctx->stream), -1);
    count_launch();
    return 1;
}

int vxb_requantize_linear_device(VxbContext* ctx, const void* x, uint64_t elements, float input_scale,
                                 int32_t input_zero_point, float output_scale, int32_t output_zero_point,
                                 uint32_t input_dtype, uint32_t output_dtype, void* out) {
    if (!ctx || !x || !out) return fail(0, "null argument");
    if (!elements) return fail(0, "empty tensor");
    if (!byte_dtype(input_dtype) || !byte_dtype(output_dtype)) return fail(0, "dtypes must be I8/U8");
    if (!valid_scale(input_scale) || !valid_scale(output_scale)) return fail(0, "scales must be positive and finite");
    if (!zero_in_range(input_zero_point, input_dtype) || !zero_in_range(output_zero_point, output_dtype))
        return fail(0, "zero point outside its dtype");
    const volatile float multiplier = input_scale / output_scale;   // one fp32 division, as the reference
    if (!valid_scale(multiplier)) return fail(0, "input_scale / output_scale is not positive and finite");
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(launch_requantize_linear(x, elements, multiplier, input_zero_point, input_dtype == VXB_DTYPE_U8,
                                      output_zero_point, output_dtype == VXB_DTYPE_U8, out, ctx->stream), -1);
    count_launch();
    return 1;
}

uint32_t vxb_weight_row_bytes(const VxbWeight* w) { return w ? w->kpad : 0; }

int vxb_linear_prepared(VxbContext* ctx, const VxbWeight* w, const int8_t* q, const float* row_scales,
                        uint32_t rows, int mode, float out_scale, int32_t out_zero, void* out,
                        uint32_t ldy, int route) {
    int rc = check_common(ctx, w, q, out, ldy);
    if (rc != 1) return rc;
    if (mode < 0 || mode > 2) return fail(0, "mode must be 0, 1 or 2");
    if (mode != 0 && !row_scales) return fail(0, "row scales are required for modes 1 and 2");
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    EpilogueParams epi{};
    epi.mode = mode; epi.row_scales = row_scales; epi.ws = w->ws; epi.out = out; epi.ld = ldy;
    if (mode == kEpiF32) epi.bias_f32 = w->bias_f32;
    if (mode == kEpiI8) {
        if (!valid_scale(out_scale)) return fail(0, "output scale is not positive and finite");
        if (out_zero < -128 || out_zero > 127) return fail(0, "output zero point %d outside int8", out_zero);
        epi.bias_i32 = w->bias_i32; set_requant_divisor(epi, w, out_scale); epi.out_zero = out_zero;
        epi.out_lo = -128; epi.out_hi = 127;
    }
    return run_gemm(ctx, w, q, rows, epi, route, "prepared+");
}

int vxb_qlinear_device(VxbContext* ctx, const VxbWeight* w, const void* input, uint32_t rows,
                       float input_scale, int32_t input_zero_point, float output_scale,
                       int32_t output_zero_point, uint32_t input_dtype, uint32_t output_dtype,
                       void* output, uint32_t ldy, int route) {
    int rc = check_common(ctx, w, input, output, ldy);
    if (rc != 1) return rc;
    const bool in_u8 = input_dtype == VXB_DTYPE_U8, out_u8 = output_dtype == VXB_DTYPE_U8;
    if ((!in_u8 && input_dtype != VXB_DTYPE_I8) || (!out_u8 && output_dtype != VXB_DTYPE_I8))
        return fail(0, "activation dtypes must be I8 or U8");
    if (!valid_scale(input_scale) || !valid_scale(output_scale)) return fail(0, "scales must be positive and finite");
    if (input_zero_point < (in_u8 ? 0 : -128) || input_zero_point > (in_u8 ? 255 : 127) ||
        output_zero_point < (out_u8 ? 0 : -128) || output_zero_point > (out_u8 ? 255 : 127))
        return fail(0, "zero point outside its dtype");
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    // activations into the padded signed layout (U8 -> subtract 128 from codes and zero point)
    CUDA_TRY(ctx->q.reserve((size_t)rows * w->kpad), 0);
    CUDA_TRY(ctx->row_scales.reserve((size_t)rows * 4), 0);
    CUDA_TRY(ctx->bias_eff.reserve((size_t)w->d_out * 4), 0);
    CUDA_TRY(launch_copy_bytes_padded((const uint8_t*)input, rows, w->d_in, (uint8_t*)ctx->q.ptr, w->kpad,
                                      in_u8 ? 0x80u : 0u, ctx->stream), -1);
    CUDA_TRY(launch_fill_f32((float*)ctx->row_scales.ptr, rows, input_scale, ctx->stream), -1);
    const int32_t signed_zero = in_u8 ? input_zero_point - 128 : input_zero_point;
    CUDA_TRY(launch_fold_zero_point(w->bias_i32, w->wsum, signed_zero, (int32_t*)ctx->bias_eff.ptr,
                                    w->d_out, ctx->stream), -1);
    count_launch(3);
    EpilogueParams epi{};
    epi.mode = kEpiI8; epi.row_scales = (const float*)ctx->row_scales.ptr; epi.ws = w->ws;
    epi.bias_i32 = (const int32_t*)ctx->bias_eff.ptr; set_requant_divisor(epi, w, output_scale);
    epi.out_zero = output_zero_point; epi.out_lo = out_u8 ? 0 : -128; epi.out_hi = out_u8 ? 255 : 127;
    epi.out = output; epi.ld = ldy;
    return run_gemm(ctx, w, (const int8_t*)ctx->q.ptr, rows, epi, route, "static+");
}

int vxb_context_trace(VxbContext* ctx, unsigned long long* device_stamps) {
    if (!ctx) return fail(0, "null context");
    ctx->trace = device_stamps;
    return 1;
}

int vxb_context_set_wait_limit(VxbContext* ctx, uint64_t cycles) {
    if (!ctx) return fail(0, "null context");
    if (ensure_device(ctx) != 1) return -1;
    uint64_t units = (cycles + 1023u) >> 10;
    if (units > 0x7fffffffull) units = 0x7fffffffull;
    const int value = (int)units;   // 0 = the default limit
    CUDA_TRY(cudaMemcpyAsync(ctx->status + 1, &value, sizeof(int), cudaMemcpyHostToDevice, ctx->stream), -1);
    CUDA_TRY(cudaStreamSynchronize(ctx->stream), -1);
    return 1;
}

int vxb_selftest_wait_expiry(VxbContext* ctx) {
    if (!ctx) return fail(0, "null context");
    if (ensure_device(ctx) != 1) return -1;
    LAUNCH_TRY(launch_wait_expiry(ctx->status, ctx->stream));
    count_launch();
    return 1;
}

int vxb_selftest_div_const(VxbContext* ctx, int divisor_exponent, uint32_t neighbours, uint32_t samples,
                           uint64_t* mismatches, uint64_t* checked) {
    if (!ctx || !mismatches || !checked) return fail(0, "null argument");
    if (divisor_exponent < -100 || divisor_exponent > 100 || neighbours > 16) return fail(0, "argument out of range");
    if (ensure_device(ctx) != 1) return -1;
    unsigned long long* counts = nullptr;
    CUDA_TRY(cudaMalloc(&counts, 2 * sizeof(unsigned long long)), 0);
    cudaError_t err = cudaMemsetAsync(counts, 0, 2 * sizeof(unsigned long long), ctx->stream);
    if (err == cudaSuccess)
        err = launch_div_const_check(divisor_exponent, neighbours, samples, counts, counts + 1, ctx->sm_count, ctx->stream);
    unsigned long long host[2] = {0, 0};
    if (err == cudaSuccess) err = cudaMemcpyAsync(host, counts, sizeof host, cudaMemcpyDeviceToHost, ctx->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
    cudaFree(counts);
    count_launch();
    if (err != cudaSuccess) return fail(-1, "division self-test failed: %s", cudaGetErrorString(err));
    *mismatches = host[0]; *checked = host[1];
    return 1;
}

void vxb_inject_failure(int kind, uint32_t countdown) {
    if (kind == VXB_INJECT_LAUNCH) g_fail_launch.store(countdown);
    else if (kind == VXB_INJECT_ALLOCATION) g_fail_alloc.store(countdown);
}

int vxb_tune(const char* name, int64_t value) {
    if (!name) return 0;
    Tunables& t = tunables();
    if (!strcmp(name, "decode.pair_share_bytes")) { t.decode_pair_share_bytes = (uint32_t)value; return 1; }
    if (!strcmp(name, "decode.l2_prefetch")) { t.decode_l2_prefetch = value != 0; return 1; }
    if (!strcmp(name, "decode.fused_max_rows")) { t.decode_fused_max_rows = (uint32_t)value; return 1; }
    if (!strcmp(name, "gemm.overlap_k1")) { t.overlap_k1 = value != 0; return 1; }
    if (!strcmp(name, "gemm.overlap_gather")) { t.overlap_gather = value != 0; return 1; }
    if (!strcmp(name, "gemm.gather_tma")) { t.gather_tma = value != 0; return 1; }
    if (!strcmp(name, "gemm.overlap_ratio")) { t.overlap_ratio = (uint32_t)value; return 1; }
    return 0;
}

int vxb_context_profile(VxbContext* ctx, int enable) {
    if (!ctx) return fail(0, "null context");
    if (ensure_device(ctx) != 1) return -1;
    for (auto& v : ctx->prof_events) { for (cudaEvent_t e : v) cudaEventDestroy(e); v.clear(); }
    ctx->profiling = enable > 0 ? enable : 0;
    ctx->prof_seen[0] = ctx->prof_seen[1] = 0;
    return 1;
}

int vxb_context_profile_read(VxbContext* ctx, double* quantize_ms, uint64_t* quantize_launches,
                             double* gemm_ms, uint64_t* gemm_launches) {
    if (!ctx) return fail(0, "null context");
    if (ensure_device(ctx) != 1) return -1;
    CUDA_TRY(cudaStreamSynchronize(ctx->stream), -1);
    double ms[2] = {0.0, 0.0}; uint64_t n[2] = {0, 0};
    for (int k = 0; k < 2; k++) {
        auto& v = ctx->prof_events[k];
        for (size_t i = 0; i + 1 < v.size(); i += 2) {
            float t = 0.0f;
            if (cudaEventElapsedTime(&t, v[i], v[i + 1]) == cudaSuccess) { ms[k] += t; n[k]++; }
        }
    }
    if (quantize_ms) *quantize_ms = ms[0];
    if (quantize_launches) *quantize_launches = n[0];
    if (gemm_ms) *gemm_ms = ms[1];
    if (gemm_launches) *gemm_launches = n[1];
    return 1;
}

int vxb_linear_host(VxbContext* ctx, const VxbWeight* w, const float* x_host, uint32_t rows,
                    int requant, float out_scale, int32_t out_zero, void* y_host) {
    if (!ctx || !w || !x_host || !y_host) return fail(0, "null argument");
    if (!rows) return 1;
    if (ensure_device(ctx) != 1) return -1;
    const size_t in_row = (size_t)w->d_in * 4, out_row = (size_t)w->d_out * (requant ? 1 : 4);
    // Large batches go through in row chunks on three streams, so that the upload of chunk c+1,
    // the kernels of chunk c and the download of chunk c-1 overlap (PCIe is full duplex and is
    // what bounds this entry). Two staging buffers each way.  The chunks ramp up from 256 rows and
    // down again to 256: nothing can be downloaded before the first chunk is up and computed, and
    // nothing overlaps the download of the last one, so both are kept short, while the chunks in the
    // middle (about a sixth of the batch each) keep the number of copies small.
    std::vector<uint32_t> sizes;
    if (rows < 1024) sizes.push_back(rows);
    else {
        uint32_t big = ((rows / 6) + 127) / 128 * 128;
        if (big < 256) big = 256;
        std::vector<uint32_t> ramp;
        uint32_t ramp_rows = 0;
        for (uint32_t sz = 256; sz < big && 2 * (ramp_rows + sz) <= rows / 2; sz *= 2) { ramp.push_back(sz); ramp_rows += sz; }
        const uint32_t middle = rows - 2 * ramp_rows, count = (middle + big - 1) / big;
        const uint32_t each = ((middle + count - 1) / count + 127) / 128 * 128;
        sizes = ramp;
        for (uint32_t left = middle; left;) { const uint32_t take = left < each ? left : each; sizes.push_back(take); left -= take; }
        for (size_t i = ramp.size(); i-- > 0;) sizes.push_back(ramp[i]);
    }
    uint32_t chunk = 0;   // the largest chunk sizes the staging buffers
    for (uint32_t sz : sizes) chunk = sz > chunk ? sz : chunk;
    const uint32_t chunks = (uint32_t)sizes.size();
    CUDA_TRY(ctx->stage_in.reserve(2 * (size_t)chunk * in_row), 0);
    CUDA_TRY(ctx->stage_out.reserve(2 * (size_t)chunk * out_row), 0);
    if (!ctx->copy_in) {
        CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking), 0);
        CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking), 0);
        for (int b = 0; b < 2; b++) {
            CUDA_TRY(cudaEventCreateWithFlags(&ctx->ev_in[b], cudaEventDisableTiming), 0);
            CUDA_TRY(cudaEventCreateWithFlags(&ctx->ev_done[b], cudaEventDisableTiming), 0);
            CUDA_TRY(cudaEventCreateWithFlags(&ctx->ev_out[b], cudaEventDisableTiming), 0);
        }
        CUDA_TRY(cudaEventCreateWithFlags(&ctx->ev_start, cudaEventDisableTiming), 0);
    }
    // the copy streams start after whatever is already queued on the context's stream
    CUDA_TRY(cudaEventRecord(ctx->ev_start, ctx->stream), -1);
    CUDA_TRY(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_start, 0), -1);
    CUDA_TRY(cudaStreamWaitEvent(ctx->copy_out, ctx->ev_start, 0), -1);
    uint32_t r0 = 0;
    for (uint32_t c = 0; c < chunks; c++) {
        const int b = (int)(c & 1u);
        const uint32_t cnt = sizes[c];
        uint8_t* din = (uint8_t*)ctx->stage_in.ptr + (size_t)b * chunk * in_row;
        uint8_t* dout = (uint8_t*)ctx->stage_out.ptr + (size_t)b * chunk * out_row;
        // upload: the buffer is free once the kernels of chunk c-2 are done with it
        if (c >= 2) CUDA_TRY(cudaStreamWaitEvent(ctx->copy_in, ctx->ev_done[b], 0), -1);
        CUDA_TRY(cudaMemcpyAsync(din, (const uint8_t*)x_host + (size_t)r0 * in_row, (size_t)cnt * in_row,
                                 cudaMemcpyHostToDevice, ctx->copy_in), -1);
        CUDA_TRY(cudaEventRecord(ctx->ev_in[b], ctx->copy_in), -1);
        // kernels: need the upload, and the output buffer once chunk c-2 has been downloaded
        CUDA_TRY(cudaStreamWaitEvent(ctx->stream, ctx->ev_in[b], 0), -1);
        if (c >= 2) CUDA_TRY(cudaStreamWaitEvent(ctx->stream, ctx->ev_out[b], 0), -1);
        const int rc = requant
            ? vxb_linear_i8(ctx, w, (const float*)din, cnt, out_scale, out_zero, (int8_t*)dout, w->d_out, VXB_ROUTE_AUTO)
            : vxb_linear_f32(ctx, w, (const float*)din, cnt, (float*)dout, w->d_out, VXB_ROUTE_AUTO);
        if (rc != 1) { cudaDeviceSynchronize(); return rc == 0 && c == 0 ? 0 : -1; }
        CUDA_TRY(cudaEventRecord(ctx->ev_done[b], ctx->stream), -1);
        // download
        CUDA_TRY(cudaStreamWaitEvent(ctx->copy_out, ctx->ev_done[b], 0), -1);
        CUDA_TRY(cudaMemcpyAsync((uint8_t*)y_host + (size_t)r0 * out_row, dout, (size_t)cnt * out_row,
                                 cudaMemcpyDeviceToHost, ctx->copy_out), -1);
        CUDA_TRY(cudaEventRecord(ctx->ev_out[b], ctx->copy_out), -1);
        r0 += cnt;
    }
    // the context's stream joins the last download(s), then the caller waits on it
    for (int b = 0; b < 2; b++)
        if (chunks > (uint32_t)b) CUDA_TRY(cudaStreamWaitEvent(ctx->stream, ctx->ev_out[b], 0), -1);
    return vxb_context_synchronize(ctx) == 1 ? 1 : -1;
}

int vxb_measure_mma_issue(VxbContext* ctx, uint32_t m, uint32_t n, uint32_t accs, uint32_t per_commit,
                          uint32_t iters, double* cycles_per_mma) {
    if (!ctx || !cycles_per_mma || !iters || !per_commit || !accs) return fail(0, "bad argument");
    if (ensure_device(ctx) != 1) return -1;
    if (!ctx->tcgen05_ready) { CUDA_TRY(gemm_tcgen05_prepare(), 0); ctx->tcgen05_ready = true; }
    long long* cycles = nullptr;
    CUDA_TRY(cudaMalloc(&cycles, sizeof(long long)), 0);
    cudaError_t err = launch_mma_probe(m, n, accs, per_commit, iters, cycles, ctx->status, ctx->stream);
    long long host = 0;
    if (err == cudaSuccess) err = cudaMemcpyAsync(&host, cycles, sizeof host, cudaMemcpyDeviceToHost, ctx->stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
    cudaFree(cycles);
    count_launch();
    if (err != cudaSuccess) return fail(-1, "mma probe failed: %s", cudaGetErrorString(err));
    *cycles_per_mma = (double)host / ((double)iters * per_commit);
    return vxb_context_synchronize(ctx) == 1 ? 1 : -1;
}

int vxb_measure_i8_tensor_peak(VxbContext* ctx, uint32_t iters, double* tops) {
    if (!ctx || !tops || !iters) return fail(0, "bad argument");
    if (ensure_device(ctx) != 1) return -1;
    if (!ctx->tcgen05_ready) { CUDA_TRY(gemm_tcgen05_prepare(), 0); ctx->tcgen05_ready = true; }
    long long* cycles = nullptr;
    CUDA_TRY(cudaMalloc(&cycles, sizeof(long long) * ctx->sm_count), 0);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaError_t err = launch_i8_peak_probe(4, cycles, ctx->status, ctx->sm_count, ctx->stream);  // warm-up
    cudaEventRecord(e0, ctx->stream);
    if (err == cudaSuccess) err = launch_i8_peak_probe(iters, cycles, ctx->status, ctx->sm_count, ctx->stream);
    cudaEventRecord(e1, ctx->stream);
    count_launch(2);
    if (err == cudaSuccess) err = cudaEventSynchronize(e1);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(cycles);
    if (err != cudaSuccess) return fail(-1, "peak probe failed: %s", cudaGetErrorString(err));
    const double ops = (double)ctx->sm_count * iters * 256.0 * 2.0 * 128.0 * 256.0 * 32.0;
    *tops = ops / (ms * 1e-3) / 1e12;
    return vxb_context_synchronize(ctx) == 1 ? 1 : -1;
}

}  // extern "C"

// ---- reference-facing host-pointer entries ------------------------------------------
namespace {

struct HostKey {
    const void* weight; const void* scales; const void* bias; uint32_t d_in, d_out, kind, group;
    bool operator==(const HostKey& o) const {
        return weight == o.weight && scales == o.scales && bias == o.bias && d_in == o.d_in &&
               d_out == o.d_out && kind == o.kind && group == o.group;
    }
};
struct HostKeyHash {
    size_t operator()(const HostKey& k) const {
        size_t h = (size_t)k.weight * 1315423911u;
        h ^= (size_t)k.scales + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= (size_t)k.bias + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        h ^= ((size_t)k.d_in << 32) ^ k.d_out ^ ((size_t)k.kind << 60) ^ ((size_t)k.group << 20);
        return h;
    }
};

std::mutex g_host_mutex;
VxbContext* g_host_ctx = nullptr;
std::unordered_map<HostKey, VxbWeight*, HostKeyHash> g_host_weights;

// One process-wide context on the device named by VOLVOXAI_CUDA_DEVICE (the
// reference's own selector), default 0. Calls are serialised by g_host_mutex,
// matching the reference's single-stream synchronous backend.
int host_context(VxbContext** out) {
    if (!g_host_ctx) {
        int device = 0;
        if (const char* env = getenv("VOLVOXAI_CUDA_DEVICE")) device = atoi(env);
        int rc = vxb_context_create(device, nullptr, &g_host_ctx);
        if (rc != 1) return rc;
    }
    *out = g_host_ctx;
    return 1;
}

bool overlap(const void* a, size_t an, const void* b, size_t bn) {
    if (!an || !bn) return false;
    const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
    return x < y + bn && y < x + an;
}

// ---- device residency of host tensors (vxb_host_residency) -----------------------------------------
// The reference's CUDA backend keeps a table from host pointers to device slots, uploads only inputs
// whose host copy is newer and leaves outputs device-dirty until something on the host needs them
// (graph_ensure_input_view / graph_mark_device, native/src/backends/cuda/host/
// cuda_graph_memory_host.inc:1302-1310).  The same here, behind the host-pointer entries: with
// residency on, an output stays in its device buffer (the host copy is stale until
// vxb_host_download), and an input that is such a device-dirty tensor - or a window of one: row
// windows are interior pointers - is consumed where it lies.  Inputs the library did not produce are
// uploaded on every call: the host may have rewritten them.
struct Resident { void* dev; size_t bytes; bool dirty; };
std::map<uintptr_t, Resident> g_resident;   // keyed by host address; ranges never overlap
bool g_residency = false;

std::map<uintptr_t, Resident>::iterator resident_containing(const void* host, size_t bytes) {
    auto it = g_resident.upper_bound((uintptr_t)host);
    if (it == g_resident.begin()) return g_resident.end();
    --it;
    return ((uintptr_t)host + bytes <= it->first + it->second.bytes) ? it : g_resident.end();
}

// Makes the host copies of every resident tensor overlapping [host, host+bytes) current and drops the entries.
int resident_evict(VxbContext* ctx, const void* host, size_t bytes) {
    for (auto it = g_resident.begin(); it != g_resident.end();) {
        if (overlap(host, bytes, (const void*)it->first, it->second.bytes)) {
            if (it->second.dirty)
                CUDA_TRY(cudaMemcpyAsync((void*)it->first, it->second.dev, it->second.bytes, cudaMemcpyDeviceToHost, ctx->stream), -1);
            CUDA_TRY(cudaStreamSynchronize(ctx->stream), -1);
            cudaFree(it->second.dev);
            it = g_resident.erase(it);
        } else ++it;
    }
    return 1;
}

// Device address of an input: a device-dirty resident tensor (or a window of one) in place, else an upload
// into `staging`.
int resident_input(VxbContext* ctx, const void* host, size_t bytes, Buffer& staging, const void** dev) {
    if (g_residency) {
        auto it = resident_containing(host, bytes);
        if (it != g_resident.end() && it->second.dirty) {
            *dev = (const uint8_t*)it->second.dev + ((uintptr_t)host - it->first);
            return 1;
        }
        // an input that only straddles device-dirty tensors: their host copies are made current first
        if (it == g_resident.end()) {
            const int rc = resident_evict(ctx, host, bytes);
            if (rc != 1) return rc;
        }
    }
    CUDA_TRY(staging.reserve(bytes), 0);
    CUDA_TRY(cudaMemcpyAsync(staging.ptr, host, bytes, cudaMemcpyHostToDevice, ctx->stream), -1);
    *dev = staging.ptr;
    return 1;
}

// Device address an output is computed into: with residency its own buffer (created on first use; any
// other resident range it overlaps is written back and dropped first), else `staging`.
int resident_output(VxbContext* ctx, void* host, size_t bytes, Buffer& staging, void** dev, bool* lazy) {
    *lazy = false;
    if (g_residency) {
        auto it = g_resident.find((uintptr_t)host);
        if (it == g_resident.end() || it->second.bytes != bytes) {
            const int rc = resident_evict(ctx, host, bytes);
            if (rc != 1) return rc;
            void* d = nullptr;
            if (injected(g_fail_alloc) || cudaMalloc(&d, bytes) != cudaSuccess) return fail(0, "device allocation of a resident output failed");
            it = g_resident.emplace((uintptr_t)host, Resident{d, bytes, false}).first;
        }
        *dev = it->second.dev;
        *lazy = true;
        return 1;
    }
    CUDA_TRY(staging.reserve(bytes), 0);
    *dev = staging.ptr;
    return 1;
}

// After the kernels: the output is device-dirty (residency) or copied to the host now; then the stream is drained.
int resident_finish(VxbContext* ctx, void* host, size_t bytes, const void* dev, bool lazy) {
    if (lazy) g_resident[(uintptr_t)host].dirty = true;
    else CUDA_TRY(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream), -1);
    return vxb_context_synchronize(ctx) == 1 ? 1 : -1;
}

}  // namespace

extern "C" {

int vxb_qlinear_i8u8(const void* input, const void* weight, const float* weight_scales,
                     const int32_t* weight_zero_points, const int32_t* bias, void* output,
                     uint32_t rows, uint32_t d_in, uint32_t d_out, float input_scale,
                     int32_t input_zero_point, float output_scale, int32_t output_zero_point,
                     uint32_t input_dtype, uint32_t weight_dtype, uint32_t output_dtype) {
    if (!input || !weight || !weight_scales || !weight_zero_points || !bias || !output)
        return fail(0, "null argument");
    if (!rows || !d_in || !d_out) return fail(0, "empty shape");
    if (weight_dtype != VXB_DTYPE_I8) return fail(0, "only I8 weights are admitted");
    for (uint32_t i = 0; i < d_out; i++)
        if (weight_zero_points[i] != 0) return fail(0, "non-zero weight zero point at channel %u", i);
    const size_t in_bytes = (size_t)rows * d_in, out_bytes = (size_t)rows * d_out;
    if (overlap(output, out_bytes, input, in_bytes) || overlap(output, out_bytes, weight, (size_t)d_out * d_in) ||
        overlap(output, out_bytes, bias, (size_t)d_out * 4) || overlap(output, out_bytes, weight_scales, (size_t)d_out * 4))
        return fail(0, "output overlaps an input");
    std::lock_guard<std::mutex> lock(g_host_mutex);
    VxbContext* ctx = nullptr;
    int rc = host_context(&ctx);
    if (rc != 1) return rc;
    const HostKey key{weight, weight_scales, bias, d_in, d_out, 1u, 0u};
    VxbWeight* w = nullptr;
    auto it = g_host_weights.find(key);
    if (it != g_host_weights.end()) w = it->second;
    else {
        rc = vxb_weight_create_i8(ctx, (const int8_t*)weight, weight_scales, nullptr, bias, d_out, d_in, &w);
        if (rc != 1) return rc;
        g_host_weights.emplace(key, w);
    }
    const void* din = nullptr; void* dout = nullptr; bool lazy = false;
    if ((rc = resident_output(ctx, output, out_bytes, ctx->stage_out, &dout, &lazy)) != 1) return rc;
    if ((rc = resident_input(ctx, input, in_bytes, ctx->stage_in, &din)) != 1) return rc;
    rc = vxb_qlinear_device(ctx, w, din, rows, input_scale, input_zero_point, output_scale,
                            output_zero_point, input_dtype, output_dtype, dout, d_out, VXB_ROUTE_AUTO);
    if (rc != 1) return rc;
    return resident_finish(ctx, output, out_bytes, dout, lazy);
}

extern "C++" {
namespace {
// host buffers through the context's staging buffers: upload, one device entry, download
template <typename Fn>
int host_elementwise(const void* input, size_t in_bytes, void* output, size_t out_bytes, Fn&& device_call) {
    if (!input || !output) return fail(0, "null argument");
    if (overlap(output, out_bytes, input, in_bytes)) return fail(0, "output overlaps the input");
    std::lock_guard<std::mutex> lock(g_host_mutex);
    VxbContext* ctx = nullptr;
    int rc = host_context(&ctx);
    if (rc != 1) return rc;
    const void* din = nullptr; void* dout = nullptr; bool lazy = false;
    if ((rc = resident_output(ctx, output, out_bytes, ctx->stage_out, &dout, &lazy)) != 1) return rc;
    if ((rc = resident_input(ctx, input, in_bytes, ctx->stage_in, &din)) != 1) return rc;
    rc = device_call(ctx, const_cast<void*>(din), dout);
    if (rc != 1) return rc;
    return resident_finish(ctx, output, out_bytes, dout, lazy);
}
}  // namespace
}  // extern "C++"

int vxb_quantize_typed_f32_i8u8(const float* input, uint32_t elements, void* output, float output_scale,
                                int32_t output_zero_point, uint32_t output_dtype) {
    if (!elements) return fail(0, "empty tensor");
    return host_elementwise(input, (size_t)elements * 4, output, elements, [&](VxbContext* ctx, void* in, void* out) {
        return vxb_quantize_linear_device(ctx, (const float*)in, elements, output_scale, output_zero_point, output_dtype, out);
    });
}

int vxb_dequantize_typed_i8u8_f32(const void* input, uint32_t elements, float input_scale, int32_t input_zero_point,
                                  uint32_t input_dtype, float* output) {
    if (!elements) return fail(0, "empty tensor");
    return host_elementwise(input, elements, output, (size_t)elements * 4, [&](VxbContext* ctx, void* in, void* out) {
        return vxb_dequantize_linear_device(ctx, in, elements, input_scale, input_zero_point, input_dtype, (float*)out);
    });
}

int vxb_requantize_linear_i8u8(const void* input, uint32_t input_elements, void* output, uint32_t output_elements,
                               float input_scale, int32_t input_zero_point, float output_scale,
                               int32_t output_zero_point, uint32_t input_dtype, uint32_t output_dtype) {
    if (!input_elements || input_elements != output_elements) return fail(0, "element counts differ or are zero");
    return host_elementwise(input, input_elements, output, output_elements, [&](VxbContext* ctx, void* in, void* out) {
        return vxb_requantize_linear_device(ctx, in, input_elements, input_scale, input_zero_point, output_scale,
                                            output_zero_point, input_dtype, output_dtype, out);
    });
}

int vxb_cuda_graph_llm_f32(const VxbLLMOpArgs* a) {
    if (!a) return fail(0, "null descriptor");
    if (a->kind != VXB_OP_PACKED_LINEAR) return fail(0, "operator %d is not PackedLinear", a->kind);
    if ((a->groups != 8 && a->groups != 4) || a->normalize != 8)
        return fail(0, "only weight bits 8 or 4 with activation bits 8 are admitted");
    if (a->key_dim <= 0 || a->value_dim <= 0 || a->batch <= 0 || a->sequence <= 0) return fail(0, "bad shape");
    if (!a->x[0] || !a->x[1] || !a->x[2] || !a->y[0]) return fail(0, "null tensor");
    const uint32_t k = (uint32_t)a->key_dim, n = (uint32_t)a->value_dim;
    const uint64_t rows64 = (uint64_t)a->batch * (uint64_t)a->sequence;
    if (rows64 > 0xffffffffull) return fail(0, "too many rows");
    // window: whole rows only (the generation path asks for exactly the last row)
    uint64_t first = a->first_unit, units = a->unit_count ? a->unit_count : rows64 * n;
    if (first > rows64 * n || units > rows64 * n - first) return fail(0, "window outside the output");
    if (first % n != 0 || units % n != 0) return fail(0, "ragged output windows are not admitted");
    if (a->first_unit != 0 && a->unit_count == 0) return fail(0, "first_unit without unit_count");
    const uint32_t row0 = (uint32_t)(first / n), rows = (uint32_t)(units / n);
    if (!rows) return 1;
    if (a->rate != 32 && a->rate != 64 && a->rate != 128 && a->rate != 256) return fail(0, "group size %d is not 32/64/128/256", a->rate);
    {
        // the output window must not overlap any source, as the reference's entry checks before it
        // maps anything (ranges_overlap in native/src/backends/cuda/host/cuda_graph_llm_host.inc:111-186)
        const uint32_t bits = (uint32_t)a->groups, groups = (k + (uint32_t)a->rate - 1) / (uint32_t)a->rate;
        const size_t out_b = (size_t)rows * n * 4;
        const float* out_p = a->y[0] + (size_t)row0 * n;
        if (overlap(out_p, out_b, a->x[0], (size_t)rows64 * k * 4) ||
            overlap(out_p, out_b, a->x[1], (size_t)n * ((k * bits + 31) / 32) * 4) ||
            overlap(out_p, out_b, a->x[2], (size_t)n * groups * 4) ||
            (a->x[3] && overlap(out_p, out_b, a->x[3], (size_t)n * 4)))
            return fail(0, "output overlaps an input");
    }

    std::lock_guard<std::mutex> lock(g_host_mutex);
    VxbContext* ctx = nullptr;
    int rc = host_context(&ctx);
    if (rc != 1) return rc;
    const HostKey key{a->x[1], a->x[2], a->x[3], k, n, a->groups == 4 ? 3u : 2u, (uint32_t)a->rate};
    VxbWeight* w = nullptr;
    auto it = g_host_weights.find(key);
    if (it != g_host_weights.end()) w = it->second;
    else {
        rc = a->groups == 4
            ? vxb_weight_create_w4_words(ctx, (const int32_t*)a->x[1], a->x[2], a->x[3], n, k, (uint32_t)a->rate, &w)
            : vxb_weight_create_w8_words(ctx, (const int32_t*)a->x[1], a->x[2], a->x[3], n, k, (uint32_t)a->rate, &w);
        if (rc != 1) return rc;
        g_host_weights.emplace(key, w);
    }
    const size_t in_bytes = (size_t)rows * k * 4, out_bytes = (size_t)rows * n * 4;
    const void* din = nullptr; void* dout = nullptr; bool lazy = false;
    float* y_host = a->y[0] + (size_t)row0 * n;
    if (rows != rows64) {
        // a partial window keeps the bytes outside it: computed through staging and written to the host at
        // once; a resident copy of the tensor is brought home first so that both stay one tensor
        if (g_residency && (rc = resident_evict(ctx, a->y[0], (size_t)rows64 * n * 4)) != 1) return rc;
        CUDA_TRY(ctx->stage_out.reserve(out_bytes), 0);
        dout = ctx->stage_out.ptr;
    } else if ((rc = resident_output(ctx, y_host, out_bytes, ctx->stage_out, &dout, &lazy)) != 1) return rc;
    if ((rc = resident_input(ctx, a->x[0] + (size_t)row0 * k, in_bytes, ctx->stage_in, &din)) != 1) return rc;
    rc = vxb_linear_f32(ctx, w, (const float*)din, rows, (float*)dout, n, VXB_ROUTE_AUTO);
    if (rc != 1) return rc == 0 ? 0 : -1;
    return resident_finish(ctx, y_host, out_bytes, dout, lazy);
}

int vxb_cuda_graph_packed_linear_decode_f32(const float* input, const int32_t* packed_weights,
                                            const float* weight_scales, const float* bias,
                                            float* output, uint32_t input_width,
                                            uint32_t output_width, uint32_t weight_bits,
                                            uint32_t activation_bits) {
    VxbLLMOpArgs a;
    memset(&a, 0, sizeof a);
    a.kind = VXB_OP_PACKED_LINEAR; a.batch = 1; a.sequence = 1;
    a.key_dim = (int32_t)input_width; a.value_dim = (int32_t)output_width;
    a.groups = (int32_t)weight_bits; a.normalize = (int32_t)activation_bits; a.rate = 128;
    a.x[0] = input; a.x[1] = (const float*)packed_weights; a.x[2] = weight_scales; a.x[3] = bias;
    a.y[0] = output;
    return vxb_cuda_graph_llm_f32(&a);
}

int vxb_host_residency(int enable) {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    if (!enable && g_residency && g_host_ctx) {
        // leaving the mode: every device-dirty tensor goes home first
        for (auto& kv : g_resident)
            if (kv.second.dirty) {
                CUDA_TRY(cudaMemcpyAsync((void*)kv.first, kv.second.dev, kv.second.bytes, cudaMemcpyDeviceToHost, g_host_ctx->stream), -1);
                kv.second.dirty = false;
            }
        CUDA_TRY(cudaStreamSynchronize(g_host_ctx->stream), -1);
    }
    g_residency = enable != 0;
    return 1;
}

int vxb_host_download(const void* host) {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    if (!g_host_ctx) return 1;
    bool found = host == nullptr;
    for (auto& kv : g_resident) {
        if (host && !overlap(host, 1, (const void*)kv.first, kv.second.bytes)) continue;
        found = true;
        if (!kv.second.dirty) continue;
        CUDA_TRY(cudaMemcpyAsync((void*)kv.first, kv.second.dev, kv.second.bytes, cudaMemcpyDeviceToHost, g_host_ctx->stream), -1);
        kv.second.dirty = false;
    }
    CUDA_TRY(cudaStreamSynchronize(g_host_ctx->stream), -1);
    return found ? 1 : fail(0, "no resident tensor at this host address");
}

int vxb_host_invalidate(const void* host) {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    for (auto it = g_resident.begin(); it != g_resident.end();) {
        if (!host || overlap(host, 1, (const void*)it->first, it->second.bytes)) { cudaFree(it->second.dev); it = g_resident.erase(it); }
        else ++it;
    }
    return 1;
}

void vxb_host_cache_clear(void) {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    for (auto& kv : g_host_weights) vxb_weight_destroy(kv.second);
    g_host_weights.clear();
    for (auto& kv : g_resident) cudaFree(kv.second.dev);   // device copies are dropped, not written back
    g_resident.clear();
    if (g_host_ctx) { vxb_context_destroy(g_host_ctx); g_host_ctx = nullptr; }
}

}  // extern "C"
