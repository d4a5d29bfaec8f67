// Variant table, launch planning and registry rows (declarations: include/vxb200_plan.h).
// Host code only; nothing here touches a device, so tests drive it on a CPU-only box.
// Counterpart of vx_cuda_packed_plan / vx_cuda_packed_select
// (native/src/backends/cuda/packed_launch_plan.h:33-125).
#include "../../include/vxb200_plan.h"
#include "../../include/vxb200_w8a8.h"
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>

using namespace vxb;

namespace {

const VxbVariant kVariants[] = {
#define VXB_VARIANT_ROW(id, route, label, symbol, bm, bn, bk, threads, cluster, smem, min_rows, max_rows, epi, weights, group, flags, prio) \
    {#id, route, label, symbol, bm, bn, bk, threads, cluster, smem, min_rows, max_rows, epi, weights, group, flags, prio},
    VXB_VARIANTS(VXB_VARIANT_ROW)
#undef VXB_VARIANT_ROW
};

int refuse(char* why, uint32_t bytes, const char* fmt, ...) {
    if (why && bytes) {
        va_list ap; va_start(ap, fmt);
        vsnprintf(why, bytes, fmt, ap);
        va_end(ap);
    }
    return 0;
}

uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

// Admission of one variant for one query (the fields of the table, nothing else).
bool admitted(const VxbVariant& v, const VxbPlanQuery& q, char* why, uint32_t bytes) {
    if (!(v.weight_mask & q.weight_kind)) { refuse(why, bytes, "%s does not serve this weight kind", v.id); return false; }
    if (!(v.epilogue_mask & q.epilogue)) { refuse(why, bytes, "%s does not produce this output", v.id); return false; }
    if (q.rows < v.min_rows || (v.max_rows && q.rows > v.max_rows)) {
        refuse(why, bytes, "%s serves %u..%u rows (got %u)", v.id, v.min_rows, v.max_rows, q.rows);
        return false;
    }
    if (v.group_size && v.group_size != q.group_size) { refuse(why, bytes, "%s needs group size %u", v.id, v.group_size); return false; }
    if (q.n_peers && !(v.flags & VXB_VF_PEERS)) { refuse(why, bytes, "%s has no peer stores", v.id); return false; }
    if (q.n_peers && v.cluster > 1 && (!q.out_store_aligned || q.epilogue != VXB_EPI_I8)) {
        refuse(why, bytes, "%s stores to peers as TMA tiles only: int8 output, 16-byte aligned buffers", v.id);
        return false;
    }
    if (q.fused_tail && !(v.flags & VXB_VF_FUSED_TAIL)) { refuse(why, bytes, "%s has no fused epilogue tail", v.id); return false; }
    if (v.flags & VXB_VF_TILE_STORE) {
        if (!q.out_store_aligned) { refuse(why, bytes, "%s needs a 16-byte aligned output base and row pitch", v.id); return false; }
        if (q.fused_tail & 2u) { refuse(why, bytes, "%s has no SiLU*Mul tail", v.id); return false; }
    }
    if (v.cluster > 1 && q.pair_clusters == 0) { refuse(why, bytes, "no co-resident CTA pairs on this device"); return false; }
    if (v.flags & VXB_VF_FUSED_K1) {
        if (!q.fp32_input) { refuse(why, bytes, "%s starts from fp32 rows", v.id); return false; }
        if ((q.k & 3u) || round_up(q.k, kKAlign) > 8192u || q.n > 256u * (q.sm_count ? q.sm_count : 148u)) {
            refuse(why, bytes, "%s needs d_in %% 4 == 0, a padded K of at most 8192 and one channel tile per CTA", v.id);
            return false;
        }
    }
    return true;
}

// Grid, threads and cluster of the chosen variant; false when the kernel has no launch shape.
bool geometry(VxbVariantId id, const VxbPlanQuery& q, VxbLaunchPlan* p) {
    const VxbVariant& v = kVariants[id];
    const uint32_t kpad = round_up(q.k, kKAlign), sms = q.sm_count ? q.sm_count : 148u;
    p->variant = id; p->route = v.route;
    p->tile_rows = v.tile_rows; p->tile_columns = v.tile_columns; p->tile_k = v.tile_k;
    p->threads = v.threads; p->cluster = v.cluster;
    switch (id) {
        case VXB_VARIANT_DECODE_ROWS: case VXB_VARIANT_DECODE_FUSED: {
            DecodeRowsArgs a{};
            a.rows = q.rows; a.n = q.n; a.kpad = kpad;
            if (id == VXB_VARIANT_DECODE_FUSED) { a.x_f32 = reinterpret_cast<const float*>(uintptr_t(16)); a.k = q.k; }
            decode_rows_plan(q.n, (int)sms, &a.tile_rows, &a.tiles_per_cta);
            a.w_stage_bytes = round_up(a.tile_rows * kKAlign, 1024u);
            if (!decode_rows_configure(a)) return false;
            p->tile_rows = decode_rows_token_slots(q.rows);
            p->tile_columns = a.tile_rows;
            p->grid = ceil_div(q.n, a.tiles_per_cta * a.tile_rows);
            p->threads = decode_rows_threads(a.pair != 0);
            return true;
        }
        case VXB_VARIANT_DECODE_STREAMK: {
            const uint64_t units = (uint64_t)ceil_div(q.n, 128) * (kpad / 128);
            p->tile_rows = decode_token_slots(q.rows);
            p->grid = units < sms ? (uint32_t)units : sms;
            p->workspace_bytes += (uint64_t)128 * q.n * 4 + (uint64_t)ceil_div(q.n, 128) * 4;
            return true;
        }
        case VXB_VARIANT_GEMV_DP4A: case VXB_VARIANT_GEMV_GROUPED: case VXB_VARIANT_GEMV_W4_GROUPED: {
            const GemvShape s = gemv_shape(id == VXB_VARIANT_GEMV_DP4A ? 0 : id == VXB_VARIANT_GEMV_GROUPED ? 1 : 2,
                                           q.rows, q.n, kpad, (int)sms);
            p->tile_rows = s.mr; p->tile_columns = 8 * s.ch; p->tile_k = s.kchunk; p->grid = s.grid;
            return true;
        }
        case VXB_VARIANT_SIMT_DP4A:
            p->grid = ceil_div(q.n, 128) * q.rows; p->tile_rows = 1;
            return true;
        case VXB_VARIANT_DP4A_GROUPED:
            p->grid = ceil_div(q.n, 128) * (q.rows == 1 ? 1 : ceil_div(q.rows, 4));
            return true;
        case VXB_VARIANT_TCGEN05: case VXB_VARIANT_TCGEN05_WIDE: case VXB_VARIANT_GROUPED_TCGEN05: {
            const uint32_t tiles = ceil_div(q.rows, v.tile_rows) * ceil_div(q.n, v.tile_columns);
            p->grid = tiles < sms ? tiles : sms;
            return true;
        }
        case VXB_VARIANT_TCGEN05_PAIR: {
            const uint32_t tiles = ceil_div(q.rows, v.tile_rows) * ceil_div(q.n, v.tile_columns);
            p->grid = 2 * (tiles < q.pair_clusters ? tiles : q.pair_clusters);
            return true;
        }
        default: return false;
    }
}

// The per-row quantizer in front of the GEMM when the call starts from fp32 activations
// (the selection rule of launch_quantize_rows, for aligned buffers).
void plan_quantizer(const VxbPlanQuery& q, VxbLaunchPlan* p) {
    const uint32_t kpad = round_up(q.k, kKAlign);
    p->workspace_bytes += (uint64_t)q.rows * kpad + (uint64_t)q.rows * 4;
    p->launches += 1;
    if (q.k % 4 != 0) {
        p->quantizer = VXB_QUANTIZER_SCALAR; p->quantizer_grid = ceil_div(q.rows, 8); p->quantizer_cluster = 1;
        return;
    }
    const uint32_t words = kpad / 4;
    if (q.rows <= 32 && words >= 512 && words <= 8u * 256u * 8u) {
        const uint32_t per = ceil_div(words, 256);
        p->quantizer = VXB_QUANTIZER_CLUSTER;
        p->quantizer_cluster = per >= 8 ? 8 : per >= 4 ? 4 : 2;
        p->quantizer_grid = p->quantizer_cluster * q.rows;
        return;
    }
    const uint32_t tpr = q.k <= 256 ? 8 : q.k <= 1024 ? 32 : q.k <= 2048 ? 64 : q.k <= 4096 ? 128 : 256;
    p->quantizer = VXB_QUANTIZER_VEC; p->quantizer_cluster = 1;
    p->quantizer_grid = ceil_div(q.rows, 256 / tpr);
}

}  // namespace

extern "C" {

uint32_t vxb_variant_count(void) { return VXB_VARIANT_COUNT; }

const VxbVariant* vxb_variant_info(uint32_t index) { return index < VXB_VARIANT_COUNT ? &kVariants[index] : nullptr; }

int vxb_plan(const VxbPlanQuery* query, VxbLaunchPlan* out, char* why, uint32_t why_bytes) {
    if (why && why_bytes) why[0] = 0;
    if (!query || !out) return refuse(why, why_bytes, "null argument");
    const VxbPlanQuery& q = *query;
    if (!q.rows || !q.k || !q.n) return refuse(why, why_bytes, "empty shape");
    if (q.weight_kind != VXB_WEIGHT_PER_CHANNEL && q.weight_kind != VXB_WEIGHT_GROUPED && q.weight_kind != VXB_WEIGHT_W4_WORDS)
        return refuse(why, why_bytes, "weight kind must be one VXB_WEIGHT_* bit");
    if (q.epilogue != VXB_EPI_ACC && q.epilogue != VXB_EPI_F32 && q.epilogue != VXB_EPI_I8)
        return refuse(why, why_bytes, "epilogue must be one VXB_EPI_* bit");
    const bool grouped = q.weight_kind != VXB_WEIGHT_PER_CHANNEL;
    if (grouped && q.group_size != 32 && q.group_size != 64 && q.group_size != 128 && q.group_size != 256)
        return refuse(why, why_bytes, "group size %u is not 32/64/128/256", q.group_size);
    if ((uint64_t)q.k * 127u * 128u > 2147483647ull) return refuse(why, why_bytes, "d_in %u can overflow the int32 accumulator", q.k);
    if (q.n_peers > 7) return refuse(why, why_bytes, "at most 7 peers");
    const uint32_t sms = q.sm_count ? q.sm_count : 148u;

    memset(out, 0, sizeof *out);
    out->launches = 1;
    int chosen = -1;
    if (q.requested_route != VXB_ROUTE_AUTO) {
        // an explicit route is honoured or refused, never replaced by another kernel
        if (grouped && q.requested_route != VXB_ROUTE_SIMT)
            return refuse(why, why_bytes, "weights with grouped scales take the automatic route only");
        for (int i = 0; i < VXB_VARIANT_COUNT; i++)
            if (kVariants[i].route == q.requested_route && (kVariants[i].weight_mask & q.weight_kind)) { chosen = i; break; }
        if (chosen < 0) return refuse(why, why_bytes, "no kernel variant has route %d", q.requested_route);
        if (!admitted(kVariants[chosen], q, why, why_bytes)) return 0;
    } else if (grouped) {
        if (q.epilogue != VXB_EPI_F32) return refuse(why, why_bytes, "weights with grouped scales produce fp32 output only");
        if (q.fused_tail) return refuse(why, why_bytes, "weights with grouped scales have no fused epilogue");
        // decode: a warp per channel streams the weights once (over the 4-bit words when they were kept);
        // from three rows on the tensor-core kernel is faster at large weights
        const uint64_t weight_bytes = (uint64_t)round_up(q.k, kKAlign) * q.n;
        if (q.rows <= 2 && q.weight_kind == VXB_WEIGHT_W4_WORDS) chosen = VXB_VARIANT_GEMV_W4_GROUPED;
        else if (q.rows <= 2 || (q.rows <= 4 && weight_bytes <= (32ull << 20))) chosen = VXB_VARIANT_GEMV_GROUPED;
        else chosen = VXB_VARIANT_GROUPED_TCGEN05;
        if (!admitted(kVariants[chosen], q, why, why_bytes)) return 0;
    } else {
        if (q.n_peers) {
            // fused all-gather: the single-CTA kernel with its 128-byte store tiles, unless the launch is clearly
            // MMA-bound (padded K of at least 3424 per peer, 1.6 times the break-even of gather_is_link_bound):
            // then the pairs of CTAs, whose 64-byte store tiles use the links less well, when their tile stores
            // are possible.  Measured: 2 GPUs, K 4096: 174 us paired against 190; 4 GPUs, K 8192 (1.28 times
            // the break-even): 569 us paired against 508.
            const uint32_t tiles = ceil_div(q.rows, 128) * ceil_div(q.n, 256);
            char unused[8];
            chosen = VXB_VARIANT_TCGEN05;
            if (q.rows > 128 && tiles >= 2u * sms && (uint64_t)q.n_peers * 3424u <= round_up(q.k, kKAlign) &&
                admitted(kVariants[VXB_VARIANT_TCGEN05_PAIR], q, unused, sizeof unused)) chosen = VXB_VARIANT_TCGEN05_PAIR;
        }
        else if (q.rows <= 128) {
            chosen = VXB_VARIANT_DECODE_ROWS;
            char unused[8];
            // one or two fp32 rows: the single-launch form.  From three rows on every CTA repeating the
            // quantization costs more than the separate cluster quantizer (17.1 against 15.5 us per
            // step at 8 rows, K 4096, N 14336), so the two-launch form stays.
            if (q.fp32_input && q.rows <= tunables().decode_fused_max_rows &&
                admitted(kVariants[VXB_VARIANT_DECODE_FUSED], q, unused, sizeof unused)) chosen = VXB_VARIANT_DECODE_FUSED;
        }
        else {
            // pairs of CTAs on 256 x 256 tiles once there are at least two waves of 128 x 256 tiles
            const uint32_t tiles = ceil_div(q.rows, 128) * ceil_div(q.n, 256);
            chosen = (q.pair_clusters > 0 && tiles >= 2u * sms) ? VXB_VARIANT_TCGEN05_PAIR : VXB_VARIANT_TCGEN05;
            // 32-bit outputs at short K are bound by the output, not by the tensor pipe
            char unused[8];
            if (q.epilogue != VXB_EPI_I8 && round_up(q.k, kKAlign) <= VXB_WIDE_MAX_KPAD &&
                admitted(kVariants[VXB_VARIANT_TCGEN05_WIDE], q, unused, sizeof unused)) chosen = VXB_VARIANT_TCGEN05_WIDE;
        }
        if (!admitted(kVariants[chosen], q, why, why_bytes)) return 0;
    }
    if (!geometry((VxbVariantId)chosen, q, out))
        return refuse(why, why_bytes, "no launch shape for %s (rows %u, d_out %u)", kVariants[chosen].id, q.rows, q.n);
    if (q.fp32_input && !(kVariants[chosen].flags & VXB_VF_FUSED_K1)) plan_quantizer(q, out);
    return 1;
}

uint32_t vxb_registry_row(uint32_t index, char* out, uint32_t out_bytes) {
    if (index >= VXB_VARIANT_COUNT || !out || !out_bytes) return 0;
    const VxbVariant& v = kVariants[index];
    const bool grouped = (v.weight_mask & VXB_WEIGHT_PER_CHANNEL) == 0;
    // PackedLinear (R1) is served by every variant; the static QLinear operator (R2) by the
    // per-channel kernels that produce int8
    const char* ops = (!grouped && (v.epilogue_mask & VXB_EPI_I8)) ? "PackedLinear,QLinear" : "PackedLinear";
    const char* phase = v.max_rows && v.max_rows <= 128 ? "decode" : (v.flags & VXB_VF_VERIFY) ? "any" : "prefill";
    const bool tensor = strstr(v.route_label, "tcgen05") != nullptr;
    const int n = snprintf(out, out_bytes,
                           "cuda.packed-linear.%s | native-cuda | %s | w8a8-%s | %s | %s | cuda.sm100a-route-predicate | "
                           "cuda.device-residency,%s | %u",
                           v.route_label, ops, grouped ? "grouped" : "per-channel", phase, v.kernel,
                           tensor ? "cuda.sm100a-tcgen05" : "cuda.sm61-dp4a", v.priority);
    return n > 0 && (uint32_t)n < out_bytes ? (uint32_t)n : 0;
}

}  // extern "C"
