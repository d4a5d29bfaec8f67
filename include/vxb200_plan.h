/*
 * vxb200_plan.h - the kernel variants of the B200 W8A8 linear route, their admission
 * facts and launch geometry, and the pure planning function that picks one.
 *
 * Counterpart of the reference's packed launch planning: the variant table
 * VxCudaPackedVariant with its X-macro rows
 * (native/src/backends/cuda/packed_launch_plan.h:15-31,
 *  native/src/backends/cuda/host/cuda_forward_function_registry_host.inc:308-334),
 * vx_cuda_packed_plan / vx_cuda_packed_select (packed_launch_plan.h:33-125) and the
 * public registry rows KernelVariant{id, backend, operator, profile, phase,
 * entrypoint_id, predicate_id, required_feature, priority}
 * (proto/kernel_registry.proto:116-126).  As there, one row per kernel carries
 * everything a launch needs, the selector never infers a kernel from a row count
 * alone, and the functions below need no GPU: tests call them on a CPU-only box.
 *
 * The library's own dispatch (vxb_linear_*, the reference-facing entries) goes
 * through vxb_plan(), so what a test sees here is what a call launches.
 */
#ifndef VXB200_PLAN_H
#define VXB200_PLAN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define VXB_PLAN_API __attribute__((visibility("default")))
#else
#define VXB_PLAN_API
#endif

/* Epilogue masks (which outputs a variant can produce). */
#define VXB_EPI_ACC 1u  /* raw int32 accumulators */
#define VXB_EPI_F32 2u  /* dequant + bias, fp32 (E1) */
#define VXB_EPI_I8 4u   /* requantized int8 / uint8 (E2) */
/* Weight kinds (how the scales are stored). */
#define VXB_WEIGHT_PER_CHANNEL 1u /* one scale per output channel */
#define VXB_WEIGHT_GROUPED 2u     /* PackedLinear group scales that differ within a channel */
#define VXB_WEIGHT_W4_WORDS 4u    /* grouped, and the 4-bit words are kept for the nibble-streaming kernel */
/* Variant flags. */
#define VXB_VF_AUTO 1u        /* eligible for automatic selection */
#define VXB_VF_PEERS 2u       /* epilogue can store to peer GPUs (fused all-gather); clustered variants only as TMA \
                                 tile stores, i.e. into buffers whose base, row pitch and width are multiples of 16 bytes */
#define VXB_VF_FUSED_TAIL 4u  /* carries the residual-Add / SiLU*Mul tails of the fp32 epilogue */
#define VXB_VF_VERIFY 8u      /* verification kernel: explicit request only */
#define VXB_VF_FUSED_K1 16u   /* quantizes the fp32 rows itself: one launch per linear, fp32 input only */
#define VXB_VF_TILE_STORE 32u /* 32-bit outputs leave as TMA tile stores: output base, row pitch and width multiples of 16 bytes, \
                                 residual Add as the only fused tail */

/*
 * Variant rows.  Fields:
 *   id, route (VXB_ROUTE_* of vxb200_w8a8.h), route label (the tail vxb_last_route() reports),
 *   kernel symbol, tile rows (0 = token slots chosen from the row count), tile columns
 *   (0 = ceil(d_out / SMs) whole channels per CTA), tile K bytes, threads per CTA, CTAs per cluster,
 *   dynamic shared memory bound in bytes, minimum rows, maximum rows (0 = unbounded),
 *   epilogue mask, weight-kind mask, required group size (0 = any), flags, registry priority.
 */
#define VXB_VARIANTS(X) \
    X(DECODE_ROWS,      4, "decode-rows-tcgen05-i8",    "decode_rows_kernel",             0,   0, 128, 544, 1, 204800,   1, 128, 7u, 1u, 0, 1u | 4u,      700) \
    X(DECODE_FUSED,     7, "decode-fused-tcgen05-i8",   "decode_rows_kernel",             0,   0, 128, 544, 1, 204800,   1,   8, 7u, 1u, 0, 1u | 4u | 16u, 720) \
    X(DECODE_STREAMK,   5, "decode-streamk-tcgen05-i8", "decode_i8_tcgen05_kernel",       0, 128, 128, 192, 1, 107520,   1, 128, 7u, 1u, 0, 0u,           300) \
    X(GEMV_DP4A,        1, "gemv-dp4a",                 "gemv_dp4a_kernel",               0,   0,   0, 256, 1,  65536,   1,  32, 7u, 1u, 0, 0u,           200) \
    X(SIMT_DP4A,        3, "simt-dp4a",                 "gemm_simt_kernel",               4, 128,   0, 128, 1,      0,   1,   0, 7u, 1u, 0, 8u,             1) \
    X(TCGEN05,          2, "tcgen05-i8",                "gemm_i8_tcgen05_kernel",       128, 256, 128, 352, 1, 223000,   1,   0, 7u, 1u, 0, 1u | 2u | 4u,  600) \
    X(TCGEN05_PAIR,     6, "tcgen05-pair-i8",           "gemm_i8_pair_kernel",          256, 256, 256, 352, 2, 223000,   1,   0, 7u, 1u, 0, 1u | 2u | 4u,  650) \
    X(TCGEN05_WIDE,     8, "tcgen05-wide-i8",           "gemm_i8_wide_kernel",          128, 256, 128, 608, 1, 231000,   1,   0, 3u, 1u, 0, 1u | 4u | 32u, 640) \
    X(GROUPED_TCGEN05,  0, "tcgen05-grouped-i8",        "gemm_i8_grouped_tcgen05_kernel", 128, 128, 128, 320, 1, 223000,   1,   0, 2u, 6u, 0, 1u,           500) \
    X(GEMV_GROUPED,     0, "gemv-grouped",              "gemv_grouped_kernel",            0,   0,   0, 256, 1,  65536,   1,   4, 2u, 6u, 0, 1u,           550) \
    X(GEMV_W4_GROUPED,  0, "gemv-w4-grouped",           "gemv_w4_grouped_kernel",         0,   0,   0, 256, 1,  65536,   1,   2, 2u, 4u, 0, 1u,           560) \
    X(DP4A_GROUPED,     3, "dp4a-grouped",              "gemm_grouped_kernel",            4, 128,   0, 128, 1,      0,   1,   0, 2u, 6u, 0, 8u,             2)

typedef enum VxbVariantId {
#define VXB_VARIANT_ENUM(id, route, label, symbol, bm, bn, bk, threads, cluster, smem, min_rows, max_rows, epi, weights, group, flags, prio) \
    VXB_VARIANT_##id,
    VXB_VARIANTS(VXB_VARIANT_ENUM)
#undef VXB_VARIANT_ENUM
    VXB_VARIANT_COUNT
} VxbVariantId;

typedef struct VxbVariant {
    const char* id;          /* "DECODE_ROWS" */
    int32_t route;           /* VXB_ROUTE_*; 0 = reachable through the automatic route only */
    const char* route_label; /* what vxb_last_route() shows for it */
    const char* kernel;      /* __global__ symbol (template name without arguments) */
    uint32_t tile_rows, tile_columns, tile_k, threads, cluster, shared_bytes_max;
    uint32_t min_rows, max_rows, epilogue_mask, weight_mask, group_size, flags, priority;
} VxbVariant;

/* What a caller is about to ask for. */
typedef struct VxbPlanQuery {
    uint32_t rows, k, n;     /* tokens, d_in, d_out */
    uint32_t weight_kind;    /* one VXB_WEIGHT_* bit */
    uint32_t group_size;     /* 32/64/128/256 for grouped kinds, else 0 */
    uint32_t epilogue;       /* one VXB_EPI_* bit */
    int32_t requested_route; /* VXB_ROUTE_AUTO or an explicit VXB_ROUTE_* */
    uint32_t n_peers;        /* > 0: fused all-gather into peer buffers */
    uint32_t fused_tail;     /* tails of the fp32 epilogue: bit 0 residual Add, bit 1 SiLU*Mul over channel pairs */
    uint32_t fp32_input;     /* the call starts from fp32 activations (a K1 quantizer is part of it) */
    uint32_t sm_count;       /* SMs of the device (148 on a B200) */
    uint32_t pair_clusters;  /* co-resident clusters of two the device grants the pair kernel (0: none) */
    uint32_t out_store_aligned; /* the output's (and every peer buffer's) base, row pitch and width are multiples of 16 bytes \
                                   (TMA tile stores possible) */
} VxbPlanQuery;

/* Per-row quantizer (K1) chosen for calls that start from fp32 activations. */
typedef enum VxbQuantizerId {
    VXB_QUANTIZER_NONE = 0,   /* prepared int8 activations, or quantization fused into the GEMV */
    VXB_QUANTIZER_SCALAR,     /* quantize_rows_scalar: any width / alignment, one warp per row */
    VXB_QUANTIZER_VEC,        /* quantize_rows_vec<TPR>: row cached in registers, 128-bit loads */
    VXB_QUANTIZER_CLUSTER     /* quantize_rows_cluster<S>: few long rows shared by 2/4/8 CTAs */
} VxbQuantizerId;

typedef struct VxbLaunchPlan {
    int32_t variant;         /* VxbVariantId */
    int32_t route;           /* the variant's VXB_ROUTE_* (0 for automatic-only variants) */
    uint32_t tile_rows, tile_columns, tile_k;
    uint32_t grid, threads, cluster;
    uint32_t launches;       /* kernel launches of the whole call (quantizer included) */
    int32_t quantizer;       /* VxbQuantizerId */
    uint32_t quantizer_grid, quantizer_cluster;
    uint64_t workspace_bytes; /* context scratch the call needs (quantized rows, scales, split-K partials) */
} VxbLaunchPlan;

#define VXB_WIDE_MAX_KPAD 1536u /* measured: equal at 2048, slower beyond (three pipeline stages) */

VXB_PLAN_API uint32_t vxb_variant_count(void);
/* NULL when index is out of range. */
VXB_PLAN_API const VxbVariant* vxb_variant_info(uint32_t index);

/* Builds the launch plan of one call or refuses it.  Returns 1 and fills *out, or 0 with the
 * reason in `why` (optional buffer).  An explicit route is honoured or refused, never replaced;
 * the automatic route picks, among the admitted variants flagged VXB_VF_AUTO, by these rules:
 *   per-channel scales: rows <= 128 -> the decode kernel (its single-launch form, which quantizes the
 *     rows itself, for fp32 input of one or two rows with a padded K of at most 8192 and d_in a
 *     multiple of 4; an explicit request admits it up to 8 rows), else the tensor-core GEMM, by pairs
 *     of CTAs once there are two waves of 128 x 256 tiles; 32-bit outputs with a padded K of at most
 *     VXB_WIDE_MAX_KPAD (the output, not the tensor pipe, bounds those launches) take the kernel
 *     built for them (sixteen epilogue warps, TMA tile stores) when the output is 16-byte aligned;
 *   grouped scales: 1-2 rows (3-4 with <= 32 MB of weights) -> the streaming GEMV (over the 4-bit
 *     words when kept), else the tensor-core kernel with a per-group accumulator drain. */
VXB_PLAN_API int vxb_plan(const VxbPlanQuery* query, VxbLaunchPlan* out, char* why, uint32_t why_bytes);

/* One kernel-registry row per variant, in the reference's KernelVariant field order:
 *   id | backend | operator | profile | phase | entrypoint_id | predicate_id | required_feature | priority
 * e.g. "cuda.packed-linear.tcgen05-pair-i8 | native-cuda | PackedLinear,QLinear | ...".  Returns the
 * number of characters written (0 when index is out of range or the buffer is too small). */
VXB_PLAN_API uint32_t vxb_registry_row(uint32_t index, char* out, uint32_t out_bytes);

#ifdef __cplusplus
}
#endif
#endif /* VXB200_PLAN_H */
