"""ctypes binding of libvxb200.so (the C ABI declared in include/vxb200_w8a8.h).

Loading fails loudly: there is no CPU or PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libvxb200.so")

DT_U8, DT_I8 = 5, 6
OP_PACKED_LINEAR = 1036
ROUTE_AUTO, ROUTE_GEMV, ROUTE_TCGEN05, ROUTE_SIMT, ROUTE_DECODE, ROUTE_DECODE_STREAMK = 0, 1, 2, 3, 4, 5
ROUTE_TCGEN05_PAIR = 6
ROUTE_DECODE_FUSED = 7
ROUTE_TCGEN05_WIDE = 8

# Every symbol include/vxb200_w8a8.h declares.
EXPORTS = [
    "vxb_abi_version", "vxb_last_error", "vxb_last_route", "vxb_launch_count",
    "vxb_context_create", "vxb_context_destroy", "vxb_context_set_stream",
    "vxb_context_synchronize", "vxb_weight_create_i8", "vxb_weight_create_w8_words",
    "vxb_weight_destroy", "vxb_weight_d_in", "vxb_weight_d_out", "vxb_weight_device_bytes",
    "vxb_quantize_rows", "vxb_linear_f32", "vxb_linear_i8", "vxb_linear_acc_i32",
    "vxb_qlinear_device", "vxb_weight_row_bytes", "vxb_linear_prepared", "vxb_linear_host", "vxb_context_profile", "vxb_context_profile_read",
    "vxb_measure_i8_tensor_peak", "vxb_peer_alloc", "vxb_peer_open",
    "vxb_peer_close", "vxb_peer_free", "vxb_linear_i8_gather", "vxb_peer_barrier", "vxb_linear_f32_fused", "vxb_weight_create_w4_words",
    "vxb_rmsnorm_quantize_rows", "vxb_rmsnorm_linear_f32_fused", "vxb_quantize_linear_device",
    "vxb_dequantize_linear_device", "vxb_requantize_linear_device", "vxb_quantize_typed_f32_i8u8",
    "vxb_dequantize_typed_i8u8_f32", "vxb_requantize_linear_i8u8", "vxb_decode_linear_f32_noalloc", "vxb_qlinear_i8u8",
    "vxb_cuda_graph_llm_f32", "vxb_cuda_graph_packed_linear_decode_f32", "vxb_host_cache_clear",
    "vxb_host_residency", "vxb_host_download", "vxb_host_invalidate",
]


# include/vxb200_plan.h: variant table, launch planning, registry rows (no GPU needed).
PLAN_EXPORTS = ["vxb_variant_count", "vxb_variant_info", "vxb_plan", "vxb_registry_row"]
# include/vxb200_package.h: graph.json + SafeTensors loader and the device-resident forward pass.
PACKAGE_EXPORTS = ["vxb_package_open", "vxb_package_close", "vxb_package_node_count", "vxb_package_node_op",
                   "vxb_package_io_count", "vxb_package_io_name", "vxb_package_io_dtype", "vxb_package_io_rank",
                   "vxb_package_io_dim", "vxb_package_io_bytes", "vxb_program_compile", "vxb_program_destroy",
                   "vxb_program_device_bytes", "vxb_program_route_evidence", "vxb_program_execute"]
DT_F32, DT_I32 = 18, 16
# volvoxai_b200/csrc/diag.h: diagnostics and self-tests, not part of the drop-in boundary.
DIAG_EXPORTS = ["vxb_context_trace", "vxb_measure_mma_issue", "vxb_context_set_wait_limit",
                "vxb_selftest_wait_expiry", "vxb_selftest_div_const", "vxb_inject_failure", "vxb_tune"]

EPI_ACC, EPI_F32, EPI_I8 = 1, 2, 4
WEIGHT_PER_CHANNEL, WEIGHT_GROUPED, WEIGHT_W4_WORDS = 1, 2, 4
VF_AUTO, VF_PEERS, VF_FUSED_TAIL, VF_VERIFY, VF_FUSED_K1 = 1, 2, 4, 8, 16
INJECT_LAUNCH, INJECT_ALLOCATION = 1, 2


class Variant(C.Structure):
    """VxbVariant of include/vxb200_plan.h."""
    _fields_ = [("id", C.c_char_p), ("route", C.c_int32), ("route_label", C.c_char_p), ("kernel", C.c_char_p)] + [
        (n, C.c_uint32) for n in ("tile_rows", "tile_columns", "tile_k", "threads", "cluster", "shared_bytes_max",
                                  "min_rows", "max_rows", "epilogue_mask", "weight_mask", "group_size", "flags",
                                  "priority")]


class PlanQuery(C.Structure):
    """VxbPlanQuery of include/vxb200_plan.h."""
    _fields_ = [("rows", C.c_uint32), ("k", C.c_uint32), ("n", C.c_uint32), ("weight_kind", C.c_uint32),
                ("group_size", C.c_uint32), ("epilogue", C.c_uint32), ("requested_route", C.c_int32),
                ("n_peers", C.c_uint32), ("fused_tail", C.c_uint32), ("fp32_input", C.c_uint32),
                ("sm_count", C.c_uint32), ("pair_clusters", C.c_uint32), ("out_store_aligned", C.c_uint32)]


class LaunchPlan(C.Structure):
    """VxbLaunchPlan of include/vxb200_plan.h."""
    _fields_ = [("variant", C.c_int32), ("route", C.c_int32), ("tile_rows", C.c_uint32), ("tile_columns", C.c_uint32),
                ("tile_k", C.c_uint32), ("grid", C.c_uint32), ("threads", C.c_uint32), ("cluster", C.c_uint32),
                ("launches", C.c_uint32), ("quantizer", C.c_int32), ("quantizer_grid", C.c_uint32),
                ("quantizer_cluster", C.c_uint32), ("workspace_bytes", C.c_uint64)]


class LLMOpArgs(C.Structure):
    """Field-for-field mirror of the reference's VxLLMOpArgs
    (native/src/kernels/llm_ops.h:38-53)."""
    _fields_ = [(n, C.c_int32) for n in (
        "kind", "batch", "sequence", "keys", "heads", "kv_heads", "key_dim", "value_dim",
        "streams", "groups", "rate", "window", "top_k", "iterations",
        "index_heads", "index_dim", "rotary_dim", "rotary_offset",
        "normalize", "causal", "interleaved", "mask_mode")] + [
        ("eps", C.c_float), ("hc_eps", C.c_float), ("scale", C.c_float),
        ("x", C.c_void_p * 8), ("y", C.c_void_p * 3),
        ("mask", C.c_void_p), ("positions", C.c_void_p),
        ("x_elements", C.c_uint64 * 8), ("y_elements", C.c_uint64 * 3),
        ("mask_elements", C.c_uint64), ("position_elements", C.c_uint64),
        ("query_offset", C.c_int32), ("first_unit", C.c_uint64), ("unit_count", C.c_uint64)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m volvoxai_b200.build` "
            "(nvcc, sm_100a). There is no fallback path.")
    L = C.CDLL(LIB_PATH)
    vp, u32, i32, f32 = C.c_void_p, C.c_uint32, C.c_int32, C.c_float
    L.vxb_abi_version.restype = u32
    L.vxb_last_error.restype = C.c_char_p
    L.vxb_last_route.restype = C.c_char_p
    L.vxb_launch_count.restype = C.c_uint64
    L.vxb_context_create.argtypes = [C.c_int, vp, C.POINTER(vp)]
    L.vxb_context_destroy.argtypes = [vp]
    L.vxb_context_destroy.restype = None
    L.vxb_context_set_stream.argtypes = [vp, vp]
    L.vxb_context_synchronize.argtypes = [vp]
    L.vxb_weight_create_i8.argtypes = [vp, vp, vp, vp, vp, u32, u32, C.POINTER(vp)]
    L.vxb_weight_create_w8_words.argtypes = [vp, vp, vp, vp, u32, u32, u32, C.POINTER(vp)]
    L.vxb_weight_create_w4_words.argtypes = [vp, vp, vp, vp, u32, u32, u32, C.POINTER(vp)]
    L.vxb_weight_destroy.argtypes = [vp]
    L.vxb_weight_destroy.restype = None
    L.vxb_weight_d_in.argtypes = [vp]
    L.vxb_weight_d_in.restype = u32
    L.vxb_weight_d_out.argtypes = [vp]
    L.vxb_weight_d_out.restype = u32
    L.vxb_weight_device_bytes.argtypes = [vp]
    L.vxb_weight_device_bytes.restype = C.c_uint64
    L.vxb_quantize_rows.argtypes = [vp, vp, u32, u32, vp, u32, vp, vp]
    L.vxb_linear_f32.argtypes = [vp, vp, vp, u32, vp, u32, C.c_int]
    L.vxb_linear_i8.argtypes = [vp, vp, vp, u32, f32, i32, vp, u32, C.c_int]
    L.vxb_linear_acc_i32.argtypes = [vp, vp, vp, u32, vp, vp, vp, C.c_int]
    L.vxb_qlinear_device.argtypes = [vp, vp, vp, u32, f32, i32, f32, i32, u32, u32, vp, u32, C.c_int]
    L.vxb_weight_row_bytes.argtypes = [vp]
    L.vxb_weight_row_bytes.restype = u32
    L.vxb_linear_prepared.argtypes = [vp, vp, vp, vp, u32, C.c_int, f32, i32, vp, u32, C.c_int]
    L.vxb_linear_host.argtypes = [vp, vp, vp, u32, C.c_int, f32, i32, vp]
    L.vxb_context_trace.argtypes = [vp, vp]
    L.vxb_context_set_wait_limit.argtypes = [vp, C.c_uint64]
    L.vxb_selftest_wait_expiry.argtypes = [vp]
    L.vxb_selftest_div_const.argtypes = [vp, C.c_int, u32, u32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    L.vxb_inject_failure.argtypes = [C.c_int, u32]
    L.vxb_inject_failure.restype = None
    L.vxb_tune.argtypes = [C.c_char_p, C.c_int64]
    L.vxb_package_open.argtypes = [C.c_char_p, C.POINTER(C.c_char_p), C.c_size_t, C.POINTER(vp)]
    L.vxb_package_close.argtypes = [vp]
    L.vxb_package_close.restype = None
    L.vxb_package_node_count.argtypes = [vp]
    L.vxb_package_node_count.restype = u32
    L.vxb_package_node_op.argtypes = [vp, u32]
    L.vxb_package_node_op.restype = C.c_char_p
    L.vxb_package_io_count.argtypes = [vp, C.c_int]
    L.vxb_package_io_count.restype = u32
    L.vxb_package_io_name.argtypes = [vp, C.c_int, u32]
    L.vxb_package_io_name.restype = C.c_char_p
    for name in ("vxb_package_io_dtype", "vxb_package_io_rank"):
        getattr(L, name).argtypes = [vp, C.c_int, u32]
        getattr(L, name).restype = u32
    L.vxb_package_io_dim.argtypes = [vp, C.c_int, u32, u32]
    L.vxb_package_io_dim.restype = C.c_int64
    L.vxb_package_io_bytes.argtypes = [vp, C.c_int, u32]
    L.vxb_package_io_bytes.restype = C.c_uint64
    L.vxb_program_compile.argtypes = [vp, vp, C.POINTER(vp)]
    L.vxb_program_destroy.argtypes = [vp]
    L.vxb_program_destroy.restype = None
    L.vxb_program_device_bytes.argtypes = [vp]
    L.vxb_program_device_bytes.restype = C.c_uint64
    L.vxb_program_route_evidence.argtypes = [vp]
    L.vxb_program_route_evidence.restype = C.c_char_p
    L.vxb_program_execute.argtypes = [vp, C.POINTER(vp), C.POINTER(C.c_size_t), u32, C.POINTER(vp), C.POINTER(C.c_size_t), u32]
    L.vxb_variant_count.restype = u32
    L.vxb_variant_info.argtypes = [u32]
    L.vxb_variant_info.restype = C.POINTER(Variant)
    L.vxb_plan.argtypes = [C.POINTER(PlanQuery), C.POINTER(LaunchPlan), C.c_char_p, u32]
    L.vxb_registry_row.argtypes = [u32, C.c_char_p, u32]
    L.vxb_registry_row.restype = u32
    L.vxb_context_profile.argtypes = [vp, C.c_int]
    L.vxb_context_profile_read.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(C.c_uint64),
                                           C.POINTER(C.c_double), C.POINTER(C.c_uint64)]
    u64 = C.c_uint64
    L.vxb_quantize_linear_device.argtypes = [vp, vp, u64, f32, i32, u32, vp]
    L.vxb_dequantize_linear_device.argtypes = [vp, vp, u64, f32, i32, u32, vp]
    L.vxb_requantize_linear_device.argtypes = [vp, vp, u64, f32, i32, f32, i32, u32, u32, vp]
    L.vxb_quantize_typed_f32_i8u8.argtypes = [vp, u32, vp, f32, i32, u32]
    L.vxb_dequantize_typed_i8u8_f32.argtypes = [vp, u32, f32, i32, u32, vp]
    L.vxb_requantize_linear_i8u8.argtypes = [vp, u32, vp, u32, f32, i32, f32, i32, u32, u32]
    L.vxb_linear_f32_fused.argtypes = [vp, vp, vp, u32, vp, u32, vp, u32, C.c_int]
    L.vxb_rmsnorm_quantize_rows.argtypes = [vp, vp, vp, C.c_float, u32, u32, vp, vp, u32, vp, vp]
    L.vxb_rmsnorm_linear_f32_fused.argtypes = [vp, vp, vp, vp, C.c_float, vp, u32, vp, u32, C.c_int]
    L.vxb_peer_alloc.argtypes = [C.c_size_t, C.POINTER(vp), C.c_char_p]
    L.vxb_peer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.vxb_peer_close.argtypes = [vp]
    L.vxb_peer_free.argtypes = [vp]
    L.vxb_linear_i8_gather.argtypes = [vp, vp, vp, u32, f32, i32, vp, u32, C.POINTER(vp), u32]
    L.vxb_peer_barrier.argtypes = [vp, vp, C.POINTER(vp), C.POINTER(u32), u32, u32, u32]
    L.vxb_measure_mma_issue.argtypes = [vp, u32, u32, u32, u32, u32, C.POINTER(C.c_double)]
    L.vxb_measure_i8_tensor_peak.argtypes = [vp, u32, C.POINTER(C.c_double)]
    L.vxb_decode_linear_f32_noalloc.argtypes = [vp, vp, u32, vp, vp, vp, u32, u32, vp, u32, vp,
                                                C.c_int, C.c_char_p, C.c_size_t]
    L.vxb_qlinear_i8u8.argtypes = [vp, vp, vp, vp, vp, vp, u32, u32, u32, f32, i32, f32, i32,
                                   u32, u32, u32]
    L.vxb_cuda_graph_llm_f32.argtypes = [C.POINTER(LLMOpArgs)]
    L.vxb_cuda_graph_packed_linear_decode_f32.argtypes = [vp, vp, vp, vp, vp, u32, u32, u32, u32]
    L.vxb_host_cache_clear.restype = None
    L.vxb_host_residency.argtypes = [C.c_int]
    L.vxb_host_download.argtypes = [vp]
    L.vxb_host_invalidate.argtypes = [vp]
    for name in EXPORTS:
        fn = getattr(L, name)
        if fn.restype is C.c_int and name.startswith("vxb_") and name not in (
                "vxb_last_error", "vxb_last_route"):
            fn.restype = C.c_int
    _lib = L
    return L


def last_error() -> str:
    return load().vxb_last_error().decode(errors="replace")


def last_route() -> str:
    return load().vxb_last_route().decode(errors="replace")
