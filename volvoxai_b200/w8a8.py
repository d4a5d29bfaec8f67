"""Host-side mirror of the reference's operator interface for the W8A8 linear,
on top of the C ABI (include/vxb200_w8a8.h).

Two levels, as in the C header:

* ``Context`` / ``Weight`` / ``linear_*``: device-resident tensors (torch is
  used for device memory and streams only; every kernel is in libvxb200.so).
* ``qlinear_i8u8`` / ``packed_linear`` / ``packed_linear_decode``: NumPy host
  arrays in and out, the argument order, admission rules and tri-state return
  (1 handled / 0 declined / -1 failed) of the reference's CUDA backend hooks
  ``VxW8A8Ops.qlinear_i8u8`` (native/src/backends/w8a8_device_ops.h:15-17) and
  ``cuda_graph_llm_f32`` / ``cuda_graph_packed_linear_decode_f32``
  (native/src/backends/cuda_engine.h:13-19).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import (DT_I8, DT_U8, OP_PACKED_LINEAR, ROUTE_AUTO, ROUTE_DECODE, ROUTE_DECODE_FUSED, ROUTE_DECODE_STREAMK, ROUTE_TCGEN05_PAIR, ROUTE_TCGEN05_WIDE,
                   ROUTE_GEMV, ROUTE_SIMT,
                   ROUTE_TCGEN05, LLMOpArgs, last_error, last_route)

__all__ = ["Context", "Weight", "W8A8Error", "variants", "plan", "registry_rows", "qlinear_i8u8", "packed_linear",
           "packed_linear_decode", "host_cache_clear", "host_residency", "host_download", "host_invalidate", "launch_count", "last_error",
           "quantize_typed_f32_i8u8", "dequantize_typed_i8u8_f32", "requantize_linear_i8u8", "last_route", "ROUTE_AUTO", "ROUTE_GEMV", "ROUTE_TCGEN05", "ROUTE_SIMT", "ROUTE_DECODE", "ROUTE_DECODE_STREAMK", "ROUTE_TCGEN05_PAIR", "ROUTE_DECODE_FUSED", "ROUTE_TCGEN05_WIDE",
           "DT_I8", "DT_U8"]


class W8A8Error(RuntimeError):
    """Raised by the device-level wrappers when the library declines (0) or fails (-1)."""

    def __init__(self, code: int):
        self.code = code
        super().__init__(f"libvxb200 returned {code}: {last_error()}")


def _check(code: int) -> None:
    if code != 1:
        raise W8A8Error(code)


def _ptr(a) -> C.c_void_p:
    if a is None:
        return C.c_void_p(0)
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    return C.c_void_p(a.data_ptr())  # torch tensor


def launch_count() -> int:
    return int(_lib.load().vxb_launch_count())


def variants() -> list[dict]:
    """The kernel variant table (include/vxb200_plan.h) as dictionaries."""
    L = _lib.load()
    out = []
    for i in range(L.vxb_variant_count()):
        v = L.vxb_variant_info(i).contents
        row = {name: getattr(v, name) for name, _ in _lib.Variant._fields_}
        for key in ("id", "route_label", "kernel"):
            row[key] = row[key].decode()
        out.append(row)
    return out


def plan(rows: int, k: int, n: int, *, weight_kind: int = _lib.WEIGHT_PER_CHANNEL, group_size: int = 0,
         epilogue: int = _lib.EPI_F32, route: int = ROUTE_AUTO, n_peers: int = 0, fused_tail=False,
         fp32_input: bool = True, sm_count: int = 148, pair_clusters: int = 74, out_store_aligned: bool = True):
    """vxb_plan(): the launch plan of one call (a dict with the variant's id added) or
    (None, reason) when it is refused.  Needs no GPU."""
    L = _lib.load()
    # fused_tail: False / True (residual Add) or the bit mask itself (1 residual Add, 2 SiLU*Mul)
    q = _lib.PlanQuery(rows, k, n, weight_kind, group_size, epilogue, route, n_peers, int(fused_tail),
                       1 if fp32_input else 0, sm_count, pair_clusters, 1 if out_store_aligned else 0)
    out = _lib.LaunchPlan()
    why = C.create_string_buffer(200)
    if L.vxb_plan(C.byref(q), C.byref(out), why, len(why)) != 1:
        return None, why.value.decode()
    d = {name: getattr(out, name) for name, _ in _lib.LaunchPlan._fields_}
    d["id"] = L.vxb_variant_info(out.variant).contents.id.decode()
    return d, ""


def registry_rows() -> list[str]:
    """One kernel-registry row per variant, in the reference's KernelVariant field order."""
    L = _lib.load()
    rows = []
    for i in range(L.vxb_variant_count()):
        buf = C.create_string_buffer(512)
        if L.vxb_registry_row(i, buf, len(buf)):
            rows.append(buf.value.decode())
    return rows


def inject_failure(kind: int, countdown: int) -> None:
    """Host-side failure injection (diag.h): refuse the countdown-th launch (kind 1) or scratch
    allocation (kind 2) from now; countdown 0 disarms."""
    _lib.load().vxb_inject_failure(kind, countdown)


def tune(name: str, value: int) -> bool:
    return _lib.load().vxb_tune(name.encode(), int(value)) == 1


class Context:
    """Device + stream + reusable scratch (one per thread of use)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._L = _lib.load()
        self.device = device
        h = C.c_void_p(0)
        _check(self._L.vxb_context_create(device, C.c_void_p(stream or 0), C.byref(h)))
        self.handle = h

    def set_stream(self, stream: int | None) -> None:
        _check(self._L.vxb_context_set_stream(self.handle, C.c_void_p(stream or 0)))

    def use_torch_stream(self) -> None:
        import torch
        self.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    def synchronize(self) -> None:
        _check(self._L.vxb_context_synchronize(self.handle))

    def set_wait_limit(self, cycles: int) -> None:
        """Limit of every bounded device wait, in SM clocks (0 = the default, about 2 s)."""
        _check(self._L.vxb_context_set_wait_limit(self.handle, int(cycles)))

    def selftest_wait_expiry(self) -> None:
        """Launches the kernel whose only wait runs out by design (diag.h)."""
        _check(self._L.vxb_selftest_wait_expiry(self.handle))

    def selftest_div_const(self, exponent: int, neighbours: int = 2, samples: int = 64):
        """(mismatches, divisions checked) of div_const against the IEEE divide over every divisor
        significand at the given exponent."""
        bad, done = C.c_uint64(0), C.c_uint64(0)
        _check(self._L.vxb_selftest_div_const(self.handle, exponent, neighbours, samples, C.byref(bad), C.byref(done)))
        return bad.value, done.value

    def measure_i8_tensor_peak(self, iters: int = 200) -> float:
        out = C.c_double(0.0)
        _check(self._L.vxb_measure_i8_tensor_peak(self.handle, iters, C.byref(out)))
        return out.value

    def trace(self, stamps) -> None:
        """Decode-kernel time stamps into the int64 CUDA tensor `stamps` ([ctas, 8]); None stops."""
        _check(self._L.vxb_context_trace(self.handle, _ptr(stamps) if stamps is not None else None))

    def profile(self, enable) -> None:
        """Start (True, or an int n > 1 to bracket only every n-th launch of each kind) or stop (False)
        per-kernel event timing; both clear the record."""
        _check(self._L.vxb_context_profile(self.handle, int(enable)))

    def profile_read(self) -> dict:
        qms, qn, gms, gn = C.c_double(0), C.c_uint64(0), C.c_double(0), C.c_uint64(0)
        _check(self._L.vxb_context_profile_read(self.handle, C.byref(qms), C.byref(qn),
                                                C.byref(gms), C.byref(gn)))
        return {"quantize_ms": qms.value, "quantize_launches": qn.value,
                "gemm_ms": gms.value, "gemm_launches": gn.value}

    def linear_host(self, w: "Weight", x_host, y_host, requant: bool = False,
                    out_scale: float = 1.0, out_zero: int = 0) -> None:
        """Whole op on HOST buffers (NumPy arrays or pinned torch CPU tensors):
        h2d copy, kernels, d2h copy, wait."""
        rows = x_host.shape[0]
        _check(self._L.vxb_linear_host(self.handle, w.handle, _ptr(x_host), rows,
                                       1 if requant else 0, float(out_scale), int(out_zero),
                                       _ptr(y_host)))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._L.vxb_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- device-pointer entries (torch tensors on this device) ----
    def quantize_rows(self, x, ldq: int | None = None):
        """fp32 [rows,k] -> (int8 [rows,ldq], fp32 scales [rows], int32 valid [rows])."""
        import torch
        rows, k = x.shape
        ldq = ldq or k
        q = torch.empty((rows, ldq), dtype=torch.int8, device=x.device)
        s = torch.empty(rows, dtype=torch.float32, device=x.device)
        v = torch.empty(rows, dtype=torch.int32, device=x.device)
        _check(self._L.vxb_quantize_rows(self.handle, _ptr(x), rows, k, _ptr(q), ldq, _ptr(s), _ptr(v)))
        return q, s, v

    def rmsnorm_quantize_rows(self, x, norm_weight, epsilon: float, ldq: int | None = None,
                              want_norm: bool = True):
        """RMSNorm folded into the quantizer: -> (normalized fp32 rows or None, q, scales, valid)."""
        import torch
        rows, k = x.shape
        ldq = ldq or k
        q = torch.empty((rows, ldq), dtype=torch.int8, device=x.device)
        s = torch.empty(rows, dtype=torch.float32, device=x.device)
        v = torch.empty(rows, dtype=torch.int32, device=x.device)
        y = torch.empty_like(x) if want_norm else None
        _check(self._L.vxb_rmsnorm_quantize_rows(self.handle, _ptr(x), _ptr(norm_weight), float(epsilon), rows, k,
                                                 _ptr(y) if want_norm else None, _ptr(q), ldq, _ptr(s), _ptr(v)))
        return y, q, s, v

    def rmsnorm_linear_f32_fused(self, w: "Weight", x, norm_weight, epsilon: float, silu_mul: bool = False,
                                 norm_out=None, out=None):
        """RMSNorm -> quantize -> linear (+ silu(gate) * up over interleaved channel pairs)."""
        import torch
        rows = x.shape[0]
        width = w.d_out // 2 if silu_mul else w.d_out
        if out is None:
            out = torch.empty((rows, width), dtype=torch.float32, device=x.device)
        _check(self._L.vxb_rmsnorm_linear_f32_fused(self.handle, w.handle, _ptr(x), _ptr(norm_weight), float(epsilon),
                                                    _ptr(norm_out) if norm_out is not None else None, rows,
                                                    _ptr(out), out.stride(0), 1 if silu_mul else 0))
        return out

    def linear_f32(self, w: "Weight", x, out=None, route: int = ROUTE_AUTO):
        import torch
        rows = x.shape[0]
        if out is None:
            out = torch.empty((rows, w.d_out), dtype=torch.float32, device=x.device)
        _check(self._L.vxb_linear_f32(self.handle, w.handle, _ptr(x), rows, _ptr(out),
                                      out.stride(0), route))
        return out

    def linear_f32_fused(self, w: "Weight", x, residual=None, silu_mul: bool = False, out=None):
        """fp32 linear with a fused tail: + residual, or silu(gate) * up over interleaved channel
        pairs (output d_out / 2 wide)."""
        import torch
        rows = x.shape[0]
        width = w.d_out // 2 if silu_mul else w.d_out
        if out is None:
            out = torch.empty((rows, width), dtype=torch.float32, device=x.device)
        _check(self._L.vxb_linear_f32_fused(self.handle, w.handle, _ptr(x), rows, _ptr(out), out.stride(0),
                                            _ptr(residual) if residual is not None else None,
                                            residual.stride(0) if residual is not None else 0,
                                            1 if silu_mul else 0))
        return out

    def linear_i8(self, w: "Weight", x, out_scale: float, out_zero: int = 0, out=None,
                  route: int = ROUTE_AUTO):
        import torch
        rows = x.shape[0]
        if out is None:
            out = torch.empty((rows, w.d_out), dtype=torch.int8, device=x.device)
        _check(self._L.vxb_linear_i8(self.handle, w.handle, _ptr(x), rows, float(out_scale),
                                     int(out_zero), _ptr(out), out.stride(0), route))
        return out

    def linear_acc_i32(self, w: "Weight", x, route: int = ROUTE_AUTO, want_q: bool = False):
        import torch
        rows = x.shape[0]
        acc = torch.empty((rows, w.d_out), dtype=torch.int32, device=x.device)
        q = torch.empty((rows, w.d_in), dtype=torch.int8, device=x.device) if want_q else None
        s = torch.empty(rows, dtype=torch.float32, device=x.device) if want_q else None
        _check(self._L.vxb_linear_acc_i32(self.handle, w.handle, _ptr(x), rows, _ptr(acc),
                                          _ptr(q), _ptr(s), route))
        return (acc, q, s) if want_q else acc

    def prepare(self, w: "Weight", x):
        """Quantize rows into the weight's padded row layout: (int8 [rows,row_bytes], scales)."""
        q, s, _ = self.quantize_rows(x, ldq=w.row_bytes)
        return q, s

    def linear_prepared(self, w: "Weight", q, row_scales, out, mode: int = 1, out_scale: float = 1.0,
                        out_zero: int = 0, route: int = ROUTE_AUTO):
        """GEMM + epilogue over already-quantized rows (mode 0 int32 / 1 fp32 / 2 int8)."""
        _check(self._L.vxb_linear_prepared(self.handle, w.handle, _ptr(q), _ptr(row_scales),
                                           q.shape[0], mode, float(out_scale), int(out_zero),
                                           _ptr(out), out.stride(0), route))
        return out

    # ---- boundary of a static W8A8 island (torch CUDA tensors) ----
    def quantize_linear(self, x, scale: float, zero_point: int = 0, unsigned: bool = False):
        import torch
        out = torch.empty(x.shape, dtype=torch.uint8 if unsigned else torch.int8, device=x.device)
        _check(self._L.vxb_quantize_linear_device(self.handle, _ptr(x), x.numel(), float(scale), int(zero_point),
                                                  DT_U8 if unsigned else DT_I8, _ptr(out)))
        return out

    def dequantize_linear(self, x, scale: float, zero_point: int = 0):
        import torch
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        _check(self._L.vxb_dequantize_linear_device(self.handle, _ptr(x), x.numel(), float(scale), int(zero_point),
                                                    DT_U8 if x.dtype == torch.uint8 else DT_I8, _ptr(out)))
        return out

    def requantize_linear(self, x, input_scale: float, input_zero_point: int, output_scale: float,
                          output_zero_point: int, unsigned: bool = False):
        import torch
        out = torch.empty(x.shape, dtype=torch.uint8 if unsigned else torch.int8, device=x.device)
        _check(self._L.vxb_requantize_linear_device(self.handle, _ptr(x), x.numel(), float(input_scale),
                                                    int(input_zero_point), float(output_scale), int(output_zero_point),
                                                    DT_U8 if x.dtype == torch.uint8 else DT_I8,
                                                    DT_U8 if unsigned else DT_I8, _ptr(out)))
        return out

    def qlinear_device(self, w: "Weight", x, input_scale, input_zero, output_scale, output_zero,
                       out_unsigned: bool = False, route: int = ROUTE_AUTO):
        import torch
        rows = x.shape[0]
        in_dt = DT_U8 if x.dtype == torch.uint8 else DT_I8
        out = torch.empty((rows, w.d_out), dtype=torch.uint8 if out_unsigned else torch.int8,
                          device=x.device)
        _check(self._L.vxb_qlinear_device(self.handle, w.handle, _ptr(x), rows, float(input_scale),
                                          int(input_zero), float(output_scale), int(output_zero),
                                          in_dt, DT_U8 if out_unsigned else DT_I8, _ptr(out),
                                          out.stride(0), route))
        return out


class Weight:
    """One linear's weights on the device, repacked once (the compile-time step)."""

    def __init__(self, ctx: Context, handle):
        self._L = ctx._L
        self.ctx = ctx
        self.handle = handle
        self.d_in = int(self._L.vxb_weight_d_in(handle))
        self.d_out = int(self._L.vxb_weight_d_out(handle))
        self.row_bytes = int(self._L.vxb_weight_row_bytes(handle))

    @classmethod
    def from_i8(cls, ctx: Context, w: np.ndarray, ws: np.ndarray, bias_f32=None, bias_i32=None):
        """int8 [d_out,d_in] + fp32 scale [d_out] (the W8A8 SafeTensors layout)."""
        w = np.ascontiguousarray(w, np.int8)
        ws = np.ascontiguousarray(ws, np.float32)
        bf = None if bias_f32 is None else np.ascontiguousarray(bias_f32, np.float32)
        bi = None if bias_i32 is None else np.ascontiguousarray(bias_i32, np.int32)
        h = C.c_void_p(0)
        _check(ctx._L.vxb_weight_create_i8(ctx.handle, _ptr(w), _ptr(ws), _ptr(bf), _ptr(bi),
                                           w.shape[0], w.shape[1], C.byref(h)))
        return cls(ctx, h)

    @classmethod
    def from_w8_words(cls, ctx: Context, words: np.ndarray, group_scales: np.ndarray, d_in: int,
                      group_size: int, bias_f32=None):
        """PackedLinear W8 storage: I32 words [d_out,ceil(d_in/4)] + group scales."""
        words = np.ascontiguousarray(words).view(np.int32)
        gs = np.ascontiguousarray(group_scales, np.float32)
        bf = None if bias_f32 is None else np.ascontiguousarray(bias_f32, np.float32)
        h = C.c_void_p(0)
        _check(ctx._L.vxb_weight_create_w8_words(ctx.handle, _ptr(words), _ptr(gs), _ptr(bf),
                                                 words.shape[0], d_in, group_size, C.byref(h)))
        return cls(ctx, h)

    @classmethod
    def from_w4_words(cls, ctx: Context, words: np.ndarray, group_scales: np.ndarray, d_in: int,
                      group_size: int, bias_f32=None):
        """PackedLinear W4 storage: I32 words [d_out,ceil(d_in/8)] of eight 4-bit codes
        (weight = code - 8) + group scales; unpacked to int8 on load."""
        words = np.ascontiguousarray(words).view(np.int32)
        gs = np.ascontiguousarray(group_scales, np.float32)
        bf = None if bias_f32 is None else np.ascontiguousarray(bias_f32, np.float32)
        h = C.c_void_p(0)
        _check(ctx._L.vxb_weight_create_w4_words(ctx.handle, _ptr(words), _ptr(gs), _ptr(bf),
                                                 words.shape[0], d_in, group_size, C.byref(h)))
        return cls(ctx, h)

    @property
    def device_bytes(self) -> int:
        return int(self._L.vxb_weight_device_bytes(self.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._L.vxb_weight_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- reference-facing host entries (NumPy in / out, tri-state int return) ----

def qlinear_i8u8(input, weight, weight_scales, weight_zero_points, bias, output,
                 input_scale, input_zero_point, output_scale, output_zero_point) -> int:
    """Same argument meaning and order as ``VxW8A8Ops.qlinear_i8u8``; dtypes are taken from
    the arrays (int8 / uint8). Writes ``output`` in place. Returns 1 / 0 / -1."""
    L = _lib.load()
    rows, d_in = input.shape
    d_out = weight.shape[0]

    def dt(a):
        return DT_U8 if a.dtype == np.uint8 else DT_I8
    for a in (input, weight, output):
        if a.dtype not in (np.int8, np.uint8) or not a.flags.c_contiguous:
            raise TypeError("byte tensors must be contiguous int8/uint8 arrays")
    ws = np.ascontiguousarray(weight_scales, np.float32)
    wz = np.ascontiguousarray(weight_zero_points, np.int32)
    b = np.ascontiguousarray(bias, np.int32)
    return int(L.vxb_qlinear_i8u8(_ptr(input), _ptr(weight), _ptr(ws), _ptr(wz), _ptr(b),
                                  _ptr(output), rows, d_in, d_out, float(input_scale),
                                  int(input_zero_point), float(output_scale),
                                  int(output_zero_point), dt(input), dt(weight), dt(output)))


def _np_dt(a):
    return DT_U8 if a.dtype == np.uint8 else DT_I8


def quantize_typed_f32_i8u8(input, output, output_scale, output_zero_point) -> int:
    """``VxW8A8Ops.quantize_typed_f32_i8u8``: fp32 NumPy array -> int8/uint8 array in place."""
    return int(_lib.load().vxb_quantize_typed_f32_i8u8(_ptr(input), input.size, _ptr(output), float(output_scale),
                                                       int(output_zero_point), _np_dt(output)))


def dequantize_typed_i8u8_f32(input, input_scale, input_zero_point, output) -> int:
    """``VxW8A8Ops.dequantize_typed_i8u8_f32``: int8/uint8 NumPy array -> fp32 array in place."""
    return int(_lib.load().vxb_dequantize_typed_i8u8_f32(_ptr(input), input.size, float(input_scale),
                                                         int(input_zero_point), _np_dt(input), _ptr(output)))


def requantize_linear_i8u8(input, output, input_scale, input_zero_point, output_scale, output_zero_point) -> int:
    """``VxW8A8Ops.requantize_linear_i8u8``: byte array -> byte array of another quantized domain."""
    return int(_lib.load().vxb_requantize_linear_i8u8(_ptr(input), input.size, _ptr(output), output.size,
                                                      float(input_scale), int(input_zero_point), float(output_scale),
                                                      int(output_zero_point), _np_dt(input), _np_dt(output)))


def packed_linear(x, words, scales, bias, y, *, weight_bits=8, group_size=128,
                  activation_bits=8, first_unit=0, unit_count=0) -> int:
    """PackedLinear through the ``cuda_graph_llm_f32`` drop-in: builds the reference's
    VxLLMOpArgs descriptor (kind=1036, key_dim=K, value_dim=N, rate=group size,
    groups=weight bits, normalize=activation bits, batch*sequence=rows) and calls the C
    entry. ``y`` (fp32 [rows,N]) is written in place inside the window. Returns 1/0/-1."""
    L = _lib.load()
    for a, t in ((x, np.float32), (scales, np.float32), (y, np.float32)):
        if a.dtype != t or not a.flags.c_contiguous:
            raise TypeError("x, scales and y must be contiguous float32 arrays")
    words = np.ascontiguousarray(words).view(np.int32)
    rows, k = x.shape
    a = LLMOpArgs()
    a.kind, a.batch, a.sequence = OP_PACKED_LINEAR, 1, rows
    a.key_dim, a.value_dim = k, words.shape[0]
    a.groups, a.rate, a.normalize = weight_bits, group_size, activation_bits
    a.x[0], a.x[1], a.x[2] = x.ctypes.data, words.ctypes.data, scales.ctypes.data
    a.x[3] = bias.ctypes.data if bias is not None else None
    a.y[0] = y.ctypes.data
    a.x_elements[0], a.x_elements[1], a.x_elements[2] = x.size, words.size, scales.size
    a.y_elements[0] = y.size
    a.first_unit, a.unit_count = first_unit, unit_count
    keep = (x, words, scales, bias, y)  # noqa: F841  (alive across the call)
    return int(L.vxb_cuda_graph_llm_f32(C.byref(a)))


def packed_linear_decode(x, words, scales, bias, y, *, weight_bits=8, activation_bits=8) -> int:
    """One-row decode entry (``cuda_graph_packed_linear_decode_f32``), group size 128."""
    L = _lib.load()
    words = np.ascontiguousarray(words).view(np.int32)
    return int(L.vxb_cuda_graph_packed_linear_decode_f32(
        _ptr(x), _ptr(words), _ptr(scales), _ptr(bias), _ptr(y), x.shape[-1], words.shape[0],
        weight_bits, activation_bits))


def host_cache_clear() -> None:
    _lib.load().vxb_host_cache_clear()


def host_residency(enable: bool) -> int:
    """Outputs of the reference-facing entries stay on the device (host copies stale until
    host_download) and feed later entries in place; see vxb_host_residency."""
    return int(_lib.load().vxb_host_residency(1 if enable else 0))


def host_download(array=None) -> int:
    """Makes the host copy of a device-resident output current (None: every tensor)."""
    return int(_lib.load().vxb_host_download(_ptr(array)))


def host_invalidate(array=None) -> int:
    """The host wrote this buffer itself: drop its device copy (None: all)."""
    return int(_lib.load().vxb_host_invalidate(_ptr(array)))
