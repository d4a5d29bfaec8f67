"""ctypes bindings for the two CPU checkers (test infrastructure only).

``Oracle``  -> oracle/liboracle.so, the plain-C restatement (w8a8_oracle.c).
``Ref``     -> oracle/_ref/libvxref.so, the reference's own CPU kernels compiled
               from its sources by oracle/Makefile (``Ref.available()`` is False
               when that library was never built).

Only tests/, the smoke run and the benchmark's CPU-baseline legs import this
module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libvxref.so")

# VX_DTYPE_* values of the reference (native/include/volvoxai_enums.h:479-480).
DT_U8, DT_I8 = 5, 6


def reference_root() -> str:
    """Where the reference checkout lies: $VX_REFERENCE, else a checkout named `reference`
    beside this repository."""
    return os.environ.get("VX_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str | None = None) -> None:
    """Compile liboracle.so and, when the reference checkout exists, _ref."""
    subprocess.run(["make", "-s", "-C", HERE, f"REF={ref_root or reference_root()}", "all"], check=True)


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build()
        L = self.lib = C.CDLL(ORACLE_SO)
        L.vxo_round_i8.restype = C.c_int32
        L.vxo_round_i8.argtypes = [C.c_float]
        L.vxo_round_ties_even.restype = C.c_int32
        L.vxo_round_ties_even.argtypes = [C.c_float]
        L.vxo_multiplier.restype = C.c_int
        L.vxo_multiplier.argtypes = [C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]
        L.vxo_gemm_i32.restype = C.c_int
        L.vxo_requant_rows.restype = C.c_int
        L.vxo_qlinear_i8u8.restype = C.c_int
        L.vxo_packed_linear_w8_grouped.restype = C.c_int
        L.vxo_packed_linear_w4_grouped.restype = C.c_int
        L.vxo_w8a8_linear.restype = C.c_int
        L.vxo_div_const_mismatches.restype = C.c_uint64
        L.vxo_div_const_mismatches.argtypes = [C.c_float, C.c_uint64, C.c_uint64, C.c_int, C.c_int]

    def div_const_mismatches(self, d, count, seed=1, lo_exp=-60, hi_exp=60):
        return int(self.lib.vxo_div_const_mismatches(float(np.float32(d)), count, seed, lo_exp, hi_exp))

    def round_i8(self, v):
        return int(self.lib.vxo_round_i8(float(np.float32(v))))

    def round_ties_even(self, v):
        return int(self.lib.vxo_round_ties_even(float(np.float32(v))))

    def multiplier(self, i, w, o):
        out = C.c_float(0)
        ok = self.lib.vxo_multiplier(float(np.float32(i)), float(np.float32(w)),
                                     float(np.float32(o)), C.byref(out))
        return (np.float32(out.value) if ok else None)

    def quantize_rows(self, x):
        x = _f32(x)
        rows, k = x.shape
        q = np.zeros((rows, k), np.int8)
        s = np.zeros(rows, np.float32)
        v = np.zeros(rows, np.int32)
        self.lib.vxo_quantize_rows(_p(x, C.c_float), C.c_uint64(rows), C.c_uint32(k),
                                   _p(q, C.c_int8), C.c_uint64(k), _p(s, C.c_float),
                                   _p(v, C.c_int32))
        return q, s, v

    def gemm_i32(self, q, w):
        q = np.ascontiguousarray(q, np.int8)
        w = np.ascontiguousarray(w, np.int8)
        rows, k = q.shape
        n = w.shape[0]
        acc = np.zeros((rows, n), np.int32)
        ok = self.lib.vxo_gemm_i32(_p(q, C.c_int8), C.c_uint64(k), _p(w, C.c_int8),
                                   C.c_uint64(k), C.c_uint64(rows), C.c_uint32(k),
                                   C.c_uint32(n), _p(acc, C.c_int32))
        if not ok:
            raise OverflowError("accumulator left int32 range")
        return acc

    def dequant_bias(self, acc, row_scales, valid, ws, bias):
        acc = np.ascontiguousarray(acc, np.int32)
        rows, n = acc.shape
        y = np.zeros((rows, n), np.float32)
        rs, wsc = _f32(row_scales), _f32(ws)
        va = np.ascontiguousarray(valid, np.int32) if valid is not None else None
        b = _f32(bias) if bias is not None else None
        self.lib.vxo_dequant_bias_f32(_p(acc, C.c_int32), C.c_uint64(rows), C.c_uint32(n),
                                      _p(rs, C.c_float), _p(va, C.c_int32), _p(wsc, C.c_float),
                                      _p(b, C.c_float), _p(y, C.c_float))
        return y

    def requant_rows(self, acc, row_scales, valid, ws, bias_i32, out_scale, out_zero,
                     unsigned=False):
        acc = np.ascontiguousarray(acc, np.int32)
        rows, n = acc.shape
        out = np.zeros((rows, n), np.uint8)
        rs, wsc = _f32(row_scales), _f32(ws)
        va = np.ascontiguousarray(valid, np.int32) if valid is not None else None
        b = np.ascontiguousarray(bias_i32, np.int32) if bias_i32 is not None else None
        ok = self.lib.vxo_requant_rows(_p(acc, C.c_int32), C.c_uint64(rows), C.c_uint32(n),
                                       _p(rs, C.c_float), _p(va, C.c_int32),
                                       _p(wsc, C.c_float), _p(b, C.c_int32),
                                       C.c_float(out_scale), C.c_int32(out_zero),
                                       C.c_int(1 if unsigned else 0), _p(out, C.c_uint8))
        if not ok:
            return None
        return out if unsigned else out.view(np.int8)

    def packed_linear_w8_grouped(self, x, words, scales, group, bias):
        x = _f32(x)
        rows, k = x.shape
        words = np.ascontiguousarray(words).view(np.uint32)
        n = words.shape[0]
        sc = _f32(scales)
        b = _f32(bias) if bias is not None else None
        y = np.zeros((rows, n), np.float32)
        st = self.lib.vxo_packed_linear_w8_grouped(
            _p(x, C.c_float), C.c_uint64(rows), C.c_uint32(k), C.c_uint32(n),
            _p(words, C.c_uint32), _p(sc, C.c_float), C.c_uint32(group),
            _p(b, C.c_float), _p(y, C.c_float))
        if st != 0:
            raise ValueError("oracle refused the packed linear")
        return y

    def packed_linear_w4_grouped(self, x, words, scales, group, bias):
        x = _f32(x)
        rows, k = x.shape
        words = np.ascontiguousarray(words).view(np.uint32)
        n = words.shape[0]
        sc = _f32(scales)
        b = _f32(bias) if bias is not None else None
        y = np.zeros((rows, n), np.float32)
        st = self.lib.vxo_packed_linear_w4_grouped(
            _p(x, C.c_float), C.c_uint64(rows), C.c_uint32(k), C.c_uint32(n),
            _p(words, C.c_uint32), _p(sc, C.c_float), C.c_uint32(group),
            _p(b, C.c_float), _p(y, C.c_float))
        if st != 0:
            raise ValueError("oracle refused the packed linear")
        return y

    def qlinear_i8u8(self, x, w, bias, ws, wz, in_scale, in_zero, out_scale, out_zero,
                     out_unsigned=False):
        x = np.ascontiguousarray(x)
        w = np.ascontiguousarray(w)
        rows, k = x.shape
        n = w.shape[0]
        out = np.zeros((rows, n), np.uint8 if out_unsigned else np.int8)
        b = np.ascontiguousarray(bias, np.int32)
        wsc = _f32(ws)
        z = np.ascontiguousarray(wz, np.int32)
        ok = self.lib.vxo_qlinear_i8u8(
            x.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p), _p(b, C.c_int32),
            _p(wsc, C.c_float), _p(z, C.c_int32), out.ctypes.data_as(C.c_void_p),
            C.c_uint32(rows), C.c_uint32(k), C.c_uint32(n), C.c_float(in_scale),
            C.c_int32(in_zero), C.c_float(out_scale), C.c_int32(out_zero),
            C.c_int(x.dtype == np.uint8), C.c_int(w.dtype == np.uint8),
            C.c_int(1 if out_unsigned else 0))
        return out if ok else None

    def rmsnorm_rows(self, x, weight, eps):
        x, weight = _f32(x), _f32(weight)
        y = np.zeros_like(x)
        self.lib.vxo_rmsnorm_rows.restype = None
        self.lib.vxo_rmsnorm_rows(_p(x, C.c_float), _p(weight, C.c_float), _p(y, C.c_float), C.c_uint32(x.shape[0]),
                                  C.c_uint32(x.shape[1]), C.c_double(float(np.float32(eps))))
        return y

    def quantize_linear(self, x, scale, zero, out_unsigned=False):
        x = _f32(x).reshape(-1)
        out = np.zeros(x.size, np.uint8 if out_unsigned else np.int8)
        ok = self.lib.vxo_quantize_linear(_p(x, C.c_float), C.c_uint64(x.size), C.c_float(scale), C.c_int32(zero),
                                          C.c_int(1 if out_unsigned else 0), out.ctypes.data_as(C.c_void_p))
        return out if ok else None

    def dequantize_linear(self, x, scale, zero):
        x = np.ascontiguousarray(x).reshape(-1)
        out = np.zeros(x.size, np.float32)
        self.lib.vxo_dequantize_linear(x.ctypes.data_as(C.c_void_p), C.c_uint64(x.size), C.c_float(scale),
                                       C.c_int32(zero), C.c_int(1 if x.dtype == np.uint8 else 0), _p(out, C.c_float))
        return out

    def requantize_linear(self, x, in_scale, in_zero, out_scale, out_zero, out_unsigned=False):
        x = np.ascontiguousarray(x).reshape(-1)
        out = np.zeros(x.size, np.uint8 if out_unsigned else np.int8)
        ok = self.lib.vxo_requantize_linear(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
                                            C.c_uint64(x.size), C.c_float(in_scale), C.c_int32(in_zero),
                                            C.c_float(out_scale), C.c_int32(out_zero),
                                            C.c_int(1 if x.dtype == np.uint8 else 0), C.c_int(1 if out_unsigned else 0))
        return out if ok else None

    def w8a8_linear(self, x, w, ws, bias=None, bias_i32=None, out_scale=1.0, out_zero=0,
                    requant=False):
        """Whole op on the CPU (quantize -> int32 GEMM -> E1/E2)."""
        x = _f32(x)
        w = np.ascontiguousarray(w, np.int8)
        rows, k = x.shape
        n = w.shape[0]
        q = np.zeros((rows, k), np.int8)
        acc = np.zeros((rows, n), np.int32)
        rs = np.zeros(rows, np.float32)
        va = np.zeros(rows, np.int32)
        out = np.zeros((rows, n), np.int8 if requant else np.float32)
        wsc = _f32(ws)
        b = _f32(bias) if bias is not None else None
        bi = np.ascontiguousarray(bias_i32, np.int32) if bias_i32 is not None else None
        ok = self.lib.vxo_w8a8_linear(
            _p(x, C.c_float), C.c_uint64(rows), C.c_uint32(k), C.c_uint32(n),
            _p(w, C.c_int8), _p(wsc, C.c_float), _p(b, C.c_float), _p(bi, C.c_int32),
            C.c_float(out_scale), C.c_int32(out_zero), C.c_int(1 if requant else 0),
            _p(q, C.c_int8), _p(acc, C.c_int32), _p(rs, C.c_float), _p(va, C.c_int32),
            out.ctypes.data_as(C.c_void_p))
        if not ok:
            return None
        return {"q": q, "acc": acc, "row_scales": rs, "valid": va, "out": out}


class Ref:
    """The reference's own CPU kernels (oracle/_ref/libvxref.so)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self):
        if not self.available():
            raise FileNotFoundError(REF_SO)
        L = self.lib = C.CDLL(REF_SO)
        L.ref_round_i8.restype = C.c_int32
        L.ref_round_i8.argtypes = [C.c_float]
        L.ref_round_ties_even.restype = C.c_int32
        L.ref_round_ties_even.argtypes = [C.c_float]
        L.ref_dot_i8.restype = C.c_int32
        L.ref_isa_name.restype = C.c_char_p
        L.ref_packed_q8_size.restype = C.c_uint32
        L.ref_multiplier.argtypes = [C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]
        L.ref_requantize_accumulator.restype = C.c_int32
        L.ref_requantize_accumulator.argtypes = [C.c_int64, C.c_float, C.c_int32,
                                                 C.c_int32, C.c_int32]

    def isa(self) -> str:
        return self.lib.ref_isa_name().decode()

    def round_i8(self, v):
        return int(self.lib.ref_round_i8(float(np.float32(v))))

    def round_ties_even(self, v):
        return int(self.lib.ref_round_ties_even(float(np.float32(v))))

    def multiplier(self, i, w, o):
        out = C.c_float(0)
        ok = self.lib.ref_multiplier(float(np.float32(i)), float(np.float32(w)),
                                     float(np.float32(o)), C.byref(out))
        return np.float32(out.value) if ok else None

    def requantize_accumulator(self, acc, mult, oz, lo, hi):
        return int(self.lib.ref_requantize_accumulator(int(acc), float(np.float32(mult)),
                                                       int(oz), int(lo), int(hi)))

    def prepare_i8(self, row):
        row = _f32(row)
        k = row.shape[0]
        q = np.zeros(k, np.int8)
        s = C.c_float(0)
        finite = self.lib.ref_prepare_i8(_p(row, C.c_float), C.c_uint32(k), _p(q, C.c_int8),
                                         C.byref(s))
        return q, np.float32(s.value), int(finite)

    def quantize_rows(self, x):
        x = _f32(x)
        rows, k = x.shape
        q = np.zeros((rows, k), np.int8)
        s = np.zeros(rows, np.float32)
        v = np.zeros(rows, np.int32)
        for r in range(rows):
            q[r], s[r], v[r] = self.prepare_i8(x[r])
        return q, s, v

    def prepare_rows(self, x, q=None, scales=None):
        """Quantize every row (threaded through the reference's pool when a scope is open)."""
        x = _f32(x)
        rows, k = x.shape
        q = np.zeros((rows, k), np.int8) if q is None else q
        scales = np.zeros(rows, np.float32) if scales is None else scales
        self.lib.ref_prepare_rows(_p(x, C.c_float), C.c_uint32(rows), C.c_uint32(k),
                                  _p(q, C.c_int8), _p(scales, C.c_float))
        return q, scales

    def dot_i8(self, q, words, count, bits=8):
        q = np.ascontiguousarray(q, np.int8)
        words = np.ascontiguousarray(words).view(np.uint32)
        return int(self.lib.ref_dot_i8(_p(q, C.c_int8), _p(words, C.c_uint32),
                                       C.c_uint32(count), C.c_uint32(bits)))

    def packed_linear(self, x, words, scales, group, bias, bits=8, first_unit=0, unit_count=0,
                      y=None):
        x = _f32(x)
        rows, k = x.shape
        words = np.ascontiguousarray(words).view(np.uint32)
        n = words.shape[0]
        sc = _f32(scales)
        b = _f32(bias) if bias is not None else None
        if y is None:
            y = np.zeros((rows, n), np.float32)
        st = self.lib.ref_packed_linear(
            _p(x, C.c_float), C.c_uint32(rows), C.c_uint32(k), C.c_uint32(n),
            _p(words, C.c_uint32), _p(sc, C.c_float), C.c_uint32(group), C.c_uint32(bits),
            _p(b, C.c_float), _p(y, C.c_float), C.c_uint64(first_unit), C.c_uint64(unit_count))
        if st != 0:
            raise ValueError("reference refused the packed linear")
        return y

    def _dt(self, a):
        return DT_U8 if a.dtype == np.uint8 else DT_I8

    def qlinear_portable(self, x, w, bias, ws, wz, in_scale, in_zero, out_scale, out_zero,
                         out_unsigned=False):
        x, w = np.ascontiguousarray(x), np.ascontiguousarray(w)
        rows, k = x.shape
        n = w.shape[0]
        out = np.zeros((rows, n), np.uint8 if out_unsigned else np.int8)
        b = np.ascontiguousarray(bias, np.int32)
        wsc = _f32(ws)
        z = np.ascontiguousarray(wz, np.int32)
        ok = self.lib.ref_qlinear_portable(
            x.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p), _p(b, C.c_int32),
            _p(wsc, C.c_float), _p(z, C.c_int32), out.ctypes.data_as(C.c_void_p),
            C.c_uint32(rows), C.c_uint32(k), C.c_uint32(n), C.c_float(in_scale),
            C.c_int32(in_zero), C.c_float(out_scale), C.c_int32(out_zero),
            C.c_uint32(self._dt(x)), C.c_uint32(self._dt(w)), C.c_uint32(self._dt(out)))
        return out if ok else None

    def rmsnorm_rows(self, x, weight, eps):
        x, weight = _f32(x), _f32(weight)
        y = np.zeros_like(x)
        self.lib.ref_rmsnorm_rows.restype = None
        self.lib.ref_rmsnorm_rows(_p(x, C.c_float), _p(weight, C.c_float), _p(y, C.c_float), C.c_uint32(x.shape[0]),
                                  C.c_uint32(x.shape[1]), C.c_double(float(np.float32(eps))))
        return y

    def quantize_linear(self, x, scale, zero, out_unsigned=False):
        x = _f32(x).reshape(-1)
        out = np.zeros(x.size, np.uint8 if out_unsigned else np.int8)
        ok = self.lib.ref_quantize_linear(_p(x, C.c_float), C.c_uint32(x.size), C.c_float(scale), C.c_int32(zero),
                                          C.c_uint32(self._dt(out)), out.ctypes.data_as(C.c_void_p))
        return out if ok else None

    def dequantize_linear(self, x, scale, zero):
        x = np.ascontiguousarray(x).reshape(-1)
        out = np.zeros(x.size, np.float32)
        ok = self.lib.ref_dequantize_linear(x.ctypes.data_as(C.c_void_p), C.c_uint32(x.size), C.c_float(scale),
                                            C.c_int32(zero), C.c_uint32(self._dt(x)), _p(out, C.c_float))
        return out if ok else None

    def requantize_linear(self, x, in_scale, in_zero, out_scale, out_zero, out_unsigned=False):
        x = np.ascontiguousarray(x).reshape(-1)
        out = np.zeros(x.size, np.uint8 if out_unsigned else np.int8)
        ok = self.lib.ref_requantize_linear(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p),
                                            C.c_uint32(x.size), C.c_float(in_scale), C.c_int32(in_zero),
                                            C.c_float(out_scale), C.c_int32(out_zero),
                                            C.c_uint32(self._dt(x)), C.c_uint32(self._dt(out)))
        return out if ok else None

    def pack_q8(self, w):
        w = np.ascontiguousarray(w)
        n, k = w.shape
        size = int(self.lib.ref_packed_q8_size(C.c_uint32(k), C.c_uint32(n)))
        buf = np.zeros(size + 64, np.uint8)
        off = (-buf.ctypes.data) % 64
        packed = buf[off:off + size]
        ok = self.lib.ref_pack_q8(packed.ctypes.data_as(C.c_void_p), C.c_uint32(size),
                                  w.ctypes.data_as(C.c_void_p), C.c_uint32(k), C.c_uint32(n),
                                  C.c_uint32(self._dt(w)))
        if not ok:
            raise ValueError("reference refused to pack the weight")
        return packed

    def qlinear_packed(self, x, packed, w_dtype, n, bias, ws, wz, in_scale, in_zero, out_scale,
                       out_zero, out=None, out_unsigned=False):
        x = np.ascontiguousarray(x)
        rows, k = x.shape
        if out is None:
            out = np.zeros((rows, n), np.uint8 if out_unsigned else np.int8)
        b = np.ascontiguousarray(bias, np.int32)
        wsc = _f32(ws)
        z = np.ascontiguousarray(wz, np.int32)
        ok = self.lib.ref_qlinear_packed(
            x.ctypes.data_as(C.c_void_p), packed.ctypes.data_as(C.c_void_p), _p(b, C.c_int32),
            _p(wsc, C.c_float), _p(z, C.c_int32), out.ctypes.data_as(C.c_void_p),
            C.c_uint32(rows), C.c_uint32(k), C.c_uint32(n), C.c_float(in_scale),
            C.c_int32(in_zero), C.c_float(out_scale), C.c_int32(out_zero),
            C.c_uint32(self._dt(x)), C.c_uint32(DT_U8 if w_dtype == np.uint8 else DT_I8),
            C.c_uint32(self._dt(out)))
        return out if ok else None

    def threads_enter(self, t):
        return int(self.lib.ref_threads_enter(C.c_int(t)))

    def threads_leave(self):
        self.lib.ref_threads_leave()
