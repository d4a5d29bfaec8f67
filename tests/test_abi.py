"""CPU-only checks of the drop-in boundary: the shared library loads, exports every
symbol the public header declares, mirrors the reference descriptor layout, and its
admission rules decline (return 0) without touching a device."""
import ctypes as C
import os
import re

import numpy as np

from volvoxai_b200 import _lib, w8a8
from tests import workloads as wl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(*path):
    text = open(os.path.join(ROOT, *path)).read()
    return sorted(set(re.findall(r"VXB_(?:PLAN_)?API[^;(]*?\b(vxb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    """The boundary header, the planning header and the diagnostic header: every declared entry is
    exported by the built library, and the ctypes mirror lists exactly those names."""
    L = _lib.load()
    names = declared_symbols("include", "vxb200_w8a8.h")
    assert len(names) >= 20
    plan = declared_symbols("include", "vxb200_plan.h")
    package = declared_symbols("include", "vxb200_package.h")
    assert sorted(_lib.PACKAGE_EXPORTS) == package
    diag = declared_symbols("volvoxai_b200", "csrc", "diag.h")
    for n in names + plan + package + diag:
        assert hasattr(L, n), n
    assert sorted(_lib.EXPORTS) == names
    assert sorted(_lib.PLAN_EXPORTS) == plan
    assert sorted(_lib.DIAG_EXPORTS) == diag
    assert not set(diag) & set(names), "diagnostics leaked into the boundary header"
    assert L.vxb_abi_version() == 1


def test_descriptor_layout_matches_reference_struct():
    # sizeof(VxLLMOpArgs) == 336, x at 104, first_unit at 320 on LP64
    # (native/src/kernels/llm_ops.h:38-53)
    assert C.sizeof(_lib.LLMOpArgs) == 336
    assert _lib.LLMOpArgs.x.offset == 104
    assert _lib.LLMOpArgs.first_unit.offset == 320
    assert _lib.LLMOpArgs.unit_count.offset == 328


def test_packed_linear_admission_declines_on_host():
    x = np.zeros((2, 64), np.float32)
    w = np.zeros((4, 64), np.int8)
    words = wl.pack_w8_words(w)
    scales = np.ones((4, 1), np.float32)
    y = np.full((2, 4), 7.0, np.float32)
    # W2 / W3 storage and A16 / F32 arithmetic stay with the reference's own routes (W4 and W8 with
    # A8 arithmetic are admitted); so does a group size outside 32..256
    assert w8a8.packed_linear(x, words, scales, None, y, weight_bits=2, group_size=64) == 0
    assert w8a8.packed_linear(x, words, scales, None, y, weight_bits=3, group_size=64) == 0
    assert w8a8.packed_linear(x, words, scales, None, y, group_size=48) == 0
    assert w8a8.packed_linear(x, words, scales, None, y, activation_bits=16, group_size=64) == 0
    assert w8a8.packed_linear(x, words, scales, None, y, activation_bits=32, group_size=64) == 0
    # ragged window, window past the end, first_unit without a count
    assert w8a8.packed_linear(x, words, scales, None, y, group_size=64, first_unit=1, unit_count=4) == 0
    assert w8a8.packed_linear(x, words, scales, None, y, group_size=64, first_unit=4, unit_count=8) == 0
    assert w8a8.packed_linear(x, words, scales, None, y, group_size=64, first_unit=4, unit_count=0) == 0
    # an output window that overlaps a source is declined as the reference's entry declines it
    both = np.zeros(2 * 64 + 2 * 4, np.float32)
    assert w8a8.packed_linear(both[:128].reshape(2, 64), words, scales, None, both[124:132].reshape(2, 4), group_size=64) == 0
    assert "overlap" in w8a8.last_error()
    assert (y == 7.0).all()  # declined before touching the output


def test_qlinear_admission_declines_on_host():
    x = np.zeros((2, 8), np.int8)
    w = np.zeros((3, 8), np.int8)
    ws = np.ones(3, np.float32)
    z = np.zeros(3, np.int32)
    out = np.full((2, 3), 9, np.int8)
    assert w8a8.qlinear_i8u8(x, w.view(np.uint8), ws, z, z, out, 1.0, 0, 1.0, 0) == 0  # U8 weights
    assert w8a8.qlinear_i8u8(x, w, ws, np.array([0, 1, 0], np.int32), z, out, 1.0, 0, 1.0, 0) == 0
    both = np.zeros(2 * 8 + 2 * 3, np.int8)
    xin, alias = both[:16].reshape(2, 8), both[12:18].reshape(2, 3)
    assert w8a8.qlinear_i8u8(xin, w, ws, z, z, alias, 1.0, 0, 1.0, 0) == 0  # output overlaps input
    assert (out == 9).all()
