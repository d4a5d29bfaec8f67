"""The reference's own parity matrix for PackedLinear, driven through the drop-in for
cuda_graph_llm_f32 (host pointers, tri-state return) and compared bit for bit with the
reference's CPU forward (oracle/_ref, compiled from the reference's sources; the restated oracle
stands in where that library is absent).

Mirrored cases:
  * the 76 generated boundary cases of tools/packed_linear_cases.py:65-86 (row counts around the
    tile sizes 4..64, K = G-1 / G / G+1, N = 3 / 4 / 5, every weight width and group size);
  * the whole-operator width list x N {1,3,4,5,13,19} x group size x input mode of
    native/tests/test_packed_linear_i8.c:207-285, with its partial output windows;
  * the row counts {1,...,66,128,130,402} of native/tests/test_packed_linear_i8.c:403-470.
Weight widths 8 and 4 are served (A8 arithmetic); widths 2 and 3 must be declined with the output
untouched, so that the reference's own routes keep serving them.  Group scales are random per
group, so every case takes the exact per-group arithmetic.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TILES = (4, 8, 16, 32, 64)
GROUPS = (32, 64, 128, 256)
WIDTHS = [1, 2, 3, 7, 8, 9, 10, 11, 15, 16, 17, 21, 22, 23, 24, 25, 31, 32, 33, 39, 40, 41, 47, 48, 49, 55, 56, 57,
          63, 64, 65, 255, 256, 257, 320, 1280, 1283]
COLUMNS = [1, 3, 4, 5, 13, 19]
ROW_COUNTS = [1, 2, 3, 4, 6, 7, 8, 10, 16, 17, 31, 32, 33, 63, 64, 65, 66, 128, 130, 402]


@pytest.fixture(scope="module")
def torch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


@pytest.fixture(scope="module")
def truth(oracle):
    """(x, words, scales, group, bias, bits) -> fp32 [rows, n] of the reference's forward."""
    from oracle.bindings import Ref
    if Ref.available():
        ref = Ref()
        return lambda x, words, scales, group, bias, bits: ref.packed_linear(x, words, scales, group, bias, bits=bits)

    def restated(x, words, scales, group, bias, bits):
        fn = oracle.packed_linear_w8_grouped if bits == 8 else oracle.packed_linear_w4_grouped
        return fn(x, words, scales, group, bias)
    return restated


def generated_boundaries():
    """Restatement of generated_boundaries() (tools/packed_linear_cases.py:65-86): tuples
    (family, rows, k, n, bits, group)."""
    cases = []
    rows = {1, 2, *(tile + offset for tile in TILES for offset in (-1, 0, 1, 2, 3))}
    cases += [("row_boundaries", r, 2 * GROUPS[0], 8, 4, 32) for r in sorted(rows)]
    for r in (2, 5):
        for k in (GROUPS[0] - 1, GROUPS[0], GROUPS[0] + 1):
            for n in (3, 4, 5):
                cases.append(("tails", r, k, n, 4, 32))
    for bits in (2, 3, 4, 8):
        for r in (2, 8):
            cases.append(("bit_controls", r, 2 * GROUPS[0], 8, bits, 32))
    for group in GROUPS:
        for k in (group - 1, group, group + 1):
            for r in (2, 17):
                cases.append(("group_controls", r, k, 8, 4, group))
    return sorted(cases)


def random_package(rng, k, n, bits, group):
    """Random codes as canonical PackedLinear words (padding = the encoded zero) + random positive
    group scales of the reference's test recipe ((1 + r % 101) * 0.00013)."""
    per_word = 32 // bits
    row_words = (k * bits + 31) // 32
    codes = rng.integers(0, 1 << bits, size=(n, row_words * per_word), dtype=np.uint32)
    codes[:, k:] = 1 << (bits - 1)
    shifts = (np.arange(per_word, dtype=np.uint32) * np.uint32(bits))
    words = (codes.reshape(n, row_words, per_word) << shifts).sum(axis=2, dtype=np.uint32)
    groups = (k + group - 1) // group
    scales = ((1 + rng.integers(0, 101, size=(n, groups))) * 0.00013).astype(np.float32)
    return np.ascontiguousarray(words.view(np.int32)), scales


def reference_inputs(rng, rows, k, mode):
    """Input rows of the reference's whole-operator test (test_packed_linear_i8.c:219-233): integer
    grids at two scales, a zero row, a subnormal row, a huge row, half-integer ties; mode 1 adds
    NaN / -Inf / +Inf rows, mode 2 is all +-0."""
    x = np.empty((rows, k), np.float32)
    j = np.arange(k)
    for r in range(rows):
        scale = np.float32(0.0073 if r % 2 else 0.125)
        x[r] = (rng.integers(0, 255, size=k) - 127).astype(np.float32) * scale
        x[r, 0] = np.float32(127.0) * scale
        if r == 1:
            x[r] = 0.0
        if r == 2:
            x[r] = (j % 9 - 4).astype(np.float32) * np.float32(2.0 ** -148)
        if r == 3:
            x[r] = (j % 255 - 127).astype(np.float32) * np.float32(2.0 ** 120)
        if r == 4:
            x[r] = np.where(j == 0, 127.0, (j % 19) - 9.5).astype(np.float32)
    if mode == 1:
        x[2 % rows, 0] = np.nan
        if rows > 8:
            x[7, 0], x[8, 0] = -np.inf, np.inf
    if mode == 2:
        x[:] = np.where((np.arange(rows * k) % 2).reshape(rows, k) == 1, -0.0, 0.0).astype(np.float32)
    return x


def same_bits(got, want):
    nan = np.isnan(want)
    return np.array_equal(np.isnan(got), nan) and np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


class Keeper:
    """Host arrays stay alive until the cached weights keyed by their addresses are dropped."""

    def __init__(self):
        self.alive = []

    def keep(self, *arrays):
        from volvoxai_b200 import w8a8
        self.alive.append(arrays)
        if len(self.alive) >= 128:
            w8a8.host_cache_clear()
            self.alive.clear()


def test_generated_boundary_cases(torch, truth):
    from volvoxai_b200 import w8a8
    w8a8.host_cache_clear()
    cases = generated_boundaries()
    assert len(cases) == 76
    rng = np.random.default_rng(20261027)
    keeper = Keeper()
    served = 0
    for family, rows, k, n, bits, group in cases:
        words, scales = random_package(rng, k, n, bits, group)
        x = rng.normal(0, 0.2, (rows, k)).astype(np.float32)
        x[0] = 0
        if rows > 2:
            x[-1, 0] = np.nan
        if rows > 4:
            x[1] *= np.float32(2.0 ** -120)
        bias = rng.normal(0, 0.02, n).astype(np.float32)
        y = np.full((rows, n), 12345.0, np.float32)
        rc = w8a8.packed_linear(x, words, scales, bias, y, weight_bits=bits, group_size=group)
        if bits in (2, 3):
            assert rc == 0 and (y == 12345.0).all(), (family, rows, k, n, bits, group)
        else:
            assert rc == 1, (family, rows, k, n, bits, group, w8a8.last_error())
            assert same_bits(y, truth(x, words, scales, group, bias, bits)), (family, rows, k, n, bits, group)
            served += 1
        keeper.keep(x, words, scales, bias, y)
    assert served == 72
    w8a8.host_cache_clear()


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("group", GROUPS)
def test_whole_operator_widths_columns_modes_and_windows(torch, truth, bits, group):
    from volvoxai_b200 import w8a8
    w8a8.host_cache_clear()
    rng = np.random.default_rng(bits * 1000 + group)
    keeper = Keeper()
    rows = 11
    for k in WIDTHS:
        for n in COLUMNS:
            words, scales = random_package(rng, k, n, bits, group)
            bias_all = ((np.arange(n) - 9) * 0.03125).astype(np.float32)
            for mode in range(3):
                x = reference_inputs(rng, rows, k, mode)
                bias = None if mode == 2 else bias_all
                want = truth(x, words, scales, group, bias, bits)
                # the five output windows of the reference's test: everything, three ragged ones
                # (declined here with the output untouched) and one of whole rows
                for first, count in ((0, 0), (1, rows * n - 2), (n - 1, 4 * n + 2), (n + 2, 3 * n - 2), (n, 8 * n)):
                    y = np.full((rows, n), 12345.0, np.float32)
                    rc = w8a8.packed_linear(x, words, scales, bias, y, weight_bits=bits, group_size=group,
                                            first_unit=first, unit_count=count)
                    whole_rows = first % n == 0 and count % n == 0
                    if not whole_rows:
                        assert rc == 0 and (y == 12345.0).all(), (k, n, mode, first, count)
                        continue
                    assert rc == 1, (k, n, mode, first, count, w8a8.last_error())
                    end = first + (count if count else rows * n)
                    flat, inside = y.reshape(-1), np.zeros(rows * n, bool)
                    inside[first:end] = True
                    assert (flat[~inside] == 12345.0).all(), (k, n, mode, first, count)
                    assert same_bits(flat[inside], want.reshape(-1)[inside]), (k, n, mode, first, count)
                    keeper.keep(y)
                keeper.keep(x)
            keeper.keep(words, scales, bias_all)
    w8a8.host_cache_clear()


@pytest.mark.parametrize("fixture", range(20))
def test_row_counts(torch, truth, fixture):
    """The reference's row-tile fixtures: every storage / group pair at K = 65, N = 8 (widths 2 and 3
    declined), then realistic W4 widths (K 320 and 1283, N 20, group 32) and W3 (declined)."""
    from volvoxai_b200 import w8a8
    w8a8.host_cache_clear()
    bits = (2, 3, 4, 8)[fixture // 4] if fixture < 16 else 4 if fixture < 18 else 3
    group = 32 << (fixture % 4) if fixture < 16 else 32
    k, n = (65, 8) if fixture < 16 else (320 if fixture % 2 == 0 else 1283, 20)
    rng = np.random.default_rng(900 + fixture)
    words, scales = random_package(rng, k, n, bits, group)
    bias = rng.normal(0, 0.5, n).astype(np.float32)
    full = np.empty((402, k), np.float32)
    for r in range(402):
        full[r] = (rng.integers(0, 255, size=k) - 127).astype(np.float32) * np.float32((1 + r % 4) * 0.03125)
    full[5] = 0
    full[9, k // 2] = np.inf
    for rows in ROW_COUNTS:
        x = np.ascontiguousarray(full[:rows])
        y = np.full((rows, n), 12345.0, np.float32)
        rc = w8a8.packed_linear(x, words, scales, bias, y, weight_bits=bits, group_size=group)
        if bits in (2, 3):
            assert rc == 0 and (y == 12345.0).all()
            continue
        assert rc == 1, (rows, w8a8.last_error())
        assert same_bits(y, truth(x, words, scales, group, bias, bits)), rows
    w8a8.host_cache_clear()
