"""Device residency behind the reference-facing host entries.

The reference's CUDA backend uploads an input only when its host copy is newer and leaves outputs on
the device until the host needs them (native/src/backends/cuda/host/cuda_graph_memory_host.inc:
1302-1310).  With vxb_host_residency(1) a chain of nodes bound through the host-pointer entries does
the same: intermediates never reach the host, results are byte-identical to the upload/download-
every-call form, and the ownership rule (download before reading, invalidate after writing) holds."""
import numpy as np
import pytest

from volvoxai_b200 import w8a8

pytestmark = pytest.mark.gpu

SENTINEL_I8, SENTINEL_F32 = -77, -12345.5


@pytest.fixture(autouse=True)
def _fresh_host_state():
    w8a8.host_cache_clear()
    yield
    w8a8.host_residency(False)
    w8a8.host_cache_clear()


def _island(rng, rows=96, k=192, h=320, n=136):
    x = (rng.standard_normal((rows, k)) * 1.7).astype(np.float32)
    w1 = rng.integers(-127, 128, (h, k), dtype=np.int8)
    w2 = rng.integers(-127, 128, (n, h), dtype=np.int8)
    s1 = rng.uniform(0.002, 0.01, h).astype(np.float32)
    s2 = rng.uniform(0.002, 0.01, n).astype(np.float32)
    b1 = rng.integers(-500, 500, h, dtype=np.int32)
    b2 = rng.integers(-500, 500, n, dtype=np.int32)
    return x, (w1, s1, b1), (w2, s2, b2)


def _run_island(x, l1, l2, bufs):
    """QuantizeLinear -> QLinear -> QLinear -> DequantizeLinear through the host entries."""
    q, h, o, y = bufs
    (w1, s1, b1), (w2, s2, b2) = l1, l2
    z1, z2 = np.zeros(len(s1), np.int32), np.zeros(len(s2), np.int32)
    assert w8a8.quantize_typed_f32_i8u8(x, q, 0.05, 3) == 1
    assert w8a8.qlinear_i8u8(q, w1, s1, z1, b1, h, 0.05, 3, 0.9, -4) == 1
    assert w8a8.qlinear_i8u8(h, w2, s2, z2, b2, o, 0.9, -4, 1.3, 5) == 1
    assert w8a8.dequantize_typed_i8u8_f32(o, 1.3, 5, y) == 1


def _buffers(x, l1, l2):
    rows = x.shape[0]
    return (np.full(x.shape, SENTINEL_I8, np.int8), np.full((rows, len(l1[1])), SENTINEL_I8, np.int8),
            np.full((rows, len(l2[1])), SENTINEL_I8, np.int8), np.full((rows, len(l2[1])), SENTINEL_F32, np.float32))


def test_chain_keeps_intermediates_on_the_device_and_matches_the_eager_form():
    rng = np.random.default_rng(41)
    x, l1, l2 = _island(rng)
    want = _buffers(x, l1, l2)
    _run_island(x, l1, l2, want)                    # residency off: every tensor reaches the host
    assert not (want[1] == SENTINEL_I8).all()

    assert w8a8.host_residency(True) == 1
    got = _buffers(x, l1, l2)
    _run_island(x, l1, l2, got)
    for a in got:                                    # nothing was downloaded: host copies are stale
        assert (a == (SENTINEL_F32 if a.dtype == np.float32 else SENTINEL_I8)).all()
    assert w8a8.host_download(got[3]) == 1           # the island's output only
    np.testing.assert_array_equal(got[3], want[3])
    assert (got[1] == SENTINEL_I8).all() and (got[2] == SENTINEL_I8).all()
    assert w8a8.host_download(None) == 1             # everything
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    # a second pass over the same buffers reuses the device tensors and gives the same bytes
    _run_island(x * 0.5, l1, l2, got)
    _run_island(x * 0.5, l1, l2, want)               # (residency on: `want` buffers become resident too)
    assert w8a8.host_download(None) == 1
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)


def test_row_window_of_a_resident_tensor_is_read_in_place():
    rng = np.random.default_rng(43)
    x, l1, _ = _island(rng, rows=64)
    w1, s1, b1 = l1
    z1 = np.zeros(len(s1), np.int32)
    q = np.zeros(x.shape, np.int8)
    want = np.zeros((16, len(s1)), np.int8)
    assert w8a8.quantize_typed_f32_i8u8(x, q, 0.05, 0) == 1
    assert w8a8.qlinear_i8u8(q[32:48], w1, s1, z1, b1, want, 0.05, 0, 0.9, 0) == 1

    w8a8.host_residency(True)
    q2 = np.full(x.shape, SENTINEL_I8, np.int8)
    got = np.zeros_like(want)
    assert w8a8.quantize_typed_f32_i8u8(x, q2, 0.05, 0) == 1
    assert (q2 == SENTINEL_I8).all()
    assert w8a8.qlinear_i8u8(q2[32:48], w1, s1, z1, b1, got, 0.05, 0, 0.9, 0) == 1   # interior pointer
    assert w8a8.host_download(got) == 1
    np.testing.assert_array_equal(got, want)
    assert w8a8.host_download(q2[40:41]) == 1          # any address inside the tensor names it
    np.testing.assert_array_equal(q2, q)
    assert w8a8.host_download(np.zeros(4, np.int8)) == 0 and "no resident tensor" in w8a8.last_error()


def test_plain_host_inputs_are_uploaded_every_call_and_invalidate_drops_device_copies():
    rng = np.random.default_rng(47)
    x = rng.standard_normal(4096).astype(np.float32)
    q = np.zeros(4096, np.int8)
    w8a8.host_residency(True)
    assert w8a8.quantize_typed_f32_i8u8(x, q, 0.05, 0) == 1
    x *= 2.0                                           # the host rewrites a plain input: no announcement needed
    assert w8a8.quantize_typed_f32_i8u8(x, q, 0.05, 0) == 1
    assert w8a8.host_download(q) == 1
    want = np.zeros(4096, np.int8)
    w8a8.host_residency(False)
    assert w8a8.quantize_typed_f32_i8u8(x, want, 0.05, 0) == 1
    np.testing.assert_array_equal(q, want)

    # the host overwrites a tensor the library produced: invalidate, then the new host bytes are what is read
    w8a8.host_residency(True)
    f = np.zeros(4096, np.float32)
    assert w8a8.quantize_typed_f32_i8u8(x, q, 0.05, 0) == 1
    q[:] = 7
    assert w8a8.host_invalidate(q) == 1
    assert w8a8.dequantize_typed_i8u8_f32(q, 0.5, 0, f) == 1
    assert w8a8.host_download(f) == 1
    np.testing.assert_array_equal(f, np.full(4096, 3.5, np.float32))


def test_leaving_residency_brings_every_output_home_and_partial_windows_write_through():
    rng = np.random.default_rng(53)
    rows, k, n = 12, 256, 96
    x = rng.standard_normal((rows, k)).astype(np.float32)
    words = rng.integers(-127, 128, (n, k), dtype=np.int8).view(np.int32)
    scales = rng.uniform(0.002, 0.01, (n, k // 128)).astype(np.float32)
    want = np.zeros((rows, n), np.float32)
    assert w8a8.packed_linear(x, words, scales, None, want) == 1

    w8a8.host_residency(True)
    y = np.full((rows, n), SENTINEL_F32, np.float32)
    assert w8a8.packed_linear(x, words, scales, None, y) == 1
    assert (y == SENTINEL_F32).all()
    # a one-row window (the generation path's last row) is written to the host at once and first
    # brings the resident tensor home, so the rows outside the window are current too
    assert w8a8.packed_linear(x, words, scales, None, y, first_unit=(rows - 1) * n, unit_count=n) == 1
    np.testing.assert_array_equal(y, want)

    y2 = np.full((rows, n), SENTINEL_F32, np.float32)
    assert w8a8.packed_linear(x, words, scales, None, y2) == 1
    assert (y2 == SENTINEL_F32).all()
    assert w8a8.host_residency(False) == 1             # leaving the mode downloads what is still device-dirty
    np.testing.assert_array_equal(y2, want)
