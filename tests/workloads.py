"""Benchmark and test input generators (not part of the product package).

Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations, plus the weight authoring arithmetic that produces
W8A8 packages.  NumPy only; no dataset, checkpoint or reference file is read.

Authoring follows the reference's producer so that the synthetic weights look
like a real package:
  * per-output-channel symmetric int8 (native/src/training/quantization.c:258-306):
    scale = f32(absmax / 127 evaluated in double), 1.0 for an all-zero channel;
    w = ties-to-even(double(v) / double(scale)) clamped to +-127;
  * I32 accumulator-domain bias (native/src/training/quantization.c:391-414):
    b = ties-to-even(f32(bias / f32(input_scale * weight_scale)));
  * W8 PackedLinear words (docs/packed-linear-design.md:24-41): byte j of a
    row's little-endian words holds code = w + 128, final-word padding = 0x80,
    scales [N, ceil(K/G)].
"""
from __future__ import annotations

import functools

import numpy as np

# (K, N) pairs of the configurations
GEMV_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]
GEMV_ROWS = [1, 4, 8, 16, 32]
GEMM_SHAPES = [(4096, 14336), (8192, 28672), (4096, 128256)]
GEMM_ROWS = [2048, 4096, 8192, 16384]
SMOLLM2_LINEARS = {"q": (576, 576), "k": (576, 192), "v": (576, 192), "o": (576, 576),
                   "gate": (576, 1536), "up": (576, 1536), "down": (1536, 576)}
QWEN3_LINEARS = {"q": (1024, 2048), "k": (1024, 1024), "v": (1024, 1024), "o": (2048, 1024),
                 "gate": (1024, 3072), "up": (1024, 3072), "down": (3072, 1024)}


# Linear layers of the two decoder configurations: name -> (K, N); every layer has one of each.
SMOLLM2_135M = {"layers": 30, "rows": 8 * 512,
                "linears": {"q": (576, 576), "k": (576, 192), "v": (576, 192), "o": (576, 576),
                            "gate": (576, 1536), "up": (576, 1536), "down": (1536, 576)}}
QWEN3_0_6B = {"layers": 28, "rows": 64,
              "linears": {"q": (1024, 2048), "k": (1024, 1024), "v": (1024, 1024), "o": (2048, 1024),
                          "gate": (1024, 3072), "up": (1024, 3072), "down": (3072, 1024)}}


def quantize_weight_per_channel(wf: np.ndarray):
    """fp32 [N,K] -> (int8 [N,K], fp32 scales [N]) as the reference's PTQ packer does."""
    wf = np.asarray(wf, np.float32)
    amax = np.abs(wf).max(axis=1).astype(np.float64)
    scale = np.where(amax == 0.0, 1.0, amax / 127.0).astype(np.float32)
    scale = np.where(scale == 0.0, np.finfo(np.float32).tiny, scale).astype(np.float32)
    q = np.rint(wf.astype(np.float64) / scale.astype(np.float64)[:, None])
    return np.clip(q, -127, 127).astype(np.int8), scale


def bias_to_i32(bias: np.ndarray, input_scale: float, ws: np.ndarray) -> np.ndarray:
    acc_scale = (np.float32(input_scale) * np.asarray(ws, np.float32)).astype(np.float32)
    ratio = (np.asarray(bias, np.float32) / acc_scale).astype(np.float32)
    return np.rint(ratio.astype(np.float64)).astype(np.int32)


def pack_w8_words(w: np.ndarray) -> np.ndarray:
    """int8 [N,K] -> uint32 words [N, ceil(K/4)] in offset-binary W8 storage."""
    w = np.asarray(w, np.int8)
    n, k = w.shape
    kw = (k + 3) // 4
    codes = np.full((n, kw * 4), 0x80, np.uint8)
    codes[:, :k] = (w.astype(np.int16) + 128).astype(np.uint8)
    return codes.view("<u4").reshape(n, kw).copy()


def pack_w4_words(w: np.ndarray) -> np.ndarray:
    """int8 weights in [-8, 7] [N,K] -> PackedLinear W4 words [N, ceil(K/8)] (int32): eight codes per
    word, earlier K in lower bits, code = w + 8, padding codes 8 (the encoded zero)."""
    n, k = w.shape
    kw = (k + 7) // 8
    codes = np.full((n, kw * 8), 8, np.uint32)
    codes[:, :k] = (w.astype(np.int32) + 8).astype(np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))
    return (codes.reshape(n, kw, 8) << shifts).sum(axis=2, dtype=np.uint32).view(np.int32)


def group_scales(ws: np.ndarray, k: int, group: int) -> np.ndarray:
    """Per-channel scales expressed as PackedLinear group scales [N, ceil(K/G)]."""
    groups = (k + group - 1) // group
    return np.repeat(np.asarray(ws, np.float32)[:, None], groups, axis=1).copy()


def single_linear(rows=64, k=576, n=1536, seed=0):
    """Configuration 1: x~N(0,1), W~N(0,0.02) per-channel int8, bias~N(0,0.01)."""
    x = np.random.default_rng(seed).standard_normal((rows, k), dtype=np.float32)
    wf = (np.random.default_rng(seed + 1).standard_normal((n, k), dtype=np.float32)
          * np.float32(0.02))
    bias = (np.random.default_rng(seed + 2).standard_normal(n, dtype=np.float32)
            * np.float32(0.01))
    w, ws = quantize_weight_per_channel(wf)
    return {"x": x, "w": w, "ws": ws, "bias": bias}


def gemv_case(rows, k, n, seed=0):
    """Configuration 4: x~N(0,1); int8 weights uniform [-127,127]; scales U(0.001,0.02)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, k), dtype=np.float32)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    return {"x": x, "w": w, "ws": ws, "bias": None}


def gemm_activations(rows, k, seed=0):
    """Configuration 5 activations: N(0,1) with a fixed random 1% of the K channels x20."""
    rng = np.random.default_rng([seed, 0xA])
    x = rng.standard_normal((rows, k), dtype=np.float32)
    outliers = rng.choice(k, size=max(1, k // 100), replace=False)
    x[:, outliers] *= np.float32(20.0)
    return x


@functools.lru_cache(maxsize=1)
def gemm_weights_cached(n, k, seed=0):
    """gemm_weights with the last result kept (read-only use): the multi-hundred-MB shapes take
    seconds to draw and several tests share them."""
    return gemm_weights(n, k, seed)


def gemm_weights(n, k, seed=0):
    """Configuration 5 weights for n output channels, drawn directly as int8 codes with the
    distribution per-channel quantization of N(0,0.02) produces (|code| max pinned at 127,
    scale = channel absmax/127 with absmax ~ 4.2 sigma), without an fp32 master."""
    rng = np.random.default_rng([seed, 0xB])
    w = np.empty((n, k), np.int8)
    step = max(1, (1 << 25) // k)
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        z = rng.standard_normal((hi - lo, k), dtype=np.float32)
        z *= np.float32(127.0 / 4.2)
        np.clip(np.rint(z, out=z), -127, 127, out=z)
        w[lo:hi] = z.astype(np.int8)
    w[:, 0] = 127
    ws = (np.float32(0.02 * 4.2 / 127.0) * rng.uniform(0.9, 1.1, size=n)).astype(np.float32)
    return w, ws


def gemm_case(rows, k, n, seed=0, weights_fast=False):
    """Configuration 5: x~N(0,1) with 1% outlier channels x20; W~N(0,0.02) per channel.
    ``weights_fast`` draws the int8 codes directly (gemm_weights) instead of authoring from
    an fp32 master, for the multi-GB shapes."""
    x = gemm_activations(rows, k, seed)
    if weights_fast:
        w, ws = gemm_weights_cached(n, k, seed)
    else:
        wf = (np.random.default_rng([seed, 0xC]).standard_normal((n, k), dtype=np.float32)
              * np.float32(0.02))
        w, ws = quantize_weight_per_channel(wf)
    return {"x": x, "w": w, "ws": ws, "bias": None}


def static_out_scale(y: np.ndarray) -> np.float32:
    """Static output scale for the requantizing epilogue: 99.9th percentile |y| / 127."""
    finite = np.abs(y[np.isfinite(y)])
    if finite.size == 0:
        return np.float32(1.0)
    p = np.percentile(finite, 99.9)
    return np.float32(p / 127.0) if p > 0 else np.float32(1.0)
