#!/usr/bin/env python3
"""Benchmark of the W8A8 linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this repository's CUDA route
    python bench.py --impl reference [--gpus N] [--steps K] [--warmup W]   # reference CPU route

A step is one pass of the hot path (per-token quantize -> int8 GEMM -> fused epilogue) over
one batch of synthetic input.  Default workload: the compute-bound GEMM of the benchmark
configurations, M=8192 tokens, K=4096, N=14336, requantizing (int8) epilogue, with the
output channels N sharded across the GPUs of one node when N > 1 GPU and the int8 output
replicated on every GPU by peer stores from the GEMM epilogue (the all-gather fused into the
kernel; the NCCL all-gather of the slabs is timed beside it under "exchange").
Rank 0 prints ONE JSON line.

  value      2*M*K*N / step time, inputs resident in HBM, CUDA events on the launching
             stream, max over ranks (includes the output exchange when n_gpus > 1)
  e2e        the same metric through the host-pointer entry vxb_linear_host: pinned host
             buffers, host->device and device->host copies inside the timed region
  roofline   the tcgen05 GEMM kernel alone, timed live by event pairs inside the timed loop
  cpu_baseline  the reference's own CPU kernels (oracle/_ref) on this box's host cores, on a
             bounded row sample of the same workload (rank 0, N=1 only)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tests import workloads as wl  # noqa: E402

NOMINAL_I8_TOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


# ---------------------------------------------------------------------------------------------
# clocks: NVML sampling thread (read-only) during the timed region
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting"}

    def __init__(self, device_index: int, period_s: float = 0.005):
        self.samples, self.reasons, self.power = [], set(), []
        self.period = period_s
        self._stop = threading.Event()
        self._thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = device_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if device_index < len(ids) and ids[device_index].isdigit():
                    phys = int(ids[device_index])
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _once(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
            self.power.append(self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._once()
            self._stop.wait(self.period)

    def start(self):
        if self.nv is None:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def sample_now(self):
        if self.nv is not None:
            self._once()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------------------------
# reference / CPU legs
# ---------------------------------------------------------------------------------------------
def cpu_reference_run(rows, k, n, steps, warmup, budget_s=None, seed=0):
    """Times the reference's own CPU kernels on a row sample of the workload: per-row int8
    preparation (vx_packed_prepare_i8_*) + packed int8 GEMM with requantization
    (vx_qlinear_i8u8_packed), all host threads through the reference's thread pool.
    Falls back to the scalar oracle port when oracle/_ref was not built."""
    from oracle.bindings import Oracle, Ref
    cores = os.cpu_count() or 1
    x = wl.gemm_activations(rows, k, seed)
    w, ws = wl.gemm_weights(n, k, seed)
    zeros = np.zeros(n, np.int32)
    ops = 2.0 * rows * k * n
    if Ref.available():
        ref = Ref()
        got = ref.threads_enter(cores)
        threads = got if got > 0 else 1
        packed = ref.pack_q8(w)
        q = np.zeros((rows, k), np.int8)
        scales = np.zeros(rows, np.float32)
        out = np.zeros((rows, n), np.int8)

        def step():
            ref.prepare_rows(x, q, scales)
            # R2's activation scale is per tensor; the arithmetic cost does not depend on it
            ok = ref.qlinear_packed(q, packed, np.int8, n, zeros, ws, zeros, float(scales.mean()), 0,
                                    0.05, 0, out=out)
            assert ok is not None
        kind, isa = "reference", ref.isa()
        label = (f"vx_packed_prepare_i8 + vx_qlinear_i8u8_packed (isa {isa}) on rows 0..{rows - 1} "
                 f"of the workload (the row sample; times scale with the row count), K={k}, N={n}")
    else:
        orc = Oracle()
        threads = 1

        def step():
            orc.w8a8_linear(x, w, ws, requant=True, out_scale=0.05)
        kind = "port"
        label = f"scalar oracle port on rows 0..{rows - 1}, K={k}, N={n}"
    for _ in range(warmup):
        step()
    times = []
    t_begin = time.perf_counter()
    for i in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if budget_s is not None and time.perf_counter() - t_begin > budget_s and i >= 2:
            break
    if kind == "reference":
        ref.threads_leave()
    total = float(np.sum(times))
    return {"tops": ops * len(times) / total / 1e12, "ms_per_step": 1e3 * total / len(times),
            "steps": len(times), "cores": threads, "kind": kind, "sample": label}


def cpu_reference_variants(k, n, seed=0, rows=64, budget_s=2.5):
    """The other CPU figures beside the headline baseline, each on a `rows`-row sample and a
    bounded time: the reference's two routes (R1 = vx_packed_linear_forward on W8/G128 words
    whose group scales repeat the channel scale, fp32 output; R2 = prepare +
    vx_qlinear_i8u8_packed, int8 output) at one thread and at every host thread."""
    from oracle.bindings import Ref
    if not Ref.available():
        return None
    ref = Ref()
    cores = os.cpu_count() or 1
    x = wl.gemm_activations(rows, k, seed)
    w, ws = wl.gemm_weights(n, k, seed)
    words = wl.pack_w8_words(w)
    gsc = wl.group_scales(ws, k, 128)
    packed = ref.pack_q8(w)
    zeros = np.zeros(n, np.int32)
    q = np.zeros((rows, k), np.int8); scales = np.zeros(rows, np.float32)
    out8 = np.zeros((rows, n), np.int8); y = np.zeros((rows, n), np.float32)
    ops = 2.0 * rows * k * n

    def r1():
        ref.packed_linear(x, words, gsc, 128, None, y=y)

    def r2():
        ref.prepare_rows(x, q, scales)
        ref.qlinear_packed(q, packed, np.int8, n, zeros, ws, zeros, float(scales.mean()), 0, 0.05, 0, out=out8)

    res = {"rows": rows, "isa": ref.isa()}
    for threads in (1, cores):
        got = ref.threads_enter(threads)
        for name, fn in (("r1_packed_linear_forward", r1), ("r2_prepare_qlinear_packed", r2)):
            fn()
            t0 = time.perf_counter(); cnt = 0
            while True:
                fn(); cnt += 1
                if time.perf_counter() - t0 > budget_s or cnt >= 200:
                    break
            res[f"{name}_tops_t{got if got > 0 else 1}"] = ops * cnt / (time.perf_counter() - t0) / 1e12
        ref.threads_leave()
    return res


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m, k, n = args.rows, args.k, args.n
    rows = min(m, args.cpu_rows)
    r = cpu_reference_run(rows, k, n, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "w8a8_linear_int8_tops", "value": r["tops"], "unit": "TOPS",
        "n_gpus": args.gpus, "steps": r["steps"], "warmup": args.warmup,
        # each timed step is the first `rows` rows of the workload (a bounded CPU sample): ms_per_step is
        # that time scaled to the configuration's row count, so that value = 2MKN / ms_per_step holds
        "ms_per_step": r["ms_per_step"] * (m / rows), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        # the configuration this arm is compared on is the GPU arm's at the same N (the CPU route itself
        # does not shard: it runs on rank 0's host cores)
        "config": workload_config(args, int(os.environ.get("WORLD_SIZE", "1"))),
        "sampled_rows": rows, "sample_ms_per_step": r["ms_per_step"],
        "cpu_baseline": {"value": r["tops"], "unit": "TOPS", "cores": r["cores"], "kind": r["kind"],
                         "sample": r["sample"]},
        "e2e": {"value": r["tops"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    return {"workload": f"w8a8_linear_gemm_M{args.rows}_K{args.k}_N{args.n}_requant_int8",
            "rows": args.rows, "k": args.k, "n": args.n, "epilogue": "requant_int8",
            "activations": "fp32 N(0,1), 1% outlier channels x20, per-token int8",
            "weights": "int8 per-output-channel, N(0,0.02)-shaped codes",
            "parallelism": f"n_shard{world}" + ("+fused_peer_store_allgather_int8" if world > 1 else ""),
            "l2": "inputs larger than L2 (x 134 MB + W 59 MB + out 117 MB per step at N=1)"}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def gemv_sweep(torch, ctx, w8a8, peaks, launches=24, replays=5):
    """Decode sweep (M in 1..32 x three (K,N) shapes).  Per case: the skinny kernel alone
    (prepared activations) for both small-M routes, and the whole step (quantizer + kernel).
    Each measurement replays a CUDA graph of `launches` back-to-back launches between two
    events, so host launch cost is not in the number.  Weights rotate through more than 2x L2
    of distinct copies, so every launch streams from HBM."""
    out = []
    routes = {"decode_tcgen05": w8a8.ROUTE_DECODE, "gemv_dp4a": w8a8.ROUTE_GEMV}
    side = torch.cuda.Stream()

    def graph_ms(fn):
        """ms per launch of fn(i), i = 0..launches-1, replayed from a CUDA graph."""
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            ctx.use_torch_stream()
            for i in range(launches):
                fn(i)
        ctx.use_torch_stream()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / (launches * replays)

    for (k, n) in wl.GEMV_SHAPES:
        copies = max(2, int(np.ceil(300e6 / (k * n))))
        rng = np.random.default_rng(k + n)
        base_w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
        weights = [w8a8.Weight.from_i8(ctx, np.roll(base_w, c, axis=0), ws) for c in range(copies)]
        for rows in wl.GEMV_ROWS:
            x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda()
            y = torch.empty((rows, n), dtype=torch.float32, device="cuda")
            q, sc = ctx.prepare(weights[0], x)
            algo_bytes = k * n + 4 * n + 4 * rows * k + 4 * rows * n
            rec = {"rows": rows, "k": k, "n": n, "algorithmic_bytes": algo_bytes}
            for name, route in routes.items():
                ms = graph_ms(lambda i, route=route: ctx.linear_prepared(
                    weights[i % copies], q, sc, y, mode=1, route=route))
                rec[name] = {"kernel_us": ms * 1e3, "gbs": algo_bytes / (ms * 1e-3) / 1e9,
                             "frac_of_measured": algo_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                             "frac_of_nominal_8000": algo_bytes / (ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS}
            ms = graph_ms(lambda i: ctx.linear_f32(weights[i % copies], x, out=y))
            rec["step_auto"] = {"route": w8a8.last_route(), "step_us": ms * 1e3,
                                "gbs": algo_bytes / (ms * 1e-3) / 1e9}
            out.append(rec)
        for wt in weights:
            wt.close()
    return out


def model_linear_stacks(torch, ctx, w8a8, peaks, replays=5):
    """The W8A8 linears of the two decoder configurations, all layers with their own weights, one
    CUDA graph per pass (fp32 epilogue): the prefill batch of the SmolLM2-135M shape (8 x 512
    tokens) and one decode step of the Qwen3-0.6B shape at batch 64.  Two ways of calling:
    "per_linear" = seven vxb_linear_f32 calls per layer (quantizer + GEMM each); "shared" = what
    the reference's fused decode patterns do with the same arithmetic: q/k/v and gate/up read
    the same activations, so their weights are concatenated along the output channels and the
    activations are quantized once (vxb_quantize_rows + vxb_linear_prepared): four quantizer and
    four GEMM launches per layer.  Only the linears run here (no attention, norms or embedding),
    so tokens/s is the rate the linear stack alone would allow."""
    out = {}
    for name, cfg in (("smollm2_135m_prefill_8x512", wl.SMOLLM2_135M), ("qwen3_0.6b_decode_b64", wl.QWEN3_0_6B)):
        rows, layers, lin = cfg["rows"], cfg["layers"], cfg["linears"]
        rng = np.random.default_rng(layers)
        groups = [("q", "k", "v"), ("o",), ("gate", "up"), ("down",)]
        per_linear, shared, ops, wbytes, iobytes = [], [], 0.0, 0, 0
        for layer in range(layers):
            raw = {}
            for lname, (k, n) in lin.items():
                raw[lname] = (rng.integers(-127, 128, size=(n, k), dtype=np.int8),
                              rng.uniform(0.001, 0.02, size=n).astype(np.float32))
                ops += 2.0 * rows * k * n
                wbytes += k * n + 4 * n
                iobytes += 4 * rows * n
            iobytes += sum(4 * rows * lin[g[0]][0] for g in groups)     # each distinct input read once
            per_linear.append({ln: w8a8.Weight.from_i8(ctx, *raw[ln]) for ln in lin})
            shared.append([w8a8.Weight.from_i8(ctx, np.concatenate([raw[ln][0] for ln in g]),
                                               np.concatenate([raw[ln][1] for ln in g])) for g in groups])
        xs = {k: torch.randn(rows, k, device="cuda") for k in {kn[0] for kn in lin.values()}}
        ys = {n: torch.empty(rows, n, device="cuda") for n in
              {kn[1] for kn in lin.values()} | {sum(lin[ln][1] for ln in g) for g in groups}}

        def pass_per_linear():
            for row in per_linear:
                for lname, (k, n) in lin.items():
                    ctx.linear_f32(row[lname], xs[k], out=ys[n])

        def pass_shared():
            for row in shared:
                for g, wt in zip(groups, row):
                    q, sc = ctx.prepare(wt, xs[lin[g[0]][0]])
                    ctx.linear_prepared(wt, q, sc, ys[wt.d_out], mode=1)

        rec = {"rows": rows, "layers": layers, "weight_bytes": wbytes, "activation_bytes": iobytes}
        for label, fn in (("per_linear", pass_per_linear), ("shared", pass_shared)):
            fn()
            route = w8a8.last_route()
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                ctx.use_torch_stream()
                fn()
            ctx.use_torch_stream()
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(replays):
                g.replay()
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1) / replays
            rec[label] = {"launches_per_layer": 14 if label == "per_linear" else 8, "ms_per_pass": ms,
                          "tokens_per_s_linears_only": rows / (ms * 1e-3), "tops": ops / (ms * 1e-3) / 1e12,
                          "gbs": (wbytes + iobytes) / (ms * 1e-3) / 1e9,
                          "frac_of_measured_hbm": (wbytes + iobytes) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "last_route": route}
        out[name] = rec
        for row in per_linear:
            for wt in row.values():
                wt.close()
        for row in shared:
            for wt in row:
                wt.close()
    return out


def widened_rows(torch, ctx, w8a8, peaks, replays=10):
    """Kernels of the rows next to the headline path, timed alone with CUDA events (inputs larger than
    L2 or an L2 flush between launches is not applied here: these are secondary figures): the GEMM for
    weights with grouped scales (G = 128, the exporter's default; also W4 storage, which is unpacked to
    int8 at load and takes the same kernel) and RMSNorm folded into the quantizer."""
    out = {}
    rows, k, n, group = 4096, 4096, 4096, 128
    rng = np.random.default_rng(77)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    gs = rng.uniform(0.001, 0.02, size=(n, k // group)).astype(np.float32)
    x = torch.randn(rows, k, device="cuda")
    y = torch.empty(rows, n, device="cuda")

    def time_us(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e3 / replays

    for label, weight in (("w8_g128", w8a8.Weight.from_w8_words(ctx, wl.pack_w8_words(w), gs, k, group)),
                          ("w4_g128", w8a8.Weight.from_w4_words(ctx, wl.pack_w4_words((w >> 4).astype(np.int8)), gs, k, group))):
        q, sc = ctx.prepare(weight, x)
        us = time_us(lambda: ctx.linear_prepared(weight, q, sc, y, mode=1))
        out["grouped_gemm_" + label] = {"rows": rows, "k": k, "n": n, "kernel_us": us,
                                        "tops": 2.0 * rows * k * n / us / 1e6, "route": w8a8.last_route()}
        weight.close()
    rows = 8192
    x = torch.randn(rows, k, device="cuda")
    gamma = torch.rand(k, device="cuda") + 0.5
    plain = time_us(lambda: ctx.quantize_rows(x))
    fused = time_us(lambda: ctx.rmsnorm_quantize_rows(x, gamma, 1e-6, want_norm=False))
    kept = time_us(lambda: ctx.rmsnorm_quantize_rows(x, gamma, 1e-6, want_norm=True))
    out["rmsnorm_quantize"] = {"rows": rows, "k": k, "quantize_us": plain, "rmsnorm_quantize_us": fused,
                               "rmsnorm_quantize_keep_rows_us": kept,
                               "note": "times include the output allocation of the Python mirror"}
    return out


def gemm_sweep(torch, ctx, w8a8, peaks, i8_probe, steps=12):
    """All twelve shapes of the compute-bound sweep (M in 2048..16384 x three (K, N) pairs), requantizing
    epilogue, one GPU: step time (quantizer + GEMM, inputs resident in HBM, CUDA events) and the GEMM
    kernel's own time (event pairs inside the library), as TOPS and as fractions of the resident-operand
    kind::i8 probe and of 2 x the measured bf16 rate.  Weights are drawn on the device (N(0, 30)-shaped
    codes clamped to +-127): the timing does not depend on their values."""
    out = []
    peak2 = 2.0 * peaks["bf16_tflops"]
    for (k, n) in wl.GEMM_SHAPES:
        gen = torch.Generator(device="cuda").manual_seed(k + n)
        codes = torch.randn((n, k), device="cuda", generator=gen).mul_(30.0).round_().clamp_(-127, 127).to(torch.int8)
        ws = np.full(n, 0.02 * 4.2 / 127.0, np.float32)
        weight = w8a8.Weight.from_i8(ctx, codes.cpu().numpy(), ws)
        del codes
        for m in wl.GEMM_ROWS:
            x = torch.randn((m, k), device="cuda", generator=gen)
            y = torch.empty((m, n), dtype=torch.int8, device="cuda")
            for _ in range(3):
                ctx.linear_i8(weight, x, 0.05, 0, out=y)
            torch.cuda.synchronize()
            ctx.profile(4)   # every fourth step's GEMM is bracketed by events (they break the launch chain)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                ctx.linear_i8(weight, x, 0.05, 0, out=y)
            e1.record()
            e1.synchronize()
            prof = ctx.profile_read()
            ctx.profile(False)
            step_ms, kern_ms = e0.elapsed_time(e1) / steps, prof["gemm_ms"] / max(1, prof["gemm_launches"])
            ops = 2.0 * m * k * n
            out.append({"rows": m, "k": k, "n": n, "route": w8a8.last_route(), "step_ms": step_ms, "kernel_ms": kern_ms,
                        "step_tops": ops / step_ms / 1e9, "kernel_tops": ops / kern_ms / 1e9,
                        "step_frac_of_nominal_4500": ops / step_ms / 1e9 / NOMINAL_I8_TOPS,
                        "kernel_frac_of_i8_probe": ops / kern_ms / 1e9 / i8_probe,
                        "kernel_frac_of_2x_bf16": ops / kern_ms / 1e9 / peak2})
            del x, y
        weight.close()
    return out


def sharded_wide_shapes(torch, dist, ctx, w8a8, sharded, world, rank, timed, steps=10):
    """The two widest configured layers at M 8192, N-sharded over `world` GPUs: the step with the int8
    output replicated by the fused peer-store all-gather and the step with outputs left sharded (what
    a row-parallel consumer takes).  All ranks call this; the activations are rank 0's, broadcast."""
    out = []
    for (m, k, n) in ((8192, 8192, 28672), (8192, 4096, 128256)):
        lo, hi = sharded.shard_bounds(n, world, rank)
        n_local = hi - lo
        w_local, ws_local = wl.gemm_weights(n_local, k, seed=2000 + rank)
        weight = w8a8.Weight.from_i8(ctx, w_local, ws_local)
        x = torch.empty((m, k), dtype=torch.float32, device="cuda")
        if rank == 0:
            x.copy_(torch.from_numpy(wl.gemm_activations(m, k, seed=3)))
        dist.broadcast(x, 0)
        scale_t = torch.zeros(1, dtype=torch.float32, device="cuda")
        if rank == 0:
            smp = ctx.linear_f32(weight, x[:16])
            ctx.synchronize()
            scale_t[0] = float(wl.static_out_scale(smp.cpu().numpy()))
        dist.broadcast(scale_t, 0)
        out_scale = float(scale_t.item())
        lin = sharded.NShardedLinear(
            n, world, rank, lambda xx, o, w=weight, s=out_scale: ctx.linear_i8(w, xx, s, 0, out=o), torch.int8, "cuda")
        fused = sharded.FusedGatherLinear(ctx, weight, n, world, rank, rows=m)
        for _ in range(3):
            fused.forward(x, out_scale)
            lin.forward_sharded(x)
        fused_ms = timed(lambda: fused.forward(x, out_scale), steps) / steps
        shard_ms = timed(lambda: lin.forward_sharded(x), steps) / steps
        # the replicated result equals every rank's own slab where they overlap
        y_rep = fused.forward(x, out_scale)
        own_ok = bool(torch.equal(y_rep[:, lo:hi], lin.forward_sharded(x)))
        flags = [None] * world
        dist.all_gather_object(flags, own_ok)
        ops = 2.0 * m * k * n
        recv = m * (n - n_local)
        out.append({"rows": m, "k": k, "n": n, "n_gpus": world,
                    "fused_ms": fused_ms, "fused_tops": ops / (fused_ms * 1e-3) / 1e12,
                    "sharded_ms": shard_ms, "sharded_tops": ops / (shard_ms * 1e-3) / 1e12,
                    "nvlink_recv_bytes_per_gpu": int(recv), "nvlink_floor_ms": recv / 770e9 * 1e3,
                    "mma_floor_ms": ops / world / (2.0 * measured_peaks()["bf16_tflops"] * 1e12) * 1e3,
                    "replicated_equals_own_slab_on_every_rank": all(flags)})
        fused.close()
        weight.close()
        del x, lin, y_rep
        torch.cuda.empty_cache()
    return out


def sustained_run(torch, step, ops, device_index, seconds=2.5):
    """Back-to-back steps for `seconds` with the clock sampler at 5 ms: the sustained rate under the power
    cap next to the burst figure of the short timed loop (median SM clock, TOPS, and TOPS scaled to the
    maximum SM clock)."""
    sampler = ClockSampler(device_index, period_s=0.005)
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    t0 = time.perf_counter()
    count = 0
    e0.record()
    while time.perf_counter() - t0 < seconds:
        for _ in range(50):
            step()
        count += 50
        torch.cuda.current_stream().synchronize() if count % 500 == 0 else None
    e1.record()
    e1.synchronize()
    sampler.stop()
    ms = e0.elapsed_time(e1) / count
    clocks = sampler.summary()
    tops = ops / ms / 1e9
    mhz, top = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
    return {"seconds": e0.elapsed_time(e1) / 1e3, "steps": count, "ms_per_step": ms, "tops": tops, "clocks": clocks,
            "tops_at_max_clock": tops * top / mhz if mhz and top else None}


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    from volvoxai_b200 import w8a8

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL's own banner goes to stderr: stdout carries the one JSON line only
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = measured_peaks()
    from volvoxai_b200 import sharded
    m, k, n = args.rows, args.k, args.n
    lo, hi = sharded.shard_bounds(n, world, rank)
    n_local = hi - lo

    ctx = w8a8.Context(local)
    ctx.use_torch_stream()

    # weights of this rank's output-channel shard (contiguous channel range), activations replicated
    w_local, ws_local = wl.gemm_weights(n_local, k, seed=1000 + rank)
    weight = w8a8.Weight.from_i8(ctx, w_local, ws_local)
    x_host_np = wl.gemm_activations(m, k, seed=0)
    x_dev = torch.from_numpy(x_host_np).cuda()

    # static output scale: 99.9th percentile |y| / 127 of this library's own fp32 output on a sample
    # (rows 0..15 of rank 0's shard), broadcast to all ranks
    out_scale_t = torch.zeros(1, dtype=torch.float32, device="cuda")
    if rank == 0:
        smp = ctx.linear_f32(weight, x_dev[:16])
        ctx.synchronize()
        out_scale_t[0] = float(wl.static_out_scale(smp.cpu().numpy()))
    if world > 1:
        dist.broadcast(out_scale_t, 0)
    out_scale = float(out_scale_t.item())

    lin = sharded.NShardedLinear(
        n, world, rank, lambda x, out: ctx.linear_i8(weight, x, out_scale, 0, out=out), torch.int8, "cuda")
    y_local = lin.forward_sharded(x_dev)

    # N > 1: the all-gather is fused into the GEMM epilogue (peer stores over NVLink into every
    # rank's replicated output buffer); the NCCL all-gather of the slabs is timed beside it
    fused = sharded.FusedGatherLinear(ctx, weight, n, world, rank, rows=m) if world > 1 else None

    def step(gather=True):
        if world > 1 and gather:
            fused.forward(x_dev, out_scale)
        else:
            lin.forward_sharded(x_dev)

    def step_nccl():
        lin.forward_gathered(x_dev)   # local slab + NCCL all-gather of the int8 slabs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, count):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(count):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    sampler = ClockSampler(local)
    launches0 = w8a8.launch_count()
    # the GEMM is bracketed by events on every 8th step only: an event between two launches keeps the later
    # one from starting as a programmatic dependent of the earlier, which costs 12 us per step at N = 2
    prof_stride = 8 if args.steps >= 16 else 1
    ctx.profile(prof_stride)
    sampler.start()
    total_ms = timed(step, args.steps)
    sampler.sample_now()
    sampler.stop()
    prof = ctx.profile_read()
    ctx.profile(False)
    launches = w8a8.launch_count() - launches0
    ctx.synchronize()

    step_route = w8a8.last_route()
    ops = 2.0 * m * k * n
    ms_per_step = total_ms / args.steps
    value = ops / (ms_per_step * 1e-3) / 1e12

    # kernel-only view (outputs left N-sharded): the same loop without the all-gather
    nogather_ms = timed(lambda: step(False), args.steps) / args.steps if world > 1 else ms_per_step
    exchange = None
    if world > 1:
        for _ in range(3):
            step_nccl()
        nccl_ms = timed(step_nccl, args.steps) / args.steps
        y_rep = fused.forward(x_dev, out_scale)
        same_as_nccl = bool(torch.equal(y_rep, lin.forward(x_dev)))
        # the gathered output against the CPU oracle (the checker, outside every timed region): rows
        # 0..15 x the first 256 channels of EVERY rank's shard, as they arrived in rank 0's buffer
        samples = [None] * world
        dist.all_gather_object(samples, (lo, w_local[:256], ws_local[:256]))
        matches_oracle = None
        if rank == 0:
            from oracle.bindings import Oracle
            orc = Oracle()
            got = y_rep[:16].cpu().numpy()
            matches_oracle = True
            for (lo_r, w_r, ws_r) in samples:
                if len(ws_r) == 0:
                    continue
                want = orc.w8a8_linear(x_host_np[:16], w_r, ws_r, requant=True, out_scale=out_scale)["out"]
                matches_oracle = matches_oracle and bool(np.array_equal(got[:, lo_r:lo_r + len(ws_r)], want))
        # lower bound of any exchange that replicates the int8 output: the bytes each GPU must
        # receive over NVLink at the measured peer-copy rate (770 GB/s per direction)
        recv_bytes = m * (n - n_local)
        exchange = {"fused_peer_store_ms": ms_per_step, "nccl_allgather_ms": nccl_ms,
                    "sharded_no_exchange_ms": nogather_ms,
                    "nvlink_recv_bytes_per_gpu": int(recv_bytes),
                    "nvlink_floor_ms": recv_bytes / 770e9 * 1e3,
                    "fused_matches_nccl_path": same_as_nccl, "matches_oracle": matches_oracle}
        if rank == 0 and not (same_as_nccl and matches_oracle):
            raise RuntimeError(f"multi-GPU output check failed: nccl path {same_as_nccl}, oracle {matches_oracle}")

    # roofline of the dominant kernel (the tcgen05 GEMM of this rank's shard)
    # a large batch is cut in two (the quantizer of the later rows runs under the GEMM of the first ones):
    # the GEMM's time per step is the sum over its launches of that step
    launches_per_step = 1.0   # one GEMM launch per step (the two-chunk overlap form is off by default)
    gemm_ms = prof["gemm_ms"] / max(1, prof["gemm_launches"]) * launches_per_step
    # the quantizer alone over the whole batch, timed outside the step loop
    for _ in range(3):
        ctx.quantize_rows(x_dev, ldq=weight.row_bytes)
    qe0, qe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    qe0.record()
    for _ in range(10):
        ctx.quantize_rows(x_dev, ldq=weight.row_bytes)
    qe1.record()
    qe1.synchronize()
    quant_ms = qe0.elapsed_time(qe1) / 10
    ops_local = 2.0 * m * k * n_local
    achieved = ops_local / (gemm_ms * 1e-3) / 1e12
    peak = 2.0 * peaks["bf16_tflops"]
    i8_probe = ctx.measure_i8_tensor_peak(200)
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "traffic": None,
        "kernel": "gemm_i8_pair_kernel" if "pair" in step_route else "gemm_i8_tcgen05_kernel", "kernel_ms": gemm_ms,
        "kernel_launches_per_step": launches_per_step, "kernel_launches_timed": int(prof["gemm_launches"]),
        "kernel_timing": f"CUDA event pairs around every {prof_stride}th step's launch inside the timed region",
        "route": step_route,
        "peak_source": f"2 x bf16_tflops (cuBLAS bf16 burst, {peaks['_source']}) as the dense int8 rate",
        "i8_probe_tops": i8_probe, "frac_of_i8_probe": achieved / i8_probe,
        "frac_of_nominal_4500": achieved / NOMINAL_I8_TOPS,
        "quantize_kernel_ms": quant_ms,
        "quantize_note": "whole-batch quantizer timed alone (allocation of its outputs included); inside a step it runs in front of the GEMM",
        "quantize_gbs": (5.0 * m * k + 4.0 * m) / (quant_ms * 1e-3) / 1e9 if quant_ms > 0 else None,
        "quantize_frac_of_hbm": ((5.0 * m * k + 4.0 * m) / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
                                 if quant_ms > 0 else None),
    }
    # DRAM traffic per launch, scaled from the ncu capture of a smaller launch of the same kernel
    # (M 4096, K 4096, N 14336: dram read 75.73 MB = 1.003 x (M + N_local) x Kpad, dram write 29.4 MB =
    # 0.50 x M x N_local; see profiles/gemm_i8_pair_M4096_K4096_N14336.md). Reads grow with
    # (M + N) x K, writes with M x N.
    kpad = (k + 127) // 128 * 128
    roofline["traffic"] = 1.003 * (m + n_local) * kpad + 0.50 * m * n_local
    roofline["traffic_source"] = "ncu dram__bytes_read+write of the M4096 launch, scaled by (M+N)K and MN"
    roofline["algorithmic_bytes"] = (m + n_local) * kpad + m * n_local
    if world > 1:
        # fused GEMM + all-gather kernel: the target time is the slower of the MMAs at the measured
        # tensor peak and the bytes this GPU must send over NVLink at the measured peer-copy rate
        send_bytes = m * n_local * (world - 1)
        t_mma, t_link = ops_local / (peak * 1e12) * 1e3, send_bytes / 770e9 * 1e3
        roofline["fused"] = {"bound": "nvlink" if t_link > t_mma else "tensor", "mma_ms": t_mma,
                             "nvlink_ms": t_link, "nvlink_send_bytes": int(send_bytes),
                             "nvlink_gbs_peak": 770.0, "target_ms": max(t_mma, t_link),
                             "kernel_ms": gemm_ms, "frac": max(t_mma, t_link) / gemm_ms}

    # end to end through the host-pointer entry: pinned host buffers, copies inside the region
    y_pin = torch.empty((m, n_local), dtype=torch.int8).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    if world == 1:
        x_pin = torch.from_numpy(x_host_np).pin_memory()
        e2e_api = "vxb_linear_host"

        def e2e_step():
            ctx.linear_host(weight, x_pin, y_pin, requant=True, out_scale=out_scale)
    else:
        # every rank uploads M / N rows, quantizes them, all-gathers the int8 codes over NVLink and
        # downloads its channel slab: host traffic per step does not grow with the number of GPUs
        rows_local = m // world
        x_pin = torch.from_numpy(x_host_np[rank * rows_local:(rank + 1) * rows_local]).pin_memory()
        host_lin = sharded.RowShardedHostLinear(ctx, weight, m, k, world, rank)
        e2e_api = "RowShardedHostLinear (vxb_quantize_rows + NCCL all-gather of int8 rows + vxb_linear_prepared)"

        def e2e_step():
            host_lin.forward(x_pin, y_pin, out_scale)
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_s.item()) * 1e3 / e2e_steps
    # the host result must equal the device-resident result
    same = bool(torch.equal(y_pin.cuda(), y_local))
    e2e = {"value": ops / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
           "steps": e2e_steps, "h2d_bytes_per_step": int(x_pin.numel() * 4) * world,
           "d2h_bytes_per_step": int(y_pin.numel()) * world, "api": e2e_api,
           "matches_device_result": same}

    line = {
        "metric": "w8a8_linear_int8_tops", "value": value, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(args, world),
        "clocks": sampler.summary(), "e2e": e2e, "gpu_launches": int(launches),
        "roofline": roofline,
        "kernel_only": {"value": ops / (nogather_ms * 1e-3) / 1e12, "unit": "TOPS",
                        "ms_per_step": nogather_ms, "note": "outputs left N-sharded (no all-gather)"},
    }
    if exchange is not None:
        line["exchange"] = exchange

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = cpu_reference_run(min(m, args.cpu_rows), k, n, steps=1000, warmup=1, budget_s=args.cpu_seconds)
        line["cpu_baseline"] = {"value": r["tops"], "unit": "TOPS", "cores": r["cores"],
                                "kind": r["kind"], "sample": r["sample"] + f", {r['steps']} repeats"}
        if not args.no_extras:
            line["cpu_baseline"]["routes"] = cpu_reference_variants(k, n)
    elif rank == 0:
        line["cpu_baseline"] = None
    if rank == 0 and world == 1 and not args.no_extras:
        line["extras"] = {"gemm_sweep": gemm_sweep(torch, ctx, w8a8, peaks, i8_probe),
                          "sustained": sustained_run(torch, step, ops, local),
                          "gemv_sweep": gemv_sweep(torch, ctx, w8a8, peaks),
                          "model_linear_stacks": model_linear_stacks(torch, ctx, w8a8, peaks),
                          "widened_rows": widened_rows(torch, ctx, w8a8, peaks)}

    if world > 1 and not args.no_extras:
        wide = sharded_wide_shapes(torch, dist, ctx, w8a8, sharded, world, rank, timed)
        if rank == 0:
            line["extras"] = {"sharded_wide_shapes": wide}

    weight.close()
    ctx.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def decode_arm(args):
    """--workload decode: one decode-shaped linear (rows <= 128) on one GPU. A step is the
    quantizer + the weight-streaming kernel on device-resident fp32 activations; weights rotate
    through more than 2x L2 of distinct copies. Prints one JSON line with the HBM roofline of the
    decode kernel (prepared activations, CUDA-graph replay of back-to-back launches)."""
    import torch
    import torch.distributed as dist
    from volvoxai_b200 import w8a8
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    # N > 1: every GPU serves its own sequences against its own copy of the layer ("replicas only": at
    # decode sizes an N-shard would trade a 10 us weight stream for an exchange of the same order)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = measured_peaks()
    rows, k, n = args.rows, args.k, args.n
    ctx = w8a8.Context(local)
    ctx.use_torch_stream()
    rng = np.random.default_rng(7)
    copies = max(2, int(np.ceil(300e6 / (k * n))))
    base_w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
    weights = [w8a8.Weight.from_i8(ctx, np.roll(base_w, c, axis=0), ws) for c in range(copies)]
    x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float32)).cuda()
    y = torch.empty((rows, n), dtype=torch.float32, device="cuda")
    q, sc = ctx.prepare(weights[0], x)
    algo_bytes = k * n + 4 * n + 4 * rows * k + 4 * rows * n
    side = torch.cuda.Stream()

    def replay_ms(fn, launches):
        for i in range(max(3, args.warmup)):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            ctx.use_torch_stream()
            for i in range(launches):
                fn(i)
        ctx.use_torch_stream()
        g.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / launches], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)   # the slowest replica's time counts
        return float(ms.item())

    launches0 = w8a8.launch_count()
    step_ms = replay_ms(lambda i: ctx.linear_f32(weights[i % copies], x, out=y), args.steps)
    launches = w8a8.launch_count() - launches0
    route = w8a8.last_route()
    kern_ms = replay_ms(lambda i: ctx.linear_prepared(weights[i % copies], q, sc, y, mode=1), args.steps)
    gbs = algo_bytes / (kern_ms * 1e-3) / 1e9
    line = {
        "metric": "w8a8_decode_linear_hbm_gbs", "value": world * algo_bytes / (step_ms * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": f"w8a8_linear_decode_M{rows}_K{k}_N{n}_f32", "rows": rows, "k": k, "n": n,
                   "route": route, "parallelism": "replicas only" if world > 1 else "one GPU",
                   "rows_per_s": world * rows / (step_ms * 1e-3),
                   "l2": f"{copies} distinct weight copies rotate (> 2x L2)",
                   "timing": "CUDA-graph replay of back-to-back launches between two events"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": None, "kernel": "decode_rows_kernel",
                     "kernel_us": kern_ms * 1e3, "algorithmic_bytes": algo_bytes,
                     "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS, "peak_source": peaks["_source"]},
    }
    for wt in weights:
        wt.close()
    ctx.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def prefill_arm(args):
    """--workload prefill: one prefill-shaped linear with fp32 output (dequantization + bias) on one GPU,
    the output-write-bound case of small models (default M 4096, K 576, N 14336).  A step is the quantizer
    + the GEMM on device-resident fp32 activations; outputs rotate through buffers larger than L2.  Prints
    one JSON line with the HBM roofline of the GEMM (prepared activations, CUDA-graph replay)."""
    import torch
    from volvoxai_b200 import w8a8
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    peaks = measured_peaks()
    rows, k, n = args.rows, args.k, args.n
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    w_np, ws_np = wl.gemm_weights(n, k, seed=9)
    bias = np.random.default_rng(9).standard_normal(n).astype(np.float32) * 0.01
    weight = w8a8.Weight.from_i8(ctx, w_np, ws_np, bias_f32=bias)
    x = torch.from_numpy(wl.gemm_activations(rows, k, seed=10)).cuda()
    copies = max(2, int(np.ceil(300e6 / (4.0 * rows * n))))
    ys = [torch.empty((rows, n), dtype=torch.float32, device="cuda") for _ in range(copies)]
    q, sc = ctx.prepare(weight, x)
    kpad = (k + 127) // 128 * 128
    algo_bytes = rows * kpad + n * kpad + 8 * n + 4 * rows + 4 * rows * n
    side = torch.cuda.Stream()

    def replay_ms(fn, launches):
        for i in range(max(3, args.warmup)):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            ctx.use_torch_stream()
            for i in range(launches):
                fn(i)
        ctx.use_torch_stream()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / launches

    launches0 = w8a8.launch_count()
    step_ms = replay_ms(lambda i: ctx.linear_f32(weight, x, out=ys[i % copies]), args.steps)
    launches = w8a8.launch_count() - launches0
    route = w8a8.last_route()
    kern_ms = replay_ms(lambda i: ctx.linear_prepared(weight, q, sc, ys[i % copies], mode=1), args.steps)
    gbs = algo_bytes / (kern_ms * 1e-3) / 1e9
    line = {
        "metric": "w8a8_prefill_linear_f32_hbm_gbs", "value": (algo_bytes + 4.0 * rows * k) / (step_ms * 1e-3) / 1e9,
        "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"w8a8_linear_prefill_M{rows}_K{k}_N{n}_f32", "rows": rows, "k": k, "n": n,
                   "route": route, "l2": f"{copies} output buffers rotate (> 2x L2 with the operands)",
                   "timing": "CUDA-graph replay of back-to-back launches between two events"},
        "gpu_launches": int(launches),
        "tops": 2.0 * rows * k * n / (step_ms * 1e-3) / 1e12,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                     "kernel": "gemm_i8_wide_kernel" if "wide" in route else "gemm_i8_pair_kernel" if "pair" in route else "gemm_i8_tcgen05_kernel",
                     "kernel_us": kern_ms * 1e3, "algorithmic_bytes": algo_bytes,
                     "output_write_gbs": 4.0 * rows * n / (kern_ms * 1e-3) / 1e9,
                     "frac_of_nominal_8000": gbs / NOMINAL_HBM_GBS, "peak_source": peaks["_source"]},
    }
    weight.close()
    ctx.close()
    print(json.dumps(line), flush=True)


def decoder_arm(args):
    """`--workload decoder --model smollm2|qwen3 [--gpus N]`: the two model-shaped configurations end to
    end.  smollm2: prefill of 8 x 512 tokens through the 30-layer SmolLM2-135M-shaped decoder (tokens/s);
    qwen3: greedy decode at batch 64 from 256-token prompts for 128 new tokens through the 28-layer
    Qwen3-0.6B-shaped decoder with the paged KV cache (block 16), the decode step replayed from a CUDA
    graph (new tokens/s).  Random-initialised weights, uniform random token ids.  Every W8A8 linear runs
    in this library (fused RMSNorm / SiLU*Mul / residual forms); embedding, rotary, attention, KV-cache
    indexing and the fp32 lm_head are PyTorch glue, and the line says how much of the step the
    library's kernels account for.  With N > 1 every GPU runs an independent replica (the path has no
    exchange step at these layer sizes): value is the sum over replicas, scaling weak."""
    import torch
    import torch.distributed as dist
    from tests import decoder_harness as dh
    from volvoxai_b200 import w8a8
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = measured_peaks()
    ctx = w8a8.Context(local)
    ctx.use_torch_stream()
    prefill = args.model == "smollm2"
    cfg = dh.SMOLLM2_135M if prefill else dh.QWEN3_0_6B
    model = dh.W8A8Decoder(cfg, ctx, w8a8, seed=rank)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    sampler = ClockSampler(local)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if prefill:
        batch, seq, steps = 8, 512, max(3, min(args.steps, 20))
        tokens = torch.randint(0, cfg["vocab"], (batch, seq), device="cuda", generator=gen)
        model.allocate_cache(batch, seq)
        for _ in range(max(3, args.warmup)):
            model.prefill(tokens)
        sync_all()
        # the library's share of one pass: the same pass eagerly with per-kernel event pairs
        before = w8a8.launch_count()
        ctx.profile(True)
        model.prefill(tokens)
        prof = ctx.profile_read(); ctx.profile(False)
        lib_ms = prof["quantize_ms"] + prof["gemm_ms"]
        launches_in_a_step = w8a8.launch_count() - before
        # the timed passes replay a CUDA graph of one prefill (the glue is hundreds of small PyTorch launches
        # per pass: launched eagerly, the host, not the GPU, sets the pace); eager if the capture is refused
        note = "prefill pass replayed from a CUDA graph"
        graph = None
        try:
            side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                ctx.use_torch_stream()
                model.prefill(tokens)
            ctx.use_torch_stream()
            graph.replay()
        except Exception as exc:   # noqa: BLE001 - any capture failure falls back to the eager loop
            graph, note = None, f"eager PyTorch glue between the library's launches (graph capture refused: {type(exc).__name__})"
            ctx.use_torch_stream()
        sync_all()
        launches0 = w8a8.launch_count()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            if graph is not None:
                graph.replay()
            else:
                model.prefill(tokens)
        e1.record()
        sync_all()
        sampler.sample_now(); sampler.stop()
        ms = e0.elapsed_time(e1) / steps
        units = batch * seq
        workload = "smollm2_135m_shape_prefill_8x512"
        metric = "w8a8_decoder_prefill_tokens_per_s"
    else:
        batch, prompt, new = 64, 256, 128
        steps = new
        tokens = torch.randint(0, cfg["vocab"], (batch, prompt), device="cuda", generator=gen)
        model.allocate_cache(batch, prompt + new, dtype=torch.bfloat16)
        logits = model.prefill(tokens)
        tok = logits.argmax(-1)
        pos = torch.full((batch, 1), prompt, dtype=torch.int64, device="cuda")
        model.decode_step(tok, pos)           # warm-up (writes position `prompt`; rewritten by the first timed step)
        torch.cuda.synchronize()
        side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ctx.use_torch_stream()
            out = model.decode_step(tok, pos)
            tok.copy_(out.argmax(-1))
            pos.add_(1)
        ctx.use_torch_stream()
        pos.fill_(prompt)
        for _ in range(3):
            graph.replay()
        pos.fill_(prompt)
        sync_all()
        launches0 = w8a8.launch_count()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(new):
            graph.replay()
        e1.record()
        sync_all()
        sampler.sample_now(); sampler.stop()
        ms = e0.elapsed_time(e1) / new
        units = batch
        # the library's share of one step: the same step eagerly with per-kernel event pairs
        pos.fill_(prompt)
        before = w8a8.launch_count()
        ctx.profile(True)
        model.decode_step(tok, pos)
        prof = ctx.profile_read(); ctx.profile(False)
        lib_ms = prof["quantize_ms"] + prof["gemm_ms"]
        launches_in_a_step = w8a8.launch_count() - before
        workload = "qwen3_0.6b_shape_decode_b64_prompt256_new128_paged_kv16"
        metric, note = "w8a8_decoder_decode_tokens_per_s", "decode step replayed from a CUDA graph; bf16 paged KV cache"
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    launches_per_step = 8 * cfg["layers"]
    weight_bytes = model.weight_bytes
    line = {
        "metric": metric, "value": world * units / (ms_max * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": ms_max, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload, "layers": cfg["layers"], "hidden": cfg["hidden"], "parallelism": f"replicas{world}",
                   "l2": "weights of all layers (> L2) stream once per step", "glue": note},
        # kernels of this library inside the timed region: a replayed graph launches what one captured step holds
        "clocks": sampler.summary(), "gpu_launches": int(launches_in_a_step * steps),
        "library": {"launches_per_step": launches_per_step, "kernels_ms_per_step": lib_ms, "share_of_step": lib_ms / ms_max,
                    "weight_bytes": weight_bytes, "route": w8a8.last_route()},
        "roofline": {"bound": "hbm", "achieved": weight_bytes / (lib_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": weight_bytes / (lib_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                     "kernel": "W8A8 linear launches of one step (quantizers + decode / GEMM kernels)",
                     "note": "weight bytes of all layers / time inside the library's kernels"},
    }
    model.close()
    ctx.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def grouped_arm(args):
    """`--workload grouped --rows M --k K --n N --group G`: the linear over PackedLinear storage whose
    group scales differ within a channel (fp32 output), quantizer + grouped-scale GEMM per step on
    device-resident activations. A secondary figure (one JSON line, tensor roofline of the
    grouped kernel); the ncu summaries of that kernel were taken with this command."""
    import torch
    from volvoxai_b200 import w8a8
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    peaks = measured_peaks()
    rows, k, n, group = args.rows, args.k, args.n, args.group
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    rng = np.random.default_rng(11)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    gs = rng.uniform(0.001, 0.02, size=(n, (k + group - 1) // group)).astype(np.float32)
    weight = w8a8.Weight.from_w8_words(ctx, wl.pack_w8_words(w), gs, k, group)
    x = torch.randn(rows, k, device="cuda")
    y = torch.empty((rows, n), dtype=torch.float32, device="cuda")
    q, sc = ctx.prepare(weight, x)

    def timed(fn, count):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(count):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / count

    launches0 = w8a8.launch_count()
    step_ms = timed(lambda: ctx.linear_f32(weight, x, out=y), args.steps)
    launches = w8a8.launch_count() - launches0
    route = w8a8.last_route()
    kern_ms = timed(lambda: ctx.linear_prepared(weight, q, sc, y, mode=1), args.steps)
    ops = 2.0 * rows * k * n
    peak = 2.0 * peaks["bf16_tflops"]
    line = {
        "metric": "w8a8_grouped_linear_int8_tops", "value": ops / (step_ms * 1e-3) / 1e12, "unit": "TOPS",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"w8a8_linear_grouped_M{rows}_K{k}_N{n}_G{group}_f32", "rows": rows, "k": k, "n": n,
                   "group": group, "route": route, "l2": "activations + weights + output exceed L2 at the default shape"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": ops / (kern_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": ops / (kern_ms * 1e-3) / 1e12 / peak, "traffic": None,
                     "kernel": "gemm_i8_grouped_tcgen05_kernel", "kernel_ms": kern_ms, "peak_source": peaks["_source"]},
    }
    weight.close()
    ctx.close()
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm", choices=["gemm", "decode", "grouped", "decoder", "prefill"])
    ap.add_argument("--model", default="qwen3", choices=["smollm2", "qwen3"], help="architecture of --workload decoder")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--group", type=int, default=128, help="scale group size of --workload grouped")
    ap.add_argument("--cpu-rows", type=int, default=512, help="row sample for the CPU legs")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    args = ap.parse_args()
    if args.rows is None:
        args.rows = 8 if args.workload == "decode" else 4096 if args.workload in ("grouped", "prefill") else 8192
    if args.workload == "prefill" and (args.k, args.n) == (4096, 14336):
        args.k = 576
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "decode":
        decode_arm(args)
    elif args.workload == "grouped":
        grouped_arm(args)
    elif args.workload == "decoder":
        decoder_arm(args)
    elif args.workload == "prefill":
        prefill_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
