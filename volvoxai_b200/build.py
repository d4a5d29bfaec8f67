"""Builds libvxb200.so (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m volvoxai_b200.build            # rebuild when sources are newer
    python -m volvoxai_b200.build --force

nvcc cross-compiles without a GPU present.  cudart is linked statically so the
library has no run-time dependency beyond the driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libvxb200.so")
SOURCES = ["api.cu", "plan.cu", "package.cu", "selftest.cu", "quantize.cu", "gemv.cu", "gemm_tcgen05.cu", "gemm_pair_tcgen05.cu", "gemm_wide_tcgen05.cu", "gemm_grouped_tcgen05.cu", "decode_tcgen05.cu", "decode_rows.cu", "boundary_ops.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "tcgen05.cuh"), os.path.join(CSRC, "diag.h"), os.path.join(ROOT, "include", "vxb200_w8a8.h"), os.path.join(ROOT, "include", "vxb200_plan.h"), os.path.join(ROOT, "include", "vxb200_package.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--fmad=false",            # every epilogue multiply/add is separately rounded
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static", "-shared", "--threads", "0",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libvxb200.so")
    return LIB


PROVIDER_LIB = os.path.join(PKG, "libvxb200_provider.so")
PROVIDER_SRC = os.path.join(PKG, "provider", "vxb200_provider.c")


def reference_include() -> str | None:
    """Where the reference's public headers lie: $VX_REFERENCE/native/include, else a checkout named
    `reference` beside this repository; None when neither exists."""
    root = os.environ.get("VX_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    inc = os.path.join(root, "native", "include")
    return inc if os.path.exists(os.path.join(inc, "volvoxai_backend.h")) else None


def build_provider(force: bool = False) -> str | None:
    """Builds libvxb200_provider.so (the VxBackendProvider of this route) against the reference's own
    header.  Needs the reference checkout; returns None (and keeps any prebuilt library) without it."""
    inc = reference_include()
    if inc is None:
        return PROVIDER_LIB if os.path.exists(PROVIDER_LIB) else None
    deps = [PROVIDER_SRC, os.path.join(ROOT, "include", "vxb200_package.h"), os.path.join(inc, "volvoxai_backend.h")]
    if not force and os.path.exists(PROVIDER_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(PROVIDER_LIB) for d in deps):
        return PROVIDER_LIB
    cmd = ["gcc", "-std=gnu11", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-I", inc, "-o", PROVIDER_LIB, PROVIDER_SRC,
           "-L", PKG, "-l:libvxb200.so", "-Wl,-rpath,$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("gcc failed building libvxb200_provider.so")
    return PROVIDER_LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--force" in sys.argv)
    print(LIB)
    print(build_provider(force="--force" in sys.argv))
