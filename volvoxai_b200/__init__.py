"""B200-native (sm_100a) W8A8 linear: per-token int8 activation quantization, a
TMA-fed tcgen05 kind::i8 GEMM with TMEM accumulators (or a bandwidth-bound GEMV
for decode), and a fused dequant+bias / requant epilogue, behind the C ABI in
include/vxb200_w8a8.h.  See volvoxai_b200.w8a8 for the host-side interface."""
from .w8a8 import *  # noqa: F401,F403
