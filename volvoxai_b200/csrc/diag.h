/*
 * diag.h - diagnostic and self-test entry points of libvxb200.so.
 *
 * Not part of the drop-in boundary (include/vxb200_w8a8.h): nothing here has a
 * counterpart a host of the reference would bind.  The tests and the benchmark
 * use these to measure the hardware facts the kernels were sized by, to prove
 * arithmetic shortcuts exhaustively on the device, and to exercise failure
 * paths from the host without faulting a GPU.
 */
#ifndef VXB200_DIAG_H
#define VXB200_DIAG_H

#include "../../include/vxb200_w8a8.h"

#ifdef __cplusplus
extern "C" {
#endif

/* While device_stamps is not NULL, every launch of the decode kernel (route DECODE) writes 8
 * %globaltimer values (ns) per CTA into device_stamps[cta*8 + slot]: 0 entry, 1 prologue done,
 * 2 first weight tile landed, 3 last MMA issued, 4 accumulator ready, 5 last output stored,
 * 6 preceding kernel finished (programmatic dependency), 7 exit.  The buffer must hold
 * 8 * ceil(d_out / channels-per-CTA) <= 8 * d_out values.  The pointer is read at launch (a
 * captured launch keeps the pointer it was captured with). */
VXB_API int vxb_context_trace(VxbContext* ctx, unsigned long long* device_stamps);

/* On one SM, `iters` rounds of `per_commit` kind::i8 MMAs of shape m x n x 32 cycling through
 * `accs` TMEM accumulators, one commit + wait per round; returns SM clocks per MMA. */
VXB_API int vxb_measure_mma_issue(VxbContext* ctx, uint32_t m, uint32_t n, uint32_t accs, uint32_t per_commit,
                          uint32_t iters, double* cycles_per_mma);

/* Limit of every bounded device wait of this context's launches, in SM clocks (0 restores the
 * default of about 2 s).  Read by a kernel when it starts. */
VXB_API int vxb_context_set_wait_limit(VxbContext* ctx, uint64_t cycles);

/* Self-test of the bounded-wait path: one CTA allocates TMEM, initialises an mbarrier that
 * nothing ever arrives on and waits for it with the context's limit.  The wait expires, the
 * kernel raises the status word, frees its TMEM and returns; the next
 * vxb_context_synchronize() therefore returns -1 once and the context stays usable.  No trap,
 * no fault, no unbounded wait.  Returns 1 when the kernel was launched. */
VXB_API int vxb_selftest_wait_expiry(VxbContext* ctx);

/* Exhaustive device check of the constant-divisor division used by the quantizer and the
 * requantizing epilogue (div_const: correctly rounded reciprocal + two FMA corrections) against
 * the IEEE divide.  For every one of the 2^23 significands of the divisor d (exponent
 * `divisor_exponent`, unbiased), numerators are taken around every half-integer quotient
 * t = 0.5 .. 127.5 (a = RN(t * d) and its `neighbours` fp32 neighbours on both sides) plus
 * `samples` pseudo-random numerators per divisor; *mismatches receives how many quotients
 * differ in any bit (divisors with an all-ones significand are skipped: the kernels use the
 * IEEE divide for them).  *checked receives the number of divisions compared. */
VXB_API int vxb_selftest_div_const(VxbContext* ctx, int divisor_exponent, uint32_t neighbours, uint32_t samples,
                           uint64_t* mismatches, uint64_t* checked);

/* Host-side failure injection, the counterpart of the reference's recording fakes with
 * fail_at / fail_view (tools/tests/test_cuda_packed_decode.py:135-171).  kind 1: the
 * `countdown`-th kernel launch from now is refused as if the driver had rejected it (the entry
 * returns -1: work may already be queued); kind 2: the `countdown`-th scratch allocation from
 * now is refused (the entry returns 0 before the output is touched).  countdown 0 disarms.
 * Process-wide; meant for single-threaded tests. */
enum { VXB_INJECT_LAUNCH = 1, VXB_INJECT_ALLOCATION = 2 };
VXB_API void vxb_inject_failure(int kind, uint32_t countdown);

/* Internal tunables by name (experiments; every default is what the library ships with):
 *   "decode.pair_share_bytes"   largest per-CTA weight share run as two CTAs per SM
 *   "decode.l2_prefetch"        1: the decode kernel's weight producers ask L2 for the tile one
 *                               ring-depth ahead of the copy they issue
 *   "decode.fused_max_rows"     fp32 rows up to which the automatic route takes the decode kernel's single-launch
 *                               form (default 2; the kernel serves up to 8)
 *   "gemm.overlap_ratio"        rows_first / rows_rest >= this / d_out when a batch is cut in two (1755)
 *   "gemm.overlap_k1"           1: batches of 2048 rows or more are cut in two so that the quantizer of the
 *                               later rows runs under the GEMM of the first ones (default 0: measured slower)
 *   "gemm.overlap_gather"       1: the same split for a link-bound fused all-gather launch, with the 128-register
 *                               build of its kernel (default 0: measured slower)
 *   "gemm.gather_tma"           1 (default): the fused all-gather's flush is one TMA tile store per destination and
 *                               warp; 0: per-lane 16-byte stores of 256-byte row segments
 * Returns 1, or 0 for an unknown name. */
VXB_API int vxb_tune(const char* name, int64_t value);

#ifdef __cplusplus
}
#endif
#endif /* VXB200_DIAG_H */
