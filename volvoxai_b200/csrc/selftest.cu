// Device self-tests behind the diagnostic entry points (diag.h): the bounded-wait expiry path
// and the exhaustive check of the constant-divisor division.  Neither faults, traps nor waits
// without a limit.
#include "tcgen05.cuh"

namespace vxb {

namespace {

using namespace tc;

// One CTA: TMEM allocated, an mbarrier nobody arrives on, one thread waits for it with the
// launch's limit.  On expiry the status word is raised, TMEM is freed and the kernel returns.
__global__ void __launch_bounds__(128, 1)
wait_expiry_kernel(int* status) {
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_ptr;
    __shared__ int abort_flag[2];
    const uint32_t warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); arm_abort(abort_flag, status); fence_barrier_init(); }
    if (warp == 0) { tmem_alloc(smem_u32(&tmem_ptr), 32); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_ptr;
    if (threadIdx.x == 32) (void)mbar_wait(smem_u32(&bar), 0u, abort_flag);   // phase 0 never completes
    tc_fence_before();
    __syncthreads();
    if (abort_flag[0] && threadIdx.x == 0 && status) atomicExch(status, 5);
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem_base, 32);
}

__device__ __forceinline__ uint32_t lcg(uint32_t& s) { s = s * 1664525u + 1013904223u; return s; }

// Every divisor significand (grid-stride), numerators around every half-integer quotient and
// pseudo-random ones: div_const against the IEEE divide, bit for bit.
__global__ void __launch_bounds__(256)
div_const_check_kernel(int exponent, uint32_t neighbours, uint32_t samples, unsigned long long* mismatches,
                       unsigned long long* checked) {
    unsigned long long bad = 0, done = 0;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t sig = blockIdx.x * blockDim.x + threadIdx.x; sig < 0x7fffffu; sig += stride) {   // all-ones excluded
        const float d = __uint_as_float(((uint32_t)(exponent + 127) << 23) | sig);
        const float rcp = __frcp_rn(d);
        for (uint32_t h = 0; h < 128; h++) {
            const float t = (float)h + 0.5f;
            const uint32_t a0 = __float_as_uint(__fmul_rn(t, d));
            for (int j = -(int)neighbours; j <= (int)neighbours; j++) {
                const float a = __uint_as_float(a0 + (uint32_t)j);
                const float want = __fdiv_rn(a, d), got = div_const(a, d, rcp);
                bad += __float_as_uint(want) != __float_as_uint(got);
                // the sign-symmetric case
                bad += __float_as_uint(__fdiv_rn(-a, d)) != __float_as_uint(div_const(-a, d, rcp));
                done += 2;
            }
        }
        uint32_t seed = sig * 2654435761u + 12345u;
        for (uint32_t i = 0; i < samples; i++) {
            // quotients between 2^-20 and 2^8
            const uint32_t r = lcg(seed);
            const int e = exponent + (int)(lcg(seed) % 29u) - 20;
            const float a = __uint_as_float(((uint32_t)(e + 127) << 23) | (r & 0x7fffffu));
            bad += __float_as_uint(__fdiv_rn(a, d)) != __float_as_uint(div_const(a, d, rcp));
            done++;
        }
    }
    // block reduction, one atomic per block
    __shared__ unsigned long long s_bad[8], s_done[8];
    for (int off = 16; off > 0; off >>= 1) {
        bad += __shfl_xor_sync(0xffffffffu, bad, off);
        done += __shfl_xor_sync(0xffffffffu, done, off);
    }
    if ((threadIdx.x & 31) == 0) { s_bad[threadIdx.x >> 5] = bad; s_done[threadIdx.x >> 5] = done; }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long b = 0, c = 0;
        for (int i = 0; i < 8; i++) { b += s_bad[i]; c += s_done[i]; }
        atomicAdd(mismatches, b);
        atomicAdd(checked, c);
    }
}

// Cross-GPU barrier of the N-sharded linear: thread t tells peer t that this rank has reached `epoch`
// (a release store at system scope into the peer's flag array, after a system-scope fence that
// orders this GPU's earlier peer stores before it) and then waits, with the launch's limit, until
// peer t's flag in this GPU's own array has reached the epoch too.  Every rank runs this kernel
// on its own GPU at the same point of its stream, so each waits only for kernels that are already
// queued on other GPUs; a rank that never arrives makes the wait run out, which raises the
// status word instead of hanging.
__global__ void __launch_bounds__(32, 1)
peer_barrier_kernel(uint32_t* my_flags, PeerBarrierArgs args, int* status) {
    const uint32_t t = threadIdx.x;
    // launched as a programmatic dependent: resident while the kernel before it still runs, and letting the
    // launch after it become resident in turn; the wait returns when that kernel (the GEMM whose peer stores
    // this barrier orders) has completed and its stores have been performed
    pdl_release();
    pdl_wait();
    if (t >= args.n_peers) return;
    __threadfence_system();
    uint32_t* remote = args.peer_flags[t] + args.my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(args.epoch) : "memory");
    const uint32_t* mine = my_flags + args.peer_ranks[t];
    int limit = status ? status[1] : 0;
    if (limit <= 0) limit = kDefaultWaitLimitKcycles;
    const long long t0 = clock64();
    for (uint32_t spins = 0;; spins++) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int32_t)(seen - args.epoch) >= 0) break;
        if ((spins & 63u) == 63u && clock64() - t0 > ((long long)limit << 10)) {
            if (status) atomicExch(status, 6);
            break;
        }
    }
}

}  // namespace

cudaError_t launch_peer_barrier(uint32_t* my_flags, const PeerBarrierArgs& args, int* status, cudaStream_t stream) {
    return launch_pdl(peer_barrier_kernel, dim3(1), dim3(32), 0, stream, my_flags, args, status);
}

cudaError_t launch_wait_expiry(int* status, cudaStream_t stream) {
    wait_expiry_kernel<<<1, 128, 0, stream>>>(status);
    return cudaGetLastError();
}

cudaError_t launch_div_const_check(int exponent, uint32_t neighbours, uint32_t samples, unsigned long long* mismatches,
                                   unsigned long long* checked, int sm_count, cudaStream_t stream) {
    div_const_check_kernel<<<sm_count * 8, 256, 0, stream>>>(exponent, neighbours, samples, mismatches, checked);
    return cudaGetLastError();
}

}  // namespace vxb
