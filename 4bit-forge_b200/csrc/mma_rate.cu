// Diagnostic: how many cycles one tcgen05.mma kind::tf32 M128 x N x K8 costs on this part when a single thread issues
// them back to back (operands in shared memory, MN-major, fp32 accumulator in tensor memory), with every SM busy.
//
// The column solver and the blocked Cholesky are built from exactly this instruction (TF32 x3), so its issue rate is
// their ceiling: 128 * N * 8 * 2 flop per that many cycles per SM.  The benchmark measures it on the GPU it runs on
// instead of assuming a TF32 peak.  The operands are zeros: nothing is computed that anyone reads.
#include "common.cuh"
#include "tcgen05.cuh"

using namespace forge;

namespace {

__global__ void __launch_bounds__(128) mma_rate_kernel(int N, int iters, int pattern, long long *cycles, int32_t *status) {
    using namespace forge::tc;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *buf = smem_raw + (base - smem_u32(smem_raw));
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5;
    // A piece (4 KB) at 0, B pieces (up to N = 256: 8 KB) at 8 KB
    for (int i = tid; i < 16 * 1024 / 4; i += 128)
        reinterpret_cast<float *>(buf)[i] = pattern ? 1e-3f * (float)((i * 2654435761u >> 20) & 1023u) - 0.5f : 0.0f;
    if (tid == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)),
                     "r"(256u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    if (tid == 0) {
        const uint32_t id = idesc_tf32((uint32_t)N);
        const uint64_t a = make_desc_tf32(base), b = make_desc_tf32(base + 8192);
        const long long t0 = clock64();
        for (int i = 0; i < iters; ++i) umma_tf32(tmem, a, b, id, i > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar));
        const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag);      // bounded
        const long long t1 = clock64();
        if (blockIdx.x == 0) cycles[0] = t1 - t0;
        if (!ok && status) atomicExch(status, FORGE_ERR_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

}  // namespace

extern "C" int forge_selftest_mma_rate(int N, int iters, int pattern, int64_t *cycles, int32_t *status, void *stream) {
    FORGE_REQUIRE(cycles, "null pointer");
    FORGE_REQUIRE(N == 64 || N == 128 || N == 256, "N must be 64, 128 or 256");
    FORGE_REQUIRE(iters > 0 && iters <= 100000, "iters must be in [1, 100000]");
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = 16 * 1024 + 1024;
    mma_rate_kernel<<<sms, 128, smem, (cudaStream_t)stream>>>(N, iters, pattern, reinterpret_cast<long long *>(cycles), status);
    FORGE_NOTE_LAUNCH();
    return check_launch("forge_selftest_mma_rate");
}
