// Inference GEMM over the sparse 1:4 + int4 "Wpair" layout:  Y[n, r] = bf16( sum_c X[n, c] * What[r, c] ).
//
// What is never materialised.  A packet is the two 64-bit words of one weight row for 64 input channels
// (forge_pack_sparse14 / pack_sparsegptq14_to_u64x2): per 32-channel half a bf16 scale, eight 2-bit positions (which
// of the four channels of a group survived) and eight 4-bit codes (value = code - 8).  So a half contributes
//   scale * sum_{i<8} X[n, base + 4 i + pos_i] * (code_i - 8)
// with exactly eight multiply-adds instead of thirty-two; pruned groups carry code 8 and add zero.
// Replaces moe_proj_unstructured_sparse14_int4symq_gemm, forge/backend/cuda/sparse14_gemm.cu:49-140 (kernel) and
// :282-374 (launcher), with the same arithmetic in the same order — fp32, fused multiply-adds, one rounding to bf16
// at the end — so the outputs are bit-identical to that kernel's.
//
// Decode-time shape (a few tokens per expert) is bound by the packet stream: 16 bytes per (row, 64 channels).
// One thread owns one output row, so a warp's packets for a channel block are one 512-byte line (Wpair is
// [G2, R, 2], rows contiguous); the token tile of X sits in shared memory as bf16 and is gathered by position
// directly (the 32 lanes of a warp read inside one 64-byte window: no bank conflict), instead of the reference's
// eight warp shuffles per token and half.  Packets are fetched four channel blocks ahead.  No padding of X or Y is
// needed: tails of N, R and C are handled in the kernel.
#include "common.cuh"

using namespace forge;

namespace {

constexpr int kRows = 128;      // output rows per CTA (one per thread)
constexpr int kAhead = 4;       // packets in flight per thread

template <int NT>
__global__ void __launch_bounds__(kRows) sparse14_gemm_kernel(const ulonglong2 *__restrict__ Wpair,
                                                              const __nv_bfloat16 *__restrict__ X, int64_t ldx,
                                                              __nv_bfloat16 *__restrict__ Y, int64_t N, int64_t R,
                                                              int64_t C, int64_t G2) {
    extern __shared__ __nv_bfloat16 Xs[];      // [NT][Cp], Cp = 64 G2 (zero padded)
    const int64_t Cp = G2 * 64;
    const int64_t n0 = (int64_t)blockIdx.x * NT;
    const int tid = threadIdx.x;
    const int64_t r = (int64_t)blockIdx.y * kRows + tid;
    const bool valid_r = r < R;
    for (int64_t t = tid; t < (int64_t)NT * Cp; t += kRows) {
        const int64_t n = n0 + t / Cp, c = t % Cp;
        Xs[t] = (n < N && c < C) ? X[n * ldx + c] : __float2bfloat16(0.0f);
    }
    __syncthreads();
    float acc[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n] = 0.0f;
    const ulonglong2 zero = make_ulonglong2(0ull, 0ull);
    ulonglong2 pk[kAhead];
#pragma unroll
    for (int d = 0; d < kAhead; ++d) pk[d] = (valid_r && d < G2) ? __ldg(Wpair + (int64_t)d * R + r) : zero;
    for (int64_t g2 = 0; g2 < G2; g2 += kAhead) {
#pragma unroll
        for (int d = 0; d < kAhead; ++d) {
            if (g2 + d >= G2) break;
            const ulonglong2 cur = pk[d];
            const int64_t nx = g2 + d + kAhead;
            pk[d] = (valid_r && nx < G2) ? __ldg(Wpair + nx * R + r) : zero;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint64_t u = half == 0 ? cur.x : cur.y;
                const uint32_t qw32 = (uint32_t)u, hi = (uint32_t)(u >> 32);
                const uint32_t idx16 = hi & 0xFFFFu;
                const float scale = __uint_as_float(hi & 0xFFFF0000u);      // the bf16 scale, widened exactly
                const __nv_bfloat16 *xb = Xs + (g2 + d) * 64 + half * 32;
                float sum[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) sum[n] = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t ch = 4u * i + ((idx16 >> (2 * i)) & 3u);
                    const float w = (float)(int)((qw32 >> (4 * i)) & 0xFu) - 8.0f;
#pragma unroll
                    for (int n = 0; n < NT; ++n) sum[n] = fmaf(__bfloat162float(xb[n * Cp + ch]), w, sum[n]);
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) acc[n] = fmaf(sum[n], scale, acc[n]);
            }
        }
    }
    if (valid_r) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
            if (n0 + n < N) Y[(n0 + n) * R + r] = __float2bfloat16_rn(acc[n]);
    }
}

template <int NT>
int launch(const ulonglong2 *W, const __nv_bfloat16 *X, int64_t ldx, __nv_bfloat16 *Y, int64_t N, int64_t R, int64_t C,
           int64_t G2, cudaStream_t st) {
    const size_t smem = (size_t)NT * G2 * 64 * sizeof(__nv_bfloat16);
    if (smem > 200 * 1024) return -1;
    cudaFuncSetAttribute(sparse14_gemm_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   // per device
    dim3 grid((unsigned)cdiv(N, NT), (unsigned)cdiv(R, kRows));
    sparse14_gemm_kernel<NT><<<grid, kRows, smem, st>>>(W, X, ldx, Y, N, R, C, G2);
    FORGE_NOTE_LAUNCH();
    return 0;
}

}  // namespace

extern "C" int forge_sparse14_gemm(const uint64_t *wpair, const void *X_bf16, int64_t ldx, int64_t N, int64_t R, int64_t C,
                                   void *Y_bf16, void *stream) {
    FORGE_REQUIRE(wpair && X_bf16 && Y_bf16, "null pointer");
    FORGE_REQUIRE(N >= 0 && R > 0 && C > 0 && ldx >= C, "bad sizes");
    FORGE_REQUIRE((uintptr_t)wpair % 16 == 0, "wpair must be 16-byte aligned");
    if (N == 0) return FORGE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t G2 = cdiv(C, 64);
    const ulonglong2 *W = reinterpret_cast<const ulonglong2 *>(wpair);
    const __nv_bfloat16 *X = (const __nv_bfloat16 *)X_bf16;
    __nv_bfloat16 *Y = (__nv_bfloat16 *)Y_bf16;
    // token tile: as many tokens per pass over the packets as there are (up to 8) and as shared memory holds
    int rc = -1;
    if (N >= 8) rc = launch<8>(W, X, ldx, Y, N, R, C, G2, st);
    if (rc != 0 && N >= 4) rc = launch<4>(W, X, ldx, Y, N, R, C, G2, st);
    if (rc != 0 && N >= 2) rc = launch<2>(W, X, ldx, Y, N, R, C, G2, st);
    if (rc != 0) rc = launch<1>(W, X, ldx, Y, N, R, C, G2, st);
    if (rc != 0) {
        set_error("forge_sparse14_gemm: C = %lld does not fit the shared-memory token tile", (long long)C);
        return FORGE_ERR_UNSUPPORTED;
    }
    return check_launch("forge_sparse14_gemm");
}
