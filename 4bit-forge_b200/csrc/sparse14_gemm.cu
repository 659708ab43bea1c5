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

// acc[n] = sum over the packets of weight row r (Wpair = [G2, R] packets of one matrix) against the token tile Xs
// ([NT][Cp] bf16 in shared memory), in the reference kernel's order of operations.
template <int NT>
__device__ __forceinline__ void row_times_tile(const ulonglong2 *__restrict__ Wpair, int64_t r, int64_t R, int64_t G2,
                                               bool valid_r, const __nv_bfloat16 *Xs, int64_t Cp, float (&acc)[NT]) {
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
}

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
    row_times_tile<NT>(Wpair, r, R, G2, valid_r, Xs, Cp, acc);
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


// ---------------------------------------------------------------------------------------------------------------
// Grouped forms for a mixture-of-experts layer whose routed rows are sorted by expert ("permuted"): rows
// [offsets[e], offsets[e+1]) belong to expert e, W = [E, G2, R] packets.  Interfaces of
// usp14w4a16sym_sm80_fused_moe_w13_gemm / _w2_gemm (forge/backend/cuda/fused_moe_usp14w4a16_gemm.cu:1028-1140):
//   W13: R = 2 I, gate rows [0, I), up rows [I, 2 I) (:722-723);  X2[m, i] = bf16( silu(g) * u ) with g, u the fp32
//        sums and silu(g) = g / (1 + expf(-g)) (:398-439): one rounding, at the store;
//   W2:  Y[m, r] = bf16( sum ), the per-expert GEMM above on every expert's rows.
// `active` lists the experts to run (the reference's `U`); `token_idx`, when given, maps a permuted position to its
// row of X, so the layer input needs no permuted copy.  Same thread-per-row packet stream as above; a CTA walks the
// token tiles of its (expert, row tile) with a stride of gridDim.x.
// ---------------------------------------------------------------------------------------------------------------
template <int NT, bool SWIGLU>
__global__ void __launch_bounds__(kRows) sparse14_moe_kernel(const ulonglong2 *__restrict__ W,
                                                             const __nv_bfloat16 *__restrict__ X, int64_t ldx,
                                                             int64_t x_rows, const int32_t *__restrict__ token_idx,
                                                             const int64_t *__restrict__ offsets,
                                                             const int32_t *__restrict__ active,
                                                             __nv_bfloat16 *__restrict__ out, int64_t N, int64_t R,
                                                             int64_t C, int64_t G2) {
    extern __shared__ __nv_bfloat16 Xs[];      // [NT][Cp]
    const int64_t Cp = G2 * 64;
    const int64_t e = (int64_t)active[blockIdx.y];
    const int64_t m_begin = max((int64_t)0, offsets[e]), m_end = min(N, offsets[e + 1]);
    const int64_t Rout = SWIGLU ? R / 2 : R;
    const int tid = threadIdx.x;
    const int64_t r = (int64_t)blockIdx.z * kRows + tid;
    const bool valid_r = r < Rout;
    const ulonglong2 *We = W + e * G2 * R;
    for (int64_t m0 = m_begin + (int64_t)blockIdx.x * NT; m0 < m_end; m0 += (int64_t)gridDim.x * NT) {
        for (int64_t t = tid; t < (int64_t)NT * Cp; t += kRows) {
            const int64_t m = m0 + t / Cp, c = t % Cp;
            __nv_bfloat16 v = __float2bfloat16(0.0f);
            if (m < m_end && c < C) {
                const int64_t row = token_idx ? (int64_t)token_idx[m] : m;
                if (row >= 0 && row < x_rows) v = X[row * ldx + c];
            }
            Xs[t] = v;
        }
        __syncthreads();
        float acc[NT];
        row_times_tile<NT>(We, r, R, G2, valid_r, Xs, Cp, acc);
        if (SWIGLU) {
            float up[NT];
            row_times_tile<NT>(We, r + Rout, R, G2, valid_r, Xs, Cp, up);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float g = acc[n];
                const float sig = 1.0f / (1.0f + expf(-g));
                acc[n] = (g * sig) * up[n];
            }
        }
        if (valid_r) {
#pragma unroll
            for (int n = 0; n < NT; ++n)
                if (m0 + n < m_end) out[(m0 + n) * Rout + r] = __float2bfloat16_rn(acc[n]);
        }
        __syncthreads();
    }
}

template <int NT, bool SWIGLU>
int launch_moe(const ulonglong2 *W, const __nv_bfloat16 *X, int64_t ldx, int64_t x_rows, const int32_t *token_idx,
               const int64_t *offsets, const int32_t *active, int n_active, __nv_bfloat16 *out, int64_t N, int64_t R,
               int64_t C, int64_t G2, cudaStream_t st) {
    const size_t smem = (size_t)NT * G2 * 64 * sizeof(__nv_bfloat16);
    if (smem > 200 * 1024) return -1;
    cudaFuncSetAttribute(sparse14_moe_kernel<NT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int64_t Rout = SWIGLU ? R / 2 : R;
    // token-tile slots per (expert, row tile): enough CTAs for a few waves, never more than the tiles of the whole
    // list (an expert with more tiles than slots loops)
    const int64_t tiles = cdiv(N, (int64_t)NT), per = cdiv((int64_t)148 * 8, (int64_t)n_active * cdiv(Rout, (int64_t)kRows));
    dim3 grid((unsigned)max((int64_t)1, min(tiles, per)), (unsigned)n_active, (unsigned)cdiv(Rout, (int64_t)kRows));
    sparse14_moe_kernel<NT, SWIGLU><<<grid, kRows, smem, st>>>(W, X, ldx, x_rows, token_idx, offsets, active, out, N, R,
                                                               C, G2);
    FORGE_NOTE_LAUNCH();
    return 0;
}

template <bool SWIGLU>
int moe_entry(const char *what, const uint64_t *W, const void *X_bf16, int64_t ldx, int64_t x_rows,
              const int32_t *token_idx, const int64_t *offsets, const int32_t *active, int n_active, int64_t N,
              int64_t R, int64_t C, void *out_bf16, void *stream) {
    if (!(W && X_bf16 && offsets && active && out_bf16)) { set_error("%s: null pointer", what); return FORGE_ERR_INVALID; }
    if (!(N >= 0 && R > 0 && C > 0 && ldx >= C && x_rows >= 0 && n_active >= 0 && n_active <= 65535) ||
        (SWIGLU && (R & 1))) {
        set_error("%s: bad sizes", what);
        return FORGE_ERR_INVALID;
    }
    if ((uintptr_t)W % 16 != 0) { set_error("%s: W must be 16-byte aligned", what); return FORGE_ERR_INVALID; }
    if (N == 0 || n_active == 0) return FORGE_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t G2 = cdiv(C, (int64_t)64);
    const ulonglong2 *Wp = reinterpret_cast<const ulonglong2 *>(W);
    const __nv_bfloat16 *X = (const __nv_bfloat16 *)X_bf16;
    __nv_bfloat16 *out = (__nv_bfloat16 *)out_bf16;
    // decode-time lists hold a few rows per expert: eight-token tiles, smaller when shared memory asks for it
    int rc = launch_moe<8, SWIGLU>(Wp, X, ldx, x_rows, token_idx, offsets, active, n_active, out, N, R, C, G2, st);
    if (rc != 0) rc = launch_moe<4, SWIGLU>(Wp, X, ldx, x_rows, token_idx, offsets, active, n_active, out, N, R, C, G2, st);
    if (rc != 0) rc = launch_moe<2, SWIGLU>(Wp, X, ldx, x_rows, token_idx, offsets, active, n_active, out, N, R, C, G2, st);
    if (rc != 0) rc = launch_moe<1, SWIGLU>(Wp, X, ldx, x_rows, token_idx, offsets, active, n_active, out, N, R, C, G2, st);
    if (rc != 0) {
        set_error("%s: C = %lld does not fit the shared-memory token tile", what, (long long)C);
        return FORGE_ERR_UNSUPPORTED;
    }
    return check_launch(what);
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

extern "C" int forge_sparse14_moe_w13_swiglu(const uint64_t *w13, const void *X_bf16, int64_t ldx, int64_t x_rows,
                                             const int32_t *token_idx, const int64_t *offsets, const int32_t *active,
                                             int n_active, int64_t N, int64_t R, int64_t C, void *X2_bf16,
                                             void *stream) {
    return moe_entry<true>("forge_sparse14_moe_w13_swiglu", w13, X_bf16, ldx, x_rows, token_idx, offsets, active,
                           n_active, N, R, C, X2_bf16, stream);
}

extern "C" int forge_sparse14_moe_w2(const uint64_t *w2, const void *X2_bf16, int64_t ldx, int64_t x_rows,
                                     const int32_t *token_idx, const int64_t *offsets, const int32_t *active,
                                     int n_active, int64_t N, int64_t R, int64_t C, void *Y_bf16, void *stream) {
    return moe_entry<false>("forge_sparse14_moe_w2", w2, X2_bf16, ldx, x_rows, token_idx, offsets, active, n_active, N,
                            R, C, Y_bf16, stream);
}
