// Fused GPTQ / SparseGPT-1:4 column solver.
//
// The rows of a weight matrix (the R axis) are independent given the factor U, so a CTA owns a strip
// of 128 rows — one thread per row — and walks ALL column blocks itself: no grid-wide sync and one
// launch per batch of matrices, instead of the reference's C/32 kernel launches plus C/32 skinny
// GEMMs per matrix (forge/backend/cuda/solver.cu:124-151).
//
// For a 128-column block starting at column bs a thread holds its row's 128 values in registers:
//   1. x[k] = W[bs+k] - sum_{j<bs} err_j * U[j, bs+k]      lazy ("left-looking") update from every
//      earlier column: the errors E[j, r] stream from global memory, the U panel [32 x 128] is staged
//      in shared memory by cp.async, double buffered;
//   2. four 32-column sub-blocks: quantise column t, err = x_t - deq_t, x_k -= U[t,k]*err for the
//      rest of the sub-block (registers, U row broadcast from shared memory), then the sub-block's 32
//      errors update the remaining columns of the block.
// The arithmetic per element is the reference's (quantize_scalar, solver.cu:9-22; x_k update by
// fmaf(-u, err, x), solver.cu:90-93); only the summation order of the lazy update differs from the
// reference's fp32 GEMM.  The SparseGPT variant adds the keep-1-of-4 choice on the error-compensated
// values (solver_sparsegptq14.cu:80-120).
//
// Layouts: the kernel works on Wt [C,R] (permuted columns, rows contiguous) so that every global
// access is coalesced across the 128 row-threads; the batched entry point builds Wt from W [R,C] with
// a tiled transpose-gather and scatters the codes back to [R,C] in the original column order.
#include "common.cuh"

using namespace forge;

namespace {

constexpr int kBlk = 128;     // columns per block == rows per CTA == threads per CTA
constexpr int kSub = 32;      // columns per sub-block
constexpr int kChunkFloats = kSub * kBlk;
constexpr float kEps = 1e-12f;

struct SolveParams {
    float *Wt;             // [nb][C][R]  in: weights (permuted, transposed); see E / write_deq
    float *E;              // [nb][C][R]  error rows; may alias Wt when write_deq == 0
    const float *U;        // [nu][C][C]
    const float *uvec;     // [nu][C]     sparse only: 1/diag (uvec_is_diag==0) or diag (==1)
    const int32_t *u_map;  // [nb] or null
    const float *scales;   // MODE 0: [nb][R][G]   MODE 1: [nb][C][R]
    const float *qzeros;
    const int32_t *perm;   // [nu][C] or null (MODE 0)
    uint8_t *q;            // [nb][C][R]
    uint32_t *M;           // [nb][ceil(C/32)][R]
    int64_t R, C, G;
    int gs, maxq, write_deq, uvec_is_diag;
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool pred) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Stage U[j0..j0+32, bs..bs+128) (and optionally E[j0..j0+32, r0..r0+128)) into shared memory.
__device__ __forceinline__ void load_chunk(float *us, float *es, const float *U, const float *E, int64_t C,
                                           int64_t R, int64_t j0, int64_t bs, int64_t r0, bool want_e,
                                           bool vecU, bool vecE, int tid) {
    if (vecU) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int v = tid + 128 * i;  // float4 index in the chunk: row = v/32, col4 = v%32
            const int jj = v >> 5, k = (v & 31) * 4;
            const bool ok = (j0 + jj < C) && (bs + k < C);
            const float *src = ok ? (U + (j0 + jj) * C + bs + k) : U;
            cp_async16(us + jj * kBlk + k, src, ok);
        }
    } else {
        for (int v = tid; v < kChunkFloats; v += 128) {
            const int jj = v >> 7, k = v & 127;
            us[v] = ((j0 + jj < C) && (bs + k < C)) ? U[(j0 + jj) * C + bs + k] : 0.0f;
        }
    }
    if (want_e) {
        if (vecE) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int v = tid + 128 * i;
                const int jj = v >> 5, k = (v & 31) * 4;
                const bool ok = (j0 + jj < C) && (r0 + k < R);
                const float *src = ok ? (E + (j0 + jj) * R + r0 + k) : E;
                cp_async16(es + jj * kBlk + k, src, ok);
            }
        } else {
            for (int v = tid; v < kChunkFloats; v += 128) {
                const int jj = v >> 7, k = v & 127;
                es[v] = ((j0 + jj < C) && (r0 + k < R)) ? E[(j0 + jj) * R + r0 + k] : 0.0f;
            }
        }
    }
}

// forge/backend/cuda/solver.cu:9-22 with the multiply-add of `x * inv_s + q0` fused, as nvcc's default
// contraction does for the reference build.
__device__ __forceinline__ void quantize_scalar(float x, float s, float q0, float maxq, float &err, float &deq,
                                                uint8_t &qb) {
    const float inv_s = __fdiv_rn(1.0f, __fadd_rn(s, kEps));
    // clamp(rint(b), 0, maxq) == rint(clamp(b, 0, maxq)), and rint on [0, 2^22) is an add of 1.5 * 2^23
    float q = fminf(fmaxf(fmaf(x, inv_s, q0), 0.0f), maxq);
    q = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
    deq = fmaf(q, s, -__fmul_rn(q0, s));
    err = __fsub_rn(x, deq);
    qb = (uint8_t)(int)q;
}

template <int MODE, bool SPARSE, int S>
__device__ __forceinline__ void solve_subblock(float (&x)[kBlk], const float *us, float *es,
                                               const float *uinv_s, const SolveParams &p, int b, int u,
                                               int64_t bs, int64_t r, bool active, float *Wt, float *E, int tid) {
    const int64_t R = p.R, C = p.C;
    const float maxq = (float)p.maxq;
    uint32_t maskbits = 0u;
#pragma unroll
    for (int t = 0; t < kSub; ++t) {
        const int kk = S * kSub + t;
        const int64_t c = bs + kk;
        float err = 0.0f;
        if (c < C) {
            if (SPARSE && (t % 4 == 0)) {
                float best = -1e30f;
                int bidx = -1;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (active && (c + k < C)) {
                        const float sc = fabsf(__fmul_rn(x[kk + k], uinv_s[kk + k]));
                        if (best < sc) { best = sc; bidx = k; }
                    }
                }
                if (bidx > -1) maskbits |= (1u << (t + bidx));
            }
            float deq = 0.0f;
            uint8_t qb = 0;
            const bool keep = SPARSE ? (((maskbits >> t) & 1u) != 0u) : true;
            if (keep && (active || !SPARSE)) {
                float s = 1.0f, q0 = 0.0f;
                if (active) {
                    if (MODE == 0) {
                        const int64_t oc = p.perm ? (int64_t)p.perm[(int64_t)u * C + c] : c;
                        const int64_t gi = ((int64_t)b * R + r) * p.G + oc / p.gs;
                        s = __ldg(p.scales + gi);
                        q0 = __ldg(p.qzeros + gi);
                    } else {
                        const int64_t gi = ((int64_t)b * C + c) * R + r;
                        s = __ldg(p.scales + gi);
                        q0 = __ldg(p.qzeros + gi);
                    }
                }
                quantize_scalar(x[kk], s, q0, maxq, err, deq, qb);
            } else {
                err = x[kk];  // pruned weight: the whole value is the error (solver_sparsegptq14.cu:118-120)
            }
            if (active) {
                p.q[((int64_t)b * C + c) * R + r] = qb;
                if (p.write_deq) Wt[c * R + r] = deq;
                E[c * R + r] = err;
            }
        }
        es[t * kBlk + tid] = err;
        // rank-1 update of the rest of the sub-block; U row t broadcast from shared memory
        const float4 *urow = reinterpret_cast<const float4 *>(us + t * kBlk + S * kSub);
#pragma unroll
        for (int k4 = 0; k4 < kSub / 4; ++k4) {
            if (4 * k4 + 3 > t) {
                const float4 u4 = urow[k4];
                if (4 * k4 + 0 > t) x[S * kSub + 4 * k4 + 0] = fmaf(-u4.x, err, x[S * kSub + 4 * k4 + 0]);
                if (4 * k4 + 1 > t) x[S * kSub + 4 * k4 + 1] = fmaf(-u4.y, err, x[S * kSub + 4 * k4 + 1]);
                if (4 * k4 + 2 > t) x[S * kSub + 4 * k4 + 2] = fmaf(-u4.z, err, x[S * kSub + 4 * k4 + 2]);
                if (4 * k4 + 3 > t) x[S * kSub + 4 * k4 + 3] = fmaf(-u4.w, err, x[S * kSub + 4 * k4 + 3]);
            }
        }
    }
    if (SPARSE && active && (bs + S * kSub < C))
        p.M[((int64_t)b * ((C + 31) / 32) + ((bs + S * kSub) >> 5)) * R + r] = maskbits;
    // the sub-block's errors update the later columns of the block
    if (S < 3) {
#pragma unroll 2
        for (int t = 0; t < kSub; ++t) {
            const float e = es[t * kBlk + tid];
            const float4 *urow = reinterpret_cast<const float4 *>(us + t * kBlk);
#pragma unroll
            for (int k4 = (S + 1) * (kSub / 4); k4 < kBlk / 4; ++k4) {
                const float4 u4 = urow[k4];
                x[4 * k4 + 0] = fmaf(-u4.x, e, x[4 * k4 + 0]);
                x[4 * k4 + 1] = fmaf(-u4.y, e, x[4 * k4 + 1]);
                x[4 * k4 + 2] = fmaf(-u4.z, e, x[4 * k4 + 2]);
                x[4 * k4 + 3] = fmaf(-u4.w, e, x[4 * k4 + 3]);
            }
        }
    }
}

template <int MODE, bool SPARSE>
__global__ void __launch_bounds__(128, 3) solve_kernel(const SolveParams p) {
    extern __shared__ float4 smem4[];
    float *smem = reinterpret_cast<float *>(smem4);
    float *Us = smem;                        // [2][32][128]
    float *Es = smem + 2 * kChunkFloats;     // [2][32][128]
    float *uinv_s = Es + 2 * kChunkFloats;   // [128]
    const int tid = threadIdx.x;
    const int b = blockIdx.y;
    const int u = p.u_map ? p.u_map[b] : b;
    const int64_t R = p.R, C = p.C;
    const int64_t r0 = (int64_t)blockIdx.x * kBlk;
    const int64_t r = r0 + tid;
    const bool active = r < R;
    float *Wt = p.Wt + (int64_t)b * C * R;
    float *E = p.E + (int64_t)b * C * R;
    const float *U = p.U + (int64_t)u * C * C;
    const bool vecU = (C % 4 == 0) && ((reinterpret_cast<uintptr_t>(U) & 15) == 0);
    const bool vecE = (R % 4 == 0) && ((reinterpret_cast<uintptr_t>(E) & 15) == 0);

    for (int64_t bs = 0; bs < C; bs += kBlk) {
        float x[kBlk];
#pragma unroll
        for (int k = 0; k < kBlk; ++k) x[k] = (active && (bs + k < C)) ? Wt[(bs + k) * R + r] : 0.0f;
        if (SPARSE) {
            const int64_t c = bs + tid;
            float v = 1.0f;
            if (c < C) {
                v = p.uvec[(int64_t)u * C + c];
                if (p.uvec_is_diag) v = __fdiv_rn(1.0f, v);
            }
            uinv_s[tid] = v;
        }
        const int nleft = (int)(bs / kSub);
        const int nchunk = nleft + 4;
        // chunk ch < nleft: rows [32ch, 32ch+32) of U and E;  else: rows of the block itself (U only)
        load_chunk(Us, Es, U, E, C, R, 0 < nleft ? 0 : bs, bs, r0, 0 < nleft, vecU, vecE, tid);
        cp_async_commit();
        for (int ch = 0; ch < nchunk; ++ch) {
            const int buf = ch & 1;
            if (ch + 1 < nchunk) {
                const int nx = ch + 1;
                const int64_t j0 = (nx < nleft) ? (int64_t)nx * kSub : bs + (int64_t)(nx - nleft) * kSub;
                load_chunk(Us + (buf ^ 1) * kChunkFloats, Es + (buf ^ 1) * kChunkFloats, U, E, C, R, j0, bs, r0,
                           nx < nleft, vecU, vecE, tid);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            const float *us = Us + buf * kChunkFloats;
            float *es = Es + buf * kChunkFloats;
            if (ch < nleft) {
#pragma unroll 2
                for (int jj = 0; jj < kSub; ++jj) {
                    const float e = es[jj * kBlk + tid];
                    const float4 *urow = reinterpret_cast<const float4 *>(us + jj * kBlk);
#pragma unroll
                    for (int k4 = 0; k4 < kBlk / 4; ++k4) {
                        const float4 u4 = urow[k4];
                        x[4 * k4 + 0] = fmaf(-u4.x, e, x[4 * k4 + 0]);
                        x[4 * k4 + 1] = fmaf(-u4.y, e, x[4 * k4 + 1]);
                        x[4 * k4 + 2] = fmaf(-u4.z, e, x[4 * k4 + 2]);
                        x[4 * k4 + 3] = fmaf(-u4.w, e, x[4 * k4 + 3]);
                    }
                }
            } else {
                switch (ch - nleft) {
                    case 0: solve_subblock<MODE, SPARSE, 0>(x, us, es, uinv_s, p, b, u, bs, r, active, Wt, E, tid); break;
                    case 1: solve_subblock<MODE, SPARSE, 1>(x, us, es, uinv_s, p, b, u, bs, r, active, Wt, E, tid); break;
                    case 2: solve_subblock<MODE, SPARSE, 2>(x, us, es, uinv_s, p, b, u, bs, r, active, Wt, E, tid); break;
                    default: solve_subblock<MODE, SPARSE, 3>(x, us, es, uinv_s, p, b, u, bs, r, active, Wt, E, tid); break;
                }
            }
            __syncthreads();  // the next iteration refills the other buffer, the one after it this one
        }
    }
}

// perm_inv[u][perm[u][i]] = i
__global__ void perm_inverse_kernel(const int32_t *__restrict__ perm, int64_t C, int32_t *__restrict__ perm_inv) {
    const int u = blockIdx.y;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < C) perm_inv[(int64_t)u * C + perm[(int64_t)u * C + i]] = (int32_t)i;
}

// Wt[b][pos(c)][r] = float(W[b][r][c]); pos = perm_inv (identity when null).  32x32 tiles.
__global__ void transpose_gather_kernel(const void *__restrict__ W, int dtype, int64_t R, int64_t C,
                                        const int32_t *__restrict__ perm_inv, const int32_t *__restrict__ u_map,
                                        float *__restrict__ Wt) {
    __shared__ float tile[32][33];
    const int b = blockIdx.z;
    const int u = u_map ? u_map[b] : b;
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;  // block (32, 8)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + ty + 8 * i, c = c0 + tx;
        float v = 0.0f;
        if (r < R && c < C) v = ld_as_f32(W, dtype, ((int64_t)b * R + r) * C + c);
        tile[ty + 8 * i][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t c = c0 + ty + 8 * i, r = r0 + tx;
        if (r < R && c < C) {
            const int64_t pos = perm_inv ? (int64_t)perm_inv[(int64_t)u * C + c] : c;
            Wt[((int64_t)b * C + pos) * R + r] = tile[tx][ty + 8 * i];
        }
    }
}

// qweight[b][r][c] = qt[b][pos(c)][r]
__global__ void untranspose_codes_kernel(const uint8_t *__restrict__ qt, int64_t R, int64_t C,
                                         const int32_t *__restrict__ perm_inv, const int32_t *__restrict__ u_map,
                                         uint8_t *__restrict__ qweight) {
    __shared__ uint8_t tile[32][33];
    const int b = blockIdx.z;
    const int u = u_map ? u_map[b] : b;
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t c = c0 + ty + 8 * i, r = r0 + tx;
        uint8_t v = 0;
        if (r < R && c < C) {
            const int64_t pos = perm_inv ? (int64_t)perm_inv[(int64_t)u * C + c] : c;
            v = qt[((int64_t)b * C + pos) * R + r];
        }
        tile[ty + 8 * i][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + ty + 8 * i, c = c0 + tx;
        if (r < R && c < C) qweight[((int64_t)b * R + r) * C + c] = tile[tx][ty + 8 * i];
    }
}

constexpr size_t kSolveSmem = (4 * kChunkFloats + kBlk) * sizeof(float);

template <int MODE, bool SPARSE>
int launch_solve(const SolveParams &p, int nb, cudaStream_t st) {
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(solve_kernel<MODE, SPARSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kSolveSmem);
        attr_done = true;
    }
    dim3 grid((unsigned)cdiv(p.R, kBlk), (unsigned)nb);
    solve_kernel<MODE, SPARSE><<<grid, kBlk, kSolveSmem, st>>>(p); FORGE_NOTE_LAUNCH();
    return check_launch("forge_gptq_solve");
}

inline int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

}  // namespace

extern "C" int64_t forge_solve_workspace_bytes(int nb, int64_t R, int64_t C) {
    return align256((int64_t)nb * C * R * 4) + align256((int64_t)nb * C * R) + align256((int64_t)nb * C * 4) + 256;
}

extern "C" int forge_gptq_solve_cr(float *Wt, const float *U, const float *uinv, const float *scales,
                                   const float *qzeros, int bits, int64_t R, int64_t C, int sparse14, uint8_t *q,
                                   uint32_t *M, void *ws, void *stream) {
    FORGE_REQUIRE(Wt && U && scales && qzeros && q && ws, "null pointer");
    FORGE_REQUIRE(R > 0 && C > 0 && bits >= 1 && bits <= 8, "bad sizes");
    FORGE_REQUIRE(!sparse14 || (uinv && M), "sparse14 needs uinv and M");
    FORGE_REQUIRE((uintptr_t)ws % 16 == 0, "workspace must be 16-byte aligned");
    SolveParams p{};
    p.Wt = Wt; p.E = (float *)ws; p.U = U; p.uvec = uinv; p.u_map = nullptr;
    p.scales = scales; p.qzeros = qzeros; p.perm = nullptr; p.q = q; p.M = M;
    p.R = R; p.C = C; p.G = 0; p.gs = 1; p.maxq = (1 << bits) - 1; p.write_deq = 1; p.uvec_is_diag = 0;
    cudaStream_t st = (cudaStream_t)stream;
    return sparse14 ? launch_solve<1, true>(p, 1, st) : launch_solve<1, false>(p, 1, st);
}

extern "C" int forge_gptq_solve_batched(const void *W, int w_dtype, int nb, int64_t R, int64_t C, const float *U,
                                        const float *udiag, const int32_t *u_map, const int32_t *perm, int nu,
                                        const float *scales, const float *qzeros, int gs, int bits, int sparse14,
                                        uint8_t *qweight, uint32_t *M, void *ws, void *stream) {
    FORGE_REQUIRE(W && U && scales && qzeros && qweight && ws, "null pointer");
    FORGE_REQUIRE(nb > 0 && R > 0 && C > 0 && gs > 0 && bits >= 1 && bits <= 8, "bad sizes");
    FORGE_REQUIRE(!sparse14 || (udiag && M), "sparse14 needs udiag and M");
    FORGE_REQUIRE(w_dtype == FORGE_DTYPE_F32 || w_dtype == FORGE_DTYPE_BF16, "bad dtype");
    FORGE_REQUIRE((uintptr_t)ws % 256 == 0, "workspace must be 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    char *wsp = (char *)ws;
    float *Wt = (float *)wsp;
    wsp += align256((int64_t)nb * C * R * 4);
    uint8_t *qt = (uint8_t *)wsp;
    wsp += align256((int64_t)nb * C * R);
    int32_t *perm_inv = nullptr;
    if (perm) {
        FORGE_REQUIRE(nu > 0 && nu <= nb, "nu must be in [1, nb]");
        perm_inv = (int32_t *)wsp;
        perm_inverse_kernel<<<dim3((unsigned)cdiv(C, 256), nu), 256, 0, st>>>(perm, C, perm_inv); FORGE_NOTE_LAUNCH();
    }
    dim3 tgrid((unsigned)cdiv(C, 32), (unsigned)cdiv(R, 32), nb);
    transpose_gather_kernel<<<tgrid, dim3(32, 8), 0, st>>>(W, w_dtype, R, C, perm_inv, u_map, Wt); FORGE_NOTE_LAUNCH();
    SolveParams p{};
    p.Wt = Wt; p.E = Wt; p.U = U; p.uvec = udiag; p.u_map = u_map;
    p.scales = scales; p.qzeros = qzeros; p.perm = perm; p.q = qt; p.M = M;
    p.R = R; p.C = C; p.G = cdiv(C, gs); p.gs = gs; p.maxq = (1 << bits) - 1; p.write_deq = 0; p.uvec_is_diag = 1;
    int rc = sparse14 ? launch_solve<0, true>(p, nb, st) : launch_solve<0, false>(p, nb, st);
    if (rc != FORGE_OK) return rc;
    untranspose_codes_kernel<<<tgrid, dim3(32, 8), 0, st>>>(qt, R, C, perm_inv, u_map, qweight); FORGE_NOTE_LAUNCH();
    return check_launch("forge_gptq_solve_batched");
}
