// Fused GPTQ / SparseGPT-1:4 column solver.
//
// The rows of a weight matrix (the R axis) are independent given the factor U, so a CTA owns a strip
// of 128 rows — one thread per row — and walks ALL column blocks itself: no grid-wide sync and one
// launch per batch of matrices, instead of the reference's C/32 kernel launches plus C/32 skinny
// GEMMs per matrix (forge/backend/cuda/solver.cu:124-151).
//
// Two builds of the same algorithm live here.  The default (solve_tc_kernel, further down) puts every product
// that crosses a 32-column sub-block boundary on the tensor cores; solve_kernel is the all-FMA build for shapes
// the tensor-core build does not take and for cross-checks (FORGE_SOLVER_IMPL=simt).  In solve_kernel, for a
// 128-column block starting at column bs a thread holds its row's 128 values in registers:
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
#include <type_traits>
#include "tcgen05.cuh"
#include <stdlib.h>
#include <string.h>

using namespace forge;
using forge::tc::kKS;
using forge::tc::kPieceBytes;
using forge::tc::idesc_tf32;
using forge::tc::make_desc_tf32;
using forge::tc::piece_offset;
using forge::tc::umma_tf32;
using forge::tc::umma_tf32_ts;
using forge::tc::idesc_tf32_ts;
using forge::tc::tf32_round;
using forge::tc::split4;

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
    int alt;               // 1: U holds -Vt (inversion-free form) and the propagated quantity is w - deq
    int meta_t;            // MODE 0: the tables are transposed, [nb][G][R] (a column's 128 rows are contiguous)
    int gs_shift;          // log2(gs) when gs is a power of two, else -1
    const uint8_t *usplit; // [nu] pre-split hi/lo operand pieces of U (forge_solve_split_u), or null
    int64_t usplit_stride; // bytes per Hessian slot
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool pred) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz));
}
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gsrc, bool pred) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = pred ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz));
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

// Scale / zero of (row r, column c).  MODE 0: per-group tables [nb][R][G], the group follows the ORIGINAL
// column index (forge/gptq.py:251-252); MODE 1: per-element tables [nb][C][R].
template <int MODE>
__device__ __forceinline__ void load_meta(const SolveParams &p, int b, int u, int64_t r, int64_t c, bool active,
                                          float &s, float &q0) {
    s = 1.0f;
    q0 = 0.0f;
    if (!active || c >= p.C) return;
    int64_t gi;
    if (MODE == 0) {
        const uint32_t oc = p.perm ? (uint32_t)p.perm[(int64_t)u * p.C + c] : (uint32_t)c;
        const int64_t g = p.gs_shift >= 0 ? (int64_t)(oc >> p.gs_shift) : (int64_t)(oc / (uint32_t)p.gs);
        gi = p.meta_t ? ((int64_t)b * p.G + g) * p.R + r : ((int64_t)b * p.R + r) * p.G + g;
    } else {
        gi = ((int64_t)b * p.C + c) * p.R + r;
    }
    s = __ldg(p.scales + gi);
    q0 = __ldg(p.qzeros + gi);
}

template <int MODE, bool SPARSE, int S>
__device__ __forceinline__ void solve_subblock(float (&x)[kBlk], const float *us, float *es,
                                               const float *uinv_s, const SolveParams &p, int b, int u,
                                               int64_t bs, int64_t r, bool active, float *Wt, float *E, int tid) {
    const int64_t R = p.R, C = p.C;
    const float maxq = (float)p.maxq;
    uint32_t maskbits = 0u;
    // When the columns are not permuted and a group spans whole sub-blocks, one (scale, zero) pair serves
    // the 32 columns; otherwise the pair of the NEXT column is fetched while the current one is solved.
    const bool uniform_meta = (MODE == 0) && (p.perm == nullptr) && (p.gs % kSub == 0);
    float s_nx, q0_nx;
    load_meta<MODE>(p, b, u, r, bs + S * kSub, active, s_nx, q0_nx);
    // Output pointers advance by one column (R elements) per step.  The empty asm makes each advance opaque:
    // otherwise the 32 x 3 addresses of the unrolled loop are all formed up front and, at two registers
    // each, evict the row's values to local memory.
    uint8_t *qp = p.q + ((int64_t)b * C + bs + S * kSub) * R + r;
    float *ep = E + (bs + S * kSub) * R + r;
    float *wp = Wt + (bs + S * kSub) * R + r;
#pragma unroll
    for (int t = 0; t < kSub; ++t) {
        // keep the loads of later columns from being hoisted over this point: fully unrolled, they would
        // otherwise all be issued up front and push the row's 128 values out of the register file
        asm volatile("" ::: "memory");
        const int kk = S * kSub + t;
        const int64_t c = bs + kk;
        const float s = s_nx, q0 = q0_nx;
        if (!uniform_meta && t + 1 < kSub) load_meta<MODE>(p, b, u, r, c + 1, active, s_nx, q0_nx);
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
                quantize_scalar(x[kk], s, q0, maxq, err, deq, qb);
            } else {
                err = x[kk];  // pruned weight: the whole value is the error (solver_sparsegptq14.cu:118-120)
            }
            if (active) {
                *qp = qb;
                if (p.write_deq) *wp = deq;
                *ep = err;
            }
        }
        qp += R; ep += R; wp += R;
        asm volatile("" : "+l"(qp), "+l"(ep), "+l"(wp));
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
#pragma unroll 1
        for (int t = 0; t < kSub; ++t) {
            const float e = es[t * kBlk + tid];
            const float4 *urow = reinterpret_cast<const float4 *>(us + t * kBlk);
#pragma unroll
            for (int k4 = (S + 1) * (kSub / 4); k4 < kBlk / 4; ++k4) {
                // at most eight panel loads (32 registers) in flight next to the row's 128 values
                if ((k4 & 7) == 0) asm volatile("" ::: "memory");
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
#pragma unroll 1
                for (int jj = 0; jj < kSub; ++jj) {
                    const float e = es[jj * kBlk + tid];
                    const float4 *urow = reinterpret_cast<const float4 *>(us + jj * kBlk);
#pragma unroll
                    for (int k4 = 0; k4 < kBlk / 4; ++k4) {
                        if ((k4 & 7) == 0) asm volatile("" ::: "memory");
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


// ================================================================================================
// Tensor-core build of the same solver.  Every update of a not-yet-solved column by the errors of an
// earlier column,  x[r, k] -= err[j, r] * U[j, k],  that crosses a 32-column sub-block boundary runs on
// tcgen05 as a  M=128 (rows) x N (columns) x K=8  TF32 GEMM per k-step, accumulated in 128 TMEM columns
// (one TMEM lane = one weight row).  Per 128-column block:
//   far   : acc[:, 0:128]   = sum_{j < bs}           err_j U[j, bs:bs+128]       (bs/8 k-steps, N = 128)
//   near s: acc[:, 32s:128] += sum_{j in sub-block s-1} err_j U[j, bs+32s:bs+128]  (4 k-steps, N = 128-32s)
// and a row-thread only ever holds the 32 values of the sub-block it is solving:
//   x[0:32] = W[:, sub-block] - tcgen05.ld(acc[:, 32s:32s+32]), then the sequential in-register solve with
//   the 32x32 triangle of U from shared memory.  Nothing but that triangle is left on the FMA pipe.
//
// fp32 fidelity: an operand v is split as  hi = tf32(v) (round to nearest on the bit pattern),
// lo = tf32(v - hi);  acc += Ehi*Uhi + Elo*Uhi + Ehi*Ulo  (three MMAs per k-step).  The dropped Elo*Ulo
// term and the truncation of lo are ~2^-21 relative, the size of fp32 rounding in a dot product.
//
// Both operands are "MN-major": the errors are [j][r] with the 128 rows of the strip contiguous, the U
// panel is [j][bs..bs+128) with the block columns contiguous.  A k-step piece is [8 j][128] fp32 in the
// swizzle layout that 32-bit MN-major operands require (see make_desc_tf32).  The four row warps are the
// producers: far k-steps bring E and U in with cp.async through a small raw ring (each thread reads back only
// the chunks it copied itself; holding prefetched k-steps in registers instead spills at 128 registers/thread),
// near k-steps take the errors straight from the registers that just produced them; the hi/lo pieces are
// stored with the swizzle, published to the async proxy, and the stage's mbarrier is arrived on.  Warp 4
// issues the MMAs and commits.  Every wait is bounded; a CTA that gives up sets the status word.
// ================================================================================================
constexpr int kTcThreads = 160;
constexpr int kTcStageBytes = 4 * kPieceBytes;      // Ehi, Elo, Uhi, Ulo
// Operand ring depth.  Two stages keep three CTAs per SM (the serial column chain wants the warps); with the U pieces
// pre-split in global memory and brought in by bulk copies, a four-stage ring (two CTAs per SM) keeps the tensor
// pipe fed through the long far phases of wide matrices.
constexpr int kTcStagesShallow = 2, kTcStagesDeep = 4;
constexpr int kUsubLd = kSub;                        // staged triangle: row t holds U[t][t+1 ...], zero padded
constexpr int kUsubFloats = kSub * kUsubLd;
// raw fp32 k-steps in flight (cp.async) in the far phase: 2 where the launch fills the GPU (a third would cost the third
// CTA per SM its shared memory), 6 where there are at most two CTAs per SM anyway and latency is all that counts
constexpr int kTcRawFull = 2, kTcRawDeep = 6;
// one raw k-step: [E row jA, E row jA+4 (, U row jA, U row jA+4)][128 threads][16 B]; U only when it is not pre-split
constexpr int tc_raw_bytes(bool tmau) { return (tmau ? 2 : 4) * 128 * 16; }
constexpr size_t tc_smem_bytes(int stages, int raw, bool tmau, bool tmema = false) {
    return (size_t)stages * (tmema ? 4 * 2 * kPieceBytes : kTcStageBytes) + 1024 + 2 * kUsubFloats * sizeof(float) +
           kSub * kBlk * sizeof(float) + kBlk * sizeof(float) + 512 +
           (tmema ? (size_t)kSub * kBlk * 5 : (size_t)raw * tc_raw_bytes(tmau));   // TMEMA: staged (scale, zero) pairs
}
// TMEMA build: the error operand of the MMAs lives in tensor memory.  A row thread owns one TMEM lane, so it can put
// its own row's eight errors of a k-step (hi and lo parts, 16 columns) there with one tcgen05.st, straight from the
// registers that loaded or produced them: no shared-memory staging of the errors at all (the shared-memory pipe,
// not the tensor pipe, is what bounds the build that stages both operands).  Columns [0,128) hold the accumulator,
// [128, 128 + 16 stages) the error stages.
// A sixth warp does nothing but bring the [Uhi | Ulo] pairs in, as far ahead as the ring allows and independently of
// the row threads: a row thread that is waiting for its error rows from HBM must not hold back the requests for U.
// A stage of this build is FOUR k-steps (32 error rows: 64 TMEM columns, four pairs = 32 KB of U, twelve MMAs): the
// hand-over between the row threads, the loader and the MMA warp (two barrier waits, fences, one commit) costs
// several hundred cycles whatever it carries, more than the three MMAs of a single k-step take.
constexpr int kTmemaStages = 2;
constexpr int kTmemaKPerStage = 4;
constexpr uint32_t kTmemaCols = 256;
constexpr int kTmemaThreads = 192;
constexpr int kPrefetchGroups = 4;   // error rows are requested into L2 this many 32-row groups ahead of their use
// Pre-split U: for column block cb (128 columns) the k-steps ks = 0 .. 16 (cb + 1) - 1 (8 rows of U each: every row
// above the block, then the block's own rows for the near updates), one [hi piece | lo piece] pair of 8 KB per
// k-step, k-steps of a block contiguous, blocks in order: pair index = 8 cb (cb + 1) + ks.
constexpr int kPairBytes = 2 * kPieceBytes;
__host__ __device__ inline int64_t usplit_pair_index(int64_t cb, int64_t ks) { return 8 * cb * (cb + 1) + ks; }
__host__ __device__ inline int64_t usplit_bytes_per_slot(int64_t C) {
    const int64_t nblk = (C + kBlk - 1) / kBlk;
    return 8 * nblk * (nblk + 1) * (int64_t)kPairBytes;
}

__device__ __forceinline__ void rows_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// A load the compiler must issue where it is written (volatile asm keeps its place among the barrier waits): the far
// phase asks for the next group of error rows BEFORE it works on the current one; left to the scheduler, the loads
// sink to their first use and every group pays a full HBM latency.
// The error rows stream through once per column block and are gone from L2 long before the next block wants them:
// no L1 allocation, first to be evicted from L2 (policy from l2_policy_evict_first).
__device__ __forceinline__ float ldg_here(const float *p, uint64_t policy) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(policy));
    return v;
}

// Cycle accounting of one CTA of the tensor-memory build (-DFORGE_SOLVER_PROFILE only; never in the shipped library):
// where the row threads, the MMA warp and the U loader spend their time.  Read back with forge_debug_solver_profile.
#ifdef FORGE_SOLVER_PROFILE
__device__ unsigned long long g_prof[32];
__device__ int g_prof_dbg;   // bit 0: skip the Elo*Uhi MMA, bit 1: skip the Ehi*Ulo MMA, bit 2: N = 64 (timing experiments)
#define PROF_T0() const long long _pt0 = clock64()
#define PROF_ADD(slot) do { pacc[slot] += (unsigned long long)(clock64() - _pt0); } while (0)
#else
#define PROF_T0() do {} while (0)
#define PROF_ADD(slot) do {} while (0)
#endif

template <int MODE, bool SPARSE, int kTcRaw, int kTcStages, bool TMAU, bool TMEMA = false>
__global__ void __launch_bounds__(TMEMA ? kTmemaThreads : kTcThreads, ((TMEMA || kTcStages > 2) ? 2 : 3))
solve_tc_kernel(const SolveParams p, int32_t *status) {
    using namespace forge::tc;
    static_assert(!TMEMA || TMAU, "the tensor-memory build takes U from the pre-split pieces");
    static_assert(kTcStages <= 8, "eight barriers per kind");
    extern __shared__ uint8_t smem_raw[];
    constexpr int kTcRawBytes = tc_raw_bytes(TMAU);
    constexpr int kStageStride = TMEMA ? kTmemaKPerStage * kPairBytes : kTcStageBytes;   // TMEMA: four [Uhi | Ulo] pairs
    constexpr int kUoff = TMEMA ? 0 : 2 * kPieceBytes;
    constexpr uint32_t kTmemCols = TMEMA ? kTmemaCols : 128u;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring = smem_raw + (smem_base - smem_u32(smem_raw));
    float *Usub = reinterpret_cast<float *>(ring + kTcStages * kStageStride);  // [2][32][32]
    float *es = Usub + 2 * kUsubFloats;                                          // [32][128] errors of a sub-block
    float *uinv_s = es + kSub * kBlk;                                            // [128]
    // barriers: full[<=8] (operands staged by the row threads), empty[<=8] at +8, acc at +16, full_u[<=8] at +24
    // (TMEMA: the bulk copies of U, tracked apart from the rows' arrivals)
    uint64_t *bars = reinterpret_cast<uint64_t *>(uinv_s + kBlk);
    uint8_t *raw = reinterpret_cast<uint8_t *>(bars) + 512;                      // [kTcRaw][8 KB]
    // TMEMA (no raw ring): the scale and the zero point of the 32 columns of a sub-block for this CTA's rows, staged
    // before the column chain; each thread writes and reads its own column of the two arrays
    float *meta_s = reinterpret_cast<float *>(raw);                              // [32][128]
    uint8_t *meta_z = raw + kSub * kBlk * sizeof(float);                          // [32][128], zero points are integers
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 40);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + 8), bar_acc = smem_u32(bars + 16);
    const uint32_t bar_full_u = smem_u32(bars + 24);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            // TMAU without TMEMA: + the row thread that announces the bulk copy of U
            mbar_init(bar_full + 8 * s, kBlk + ((TMAU && !TMEMA) ? 1 : 0));
            mbar_init(bar_empty + 8 * s, 1);
            if (TMEMA) mbar_init(bar_full_u + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    const uint32_t tmem_e = tmem_base + 128u;      // TMEMA: error stages of 4 k-steps x 16 columns (hi 8, lo 8)
#ifdef FORGE_SOLVER_PROFILE
    const bool prof_on = TMEMA && blockIdx.x == 3 && blockIdx.y == 5 && (threadIdx.x & 31) == 0 &&
                         ((threadIdx.x >> 5) == 0 || (threadIdx.x >> 5) >= 4);
    const long long prof_start = clock64();
    unsigned long long pacc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    const int prof_dbg = g_prof_dbg;
#endif

    const int b = blockIdx.y;
    const int u = p.u_map ? p.u_map[b] : b;
    const int64_t R = p.R, C = p.C;
    const int64_t r0 = (int64_t)blockIdx.x * kBlk;
    float *Wt = p.Wt + (int64_t)b * C * R;
    float *E = p.E + (int64_t)b * C * R;
    const float *U = p.U + (int64_t)u * C * C;
    const uint8_t *usp = TMAU ? p.usplit + (int64_t)u * p.usplit_stride : nullptr;
    uint32_t it = 0;       // k-steps pushed through the ring (same sequence in both roles)
    uint32_t acc_it = 0;   // accumulator hand-overs (commits by warp 4 / waits by the row warps)

    if (warp < 4) {
        const int64_t r = r0 + tid;
        const bool active = r < R;
        const float maxq = (float)p.maxq;
        // float4 slots of this thread inside a [8 j][128] piece: rows j = tid/32 and tid/32 + 4, chunk c4
        const int jA = tid >> 5, c4 = tid & 31;
        const bool e_ok = (r0 + 4 * c4) < R;
        const uint32_t sw_off[2] = {piece_offset(jA, c4), piece_offset(jA + 4, c4)};
        // scalar slot of this thread's own row in an error piece, for K row jj: piece_offset(jj, tid/4) + (tid%4)*4
        const bool uniform_meta = (MODE == 0) && (p.perm == nullptr) && (p.gs % kSub == 0);
        bool ok = true;

        for (int64_t bs = 0; bs < C; bs += kBlk) {
            const bool u_ok = (bs + 4 * c4) < C;
            // ---------------- far phase: every column before the block ----------------
            if (TMEMA && bs > 0 && ok) {
#ifdef FORGE_SOLVER_PROFILE
                const long long _pfar0 = clock64();
#endif
                // Far phase, errors through tensor memory.  A thread reads its own row's errors straight from global
                // memory (a warp's 32 rows are one 128-byte line per error row), 32 error rows = 4 k-steps at a time,
                // the next group in flight while this one is split and stored.
                const int ngroups = (int)(bs / 32);
                const uint64_t stream_pol = forge::tc::l2_policy_evict_first();
                const float *srcE = E + r;
                float cur[32], nxt[32];
                // this warp's 32 rows are one 128-byte line per error row: lane i asks for error row i of a group
                const float *pfE = E + r0 + warp * 32 + (int64_t)lane * R;
                for (int g = 0; g < kPrefetchGroups && g < ngroups; ++g)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(pfE + (int64_t)g * 32 * R));
#pragma unroll
                for (int i = 0; i < 32; ++i) cur[i] = active ? ldg_here(srcE + (int64_t)i * R, stream_pol) : 0.0f;
#pragma unroll 1
                for (int g = 0; g < ngroups && ok; ++g) {
                    if (g + kPrefetchGroups < ngroups)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(pfE + (int64_t)(g + kPrefetchGroups) * 32 * R));
                    if (g + 1 < ngroups) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            nxt[i] = active ? ldg_here(srcE + ((int64_t)(g + 1) * 32 + i) * R, stream_pol) : 0.0f;
                    }
                    {
                        const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                        {
                            PROF_T0();
                            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                            PROF_ADD(1);
                        }
                        ok = __all_sync(0xffffffffu, ok);   // tcgen05.st is warp-aligned: the whole warp goes or none
                        if (!ok) break;
                        tc_fence_after();
                        PROF_T0();
#pragma unroll
                        for (int k = 0; k < kTmemaKPerStage; ++k) {
                            uint32_t v16[16];
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) {
                                const float v = cur[8 * k + jj];
                                const float hi = tf32_round(v);
                                v16[jj] = __float_as_uint(hi);
                                v16[8 + jj] = __float_as_uint(tf32_round(__fsub_rn(v, hi)));
                            }
                            tmem_st16(tmem_e + ((uint32_t)(warp * 32) << 16) + s * 64u + (uint32_t)k * 16u, v16);
                        }
                        tmem_st_wait();
                        tc_fence_before();
                        mbar_arrive(bar_full + 8 * s);
                        PROF_ADD(2);
                        ++it;
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) cur[i] = nxt[i];
                }
#ifdef FORGE_SOLVER_PROFILE
                pacc[0] += (unsigned long long)(clock64() - _pfar0);
#endif
            }
            if (!TMEMA && bs > 0 && ok) {
                // operands travel global -> raw ring (cp.async, kTcRaw k-steps ahead, no registers held) -> hi/lo split
                // -> operand stage; a thread reads back only the 16-byte chunks it copied itself (no barrier needed).
                // TMAU: only the errors go that way; the U pieces were split once for all row strips
                // (forge_solve_split_u) and one thread brings each [hi | lo] pair in with a bulk copy.
                const int nks = (int)(bs / kKS);
                const uint32_t raw_u32 = smem_u32(raw) + (uint32_t)tid * 16u;
                const float *srcE = E + (int64_t)jA * R + r0 + 4 * c4;
                const float *srcU = U + (int64_t)jA * C + bs + 4 * c4;
                const uint8_t *upair = TMAU ? usp + usplit_pair_index(bs / kBlk, 0) * kPairBytes : nullptr;
                auto issue = [&](int ks) {
                    if (ks < nks) {
                        const uint32_t dst = raw_u32 + (uint32_t)(ks % kTcRaw) * kTcRawBytes;
                        const int64_t j = (int64_t)ks * kKS;
                        cp_async16_zfill(dst, e_ok ? srcE + j * R : E, e_ok);
                        cp_async16_zfill(dst + 2048, e_ok ? srcE + (j + 4) * R : E, e_ok);
                        if (!TMAU) {
                            cp_async16_zfill(dst + 4096, u_ok ? srcU + j * C : U, u_ok);
                            cp_async16_zfill(dst + 6144, u_ok ? srcU + (j + 4) * C : U, u_ok);
                        }
                    }
                    cp_async_commit();
                };
#pragma unroll
                for (int d = 0; d < kTcRaw; ++d) issue(d);
#pragma unroll 1
                for (int ks = 0; ks < nks && ok; ++ks) {
                    cp_async_wait<kTcRaw - 1>();
                    const uint8_t *rs = raw + (ks % kTcRaw) * kTcRawBytes + tid * 16;
                    float4 ve[2], vu[2];
                    ve[0] = *reinterpret_cast<const float4 *>(rs);
                    ve[1] = *reinterpret_cast<const float4 *>(rs + 2048);
                    if (!TMAU) {
                        vu[0] = *reinterpret_cast<const float4 *>(rs + 4096);
                        vu[1] = *reinterpret_cast<const float4 *>(rs + 6144);
                    }
                    const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                    ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    uint8_t *stage = ring + s * kTcStageBytes;
                    if (TMAU && tid == 0) {
                        mbar_arrive_expect_tx(bar_full + 8 * s, (uint32_t)kPairBytes);
                        bulk_copy_g2s(smem_base + s * kTcStageBytes + 2 * kPieceBytes, upair + (int64_t)ks * kPairBytes,
                                      (uint32_t)kPairBytes, bar_full + 8 * s);
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float4 hi, lo;
                        split4(ve[h], hi, lo);
                        *reinterpret_cast<float4 *>(stage + 0 * kPieceBytes + sw_off[h]) = hi;
                        *reinterpret_cast<float4 *>(stage + 1 * kPieceBytes + sw_off[h]) = lo;
                        if (!TMAU) {
                            split4(vu[h], hi, lo);
                            *reinterpret_cast<float4 *>(stage + 2 * kPieceBytes + sw_off[h]) = hi;
                            *reinterpret_cast<float4 *>(stage + 3 * kPieceBytes + sw_off[h]) = lo;
                        }
                    }
                    fence_proxy_async();
                    mbar_arrive(bar_full + 8 * s);
                    ++it;
                    issue(ks + kTcRaw);
                }
                cp_async_wait<0>();
            }
            if (SPARSE) {
                const int64_t c = bs + tid;
                float v = 1.0f;
                if (c < C) {
                    v = p.uvec[(int64_t)u * C + c];
                    if (p.uvec_is_diag) v = __fdiv_rn(1.0f, v);
                }
                uinv_s[tid] = v;   // read after the next rows_barrier
            }
            // ---------------- the four sub-blocks ----------------
#pragma unroll 1
            for (int sb = 0; sb < 4; ++sb) {
#ifdef FORGE_SOLVER_PROFILE
                const long long _pnr0 = clock64();
#endif
                const int64_t cs = bs + (int64_t)sb * kSub;
                float *us = Usub + (sb & 1) * kUsubFloats;
                // (1) the strict upper triangle of U[cs.., cs..] for the in-register part, row t stored from its
                // first useful element: us[t][k] = U[cs+t][cs+t+1+k] (zero past the row end), so that the column
                // loop reads a row with aligned vector loads whatever t is.  4-byte copies: the source is unaligned.
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int v = tid + 128 * i;            // 1024 elements, 8 per thread
                    const int jj = v >> 5, k = v & 31;
                    const bool okl = (k < kSub - 1 - jj) && (cs + jj < C) && (cs + jj + 1 + k < C);
                    cp_async4(us + jj * kUsubLd + k, okl ? (U + (cs + jj) * C + cs + jj + 1 + k) : U, okl);
                }
                cp_async_commit();
                // (2) near update: the previous sub-block's errors go to the later columns of the block
                if (TMEMA && sb > 0 && ok) {
                    // near update, errors of the previous sub-block from this thread's own column of the scratch: one stage
                    const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                    ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) {
                        tc_fence_after();
#pragma unroll
                        for (int i = 0; i < kTmemaKPerStage; ++i) {
                            uint32_t v16[16];
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) {
                                const float v = es[(i * kKS + jj) * kBlk + tid];
                                const float hi = tf32_round(v);
                                v16[jj] = __float_as_uint(hi);
                                v16[8 + jj] = __float_as_uint(tf32_round(__fsub_rn(v, hi)));
                            }
                            tmem_st16(tmem_e + ((uint32_t)(warp * 32) << 16) + s * 64u + (uint32_t)i * 16u, v16);
                        }
                        tmem_st_wait();
                        tc_fence_before();
                        mbar_arrive(bar_full + 8 * s);
                        ++it;
                    }
                }
                if (!TMEMA && sb > 0 && ok) {
                    float4 nu[4][2];
                    if (!TMAU) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int64_t j = cs - kSub + i * kKS + jA + 4 * h;
                                nu[i][h] = (u_ok && j < C) ? *reinterpret_cast<const float4 *>(U + j * C + bs + 4 * c4)
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (ok) {
                            const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                            if (ok) {
                                uint8_t *stage = ring + s * kTcStageBytes;
                                if (TMAU && tid == 0) {
                                    // the block's own rows follow the far k-steps in the pre-split layout
                                    const int64_t pair = usplit_pair_index(bs / kBlk, bs / kKS + (sb - 1) * 4 + i);
                                    mbar_arrive_expect_tx(bar_full + 8 * s, (uint32_t)kPairBytes);
                                    bulk_copy_g2s(smem_base + s * kTcStageBytes + 2 * kPieceBytes, usp + pair * kPairBytes,
                                                  (uint32_t)kPairBytes, bar_full + 8 * s);
                                }
#pragma unroll
                                for (int jj = 0; jj < kKS; ++jj) {
                                    const float v = es[(i * kKS + jj) * kBlk + tid];
                                    const float hi = tf32_round(v);
                                    const float lo = tf32_round(__fsub_rn(v, hi));
                                    const uint32_t off = piece_offset(jj, tid >> 2) + ((tid & 3) << 2);
                                    *reinterpret_cast<float *>(stage + 0 * kPieceBytes + off) = hi;
                                    *reinterpret_cast<float *>(stage + 1 * kPieceBytes + off) = lo;
                                }
                                if (!TMAU) {
#pragma unroll
                                    for (int h = 0; h < 2; ++h) {
                                        float4 hi, lo;
                                        split4(nu[i][h], hi, lo);
                                        *reinterpret_cast<float4 *>(stage + 2 * kPieceBytes + sw_off[h]) = hi;
                                        *reinterpret_cast<float4 *>(stage + 3 * kPieceBytes + sw_off[h]) = lo;
                                    }
                                }
                                fence_proxy_async();
                                mbar_arrive(bar_full + 8 * s);
                                ++it;
                            }
                        }
                    }
                }
                // (2b) with permuted columns (activation order) every column has its own group: its scale is a
                // dependent global load (permutation -> group -> scale).  One column of look-ahead cannot hide that, and
                // the chain then runs at one such latency per column; so the 32 pairs are fetched here, eight at a time,
                // where the thread is about to wait for the accumulator anyway
                const bool staged_meta = TMEMA && !uniform_meta;
#ifdef FORGE_SOLVER_PROFILE
                const long long _pst0 = clock64();
                pacc[7] += (unsigned long long)(_pst0 - _pnr0);
#endif
                if (staged_meta) {
#pragma unroll 1
                    for (int i0 = 0; i0 < kSub; i0 += 8) {
                        // branch-free, so that the eight permutation loads, then the sixteen table loads, are all in
                        // flight together (indices are clamped into range; out-of-range slots get the neutral pair)
                        const int64_t rr = active ? r : (R - 1);
                        int64_t gi[8];
                        float sv[8], zv[8];
                        if (MODE == 0) {
                            uint32_t oc[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int64_t c = imin64(cs + i0 + i, C - 1);
                                oc[i] = p.perm ? (uint32_t)__ldg(p.perm + (int64_t)u * C + c) : (uint32_t)c;
                            }
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int64_t g = p.gs_shift >= 0 ? (int64_t)(oc[i] >> p.gs_shift)
                                                                  : (int64_t)(oc[i] / (uint32_t)p.gs);
                                gi[i] = p.meta_t ? ((int64_t)b * p.G + g) * R + rr : ((int64_t)b * R + rr) * p.G + g;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) gi[i] = ((int64_t)b * C + imin64(cs + i0 + i, C - 1)) * R + rr;
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            sv[i] = __ldg(p.scales + gi[i]);
                            zv[i] = __ldg(p.qzeros + gi[i]);
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const bool in = active && (cs + i0 + i < C);
                            meta_s[(i0 + i) * kBlk + tid] = in ? sv[i] : 1.0f;
                            meta_z[(i0 + i) * kBlk + tid] = in ? (uint8_t)(int)zv[i] : (uint8_t)0;
                        }
                    }
                }
#ifdef FORGE_SOLVER_PROFILE
                pacc[6] += (unsigned long long)(clock64() - _pst0);
                const long long _px0 = clock64();
#endif
                // (3) x = W - acc for the 32 columns of this sub-block
                // es[.][tid] is this thread's own column of the scratch: the near update above has consumed the previous
                // sub-block's errors, so it now holds this sub-block's original weights until each is replaced by its error
                float x[kSub];
#pragma unroll
                for (int i = 0; i < kSub; ++i) {
                    x[i] = (active && (cs + i < C)) ? Wt[(cs + i) * R + r] : 0.0f;
                    es[i * kBlk + tid] = x[i];
                }
                if (bs > 0 || sb > 0) {
                    PROF_T0();
                    if (ok) ok = mbar_wait(bar_acc, acc_it & 1u, abort_flag);
                    PROF_ADD(4);
                    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-aligned: the whole warp goes or none
                    if (ok) {
                        tc_fence_after();
                        uint32_t v[32];
                        tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(sb * kSub), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < kSub; ++i) x[i] = __fsub_rn(x[i], __uint_as_float(v[i]));
                        tc_fence_before();
                    }
                    ++acc_it;
                }
                // (4) every row thread passes here, whether its waits succeeded or not; a thread that gave up
                // raised the abort flag before, so all of them leave together
                cp_async_wait<0>();
                rows_barrier();
                if (*abort_flag) break;
#ifdef FORGE_SOLVER_PROFILE
                const long long _pch0 = clock64();
                pacc[3] += (unsigned long long)(_pch0 - _px0);
#endif
                // (5) sequential solve of the 32 columns.  The loop is rolled: x and w slide down by one register per
                // column, so that the column being solved is always x[0] and every index is static.  (Fully unrolled,
                // the 32 x ~80 instructions run once per pass and the warp stalls on instruction fetch.)
                uint32_t maskbits = 0u;
                float s_nx = 1.0f, q0_nx = 0.0f;
                if (!staged_meta) load_meta<MODE>(p, b, u, r, cs, active, s_nx, q0_nx);
                uint8_t *qp = p.q + ((int64_t)b * C + cs) * R + r;
                float *ep = E + cs * R + r;
                float *wp = Wt + cs * R + r;
                float inv_s = 0.0f, nq0s = 0.0f;
                // One column.  W = width of the live window: at column t only x[1 .. 31-t] are still unsolved, so the
                // loop runs in four quarters with W = 32, 24, 16, 8 and each quarter propagates along W-1 entries only.
                auto column = [&](auto wtag, const int t) {
                    constexpr int W = decltype(wtag)::value;
                    const int64_t c = cs + t;
                    // the row of U this column propagates along: in flight while the column is quantised
                    // (first half now, second half after the quantisation: holding all of it across the chain spills)
                    float4 u4[W / 4];
                    const float4 *urow = reinterpret_cast<const float4 *>(us + t * kUsubLd);
                    constexpr int kFirst = (W / 8 > 0) ? W / 8 : 1;
#pragma unroll
                    for (int k4 = 0; k4 < kFirst; ++k4) u4[k4] = urow[k4];
                    const float w_t = es[t * kBlk + tid];   // the column's original weight; replaced by its error below
                    const float sc = staged_meta ? meta_s[t * kBlk + tid] : s_nx;
                    const float q0 = staged_meta ? (float)meta_z[t * kBlk + tid] : q0_nx;
                    if (!uniform_meta || t == 0) {
                        inv_s = __fdiv_rn(1.0f, __fadd_rn(sc, kEps));
                        nq0s = -__fmul_rn(q0, sc);
                    }
                    if (!staged_meta && !uniform_meta && t + 1 < kSub) load_meta<MODE>(p, b, u, r, c + 1, active, s_nx, q0_nx);
                    float err = 0.0f;
                    if (c < C) {
                        if (SPARSE && (t & 3) == 0) {
                            float best = -1e30f;
                            int bidx = -1;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                if (active && (c + k < C)) {
                                    const float sv = fabsf(__fmul_rn(x[k], uinv_s[sb * kSub + t + k]));
                                    if (best < sv) { best = sv; bidx = k; }
                                }
                            }
                            if (bidx > -1) maskbits |= (1u << (t + bidx));
                        }
                        float deq = 0.0f;
                        uint8_t qb = 0;
                        const bool keep = SPARSE ? (((maskbits >> t) & 1u) != 0u) : true;
                        if (keep && (active || !SPARSE)) {
                            // quantize_scalar with the reciprocal and -q0*s hoisted (same operations, same rounding)
                            float q = fminf(fmaxf(fmaf(x[0], inv_s, q0), 0.0f), maxq);
                            q = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
                            deq = fmaf(q, sc, nq0s);
                            err = __fsub_rn(x[0], deq);
                            qb = (uint8_t)(int)q;
                        } else {
                            err = x[0];
                        }
                        if (p.alt) err = __fsub_rn(w_t, deq);  // inversion-free form propagates w - deq
                        if (active) {
                            *qp = qb;
                            if (p.write_deq) *wp = deq;
                            *ep = err;
                        }
                    }
                    qp += R; ep += R; wp += R;
                    es[t * kBlk + tid] = err;
                    // x[k] <- x[k+1] - U[t][t+1+k] * err ; past the end of the row the staged value is zero
#pragma unroll
                    for (int k4 = kFirst; k4 < W / 4; ++k4) u4[k4] = urow[k4];
#pragma unroll
                    for (int k4 = 0; k4 < W / 4; ++k4) {
                        x[4 * k4 + 0] = fmaf(-u4[k4].x, err, x[4 * k4 + 1]);
                        x[4 * k4 + 1] = fmaf(-u4[k4].y, err, x[4 * k4 + 2]);
                        x[4 * k4 + 2] = fmaf(-u4[k4].z, err, x[4 * k4 + 3]);
                        if (k4 < W / 4 - 1) x[4 * k4 + 3] = fmaf(-u4[k4].w, err, x[4 * k4 + 4]);
                    }
                    x[W - 1] = 0.0f;
                };
#pragma unroll 1
                for (int t = 0; t < 8; ++t) column(std::integral_constant<int, 32>{}, t);
#pragma unroll 1
                for (int t = 8; t < 16; ++t) column(std::integral_constant<int, 24>{}, t);
#pragma unroll 1
                for (int t = 16; t < 24; ++t) column(std::integral_constant<int, 16>{}, t);
#pragma unroll 1
                for (int t = 24; t < 32; ++t) column(std::integral_constant<int, 8>{}, t);
                if (SPARSE && active && (cs < C)) p.M[((int64_t)b * ((C + 31) / 32) + (cs >> 5)) * R + r] = maskbits;
#ifdef FORGE_SOLVER_PROFILE
                pacc[5] += (unsigned long long)(clock64() - _pch0);
#endif
            }
            // the errors of this block must be visible to the far-phase loads of the next one
            rows_barrier();
            if (*abort_flag) break;
        }
        cp_async_wait<0>();
    } else if (TMEMA && warp == 5) {
        // ---- U loader: the pairs of every k-step in the order the MMAs take them (per block: the far k-steps, then the
        // twelve near ones), each into its ring slot as soon as the MMAs that last read the slot have completed
        if (lane == 0) {
            bool ok = true;
            const uint64_t keep = l2_policy_evict_last();
            for (int64_t bs = 0; bs < C && ok; bs += kBlk) {
                const int64_t first = usplit_pair_index(bs / kBlk, 0);
                const int n_stages = (int)(bs / kKS) / kTmemaKPerStage + 3;    // far stages, then the three near ones
                for (int sg = 0; sg < n_stages && ok; ++sg) {
                    const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                    {
                        PROF_T0();
                        ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                        PROF_ADD(8);
                    }
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_full_u + 8 * s, (uint32_t)kStageStride);
                    bulk_copy_g2s_hint(smem_base + s * kStageStride,
                                       usp + (first + (int64_t)sg * kTmemaKPerStage) * kPairBytes, (uint32_t)kStageStride,
                                       bar_full_u + 8 * s, keep);
                    ++it;
                }
            }
        }
        __syncwarp();
    } else if (TMEMA) {
        // ---- MMA issuer, stages of four k-steps: errors from tensor memory, U pairs from the ring
        bool ok = true;
        const uint32_t id_far = idesc_tf32_ts(128);
        auto stage_mmas = [&](uint32_t s, uint32_t d, uint32_t boff, uint32_t id, bool first_accumulates) {
            const uint32_t e0 = tmem_e + s * 64u;
            const uint64_t u0 = make_desc_tf32(smem_base + s * kStageStride + boff);
#pragma unroll
            for (int k = 0; k < kTmemaKPerStage; ++k) {
                // descriptors address in 16-byte units: a pair is 8 KB = 512 units on, its lo piece 256 units on
                const uint64_t uhi = u0 + (uint64_t)(k * (kPairBytes >> 4));
                const uint64_t ulo = uhi + (uint64_t)(kPieceBytes >> 4);
                const uint32_t ehi = e0 + (uint32_t)k * 16u, elo = ehi + 8u;
#ifdef FORGE_SOLVER_PROFILE
                umma_tf32_ts(d, ehi, uhi, id, (k > 0 || first_accumulates) ? 1u : 0u);
                if (!(prof_dbg & 1)) umma_tf32_ts(d, elo, uhi, id, 1u);
                if (!(prof_dbg & 2)) umma_tf32_ts(d, ehi, ulo, id, 1u);
#else
                umma_tf32_ts(d, ehi, uhi, id, (k > 0 || first_accumulates) ? 1u : 0u);
                umma_tf32_ts(d, elo, uhi, id, 1u);
                umma_tf32_ts(d, ehi, ulo, id, 1u);
#endif
            }
        };
        for (int64_t bs = 0; bs < C && ok; bs += kBlk) {
            if (bs > 0) {
                const int nst = (int)(bs / kKS) / kTmemaKPerStage;
                for (int sg = 0; sg < nst && ok; ++sg) {
                    const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                    {
                        PROF_T0();
                        ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                        PROF_ADD(9);
                    }
                    {
                        PROF_T0();
                        if (ok) ok = mbar_wait(bar_full_u + 8 * s, ph, abort_flag);
                        PROF_ADD(10);
                    }
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        PROF_T0();
                        stage_mmas(s, tmem_base, 0u, id_far, sg > 0);
                        umma_commit(bar_empty + 8 * s);
                        PROF_ADD(11);
                    }
                    __syncwarp();
                    ++it;
                }
                if (!ok) break;
                if (lane == 0) umma_commit(bar_acc);
                __syncwarp();
            }
            for (int sb = 1; sb < 4 && ok; ++sb) {
                const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                if (ok) ok = mbar_wait(bar_full_u + 8 * s, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    // skip the MN blocks of the solved sub-blocks; block 0 has no far phase: its first near stage
                    // starts the accumulator columns it covers
                    stage_mmas(s, tmem_base + (uint32_t)(sb * kSub), (uint32_t)sb * 1024u,
                               idesc_tf32_ts((uint32_t)(kBlk - sb * kSub)), bs > 0 || sb > 1);
                    umma_commit(bar_empty + 8 * s);
                    umma_commit(bar_acc);
                }
                __syncwarp();
                ++it;
            }
        }
    } else {
        bool ok = true;
        for (int64_t bs = 0; bs < C && ok; bs += kBlk) {
            if (bs > 0) {
                const int nks = (int)(bs / kKS);
                for (int ks = 0; ks < nks && ok; ++ks) {
                    const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                    {
                        PROF_T0();
                        ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                        PROF_ADD(9);
                    }
                    {
                        PROF_T0();
                        if (ok && TMEMA) ok = mbar_wait(bar_full_u + 8 * s, ph, abort_flag);
                        PROF_ADD(10);
                    }
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t st = smem_base + s * kStageStride;
                        const uint64_t uhi = make_desc_tf32(st + kUoff), ulo = make_desc_tf32(st + kUoff + kPieceBytes);
                        {
                            const uint64_t ehi = make_desc_tf32(st), elo = make_desc_tf32(st + kPieceBytes);
                            const uint32_t id = idesc_tf32(128);
                            umma_tf32(tmem_base, ehi, uhi, id, ks > 0 ? 1u : 0u);
                            umma_tf32(tmem_base, elo, uhi, id, 1u);
                            umma_tf32(tmem_base, ehi, ulo, id, 1u);
                        }
                        umma_commit(bar_empty + 8 * s);
                    }
                    __syncwarp();
                    ++it;
                }
                if (!ok) break;
                if (lane == 0) umma_commit(bar_acc);
                __syncwarp();
            }
            for (int sb = 1; sb < 4 && ok; ++sb) {
                for (int i = 0; i < 4 && ok; ++i) {
                    const uint32_t s = it % kTcStages, ph = (it / kTcStages) & 1u;
                    ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                    if (ok && TMEMA) ok = mbar_wait(bar_full_u + 8 * s, ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t st = smem_base + s * kStageStride;
                        const uint32_t boff = (uint32_t)sb * 1024u;  // skip the MN blocks of the solved sub-blocks
                        const uint64_t uhi = make_desc_tf32(st + kUoff + boff);
                        const uint64_t ulo = make_desc_tf32(st + kUoff + kPieceBytes + boff);
                        const uint32_t d = tmem_base + (uint32_t)(sb * kSub);
                        // block 0 has no far phase: its first near step starts the accumulator columns it covers
                        const uint32_t acc = (bs > 0 || sb > 1 || i > 0) ? 1u : 0u;
                        {
                            const uint64_t ehi = make_desc_tf32(st), elo = make_desc_tf32(st + kPieceBytes);
                            const uint32_t id = idesc_tf32((uint32_t)(kBlk - sb * kSub));
                            umma_tf32(d, ehi, uhi, id, acc);
                            umma_tf32(d, elo, uhi, id, 1u);
                            umma_tf32(d, ehi, ulo, id, 1u);
                        }
                        umma_commit(bar_empty + 8 * s);
                    }
                    __syncwarp();
                    ++it;
                }
                if (!ok) break;
                if (lane == 0) umma_commit(bar_acc);
                __syncwarp();
            }
        }
    }
#ifdef FORGE_SOLVER_PROFILE
    if (prof_on) {
        const int slot = warp == 0 ? 16 : (warp == 4 ? 17 : (warp == 5 ? 18 : 19));
        g_prof[slot] += (unsigned long long)(clock64() - prof_start);
        for (int i = 0; i < 12; ++i) g_prof[i] += pacc[i];
    }
#endif
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0 && status) atomicExch(status, FORGE_ERR_TIMEOUT);
        if (TMAU) {
            // a CTA that gave up may still have bulk copies of U in flight towards its shared memory: give them time
            // to land (bounded; they take microseconds) before the CTA returns
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000LL) {}
        }
    }
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// [hi | lo] operand pieces of U for the tensor-core solver (layout: usplit_pair_index).  One CTA per pair: 128 threads,
// each two 16-byte chunks (rows j and j + 4 of the k-step), exactly the slots the solver's own producers would write.
__global__ void __launch_bounds__(128) split_u_kernel(const float *__restrict__ Uall, int64_t C, uint8_t *__restrict__ out,
                                                      int64_t out_stride) {
    const int64_t ks = blockIdx.x, cb = blockIdx.y;
    if (ks >= 16 * (cb + 1)) return;
    const int u = blockIdx.z;
    const float *U = Uall + (int64_t)u * C * C;
    uint8_t *pair = out + (int64_t)u * out_stride + usplit_pair_index(cb, ks) * kPairBytes;
    const int tid = threadIdx.x, jA = tid >> 5, c4 = tid & 31;
    const int64_t col = cb * kBlk + 4 * c4;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int64_t j = ks * kKS + jA + 4 * h;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < C && col < C) v = *reinterpret_cast<const float4 *>(U + j * C + col);
        float4 hi, lo;
        split4(v, hi, lo);
        const uint32_t off = piece_offset(jA + 4 * h, c4);
        *reinterpret_cast<float4 *>(pair + off) = hi;
        *reinterpret_cast<float4 *>(pair + kPieceBytes + off) = lo;
    }
}

// [nb][R][G] -> [nb][G][R] for the scale and zero tables: the solver's 128 row threads then read one column's
// entries from consecutive addresses
__global__ void transpose_meta_kernel(const float *__restrict__ s_in, const float *__restrict__ z_in, int64_t R, int64_t G,
                                      float *__restrict__ s_out, float *__restrict__ z_out) {
    __shared__ float ts[32][33], tz[32][33];
    const int b = blockIdx.z;
    const int64_t g0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;  // block (32, 8)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + ty + 8 * i, g = g0 + tx;
        if (r < R && g < G) {
            ts[ty + 8 * i][tx] = s_in[((int64_t)b * R + r) * G + g];
            tz[ty + 8 * i][tx] = z_in[((int64_t)b * R + r) * G + g];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t g = g0 + ty + 8 * i, r = r0 + tx;
        if (r < R && g < G) {
            s_out[((int64_t)b * G + g) * R + r] = ts[tx][ty + 8 * i];
            z_out[((int64_t)b * G + g) * R + r] = tz[tx][ty + 8 * i];
        }
    }
}

// perm_inv[u][perm[u][i]] = i
__global__ void perm_inverse_kernel(const int32_t *__restrict__ perm, int64_t C, int32_t *__restrict__ perm_inv) {
    const int u = blockIdx.y;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < C) perm_inv[(int64_t)u * C + perm[(int64_t)u * C + i]] = (int32_t)i;
}

// Wt[b][pos(c)][r] = float(W[b][r][c]); pos = perm_inv (identity when null).  64 x 64 tiles, 256 threads: rows of W are
// read in 8- or 16-byte pieces (four weights per thread), rows of Wt written as float4 (16 threads per 256-byte row).
__global__ void __launch_bounds__(256) transpose_gather_kernel(const void *__restrict__ W, int dtype, int64_t R, int64_t C,
                                                               const int32_t *__restrict__ perm_inv,
                                                               const int32_t *__restrict__ u_map, float *__restrict__ Wt) {
    __shared__ float tile[64][65];      // [r][c]
    const int b = blockIdx.z;
    const int u = u_map ? u_map[b] : b;
    const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
    const int tid = threadIdx.x, q16 = tid & 15, row16 = tid >> 4;
    const bool vec_in = (C % 4 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + row16 + 16 * i, c = c0 + 4 * q16;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < R && c < C) {
            const int64_t idx = ((int64_t)b * R + r) * C + c;
            if (vec_in && c + 3 < C) {
                if (dtype == FORGE_DTYPE_BF16) {
                    const uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __nv_bfloat16 *>(W) + idx);
                    v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
                    v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
                } else {
                    const float4 raw = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(W) + idx);
                    v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < C) v[e] = ld_as_f32(W, dtype, idx + e);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) tile[row16 + 16 * i][4 * q16 + e] = v[e];
    }
    __syncthreads();
    const bool vec_out = (R % 4 == 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t c = c0 + row16 + 16 * i, r = r0 + 4 * q16;
        if (c < C && r < R) {
            const int64_t pos = perm_inv ? (int64_t)perm_inv[(int64_t)u * C + c] : c;
            float *dst = Wt + ((int64_t)b * C + pos) * R + r;
            const int cl = row16 + 16 * i;
            if (vec_out && r + 3 < R) {
                *reinterpret_cast<float4 *>(dst) =
                    make_float4(tile[4 * q16][cl], tile[4 * q16 + 1][cl], tile[4 * q16 + 2][cl], tile[4 * q16 + 3][cl]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (r + e < R) dst[e] = tile[4 * q16 + e][cl];
            }
        }
    }
}

// qweight[b][r][c] = qt[b][pos(c)][r].  64 x 64 byte tiles, 256 threads, four codes (one 32-bit word) per access on both
// sides.
__global__ void __launch_bounds__(256) untranspose_codes_kernel(const uint8_t *__restrict__ qt, int64_t R, int64_t C,
                                                                const int32_t *__restrict__ perm_inv,
                                                                const int32_t *__restrict__ u_map,
                                                                uint8_t *__restrict__ qweight) {
    __shared__ uint8_t tile[64][68];    // [c][r]
    const int b = blockIdx.z;
    const int u = u_map ? u_map[b] : b;
    const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
    const int tid = threadIdx.x, q16 = tid & 15, row16 = tid >> 4;
    const bool vec_in = (R % 4 == 0), vec_out = (C % 4 == 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t c = c0 + row16 + 16 * i, r = r0 + 4 * q16;
        uint32_t w = 0;
        if (c < C && r < R) {
            const int64_t pos = perm_inv ? (int64_t)perm_inv[(int64_t)u * C + c] : c;
            const uint8_t *src = qt + ((int64_t)b * C + pos) * R + r;
            if (vec_in && r + 3 < R) {
                w = *reinterpret_cast<const uint32_t *>(src);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (r + e < R) w |= (uint32_t)src[e] << (8 * e);
            }
        }
        *reinterpret_cast<uint32_t *>(&tile[row16 + 16 * i][4 * q16]) = w;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t r = r0 + row16 + 16 * i, c = c0 + 4 * q16;
        if (r < R && c < C) {
            const int rl = row16 + 16 * i;
            const uint32_t w = (uint32_t)tile[4 * q16][rl] | ((uint32_t)tile[4 * q16 + 1][rl] << 8) |
                               ((uint32_t)tile[4 * q16 + 2][rl] << 16) | ((uint32_t)tile[4 * q16 + 3][rl] << 24);
            uint8_t *dst = qweight + ((int64_t)b * R + r) * C + c;
            if (vec_out && c + 3 < C) {
                *reinterpret_cast<uint32_t *>(dst) = w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < C) dst[e] = (uint8_t)(w >> (8 * e));
            }
        }
    }
}

constexpr size_t kSolveSmem = (4 * kChunkFloats + kBlk) * sizeof(float);

// The tensor-core build needs 16-byte aligned float4 rows (R % 4 == 0, C % 4 == 0); otherwise, or when
// FORGE_SOLVER_IMPL=simt is set in the environment (cross-checks), the plain-FMA build runs.
inline bool use_tc_solver(const SolveParams &p) {
    const char *e = getenv("FORGE_SOLVER_IMPL");
    if (e && strcmp(e, "simt") == 0) return false;
    return (p.R % 4 == 0) && (p.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.U) & 15) == 0) &&
           ((reinterpret_cast<uintptr_t>(p.E) & 15) == 0);
}

template <int MODE, bool SPARSE>
int launch_solve(const SolveParams &p, int nb, int32_t *status, cudaStream_t st) {
    dim3 grid((unsigned)cdiv(p.R, kBlk), (unsigned)nb);
    if (!use_tc_solver(p)) {
        cudaFuncSetAttribute(solve_kernel<MODE, SPARSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSolveSmem);
        solve_kernel<MODE, SPARSE><<<grid, kBlk, kSolveSmem, st>>>(p); FORGE_NOTE_LAUNCH();
        return check_launch("forge_gptq_solve");
    }
    // per-device attributes (more than 48 KB of dynamic shared memory): set on the device that is current for this call
    auto go = [&](auto kernel, size_t smem, int threads = kTcThreads) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kernel<<<grid, threads, smem, st>>>(p, status); FORGE_NOTE_LAUNCH();
    };
    const bool few = (int64_t)grid.x * grid.y <= 2 * 148;
    if (p.usplit) {
        // U pre-split.  Wide matrices (long far phases) and small launches: errors through tensor memory, two CTAs per
        // SM (256 TMEM columns each); FORGE_SOLVER_IMPL=smem keeps the shared-memory staging of the errors there too
        // (cross-checks).  Other launches keep three CTAs per SM for the serial column chain.
        const char *e = getenv("FORGE_SOLVER_IMPL");
        const bool smem_e = e && strcmp(e, "smem") == 0;
        if ((p.C >= 4096 || few) && !smem_e)
            go(solve_tc_kernel<MODE, SPARSE, 1, kTmemaStages, true, true>, tc_smem_bytes(kTmemaStages, 0, true, true),
               kTmemaThreads);
        else if (p.C >= 4096 || few)
            go(solve_tc_kernel<MODE, SPARSE, 4, kTcStagesDeep, true>, tc_smem_bytes(kTcStagesDeep, 4, true));
        else go(solve_tc_kernel<MODE, SPARSE, 4, kTcStagesShallow, true>, tc_smem_bytes(kTcStagesShallow, 4, true));
    } else if (few) {
        go(solve_tc_kernel<MODE, SPARSE, kTcRawDeep, kTcStagesShallow, false>, tc_smem_bytes(kTcStagesShallow, kTcRawDeep, false));
    } else {
        go(solve_tc_kernel<MODE, SPARSE, kTcRawFull, kTcStagesShallow, false>, tc_smem_bytes(kTcStagesShallow, kTcRawFull, false));
    }
    return check_launch("forge_gptq_solve");
}

inline int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

}  // namespace

#ifdef FORGE_SOLVER_PROFILE
// profiling build only: copy the cycle counters out (32 x u64) and clear them
extern "C" int forge_debug_solver_set(int dbg) {
    cudaMemcpyToSymbol(g_prof_dbg, &dbg, sizeof(int));
    return 0;
}
extern "C" int forge_debug_solver_profile(unsigned long long *out32) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out32, g_prof, sizeof(unsigned long long) * 32);
    unsigned long long zero[32] = {0};
    cudaMemcpyToSymbol(g_prof, zero, sizeof(zero));
    return 0;
}
#endif

extern "C" int64_t forge_solve_split_u_bytes(int nu, int64_t C) {
    return (C > 0 && C % 4 == 0 && nu > 0) ? (int64_t)nu * usplit_bytes_per_slot(C) : 0;
}

extern "C" int forge_solve_split_u(const float *U, int nu, int64_t C, void *usplit, void *stream) {
    FORGE_REQUIRE(U && usplit, "null pointer");
    FORGE_REQUIRE(nu > 0 && C > 0 && C % 4 == 0, "C must be a positive multiple of 4");
    FORGE_REQUIRE((uintptr_t)U % 16 == 0 && (uintptr_t)usplit % 16 == 0, "U and usplit must be 16-byte aligned");
    const int64_t nblk = cdiv(C, kBlk);
    FORGE_REQUIRE(nblk <= 65535 && nu <= 65535, "too many column blocks / slots for one launch");
    split_u_kernel<<<dim3((unsigned)(16 * nblk), (unsigned)nblk, (unsigned)nu), 128, 0, (cudaStream_t)stream>>>(
        U, C, (uint8_t *)usplit, usplit_bytes_per_slot(C));
    FORGE_NOTE_LAUNCH();
    return check_launch("forge_solve_split_u");
}

// transposed scale / zero tables: the group size is not known here, 32 (the smallest the grid kernels take) bounds it
static inline int64_t meta_t_bytes(int nb, int64_t R, int64_t C) { return align256((int64_t)nb * R * (C / 32 + 1) * 4); }

extern "C" int64_t forge_solve_workspace_bytes(int nb, int64_t R, int64_t C) {
    return align256((int64_t)nb * C * R * 4) + align256((int64_t)nb * C * R) + align256((int64_t)nb * C * 4) +
           2 * meta_t_bytes(nb, R, C) + 256;
}

extern "C" int forge_gptq_solve_cr(float *Wt, const float *U, const float *uinv, const float *scales,
                                   const float *qzeros, int bits, int64_t R, int64_t C, int sparse14, uint8_t *q,
                                   uint32_t *M, void *ws, int32_t *status, void *stream) {
    FORGE_REQUIRE(Wt && U && scales && qzeros && q && ws, "null pointer");
    FORGE_REQUIRE(R > 0 && C > 0 && bits >= 1 && bits <= 8, "bad sizes");
    FORGE_REQUIRE(!sparse14 || (uinv && M), "sparse14 needs uinv and M");
    FORGE_REQUIRE((uintptr_t)ws % 16 == 0, "workspace must be 16-byte aligned");
    SolveParams p{};
    p.Wt = Wt; p.E = (float *)ws; p.U = U; p.uvec = uinv; p.u_map = nullptr;
    p.scales = scales; p.qzeros = qzeros; p.perm = nullptr; p.q = q; p.M = M;
    p.R = R; p.C = C; p.G = 0; p.gs = 1; p.maxq = (1 << bits) - 1; p.write_deq = 1; p.uvec_is_diag = 0;
    p.gs_shift = 0;
    cudaStream_t st = (cudaStream_t)stream;
    return sparse14 ? launch_solve<1, true>(p, 1, status, st) : launch_solve<1, false>(p, 1, status, st);
}

extern "C" int forge_gptq_solve_batched(const void *W, int w_dtype, int nb, int64_t R, int64_t C, const float *U,
                                        const float *udiag, const int32_t *u_map, const int32_t *perm, int nu,
                                        const float *scales, const float *qzeros, int gs, int bits, int sparse14,
                                        int form, const void *usplit, uint8_t *qweight, uint32_t *M, void *ws,
                                        int32_t *status, void *stream) {
    FORGE_REQUIRE(W && U && scales && qzeros && qweight && ws, "null pointer");
    FORGE_REQUIRE(!usplit || ((uintptr_t)usplit % 16 == 0 && C % 4 == 0 && R % 4 == 0),
                  "usplit needs 16-byte alignment and R, C multiples of 4");
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
    int32_t *perm_inv = (int32_t *)wsp;
    wsp += align256((int64_t)nb * C * 4);
    float *scales_t = nullptr, *qzeros_t = nullptr;
    const int64_t G = cdiv(C, gs);
    if (gs >= 32) {
        scales_t = (float *)wsp;
        qzeros_t = (float *)(wsp + meta_t_bytes(nb, R, C));
        transpose_meta_kernel<<<dim3((unsigned)cdiv(G, 32), (unsigned)cdiv(R, 32), nb), dim3(32, 8), 0, st>>>(
            scales, qzeros, R, G, scales_t, qzeros_t);
        FORGE_NOTE_LAUNCH();
    }
    if (!perm) perm_inv = nullptr;
    if (perm) {
        FORGE_REQUIRE(nu > 0 && nu <= nb, "nu must be in [1, nb]");
        perm_inverse_kernel<<<dim3((unsigned)cdiv(C, 256), nu), 256, 0, st>>>(perm, C, perm_inv); FORGE_NOTE_LAUNCH();
    }
    dim3 tgrid((unsigned)cdiv(C, 64), (unsigned)cdiv(R, 64), nb);
    transpose_gather_kernel<<<tgrid, 256, 0, st>>>(W, w_dtype, R, C, perm_inv, u_map, Wt); FORGE_NOTE_LAUNCH();
    SolveParams p{};
    p.Wt = Wt; p.E = Wt; p.U = U; p.uvec = udiag; p.u_map = u_map;
    p.scales = scales_t ? scales_t : scales; p.qzeros = scales_t ? qzeros_t : qzeros; p.meta_t = scales_t ? 1 : 0;
    p.perm = perm; p.q = qt; p.M = M;
    p.R = R; p.C = C; p.G = G; p.gs = gs; p.maxq = (1 << bits) - 1; p.write_deq = 0; p.uvec_is_diag = 1;
    p.gs_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
        if ((1 << sft) == gs) p.gs_shift = sft;
    p.alt = form ? 1 : 0;
    p.usplit = (const uint8_t *)usplit;
    p.usplit_stride = usplit ? usplit_bytes_per_slot(C) : 0;
    if (p.alt && !use_tc_solver(p)) {
        set_error("forge_gptq_solve_batched: the inversion-free form needs R %% 4 == 0 and C %% 4 == 0");
        return FORGE_ERR_UNSUPPORTED;
    }
    int rc = sparse14 ? launch_solve<0, true>(p, nb, status, st) : launch_solve<0, false>(p, nb, status, st);
    if (rc != FORGE_OK) return rc;
    untranspose_codes_kernel<<<tgrid, 256, 0, st>>>(qt, R, C, perm_inv, u_map, qweight); FORGE_NOTE_LAUNCH();
    return check_launch("forge_gptq_solve_batched");
}
