// Batched Cholesky -> unit-diagonal upper factor of the inverse, for all Hessians of a layer at once.
//
// The reference (forge/gptq.py:156-170) runs three LAPACK-style calls per matrix:
//   L = chol(Hp);  Hinv = cholesky_inverse(L);  T = chol(Hinv, upper);  U = T / diag(T)
// (4/3 C^3 flop).  The same U follows from ONE Cholesky of the index-reversed matrix and ONE
// triangular inverse (2/3 C^3 flop):  with J the reversal permutation and  J Hp J = L L^T,
//   T = J L^-1 J   (upper, T^T T = Hp^-1),   U = diag(T)^-1 T = J [diag(L) L^-1] J .
// The caller hands in A = J Hp J (forge_hessian_gather_damp writes it that way), so everything here
// is a plain lower Cholesky plus a lower triangular inverse whose rows are scaled by diag(L) as they
// are produced; one last pass rotates the result by 180 degrees into the upper triangle.
//
// Blocked right-looking factorisation, every step batched over the matrices, blocked on two levels:
//   diag   : factor the 64x64 diagonal block in registers (one thread per row), invert it (Dinv), emit the
//            matching diagonal block of the scaled inverse and udiag;
//   panel  : rows below  <-  rows below * Dinv^T   (TRSM as a GEMM); the result is also stored transposed in
//            the unused upper triangle so that the update reads both operands with unit stride;
//   update : inside an outer block of 256 (512 for large matrices) columns, the panel updates only the rest of
//            that outer block (K = 64); once the outer block is done it updates everything behind it in ONE pass
//            (K = 256 / 512).  The update is a TF32 x3 GEMM on tcgen05 (fp32 fidelity through a hi/lo split, see
//            tcgen05.cuh) with a vector red.global.add epilogue; an all-FMA version (chol_syrk_kernel) serves
//            shapes the vector path does not take and the cross-check FORGE_SYRK_IMPL=simt.
// forge_chol_factor_batched stops there and hands the solver the factor itself (scaled, negated, rotated:
// rotate_scale_neg_kernel); forge_chol_inv_upper_batched continues with the inverse, block column by block
// column from the right,   M[below, j] = -( M[below, below] * L[below, j] ) * Dinv_j   (fp32 FMA).
#include "common.cuh"
#include "tcgen05.cuh"
#include <stdlib.h>
#include <string.h>

using namespace forge;

namespace {

constexpr int NB = 64;        // panel width
constexpr int TM = 128;       // tile rows
constexpr int KC = 16;        // k-chunk staged in shared memory
constexpr int AS = KC + 4;    // padded row stride of the A chunk (floats)

// acc[8][TN/16] += A[TM x K] * B[K x TN].   A(i,k) = A[i*lda + k], B(k,n) = B[k*ldb + n].
// Rows i >= m_valid, columns n >= n_valid and k >= K read as zero; with tri_row0 >= 0 the A operand is
// lower triangular in global indexing: A(i,k) reads as zero when (tri_k0 + k) > (tri_row0 + i).
// 256 threads: ty = tid/16 owns rows ty + 16*ii, tx = tid%16 owns columns tx*4+e (+64 for TN=128).
template <int TN>
__device__ __forceinline__ void tile_gemm(float (&acc)[8][TN / 16], const float *__restrict__ A, int64_t lda,
                                          int m_valid, const float *__restrict__ B, int64_t ldb, int n_valid,
                                          int K, bool vec, int64_t tri_row0, int64_t tri_k0, float *As,
                                          float *Bs) {
    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    // global -> registers for chunk k0 (issued one chunk ahead of its use), registers -> shared memory later
    float4 ra[2], rb[TN / 64];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int v = tid + 256 * i;
            const int row = v >> 2, kq = (v & 3) * 4;
            float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < m_valid && k0 + kq < K) {
                const float *src = A + (int64_t)row * lda + k0 + kq;
                if (vec && k0 + kq + 3 < K) val = *reinterpret_cast<const float4 *>(src);
                else {
                    val.x = src[0];
                    if (k0 + kq + 1 < K) val.y = src[1];
                    if (k0 + kq + 2 < K) val.z = src[2];
                    if (k0 + kq + 3 < K) val.w = src[3];
                }
                if (tri_row0 >= 0) {
                    const int64_t gr = tri_row0 + row, gk = tri_k0 + k0 + kq;
                    if (gk + 0 > gr) val.x = 0.f;
                    if (gk + 1 > gr) val.y = 0.f;
                    if (gk + 2 > gr) val.z = 0.f;
                    if (gk + 3 > gr) val.w = 0.f;
                }
            }
            ra[i] = val;
        }
#pragma unroll
        for (int i = 0; i < TN / 64; ++i) {
            const int v = tid + 256 * i;
            const int row = v / (TN / 4), n4 = (v % (TN / 4)) * 4;
            float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + row < K && n4 < n_valid) {
                const float *src = B + (int64_t)(k0 + row) * ldb + n4;
                if (vec && n4 + 3 < n_valid) val = *reinterpret_cast<const float4 *>(src);
                else {
                    val.x = src[0];
                    if (n4 + 1 < n_valid) val.y = src[1];
                    if (n4 + 2 < n_valid) val.z = src[2];
                    if (n4 + 3 < n_valid) val.w = src[3];
                }
            }
            rb[i] = val;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += KC) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int v = tid + 256 * i;
            *reinterpret_cast<float4 *>(As + (v >> 2) * AS + (v & 3) * 4) = ra[i];
        }
#pragma unroll
        for (int i = 0; i < TN / 64; ++i) {
            const int v = tid + 256 * i;
            *reinterpret_cast<float4 *>(Bs + (v / (TN / 4)) * TN + (v % (TN / 4)) * 4) = rb[i];
        }
        if (k0 + KC < K) fetch(k0 + KC);  // in flight while this chunk is multiplied
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < KC; ++kk) {
            float a[8];
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) a[ii] = As[(ty + 16 * ii) * AS + kk];
            float bv[TN / 16];
            {
                const float4 b0 = *reinterpret_cast<const float4 *>(Bs + kk * TN + tx * 4);
                bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
                if (TN == 128) {
                    const float4 b1 = *reinterpret_cast<const float4 *>(Bs + kk * TN + 64 + tx * 4);
                    bv[TN / 16 - 4] = b1.x; bv[TN / 16 - 3] = b1.y; bv[TN / 16 - 2] = b1.z; bv[TN / 16 - 1] = b1.w;
                }
            }
#pragma unroll
            for (int ii = 0; ii < 8; ++ii)
#pragma unroll
                for (int jj = 0; jj < TN / 16; ++jj) acc[ii][jj] = fmaf(a[ii], bv[jj], acc[ii][jj]);
        }
        __syncthreads();
    }
}

__device__ __forceinline__ int col_of(int tx, int jj) { return (jj < 4) ? tx * 4 + jj : 64 + tx * 4 + (jj - 4); }

struct CholWs {
    float *dinv;  // [nb][nblk][2][NB][NB]  (0: Dinv, 1: Dinv^T)
};

// ---- diag: factor + invert the diagonal block of step k (one CTA of 64 threads per matrix) -----------------
// Thread i owns row i of the 64x64 block in registers (the full symmetric row, so that no update needs a
// predicate).  Both loops are ROLLED with a sliding window, so that every register index is static and the loop
// bodies stay in the instruction cache (a fully unrolled version spends its time fetching 7000 instructions that
// each run once): at step j the row's entry for column j is a[0], and the update writes a[m] <- a[m+1] - l_ij *
// l_(j+1+m),j.  Column j of the factor is published pre-shifted, Lsh[j][m] = L[j+1+m][j], which makes the reads
// aligned float4 broadcasts for the update and for the inverse alike.  The inverse is one forward substitution per
// thread (thread c solves L x = e_c, column-oriented with the same sliding window); no barrier is needed there.
__global__ void __launch_bounds__(64) chol_diag_kernel(float *__restrict__ Aall, int64_t C, int k, int nblk,
                                                        float *__restrict__ dinv_all, float *__restrict__ Uall,
                                                        float *__restrict__ udiag, int32_t *__restrict__ info) {
    __shared__ __align__(16) float Lsh[NB][NB];   // Lsh[j][m] = L[j+1+m][j], zero past the end of the column
    __shared__ float dg[NB], invd[NB];
    __shared__ int bad_col;
    const int b = blockIdx.x, i = threadIdx.x;
    float *A = Aall + (int64_t)b * C * C;
    const int64_t cb = (int64_t)k * NB;
    const int nbk = (int)imin64(NB, C - cb);
    if (i == 0) bad_col = -1;
    float a[NB];
    // the block is symmetric on entry as far as it is used: read the row from the lower triangle and its mirror
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        float v = (i == j) ? 1.0f : 0.0f;         // identity padding of a partial last block
        if (i < nbk && j < nbk) v = (j <= i) ? A[(cb + i) * C + cb + j] : A[(cb + j) * C + cb + i];
        a[j] = v;
        Lsh[j][i] = 0.0f;
    }
    __syncthreads();
    float *Acol = A + (cb + i) * C + cb;          // L[i][j] goes to Acol[j]
#pragma unroll 1
    for (int j = 0; j < NB; ++j) {
        if (i == j) {
            const float piv = a[0];
            if (!(piv > 0.0f) && bad_col < 0) bad_col = j;
            const float d = sqrtf(piv);
            dg[j] = d;
            invd[j] = __fdiv_rn(1.0f, d);
        }
        __syncthreads();
        const float lij = (i == j) ? dg[j] : __fmul_rn(a[0], invd[j]);
        if (i > j) Lsh[j][i - j - 1] = lij;
        if (i >= j && i < nbk && j < nbk) Acol[j] = lij;
        __syncthreads();
        const float4 *cj = reinterpret_cast<const float4 *>(&Lsh[j][0]);
#pragma unroll
        for (int m4 = 0; m4 < NB / 4; ++m4) {
            const float4 c4 = cj[m4];
            a[4 * m4 + 0] = fmaf(-lij, c4.x, a[4 * m4 + 1]);
            a[4 * m4 + 1] = fmaf(-lij, c4.y, a[4 * m4 + 2]);
            a[4 * m4 + 2] = fmaf(-lij, c4.z, a[4 * m4 + 3]);
            if (m4 < NB / 4 - 1) a[4 * m4 + 3] = fmaf(-lij, c4.w, a[4 * m4 + 4]);
        }
        a[NB - 1] = 0.0f;
    }
    // column c = i of the inverse:  x_r = b_r / L[r][r],  b_m <- b_m - L[m][r] x_r  (m > r), window sliding with r
#pragma unroll
    for (int m = 0; m < NB; ++m) a[m] = (m == i) ? 1.0f : 0.0f;
    float *dinv = dinv_all + ((int64_t)b * nblk + k) * 2 * NB * NB;
    float *U = Uall ? Uall + (int64_t)b * C * C : nullptr;
#pragma unroll 1
    for (int r = 0; r < NB; ++r) {
        const float xr = __fmul_rn(a[0], invd[r]);
        dinv[r * NB + i] = xr;                    // Dinv[r][c = i]
        dinv[NB * NB + i * NB + r] = xr;          // Dinv^T[c][r]
        if (U && r < nbk && i < nbk) {
            // diagonal block of  diag(L) L^-1  (unit diagonal, zero above it)
            U[(cb + r) * C + cb + i] = (i < r) ? __fmul_rn(dg[r], xr) : ((i == r) ? 1.0f : 0.0f);
        }
        const float4 *cr = reinterpret_cast<const float4 *>(&Lsh[r][0]);
#pragma unroll
        for (int m4 = 0; m4 < NB / 4; ++m4) {
            const float4 c4 = cr[m4];
            a[4 * m4 + 0] = fmaf(-xr, c4.x, a[4 * m4 + 1]);
            a[4 * m4 + 1] = fmaf(-xr, c4.y, a[4 * m4 + 2]);
            a[4 * m4 + 2] = fmaf(-xr, c4.z, a[4 * m4 + 3]);
            if (m4 < NB / 4 - 1) a[4 * m4 + 3] = fmaf(-xr, c4.w, a[4 * m4 + 4]);
        }
        a[NB - 1] = 0.0f;
    }
    if (i < nbk) udiag[(int64_t)b * C + (C - 1 - (cb + i))] = invd[i];
    if (i == 0 && bad_col >= 0 && info[b] == 0) info[b] = (int32_t)(cb + bad_col + 1);
}

// ---- panel: rows below the diagonal block <- rows * Dinv^T; also stored transposed above ------
__global__ void __launch_bounds__(256, 3) chol_panel_kernel(float *__restrict__ Aall, int64_t C, int k, int nblk,
                                                          const float *__restrict__ dinv_all, int vec,
                                                          int64_t row_end) {
    __shared__ __align__(16) float As[TM * AS];
    __shared__ __align__(16) float Bs[KC * 64];
    const int b = blockIdx.y, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    float *A = Aall + (int64_t)b * C * C;
    const int64_t cb = (int64_t)k * NB, rb = cb + NB;
    const int64_t i0 = (int64_t)blockIdx.x * TM;
    const int m_valid = (int)imin64(TM, row_end - rb - i0);     // rows [rb, row_end) only
    if (m_valid <= 0) return;
    const float *dinvT = dinv_all + ((int64_t)b * nblk + k) * 2 * NB * NB + NB * NB;
    float acc[8][4];
#pragma unroll
    for (int ii = 0; ii < 8; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.0f;
    tile_gemm<64>(acc, A + (rb + i0) * C + cb, C, m_valid, dinvT, NB, NB, NB, vec != 0, -1, 0, As, Bs);
#pragma unroll
    for (int ii = 0; ii < 8; ++ii) {
        const int i = ty + 16 * ii;
        if (i < m_valid) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int c = tx * 4 + jj;
                A[(rb + i0 + i) * C + cb + c] = acc[ii][jj];
                A[(cb + c) * C + rb + i0 + i] = acc[ii][jj];
            }
        }
    }
}

// ---- syrk: trailing lower triangle -= panel * panel^T -----------------------------------------
__global__ void __launch_bounds__(256, 2) chol_syrk_kernel(float *__restrict__ Aall, int64_t C, int k, int vec) {
    if (blockIdx.y > blockIdx.x) return;  // upper tiles are not needed
    __shared__ __align__(16) float As[TM * AS];
    __shared__ __align__(16) float Bs[KC * 128];
    const int b = blockIdx.z, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    float *A = Aall + (int64_t)b * C * C;
    const int64_t cb = (int64_t)k * NB, rb = cb + NB;
    const int64_t i0 = (int64_t)blockIdx.x * TM, j0 = (int64_t)blockIdx.y * 128;
    const int m_valid = (int)imin64(TM, C - rb - i0);
    const int n_valid = (int)imin64(128, C - rb - j0);
    if (m_valid <= 0 || n_valid <= 0) return;
    float acc[8][8];
#pragma unroll
    for (int ii = 0; ii < 8; ++ii)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) acc[ii][jj] = 0.0f;
    tile_gemm<128>(acc, A + (rb + i0) * C + cb, C, m_valid, A + cb * C + rb + j0, C, n_valid, NB, vec != 0, -1, 0,
                   As, Bs);
#pragma unroll
    for (int ii = 0; ii < 8; ++ii) {
        const int i = ty + 16 * ii;
        if (i >= m_valid) continue;
        float *row = A + (rb + i0 + i) * C + rb + j0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c0 = h * 64 + tx * 4;
            if (vec && c0 + 3 < n_valid) {
                float4 v = *reinterpret_cast<float4 *>(row + c0);
                v.x -= acc[ii][4 * h + 0]; v.y -= acc[ii][4 * h + 1];
                v.z -= acc[ii][4 * h + 2]; v.w -= acc[ii][4 * h + 3];
                *reinterpret_cast<float4 *>(row + c0) = v;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c0 + e < n_valid) row[c0 + e] -= acc[ii][4 * h + e];
            }
        }
    }
}

// ---- trailing update on the tensor cores ---------------------------------------------------------
// T[i-tile, j-tile] -= P_i P_j^T  where P = the K panel columns [kb, kb + K) already factored, T = the block of the
// matrix whose rows start at r0 (to the end) and whose columns are [r0, r0 + ncols): the lower-triangular tiles of
// that block.  A TF32 x3 GEMM with the fp32 accumulator in TMEM.  Both operands come from the TRANSPOSED copy of
// the panel in the upper triangle, Lt[kb + k][r0 + i] = L[r0 + i][kb + k], whose rows are contiguous along the tile
// rows: exactly the MN-major [8 K rows][128] pieces the tcgen05 path of the column solver uses (hi/lo split, three
// MMAs per k-step, see tcgen05.cuh).  The factorisation is blocked on two levels: inside an outer block of
// kOuter columns (twice that for large matrices) every 64-column panel updates only the rest of that outer block
// (K = 64), and the outer block as a whole updates the matrix behind it once (K = the outer block's width), so the read-modify-write of the
// trailing matrix in HBM happens once per kOuter columns instead of once per 64.  Persistent CTAs walk the tiles
// of all matrices.
constexpr int kOuter = 256;

// tile p of one matrix -> (ti, tj): rows of tiles ti = 0.. hold min(ti + 1, ntj) tiles each
__device__ __forceinline__ void syrk_tile(int p, int ntj, int &ti, int &tj) {
    const int tri = ntj * (ntj + 1) / 2;
    if (p < tri) {
        ti = 0;
        while (p > ti) { p -= ti + 1; ++ti; }
        tj = p;
    } else {
        p -= tri;
        ti = ntj + p / ntj;
        tj = p % ntj;
    }
}
__host__ __device__ __forceinline__ int syrk_tiles(int nti, int ntj) {
    return ntj * (ntj + 1) / 2 + (nti - ntj) * ntj;
}

// A 16-byte load the compiler must issue where it is written: the operand rows of four k-steps are requested together
// BEFORE the first of them is split and staged; left to the scheduler the loads sink to their first use and every k-step
// pays an L2 round trip.
__device__ __forceinline__ float4 ldg128_here(const float *p) {
    float4 v;
    asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

constexpr int kSyrkThreads = 160;
constexpr int kSyrkStages = 4;
constexpr int kSyrkStageBytes = 4 * forge::tc::kPieceBytes;   // Ahi, Alo, Bhi, Blo
constexpr size_t kSyrkSmem = (size_t)kSyrkStages * kSyrkStageBytes + 1024 + 256;

__global__ void __launch_bounds__(kSyrkThreads, 3) chol_syrk_tc_kernel(float *__restrict__ Aall, int64_t C, int64_t kb, int K,
                                                                        int64_t r0, int64_t ncols, int nb,
                                                                        int32_t *status, int64_t row_end) {
    using namespace forge::tc;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + kSyrkStages * kSyrkStageBytes);  // full[4], empty[4], acc
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 9);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kSyrkStages), bar_acc = smem_u32(bars + 8);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kSyrkStages; ++s) {
            mbar_init(bar_full + 8 * s, 128);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"(128u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    const int64_t cb = kb, rb = r0;
    const int64_t m = row_end - rb;                 // rows of the block being updated: [r0, row_end)
    const int64_t ncol = ncols < m ? ncols : m;     // its columns
    const int nti = (int)((m + 127) / 128), ntj = (int)((ncol + 127) / 128);
    const int ntri = syrk_tiles(nti, ntj);
    const int total = nb * ntri;
    uint32_t it = 0, acc_it = 0;
    const int kSteps = K / kKS;                     // 8 K rows per step

    if (warp < 4) {
        const int jA = tid >> 5, c4 = tid & 31;
        const uint32_t sw_off[2] = {piece_offset(jA, c4), piece_offset(jA + 4, c4)};
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
            const int b = tile / ntri;
            int ti, tj;
            syrk_tile(tile % ntri, ntj, ti, tj);
            float *A = Aall + (int64_t)b * C * C;
            const int64_t i0 = (int64_t)ti * 128, j0 = (int64_t)tj * 128;
            const bool diag = (ti == tj);
            const bool a_ok = (i0 + 4 * c4) < m, b_ok = (j0 + 4 * c4) < m;
            const float *srcA = A + cb * C + rb + i0 + 4 * c4;
            const float *srcB = A + cb * C + rb + j0 + 4 * c4;
            // ---- operands: K / 8 k-steps, loaded four at a time through registers
#pragma unroll 1
            for (int half = 0; half < K / 32 && ok; ++half) {
                float4 ra[4][2], rbv[4][2];
#pragma unroll
                for (int d = 0; d < 4; ++d)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int64_t row = (int64_t)(half * 4 + d) * kKS + jA + 4 * h;
                        ra[d][h] = a_ok ? ldg128_here(srcA + row * C) : make_float4(0.f, 0.f, 0.f, 0.f);
                        if (!diag) rbv[d][h] = b_ok ? ldg128_here(srcB + row * C) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                for (int d = 0; d < 4; ++d) {
                    if (!ok) break;
                    const uint32_t s = it % kSyrkStages, ph = (it / kSyrkStages) & 1u;
                    ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    uint8_t *stage = ring + s * kSyrkStageBytes;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float4 hi, lo;
                        split4(ra[d][h], hi, lo);
                        *reinterpret_cast<float4 *>(stage + 0 * kPieceBytes + sw_off[h]) = hi;
                        *reinterpret_cast<float4 *>(stage + 1 * kPieceBytes + sw_off[h]) = lo;
                        if (!diag) {
                            split4(rbv[d][h], hi, lo);
                            *reinterpret_cast<float4 *>(stage + 2 * kPieceBytes + sw_off[h]) = hi;
                            *reinterpret_cast<float4 *>(stage + 3 * kPieceBytes + sw_off[h]) = lo;
                        }
                    }
                    fence_proxy_async();
                    mbar_arrive(bar_full + 8 * s);
                    ++it;
                }
            }
            // ---- epilogue: T -= acc, one row per thread
            if (ok) ok = mbar_wait(bar_acc, acc_it & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            ++acc_it;
            if (!ok) break;
            tc_fence_after();
            const int64_t row = i0 + tid;
            float *Crow = A + (rb + row) * C + rb + j0;
#pragma unroll 1
            for (int qd = 0; qd < 4; ++qd) {
                if (j0 + qd * 32 >= ncol) break;            // columns outside the block (same for the whole CTA)
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(qd * 32), v);
                tmem_ld_wait();
                if (row < m) {
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        const int64_t col = j0 + qd * 32 + g4 * 4;
                        if (col + 3 < ncol) {
                            float4 *dst = reinterpret_cast<float4 *>(Crow + qd * 32 + g4 * 4);
                            // fire-and-forget reduction in L2 instead of load / subtract / store: the epilogue
                            // has no load round trip, and since every element gets exactly one addition per launch
                            // the result does not depend on any ordering
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                                         "f"(-__uint_as_float(v[4 * g4 + 0])), "f"(-__uint_as_float(v[4 * g4 + 1])),
                                         "f"(-__uint_as_float(v[4 * g4 + 2])), "f"(-__uint_as_float(v[4 * g4 + 3]))
                                         : "memory");
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (col + e < ncol) Crow[qd * 32 + g4 * 4 + e] -= __uint_as_float(v[4 * g4 + e]);
                        }
                    }
                }
            }
            tc_fence_before();
        }
    } else {
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
            int ti, tj;
            syrk_tile(tile % ntri, ntj, ti, tj);
            const bool diag = (ti == tj);
            for (int ks = 0; ks < kSteps && ok; ++ks) {
                const uint32_t s = it % kSyrkStages, ph = (it / kSyrkStages) & 1u;
                ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t st = smem_base + s * kSyrkStageBytes;
                    const uint64_t ahi = make_desc_tf32(st), alo = make_desc_tf32(st + kPieceBytes);
                    const uint64_t bhi = diag ? ahi : make_desc_tf32(st + 2 * kPieceBytes);
                    const uint64_t blo = diag ? alo : make_desc_tf32(st + 3 * kPieceBytes);
                    const uint32_t id = idesc_tf32(128);
                    umma_tf32(tmem_base, ahi, bhi, id, ks > 0 ? 1u : 0u);
                    umma_tf32(tmem_base, alo, bhi, id, 1u);
                    umma_tf32(tmem_base, ahi, blo, id, 1u);
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
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0 && status) atomicExch(status, FORGE_ERR_TIMEOUT);
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
    }
}

// ---- the same update on 256 x 256 tiles (the big update behind an outer block) -----------------------------------
// The 128 x 128 kernel above stages 16 KB of split operands per k-step for three 128 x 128 x 8 MMAs: shared-memory
// stores and operand loads keep the L1 / shared-memory pipe as busy as the tensor pipe (ncu: 78 % against 44 %).  A
// 256 x 256 tile stages 32 KB per k-step for SIX 128 x 256 x 8 MMAs: half the staging per multiply-add.  One CTA per SM:
// eight producer / epilogue warps (thread t owns tile row t), one MMA warp, both 128-row halves' accumulators fill
// tensor memory (2 x 256 columns).  Stage = [A0hi A1hi A0lo A1lo B0hi B1hi B0lo B1lo] (4 KB pieces): the two pieces of
// a B part are adjacent and form one N = 256 operand; on diagonal tiles B is A.
constexpr int kSyrk2Threads = 288;
constexpr int kSyrk2Stages = 4;
constexpr int kSyrk2StageBytes = 8 * forge::tc::kPieceBytes;
constexpr size_t kSyrk2Smem = (size_t)kSyrk2Stages * kSyrk2StageBytes + 1024 + 256;

__global__ void __launch_bounds__(kSyrk2Threads, 1) chol_syrk256_tc_kernel(float *__restrict__ Aall, int64_t C, int64_t kb,
                                                                            int K, int64_t r0, int nb,
                                                                            int32_t *status) {
    using namespace forge::tc;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + kSyrk2Stages * kSyrk2StageBytes);  // full[4], empty[4], acc
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 9);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kSyrk2Stages), bar_acc = smem_u32(bars + 8);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kSyrk2Stages; ++s) {
            mbar_init(bar_full + 8 * s, 256);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    const int64_t cb = kb, rb = r0;
    const int64_t m = C - rb;                       // the square block [r0, C) x [r0, C), lower tiles
    const int nt = (int)((m + 255) / 256);
    const int ntri = syrk_tiles(nt, nt);
    const int total = nb * ntri;
    uint32_t it = 0, acc_it = 0;
    const int kSteps = K / kKS;

    if (warp < 8) {
        const int half = tid >> 7, jA = (tid >> 5) & 3, c4 = tid & 31;
        const uint32_t sw_off[2] = {piece_offset(jA, c4), piece_offset(jA + 4, c4)};
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
            const int b = tile / ntri;
            int ti, tj;
            syrk_tile(tile % ntri, nt, ti, tj);
            float *A = Aall + (int64_t)b * C * C;
            const int64_t i0 = (int64_t)ti * 256, j0 = (int64_t)tj * 256;
            const bool diag = (ti == tj);
            const int64_t ia = i0 + half * 128 + 4 * c4, jb = j0 + half * 128 + 4 * c4;
            const bool a_ok = ia < m, b_ok = jb < m;
            const float *srcA = A + cb * C + rb + ia;
            const float *srcB = A + cb * C + rb + jb;
#pragma unroll 1
            for (int grp = 0; grp < K / 32 && ok; ++grp) {
                float4 ra[4][2], rbv[4][2];
#pragma unroll
                for (int d = 0; d < 4; ++d)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int64_t row = (int64_t)(grp * 4 + d) * kKS + jA + 4 * h;
                        ra[d][h] = a_ok ? ldg128_here(srcA + row * C) : make_float4(0.f, 0.f, 0.f, 0.f);
                        if (!diag) rbv[d][h] = b_ok ? ldg128_here(srcB + row * C) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                for (int d = 0; d < 4; ++d) {
                    if (!ok) break;
                    const uint32_t s = it % kSyrk2Stages, ph = (it / kSyrk2Stages) & 1u;
                    ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    uint8_t *stage = ring + s * kSyrk2StageBytes + half * kPieceBytes;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float4 hi, lo;
                        split4(ra[d][h], hi, lo);
                        *reinterpret_cast<float4 *>(stage + 0 * kPieceBytes + sw_off[h]) = hi;
                        *reinterpret_cast<float4 *>(stage + 2 * kPieceBytes + sw_off[h]) = lo;
                        if (!diag) {
                            split4(rbv[d][h], hi, lo);
                            *reinterpret_cast<float4 *>(stage + 4 * kPieceBytes + sw_off[h]) = hi;
                            *reinterpret_cast<float4 *>(stage + 6 * kPieceBytes + sw_off[h]) = lo;
                        }
                    }
                    fence_proxy_async();
                    mbar_arrive(bar_full + 8 * s);
                    ++it;
                }
            }
            // ---- epilogue: T -= acc, one row per thread (thread t <-> tile row t <-> TMEM lane t % 128 of half t / 128)
            if (ok) ok = mbar_wait(bar_acc, acc_it & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            ++acc_it;
            if (!ok) break;
            tc_fence_after();
            const int64_t row = i0 + tid;
            float *Crow = A + (rb + row) * C + rb + j0;
            const uint32_t tm = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(half * 256);
#pragma unroll 1
            for (int qd = 0; qd < 8; ++qd) {
                if (j0 + qd * 32 >= m) break;                // columns past the matrix (same for the whole CTA)
                // on a diagonal tile the columns right of this row's 32-column group boundary are never used
                uint32_t v[32];
                tmem_ld32(tm + (uint32_t)(qd * 32), v);
                tmem_ld_wait();
                if (row < m && !(diag && qd * 32 > tid)) {
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        const int64_t col = j0 + qd * 32 + g4 * 4;
                        if (col + 3 < m) {
                            float4 *dst = reinterpret_cast<float4 *>(Crow + qd * 32 + g4 * 4);
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                                         "f"(-__uint_as_float(v[4 * g4 + 0])), "f"(-__uint_as_float(v[4 * g4 + 1])),
                                         "f"(-__uint_as_float(v[4 * g4 + 2])), "f"(-__uint_as_float(v[4 * g4 + 3]))
                                         : "memory");
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (col + e < m) Crow[qd * 32 + g4 * 4 + e] -= __uint_as_float(v[4 * g4 + e]);
                        }
                    }
                }
            }
            tc_fence_before();
        }
    } else {
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
            int ti, tj;
            syrk_tile(tile % ntri, nt, ti, tj);
            const bool diag = (ti == tj);
            for (int ks = 0; ks < kSteps && ok; ++ks) {
                const uint32_t s = it % kSyrk2Stages, ph = (it / kSyrk2Stages) & 1u;
                ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t st = smem_base + s * kSyrk2StageBytes;
                    const uint64_t bhi = make_desc_tf32(st + (diag ? 0 : 4) * kPieceBytes);
                    const uint64_t blo = make_desc_tf32(st + (diag ? 2 : 6) * kPieceBytes);
                    const uint32_t id = idesc_tf32(256);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint64_t ahi = make_desc_tf32(st + h * kPieceBytes);
                        const uint64_t alo = make_desc_tf32(st + (2 + h) * kPieceBytes);
                        const uint32_t d = tmem_base + (uint32_t)(h * 256);
                        umma_tf32(d, ahi, bhi, id, ks > 0 ? 1u : 0u);
                        umma_tf32(d, alo, bhi, id, 1u);
                        umma_tf32(d, ahi, blo, id, 1u);
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
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0 && status) atomicExch(status, FORGE_ERR_TIMEOUT);
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- inverse of an outer block's factor -----------------------------------------------------------------------
// M = L11^-1 for the W x W diagonal block that starts at column ob (W = 64 P), from the 64x64 inverses the diagonal
// kernel left behind:  M[p][p] = Dinv_p,  M[p][q] = -Dinv_p * sum_{q <= r < p} L[p][r] M[r][q]  (p > q).
// CTA (q, b) owns block column q of matrix b and walks p = q .. P-1 with the finished blocks in shared memory.
// Output, row-major [W][W]: transposed != 0: MT[k][c] = M[c][k] (rows of MT are K rows of the operand of L21 = A21 M^T);
// transposed == 0: M itself (K rows of the operand of T = L21 M, triangular inverse).  Only the zero block the
// multiplication reads is cleared (the off-diagonal 64 x 64 block of a 128-column tile).  With Uall given, the blocks
// below the diagonal of  diag(L) M  also go to U[J, J] (the scaled inverse the triangular-inverse pass builds; its
// 64 x 64 diagonal blocks are the diagonal kernel's).
__global__ void __launch_bounds__(256) chol_block_inv_kernel(const float *__restrict__ Aall, int64_t C, int64_t ob,
                                                             int P, int nblk, const float *__restrict__ dinv_all,
                                                             float *__restrict__ minv_all, int transposed,
                                                             float *__restrict__ Uall) {
    extern __shared__ __align__(16) float binv_smem[];
    float *Xs = binv_smem;                 // [P][64][64]  finished blocks of this block column
    float *Ls = Xs + (int64_t)P * 4096;    // [64][65]     left operand of the current product
    float *Ss = Ls + 64 * 65;              // [64][64]     the sum before the multiplication by Dinv_p
    const int q = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int64_t W = (int64_t)P * 64;
    const float *A = Aall + (int64_t)b * C * C;
    float *MT = minv_all + (int64_t)b * W * W;
    const int kb0 = (int)(ob / 64);
    float *U = Uall ? Uall + (int64_t)b * C * C : nullptr;
    if (q & 1) {
        for (int idx = tid; idx < 1024; idx += 256) {
            const int j = idx >> 4, i4 = (idx & 15) * 4;
            // transposed: rows of k-block q against columns of c-block q - 1; else rows of block q - 1, columns of q
            float *z = transposed ? MT + (int64_t)(64 * q + j) * W + 64 * (q - 1) + i4
                                  : MT + (int64_t)(64 * (q - 1) + j) * W + 64 * q + i4;
            *reinterpret_cast<float4 *>(z) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    auto load_block = [&](const float *src, int64_t ld) {     // Ls[i][k] = src[i * ld + k]
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = (tid >> 4) + 16 * u, k4 = (tid & 15) * 4;
            const float4 v = *reinterpret_cast<const float4 *>(src + (int64_t)i * ld + k4);
            Ls[i * 65 + k4 + 0] = v.x; Ls[i * 65 + k4 + 1] = v.y; Ls[i * 65 + k4 + 2] = v.z; Ls[i * 65 + k4 + 3] = v.w;
        }
    };
    for (int p = q; p < P; ++p) {
        float acc[4][4];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = (p == q && ty * 4 + ii == tx * 4 + jj) ? 1.0f : 0.0f;
        for (int r = q; r < p; ++r) {
            load_block(A + (ob + 64 * (int64_t)p) * C + ob + 64 * (int64_t)r, C);
            __syncthreads();
            const float *Xr = Xs + (int64_t)r * 4096;
#pragma unroll 8
            for (int k = 0; k < 64; ++k) {
                const float4 bv = *reinterpret_cast<const float4 *>(Xr + k * 64 + tx * 4);
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const float a = Ls[(ty * 4 + ii) * 65 + k];
                    acc[ii][0] = fmaf(-a, bv.x, acc[ii][0]);
                    acc[ii][1] = fmaf(-a, bv.y, acc[ii][1]);
                    acc[ii][2] = fmaf(-a, bv.z, acc[ii][2]);
                    acc[ii][3] = fmaf(-a, bv.w, acc[ii][3]);
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
            *reinterpret_cast<float4 *>(Ss + (ty * 4 + ii) * 64 + tx * 4) =
                make_float4(acc[ii][0], acc[ii][1], acc[ii][2], acc[ii][3]);
        load_block(dinv_all + ((int64_t)b * nblk + kb0 + p) * 2 * NB * NB, NB);      // Dinv_p, row-major
        __syncthreads();
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.0f;
#pragma unroll 8
        for (int k = 0; k < 64; ++k) {
            const float4 bv = *reinterpret_cast<const float4 *>(Ss + k * 64 + tx * 4);
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
                const float a = Ls[(ty * 4 + ii) * 65 + k];
                acc[ii][0] = fmaf(a, bv.x, acc[ii][0]);
                acc[ii][1] = fmaf(a, bv.y, acc[ii][1]);
                acc[ii][2] = fmaf(a, bv.z, acc[ii][2]);
                acc[ii][3] = fmaf(a, bv.w, acc[ii][3]);
            }
        }
        float *Xp = Xs + (int64_t)p * 4096;
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
            *reinterpret_cast<float4 *>(Xp + (ty * 4 + ii) * 64 + tx * 4) =
                make_float4(acc[ii][0], acc[ii][1], acc[ii][2], acc[ii][3]);
        if (transposed) {
            // MT[64 q + j][64 p + i] = X_p[i][j]: four consecutive i per store
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
                *reinterpret_cast<float4 *>(MT + (int64_t)(64 * q + tx * 4 + jj) * W + 64 * p + ty * 4) =
                    make_float4(acc[0][jj], acc[1][jj], acc[2][jj], acc[3][jj]);
        } else {
#pragma unroll
            for (int ii = 0; ii < 4; ++ii)
                *reinterpret_cast<float4 *>(MT + (int64_t)(64 * p + ty * 4 + ii) * W + 64 * q + tx * 4) =
                    make_float4(acc[ii][0], acc[ii][1], acc[ii][2], acc[ii][3]);
        }
        if (U && p > q) {
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
                const int64_t r = ob + 64 * p + ty * 4 + ii;
                const float dg = A[r * C + r];            // L[r][r]
                *reinterpret_cast<float4 *>(U + r * C + ob + 64 * q + tx * 4) =
                    make_float4(dg * acc[ii][0], dg * acc[ii][1], dg * acc[ii][2], dg * acc[ii][3]);
            }
        }
        __syncthreads();
    }
}

// ---- rows below an outer block:  L21 = A21 * M11^T on the tensor cores ---------------------------------------------
// A21 = rows [ob + W, C) x columns [ob, ob + W) as the earlier outer blocks' updates left it, M11 = the block inverse
// above.  One pass replaces, for these rows, the eight panel multiplications and the eight K = 64 updates of the
// right-looking form (each a read-modify-write of the strip in HBM) by one TF32 x3 GEMM that reads A21 once.
// A CTA owns a strip of 128 rows and walks the W / 128 column tiles from the LAST to the first: tile tj needs
// columns [0, 128 (tj + 1)) of the strip (M11 is lower triangular) and overwrites columns [128 tj, 128 tj + 128), which
// no later tile of the strip reads.  The A operand is row-major in memory (k contiguous): a producer thread owns one
// row, loads 32 k-values at a time and scatters the hi / lo parts into the MN-major piece (a warp's 32 rows are 128
// contiguous bytes of a K row: no bank conflict).  B pieces come from MT exactly like the update kernel's operands.
// The result goes to the lower triangle (row-major) and, transposed, to the upper triangle, where the update kernel
// reads its operands.
//
// The same kernel serves the blocked triangular inverse (MODE 1 and 2), which walks the outer blocks from the last to
// the first:  (D L^-1)[below, J] = -(D L^-1)[below, below] * ( L[below, J] * M_JJ ),  M_JJ the block inverse:
//   MODE 1: T = L21 * M_JJ in place of L21 (B rows from the row-major block inverse, K range [128 tj, W), column tiles
//           in ascending order so that no tile overwrites columns a later one reads);
//   MODE 2: U21 = -U22 * T, U22 = the finished scaled inverse of the rows below (row-major, lower triangular: K ends
//           at the strip's last row, entries right of the diagonal read as zero), T from A.
constexpr int kTrsmThreads = 160;
template <int MODE>
__global__ void __launch_bounds__(kTrsmThreads, 3) chol_trsm_tc_kernel(float *__restrict__ Aall, float *__restrict__ Uall,
                                                                        int64_t C, int64_t ob, int W,
                                                                        const float *__restrict__ minv_all, int nb,
                                                                        int32_t *status) {
    using namespace forge::tc;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + kSyrkStages * kSyrkStageBytes);  // full[4], empty[4], acc
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 9);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kSyrkStages), bar_acc = smem_u32(bars + 8);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kSyrkStages; ++s) {
            mbar_init(bar_full + 8 * s, 128);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"(128u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    const int64_t oe = ob + W, m = C - oe;
    const int nstrips = (int)((m + 127) / 128), ntj = W / 128;
    const int total = nb * nstrips;
    uint32_t it = 0, acc_it = 0;

    if (warp < 4) {
        const int jB = tid >> 5, c4 = tid & 31;
        const uint32_t swB[2] = {piece_offset(jB, c4), piece_offset(jB + 4, c4)};
        const uint32_t rowA = (uint32_t)((tid & 3) * 4);        // byte offset of this thread's row inside a 16-byte chunk
        uint32_t swA[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) swA[j] = piece_offset(j, tid >> 2) + rowA;
        bool ok = true;
        for (int unit = blockIdx.x; unit < total && ok; unit += gridDim.x) {
            const int b = unit / nstrips;
            const int64_t i0 = (int64_t)(unit % nstrips) * 128;
            float *A = Aall + (int64_t)b * C * C;
            float *U = (MODE == 2) ? Uall + (int64_t)b * C * C : nullptr;
            const float *MT = minv_all + (int64_t)b * W * W;
            const bool a_ok = (i0 + tid) < m;
            for (int tt = 0; tt < ntj && ok; ++tt) {
                const int tj = (MODE == 0) ? ntj - 1 - tt : tt;
                // K range of this tile and where its operands start
                const int k0 = (MODE == 1) ? 128 * tj : 0;
                const int K = (MODE == 0) ? 128 * (tj + 1) : (MODE == 1) ? W - 128 * tj : (int)(i0 + 128 < m ? i0 + 128 : m);
                const float *srcA = (MODE == 2) ? U + (oe + i0 + tid) * C + oe : A + (oe + i0 + tid) * C + ob + k0;
                const float *srcB = (MODE == 2) ? A + oe * C + ob + 128 * tj + 4 * c4 : MT + (int64_t)k0 * W + 128 * tj + 4 * c4;
                const int64_t ldb = (MODE == 2) ? C : (int64_t)W;
#pragma unroll 1
                for (int half = 0; half < K / 32 && ok; ++half) {
                    float4 ra[8], rbv[4][2];
#pragma unroll
                    for (int d = 0; d < 8; ++d)
                        ra[d] = a_ok ? ldg128_here(srcA + half * 32 + 4 * d) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int d = 0; d < 4; ++d)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            rbv[d][h] = ldg128_here(srcB + (int64_t)(half * 32 + d * kKS + jB + 4 * h) * ldb);
#pragma unroll
                    for (int d = 0; d < 4; ++d) {
                        if (!ok) break;
                        const uint32_t s = it % kSyrkStages, ph = (it / kSyrkStages) & 1u;
                        ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                        if (!ok) break;
                        uint8_t *stage = ring + s * kSyrkStageBytes;
                        float av[8] = {ra[2 * d].x, ra[2 * d].y, ra[2 * d].z, ra[2 * d].w,
                                       ra[2 * d + 1].x, ra[2 * d + 1].y, ra[2 * d + 1].z, ra[2 * d + 1].w};
                        if (MODE == 2) {
                            // lower triangular operand: column k of row i counts only for k <= i
                            const int64_t kfirst = (int64_t)half * 32 + d * kKS;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (kfirst + j > i0 + tid) av[j] = 0.0f;
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float hi = tf32_round(av[j]);
                            const float lo = tf32_round(__fsub_rn(av[j], hi));
                            *reinterpret_cast<float *>(stage + 0 * kPieceBytes + swA[j]) = hi;
                            *reinterpret_cast<float *>(stage + 1 * kPieceBytes + swA[j]) = lo;
                        }
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float4 hi, lo;
                            split4(rbv[d][h], hi, lo);
                            *reinterpret_cast<float4 *>(stage + 2 * kPieceBytes + swB[h]) = hi;
                            *reinterpret_cast<float4 *>(stage + 3 * kPieceBytes + swB[h]) = lo;
                        }
                        fence_proxy_async();
                        mbar_arrive(bar_full + 8 * s);
                        ++it;
                    }
                }
                // ---- epilogue of (strip, tj): one row per thread, both orientations
                if (ok) ok = mbar_wait(bar_acc, acc_it & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                ++acc_it;
                if (!ok) break;
                tc_fence_after();
                const int64_t row = i0 + tid, col0 = ob + 128 * (int64_t)tj;
#pragma unroll 1
                for (int qd = 0; qd < 4; ++qd) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(qd * 32), v);
                    tmem_ld_wait();
                    if (row < m) {
                        const float sgn = (MODE == 2) ? -1.0f : 1.0f;
                        float *dst = ((MODE == 2) ? U : A) + (oe + row) * C + col0 + qd * 32;
#pragma unroll
                        for (int g4 = 0; g4 < 8; ++g4)
                            *reinterpret_cast<float4 *>(dst + 4 * g4) =
                                make_float4(sgn * __uint_as_float(v[4 * g4 + 0]), sgn * __uint_as_float(v[4 * g4 + 1]),
                                            sgn * __uint_as_float(v[4 * g4 + 2]), sgn * __uint_as_float(v[4 * g4 + 3]));
                        if (MODE == 0) {
                            float *dstT = A + (col0 + qd * 32) * C + oe + row;
#pragma unroll
                            for (int c = 0; c < 32; ++c) dstT[(int64_t)c * C] = __uint_as_float(v[c]);
                        }
                    }
                }
                tc_fence_before();
            }
        }
    } else {
        bool ok = true;
        for (int unit = blockIdx.x; unit < total && ok; unit += gridDim.x) {
            const int64_t i0 = (int64_t)(unit % nstrips) * 128;
            for (int tt = 0; tt < ntj && ok; ++tt) {
                const int tj = (MODE == 0) ? ntj - 1 - tt : tt;
                const int K = (MODE == 0) ? 128 * (tj + 1) : (MODE == 1) ? W - 128 * tj : (int)(i0 + 128 < m ? i0 + 128 : m);
                const int kSteps = K / kKS;
                for (int ks = 0; ks < kSteps && ok; ++ks) {
                    const uint32_t s = it % kSyrkStages, ph = (it / kSyrkStages) & 1u;
                    ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t st = smem_base + s * kSyrkStageBytes;
                        const uint64_t ahi = make_desc_tf32(st), alo = make_desc_tf32(st + kPieceBytes);
                        const uint64_t bhi = make_desc_tf32(st + 2 * kPieceBytes), blo = make_desc_tf32(st + 3 * kPieceBytes);
                        const uint32_t id = idesc_tf32(128);
                        umma_tf32(tmem_base, ahi, bhi, id, ks > 0 ? 1u : 0u);
                        umma_tf32(tmem_base, alo, bhi, id, 1u);
                        umma_tf32(tmem_base, ahi, blo, id, 1u);
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
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0 && status) atomicExch(status, FORGE_ERR_TIMEOUT);
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(128u) : "memory");
    }
}

// ---- triangular inverse, block column j: M[below,j] = -(M[below,below] L[below,j]) Dinv_j -------
__global__ void __launch_bounds__(256, 3) trtri_step_kernel(const float *__restrict__ Aall, float *__restrict__ Uall,
                                                          int64_t C, int j, int nblk,
                                                          const float *__restrict__ dinv_all, int vec) {
    __shared__ __align__(16) float As[TM * AS];
    __shared__ __align__(16) float Bs[KC * 64];
    const int b = blockIdx.y, tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const float *A = Aall + (int64_t)b * C * C;
    float *U = Uall + (int64_t)b * C * C;
    const int64_t cb = (int64_t)j * NB, rb = cb + NB;
    const int64_t i0 = (int64_t)blockIdx.x * TM;
    const int m_valid = (int)imin64(TM, C - rb - i0);
    if (m_valid <= 0) return;
    float acc[8][4];
#pragma unroll
    for (int ii = 0; ii < 8; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.0f;
    // T = M[rows, rb .. rows] * L[rb .. , cb:cb+64]; the K range ends at this tile's last row
    const int K = (int)imin64(C - rb, i0 + TM);
    tile_gemm<64>(acc, U + (rb + i0) * C + rb, C, m_valid, A + rb * C + cb, C, NB, K, vec != 0, rb + i0, rb, As, Bs);
    // park T in the destination (rows are private to this CTA), then multiply by -Dinv_j
#pragma unroll
    for (int ii = 0; ii < 8; ++ii) {
        const int i = ty + 16 * ii;
        if (i < m_valid) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) U[(rb + i0 + i) * C + cb + tx * 4 + jj] = acc[ii][jj];
        }
    }
    __threadfence_block();
    __syncthreads();
    const float *dinv = dinv_all + ((int64_t)b * nblk + j) * 2 * NB * NB;
#pragma unroll
    for (int ii = 0; ii < 8; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.0f;
    tile_gemm<64>(acc, U + (rb + i0) * C + cb, C, m_valid, dinv, NB, NB, NB, vec != 0, -1, 0, As, Bs);
#pragma unroll
    for (int ii = 0; ii < 8; ++ii) {
        const int i = ty + 16 * ii;
        if (i < m_valid) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) U[(rb + i0 + i) * C + cb + tx * 4 + jj] = -acc[ii][jj];
        }
    }
}

// ---- rotate the lower-triangular scaled inverse into the upper triangle (in place) --------------
// U[t][k] = M[C-1-t][C-1-k] for k >= t.  Sources lie on or below the diagonal, destinations on or
// above it; the diagonal is 1 on both sides, so the pass is safe in place.
__global__ void rotate_upper_kernel(float *__restrict__ Uall, int64_t C, const int32_t *__restrict__ info,
                                    float *__restrict__ udiag) {
    const int b = blockIdx.z;
    float *U = Uall + (int64_t)b * C * C;
    const bool bad = info[b] != 0;
    const int64_t t = (int64_t)blockIdx.y * 8 + threadIdx.y;
    const int64_t k = (int64_t)blockIdx.x * 32 + threadIdx.x;
    if (t >= C || k >= C) return;
    if (bad) {
        U[t * C + k] = (t == k) ? 1.0f : 0.0f;
        if (t == k) udiag[(int64_t)b * C + t] = 1.0f;
        return;
    }
    if (k > t) U[t * C + k] = U[(C - 1 - t) * C + (C - 1 - k)];
}

// Inversion-free form.  With  J Hp J = L L^T  the matrix  V = J L J  is upper triangular and  Hp = V V^T.
// Scaling its columns to a unit diagonal gives  Vt = V diag(V)^-1 = (the reference's unit factor U)^-1, and the
// column solver can work from Vt directly:  x_t = w_t + sum_{s<t} (w_s - deq_s) Vt[s,t]  is the same recurrence
// as  x_t = w_t - sum_{s<t} err_s U[s,t]  (substitute err = (w - deq) Vt).  So no triangular inverse is needed.
// This pass writes  out[s][t] = -Vt[s,t] = -L[C-1-s][C-1-t] * udiag[t]  for t > s  (udiag[t] = 1 / L[C-1-t][C-1-t]),
// 1 on the diagonal.  Sources are on or below the diagonal, destinations above it, so it may run in place.
__global__ void rotate_scale_neg_kernel(const float *__restrict__ Lall, float *__restrict__ Oall, int64_t C,
                                        const int32_t *__restrict__ info, float *__restrict__ udiag) {
    // a thread handles four consecutive destination columns t .. t+3 of row s (sources are four consecutive, reversed,
    // elements of one row of L); vector accesses where C is a multiple of 4
    const int b = blockIdx.z;
    const float *L = Lall + (int64_t)b * C * C;
    float *O = Oall + (int64_t)b * C * C;
    const bool bad = info[b] != 0;
    const int64_t s = (int64_t)blockIdx.y * 8 + threadIdx.y;
    const int64_t t0 = ((int64_t)blockIdx.x * 32 + threadIdx.x) * 4;
    if (s >= C || t0 >= C) return;
    if (bad) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int64_t t = t0 + e;
            if (t < C && t >= s) O[s * C + t] = (t == s) ? 1.0f : 0.0f;
            if (t == s) udiag[(int64_t)b * C + t] = 1.0f;
        }
        return;
    }
    if (t0 + 3 <= s) return;                       // nothing of this quad lies above the diagonal
    const float *ud = udiag + (int64_t)b * C;
    if ((C & 3) == 0 && t0 > s) {
        // whole quad above the diagonal: destination columns t0..t0+3 <- source columns C-1-t0 .. C-4-t0 (one float4)
        const float4 src = *reinterpret_cast<const float4 *>(L + (C - 1 - s) * C + (C - 4 - t0));
        const float4 d = *reinterpret_cast<const float4 *>(ud + t0);
        *reinterpret_cast<float4 *>(O + s * C + t0) =
            make_float4(-__fmul_rn(src.w, d.x), -__fmul_rn(src.z, d.y), -__fmul_rn(src.y, d.z), -__fmul_rn(src.x, d.w));
        return;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int64_t t = t0 + e;
        if (t < C && t > s) O[s * C + t] = -__fmul_rn(L[(C - 1 - s) * C + (C - 1 - t)], ud[t]);
    }
}

__global__ void unit_diag_kernel(float *__restrict__ Oall, int64_t C) {
    const int b = blockIdx.y;
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < C) Oall[(int64_t)b * C * C + t * C + t] = 1.0f;
}

__global__ void zero_lower_kernel(float *__restrict__ Uall, int64_t C) {
    const int b = blockIdx.z;
    float *U = Uall + (int64_t)b * C * C;
    const int64_t t = (int64_t)blockIdx.y * 8 + threadIdx.y;
    const int64_t k = (int64_t)blockIdx.x * 32 + threadIdx.x;
    if (t < C && k < t) U[t * C + k] = 0.0f;
}

__global__ void info_clear_kernel(int32_t *info, int nb, int32_t *status) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < nb) info[b] = 0;
    if (b == 0) *status = 0;
}

// a bounded wait of a tensor-core kernel ran out: report every matrix of the batch as not factorised
__global__ void status_to_info_kernel(int32_t *info, int nb, const int32_t *status) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < nb && *status != 0 && info[b] == 0) info[b] = 0x40000000;
}

}  // namespace

// width of the outer blocks of the two-level factorisation (measured: wider blocks pay from C ~ 4096 on)
static inline int64_t chol_outer(int64_t C) { return (C >= 4096) ? 2 * kOuter : kOuter; }

// workspace: the (Dinv, Dinv^T) pairs of every 64-column block, one inverted outer block per matrix, the status word
extern "C" int64_t forge_chol_workspace_bytes(int nb, int64_t C) {
    const int64_t nblk = cdiv(C, NB), W = chol_outer(C);
    return ((int64_t)nb * nblk * 2 * NB * NB + (int64_t)nb * W * W) * (int64_t)sizeof(float) + 256;
}

extern "C" int64_t forge_chol_workspace_bytes(int nb, int64_t C);
static void launch_factor(float *A, int nb, int64_t C, float *U, float *udiag, int32_t *info, float *dinv, int vec,
                          cudaStream_t st) {
    // the last 256 bytes of the workspace hold the status word of the tensor-core kernels
    int32_t *status = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(dinv) + forge_chol_workspace_bytes(nb, C) - 256);
    const int nblk = (int)cdiv(C, NB);
    // per-device attribute: set on the device that is current for this call
    cudaFuncSetAttribute(chol_syrk_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSyrkSmem);
    const char *env = getenv("FORGE_SYRK_IMPL");
    const bool syrk_simt = env && strcmp(env, "simt") == 0;   // cross-checks: plain-FMA trailing update
    const int64_t outer = chol_outer(C);
    float *minv = dinv + (int64_t)nb * nblk * 2 * NB * NB;
    info_clear_kernel<<<(nb + 127) / 128, 128, 0, st>>>(info, nb, status); FORGE_NOTE_LAUNCH();
    if (!vec || syrk_simt) {
        // plain right-looking form: every panel updates the whole matrix behind it
        for (int k = 0; k < nblk; ++k) {
            chol_diag_kernel<<<nb, NB, 0, st>>>(A, C, k, nblk, dinv, U, udiag, info); FORGE_NOTE_LAUNCH();
            const int64_t m = C - (int64_t)(k + 1) * NB;
            if (m > 0) {
                const unsigned nt = (unsigned)cdiv(m, TM);
                chol_panel_kernel<<<dim3(nt, nb), 256, 0, st>>>(A, C, k, nblk, dinv, vec, C); FORGE_NOTE_LAUNCH();
                chol_syrk_kernel<<<dim3(nt, nt, nb), 256, 0, st>>>(A, C, k, vec); FORGE_NOTE_LAUNCH();
            }
        }
    } else {
        // T[rows [r0, row_end), columns [r0, r0 + ncols)] -= P P^T with the K factored columns from kb on
        auto update = [&](int64_t kb, int K, int64_t r0, int64_t ncols, int64_t row_end) {
            const int64_t m = row_end - r0, nc = ncols < m ? ncols : m;
            const int total = nb * syrk_tiles((int)cdiv(m, (int64_t)128), (int)cdiv(nc, (int64_t)128));
            const int grid = total < 148 * 3 ? total : 148 * 3;
            chol_syrk_tc_kernel<<<grid, kSyrkThreads, kSyrkSmem, st>>>(A, C, kb, K, r0, ncols, nb, status, row_end);
            FORGE_NOTE_LAUNCH();
        };
        cudaFuncSetAttribute(chol_trsm_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSyrkSmem);
        cudaFuncSetAttribute(chol_syrk256_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSyrk2Smem);
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int binv_smem = (int)((outer / NB * 4096 + 64 * 65 + 4096) * sizeof(float));
        cudaFuncSetAttribute(chol_block_inv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, binv_smem);
        for (int64_t ob = 0; ob < C; ob += outer) {
            const int64_t oe = imin64(C, ob + outer);
            // the outer block's own rows: 64-column panels, right-looking inside the block
            for (int k = (int)(ob / NB); (int64_t)k * NB < oe; ++k) {
                chol_diag_kernel<<<nb, NB, 0, st>>>(A, C, k, nblk, dinv, U, udiag, info); FORGE_NOTE_LAUNCH();
                const int64_t rb = (int64_t)(k + 1) * NB;
                if (rb >= oe) continue;
                chol_panel_kernel<<<dim3((unsigned)cdiv(oe - rb, (int64_t)TM), nb), 256, 0, st>>>(A, C, k, nblk, dinv, vec, oe);
                FORGE_NOTE_LAUNCH();
                update((int64_t)k * NB, NB, rb, oe - rb, oe);
            }
            if (oe < C) {
                // the rows behind it: block inverse, ONE multiplication for the panel, ONE update of the rest
                const int P = (int)(outer / NB);
                chol_block_inv_kernel<<<dim3(P, nb), 256, binv_smem, st>>>(A, C, ob, P, nblk, dinv, minv, 1, nullptr);
                FORGE_NOTE_LAUNCH();
                const int64_t units = (int64_t)nb * cdiv(C - oe, (int64_t)128);
                chol_trsm_tc_kernel<0><<<(unsigned)(units < 148 * 3 ? units : 148 * 3), kTrsmThreads, kSyrkSmem, st>>>(
                    A, nullptr, C, ob, (int)outer, minv, nb, status);
                FORGE_NOTE_LAUNCH();
                if (C - oe > 256) {
                    const int nt2 = (int)cdiv(C - oe, (int64_t)256);
                    const int total2 = nb * syrk_tiles(nt2, nt2);
                    chol_syrk256_tc_kernel<<<total2 < sms ? total2 : sms, kSyrk2Threads, kSyrk2Smem, st>>>(
                        A, C, ob, (int)(oe - ob), oe, nb, status);
                    FORGE_NOTE_LAUNCH();
                } else {
                    update(ob, (int)(oe - ob), oe, C - oe, C);
                }
            }
        }
    }
    status_to_info_kernel<<<(nb + 127) / 128, 128, 0, st>>>(info, nb, status); FORGE_NOTE_LAUNCH();
}

extern "C" int forge_chol_factor_batched(float *A, int nb, int64_t C, float *udiag, int32_t *info, void *ws,
                                         void *stream) {
    FORGE_REQUIRE(A && udiag && info && ws, "null pointer");
    FORGE_REQUIRE(nb > 0 && C > 0, "empty batch");
    FORGE_REQUIRE((uintptr_t)ws % 16 == 0, "workspace must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = (C % 4 == 0) && ((uintptr_t)A % 16 == 0);
    launch_factor(A, nb, C, nullptr, udiag, info, (float *)ws, vec, st);
    dim3 g2((unsigned)cdiv(C, 128), (unsigned)cdiv(C, 8), nb);
    rotate_scale_neg_kernel<<<g2, dim3(32, 8), 0, st>>>(A, A, C, info, udiag); FORGE_NOTE_LAUNCH();
    unit_diag_kernel<<<dim3((unsigned)cdiv(C, 256), nb), 256, 0, st>>>(A, C); FORGE_NOTE_LAUNCH();
    return check_launch("forge_chol_factor_batched");
}

extern "C" int forge_chol_inv_upper_batched(float *A, int nb, int64_t C, float *U, float *udiag, int32_t *info,
                                            int zero_lower, void *ws, void *stream) {
    FORGE_REQUIRE(A && U && udiag && info && ws, "null pointer");
    FORGE_REQUIRE(nb > 0 && C > 0, "empty batch");
    FORGE_REQUIRE(A != U, "A must not alias U");
    FORGE_REQUIRE((uintptr_t)ws % 16 == 0, "workspace must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int nblk = (int)cdiv(C, NB);
    float *dinv = (float *)ws;
    const int vec = (C % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)U % 16 == 0);
    launch_factor(A, nb, C, U, udiag, info, dinv, vec, st);
    const char *env = getenv("FORGE_SYRK_IMPL");
    const bool simt = env && strcmp(env, "simt") == 0;
    const int64_t outer = chol_outer(C);
    if (vec && !simt && C % 128 == 0 && C > outer) {
        // blocked triangular inverse on the tensor cores, outer blocks from the last to the first: block inverse
        // (also D M_JJ into U[J, J]), T = L21 M_JJ in place, U21 = -U22 T
        float *minv = dinv + (int64_t)nb * nblk * 2 * NB * NB;
        int32_t *status = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(dinv) + forge_chol_workspace_bytes(nb, C) - 256);
        cudaFuncSetAttribute(chol_trsm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSyrkSmem);
        cudaFuncSetAttribute(chol_trsm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSyrkSmem);
        const int binv_smem = (int)((outer / NB * 4096 + 64 * 65 + 4096) * sizeof(float));
        cudaFuncSetAttribute(chol_block_inv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, binv_smem);
        for (int64_t ob = ((C - 1) / outer) * outer; ob >= 0; ob -= outer) {
            const int64_t oe = imin64(C, ob + outer);
            const int P = (int)((oe - ob) / NB);
            chol_block_inv_kernel<<<dim3(P, nb), 256, binv_smem, st>>>(A, C, ob, P, nblk, dinv, minv, 0, U);
            FORGE_NOTE_LAUNCH();
            if (oe < C) {
                const int64_t units = (int64_t)nb * cdiv(C - oe, (int64_t)128);
                const unsigned grid = (unsigned)(units < 148 * 3 ? units : 148 * 3);
                chol_trsm_tc_kernel<1><<<grid, kTrsmThreads, kSyrkSmem, st>>>(A, U, C, ob, (int)outer, minv, nb, status);
                FORGE_NOTE_LAUNCH();
                chol_trsm_tc_kernel<2><<<grid, kTrsmThreads, kSyrkSmem, st>>>(A, U, C, ob, (int)outer, minv, nb, status);
                FORGE_NOTE_LAUNCH();
            }
        }
        status_to_info_kernel<<<(nb + 127) / 128, 128, 0, st>>>(info, nb, status); FORGE_NOTE_LAUNCH();
    } else {
        for (int j = nblk - 2; j >= 0; --j) {
            const int64_t m = C - (int64_t)(j + 1) * NB;
            const unsigned nt = (unsigned)cdiv(m, TM);
            trtri_step_kernel<<<dim3(nt, nb), 256, 0, st>>>(A, U, C, j, nblk, dinv, vec); FORGE_NOTE_LAUNCH();
        }
    }
    dim3 g2((unsigned)cdiv(C, 32), (unsigned)cdiv(C, 8), nb);
    rotate_upper_kernel<<<g2, dim3(32, 8), 0, st>>>(U, C, info, udiag); FORGE_NOTE_LAUNCH();
    if (zero_lower) { zero_lower_kernel<<<g2, dim3(32, 8), 0, st>>>(U, C); FORGE_NOTE_LAUNCH(); }
    return check_launch("forge_chol_inv_upper_batched");
}
