/*
 * CPU oracle for the CUDA-only half of the 4Bit-Forge GPTQ / SparseGPT path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's CUDA kernels so that the sm_100a kernels can be checked
 * against it.  Nothing in the shipped library links or calls it; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * Parity status: PINNED.  The reference repository holds no tests or golden
 * vectors for these kernels, so the vectors were made from the reference
 * itself: its quant_grid.cu, solver.cu, solver_sparsegptq14.cu and
 * bitpacking_sparsegptq14.cu are compiled for sm_100a where they lie in the
 * reference checkout (oracle/ref_build.py -> oracle/_ref), run on a B200 by
 * tests/golden/make_golden_gpu.py, and their inputs and outputs are stored in
 * tests/golden/ref_kernels_b200.npz.  tests/test_oracle_ref_kernels.py replays
 * this file on those inputs: scales, zeros, the winning shrink factors, codes,
 * 1:4 masks and packed words are all bit-identical.  (dense int4 packing is
 * pinned against the installed compressed_tensors.pack_to_int32 instead.)
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/build.py).
 * -ffp-contract=off matters: every fused multiply-add below is an explicit
 * fmaf() exactly where the CUDA source has one (or where nvcc's default
 * -fmad=true contracts a*b+c), and nowhere else.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define FO_EPS 1e-12f

int fo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* round-to-nearest-even float -> bf16 bits (CUDA __float2bfloat16_rn) */
static inline uint16_t f32_to_bf16_rn(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* lrintf under the default rounding mode = round half to even, as on the GPU */
static inline float rint_even(float x) { return nearbyintf(x); }

/* ------------------------------------------------------------------------- *
 * Per-group min/max scale and zero.
 * Follows forge/backend/cuda/quant_grid.cu:42-99 (build_quantization_grid).
 * X is [RG, gs] fp32 row-major; outputs scales[RG], qzeros[RG].
 * ------------------------------------------------------------------------- */
void fo_absmax_grid(const float *X, int64_t RG, int64_t gs, int bits, int sym,
                    float *scales, float *qzeros) {
    const float maxq = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < RG; ++g) {
        const float *grp = X + g * gs;
        float mn = 1e30f, mx = -1e30f;               /* quant_grid.cu:63-64 */
        for (int64_t i = 0; i < gs; ++i) {
            mx = fmaxf(mx, grp[i]);
            mn = fminf(mn, grp[i]);
        }
        float s, q0;
        if (sym) {                                    /* quant_grid.cu:81-84 */
            float amax = fmaxf(fabsf(mn), fabsf(mx));
            s = fmaf(2.0f / maxq, amax, FO_EPS);  /* a*b+c: one FMA under nvcc's default -fmad=true */
            q0 = 0.5f * (maxq + 1.0f);
        } else {                                      /* quant_grid.cu:85-92 */
            s = (mx - mn) / maxq + FO_EPS;
            float q = -mn / s;
            q = rint_even(q);
            q0 = fminf(fmaxf(q, 0.0f), maxq);
        }
        scales[g] = s;
        qzeros[g] = q0;
    }
}

/* ------------------------------------------------------------------------- *
 * MSE (L^norm) shrink-factor search.
 * Follows forge/backend/cuda/quant_grid.cu:101-183.  The kernel runs one warp
 * per group: lane l holds values l, l+32, ...; the per-candidate loss is the
 * lane-local sum (in that order) reduced by a shfl_down tree (16,8,4,2,1).
 * That summation order is reproduced here.  The kernel's __logf/__expf are
 * approximate hardware functions; logf/expf stand in for them, so a candidate
 * whose loss ties another to ~1e-6 relative may be chosen differently.
 * gs must be 32, 64 or 128 (quant_grid.cu:254-284).
 * ------------------------------------------------------------------------- */
int fo_mse_grid(const float *X, float *scales, float *qzeros, const float *cand,
                int64_t RG, int64_t gs, int64_t P, int bits, float norm, int sym) {
    if (gs != 32 && gs != 64 && gs != 128) return -1;
    const int vpl = (int)(gs / 32);
    const float maxq = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < RG; ++g) {
        const float sg = scales[g], q0g = qzeros[g];
        float xmin = 0.0f;
        if (!sym) xmin = -(sg * q0g);                 /* quant_grid.cu:129-132 */
        float best_s = sg, best_q = q0g, best_loss = FLT_MAX;
        const float *grp = X + g * gs;
        for (int64_t p = 0; p < P; ++p) {
            const float s = sg * cand[p];
            const float rcp = 1.0f / (s + FO_EPS);
            float q0;
            if (sym) q0 = q0g;
            else {
                q0 = -xmin * rcp;
                q0 = fminf(fmaxf(rint_even(q0), 0.0f), maxq);
            }
            float lane[32];
            for (int l = 0; l < 32; ++l) {
                float loss = 0.0f;
                for (int i = 0; i < vpl; ++i) {       /* quant_grid.cu:158-168 */
                    float v = grp[l + 32 * i];
                    float q = rint_even(fmaf(v, rcp, q0));
                    q = fminf(fmaxf(q, 0.0f), maxq);
                    float diff = fmaf(q - q0, s, -v);
                    float e = fmaxf(fabsf(diff), 1e-20f);
                    float val = expf(logf(e) * norm);
                    loss += val;
                }
                lane[l] = loss;
            }
            for (int off = 16; off > 0; off >>= 1)    /* warpReduceSum, :15-21 */
                for (int l = 0; l < off; ++l) lane[l] += lane[l + off];
            if (lane[0] < best_loss) {                /* first minimum wins */
                best_loss = lane[0];
                best_s = s;
                best_q = q0;
            }
        }
        scales[g] = best_s;
        qzeros[g] = best_q;
    }
    return 0;
}

/* forge/backend/cuda/solver.cu:9-22 (quantize_scalar).  The source's
 * `x * inv_s + q0` is contracted to one FMA by nvcc's default -fmad=true. */
static inline void quantize_scalar(float x, float inv_s, float s, float q0, int maxq,
                                   float *err, uint8_t *qb, float *deq) {
    float biased = fmaf(x, inv_s, q0);
    long q = lrintf(biased);
    if (q < 0) q = 0;
    else if (q > maxq) q = maxq;
    *deq = fmaf((float)q, s, -q0 * s);
    *err = x - *deq;
    *qb = (uint8_t)q;
}

/* ------------------------------------------------------------------------- *
 * GPTQ front-to-back solver, and the SparseGPT 1:4 variant.
 * Follows forge/backend/cuda/solver.cu:26-154 and
 * forge/backend/cuda/solver_sparsegptq14.cu:29-200.
 *   W      [C,R] fp32, mutated to the dequantised weights
 *   U      [C,C] fp32, unit-diagonal upper factor (row-normalised)
 *   uinv   [C]   fp32 1/diag of the un-normalised factor (sparse only, else NULL)
 *   scales,qzeros [C,R] fp32 per element
 *   q      [C,R] uint8 out;  M [ceil(C/32),R] uint32 out (sparse only)
 * Columns are processed in blocks of `block` (32 in the reference); inside a
 * block every column's error is propagated to the later columns of the block
 * (rank-1, FMA), after a block the remaining rows of W get W -= U_blk^T E
 * (the reference's fp32 addmm_, solver.cu:146-150).  Rows of the weight (the
 * R axis) are independent, so threads own strips of r.
 * ------------------------------------------------------------------------- */
void fo_gptq_solve(float *W, const float *U, const float *uinv, const float *scales,
                   const float *qzeros, int bits, int64_t R, int64_t C, int block,
                   int sparse14, uint8_t *qout, uint32_t *M) {
    const int maxq = (1 << bits) - 1;
    const int64_t RS = 64; /* strip of rows handled by one thread at a time */
    const int64_t nstrip = (R + RS - 1) / RS;
#pragma omp parallel
    {
        float *E = (float *)malloc(sizeof(float) * (size_t)block * RS);
        float *acc = (float *)malloc(sizeof(float) * RS);
#pragma omp for schedule(dynamic, 1)
        for (int64_t sidx = 0; sidx < nstrip; ++sidx) {
            const int64_t r0 = sidx * RS;
            const int64_t nr = (R - r0 < RS) ? (R - r0) : RS;
            for (int64_t bs = 0; bs < C; bs += block) {
                const int64_t be = (bs + block < C) ? bs + block : C;
                const int B = (int)(be - bs);
                uint32_t maskbits[64];
                for (int64_t i = 0; i < nr; ++i) maskbits[i] = 0u;
                for (int t = 0; t < B; ++t) {
                    const int64_t cid = bs + t;
                    float *wrow = W + cid * R + r0;
                    if (sparse14 && (t % 4 == 0)) {
                        /* solver_sparsegptq14.cu:80-102: keep argmax_k |x*uinv|,
                         * first maximum wins, on the error-compensated values. */
                        for (int64_t i = 0; i < nr; ++i) {
                            float best = -1e30f;
                            int bidx = -1;
                            for (int k = 0; k < 4; ++k) {
                                if (cid + k >= C) continue;
                                float sc = fabsf(W[(cid + k) * R + r0 + i] * uinv[cid + k]);
                                if (best < sc) { best = sc; bidx = k; }
                            }
                            if (bidx > -1) maskbits[i] |= (1u << (t + bidx));
                        }
                    }
                    for (int64_t i = 0; i < nr; ++i) {
                        float err = 0.f, deq = 0.f;
                        uint8_t qb = 0;
                        int keep = 1;
                        if (sparse14) keep = (int)((maskbits[i] >> t) & 1u);
                        if (keep) {
                            float s = scales[cid * R + r0 + i];
                            float q0 = qzeros[cid * R + r0 + i];
                            float inv_s = 1.0f / (s + FO_EPS);
                            quantize_scalar(wrow[i], inv_s, s, q0, maxq, &err, &qb, &deq);
                        } else {
                            err = wrow[i];                /* solver_sparsegptq14.cu:118-120 */
                        }
                        qout[cid * R + r0 + i] = qb;
                        wrow[i] = deq;
                        E[(int64_t)t * RS + i] = err;
                    }
                    for (int k = t + 1; k < B; ++k) {     /* solver.cu:90-93 */
                        const float alpha = U[cid * C + bs + k];
                        float *xk = W + (bs + k) * R + r0;
                        const float *et = E + (int64_t)t * RS;
                        for (int64_t i = 0; i < nr; ++i) xk[i] = fmaf(-alpha, et[i], xk[i]);
                    }
                }
                if (sparse14 && M) {                      /* solver_sparsegptq14.cu:134-136 */
                    for (int64_t i = 0; i < nr; ++i) M[(bs >> 5) * R + r0 + i] = maskbits[i];
                }
                for (int64_t k = be; k < C; ++k) {        /* solver.cu:146-150 */
                    for (int64_t i = 0; i < nr; ++i) acc[i] = 0.0f;
                    for (int t = 0; t < B; ++t) {
                        const float u = U[(bs + t) * C + k];
                        const float *et = E + (int64_t)t * RS;
                        for (int64_t i = 0; i < nr; ++i) acc[i] = fmaf(u, et[i], acc[i]);
                    }
                    float *wk = W + k * R + r0;
                    for (int64_t i = 0; i < nr; ++i) wk[i] = wk[i] - acc[i];
                }
            }
        }
        free(E);
        free(acc);
    }
}

/* ------------------------------------------------------------------------- *
 * Sparse 1:4 + int4 "Wpair" packer.
 * Follows forge/backend/cuda/bitpacking_sparsegptq14.cu:58-107.
 *   q [C,R] uint8, M [G32,R] uint32, scales [G32,R] fp32 -> out [G2,R,2] uint64
 *   u64 = bf16(scale)<<48 | idx16<<32 | qw32 ; default nibble 8 ; odd tail -> 0
 * ------------------------------------------------------------------------- */
void fo_pack_sparse14(const uint8_t *q, const uint32_t *M, const float *scales,
                      int64_t C, int64_t R, int64_t G32, uint64_t *out) {
    const int64_t G2 = (G32 + 1) >> 1;
#pragma omp parallel for schedule(static)
    for (int64_t g2 = 0; g2 < G2; ++g2) {
        for (int64_t r = 0; r < R; ++r) {
            for (int h = 0; h < 2; ++h) {
                const int64_t gid = 2 * g2 + h;
                uint64_t word = 0;
                if (gid < G32) {
                    uint32_t bitmask = M[gid * R + r];
                    uint16_t idx16 = 0;
                    uint32_t qw32 = 0x88888888u;
                    for (int i = 0; i < 8; ++i) {
                        uint32_t sub = (bitmask >> (4 * i)) & 0xFu;
                        if (sub == 0u) continue;
                        int c = __builtin_ffs((int)sub) - 1;
                        idx16 |= (uint16_t)((c & 0x3) << (2 * i));
                        int64_t cid = gid * 32 + i * 4 + c;
                        if (cid < C) {
                            uint32_t qq = (uint32_t)(q[cid * R + r] & 0xFu);
                            uint32_t sh = 4u * (uint32_t)i;
                            qw32 = (qw32 & ~(0xFu << sh)) | ((qq & 0xFu) << sh);
                        }
                    }
                    uint16_t sb = f32_to_bf16_rn(scales[gid * R + r]);
                    word = ((uint64_t)sb << 48) | ((uint64_t)idx16 << 32) | (uint64_t)qw32;
                }
                out[(g2 * R + r) * 2 + h] = word;
            }
        }
    }
}

/* ------------------------------------------------------------------------- *
 * Dense int4 "pack-quantized" packer.
 * Follows pack_quantized.py:279-313 (pack_weight) and the third-party
 * compressed_tensors.compressors.pack_to_int32 it calls (version 0.15.0.1):
 *   v = int8(q) - int8(zero of the element's group)          (int8 wrap)
 *   u = uint8(int8(v + 8))                                    (no 4-bit mask)
 *   packed[r, j] = sum_{i<8} (int32(u[r, 8j+i]) << 4i)        (int32 wrap; the
 *                   columns beyond C contribute 0)
 *   q [R,C] uint8; zeros [R,G] (already integral) ; out [R, ceil(C/8)] int32
 * ------------------------------------------------------------------------- */
void fo_pack_int4(const uint8_t *q, const float *zeros, int64_t R, int64_t C, int64_t gs,
                  int32_t *out) {
    const int64_t G = (C + gs - 1) / gs;
    const int64_t CP = (C + 7) / 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < R; ++r) {
        for (int64_t j = 0; j < CP; ++j) {
            uint32_t acc = 0;
            for (int i = 0; i < 8; ++i) {
                int64_t c = 8 * j + i;
                if (c >= C) continue;
                int8_t z = (int8_t)(int)zeros[r * G + c / gs];
                int8_t v = (int8_t)((int8_t)q[r * C + c] - z);
                uint8_t u = (uint8_t)(int8_t)(v + 8);
                acc += ((uint32_t)u) << (4 * i);
            }
            out[r * CP + j] = (int32_t)acc;
        }
    }
}

/* ------------------------------------------------------------------------- *
 * Inference GEMM over the Wpair layout.
 * Follows forge/backend/cuda/sparse14_gemm.cu:49-140 (the kernel; the launcher's zero padding of X, :318-336, is
 * the bounds check below).  Per output row r, token n and 32-channel half: sum = fma(x, q4 - 8, sum) over the eight
 * groups in order, acc = fma(sum, scale, acc); Y = bf16_rn(acc).  nvcc's default contraction fuses the kernel's
 * `sum += x * w` and `acc += sum * scale`, hence the explicit fmaf here.
 *   wpair [G2,R,2] uint64, X bf16 bits [N,C] (uint16), Y bf16 bits [N,R] (uint16)
 * ------------------------------------------------------------------------- */
static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void fo_sparse14_gemm(const uint64_t *wpair, const uint16_t *X, int64_t N, int64_t R, int64_t C, uint16_t *Y) {
    const int64_t G2 = (C + 63) / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < R; ++r) {
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int64_t g2 = 0; g2 < G2; ++g2) {
                for (int half = 0; half < 2; ++half) {
                    const uint64_t u = wpair[(g2 * R + r) * 2 + half];
                    const uint32_t qw32 = (uint32_t)(u & 0xFFFFFFFFull), hi = (uint32_t)(u >> 32);
                    const uint32_t idx16 = hi & 0xFFFFu;
                    const float scale = bf16_bits_to_f32((uint16_t)(hi >> 16));
                    const int64_t base = g2 * 64 + half * 32;
                    float sum = 0.0f;
                    for (int i = 0; i < 8; ++i) {
                        const int64_t c = base + 4 * i + ((idx16 >> (2 * i)) & 3u);
                        const float w = (float)(int)((qw32 >> (4 * i)) & 0xFu) - 8.0f;
                        const float x = (c < C) ? bf16_bits_to_f32(X[n * C + c]) : 0.0f;
                        sum = fmaf(x, w, sum);
                    }
                    acc = fmaf(sum, scale, acc);
                }
            }
            Y[n * R + r] = f32_to_bf16_rn(acc);
        }
    }
}
