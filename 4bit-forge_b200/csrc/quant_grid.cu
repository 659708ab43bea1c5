// Per-group scale / zero grid: min-max, and the L^p shrink-factor search.
//
// The reference kernels (forge/backend/cuda/quant_grid.cu:42-183) give one warp to a group, lane l holding
// elements l, l+32, ..., and the candidate that wins the search depends on the order in which the per-element
// errors are summed: lane-local sum first, then a shfl_down tree.  Every kernel here reproduces that order (the
// thread-per-candidate kernels with a 6-entry stack visited in bit-reversed lane order), so scales and zeros are
// bit-identical to the reference's.  What changes is the data path and the amount of work: the weights are read
// once, in their storage type (bf16, 2 B/element, instead of an fp32 copy), min-max and search share one staging,
// and the search abandons a candidate as soon as its partial loss exceeds a finished candidate's
// (mse_prune_kernel).  Three kernels:
//   quant_grid_kernel : warp per group; min-max grids and any group size;
//   mse_grid_kernel   : exhaustive search, one thread per (group, candidate pair); group sizes 32 / 64 and the
//                       cross-check FORGE_GRID_IMPL=exhaustive;
//   mse_prune_kernel  : group size 128, up to 128 candidates, exact pruning; the default.
// The search is bound by the special-function pipe (lg2 + ex2 per element-candidate evaluated), not by HBM.
#include "common.cuh"
#include <float.h>
#include <stdlib.h>
#include <string.h>

using namespace forge;

namespace {

constexpr float kEps = 1e-12f;

template <int GS, bool BF16, bool ABSMAX>
__global__ void __launch_bounds__(256)
quant_grid_kernel(const void *__restrict__ Wv, int64_t rows, int64_t C, int64_t G, int gs_dyn, int bits,
                  int symmetric, const float *__restrict__ cand, int P, float norm,
                  float *__restrict__ scales, float *__restrict__ qzeros) {
    constexpr int VPL = (GS > 0) ? GS / 32 : 1;
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const float maxq = (float)((1 << bits) - 1);
    const int64_t n_groups = rows * G;
    const int gs = (GS > 0) ? GS : gs_dyn;

    for (int64_t g = warp_id; g < n_groups; g += warps_total) {
        const int64_t r = g / G, gi = g % G;
        const int64_t col0 = gi * gs;
        const int64_t base = r * C + col0;
        float vals[VPL];
        float sg, q0g;
        if (GS > 0) {
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int64_t c = col0 + lane + 32 * v;
                float x = 0.0f;  // zero padding of the last group (forge/gptq.py:194-195)
                if (c < C) {
                    if (BF16) x = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(Wv)[base + lane + 32 * v]);
                    else x = reinterpret_cast<const float *>(Wv)[base + lane + 32 * v];
                }
                vals[v] = x;
            }
        }
        if (ABSMAX) {
            float mn = 1e30f, mx = -1e30f;
            if (GS > 0) {
#pragma unroll
                for (int v = 0; v < VPL; ++v) { mx = fmaxf(mx, vals[v]); mn = fminf(mn, vals[v]); }
            } else {
                for (int i = lane; i < gs; i += 32) {
                    const int64_t c = col0 + i;
                    float x = 0.0f;
                    if (c < C) x = BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(Wv)[base + i])
                                        : reinterpret_cast<const float *>(Wv)[base + i];
                    mx = fmaxf(mx, x);
                    mn = fminf(mn, x);
                }
            }
            mx = warp_max(mx);
            mn = warp_min(mn);
            float s, q0;
            if (symmetric) {
                const float amax = fmaxf(fabsf(mn), fabsf(mx));
                s = fmaf(2.0f / maxq, amax, kEps);
                q0 = 0.5f * (maxq + 1.0f);
            } else {
                s = __fadd_rn(__fdiv_rn(__fsub_rn(mx, mn), maxq), kEps);
                float q = rintf(__fdiv_rn(-mn, s));
                q0 = fminf(fmaxf(q, 0.0f), maxq);
            }
            sg = __shfl_sync(0xffffffffu, s, 0);
            q0g = __shfl_sync(0xffffffffu, q0, 0);
        } else {
            sg = scales[g];
            q0g = qzeros[g];
        }

        float best_s = sg, best_q = q0g;
        if (GS > 0 && P > 0) {
            float xmin = 0.0f;
            if (!symmetric) xmin = -__fmul_rn(sg, q0g);
            float best_loss = FLT_MAX;
            constexpr int UP = 4;
            for (int p0 = 0; p0 < P; p0 += UP) {
                float loss[UP], s_[UP], q0_[UP];
#pragma unroll
                for (int u = 0; u < UP; ++u) {
                    const int p = min(p0 + u, P - 1);
                    const float s = __fmul_rn(sg, cand[p]);
                    const float rcp = __fdiv_rn(1.0f, __fadd_rn(s, kEps));
                    float q0;
                    if (symmetric) q0 = q0g;
                    else q0 = fminf(fmaxf(rintf(__fmul_rn(-xmin, rcp)), 0.0f), maxq);
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < VPL; ++i) {
                        const float v = vals[i];
                        // clamp(rint(x), 0, maxq) == rint(clamp(x, 0, maxq)); in [0, 2^22) the
                        // round-half-even of rint is the rounding of an fp32 add of 1.5 * 2^23
                        float q = fminf(fmaxf(fmaf(v, rcp, q0), 0.0f), maxq);
                        q = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
                        const float diff = fmaf(__fsub_rn(q, q0), s, -v);
                        const float e = fmaxf(fabsf(diff), 1e-20f);
                        const float val = __expf(__fmul_rn(__logf(e), norm));
                        acc = __fadd_rn(acc, val);
                    }
                    loss[u] = acc;
                    s_[u] = s;
                    q0_[u] = q0;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int u = 0; u < UP; ++u) loss[u] = __fadd_rn(loss[u], __shfl_down_sync(0xffffffffu, loss[u], o));
                }
#pragma unroll
                for (int u = 0; u < UP; ++u) {
                    if (p0 + u < P && loss[u] < best_loss) {
                        best_loss = loss[u];
                        best_s = s_[u];
                        best_q = q0_[u];
                    }
                }
            }
        }
        if (lane == 0) {
            scales[g] = best_s;
            qzeros[g] = best_q;
        }
    }
}


// Min-max grid only (no shrink-factor search), bf16 weights, groups of 128 columns that tile the row exactly: the
// HBM-bound case of the layer path.  A lane reads four consecutive weights (8 bytes), so a warp reads a whole group in
// one 256-byte access, and four groups are in flight per warp.  min / max do not depend on the order of the elements,
// so the result is bit-identical to quant_grid_kernel's.
__global__ void __launch_bounds__(256)
minmax_grid_g128_bf16_kernel(const __nv_bfloat16 *__restrict__ W, int64_t n_groups, int bits, int symmetric,
                             float *__restrict__ scales, float *__restrict__ qzeros) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const float maxq = (float)((1 << bits) - 1);
    const uint2 *src = reinterpret_cast<const uint2 *>(W);
    for (int64_t g0 = warp_id * 4; g0 < n_groups; g0 += warps_total * 4) {
        uint2 raw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            raw[k] = (g0 + k < n_groups) ? src[(g0 + k) * 32 + lane] : make_uint2(0u, 0u);
        float mn[4], mx[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a = __uint_as_float(raw[k].x << 16), b = __uint_as_float(raw[k].x & 0xFFFF0000u);
            const float c = __uint_as_float(raw[k].y << 16), d = __uint_as_float(raw[k].y & 0xFFFF0000u);
            mx[k] = fmaxf(fmaxf(a, b), fmaxf(c, d));
            mn[k] = fminf(fminf(a, b), fminf(c, d));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
                mn[k] = fminf(mn[k], __shfl_xor_sync(0xffffffffu, mn[k], o));
            }
        }
        if (lane < 4 && g0 + lane < n_groups) {
            const float hi = lane == 0 ? mx[0] : lane == 1 ? mx[1] : lane == 2 ? mx[2] : mx[3];
            const float lo = lane == 0 ? mn[0] : lane == 1 ? mn[1] : lane == 2 ? mn[2] : mn[3];
            float s, q0;
            if (symmetric) {
                const float amax = fmaxf(fabsf(lo), fabsf(hi));
                s = fmaf(2.0f / maxq, amax, kEps);
                q0 = 0.5f * (maxq + 1.0f);
            } else {
                s = __fadd_rn(__fdiv_rn(__fsub_rn(hi, lo), maxq), kEps);
                const float q = rintf(__fdiv_rn(-lo, s));
                q0 = fminf(fmaxf(q, 0.0f), maxq);
            }
            scales[g0 + lane] = s;
            qzeros[g0 + lane] = q0;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Shrink-factor search, second layout: one THREAD per (group, candidate pair) instead of one warp per
// group.  The per-candidate set-up (scale, reciprocal, zero) is then paid once per 128 elements instead
// of once per 4, and no shuffle is needed: the thread reproduces the reference warp's summation order
// by itself — 32 "lane" partial sums, each the in-order sum of elements l, l+32, ..., then the
// shfl_down tree (offsets 16, 8, 4, 2, 1) over those 32 numbers.  The group's values sit in shared
// memory as [l][i] so that one broadcast LDS.128 feeds four elements of every thread of the group.
// The per-element arithmetic is the reference's (fma, round-half-even, clamp, fma, |.|^norm through
// lg2/ex2 approximations); the search is bound by the two MUFU operations per element-candidate.
// ------------------------------------------------------------------------------------------------
constexpr int kMseThreads = 256;
constexpr int kMseCPT = 2;        // candidates per thread
constexpr int kMseMaxGroups = 8;  // groups per CTA pass

__device__ __forceinline__ float fast_lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int GS, bool BF16, bool ABSMAX>
__global__ void __launch_bounds__(kMseThreads, 4)
mse_grid_kernel(const void *__restrict__ Wv, int64_t rows, int64_t C, int64_t G, int bits, int symmetric,
                const float *__restrict__ cand, int P, float norm, float *__restrict__ scales,
                float *__restrict__ qzeros, int tpg, int gpc) {
    constexpr int VPL = GS / 32;
    __shared__ __align__(16) float vals_s[kMseMaxGroups][32 * VPL];   // [group][l][i]
    __shared__ float meta_s[kMseMaxGroups][2];
    __shared__ float loss_s[kMseMaxGroups][kMseThreads];              // per candidate (P <= 256)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float maxq = (float)((1 << bits) - 1);
    const int64_t n_groups = rows * G;
    const float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer, ties to even

    for (int64_t g0 = (int64_t)blockIdx.x * gpc; g0 < n_groups; g0 += (int64_t)gridDim.x * gpc) {
        // ---- stage the values of this pass's groups, element e of a group at [e % 32][e / 32]
        for (int idx = tid; idx < gpc * GS; idx += kMseThreads) {
            const int gl = idx / GS, e = idx % GS;
            const int64_t g = g0 + gl;
            float x = 0.0f;
            if (g < n_groups) {
                const int64_t r = g / G, c = (g % G) * GS + e;
                if (c < C) {
                    x = BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(Wv)[r * C + c])
                             : reinterpret_cast<const float *>(Wv)[r * C + c];
                }
            }
            vals_s[gl][(e & 31) * VPL + (e >> 5)] = x;
        }
        __syncthreads();
        // ---- min-max scale / zero of each group (one warp per group)
        if (warp < gpc) {
            const int64_t g = g0 + warp;
            float sg = 1.0f, q0g = 0.0f;
            if (g < n_groups) {
                if (ABSMAX) {
                    float mn = 1e30f, mx = -1e30f;
#pragma unroll
                    for (int i = 0; i < VPL; ++i) {
                        const float x = vals_s[warp][lane * VPL + i];
                        mx = fmaxf(mx, x);
                        mn = fminf(mn, x);
                    }
                    mx = warp_max(mx);
                    mn = warp_min(mn);
                    if (symmetric) {
                        sg = fmaf(2.0f / maxq, fmaxf(fabsf(mn), fabsf(mx)), kEps);
                        q0g = 0.5f * (maxq + 1.0f);
                    } else {
                        sg = __fadd_rn(__fdiv_rn(__fsub_rn(mx, mn), maxq), kEps);
                        q0g = fminf(fmaxf(rintf(__fdiv_rn(-mn, sg)), 0.0f), maxq);
                    }
                } else {
                    sg = scales[g];
                    q0g = qzeros[g];
                }
            }
            if (lane == 0) { meta_s[warp][0] = sg; meta_s[warp][1] = q0g; }
        }
        __syncthreads();
        // ---- one thread per (group, candidate pair)
        const int gl = tid / tpg, jt = tid % tpg;
        if (gl < gpc && g0 + gl < n_groups) {
            const float sg = meta_s[gl][0], q0g = meta_s[gl][1];
            const float xmin = symmetric ? 0.0f : -__fmul_rn(sg, q0g);
            float sc[kMseCPT], rcp[kMseCPT], q0[kMseCPT], hiq[kMseCPT], offq[kMseCPT];
#pragma unroll
            for (int c = 0; c < kMseCPT; ++c) {
                const int p = min(jt + c * tpg, P - 1);
                sc[c] = __fmul_rn(sg, cand[p]);
                rcp[c] = __fdiv_rn(1.0f, __fadd_rn(sc[c], kEps));
                q0[c] = symmetric ? q0g : fminf(fmaxf(rintf(__fmul_rn(-xmin, rcp[c])), 0.0f), maxq);
                hiq[c] = kMagic + maxq;       // clamp bounds and zero in the "magic" domain (all exact integers)
                offq[c] = kMagic + q0[c];
            }
            // The reference reduces the 32 lane sums with a shfl_down tree (offsets 16, 8, 4, 2, 1): node(l) at
            // offset o is node(l) + node(l + o).  Visiting the lanes in bit-reversed order (0, 16, 8, 24, 4, ...)
            // makes every tree node the sum of two ADJACENT finished subtrees, so a 6-entry stack (one entry per
            // pending subtree, as in a binary counter) reproduces the tree exactly with 6 live registers per
            // candidate instead of 32.
            float st[kMseCPT][6];
            const float4 *v4 = reinterpret_cast<const float4 *>(&vals_s[gl][0]);
#pragma unroll
            for (int idx = 0; idx < 32; ++idx) {
                const int l = ((idx & 1) << 4) | ((idx & 2) << 2) | (idx & 4) | ((idx & 8) >> 2) | ((idx & 16) >> 4);
                float v[4];
                if (VPL == 4) {
                    const float4 t = v4[l];
                    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
                } else {
#pragma unroll
                    for (int i = 0; i < VPL; ++i) v[i] = vals_s[gl][l * VPL + i];
                }
                const int pc = __builtin_popcount(idx);   // pending subtrees before this leaf
                int merges = 0;                            // trailing one bits of idx
#pragma unroll
                for (int bbit = 0; bbit < 5; ++bbit) {
                    if (((idx >> bbit) & 1) == 0) break;
                    ++merges;
                }
#pragma unroll
                for (int c = 0; c < kMseCPT; ++c) {
                    float acc = 0.0f;
#pragma unroll
                    for (int i = 0; i < VPL; ++i) {
                        // q = clamp(rint(v*rcp + q0), 0, maxq), carried as q + magic
                        float t = __fadd_rn(fmaf(v[i], rcp[c], q0[c]), kMagic);
                        t = fminf(fmaxf(t, kMagic), hiq[c]);
                        const float diff = fmaf(__fsub_rn(t, offq[c]), sc[c], -v[i]);
                        const float e = fmaxf(fabsf(diff), 1e-20f);
                        const float lg = __fmul_rn(fast_lg2(e), 0.693147182f);                  // __logf
                        const float val = fast_ex2(__fmul_rn(__fmul_rn(lg, norm), 1.44269502f));  // __expf
                        acc = __fadd_rn(acc, val);
                    }
                    st[c][pc] = acc;
#pragma unroll
                    for (int m = 0; m < 5; ++m) {
                        if (m < merges) st[c][pc - 1 - m] = __fadd_rn(st[c][pc - 1 - m], st[c][pc - m]);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < kMseCPT; ++c) {
                const int p = jt + c * tpg;
                if (p < P) loss_s[gl][p] = st[c][0];
            }
        }
        __syncthreads();
        // ---- first strictly smaller loss in candidate order wins == lexicographic minimum of (loss, candidate)
        if (warp < gpc && g0 + warp < n_groups) {
            float best = FLT_MAX;
            int bp = 0x7fffffff;
            for (int p = lane; p < P; p += 32) {
                const float l = loss_s[warp][p];
                if (l < best) { best = l; bp = p; }   // ascending p inside a lane: earlier candidate kept on ties
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int op = __shfl_xor_sync(0xffffffffu, bp, o);
                if (ob < best || (ob == best && op < bp)) { best = ob; bp = op; }
            }
            if (lane == 0) {
                const float sg = meta_s[warp][0], q0g = meta_s[warp][1];
                float bs = sg, bq = q0g;
                if (best < FLT_MAX && bp < P) {
                    bs = __fmul_rn(sg, cand[bp]);
                    if (!symmetric) {
                        const float xmin = -__fmul_rn(sg, q0g);
                        const float rc = __fdiv_rn(1.0f, __fadd_rn(bs, kEps));
                        bq = fminf(fmaxf(rintf(__fmul_rn(-xmin, rc)), 0.0f), maxq);
                    }
                }
                scales[g0 + warp] = bs;
                qzeros[g0 + warp] = bq;
            }
        }
        __syncthreads();
    }
}

// ---- the same search with exact pruning -------------------------------------------------------------------
// The loss of a candidate is a sum of positive terms, so a candidate whose PARTIAL sum already exceeds the loss of
// some fully evaluated candidate can never be the first strictly smaller one and is abandoned.  Nothing about the
// result changes: the candidates that finish are summed in exactly the order described above, and an abandoned one
// is strictly worse than a finished one (the comparison carries a 1e-4 relative margin, three orders of magnitude
// above the rounding difference between two summation orders of 128 positive fp32 terms).  What changes is the
// work: with min-max scales the best shrink factor is close to 1 for most groups, and most of the 100 candidates
// are dropped after two elements (the extremes of the group) or after their first 16.
//
// Mapping: a CTA pass takes 32 consecutive groups; lane = group, so the 32 lanes of a warp evaluate the SAME
// candidate on 32 groups and leave the loop at about the same time.  Warps draw candidates from a shared counter in
// ascending order (shrink factor 1.0 first: the likely winners finish early and tighten the bound).  The bound
// of a group starts from the loss of candidate 0 (evaluated cooperatively by the eight warps, in any order, it is
// only a bound) and is lowered with atomicMin by every candidate that finishes; a stale read is merely
// conservative.
constexpr int kPrThreads = 256;
constexpr int kPrMaxP = 128;
constexpr int kPrPitch = 33;          // row pitch (in groups) of the staged values and of the loss table
constexpr float kPrMargin = 1.0001f;

template <bool BF16, bool ABSMAX>
__global__ void __launch_bounds__(kPrThreads, 4)
mse_prune_kernel(const void *__restrict__ Wv, int64_t rows, int64_t C, int64_t G, int bits, int symmetric,
                 const float *__restrict__ cand, int P, float norm, float *__restrict__ scales,
                 float *__restrict__ qzeros) {
    constexpr int GS = 128;
    __shared__ __align__(16) float4 vals_s[32 * kPrPitch];   // [chunk l][group] = elements l, l+32, l+64, l+96
    __shared__ float loss_s[kPrMaxP * kPrPitch];             // [candidate][group]
    __shared__ float part_s[8][2][32];
    __shared__ float meta_s[4][32];                          // scale, zero, smallest and largest value
    __shared__ int bound_s[32];                              // positive floats order like their bit patterns
    __shared__ int next_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float maxq = (float)((1 << bits) - 1);
    const int64_t n_groups = rows * G;
    const float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer, ties to even
    const unsigned full = 0xffffffffu;

    for (int64_t g0 = (int64_t)blockIdx.x * 32; g0 < n_groups; g0 += (int64_t)gridDim.x * 32) {
        // ---- stage 32 groups
        for (int idx = tid; idx < 32 * GS; idx += kPrThreads) {
            const int gl = idx / GS, e = idx % GS;
            const int64_t g = g0 + gl;
            float x = 0.0f;
            if (g < n_groups) {
                const int64_t r = g / G, c = (g % G) * GS + e;
                if (c < C) {
                    x = BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(Wv)[r * C + c])
                             : reinterpret_cast<const float *>(Wv)[r * C + c];
                }
            }
            reinterpret_cast<float *>(vals_s)[((e & 31) * kPrPitch + gl) * 4 + (e >> 5)] = x;
        }
        if (tid == 0) next_s = 0;
        __syncthreads();
        const bool valid = (g0 + lane) < n_groups;
        // ---- extremes of each group (order-free), and from them the min-max scale / zero
        {
            float mn = 1e30f, mx = -1e30f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 t = vals_s[(4 * warp + k) * kPrPitch + lane];
                mx = fmaxf(fmaxf(fmaxf(mx, t.x), fmaxf(t.y, t.z)), t.w);
                mn = fminf(fminf(fminf(mn, t.x), fminf(t.y, t.z)), t.w);
            }
            part_s[warp][0][lane] = mn;
            part_s[warp][1][lane] = mx;
            __syncthreads();
            if (warp == 0) {
                mn = part_s[0][0][lane];
                mx = part_s[0][1][lane];
#pragma unroll
                for (int w = 1; w < 8; ++w) {
                    mn = fminf(mn, part_s[w][0][lane]);
                    mx = fmaxf(mx, part_s[w][1][lane]);
                }
                float sg, q0g;
                if (!ABSMAX) {
                    sg = valid ? scales[g0 + lane] : 1.0f;
                    q0g = valid ? qzeros[g0 + lane] : 0.0f;
                } else if (symmetric) {
                    sg = fmaf(2.0f / maxq, fmaxf(fabsf(mn), fabsf(mx)), kEps);
                    q0g = 0.5f * (maxq + 1.0f);
                } else {
                    sg = __fadd_rn(__fdiv_rn(__fsub_rn(mx, mn), maxq), kEps);
                    q0g = fminf(fmaxf(rintf(__fdiv_rn(-mn, sg)), 0.0f), maxq);
                }
                meta_s[0][lane] = sg;
                meta_s[1][lane] = q0g;
                meta_s[2][lane] = mn;
                meta_s[3][lane] = mx;
            }
        }
        __syncthreads();
        const float vmin = meta_s[2][lane], vmax = meta_s[3][lane];
        const float sg = meta_s[0][lane], q0g = meta_s[1][lane];
        const float xmin = symmetric ? 0.0f : -__fmul_rn(sg, q0g);
        const float hiq = kMagic + maxq;
        auto element_loss = [&](float v, float sc, float rcp, float q0, float offq) {
            // q = clamp(rint(v*rcp + q0), 0, maxq), carried as q + magic
            float t = __fadd_rn(fmaf(v, rcp, q0), kMagic);
            t = fminf(fmaxf(t, kMagic), hiq);
            const float diff = fmaf(__fsub_rn(t, offq), sc, -v);
            const float e = fmaxf(fabsf(diff), 1e-20f);
            const float lg = __fmul_rn(fast_lg2(e), 0.693147182f);                  // __logf
            return fast_ex2(__fmul_rn(__fmul_rn(lg, norm), 1.44269502f));           // __expf
        };
        // ---- starting bound: candidate 0, sixteen elements per warp
        {
            const float sc = __fmul_rn(sg, cand[0]);
            const float rcp = __fdiv_rn(1.0f, __fadd_rn(sc, kEps));
            const float q0 = symmetric ? q0g : fminf(fmaxf(rintf(__fmul_rn(-xmin, rcp)), 0.0f), maxq);
            const float offq = kMagic + q0;
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 t = vals_s[(4 * warp + k) * kPrPitch + lane];
                acc += element_loss(t.x, sc, rcp, q0, offq) + element_loss(t.y, sc, rcp, q0, offq) +
                       element_loss(t.z, sc, rcp, q0, offq) + element_loss(t.w, sc, rcp, q0, offq);
            }
            part_s[warp][0][lane] = acc;
            __syncthreads();
            if (warp == 0) {
                float b = part_s[0][0][lane];
#pragma unroll
                for (int w = 1; w < 8; ++w) b += part_s[w][0][lane];
                bound_s[lane] = __float_as_int(b * kPrMargin);
            }
            __syncthreads();
        }
        // ---- candidates, drawn in ascending order
        while (true) {
            int p = 0;
            if (lane == 0) p = atomicAdd(&next_s, 1);
            p = __shfl_sync(full, p, 0);
            if (p >= P) break;
            const float sc = __fmul_rn(sg, cand[p]);
            const float rcp = __fdiv_rn(1.0f, __fadd_rn(sc, kEps));
            const float q0 = symmetric ? q0g : fminf(fmaxf(rintf(__fmul_rn(-xmin, rcp)), 0.0f), maxq);
            const float offq = kMagic + q0;
            // bit-reversed visit order + 6-entry stack = the reference's shfl_down tree (see mse_grid_kernel)
            float st[6];
            // the smallest and the largest value are two of the 128 terms (any two, if all values are equal), and
            // under a shrunk scale they are the clipped ones: most candidates are dropped right here
            const float two = element_loss(vmin, sc, rcp, q0, offq) + element_loss(vmax, sc, rcp, q0, offq);
            bool alive = valid && !(two > __int_as_float(*reinterpret_cast<volatile int *>(&bound_s[lane])));
            if (!__any_sync(full, alive)) {
                loss_s[p * kPrPitch + lane] = FLT_MAX;
                continue;
            }
#pragma unroll
            for (int idx = 0; idx < 32; ++idx) {
                const int l = ((idx & 1) << 4) | ((idx & 2) << 2) | (idx & 4) | ((idx & 8) >> 2) | ((idx & 16) >> 4);
                const float4 t = vals_s[l * kPrPitch + lane];
                float acc = element_loss(t.x, sc, rcp, q0, offq);
                acc = __fadd_rn(acc, element_loss(t.y, sc, rcp, q0, offq));
                acc = __fadd_rn(acc, element_loss(t.z, sc, rcp, q0, offq));
                acc = __fadd_rn(acc, element_loss(t.w, sc, rcp, q0, offq));
                const int pc = __builtin_popcount(idx);
                st[pc] = acc;
#pragma unroll
                for (int m = 0; m < 5; ++m) {
                    if (((idx >> m) & 1) == 0) break;
                    st[pc - 1 - m] = __fadd_rn(st[pc - 1 - m], st[pc - m]);
                }
                if ((idx & 3) == 3 && idx != 31) {
                    float partial = st[0];
#pragma unroll
                    for (int k = 1; k < 6; ++k)
                        if (k < __builtin_popcount(idx + 1)) partial += st[k];
                    const float bnd = __int_as_float(*reinterpret_cast<volatile int *>(&bound_s[lane]));
                    alive = alive && !(partial > bnd);
                    if (!__any_sync(full, alive)) break;
                }
            }
            loss_s[p * kPrPitch + lane] = alive ? st[0] : FLT_MAX;
            if (alive) atomicMin(&bound_s[lane], __float_as_int(st[0] * kPrMargin));
        }
        __syncthreads();
        // ---- first strictly smaller loss in candidate order wins == lexicographic minimum of (loss, candidate)
#pragma unroll 1
        for (int k = 0; k < 4; ++k) {
            const int gl = 4 * warp + k;
            if (g0 + gl >= n_groups) break;
            float best = FLT_MAX;
            int bp = 0x7fffffff;
            for (int p = lane; p < P; p += 32) {
                const float l = loss_s[p * kPrPitch + gl];
                if (l < best) { best = l; bp = p; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(full, best, o);
                const int op = __shfl_xor_sync(full, bp, o);
                if (ob < best || (ob == best && op < bp)) { best = ob; bp = op; }
            }
            if (lane == 0) {
                const float sgl = meta_s[0][gl], q0l = meta_s[1][gl];
                float bs = sgl, bq = q0l;
                if (best < FLT_MAX && bp < P) {
                    bs = __fmul_rn(sgl, cand[bp]);
                    if (!symmetric) {
                        const float xm = -__fmul_rn(sgl, q0l);
                        const float rc = __fdiv_rn(1.0f, __fadd_rn(bs, kEps));
                        bq = fminf(fmaxf(rintf(__fmul_rn(-xm, rc)), 0.0f), maxq);
                    }
                }
                scales[g0 + gl] = bs;
                qzeros[g0 + gl] = bq;
            }
        }
        __syncthreads();
    }
}

template <bool ABSMAX>
int launch_grid(const void *W, int w_dtype, int64_t rows, int64_t C, int gs, int bits, int symmetric,
                const float *cand, int n_cand, float norm, float *scales, float *qzeros, cudaStream_t st) {
    const int64_t G = cdiv(C, gs);
    const int64_t n_groups = rows * G;
    const char *impl = getenv("FORGE_GRID_IMPL");
    const bool exhaustive = impl && strcmp(impl, "exhaustive") == 0;   // cross-checks: evaluate every candidate fully
    if (n_cand > 0 && n_cand <= kPrMaxP && gs == 128 && !exhaustive) {
        // two passes per CTA: short-lived CTAs, so that kernels of a higher-priority stream (the factorisation that the
        // layer driver runs beside the search) find free slots every few tens of microseconds
        const int blocks = (int)imin64(cdiv(n_groups, 64), 1 << 30);
        if (w_dtype == FORGE_DTYPE_BF16) {
            mse_prune_kernel<true, ABSMAX><<<blocks, kPrThreads, 0, st>>>(W, rows, C, G, bits, symmetric, cand, n_cand,
                                                                         norm, scales, qzeros);
        } else {
            mse_prune_kernel<false, ABSMAX><<<blocks, kPrThreads, 0, st>>>(W, rows, C, G, bits, symmetric, cand, n_cand,
                                                                          norm, scales, qzeros);
        }
        FORGE_NOTE_LAUNCH();
        return check_launch("forge_quant_grid(mse, pruned)");
    }
    if (n_cand > 0 && n_cand <= kMseThreads && (gs == 32 || gs == 64 || gs == 128)) {
        const int tpg = (n_cand + kMseCPT - 1) / kMseCPT;                 // threads per group
        int gpc = kMseThreads / tpg;                                       // groups per CTA pass
        if (gpc > kMseMaxGroups) gpc = kMseMaxGroups;
        const int blocks = (int)imin64(cdiv(n_groups, gpc), 148 * 2 * 8);
        const bool bf = (w_dtype == FORGE_DTYPE_BF16);
#define FORGE_LAUNCH_MSE(GSV)                                                                                  \
        do {                                                                                                   \
            if (bf) { mse_grid_kernel<GSV, true, ABSMAX><<<blocks, kMseThreads, 0, st>>>(                      \
                        W, rows, C, G, bits, symmetric, cand, n_cand, norm, scales, qzeros, tpg, gpc); FORGE_NOTE_LAUNCH(); } \
            else { mse_grid_kernel<GSV, false, ABSMAX><<<blocks, kMseThreads, 0, st>>>(                        \
                        W, rows, C, G, bits, symmetric, cand, n_cand, norm, scales, qzeros, tpg, gpc); FORGE_NOTE_LAUNCH(); } \
        } while (0)
        if (gs == 32) FORGE_LAUNCH_MSE(32);
        else if (gs == 64) FORGE_LAUNCH_MSE(64);
        else FORGE_LAUNCH_MSE(128);
#undef FORGE_LAUNCH_MSE
        return check_launch("forge_quant_grid(mse)");
    }
    const int threads = 256;  // 8 groups per CTA pass
    const int64_t want = cdiv(n_groups, threads / 32);
    const int blocks = (int)imin64(want, 148 * 8);
    const bool bf = (w_dtype == FORGE_DTYPE_BF16);
#define FORGE_LAUNCH_GRID(GSV)                                                                               \
    do {                                                                                                     \
        if (bf) { quant_grid_kernel<GSV, true, ABSMAX><<<blocks, threads, 0, st>>>(                            \
                    W, rows, C, G, gs, bits, symmetric, cand, n_cand, norm, scales, qzeros); FORGE_NOTE_LAUNCH(); } else { quant_grid_kernel<GSV, false, ABSMAX><<<blocks, threads, 0, st>>>(                              \
                    W, rows, C, G, gs, bits, symmetric, cand, n_cand, norm, scales, qzeros); FORGE_NOTE_LAUNCH(); }                 \
    } while (0)
    switch (gs) {
        case 32: FORGE_LAUNCH_GRID(32); break;
        case 64: FORGE_LAUNCH_GRID(64); break;
        case 128: FORGE_LAUNCH_GRID(128); break;
        default:
            if (n_cand > 0 || !ABSMAX) {
                set_error("Unsupported group_size=%d (expected 32/64/128)", gs);
                return FORGE_ERR_UNSUPPORTED;
            }
            FORGE_LAUNCH_GRID(0);
    }
#undef FORGE_LAUNCH_GRID
    return check_launch("forge_quant_grid");
}

}  // namespace

extern "C" int forge_quant_grid(const void *W, int w_dtype, int64_t rows, int64_t C, int gs, int bits,
                                int symmetric, const float *candidates, int n_cand, float norm, float *scales,
                                float *qzeros, void *stream) {
    FORGE_REQUIRE(W && scales && qzeros, "null pointer");
    FORGE_REQUIRE(rows > 0 && C > 0 && gs > 0 && bits >= 1 && bits <= 8, "bad sizes");
    FORGE_REQUIRE(n_cand == 0 || candidates, "candidates missing");
    FORGE_REQUIRE(w_dtype == FORGE_DTYPE_F32 || w_dtype == FORGE_DTYPE_BF16, "bad dtype");
    if (n_cand == 0 && gs == 128 && C % 128 == 0 && w_dtype == FORGE_DTYPE_BF16 && (uintptr_t)W % 8 == 0) {
        const int64_t n_groups = rows * (C / 128);
        const int blocks = (int)imin64(cdiv(n_groups, 8 * 4), 148 * 16);
        minmax_grid_g128_bf16_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)W, n_groups, bits,
                                                                               symmetric, scales, qzeros);
        FORGE_NOTE_LAUNCH();
        return check_launch("forge_quant_grid");
    }
    return launch_grid<true>(W, w_dtype, rows, C, gs, bits, symmetric, candidates, n_cand, norm, scales, qzeros,
                             (cudaStream_t)stream);
}

extern "C" int forge_quant_grid_mse(const void *W, int w_dtype, int64_t rows, int64_t C, int gs, int bits,
                                    int symmetric, const float *candidates, int n_cand, float norm,
                                    float *scales, float *qzeros, void *stream) {
    FORGE_REQUIRE(W && scales && qzeros && candidates, "null pointer");
    FORGE_REQUIRE(rows > 0 && C > 0 && gs > 0 && n_cand > 0 && bits >= 1 && bits <= 8, "bad sizes");
    FORGE_REQUIRE(w_dtype == FORGE_DTYPE_F32 || w_dtype == FORGE_DTYPE_BF16, "bad dtype");
    return launch_grid<false>(W, w_dtype, rows, C, gs, bits, symmetric, candidates, n_cand, norm, scales,
                              qzeros, (cudaStream_t)stream);
}
