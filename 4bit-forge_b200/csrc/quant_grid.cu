// Per-group scale / zero grid: min-max, and the L^p shrink-factor search.
//
// One warp per group, lane l holding elements l, l+32, ... exactly as the reference kernels do
// (forge/backend/cuda/quant_grid.cu:42-183), because the candidate that wins the search depends on the
// order in which the per-element errors are summed: lane-local sum first, then a shfl_down tree.  What
// changes is the data path: the weights are read once, in their storage type (bf16, 2 B/element,
// instead of an fp32 copy), the min-max pass and the search share the registers, the search is
// unrolled over candidates so that several reduction trees are in flight per warp, and the grid is a
// multiple of the SM count.  The search is bound by FP32/MUFU issue (two transcendental ops per
// element-candidate), not by HBM.
#include "common.cuh"
#include <float.h>

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

template <bool ABSMAX>
int launch_grid(const void *W, int w_dtype, int64_t rows, int64_t C, int gs, int bits, int symmetric,
                const float *cand, int n_cand, float norm, float *scales, float *qzeros, cudaStream_t st) {
    const int64_t G = cdiv(C, gs);
    const int64_t n_groups = rows * G;
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
