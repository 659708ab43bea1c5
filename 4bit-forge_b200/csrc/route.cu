// Router top-k on the device: router logits [T, E] -> chosen expert ids [T, k] (and their scores).
//
// The reference never computes this itself: the HF MoE block does it in its own forward before the
// expert hooks fire (quant.py:398-406), and the fused-experts capture re-creates the selection from
// `router_indices` (forge/utils/engine.py:228-238).  A layer-level driver that owns the whole step has
// to do it, so it is a kernel here: one warp per token, the E scores of a token spread over the 32
// lanes, "extract the maximum k times" with warp shuffles.  Two selection rules:
//   plain         : top-k over the scores (softmax is monotone, so the order of the logits is used);
//   group-limited : DeepSeek-V3 style — scores = sigmoid(logit) (+ selection bias), the experts are
//                   split into n_groups equal groups, a group's score is the sum of its two best
//                   experts, only the topk_groups best groups stay eligible, then top-k over those.
// Ties go to the lower expert index.  Ids come out in descending score order.
#include "common.cuh"

using namespace forge;

namespace {

constexpr int kMaxPerLane = 32;   // E <= 1024

struct Best {
    float v;
    int idx;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.v > a.v || (b.v == a.v && b.idx < a.idx)) ? b : a;
}
__device__ __forceinline__ Best warp_argmax(Best x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.idx = __shfl_xor_sync(0xffffffffu, x.idx, o);
        x = better(x, y);
    }
    return x;
}

// mode 0: softmax scores, plain top-k; mode 1: sigmoid scores, plain top-k; mode 2: sigmoid, group-limited.
// kPerLane = experts per lane this instance is compiled for (E <= 32 kPerLane): every scan over a token's scores is
// unrolled to exactly that length.
template <int kPerLane>
__global__ void route_topk_kernel(const float *__restrict__ logits, const float *__restrict__ bias, int64_t T, int E,
                                  int k, int mode, int n_groups, int topk_groups, int32_t *__restrict__ ids,
                                  float *__restrict__ weights) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const int npl = (E + 31) / 32;
    const float NEG = -3.0e38f;
    float sel[kPerLane];   // what the selection compares
    float raw[kPerLane];   // what is reported as the weight
    float mx = NEG;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        sel[j] = NEG;
        raw[j] = 0.0f;
        if (j < npl) {
            const int e = j * 32 + lane;
            if (e < E) {
                const float x = logits[t * E + e];
                if (mode == 0) {
                    raw[j] = x;
                    sel[j] = x;
                    mx = fmaxf(mx, x);
                } else {
                    const float s = 1.0f / (1.0f + expf(-x));
                    raw[j] = s;
                    sel[j] = bias ? s + bias[e] : s;
                }
            }
        }
    }
    float denom = 1.0f;
    if (mode == 0 && weights) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j)
            if (j < npl && j * 32 + lane < E) sum += expf(raw[j] - mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        denom = sum;
    }
    if (mode == 2) {
        // group scores: sum of the two best selection scores of each group
        const int gsz = E / n_groups;
        float gscore = NEG;   // lane g (< n_groups) keeps the score of group g
        for (int g = 0; g < n_groups; ++g) {
            float acc = 0.0f;
            int taken = -1;
            for (int rep = 0; rep < 2; ++rep) {
                Best b{NEG, 0x7fffffff};
#pragma unroll
                for (int j = 0; j < kPerLane; ++j) {
                    if (j < npl) {
                        const int e = j * 32 + lane;
                        if (e < E && e / gsz == g && e != taken) b = better(b, Best{sel[j], e});
                    }
                }
                b = warp_argmax(b);
                taken = b.idx;
                if (b.v > NEG) acc += b.v;
            }
            if (lane == g) gscore = acc;
        }
        // keep the topk_groups best groups (n_groups <= 32: one group per lane)
        unsigned keep = 0u;
        for (int rep = 0; rep < topk_groups; ++rep) {
            const bool cand = lane < n_groups && !((keep >> lane) & 1u);
            Best b{cand ? gscore : NEG, cand ? lane : 0x7fffffff};
            b = warp_argmax(b);
            if (b.idx < n_groups) keep |= 1u << b.idx;
        }
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            if (j < npl) {
                const int e = j * 32 + lane;
                if (e < E && !((keep >> (e / gsz)) & 1u)) sel[j] = NEG;
            }
        }
    }
    for (int r = 0; r < k; ++r) {
        Best b{NEG, 0x7fffffff};
        float w = 0.0f;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            if (j < npl) {
                const int e = j * 32 + lane;
                if (e < E) {
                    const Best c{sel[j], e};
                    const Best nb = better(b, c);
                    if (nb.idx != b.idx) w = raw[j];
                    b = nb;
                }
            }
        }
        const Best win = warp_argmax(b);
        if (win.idx == b.idx && b.idx < E) {   // exactly one lane owns the winner
            ids[t * k + r] = win.idx;
            if (weights) weights[t * k + r] = (mode == 0) ? expf(w - mx) / denom : w;
        }
#pragma unroll
        for (int j = 0; j < kPerLane; ++j)
            if (j < npl && j * 32 + lane == win.idx) sel[j] = NEG;
    }
}

}  // namespace

extern "C" int forge_route_topk(const float *logits, const float *bias, int64_t T, int E, int k, int mode, int n_groups,
                                int topk_groups, int32_t *topk_ids, float *topk_weights, void *stream) {
    FORGE_REQUIRE(logits && topk_ids, "null pointer");
    FORGE_REQUIRE(T >= 0 && E > 0 && E <= 32 * kMaxPerLane && k > 0 && k <= E, "bad sizes (E <= 1024, k <= E)");
    FORGE_REQUIRE(mode >= 0 && mode <= 2, "mode must be 0 (softmax), 1 (sigmoid) or 2 (sigmoid, group-limited)");
    if (mode == 2) {
        FORGE_REQUIRE(n_groups > 0 && n_groups <= 32 && E % n_groups == 0, "n_groups must divide E and be <= 32");
        FORGE_REQUIRE(topk_groups > 0 && topk_groups <= n_groups, "topk_groups must be in [1, n_groups]");
        FORGE_REQUIRE((int64_t)topk_groups * (E / n_groups) >= k, "the kept groups hold fewer than k experts");
    }
    if (T == 0) return FORGE_OK;
    const int warps = 8;
    const dim3 grid((unsigned)cdiv(T, warps)), block(warps * 32);
    cudaStream_t st = (cudaStream_t)stream;
    const int npl = (E + 31) / 32;
#define FORGE_ROUTE_LAUNCH(N) \
    route_topk_kernel<N><<<grid, block, 0, st>>>(logits, bias, T, E, k, mode, n_groups, topk_groups, topk_ids, topk_weights)
    if (npl <= 1) FORGE_ROUTE_LAUNCH(1);
    else if (npl <= 2) FORGE_ROUTE_LAUNCH(2);
    else if (npl <= 4) FORGE_ROUTE_LAUNCH(4);
    else if (npl <= 8) FORGE_ROUTE_LAUNCH(8);
    else if (npl <= 16) FORGE_ROUTE_LAUNCH(16);
    else FORGE_ROUTE_LAUNCH(32);
#undef FORGE_ROUTE_LAUNCH
    FORGE_NOTE_LAUNCH();
    return check_launch("forge_route_topk");
}
