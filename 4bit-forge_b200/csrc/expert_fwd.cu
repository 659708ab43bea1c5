// Expert forward that produces the down-projection calibration input of every local expert,
//   act[off_b + j, :] = bf16( bf16(silu(bf16(x Wg_b^T))) * bf16(x Wu_b^T) ),   x = X[token_idx[off_b + j]],
// as ONE grouped tcgen05 / TMEM GEMM launch with the routing gather fused into the operand load and
// the SwiGLU in the epilogue.  The reference gets these activations from the HF block forward, one
// expert module at a time, and hooks them at down_proj (quant.py:398-406; the fused-experts form is
// forge/utils/engine.py:228-258).
//
// Shapes per expert b: [n_b x H] * [H x 2I] with M = routed tokens (gathered rows of X), N = gate and
// up channels, K = H.  Both operands are K-major (H is the contiguous axis of X and of the weights): a
// k-tile is 64 channels = 128 bytes per row, stored with the 128-byte swizzle.  A CTA tile is 128
// tokens x (128 gate + 128 up) channels: the 128 gate rows and the 128 up rows of the weight k-tile
// sit back to back in shared memory and form ONE N = 256 operand, so a k-step is a single
// M128 x N256 x K16 MMA whose accumulator columns [0,128) are the gate and [128,256) the up
// projection of the same tokens and channels.  Two accumulators (all 512 TMEM columns) alternate, so
// the epilogue of one tile overlaps the main loop of the next.
//
// Warp roles (288 threads): warps 0-3 load (16-byte cp.async, 4-stage ring), warps 4-7 run the epilogue
// (tcgen05.ld, one TMEM lane = one token row per thread), warp 8 owns TMEM and issues the MMAs.
// Persistent CTAs walk the tile list (slot, token tile, channel tile) derived from the device-side
// offsets.  Every mbarrier wait is bounded; offsets and token indices are bounds-checked (status word).
#include "common.cuh"
#include "tcgen05.cuh"

using namespace forge;
using namespace forge::tc;

namespace {

constexpr int kMT = 128;                      // tokens per tile
constexpr int kNT = 128;                      // gate (and up) channels per tile
constexpr int kKT = 64;                       // hidden channels per k-tile (128 B of bf16)
constexpr int kABytes = kMT * 128;            // 16 KB
constexpr int kBBytes = 2 * kNT * 128;        // 32 KB: gate rows then up rows
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStages = 4;
constexpr int kLag = 2;
constexpr int kProducers = 128;
constexpr int kThreads = 288;
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 + 256;

struct FwdParams {
    const __nv_bfloat16 *X;
    int64_t n_rows, ldx, H, I;
    const int32_t *token_idx;
    int64_t list_len;
    const int64_t *offsets;
    int nb;
    const __nv_bfloat16 *Wg, *Wu;   // [nb][I][H]
    __nv_bfloat16 *out;             // [out_rows][I]
    int64_t out_rows;
    int32_t *status;
    int ntn;                        // channel tiles per expert
};

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1 KB apart (stride byte offset); the
// leading byte offset is not used by swizzled K-major layouts.
__device__ __forceinline__ uint64_t make_desc_kmajor(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// D fp32, A/B bf16, both K-major, M = 128, N = 256
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_bf16_kmajor(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// the activation exactly as the block forward rounds it: projections to bf16, silu to bf16, product to bf16
__device__ __forceinline__ __nv_bfloat16 swiglu_bf16(float acc_g, float acc_u) {
    const float g = bf16_round(acc_g), u = bf16_round(acc_u);
    const float s = bf16_round(g / (1.0f + expf(-g)));
    return __float2bfloat16_rn(s * u);
}

// Token tiles of a slot; 0 when the slot is empty or its claim does not fit the list / X / the output buffer.
__device__ __forceinline__ int64_t slot_token_tiles(const FwdParams &P, int b, int64_t &off, int64_t &n, bool &bad) {
    off = P.offsets[b];
    n = P.offsets[b + 1] - off;
    bad = !(off >= 0 && n >= 0 && off + n <= P.list_len && off + n <= P.out_rows);
    return (bad || n <= 0) ? 0 : (n + kMT - 1) / kMT;
}

__global__ void __launch_bounds__(kThreads, 1) expert_swiglu_tc_kernel(const FwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_al + kStages * kStageBytes);
    // bars[0..3] full, [4..7] empty, [8..9] acc_full, [10..11] acc_empty
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 12);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * kStages), bar_acc_empty = smem_u32(bars + 2 * kStages + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, kProducers);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full + 8 * a, 1);
            mbar_init(bar_acc_empty + 8 * a, 128);
        }
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

    const int64_t H = P.H, I = P.I;
    const int nkt = (int)((H + kKT - 1) / kKT);
    const int64_t grid = gridDim.x;
    uint32_t it = 0;          // k-tiles pushed through the ring (same sequence for producers and the MMA warp)
    uint32_t tile_iter = 0;   // tiles done by this CTA (same sequence for the MMA warp and the epilogue)

    if (warp < 4) {
        // ------------------------------ producers ------------------------------
        const int chunk = tid & 7;        // 16-byte chunk of the 128-byte row
        const int rbase = tid >> 3;       // rows rbase + 16 i
        int pend = 0;
        bool ok = true;
        int64_t base = 0;
        for (int b = 0; b < P.nb && ok; ++b) {
            int64_t off, n;
            bool bad;
            const int64_t mt = slot_token_tiles(P, b, off, n, bad);
            if (bad && tid == 0 && blockIdx.x == 0 && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
            const int64_t tb = mt * P.ntn;
            const int32_t *tl = P.token_idx ? P.token_idx + off : nullptr;
            const __nv_bfloat16 *Wgb = P.Wg + (int64_t)b * I * H, *Wub = P.Wu + (int64_t)b * I * H;
            for (int64_t t = ((int64_t)blockIdx.x - base % grid + grid) % grid; t < tb && ok; t += grid) {
                const int64_t m0 = (t / P.ntn) * kMT, n0 = (t % P.ntn) * kNT;
                const __nv_bfloat16 *arow[8];
                int64_t tokv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {     // all loads first, the checks after: eight latencies overlap
                    const int64_t kidx = m0 + rbase + 16 * i;
                    tokv[i] = (kidx < n) ? (tl ? (int64_t)tl[kidx] : off + kidx) : INT64_MIN;
                }
                bool bad_token = false;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool valid = tokv[i] >= 0 && tokv[i] < P.n_rows;   // else: not a row of X, contributes zeros
                    bad_token |= (!valid && tokv[i] != INT64_MIN);
                    arow[i] = valid ? P.X + tokv[i] * P.ldx + chunk * 8 : nullptr;
                }
                if (bad_token && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
                for (int kt = 0; kt < nkt && ok; ++kt) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                    if (!ok) break;
                    const uint32_t stage = smem_base + s * kStageBytes;
                    const int64_t k0 = (int64_t)kt * kKT;
                    const bool kin = (k0 + chunk * 8) < H;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = rbase + 16 * i;
                        const uint32_t dst = stage + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
                        const bool v = kin && arow[i] != nullptr;
                        cp_async16_zfill(dst, v ? (const void *)(arow[i] + k0) : (const void *)P.X, v);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int r = rbase + 16 * i;                      // 0..255: gate rows then up rows
                        const int64_t ch = n0 + (r & (kNT - 1));
                        const __nv_bfloat16 *wb = (r < kNT) ? Wgb : Wub;
                        const uint32_t dst = stage + kABytes +
                                             (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
                        const bool v = kin && ch < I;
                        cp_async16_zfill(dst, v ? (const void *)(wb + ch * H + k0 + chunk * 8) : (const void *)P.X, v);
                    }
                    cp_async_commit();
                    ++pend;
                    ++it;
                    if (pend > kLag) {
                        cp_async_wait<kLag>();
                        fence_proxy_async();
                        mbar_arrive(bar_full + 8 * ((it - pend) % kStages));
                        --pend;
                    }
                }
            }
            base += tb;
        }
        while (pend > 0) {  // publish the stages still in flight
            if (pend >= 2) cp_async_wait<1>();
            else cp_async_wait<0>();
            fence_proxy_async();
            mbar_arrive(bar_full + 8 * ((it - pend) % kStages));
            --pend;
        }
        cp_async_wait<0>();
    } else if (warp < 8) {
        // ------------------------------ epilogue ------------------------------
        const int q = warp - 4;            // TMEM lane quarter of this warp
        bool ok = true;
        int64_t base = 0;
        for (int b = 0; b < P.nb && ok; ++b) {
            int64_t off, n;
            bool bad;
            const int64_t mt = slot_token_tiles(P, b, off, n, bad);
            const int64_t tb = mt * P.ntn;
            for (int64_t t = ((int64_t)blockIdx.x - base % grid + grid) % grid; t < tb && ok; t += grid) {
                const int64_t m0 = (t / P.ntn) * kMT, n0 = (t % P.ntn) * kNT;
                const uint32_t buf = tile_iter & 1u;
                ok = mbar_wait(bar_acc_full + 8 * buf, (tile_iter >> 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-aligned: the whole warp goes or none
                if (!ok) break;
                tc_fence_after();
                const int64_t row = m0 + q * 32 + lane;
                __nv_bfloat16 *orow = P.out + (off + row) * I + n0;
                const bool vec_ok = (I % 8 == 0);
#pragma unroll 1
                for (int cc = 0; cc < kNT / 32; ++cc) {
                    if (n0 + cc * 32 >= I) break;   // warp-uniform
                    uint32_t vg[32], vu[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u + (uint32_t)(cc * 32);
                    tmem_ld32(taddr, vg);
                    tmem_ld32(taddr + 128u, vu);
                    tmem_ld_wait();
                    if (row < n) {
                        __align__(16) __nv_bfloat16 r[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = swiglu_bf16(__uint_as_float(vg[e]), __uint_as_float(vu[e]));
                        if (vec_ok && n0 + cc * 32 + 32 <= I) {
                            uint4 *dst = reinterpret_cast<uint4 *>(orow + cc * 32);
#pragma unroll
                            for (int v4 = 0; v4 < 4; ++v4) dst[v4] = reinterpret_cast<const uint4 *>(r)[v4];
                        } else {
#pragma unroll
                            for (int e = 0; e < 32; ++e)
                                if (n0 + cc * 32 + e < I) orow[cc * 32 + e] = r[e];
                        }
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_acc_empty + 8 * buf);
                ++tile_iter;
            }
            base += tb;
        }
    } else {
        // ------------------------------ MMA issuer (warp 8) ------------------------------
        bool ok = true;
        int64_t base = 0;
        for (int b = 0; b < P.nb && ok; ++b) {
            int64_t off, n;
            bool bad;
            const int64_t mt = slot_token_tiles(P, b, off, n, bad);
            const int64_t tb = mt * P.ntn;
            for (int64_t t = ((int64_t)blockIdx.x - base % grid + grid) % grid; t < tb && ok; t += grid) {
                const uint32_t buf = tile_iter & 1u;
                ok = mbar_wait(bar_acc_empty + 8 * buf, ((tile_iter >> 1) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                for (int kt = 0; kt < nkt && ok; ++kt) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t a_base = smem_base + s * kStageBytes;
                        const uint32_t b_base = a_base + kABytes;
#pragma unroll
                        for (int kk = 0; kk < kKT / 16; ++kk)
                            umma_bf16_kmajor(tmem_base + buf * 256u, make_desc_kmajor(a_base + kk * 32),
                                             make_desc_kmajor(b_base + kk * 32), (kt > 0 || kk > 0) ? 1u : 0u);
                        umma_commit(bar_empty + 8 * s);
                    }
                    __syncwarp();
                    ++it;
                }
                if (!ok) break;
                if (lane == 0) umma_commit(bar_acc_full + 8 * buf);
                __syncwarp();
                ++tile_iter;
            }
            base += tb;
        }
    }
    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0 && P.status) atomicExch(P.status, FORGE_ERR_TIMEOUT);
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Plain-FMA validation kernel with the same contract: one thread per output element.  Cross-checks the
// tensor-core kernel on the GPU itself (FORGE_FWD_SIMT); not on the product path otherwise.
__global__ void expert_swiglu_simt_kernel(const FwdParams P) {
    const int b = blockIdx.z;
    const int64_t off = P.offsets[b], n = P.offsets[b + 1] - off;
    if (!(off >= 0 && n >= 0 && off + n <= P.list_len && off + n <= P.out_rows)) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
        return;
    }
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P.I) return;
    const __nv_bfloat16 *wg = P.Wg + ((int64_t)b * P.I + i) * P.H, *wu = P.Wu + ((int64_t)b * P.I + i) * P.H;
    for (int64_t j = blockIdx.y; j < n; j += gridDim.y) {
        int64_t tok = P.token_idx ? (int64_t)P.token_idx[off + j] : off + j;
        if (tok < 0 || tok >= P.n_rows) {
            if (P.status) atomicExch(P.status, FORGE_ERR_INVALID);
            tok = -1;
        }
        float ag = 0.0f, au = 0.0f;
        if (tok >= 0) {
            const __nv_bfloat16 *x = P.X + tok * P.ldx;
            for (int64_t k = 0; k < P.H; ++k) {
                const float xv = __bfloat162float(x[k]);
                ag = fmaf(xv, __bfloat162float(wg[k]), ag);
                au = fmaf(xv, __bfloat162float(wu[k]), au);
            }
        }
        P.out[(off + j) * P.I + i] = swiglu_bf16(ag, au);
    }
}

}  // namespace

extern "C" int forge_expert_swiglu_grouped(const void *X_bf16, int64_t n_rows, int64_t ldx, int64_t H, int64_t I,
                                           const int32_t *token_idx, int64_t list_len, const int64_t *offsets, int nb,
                                           const void *Wg_bf16, const void *Wu_bf16, void *out_bf16, int64_t out_rows,
                                           int flags, int32_t *status, void *stream) {
    FORGE_REQUIRE(X_bf16 && offsets && Wg_bf16 && Wu_bf16 && out_bf16, "null pointer");
    FORGE_REQUIRE(nb > 0 && H > 0 && I > 0 && ldx >= H && out_rows >= 0, "bad sizes");
    FORGE_REQUIRE(n_rows >= 0 && n_rows <= 0x7fffffffLL, "n_rows must fit a 32-bit token index");
    FORGE_REQUIRE(!token_idx || list_len >= 0, "list_len must be >= 0");
    cudaStream_t st = (cudaStream_t)stream;
    FwdParams P{};
    P.X = (const __nv_bfloat16 *)X_bf16; P.n_rows = n_rows; P.ldx = ldx; P.H = H; P.I = I;
    P.token_idx = token_idx; P.list_len = token_idx ? list_len : n_rows; P.offsets = offsets; P.nb = nb;
    P.Wg = (const __nv_bfloat16 *)Wg_bf16; P.Wu = (const __nv_bfloat16 *)Wu_bf16;
    P.out = (__nv_bfloat16 *)out_bf16; P.out_rows = out_rows; P.status = status;
    P.ntn = (int)cdiv(I, kNT);
    if (flags & FORGE_FWD_SIMT) {
        dim3 grid((unsigned)cdiv(I, 128), 64, nb);
        expert_swiglu_simt_kernel<<<grid, 128, 0, st>>>(P); FORGE_NOTE_LAUNCH();
        return check_launch("forge_expert_swiglu_grouped(simt)");
    }
    FORGE_REQUIRE(H % 8 == 0 && ldx % 8 == 0, "H and ldx must be multiples of 8 (16-byte row chunks)");
    FORGE_REQUIRE((uintptr_t)X_bf16 % 16 == 0 && (uintptr_t)Wg_bf16 % 16 == 0 && (uintptr_t)Wu_bf16 % 16 == 0 &&
                      (uintptr_t)out_bf16 % 16 == 0,
                  "X, Wg, Wu and out must be 16-byte aligned");
    cudaError_t e = cudaFuncSetAttribute(expert_swiglu_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBytes);   // per-device attribute
    if (e != cudaSuccess) {
        set_error("forge_expert_swiglu_grouped: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        return FORGE_ERR_LAUNCH;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    expert_swiglu_tc_kernel<<<sms, kThreads, kSmemBytes, st>>>(P); FORGE_NOTE_LAUNCH();
    return check_launch("forge_expert_swiglu_grouped");
}
