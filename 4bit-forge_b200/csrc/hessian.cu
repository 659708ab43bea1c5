// Per-expert Hessian accumulation  H_b = beta_b * H_b + alpha_b * X_b^T X_b  as a grouped
// tcgen05 / TMEM GEMM with the routing gather fused into the operand load.
//
// Shapes: for expert b the GEMM is  [C x n_b] * [n_b x C]  with K = n_b = the tokens routed to b.
// Both operands are the SAME matrix X (bf16, [T, C] row-major, channels contiguous), read by token
// index, so both are "MN-major" for the tensor core: a K-tile of 64 tokens x 64 channels is 64
// rows of 128 bytes, stored with the 128-byte swizzle (16-byte chunk index XOR row-in-8) that the
// UMMA shared-memory descriptor expects.  The rows are fetched with 16-byte cp.async copies whose
// source row is token_idx[...] — that is the fused top-k gather: no permuted copy of X exists.
//
// One persistent CTA per SM.  A CTA tile is 256 x 256 outputs: two M=128 x N=256 x K=16 bf16 MMAs
// per k-step into two fp32 accumulators that fill the SM's 512 TMEM columns.  Per 64-token k-tile the
// CTA stages 256 + 256 channels (64 KB; 32 KB on diagonal tiles where both operands coincide), i.e.
// 128 flop per staged byte.  Only tiles on or above the diagonal are computed; the epilogue scales
// by alpha/beta and optionally mirrors into the lower triangle.
//
// Warp roles (160 threads): warps 0-3 load (cp.async, 3-stage ring, completion published to the
// async proxy by fence.proxy.async + mbarrier arrive) and later run the epilogue (tcgen05.ld, one
// TMEM lane = one output row per thread); warp 4 allocates TMEM and its lane 0 issues the MMAs and
// the tcgen05.commit that frees a stage / publishes the accumulator.
// Every mbarrier wait is bounded by a clock64 budget; on expiry the CTA raises FORGE_ERR_TIMEOUT in
// the status word, drains its copies, frees TMEM and returns.
#include "common.cuh"
#include "tcgen05.cuh"

using namespace forge;
using namespace forge::tc;

namespace {

constexpr int32_t kNoRow = INT32_MIN;         // padding slot of a k-tile (past the end of the token list)
constexpr int kTile = 256;                    // output tile edge (channels)
constexpr int kKT = 64;                       // tokens per k-tile
// The tensor core adds each k-step's products to the fp32 accumulator with truncation, not round-to-nearest: the
// accumulated bias grows with the number of k-steps (measured against float64 at 7168 channels: 2e-6 relative after
// 1024 tokens, 3e-5 after 8192, 3e-4 after 65536, all towards zero; a round-to-nearest fp32 sum stays near 2e-6).  A
// tile's token range is therefore accumulated in pieces of at most kChunkKT k-tiles; each piece is added to H in the
// epilogue in ordinary fp32 arithmetic.  With 4096 tokens per piece the error stays below 2e-5 for any token count.
constexpr int kChunkKT = 64;
constexpr int kMaxSortedSlots = 512;           // more slots than this keep their index order
constexpr int kSubBytes = kKT * 128;          // one 64-channel x 64-token sub-tile: 8 KB
constexpr int kOperandBytes = 4 * kSubBytes;  // 256 channels: 32 KB
constexpr int kStageBytes = 2 * kOperandBytes;
constexpr int kStages = 3;
constexpr int kLag = 2;                       // cp.async groups in flight per thread
constexpr int kProducerThreads = 128;
constexpr int kEpilogueThreads = 256;           // warps 5..12: two per TMEM lane quarter, one accumulator half each
constexpr int kThreads = 160 + kEpilogueThreads; // 4 producer warps, the MMA warp, 8 epilogue warps
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;

struct HessParams {
    const __nv_bfloat16 *X;
    int64_t ldx, C;
    const int32_t *token_idx;
    const int64_t *offsets;
    int64_t n_rows;    // rows of X
    int64_t list_len;  // entries of token_idx (or n_rows when the rows are contiguous)
    int nb;
    float *H;
    const int64_t *n_prev;
    int mirror;
    int32_t *status;
    int nt;    // tiles per edge
    int ntri;  // tiles per expert (upper triangle)
};

// UMMA shared-memory descriptor, MN-major operand, 128-byte swizzle:
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4 (next 64-element
//   MN block: 8 KB)   bits [32,46) stride byte offset >> 4 (next group of 8 K rows: 1 KB)
//   bits [46,48) version = 1                  bits [61,64) layout = 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(kSubBytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D fp32, A/B bf16, both MN-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((256u >> 3) << 17) |
                            ((128u >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// A slot whose offsets claim rows outside the token list (or outside X when the rows are contiguous) is skipped
// by every role alike; the status word then says FORGE_ERR_INVALID.  Nothing is read through a bad claim.
__device__ __forceinline__ bool slot_in_bounds(const HessParams &P, int64_t off, int64_t n) {
    return off >= 0 && n >= 0 && off + n <= P.list_len;
}
__device__ __forceinline__ void tile_coords(int p, int nt, int &ti, int &tj) {
    ti = 0;
    while (p >= nt - ti) { p -= nt - ti; ++ti; }
    tj = ti + p;
}

__global__ void __launch_bounds__(kThreads, 1) hessian_tc_kernel(const HessParams P) {
    extern __shared__ uint8_t smem_raw[];
    // 1 KB alignment: the swizzle pattern and the descriptors (base_offset = 0) assume it
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_al + kStages * kStageBytes);
    // bars[0..2] full, [3..5] empty, [6] acc_full, [7] acc_empty, then tmem base + abort flag
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + 3);
    const uint32_t bar_acc_full = smem_u32(bars + 6), bar_acc_empty = smem_u32(bars + 7);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, kProducerThreads);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, kEpilogueThreads);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Slots in order of decreasing token count.  Tiles go to the CTAs round-robin along this order, so tiles of similar
    // cost are neighbours: the CTAs' loads differ by at most one tile of each weight class, and the last, partly filled
    // round consists of the cheapest tiles.  (In index order every heavy slot leaves some CTAs one heavy tile ahead, and
    // with a few hot experts among many cold ones those surpluses can pile up on the same CTAs.)  Every CTA computes
    // the same order itself; results do not depend on it (a tile is still one CTA's sum).
    __shared__ int32_t s_cnt[kMaxSortedSlots];
    __shared__ int16_t s_order[kMaxSortedSlots];
    const bool sorted = P.nb <= kMaxSortedSlots;
    if (sorted) {
        for (int i = tid; i < P.nb; i += kThreads) {
            const int64_t n = P.offsets[i + 1] - P.offsets[i];
            s_cnt[i] = (int32_t)(n < 0 ? 0 : (n > 0x7fffffff ? 0x7fffffff : n));
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (sorted) {
        for (int i = tid; i < P.nb; i += kThreads) {
            const int32_t ni = s_cnt[i];
            int rank = 0;
            for (int j = 0; j < P.nb; ++j) rank += (s_cnt[j] > ni) || (s_cnt[j] == ni && j < i);
            s_order[rank] = (int16_t)i;
        }
        __syncthreads();
    }
    const uint32_t tmem_base = *tmem_holder;

    const int64_t C = P.C;
    const int total_tiles = P.nb * P.ntri;
    uint32_t it = 0;         // k-tile counter of this CTA (ring position), same sequence in both roles
    uint32_t tile_iter = 0;  // accumulator hand-overs (pieces of tiles) done by this CTA

    if (warp < 4) {
        // ------------------------------ producers + epilogue ------------------------------
        const int rsub = lane >> 3;   // row within a group of 4
        const int chunk = lane & 7;   // 16-byte chunk within the 128-byte row
        int pend = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int b = sorted ? (int)s_order[tile / P.ntri] : tile / P.ntri;
            int ti, tj;
            tile_coords(tile % P.ntri, P.nt, ti, tj);
            const int64_t off = P.offsets[b];
            const int64_t n = P.offsets[b + 1] - off;
            if (!slot_in_bounds(P, off, n)) {
                if (tid == 0 && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
                continue;
            }
            if (n <= 0) continue;
            const bool diag = (ti == tj);
            const int nkt = (int)((n + kKT - 1) / kKT);
            const int32_t *tl = P.token_idx ? P.token_idx + off : nullptr;
            bool ok = true;
            bool bad_token = false;
            const uint32_t n_rows_u = (uint32_t)P.n_rows;
            // Token indices of the k-tile about to be issued; the ones of the NEXT k-tile are loaded right after
            // this tile's copies are issued, so that their latency never sits between two stages.
            int32_t tok_cur[4], tok_nxt[4];
            auto load_tokens = [&](int kt, int32_t (&dst)[4]) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int64_t kidx = (int64_t)kt * kKT + warp * 16 + i * 4 + rsub;
                    // no check here: the value is first looked at one k-tile later, so the load's latency stays hidden
                    int32_t t = kNoRow;
                    if (kidx < n) t = tl ? tl[kidx] : (int32_t)(off + kidx);
                    dst[i] = t;
                }
            };
            const int nch = (nkt + kChunkKT - 1) / kChunkKT, kt_per = (nkt + nch - 1) / nch;
            // channel offsets of the (up to) eight 64-channel sub-tiles this thread copies a chunk of
            const int64_t chA = (int64_t)ti * kTile + chunk * 8, chB = (int64_t)tj * kTile + chunk * 8;
            for (int piece = 0; piece < nch && ok; ++piece) {
            const int kt0 = piece * kt_per, kt1 = (kt0 + kt_per < nkt) ? kt0 + kt_per : nkt;
            const bool first_piece = (piece == 0);
            load_tokens(kt0, tok_cur);
            for (int kt = kt0; kt < kt1 && ok; ++kt) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag);
                if (!ok) break;
                const uint32_t stage = smem_base + s * kStageBytes;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = warp * 16 + i * 4 + rsub;  // token row inside the k-tile
                    // a list entry that is not a row of X contributes zeros (and is reported once per tile)
                    const bool rvalid = (uint32_t)tok_cur[i] < n_rows_u;
                    bad_token |= (!rvalid && tok_cur[i] != kNoRow);
                    const __nv_bfloat16 *xrow = P.X + (int64_t)(rvalid ? tok_cur[i] : 0) * P.ldx;
                    const uint32_t drow = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
#pragma unroll
                    for (int sub = 0; sub < 8; ++sub) {
                        if (diag && sub >= 4) break;
                        const int64_t ch = (sub < 4 ? chA : chB) + (sub & 3) * 64;
                        const bool v = rvalid && (ch < C);
                        cp_async16_zfill(stage + sub * kSubBytes + drow, v ? (const void *)(xrow + ch) : (const void *)P.X, v);
                    }
                }
                if (kt + 1 < kt1) load_tokens(kt + 1, tok_nxt);
#pragma unroll
                for (int i = 0; i < 4; ++i) tok_cur[i] = tok_nxt[i];
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
            while (pend > 0) {  // publish the stages still in flight
                if (pend >= 2) cp_async_wait<1>();
                else cp_async_wait<0>();
                fence_proxy_async();
                mbar_arrive(bar_full + 8 * ((it - pend) % kStages));
                --pend;
            }
            if (!ok) break;
            }   // pieces of the token range
            if (bad_token && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
            if (!ok) break;
        }
        cp_async_wait<0>();
    } else if (warp >= 5) {
        // ------------------------------ epilogue (warps 5..12) ------------------------------
        // Warp w reads TMEM lanes 32 (w % 4) .. +31 (the hardware's rule) of accumulator half mh = (w - 5) / 4: the
        // eight warps cover the 256 x 256 tile once.  The producers meanwhile refill the operand ring for the next
        // piece or tile; the MMA warp resumes when all 256 threads have arrived on acc_empty.
        const int q = warp & 3, mh = (warp - 5) >> 2;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int b = sorted ? (int)s_order[tile / P.ntri] : tile / P.ntri;
            int ti, tj;
            tile_coords(tile % P.ntri, P.nt, ti, tj);
            const int64_t n = P.offsets[b + 1] - P.offsets[b];
            if (n <= 0 || !slot_in_bounds(P, P.offsets[b], n)) continue;
            const int nkt = (int)((n + kKT - 1) / kKT);
            const int nch = (nkt + kChunkKT - 1) / kChunkKT;
            bool ok = true;
            for (int piece = 0; piece < nch && ok; ++piece) {
            const bool first_piece = (piece == 0);
            ok = mbar_wait(bar_acc_full, tile_iter & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below is warp-aligned: the whole warp goes or none
            if (!ok) break;
            tc_fence_after();
            const int64_t np = P.n_prev ? P.n_prev[b] : 0;
            const double Ntot = (double)(np + n);
            const float alpha = (float)(2.0 / Ntot);
            const float beta = (float)((double)np / Ntot);
            float *Hb = P.H + (int64_t)b * C * C;
            {
                const int64_t m = (int64_t)ti * kTile + mh * 128 + q * 32 + lane;
#pragma unroll 1
                for (int cc = 0; cc < 8; ++cc) {
                    const int64_t n0 = (int64_t)tj * kTile + cc * 32;
                    // whole 32x32 sub-block below the diagonal or out of range: nothing to store
                    const int64_t m_lo = (int64_t)ti * kTile + mh * 128 + q * 32;
                    if (n0 + 31 < m_lo || n0 >= C || m_lo >= C) continue;  // warp-uniform
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mh * 256 + cc * 32), v);
                    tmem_ld_wait();
                    if (m < C) {
                        const bool vec_ok = (C % 4 == 0);
#pragma unroll
                        for (int g4 = 0; g4 < 8; ++g4) {
                            const int64_t nn0 = n0 + 4 * g4;
                            float val[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) val[e] = alpha * __uint_as_float(v[4 * g4 + e]);
                            if (!first_piece) {
                                // later pieces: H += alpha acc as fire-and-forget fp32 additions in L2 (round to
                                // nearest), on the entry and on its mirror image: both see the same sequence of
                                // additions, so the matrix stays exactly symmetric, and no load sits in the epilogue
                                if (vec_ok && nn0 >= m && nn0 + 3 < C) {
                                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(Hb + m * C + nn0),
                                                 "f"(val[0]), "f"(val[1]), "f"(val[2]), "f"(val[3])
                                                 : "memory");
                                    if (P.mirror) {
#pragma unroll
                                        for (int e = 0; e < 4; ++e)
                                            if (nn0 + e > m) atomicAdd(Hb + (nn0 + e) * C + m, val[e]);
                                    }
                                } else {
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        const int64_t nn = nn0 + e;
                                        if (nn < C && nn >= m) {
                                            atomicAdd(Hb + m * C + nn, val[e]);
                                            if (P.mirror && nn > m) atomicAdd(Hb + nn * C + m, val[e]);
                                        }
                                    }
                                }
                            } else if (vec_ok && nn0 >= m && nn0 + 3 < C) {
                                float4 *dst = reinterpret_cast<float4 *>(Hb + m * C + nn0);
                                if (np > 0) {
                                    const float4 old = *dst;
                                    val[0] = fmaf(beta, old.x, val[0]); val[1] = fmaf(beta, old.y, val[1]);
                                    val[2] = fmaf(beta, old.z, val[2]); val[3] = fmaf(beta, old.w, val[3]);
                                }
                                *dst = make_float4(val[0], val[1], val[2], val[3]);
                                if (P.mirror) {
#pragma unroll
                                    for (int e = 0; e < 4; ++e)
                                        if (nn0 + e > m) Hb[(nn0 + e) * C + m] = val[e];
                                }
                            } else {
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int64_t nn = nn0 + e;
                                    if (nn < C && nn >= m) {
                                        float x = val[e];
                                        if (np > 0) x = fmaf(beta, Hb[m * C + nn], x);
                                        Hb[m * C + nn] = x;
                                        if (P.mirror && nn > m) Hb[nn * C + m] = x;
                                    }
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_acc_empty);
            ++tile_iter;
            }   // pieces of the token range
            if (!ok) break;
        }
    } else {
        // ------------------------------ MMA issuer (warp 4) ------------------------------
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int b = sorted ? (int)s_order[tile / P.ntri] : tile / P.ntri;
            int ti, tj;
            tile_coords(tile % P.ntri, P.nt, ti, tj);
            const int64_t n = P.offsets[b + 1] - P.offsets[b];
            if (n <= 0 || !slot_in_bounds(P, P.offsets[b], n)) continue;
            const bool diag = (ti == tj);
            const int nkt = (int)((n + kKT - 1) / kKT);
            const int nch = (nkt + kChunkKT - 1) / kChunkKT, kt_per = (nkt + nch - 1) / nch;
            bool ok = true;
            for (int piece = 0; piece < nch && ok; ++piece) {
            const int kt0 = piece * kt_per, kt1 = (kt0 + kt_per < nkt) ? kt0 + kt_per : nkt;
            ok = mbar_wait(bar_acc_empty, (tile_iter & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            for (int kt = kt0; kt < kt1 && ok; ++kt) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_base = smem_base + s * kStageBytes;
                    const uint32_t b_base = diag ? a_base : a_base + kOperandBytes;
#pragma unroll
                    for (int kk = 0; kk < kKT / 16; ++kk) {
                        const uint64_t bdesc = make_desc(b_base + kk * 2048);
#pragma unroll
                        for (int mh = 0; mh < 2; ++mh) {
                            const uint64_t adesc = make_desc(a_base + mh * 2 * kSubBytes + kk * 2048);
                            umma_bf16(tmem_base + mh * 256, adesc, bdesc, (kt > kt0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(bar_empty + 8 * s);  // frees the stage once these MMAs have read it
                }
                __syncwarp();
                ++it;
            }
            if (!ok) break;
            if (lane == 0) umma_commit(bar_acc_full);
            __syncwarp();
            ++tile_iter;
            }   // pieces of the token range
            if (!ok) break;
        }
    }
    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0 && P.status) atomicExch(P.status, FORGE_ERR_TIMEOUT);
    if (warp == 4) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Plain-FMA validation kernel (same contract, upper triangle + optional mirror): 16x16 outputs per
// CTA, tokens staged 16 at a time.  Exists so that the tensor-core kernel can be cross-checked on the
// GPU itself; it is not on the product path unless FORGE_HESS_SIMT is passed.
__global__ void hessian_simt_kernel(const HessParams P) {
    __shared__ float xa[16][17], xb[16][17];
    const int b = blockIdx.z;
    const int64_t C = P.C;
    const int64_t m0 = (int64_t)blockIdx.y * 16, n0 = (int64_t)blockIdx.x * 16;
    if (n0 + 15 < m0) return;
    const int64_t off = P.offsets[b];
    const int64_t n = P.offsets[b + 1] - off;
    if (!slot_in_bounds(P, off, n)) {
        if (threadIdx.x == 0 && threadIdx.y == 0 && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
        return;
    }
    if (n <= 0) return;
    const int32_t *tl = P.token_idx ? P.token_idx + off : nullptr;
    const int tx = threadIdx.x, ty = threadIdx.y;
    float acc = 0.0f;
    for (int64_t k0 = 0; k0 < n; k0 += 16) {
        const int64_t kidx = k0 + ty;
        float va = 0.0f, vb = 0.0f;
        const int64_t tok = (kidx < n) ? (tl ? (int64_t)tl[kidx] : off + kidx) : -1;
        if (kidx < n && (tok < 0 || tok >= P.n_rows) && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
        if (tok >= 0 && tok < P.n_rows) {
            if (m0 + tx < C) va = __bfloat162float(P.X[tok * P.ldx + m0 + tx]);
            if (n0 + tx < C) vb = __bfloat162float(P.X[tok * P.ldx + n0 + tx]);
        }
        xa[ty][tx] = va;
        xb[ty][tx] = vb;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = fmaf(xa[k][ty], xb[k][tx], acc);
        __syncthreads();
    }
    const int64_t m = m0 + ty, nn = n0 + tx;
    if (m < C && nn < C && nn >= m) {
        const int64_t np = P.n_prev ? P.n_prev[b] : 0;
        const double Ntot = (double)(np + n);
        const float alpha = (float)(2.0 / Ntot), beta = (float)((double)np / Ntot);
        float *Hb = P.H + (int64_t)b * C * C;
        float val = alpha * acc;
        if (np > 0) val = fmaf(beta, Hb[m * C + nn], val);
        Hb[m * C + nn] = val;
        if (P.mirror && nn > m) Hb[nn * C + m] = val;
    }
}

}  // namespace

// Self-test of the bounded wait every tensor-core kernel here relies on: one CTA waits on an mbarrier that nothing
// ever arrives on, with a budget of `budget_cycles`; the wait gives up, the kernel writes FORGE_ERR_TIMEOUT to the
// status word and returns normally.  Nothing faults or hangs: this is how a lost producer would surface.
__global__ void bounded_wait_selftest_kernel(int32_t *status, long long budget_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, budget_cycles);
    __syncthreads();
    if (threadIdx.x == 0) *status = ok ? FORGE_OK : FORGE_ERR_TIMEOUT;
}

extern "C" int forge_selftest_bounded_wait(int32_t *status, int64_t budget_cycles, void *stream) {
    FORGE_REQUIRE(status, "null pointer");
    FORGE_REQUIRE(budget_cycles > 0 && budget_cycles <= 2000000000LL, "budget must be in (0, 2e9] cycles");
    bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, (long long)budget_cycles); FORGE_NOTE_LAUNCH();
    return check_launch("forge_selftest_bounded_wait");
}

extern "C" int forge_hessian_grouped(const void *X_bf16, int64_t n_rows, int64_t ldx, int64_t C,
                                     const int32_t *token_idx, int64_t list_len, const int64_t *offsets, int nb,
                                     float *H, const int64_t *n_prev, int flags, int32_t *status, void *stream) {
    FORGE_REQUIRE(X_bf16 && offsets && H, "null pointer");
    FORGE_REQUIRE(nb > 0 && C > 0 && ldx >= C, "bad sizes");
    FORGE_REQUIRE(n_rows >= 0 && n_rows <= 0x7fffffffLL, "n_rows must fit a 32-bit token index");
    FORGE_REQUIRE(!token_idx || list_len >= 0, "list_len must be >= 0");
    cudaStream_t st = (cudaStream_t)stream;
    HessParams P{};
    P.X = (const __nv_bfloat16 *)X_bf16; P.ldx = ldx; P.C = C; P.token_idx = token_idx; P.offsets = offsets;
    P.n_rows = n_rows; P.list_len = token_idx ? list_len : n_rows;
    P.nb = nb; P.H = H; P.n_prev = n_prev; P.mirror = (flags & FORGE_HESS_MIRROR) ? 1 : 0; P.status = status;
    P.nt = (int)cdiv(C, kTile);
    P.ntri = P.nt * (P.nt + 1) / 2;
    if (flags & FORGE_HESS_SIMT) {
        dim3 grid((unsigned)cdiv(C, 16), (unsigned)cdiv(C, 16), nb);
        hessian_simt_kernel<<<grid, dim3(16, 16), 0, st>>>(P); FORGE_NOTE_LAUNCH();
        return check_launch("forge_hessian_grouped(simt)");
    }
    FORGE_REQUIRE(C % 8 == 0 && ldx % 8 == 0, "C and ldx must be multiples of 8 (16-byte row chunks)");
    FORGE_REQUIRE((uintptr_t)X_bf16 % 16 == 0, "X must be 16-byte aligned");
    {   // per-device attribute: set on the device that is current for this call
        cudaError_t e = cudaFuncSetAttribute(hessian_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBytes);
        if (e != cudaSuccess) {
            set_error("forge_hessian_grouped: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return FORGE_ERR_LAUNCH;
        }
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t total = (int64_t)nb * P.ntri;
    const int grid = (int)imin64(total, sms);
    hessian_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(P); FORGE_NOTE_LAUNCH();
    return check_launch("forge_hessian_grouped");
}
