// HBM-bandwidth kernels of the path: fp8 block de-quantisation, routing lists, Hessian
// preparation (NaN scan, pruning, permutation gather + damping), code de-quantisation, and the
// two bit-exact packers.  All are plain coalesced SIMT kernels; none is GEMM-shaped.
#include "common.cuh"
#include "tcgen05.cuh"
#include <stdarg.h>

namespace forge {
static thread_local char g_err[512] = "";
void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
static long long g_launches = 0;
void note_launch() { __atomic_fetch_add(&g_launches, 1, __ATOMIC_RELAXED); }
}  // namespace forge
using namespace forge;

extern "C" long long forge_launch_count(void) { return __atomic_load_n(&forge::g_launches, __ATOMIC_RELAXED); }

extern "C" int forge_version(void) { return 100; }
extern "C" const char *forge_last_error(void) { return g_err; }

// --------------------------------------------------------------------------------------------
// fp8 e4m3 block de-quantisation
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ float fp8_e4m3_to_f32(uint8_t v) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
    return __half2float(__half(h));
}

// One thread converts 16 consecutive elements of a row (16 B in, 32 B out).
__global__ void fp8_dequant_vec16(const uint8_t *__restrict__ w, const float *__restrict__ sinv,
                                  __nv_bfloat16 *__restrict__ out, int64_t O, int64_t I, int64_t nI,
                                  int64_t so, int64_t si) {
    const int64_t vec_per_row = I / 16;
    const int64_t total = O * vec_per_row;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total;
         v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = v / vec_per_row, i0 = (v % vec_per_row) * 16;
        const uint4 raw = *reinterpret_cast<const uint4 *>(w + o * I + i0);
        const uint8_t *b = reinterpret_cast<const uint8_t *>(&raw);
        const float *srow = sinv + (o / so) * nI;
        __align__(16) __nv_bfloat16 r[16];
        if (si % 16 == 0) {
            const float s = srow[i0 / si];     // the 16 elements lie in one column tile
#pragma unroll
            for (int e = 0; e < 16; ++e) r[e] = __float2bfloat16_rn(fp8_e4m3_to_f32(b[e]) * s);
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const float s = srow[(i0 + e) / si];
                r[e] = __float2bfloat16_rn(fp8_e4m3_to_f32(b[e]) * s);
            }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + o * I + i0);
        dst[0] = reinterpret_cast<uint4 *>(r)[0];
        dst[1] = reinterpret_cast<uint4 *>(r)[1];
    }
}

__global__ void fp8_dequant_scalar(const uint8_t *__restrict__ w, const float *__restrict__ sinv,
                                   __nv_bfloat16 *__restrict__ out, int64_t O, int64_t I, int64_t nI,
                                   int64_t so, int64_t si) {
    const int64_t total = O * I;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = e / I, i = e % I;
        out[e] = __float2bfloat16_rn(fp8_e4m3_to_f32(w[e]) * sinv[(o / so) * nI + i / si]);
    }
}

extern "C" int forge_fp8_block_dequant(const void *w_fp8, const float *scale_inv, void *out_bf16, int64_t O,
                                       int64_t I, int64_t nO, int64_t nI, void *stream) {
    FORGE_REQUIRE(w_fp8 && scale_inv && out_bf16, "null pointer");
    FORGE_REQUIRE(O > 0 && I > 0 && nO > 0 && nI > 0, "empty shape");
    FORGE_REQUIRE(I % nI == 0, "I must be a multiple of the number of column tiles");
    const int64_t si = I / nI;
    const int64_t so = (cdiv(O, si) == nO) ? si : cdiv(O, nO);
    FORGE_REQUIRE(cdiv(O, so) <= nO, "scale grid has too few row tiles");
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = (I % 16 == 0) && ((uintptr_t)w_fp8 % 16 == 0) && ((uintptr_t)out_bf16 % 16 == 0);
    const int64_t work = vec ? O * (I / 16) : O * I;
    const int threads = 256;
    const int blocks = (int)imin64(cdiv(work, threads), 148 * 16);
    if (vec) { fp8_dequant_vec16<<<blocks, threads, 0, st>>>((const uint8_t *)w_fp8, scale_inv,
                                                      (__nv_bfloat16 *)out_bf16, O, I, nI, so, si); FORGE_NOTE_LAUNCH(); } else { fp8_dequant_scalar<<<blocks, threads, 0, st>>>((const uint8_t *)w_fp8, scale_inv,
                                                       (__nv_bfloat16 *)out_bf16, O, I, nI, so, si); FORGE_NOTE_LAUNCH(); }
    return check_launch("forge_fp8_block_dequant");
}

// --------------------------------------------------------------------------------------------
// routing lists: one CTA per local expert scans the [T,k] id table twice (count, then fill), so the
// tokens of an expert come out in ascending order without a sort.
// --------------------------------------------------------------------------------------------
template <bool FILL>
__global__ void route_scan_kernel(const int32_t *__restrict__ ids, int64_t T, int k, int e_begin,
                                  int32_t *__restrict__ counts, const int64_t *__restrict__ offsets,
                                  int32_t *__restrict__ lists) {
    const int e_local = blockIdx.x;
    const int e = e_begin + e_local;
    __shared__ int warp_tot[32];
    __shared__ int base_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (threadIdx.x == 0) base_s = 0;
    __syncthreads();
    const int64_t out0 = FILL ? offsets[e_local] : 0;
    for (int64_t t0 = 0; t0 < T; t0 += blockDim.x) {
        const int64_t t = t0 + threadIdx.x;
        int hit = 0;
        if (t < T) {
            for (int j = 0; j < k; ++j) hit |= (ids[t * k + j] == e);
        }
        const unsigned bal = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_tot[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < nwarp; ++w) {
            const int c = warp_tot[w];
            if (w < warp) before += c;
            total += c;
        }
        if (FILL && hit) {
            const int pos = base_s + before + __popc(bal & ((1u << lane) - 1u));
            lists[out0 + pos] = (int32_t)t;
        }
        __syncthreads();
        if (threadIdx.x == 0) base_s += total;
        __syncthreads();
    }
    if (!FILL && threadIdx.x == 0) counts[e_local] = base_s;
}

// offsets = exclusive prefix sum of counts; the `tail` dense slots behind the routed ones see every token
__global__ void route_offsets_kernel(int32_t *__restrict__ counts, int n, int tail, int64_t T,
                                     int64_t *__restrict__ offsets) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int64_t acc = 0;
        for (int i = 0; i < n; ++i) {
            offsets[i] = acc;
            acc += counts[i];
        }
        for (int i = n; i < n + tail; ++i) {
            counts[i] = (int32_t)T;
            offsets[i] = acc;
            acc += T;
        }
        offsets[n + tail] = acc;
    }
}

// token list of a dense slot: 0, 1, ..., T-1
__global__ void route_dense_fill_kernel(const int64_t *__restrict__ offsets, int n, int64_t T,
                                        int32_t *__restrict__ lists) {
    const int64_t base = offsets[n + blockIdx.y];
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < T; t += (int64_t)gridDim.x * blockDim.x)
        lists[base + t] = (int32_t)t;
}

extern "C" int forge_route_build_lists(const int32_t *topk_ids, int64_t T, int k, int e_begin, int e_count,
                                       int dense_tail, int32_t *counts, int64_t *offsets, int32_t *token_lists,
                                       void *stream) {
    FORGE_REQUIRE(counts && offsets && token_lists, "null pointer");
    FORGE_REQUIRE(T >= 0 && k > 0 && e_count >= 0 && dense_tail >= 0 && e_count + dense_tail > 0 && e_begin >= 0,
                  "bad sizes");
    FORGE_REQUIRE(e_count == 0 || topk_ids, "null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    if (e_count > 0) {
        route_scan_kernel<false><<<e_count, 512, 0, st>>>(topk_ids, T, k, e_begin, counts, nullptr, nullptr); FORGE_NOTE_LAUNCH();
    }
    route_offsets_kernel<<<1, 32, 0, st>>>(counts, e_count, dense_tail, T, offsets); FORGE_NOTE_LAUNCH();
    if (e_count > 0) {
        route_scan_kernel<true><<<e_count, 512, 0, st>>>(topk_ids, T, k, e_begin, counts, offsets, token_lists); FORGE_NOTE_LAUNCH();
    }
    if (dense_tail > 0 && T > 0) {
        route_dense_fill_kernel<<<dim3((unsigned)imin64(cdiv(T, 256), 592), dense_tail), 256, 0, st>>>(offsets, e_count, T, token_lists);
        FORGE_NOTE_LAUNCH();
    }
    return check_launch("forge_route_build_lists");
}

__global__ void counts_add_kernel(int64_t *n_prev, const int64_t *offsets, int nb) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < nb) n_prev[b] += offsets[b + 1] - offsets[b];
}
extern "C" int forge_counts_add(int64_t *n_prev, const int64_t *offsets, int nb, void *stream) {
    FORGE_REQUIRE(n_prev && offsets && nb > 0, "bad arguments");
    counts_add_kernel<<<(nb + 127) / 128, 128, 0, (cudaStream_t)stream>>>(n_prev, offsets, nb); FORGE_NOTE_LAUNCH();
    return check_launch("forge_counts_add");
}

// --------------------------------------------------------------------------------------------
// Hessian preparation
// --------------------------------------------------------------------------------------------
__global__ void scan_init_kernel(const int64_t *n_samples, int32_t *invalid, int nb) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < nb) invalid[b] = (n_samples != nullptr && n_samples[b] == 0) ? 1 : 0;
}

__global__ void scan_nan_kernel(const float *__restrict__ H, int64_t elems, int32_t *invalid) {
    const int b = blockIdx.y;
    const float *Hb = H + (int64_t)b * elems;
    int bad = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if ((elems % 4 == 0) && ((uintptr_t)Hb % 16 == 0)) {
        const float4 *H4 = reinterpret_cast<const float4 *>(Hb);
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems / 4; i += stride) {
            const float4 v = H4[i];
            bad |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += stride) {
            const float v = Hb[i];
            bad |= (v != v);
        }
    }
    bad = __any_sync(0xffffffffu, bad);
    if (bad && (threadIdx.x & 31) == 0) atomicOr(invalid + b, 1);
}

__global__ void scan_diag_kernel(const float *__restrict__ H, int64_t C, const int32_t *__restrict__ invalid,
                                 float *__restrict__ diag, uint8_t *__restrict__ pruned) {
    const int b = blockIdx.y;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const bool inv = invalid[b] != 0;
    const float d = inv ? 1.0f : H[(int64_t)b * C * C + c * C + c];
    const bool pr = (!inv) && (d == 0.0f);
    diag[(int64_t)b * C + c] = pr ? 1.0f : d;
    pruned[(int64_t)b * C + c] = pr ? 1 : 0;
}

extern "C" int forge_hessian_scan(const float *H, int nb, int64_t C, const int64_t *n_samples, float *diag,
                                  uint8_t *pruned, int32_t *invalid, void *stream) {
    FORGE_REQUIRE(H && diag && pruned && invalid, "null pointer");
    FORGE_REQUIRE(nb > 0 && C > 0, "empty batch");
    cudaStream_t st = (cudaStream_t)stream;
    scan_init_kernel<<<(nb + 127) / 128, 128, 0, st>>>(n_samples, invalid, nb); FORGE_NOTE_LAUNCH();
    const int64_t elems = C * C;
    const int bx = (int)imin64(cdiv(elems / 4 + 1, 256), 64);
    scan_nan_kernel<<<dim3(bx, nb), 256, 0, st>>>(H, elems, invalid); FORGE_NOTE_LAUNCH();
    scan_diag_kernel<<<dim3((unsigned)cdiv(C, 256), nb), 256, 0, st>>>(H, C, invalid, diag, pruned); FORGE_NOTE_LAUNCH();
    return check_launch("forge_hessian_scan");
}

// W[b,:,c] = 0 for the pruned columns c of Hessian slot u_map[b]   (forge/gptq.py:115)
__global__ void apply_pruned_kernel(void *W, int dtype, int64_t R, int64_t C, const uint8_t *__restrict__ pruned,
                                    const int32_t *__restrict__ u_map) {
    const int b = blockIdx.z;
    const int u = u_map ? u_map[b] : b;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C || !pruned[(int64_t)u * C + c]) return;
    for (int64_t r = blockIdx.y; r < R; r += gridDim.y) {
        const int64_t i = ((int64_t)b * R + r) * C + c;
        if (dtype == FORGE_DTYPE_BF16) reinterpret_cast<__nv_bfloat16 *>(W)[i] = __float2bfloat16_rn(0.0f);
        else reinterpret_cast<float *>(W)[i] = 0.0f;
    }
}
extern "C" int forge_weight_apply_pruned(void *W, int w_dtype, int nb, int64_t R, int64_t C,
                                         const uint8_t *pruned, const int32_t *u_map, void *stream) {
    FORGE_REQUIRE(W && pruned && nb > 0 && R > 0 && C > 0, "bad arguments");
    dim3 grid((unsigned)cdiv(C, 128), (unsigned)imin64(R, 64), nb);
    apply_pruned_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(W, w_dtype, R, C, pruned, u_map); FORGE_NOTE_LAUNCH();
    return check_launch("forge_weight_apply_pruned");
}

// wzero[b,c] = all_r W[b,r,c] == 0.  One thread per column, coalesced across columns; almost every
// thread leaves at r = 0.
__global__ void zero_cols_kernel(const void *__restrict__ W, int dtype, int64_t R, int64_t C,
                                 uint8_t *__restrict__ wzero) {
    const int b = blockIdx.y;
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    int allz = 1;
    for (int64_t r = 0; r < R; ++r) {
        if (ld_as_f32(W, dtype, ((int64_t)b * R + r) * C + c) != 0.0f) { allz = 0; break; }
    }
    wzero[(int64_t)b * C + c] = (uint8_t)allz;
}
extern "C" int forge_weight_zero_cols(const void *W, int w_dtype, int nb, int64_t R, int64_t C, uint8_t *wzero,
                                      void *stream) {
    FORGE_REQUIRE(W && wzero && nb > 0 && R > 0 && C > 0, "bad arguments");
    zero_cols_kernel<<<dim3((unsigned)cdiv(C, 128), nb), 128, 0, (cudaStream_t)stream>>>(W, w_dtype, R, C, wzero); FORGE_NOTE_LAUNCH();
    return check_launch("forge_weight_zero_cols");
}

__device__ __forceinline__ float hp_diag_value(const float *Hb, int64_t C, int64_t i, const int32_t *perm_b,
                                               const uint8_t *pruned_b, const uint8_t *wzero_b, bool inv) {
    if (wzero_b && wzero_b[i]) return 1.0f;
    if (inv) return 1.0f;
    const int64_t pi = perm_b ? perm_b[i] : i;
    if (pruned_b && pruned_b[pi]) return 1.0f;
    return Hb[pi * C + pi];
}

__global__ void damp_kernel(const float *__restrict__ H, int64_t C, const int32_t *__restrict__ perm,
                            const uint8_t *__restrict__ pruned, const uint8_t *__restrict__ wzero,
                            const int32_t *__restrict__ invalid, float rel_damp, float *__restrict__ damp_out) {
    const int b = blockIdx.x;
    const float *Hb = H + (int64_t)b * C * C;
    const int32_t *pb = perm ? perm + (int64_t)b * C : nullptr;
    const uint8_t *prb = pruned ? pruned + (int64_t)b * C : nullptr;
    const uint8_t *wzb = wzero ? wzero + (int64_t)b * C : nullptr;
    const bool inv = invalid ? invalid[b] != 0 : false;
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) acc += (double)hp_diag_value(Hb, C, i, pb, prb, wzb, inv);
    __shared__ double red[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
        const float mean = (float)(t / (double)C);
        damp_out[b] = rel_damp * mean;
    }
}

// One CTA per (three output rows i, matrix b): stage rows perm[i] of H in shared memory, then emit Hp[i, :] through
// the permutation, index-reversed, with the fix-ups and the damping applied.  The per-column source index and flags
// (permutation, dead channel, all-zero weight column) are gathered ONCE per CTA into a fourth shared-memory row, with
// all their (dependent: permutation -> dead flag) global loads in flight together and beside the row loads; the output
// loop then touches shared memory only.  (With the loads inside the output loop every column paid two L2 round trips
// in sequence: the kernel ran at 0.3 of the HBM roofline.)
constexpr int kGdRows = 3;
__global__ void gather_damp_kernel(const float *__restrict__ H, int64_t C, const int32_t *__restrict__ perm,
                                   const uint8_t *__restrict__ pruned, const uint8_t *__restrict__ wzero,
                                   const int32_t *__restrict__ invalid, const float *__restrict__ damp,
                                   float *__restrict__ A, float *__restrict__ Hp_out) {
    extern __shared__ __align__(16) float row[];     // [kGdRows][C] rows, then [C] column codes
    __shared__ __align__(8) uint64_t gd_bar;
    __shared__ int gd_abort;
    const int b = blockIdx.y;
    const int64_t i0 = (int64_t)blockIdx.x * kGdRows;
    const float *Hb = H + (int64_t)b * C * C;
    const int32_t *pb = perm ? perm + (int64_t)b * C : nullptr;
    const uint8_t *prb = pruned ? pruned + (int64_t)b * C : nullptr;
    const uint8_t *wzb = wzero ? wzero + (int64_t)b * C : nullptr;
    const bool inv = invalid ? invalid[b] != 0 : false;
    // Fast path (the usual case without activation order): natural order and no dead channel / zero column anywhere
    // in this matrix: a pure index reversal of the rows with the damping on the diagonal, 16 bytes per access.
    if (!pb && (C & 3) == 0) {
        int flagged = inv ? 1 : 0;
        for (int64_t c = (int64_t)threadIdx.x * 16; c < C; c += (int64_t)blockDim.x * 16) {
            if (c + 16 <= C && (C & 15) == 0) {
                if (prb) { const uint4 f = *reinterpret_cast<const uint4 *>(prb + c); flagged |= (f.x | f.y | f.z | f.w) != 0u; }
                if (wzb) { const uint4 f = *reinterpret_cast<const uint4 *>(wzb + c); flagged |= (f.x | f.y | f.z | f.w) != 0u; }
            } else {
                for (int64_t e = c; e < C && e < c + 16; ++e) flagged |= (prb && prb[e]) || (wzb && wzb[e]);
            }
        }
        if (!__syncthreads_or(flagged)) {
            const float dmp = damp[b];
            for (int rr = 0; rr < kGdRows; ++rr) {
                const int64_t i = i0 + rr;
                if (i >= C) break;
                const float4 *src = reinterpret_cast<const float4 *>(Hb + i * C);
                float *Arow = A + (int64_t)b * C * C + (C - 1 - i) * C;
                float *Hrow = Hp_out ? Hp_out + (int64_t)b * C * C + i * C : nullptr;
                for (int64_t c4 = threadIdx.x; c4 < C / 4; c4 += blockDim.x) {
                    float4 v = src[c4];
                    const int64_t j = 4 * c4;
                    if (i >= j && i < j + 4) {
                        const int k = (int)(i - j);
                        if (k == 0) v.x += dmp; else if (k == 1) v.y += dmp; else if (k == 2) v.z += dmp; else v.w += dmp;
                    }
                    if (Hrow) *reinterpret_cast<float4 *>(Hrow + j) = v;
                    *reinterpret_cast<float4 *>(Arow + (C - 4 - j)) = make_float4(v.w, v.z, v.y, v.x);
                }
            }
            return;
        }
    }
    int64_t pi[kGdRows];
    bool row_dead[kGdRows], row_wz[kGdRows], row_in[kGdRows];
#pragma unroll
    for (int rr = 0; rr < kGdRows; ++rr) {
        const int64_t i = i0 + rr;
        row_in[rr] = i < C;
        pi[rr] = row_in[rr] ? (pb ? (int64_t)pb[i] : i) : 0;
        row_dead[rr] = inv || (row_in[rr] && prb && prb[pi[rr]]);
        row_wz[rr] = row_in[rr] && wzb && wzb[i];
    }
    // The rows come in by bulk copies that one thread issues (the whole 3 x 4C bytes of a CTA in flight at once, at
    // no register cost; per-thread loads kept ~16 KB per CTA in flight and the kernel at 0.3 of the HBM roofline)
    // while all threads gather the column codes.
    const bool vec = (C & 3) == 0;
    const uint32_t bar = forge::tc::smem_u32(&gd_bar);
    if (vec) {
        if (threadIdx.x == 0) {
            gd_abort = 0;
            forge::tc::mbar_init(bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t bytes = 0;
#pragma unroll
            for (int rr = 0; rr < kGdRows; ++rr)
                if (row_in[rr] && !row_dead[rr] && !row_wz[rr]) bytes += (uint32_t)(C * 4);
            forge::tc::mbar_arrive_expect_tx(bar, bytes);
            constexpr uint32_t kPiece = 8192;
#pragma unroll
            for (int rr = 0; rr < kGdRows; ++rr) {
                if (!row_in[rr] || row_dead[rr] || row_wz[rr]) continue;
                const char *src = reinterpret_cast<const char *>(Hb + pi[rr] * C);
                const uint32_t dst = forge::tc::smem_u32(row + (int64_t)rr * C);
                for (uint32_t off = 0; off < (uint32_t)(C * 4); off += kPiece) {
                    const uint32_t n = min(kPiece, (uint32_t)(C * 4) - off);
                    forge::tc::bulk_copy_g2s(dst + off, src + off, n, bar);
                }
            }
        }
    }
    // column codes: source column pj in the low 30 bits, bit 31 = all-zero weight column at position j, bit 30 = dead
    // channel pj
    uint32_t *code = reinterpret_cast<uint32_t *>(row + (int64_t)kGdRows * C);
    for (int64_t j = threadIdx.x; j < C; j += blockDim.x) {
        const uint32_t pj = pb ? (uint32_t)__ldg(pb + j) : (uint32_t)j;
        uint32_t cw = pj;
        if (wzb && __ldg(wzb + j)) cw |= 0x80000000u;
        if (prb && __ldg(prb + pj)) cw |= 0x40000000u;
        code[j] = cw;
    }
    bool by_hand = !vec;
    if (vec && !forge::tc::mbar_wait(bar, 0, &gd_abort)) by_hand = true;   // the wait is bounded; plain loads then
    if (__syncthreads_or(by_hand ? 1 : 0)) {
#pragma unroll
        for (int rr = 0; rr < kGdRows; ++rr) {
            if (!row_in[rr] || row_dead[rr] || row_wz[rr]) continue;
            const float *src = Hb + pi[rr] * C;
            float *dst = row + (int64_t)rr * C;
            for (int64_t c = threadIdx.x; c < C; c += blockDim.x) dst[c] = src[c];
        }
        if (vec) {   // bulk copies may still be landing (with the same bytes): give them one more bounded wait
            volatile int again = 0;
            forge::tc::mbar_wait(bar, 0, &again);
        }
        __syncthreads();
    }
    const float dmp = damp[b];
    if (vec && !Hp_out) {
        // four consecutive output columns per thread: one 16-byte read of the codes, one 16-byte store per row
        for (int64_t jo = (int64_t)threadIdx.x * 4; jo < C; jo += (int64_t)blockDim.x * 4) {
            const int64_t jlo = C - 4 - jo;   // positions jlo+3, jlo+2, jlo+1, jlo <-> output columns jo .. jo+3
            const uint4 cq = *reinterpret_cast<const uint4 *>(code + jlo);
            const uint32_t cws[4] = {cq.w, cq.z, cq.y, cq.x};
#pragma unroll
            for (int rr = 0; rr < kGdRows; ++rr) {
                if (!row_in[rr]) continue;
                const int64_t i = i0 + rr;
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int64_t j = jlo + 3 - e;
                    const uint32_t cw = cws[e];
                    const int64_t pj = (int64_t)(cw & 0x3FFFFFFFu);
                    float x;
                    if (row_wz[rr] || (cw & 0x80000000u)) x = (i == j) ? 1.0f : 0.0f;
                    else if (row_dead[rr] || (cw & 0x40000000u)) x = (pi[rr] == pj) ? 1.0f : 0.0f;
                    else x = row[(int64_t)rr * C + pj];
                    if (i == j) x += dmp;
                    v[e] = x;
                }
                *reinterpret_cast<float4 *>(A + (int64_t)b * C * C + (C - 1 - i) * C + jo) =
                    make_float4(v[0], v[1], v[2], v[3]);
            }
        }
        return;
    }
    for (int64_t jo = threadIdx.x; jo < C; jo += blockDim.x) {
        const int64_t j = C - 1 - jo;  // output column jo of the reversed matrix <-> position j
        const uint32_t cw = code[j];
        const bool col_wz = (cw & 0x80000000u) != 0u, col_dead = (cw & 0x40000000u) != 0u;
        const int64_t pj = (int64_t)(cw & 0x3FFFFFFFu);
#pragma unroll
        for (int rr = 0; rr < kGdRows; ++rr) {
            if (!row_in[rr]) continue;
            const int64_t i = i0 + rr;
            float v;
            if (row_wz[rr] || col_wz) v = (i == j) ? 1.0f : 0.0f;
            else if (row_dead[rr] || col_dead) v = (pi[rr] == pj) ? 1.0f : 0.0f;
            else v = row[(int64_t)rr * C + pj];
            if (i == j) v += dmp;
            A[(int64_t)b * C * C + (C - 1 - i) * C + jo] = v;
            if (Hp_out) Hp_out[(int64_t)b * C * C + i * C + j] = v;
        }
    }
}

// The streaming form of the gather for permuted matrices (C a multiple of 4, no Hp output): persistent CTAs, each
// walking a contiguous run of (matrix, group of R rows) items.  The column codes of a matrix are gathered once per
// run of items of that matrix; the rows of item n+1 arrive by bulk copies while item n is written, so every SM keeps
// 4RC bytes of reads in flight behind its stores.
constexpr int kGsThreads = 512;
constexpr int kGsMaxRows = 12;
__global__ void __launch_bounds__(kGsThreads, 1)
gather_damp_stream_kernel(const float *__restrict__ H, int64_t C, const int32_t *__restrict__ perm,
                          const uint8_t *__restrict__ pruned, const uint8_t *__restrict__ wzero,
                          const int32_t *__restrict__ invalid, const float *__restrict__ damp,
                          float *__restrict__ A, int R, int64_t n_groups, int64_t total_items) {
    extern __shared__ __align__(16) float gs_smem[];   // [C] codes, then [2][R][C] rows
    __shared__ __align__(8) uint64_t gs_bar[2];
    __shared__ int gs_abort;
    uint32_t *code = reinterpret_cast<uint32_t *>(gs_smem);
    float *rows = gs_smem + C;
    const int64_t per = (total_items + gridDim.x - 1) / gridDim.x;
    const int64_t it0 = (int64_t)blockIdx.x * per, it1 = min(total_items, it0 + per);
    if (it0 >= it1) return;
    if (threadIdx.x == 0) {
        gs_abort = 0;
        forge::tc::mbar_init(forge::tc::smem_u32(&gs_bar[0]), 1);
        forge::tc::mbar_init(forge::tc::smem_u32(&gs_bar[1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    int64_t cur_b = -1;
    // code word of row position i of matrix b: source row in the low 30 bits, bit 31 = all-zero weight column at i,
    // bit 30 = dead channel (or a matrix flagged invalid): either bit means "nothing to load, an identity row"
    auto row_code = [&](int64_t b, int64_t i, bool inv) -> uint32_t {
        uint32_t cw;
        if (b == cur_b) cw = code[i];
        else {
            const uint32_t pi = (uint32_t)perm[b * C + i];
            cw = pi;
            if (wzero && wzero[b * C + i]) cw |= 0x80000000u;
            if (pruned && pruned[b * C + pi]) cw |= 0x40000000u;
        }
        return inv ? (cw | 0x40000000u) : cw;
    };
    // thread 0: start the row copies of item `it` into buffer `s`
    auto issue = [&](int64_t it, int s) {
        const int64_t b = it / n_groups, g = it - b * n_groups;
        const bool inv = invalid ? invalid[b] != 0 : false;
        const float *Hb = H + b * C * C;
        const uint32_t bar = forge::tc::smem_u32(&gs_bar[s]);
        uint32_t bytes = 0;
        constexpr uint32_t kPiece = 8192;
        for (int rr = 0; rr < R; ++rr) {
            const int64_t i = g * R + rr;
            if (i >= C) break;
            const uint32_t cw = row_code(b, i, inv);
            if (cw & 0xC0000000u) continue;
            const char *src = reinterpret_cast<const char *>(Hb + (int64_t)cw * C);
            const uint32_t dst = forge::tc::smem_u32(rows + ((int64_t)s * R + rr) * C);
            for (uint32_t off = 0; off < (uint32_t)(C * 4); off += kPiece)
                forge::tc::bulk_copy_g2s(dst + off, src + off, min(kPiece, (uint32_t)(C * 4) - off), bar);
            bytes += (uint32_t)(C * 4);
        }
        // the phase completes when this arrival AND the announced bytes are in (the byte count may run ahead of its
        // announcement)
        forge::tc::mbar_arrive_expect_tx(bar, bytes);
    };
    if (threadIdx.x == 0) issue(it0, 0);
    for (int64_t it = it0; it < it1; ++it) {
        const int s = (int)((it - it0) & 1);
        const uint32_t parity = (uint32_t)(((it - it0) >> 1) & 1);
        const int64_t b = it / n_groups, g = it - b * n_groups;
        if (b != cur_b) {
            // every thread has left the previous item's output loop (the barrier that ends an iteration)
            const int32_t *pb = perm + b * C;
            const uint8_t *prb = pruned ? pruned + b * C : nullptr;
            const uint8_t *wzb = wzero ? wzero + b * C : nullptr;
            for (int64_t j = threadIdx.x; j < C; j += blockDim.x) {
                const uint32_t pj = (uint32_t)__ldg(pb + j);
                uint32_t cw = pj;
                if (wzb && __ldg(wzb + j)) cw |= 0x80000000u;
                if (prb && __ldg(prb + pj)) cw |= 0x40000000u;
                code[j] = cw;
            }
            __syncthreads();
            cur_b = b;
        }
        if (threadIdx.x == 0 && it + 1 < it1) issue(it + 1, s ^ 1);
        const bool inv = invalid ? invalid[b] != 0 : false;
        const float dmp = damp[b];
        float *buf = rows + (int64_t)s * R * C;
        const bool ok = forge::tc::mbar_wait(forge::tc::smem_u32(&gs_bar[s]), parity, &gs_abort);
        if (__syncthreads_or(ok ? 0 : 1)) {
            // a bounded wait ran out: one more bounded wait, so that no copy into this buffer is left in flight, then
            // fetch this item's rows by plain loads
            volatile int again = 0;
            forge::tc::mbar_wait(forge::tc::smem_u32(&gs_bar[s]), parity, &again);
            for (int rr = 0; rr < R; ++rr) {
                const int64_t i = g * R + rr;
                if (i >= C) break;
                const uint32_t cw = row_code(b, i, inv);
                if (cw & 0xC0000000u) continue;
                const float *src = H + b * C * C + (int64_t)cw * C;
                for (int64_t c = threadIdx.x; c < C; c += blockDim.x) buf[(int64_t)rr * C + c] = src[c];
            }
            __syncthreads();
        }
        // rows outermost: a row's facts (source row, dead / zero flags, output pointer) are set up once; the inner loop
        // handles four output columns per thread with 32-bit indices, and takes a short cut when none of the four
        // column codes carries a flag (the usual case): four shared-memory reads, one 16-byte store
        const int Ci = (int)C;
        for (int rr = 0; rr < R; ++rr) {
            const int i = (int)(g * R) + rr;
            if (i >= Ci) break;
            const uint32_t cwi = code[i] | (inv ? 0x40000000u : 0u);
            const bool row_wz = (cwi & 0x80000000u) != 0u, row_dead = (cwi & 0x40000000u) != 0u;
            const uint32_t pi = cwi & 0x3FFFFFFFu;
            const float *row = buf + (int64_t)rr * C;
            float *orow = A + b * C * C + (int64_t)(Ci - 1 - i) * C;
            const bool row_plain = !row_wz && !row_dead;
            for (int jo = (int)threadIdx.x * 4; jo < Ci; jo += (int)blockDim.x * 4) {
                const int jlo = Ci - 4 - jo;   // positions jlo+3 .. jlo <-> output columns jo .. jo+3
                const uint4 cq = *reinterpret_cast<const uint4 *>(code + jlo);
                float4 v;
                if (row_plain && ((cq.x | cq.y | cq.z | cq.w) & 0xC0000000u) == 0u) {
                    v = make_float4(row[cq.w], row[cq.z], row[cq.y], row[cq.x]);
                } else {
                    const uint32_t cws[4] = {cq.w, cq.z, cq.y, cq.x};
                    float x[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = jlo + 3 - e;
                        const uint32_t cw = cws[e];
                        const uint32_t pj = cw & 0x3FFFFFFFu;
                        if (row_wz || (cw & 0x80000000u)) x[e] = (i == j) ? 1.0f : 0.0f;
                        else if (row_dead || (cw & 0x40000000u)) x[e] = (pi == pj) ? 1.0f : 0.0f;
                        else x[e] = row[pj];
                    }
                    v = make_float4(x[0], x[1], x[2], x[3]);
                }
                const int d = i - jlo;         // the diagonal position j == i is element 3 - d of this group
                if ((unsigned)d < 4u) {
                    if (d == 3) v.x += dmp; else if (d == 2) v.y += dmp; else if (d == 1) v.z += dmp; else v.w += dmp;
                }
                *reinterpret_cast<float4 *>(orow + jo) = v;
            }
        }
        __syncthreads();   // the buffer and (at a change of matrix) the code table are free again
    }
}

extern "C" int forge_hessian_gather_damp(const float *H, int nb, int64_t C, const int32_t *perm,
                                         const uint8_t *pruned, const uint8_t *wzero, const int32_t *invalid,
                                         float rel_damp, float *A, float *Hp_out, float *damp_out, void *stream) {
    FORGE_REQUIRE(H && A && damp_out, "null pointer");
    FORGE_REQUIRE(nb > 0 && C > 0, "empty batch");
    FORGE_REQUIRE(C * 4 * (kGdRows + 1) <= 200 * 1024, "C too large for the row staging buffer");
    FORGE_REQUIRE(A != H, "A must not alias H");
    FORGE_REQUIRE(C < (1 << 30), "C too large for the column codes");
    cudaStream_t st = (cudaStream_t)stream;
    damp_kernel<<<nb, 256, 0, st>>>(H, C, perm, pruned, wzero, invalid, rel_damp, damp_out); FORGE_NOTE_LAUNCH();
    const int64_t fit = ((int64_t)216 * 1024 / (C * 4) - 1) / 2;    // rows per buffer with codes + two buffers resident
    if (perm && !Hp_out && (C & 3) == 0 && fit >= 1) {
        const int R = (int)(fit < kGsMaxRows ? fit : (int64_t)kGsMaxRows);
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int64_t n_groups = cdiv(C, (int64_t)R), total = n_groups * nb;
        const size_t smem_stream = (size_t)C * 4 * (2 * R + 1);
        cudaFuncSetAttribute(gather_damp_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024);
        gather_damp_stream_kernel<<<(unsigned)(total < sms ? total : (int64_t)sms), kGsThreads, smem_stream, st>>>(
            H, C, perm, pruned, wzero, invalid, damp_out, A, R, n_groups, total);
        FORGE_NOTE_LAUNCH();
        return check_launch("forge_hessian_gather_damp");
    }
    const size_t smem = (size_t)C * 4 * (kGdRows + 1);
    // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute: set it on the device that is
    // current for this call (a process-wide "done" flag would leave a second GPU without it)
    cudaFuncSetAttribute(gather_damp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    gather_damp_kernel<<<dim3((unsigned)cdiv(C, kGdRows), nb), 256, smem, st>>>(H, C, perm, pruned, wzero, invalid,
                                                                              damp_out, A, Hp_out);
    FORGE_NOTE_LAUNCH();
    return check_launch("forge_hessian_gather_damp");
}

// --------------------------------------------------------------------------------------------
// Packed-int4 checkpoint weights (compressed-tensors "pack-quantized", e.g. Kimi-K2) -> dense:
//   out[o, i] = dtype( fp32(nibble) * sf[o, i / gs] ),  nibble i%8 of packed[o, i/8] at bits [4(i%8), +4),
//   two's-complement int4 when `symmetric`, unsigned otherwise; sf = scale, or 1/scale when scale_is_inv.
// Restates _apply_block_scale, forge/utils/io.py:722-808 (bits = 4, scales [O, I/gs]) on the device.
// One thread per packed word: 4 B in, 8 outputs (16 B of bf16) out.
// --------------------------------------------------------------------------------------------
__global__ void int4_packed_dequant_kernel(const int32_t *__restrict__ packed, const float *__restrict__ scales,
                                           int64_t O, int64_t I, int gs, int symmetric, int scale_is_inv,
                                           void *__restrict__ out, int out_dtype) {
    const int64_t IP = I / 8, total = O * IP;
    const int G = (int)(I / gs);
    const bool one_scale = (gs % 8) == 0;     // the eight values of a word share a group (the usual case)
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = w / IP;
        const int i0 = (int)(w - o * IP) * 8;
        const uint32_t word = (uint32_t)packed[w];
        const float *srow = scales + o * G;
        float sf0 = srow[i0 / gs];
        if (scale_is_inv) sf0 = __fdiv_rn(1.0f, sf0);
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            int u = (int)((word >> (4 * e)) & 0xFu);
            if (symmetric && u >= 8) u -= 16;
            float sf = sf0;
            if (!one_scale) {
                sf = srow[(i0 + e) / gs];
                if (scale_is_inv) sf = __fdiv_rn(1.0f, sf);
            }
            v[e] = __fmul_rn((float)u, sf);
        }
        if (out_dtype == FORGE_DTYPE_BF16) {
            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(out) + o * I + i0;
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
            pk.x = *reinterpret_cast<uint32_t *>(&h0); pk.y = *reinterpret_cast<uint32_t *>(&h1);
            pk.z = *reinterpret_cast<uint32_t *>(&h2); pk.w = *reinterpret_cast<uint32_t *>(&h3);
            *reinterpret_cast<uint4 *>(dst) = pk;
        } else {
            float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + o * I + i0);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
}
// The same for the usual checkpoint layout (bf16 output, every word inside one group).  A CTA walks a run of whole
// rows with 32-bit indices (the 64-bit division per word of the kernel above costs more issue slots than the memory
// system leaves); a thread keeps FOUR words in flight, taken 256 words apart, so that a warp's loads are whole 128-byte
// lines and its stores whole 512-byte runs.
constexpr int kI4Rows = 16;     // rows per CTA
__global__ void __launch_bounds__(256) int4_packed_dequant_vec4_kernel(const int32_t *__restrict__ packed,
                                                                       const float *__restrict__ scales, int64_t O,
                                                                       int64_t I, int gs, int symmetric,
                                                                       int scale_is_inv,
                                                                       __nv_bfloat16 *__restrict__ out) {
    const uint32_t IP = (uint32_t)(I / 8), G = (uint32_t)(I / gs), gw = (uint32_t)(gs / 8);   // words per row / group
    const int64_t row0 = (int64_t)blockIdx.x * kI4Rows;
    const uint32_t nrows = (uint32_t)imin64(kI4Rows, O - row0);
    const uint32_t total = nrows * IP;
    const int32_t *src = packed + row0 * IP;
    const float *srow = scales + row0 * G;
    __nv_bfloat16 *dst = out + row0 * I;
    for (uint32_t w0 = threadIdx.x; w0 < total; w0 += 4 * 256) {
        uint32_t word[4], r[4], c[4];
        float sf[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t w = w0 + q * 256;
            const bool ok = w < total;
            r[q] = ok ? w / IP : 0u;
            c[q] = ok ? w - r[q] * IP : 0u;
            word[q] = ok ? (uint32_t)__ldg(src + w) : 0u;
            sf[q] = ok ? __ldg(srow + r[q] * G + c[q] / gw) : 1.0f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (w0 + q * 256 >= total) break;
            const float s1 = scale_is_inv ? __fdiv_rn(1.0f, sf[q]) : sf[q];
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                int u = (int)((word[q] >> (4 * e)) & 0xFu);
                if (symmetric && u >= 8) u -= 16;
                v[e] = __fmul_rn((float)u, s1);
            }
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
            pk.x = *reinterpret_cast<uint32_t *>(&h0); pk.y = *reinterpret_cast<uint32_t *>(&h1);
            pk.z = *reinterpret_cast<uint32_t *>(&h2); pk.w = *reinterpret_cast<uint32_t *>(&h3);
            *reinterpret_cast<uint4 *>(dst + (int64_t)r[q] * I + (int64_t)c[q] * 8) = pk;
        }
    }
}
extern "C" int forge_int4_packed_dequant(const int32_t *packed, const float *scales, int64_t O, int64_t I, int gs,
                                         int symmetric, int scale_is_inv, void *out, int out_dtype, void *stream) {
    FORGE_REQUIRE(packed && scales && out, "null pointer");
    FORGE_REQUIRE(O > 0 && I > 0 && gs > 0, "bad sizes");
    FORGE_REQUIRE(I % 8 == 0 && I % gs == 0, "I must be a multiple of 8 and of the group size");
    FORGE_REQUIRE(out_dtype == FORGE_DTYPE_F32 || out_dtype == FORGE_DTYPE_BF16, "bad dtype");
    FORGE_REQUIRE((uintptr_t)out % 16 == 0, "output must be 16-byte aligned");
    if (out_dtype == FORGE_DTYPE_BF16 && gs % 8 == 0 && I / 8 * kI4Rows < (1ll << 31) && cdiv(O, (int64_t)kI4Rows) < (1ll << 31)) {
        const int blocks4 = (int)cdiv(O, (int64_t)kI4Rows);
        int4_packed_dequant_vec4_kernel<<<blocks4, 256, 0, (cudaStream_t)stream>>>(
            packed, scales, O, I, gs, symmetric, scale_is_inv, reinterpret_cast<__nv_bfloat16 *>(out));
        FORGE_NOTE_LAUNCH();
        return check_launch("forge_int4_packed_dequant");
    }
    const int blocks = (int)imin64(cdiv(O * (I / 8), 256), 148 * 64);
    int4_packed_dequant_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(packed, scales, O, I, gs, symmetric,
                                                                        scale_is_inv, out, out_dtype); FORGE_NOTE_LAUNCH();
    return check_launch("forge_int4_packed_dequant");
}

// --------------------------------------------------------------------------------------------
// MXFP4 checkpoint weights (gpt-oss: 16-byte blocks of 32 E2M1 codes + one E8M0 scale byte) -> dense, transposed:
//   blocks [rows, NB, 16] u8, scales [rows, NB] u8  ->  out [NB*32, rows]:
//   code 2k = low nibble of byte k, code 2k+1 = its high nibble; value = +-{0, .5, 1, 1.5, 2, 3, 4, 6}[code & 7];
//   scale = 2^(e - 127), and 2^-23 for e == 0;  out[nb*32 + c, row] = dtype(value * scale).
// Restates _dequant_mxfp4_blocks_to_fp / _e8m0_to_scale_fp32, forge/utils/io.py:505-531 (including its final
// transpose of the last two dimensions).  A CTA converts a [64 rows] x [4 blocks = 128 codes] tile through shared
// memory: 16-byte block reads (four neighbouring blocks = 64 contiguous bytes), transposed writes of 64 rows each.
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mxfp4_dequant_kernel(const uint8_t *__restrict__ blocks,
                                                            const uint8_t *__restrict__ scales, int64_t rows, int64_t NB,
                                                            void *__restrict__ out, int out_dtype) {
    // tile: 64 rows x 4 blocks (128 output columns), tile[code * 4 + block][row]; with a pitch of 72 floats the 32
    // lanes of a writing warp (8 rows x 4 blocks) hit 32 different banks, and the 8-byte reads below stay aligned
    __shared__ __align__(8) float tile[128][72];
    // signed E2M1 values by 4-bit code; sixteen words in sixteen banks, so any mix of lookups is conflict-free
    __shared__ float lut[16];
    const int tid = threadIdx.x;
    if (tid < 16) {
        const int m = tid & 7;
        const float mag = (m < 2) ? 0.5f * (float)m : __int_as_float(((126 + (m >> 1)) << 23) | ((m & 1) << 22));
        lut[tid] = (tid & 8) ? -mag : mag;
    }
    __syncthreads();
    const int64_t nb0 = (int64_t)blockIdx.x * 4, r0 = (int64_t)blockIdx.y * 64;
    {
        // read: thread -> (row = tid / 4, block = tid % 4): one 16-byte block and its scale byte
        const int rr = tid >> 2, bb = tid & 3;
        const int64_t row = r0 + rr, nb = nb0 + bb;
        if (row < rows && nb < NB) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(blocks + (row * NB + nb) * 16);
            const int e = scales[row * NB + nb];
            // 2^(e-127) is the fp32 whose exponent field is e (e = 255 gives +inf, as 2^128 does in fp32)
            const float sc = (e == 0) ? 1.1920928955078125e-07f : __int_as_float(e << 23);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const uint32_t byte = (words[k >> 2] >> (8 * (k & 3))) & 0xFFu;
                const int lo = (int)(byte & 0xFu), hi = (int)(byte >> 4);
                const float vlo = lut[lo], vhi = lut[hi];
                tile[(2 * k) * 4 + bb][rr] = __fmul_rn(vlo, sc);
                tile[(2 * k + 1) * 4 + bb][rr] = __fmul_rn(vhi, sc);
            }
        }
    }
    __syncthreads();
    // write: warp w takes columns w, w + 8, ...; a lane writes rows 2 lane, 2 lane + 1 (128 B of bf16 per warp)
    const int warp = tid >> 5, lane = tid & 31;
    const bool pair_ok = (rows & 1) == 0;
    for (int c = warp; c < 128; c += 8) {
        const int64_t nb = nb0 + (c & 3);
        if (nb >= NB) continue;
        const int64_t col = nb * 32 + (c >> 2);
        const int64_t row = r0 + 2 * lane;
        const float2 vv = *reinterpret_cast<const float2 *>(&tile[c][2 * lane]);
        const float v0 = vv.x, v1 = vv.y;
        if (out_dtype == FORGE_DTYPE_BF16) {
            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(out) + col * rows + row;
            if (pair_ok && row + 1 < rows) {
                *reinterpret_cast<__nv_bfloat162 *>(dst) = __floats2bfloat162_rn(v0, v1);
            } else {
                if (row < rows) dst[0] = __float2bfloat16_rn(v0);
                if (row + 1 < rows) dst[1] = __float2bfloat16_rn(v1);
            }
        } else {
            float *dst = reinterpret_cast<float *>(out) + col * rows + row;
            if (pair_ok && row + 1 < rows) {
                *reinterpret_cast<float2 *>(dst) = make_float2(v0, v1);
            } else {
                if (row < rows) dst[0] = v0;
                if (row + 1 < rows) dst[1] = v1;
            }
        }
    }
}
extern "C" int forge_mxfp4_dequant(const uint8_t *blocks, const uint8_t *scales, int64_t rows, int64_t NB, void *out,
                                   int out_dtype, void *stream) {
    FORGE_REQUIRE(blocks && scales && out, "null pointer");
    FORGE_REQUIRE(rows > 0 && NB > 0 && NB < 65536 * 32, "bad sizes");
    FORGE_REQUIRE(out_dtype == FORGE_DTYPE_F32 || out_dtype == FORGE_DTYPE_BF16, "bad dtype");
    FORGE_REQUIRE(cdiv(rows, 64) <= 65535, "too many rows for one launch");
    FORGE_REQUIRE((uintptr_t)blocks % 16 == 0 && (uintptr_t)out % 8 == 0, "blocks must be 16-byte aligned");
    dim3 grid((unsigned)cdiv(NB, 4), (unsigned)cdiv(rows, 64));
    mxfp4_dequant_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(blocks, scales, rows, NB, out, out_dtype); FORGE_NOTE_LAUNCH();
    return check_launch("forge_mxfp4_dequant");
}

// --------------------------------------------------------------------------------------------
// de-quantise codes: out = (q - q0) * s in fp32   (forge/utils/engine.py:93-96)
// --------------------------------------------------------------------------------------------
__global__ void dequant_kernel(const uint8_t *__restrict__ q, const float *__restrict__ scales,
                               const float *__restrict__ qzeros, int64_t rows, int64_t C, int gs, int64_t G,
                               void *__restrict__ out, int out_dtype) {
    const int64_t total = rows * C;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = e / C, c = e % C;
        const int64_t g = r * G + c / gs;
        const float w = ((float)q[e] - qzeros[g]) * scales[g];
        if (out_dtype == FORGE_DTYPE_BF16) reinterpret_cast<__nv_bfloat16 *>(out)[e] = __float2bfloat16_rn(w);
        else reinterpret_cast<float *>(out)[e] = w;
    }
}
extern "C" int forge_dequantize(const uint8_t *q, const float *scales, const float *qzeros, int64_t rows,
                                int64_t C, int gs, void *out, int out_dtype, void *stream) {
    FORGE_REQUIRE(q && scales && qzeros && out, "null pointer");
    FORGE_REQUIRE(rows > 0 && C > 0 && gs > 0, "bad sizes");
    const int64_t G = cdiv(C, gs);
    const int blocks = (int)imin64(cdiv(rows * C, 256), 148 * 32);
    dequant_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, scales, qzeros, rows, C, gs, G, out, out_dtype); FORGE_NOTE_LAUNCH();
    return check_launch("forge_dequantize");
}

// --------------------------------------------------------------------------------------------
// dense int4 packer.  Fast path (C and gs multiples of 16, 16-byte aligned rows): one thread per 16 codes — one
// 16-byte load, one zero point (the 16 codes share a group), two packed words in one 8-byte store.  General path:
// one thread per output word (8 codes), every code with its own group index.
// --------------------------------------------------------------------------------------------
constexpr int kP4Rows = 16;     // rows per CTA
__global__ void __launch_bounds__(256) pack_int4_vec16_kernel(const uint8_t *__restrict__ q,
                                                              const float *__restrict__ qzeros, int64_t rows, int C16,
                                                              int gs16, int G, int32_t *__restrict__ packed) {
    // a CTA walks a run of whole rows with 32-bit indices; a thread keeps four 16-code chunks in flight, 256 chunks
    // apart (a warp's loads are whole 512-byte runs, its stores whole 256-byte runs)
    const int64_t row0 = (int64_t)blockIdx.x * kP4Rows;
    const uint32_t nrows = (uint32_t)imin64(kP4Rows, rows - row0);
    const uint32_t total = nrows * (uint32_t)C16;
    const uint4 *src = reinterpret_cast<const uint4 *>(q) + row0 * C16;
    const float *zrow = qzeros + row0 * G;
    uint2 *dst = reinterpret_cast<uint2 *>(packed) + row0 * C16;
    for (uint32_t w0 = threadIdx.x; w0 < total; w0 += 4 * 256) {
        uint4 raw[4];
        int z[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t w = w0 + k * 256;
            const bool ok = w < total;
            const uint32_t r = ok ? w / (uint32_t)C16 : 0u;
            const uint32_t j = ok ? w - r * (uint32_t)C16 : 0u;
            raw[k] = ok ? __ldg(src + w) : make_uint4(0u, 0u, 0u, 0u);
            z[k] = ok ? (int)__ldg(zrow + r * (uint32_t)G + j / (uint32_t)gs16) : 0;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (w0 + k * 256 >= total) break;
            const uint32_t in[4] = {raw[k].x, raw[k].y, raw[k].z, raw[k].w};
            uint32_t out[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t acc = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int b = (int)((in[2 * h + (i >> 2)] >> (8 * (i & 3))) & 0xFFu);
                    // int8(code) - int8(zero) + 8, taken as a byte, shifted in: additions carry like pack_to_int32's sum
                    const uint32_t u = (uint32_t)(uint8_t)(int8_t)((int8_t)(int8_t)b - (int8_t)z[k] + 8);
                    acc += u << (4 * i);
                }
                out[h] = acc;
            }
            dst[w0 + k * 256] = make_uint2(out[0], out[1]);
        }
    }
}

__global__ void pack_int4_kernel(const uint8_t *__restrict__ q, const float *__restrict__ qzeros, int64_t rows,
                                 int64_t C, int gs, int64_t G, int64_t CP, int32_t *__restrict__ packed,
                                 int aligned8) {
    const int64_t total = rows * CP;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total;
         w += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = w / CP, j = w % CP;
        const int64_t c0 = j * 8;
        uint8_t b[8];
        if (aligned8 && c0 + 8 <= C) {
            const uint2 raw = *reinterpret_cast<const uint2 *>(q + r * C + c0);
            *reinterpret_cast<uint2 *>(b) = raw;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) b[i] = (c0 + i < C) ? q[r * C + c0 + i] : 0;
        }
        uint32_t acc = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (c0 + i < C) {
                const int8_t z = (int8_t)(int)qzeros[r * G + (c0 + i) / gs];
                const int8_t v = (int8_t)((int8_t)b[i] - z);
                const uint8_t u = (uint8_t)(int8_t)(v + 8);
                acc += ((uint32_t)u) << (4 * i);
            }
        }
        packed[w] = (int32_t)acc;
    }
}
extern "C" int forge_pack_int4(const uint8_t *q, const float *qzeros, int64_t rows, int64_t C, int gs,
                               int32_t *packed, void *stream) {
    FORGE_REQUIRE(q && qzeros && packed, "null pointer");
    FORGE_REQUIRE(rows > 0 && C > 0 && gs > 0, "bad sizes");
    const int64_t G = cdiv(C, gs), CP = cdiv(C, 8);
    if (C % 16 == 0 && gs % 16 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)packed % 8 == 0 && C / 16 < (1 << 26) &&
        cdiv(rows, (int64_t)kP4Rows) < (1ll << 31)) {
        const int blocks = (int)cdiv(rows, (int64_t)kP4Rows);
        pack_int4_vec16_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, qzeros, rows, (int)(C / 16), gs / 16, (int)G,
                                                                         packed);
        FORGE_NOTE_LAUNCH();
        return check_launch("forge_pack_int4");
    }
    const int aligned8 = (C % 8 == 0) && ((uintptr_t)q % 8 == 0);
    const int blocks = (int)imin64(cdiv(rows * CP, 256), 148 * 32);
    pack_int4_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, qzeros, rows, C, gs, G, CP, packed, aligned8); FORGE_NOTE_LAUNCH();
    return check_launch("forge_pack_int4");
}

// --------------------------------------------------------------------------------------------
// sparse 1:4 packer.  One thread per (pair of 32-column groups, row); rows are the fast index so
// that M, scales and the 16-byte output are coalesced.  Each 4-column group of the row is one
// 32-bit word of codes, so the kept code is a byte select inside a register.
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t pack_one_group(const uint32_t words[8], uint32_t bitmask, float scale,
                                                   int64_t col0, int64_t C) {
    uint32_t idx16 = 0, qw32 = 0x88888888u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t sub = (bitmask >> (4 * i)) & 0xFu;
        if (sub == 0u) continue;
        const int c = __ffs(sub) - 1;
        idx16 |= (uint32_t)(c & 3) << (2 * i);
        if (col0 + i * 4 + c < C) {
            const uint32_t qv = (words[i] >> (8 * c)) & 0xFu;
            qw32 = (qw32 & ~(0xFu << (4 * i))) | (qv << (4 * i));
        }
    }
    const __nv_bfloat16 sb = __float2bfloat16_rn(scale);
    const uint16_t sbits = *reinterpret_cast<const uint16_t *>(&sb);
    return ((uint64_t)sbits << 48) | ((uint64_t)(idx16 & 0xFFFFu) << 32) | (uint64_t)qw32;
}

__global__ void pack_sparse14_kernel(const uint8_t *__restrict__ q, const uint32_t *__restrict__ M,
                                     const float *__restrict__ scales, int64_t R, int64_t C, int64_t G32,
                                     int64_t G2, ulonglong2 *__restrict__ out, int vec_ok) {
    // blockIdx.y = matrix of the batch
    q += (int64_t)blockIdx.y * R * C;
    M += (int64_t)blockIdx.y * G32 * R;
    scales += (int64_t)blockIdx.y * G32 * R;
    out += (int64_t)blockIdx.y * G2 * R;
    const int64_t total = G2 * R;
    for (int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; tid < total;
         tid += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = tid % R, g2 = tid / R;
        ulonglong2 o;
        uint64_t halves[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t gid = 2 * g2 + h;
            if (gid >= G32) { halves[h] = 0ull; continue; }
            const int64_t col0 = gid * 32;
            uint32_t words[8];
            if (vec_ok && col0 + 32 <= C) {
                const uint4 *src = reinterpret_cast<const uint4 *>(q + r * C + col0);
                const uint4 a = src[0], bq = src[1];
                words[0] = a.x; words[1] = a.y; words[2] = a.z; words[3] = a.w;
                words[4] = bq.x; words[5] = bq.y; words[6] = bq.z; words[7] = bq.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint32_t w = 0;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int64_t cid = col0 + i * 4 + c;
                        if (cid < C) w |= (uint32_t)q[r * C + cid] << (8 * c);
                    }
                    words[i] = w;
                }
            }
            halves[h] = pack_one_group(words, M[gid * R + r], scales[gid * R + r], col0, C);
        }
        o.x = halves[0];
        o.y = halves[1];
        out[g2 * R + r] = o;
    }
}
extern "C" int forge_pack_sparse14(const uint8_t *q, const uint32_t *M, const float *scales32, int64_t R,
                                   int64_t C, uint64_t *out, void *stream) {
    FORGE_REQUIRE(q && M && scales32 && out, "null pointer");
    FORGE_REQUIRE(R > 0 && C > 0, "bad sizes");
    FORGE_REQUIRE((uintptr_t)out % 16 == 0, "output must be 16-byte aligned");
    const int64_t G32 = cdiv(C, 32), G2 = (G32 + 1) >> 1;
    const int vec_ok = (C % 16 == 0) && ((uintptr_t)q % 16 == 0);
    const int blocks = (int)imin64(cdiv(G2 * R, 256), 148 * 32);
    pack_sparse14_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q, M, scales32, R, C, G32, G2,
                                                                 (ulonglong2 *)out, vec_ok); FORGE_NOTE_LAUNCH();
    return check_launch("forge_pack_sparse14");
}

extern "C" int forge_pack_sparse14_batched(const uint8_t *q, const uint32_t *M, const float *scales32, int nb, int64_t R,
                                           int64_t C, uint64_t *out, void *stream) {
    FORGE_REQUIRE(q && M && scales32 && out, "null pointer");
    FORGE_REQUIRE(nb > 0 && nb <= 65535 && R > 0 && C > 0, "bad sizes");
    FORGE_REQUIRE((uintptr_t)out % 16 == 0, "output must be 16-byte aligned");
    const int64_t G32 = cdiv(C, 32), G2 = (G32 + 1) >> 1;
    // every matrix of the batch starts R * C bytes after the previous one: 16-byte accesses need that to be a multiple
    const int vec_ok = (C % 16 == 0) && ((uintptr_t)q % 16 == 0) && ((R * C) % 16 == 0);
    const int per = (int)imin64(cdiv(G2 * R, 256), cdiv((int64_t)148 * 32, (int64_t)nb) + 1);
    pack_sparse14_kernel<<<dim3((unsigned)per, (unsigned)nb), 256, 0, (cudaStream_t)stream>>>(
        q, M, scales32, R, C, G32, G2, (ulonglong2 *)out, vec_ok);
    FORGE_NOTE_LAUNCH();
    return check_launch("forge_pack_sparse14_batched");
}
