// Layer reconstruction loss  || X W^T - X What^T ||_F^2  per matrix, What = (q - q0) * s, on the device.
//
// This is the acceptance quantity of the path (the reference prints it per layer as the relative
// error after writing the de-quantised weights back, quant.py:491-496 with forge/utils/engine.py:72-97);
// evaluating it on the GPU lets full-width layers (7168 input channels, thousands of routed tokens)
// be checked, which a host evaluation in double precision cannot do in reasonable time.
//
// Plain tiled FMA GEMM of the routed activations with D = W - What (formed on the fly from the weight,
// the codes and the per-group scale / zero), 64 tokens x 64 weight rows per CTA step, fp32 dot products,
// squares summed in double.  A check, not a hot kernel: no tensor cores on purpose (D is not
// bf16-representable and the point is an independent number).
#include "common.cuh"

using namespace forge;

namespace {

constexpr int kT = 64, kR = 64, kK = 16;

struct ReconParams {
    const void *W;
    int w_dtype;
    const uint8_t *q;
    const float *scales, *qzeros;
    int gs;
    int64_t R, C, G;
    const __nv_bfloat16 *X;
    int64_t n_rows, ldx;
    const int32_t *token_idx;
    int64_t list_len;
    const int64_t *offsets;
    const int32_t *x_map;   // slot of (offsets) that matrix b reads, or null (= b)
    double *out;
    int32_t *status;
};

__global__ void __launch_bounds__(256) recon_loss_kernel(const ReconParams P) {
    __shared__ float xs[kK][kT + 1];
    __shared__ float ds[kK][kR + 1];
    __shared__ double red[8];
    const int b = blockIdx.z;
    const int slot = P.x_map ? P.x_map[b] : b;
    const int64_t off = P.offsets[slot], n = P.offsets[slot + 1] - off;
    if (!(off >= 0 && n >= 0 && off + n <= P.list_len)) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && P.status) atomicExch(P.status, FORGE_ERR_INVALID);
        return;
    }
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;   // tx: weight rows, ty: tokens
    const int64_t r0 = (int64_t)blockIdx.x * kR;
    const int32_t *tl = P.token_idx ? P.token_idx + off : nullptr;
    double part = 0.0;
    for (int64_t j0 = (int64_t)blockIdx.y * kT; j0 < n; j0 += (int64_t)gridDim.y * kT) {
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] = 0.0f;
        for (int64_t k0 = 0; k0 < P.C; k0 += kK) {
            // stage 64 tokens x 16 channels and 64 rows x 16 channels (4 elements of each per thread)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int e = tid + 256 * i;         // 0..1023
                const int kk = e & 15, rr = e >> 4;  // channel, token / row inside the tile
                const int64_t c = k0 + kk;
                float xv = 0.0f, dv = 0.0f;
                if (c < P.C) {
                    const int64_t j = j0 + rr;
                    if (j < n) {
                        const int64_t tok = tl ? (int64_t)tl[j] : off + j;
                        if (tok >= 0 && tok < P.n_rows) xv = __bfloat162float(P.X[tok * P.ldx + c]);
                        else if (P.status) atomicExch(P.status, FORGE_ERR_INVALID);
                    }
                    const int64_t r = r0 + rr;
                    if (r < P.R) {
                        const int64_t wi = ((int64_t)b * P.R + r) * P.C + c;
                        const int64_t gi = ((int64_t)b * P.R + r) * P.G + c / P.gs;
                        const float what = __fmul_rn(__fsub_rn((float)P.q[wi], P.qzeros[gi]), P.scales[gi]);
                        dv = ld_as_f32(P.W, P.w_dtype, wi) - what;
                    }
                }
                xs[kk][rr] = xv;
                ds[kk][rr] = dv;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < kK; ++kk) {
                float xv[4], dv[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) xv[a] = xs[kk][ty * 4 + a];
#pragma unroll
                for (int c = 0; c < 4; ++c) dv[c] = ds[kk][tx * 4 + c];
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[a][c] = fmaf(xv[a], dv[c], acc[a][c]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) part += (double)acc[a][c] * (double)acc[a][c];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) red[tid >> 5] = part;
    __syncthreads();
    if (tid == 0) {
        double s = 0.0;
        for (int w = 0; w < 8; ++w) s += red[w];
        if (s != 0.0) atomicAdd(P.out + b, s);
    }
}

__global__ void zero_doubles_kernel(double *p, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = 0.0;
}

}  // namespace

extern "C" int forge_recon_loss(const void *W, int w_dtype, const uint8_t *q, const float *scales, const float *qzeros,
                                int gs, int nb, int64_t R, int64_t C, const void *X_bf16, int64_t n_rows, int64_t ldx,
                                const int32_t *token_idx, int64_t list_len, const int64_t *offsets,
                                const int32_t *x_map, double *loss, int32_t *status, void *stream) {
    FORGE_REQUIRE(W && q && scales && qzeros && X_bf16 && offsets && loss, "null pointer");
    FORGE_REQUIRE(nb > 0 && R > 0 && C > 0 && gs > 0 && ldx >= C && n_rows >= 0, "bad sizes");
    FORGE_REQUIRE(w_dtype == FORGE_DTYPE_F32 || w_dtype == FORGE_DTYPE_BF16, "bad dtype");
    cudaStream_t st = (cudaStream_t)stream;
    ReconParams P{};
    P.W = W; P.w_dtype = w_dtype; P.q = q; P.scales = scales; P.qzeros = qzeros; P.gs = gs;
    P.R = R; P.C = C; P.G = cdiv(C, gs);
    P.X = (const __nv_bfloat16 *)X_bf16; P.n_rows = n_rows; P.ldx = ldx; P.token_idx = token_idx;
    P.list_len = token_idx ? list_len : n_rows; P.offsets = offsets; P.x_map = x_map; P.out = loss; P.status = status;
    zero_doubles_kernel<<<(nb + 127) / 128, 128, 0, st>>>(loss, nb); FORGE_NOTE_LAUNCH();
    // token tiles are walked with a stride: enough CTAs per matrix to fill the GPU even for a batch of one
    const int64_t row_tiles = cdiv(R, kR);
    int ty = (int)imin64(64, cdiv(148 * 8, row_tiles * nb));
    if (ty < 1) ty = 1;
    recon_loss_kernel<<<dim3((unsigned)row_tiles, (unsigned)ty, (unsigned)nb), 256, 0, st>>>(P); FORGE_NOTE_LAUNCH();
    return check_launch("forge_recon_loss");
}
