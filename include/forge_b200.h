/*
 * forge_b200 — C ABI of the sm_100a GPTQ / SparseGPT solver engine.
 *
 * Every entry point
 *   - is extern "C", takes plain device pointers, sizes and a CUDA stream
 *     (passed as void*; 0 = the legacy default stream),
 *   - returns FORGE_OK (0) or a FORGE_ERR_* code and never throws,
 *   - is asynchronous on `stream` and never synchronises the device,
 *   - allocates nothing: outputs and workspaces belong to the caller
 *     (forge_*_workspace_bytes() give the sizes).
 * forge_last_error() returns a per-thread description of the last failure.
 *
 * Citations name the reference interface each function replaces (paths inside
 * the reference project, Pranshu-Bahadur/4Bit-Forge).
 *
 * Notation: R = out_features, C = in_features, gs = group size,
 * G = ceil(C/gs), nb = matrices in the batch.
 */
#ifndef FORGE_B200_H
#define FORGE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FORGE_OK = 0,
    FORGE_ERR_INVALID = 1,     /* bad argument (null pointer, unsupported size) */
    FORGE_ERR_LAUNCH = 2,      /* CUDA reported an error at launch */
    FORGE_ERR_TIMEOUT = 3,     /* a bounded device-side wait ran out (status word) */
    FORGE_ERR_UNSUPPORTED = 4  /* shape / option outside what the kernels cover */
};

enum { FORGE_DTYPE_F32 = 0, FORGE_DTYPE_BF16 = 1 };

/* flags of forge_hessian_grouped */
enum {
    FORGE_HESS_MIRROR = 1,   /* also write the lower triangle (full symmetric H) */
    FORGE_HESS_SIMT = 2      /* plain-FMA validation kernel instead of tcgen05 */
};
/* flags of forge_expert_swiglu_grouped */
enum { FORGE_FWD_SIMT = 1 }; /* plain-FMA validation kernel instead of tcgen05 */
/* selection rule of forge_route_topk */
enum { FORGE_ROUTE_SOFTMAX = 0, FORGE_ROUTE_SIGMOID = 1, FORGE_ROUTE_SIGMOID_GROUPED = 2 };

int forge_version(void);
const char *forge_last_error(void);
/* number of kernels this library has launched in the calling process so far */
long long forge_launch_count(void);

/* ---- A0: DeepSeek fp8 block de-quantisation ------------------------------
 * out_bf16[o,i] = bf16( fp32(w_fp8_e4m3[o,i]) * scale_inv[o/so, i/si] ),
 * si = I/nI, so = si if ceil(O/si)==nO else ceil(O/nO).
 * Replaces forge/utils/io.py:533-563 (_apply_block_scale_inv_2d) and the fp8
 * branch of materialize_block_weights_to_fp, forge/utils/io.py:864-874. */
int forge_fp8_block_dequant(const void *w_fp8, const float *scale_inv, void *out_bf16,
                            int64_t O, int64_t I, int64_t nO, int64_t nI, void *stream);

/* ---- routing: router logits -> top-k expert ids -------------------------------
 * logits [T,E] fp32 -> topk_ids [T,k] int32 in descending score order (ties: lower expert id) and, when
 * topk_weights is not NULL, the scores of the chosen experts [T,k] (softmax probabilities / sigmoid scores).
 * mode FORGE_ROUTE_SOFTMAX / FORGE_ROUTE_SIGMOID: plain top-k.  FORGE_ROUTE_SIGMOID_GROUPED (DeepSeek-V3): the
 * experts form n_groups equal groups, a group scores the sum of its two best experts, only the topk_groups best
 * groups stay eligible.  bias [E] (may be NULL) is added to the sigmoid scores for the selection only.  E <= 1024.
 * The reference leaves this step to the HF MoE block's own forward (quant.py:398-406); the in-repo statement of
 * the selection it relies on is the fused-experts capture, forge/utils/engine.py:228-238. */
int forge_route_topk(const float *logits, const float *bias, int64_t T, int E, int k, int mode, int n_groups,
                     int topk_groups, int32_t *topk_ids, float *topk_weights, void *stream);

/* ---- routing: top-k ids -> per-expert token lists ------------------------
 * topk_ids [T,k] int32 (expert id per slot).  For the routed experts [e_begin, e_begin+e_count) followed by
 * dense_tail slots that see every token (shared experts) writes counts[e_count+dense_tail],
 * offsets[e_count+dense_tail+1] (exclusive prefix sum) and token_lists (token indices grouped by slot, ascending
 * inside each slot; capacity T*k + dense_tail*T).  Stands in for the gather the HF MoE block performs before each
 * expert's forward hook fires (quant.py:398-406; the in-repo statement is forge/utils/engine.py:228-238). */
int forge_route_build_lists(const int32_t *topk_ids, int64_t T, int k, int e_begin, int e_count, int dense_tail,
                            int32_t *counts, int64_t *offsets, int32_t *token_lists, void *stream);

/* ---- expert forward: the down-projection calibration input of every local expert --------
 * For slot b and j < n_b = offsets[b+1]-offsets[b], x = row token_idx[offsets[b]+j] of X (row offsets[b]+j when
 * token_idx is NULL):
 *   out[offsets[b]+j, :] = bf16( bf16(silu(bf16(x Wg[b]^T))) * bf16(x Wu[b]^T) )      (fp32 accumulation)
 * X bf16 [n_rows, ldx >= H]; Wg, Wu bf16 [nb, I, H]; out bf16 [out_rows, I], packed by slot.  One grouped
 * tcgen05 GEMM launch, gather fused into the load, SwiGLU in the epilogue.  H % 8 == 0.  Slots whose claim does
 * not fit the list, X or out are skipped and list entries that are not rows of X contribute zeros; the status
 * word then says FORGE_ERR_INVALID (FORGE_ERR_TIMEOUT: a bounded wait ran out).
 * Replaces the HF expert-module forward the reference hooks at down_proj (quant.py:398-406) and the fused-experts
 * recomputation of that input, forge/utils/engine.py:228-258. */
int forge_expert_swiglu_grouped(const void *X_bf16, int64_t n_rows, int64_t ldx, int64_t H, int64_t I,
                                const int32_t *token_idx, int64_t list_len, const int64_t *offsets, int nb,
                                const void *Wg_bf16, const void *Wu_bf16, void *out_bf16, int64_t out_rows,
                                int flags, int32_t *status, void *stream);

/* ---- A2: per-expert Hessian accumulation ---------------------------------
 * For b in [0,nb):  n = offsets[b+1]-offsets[b];  N = n_prev[b] + n;
 *   H[b] = (n_prev[b]/N) * H[b] + (2/N) * sum_{t in list b} x_t^T x_t   (n > 0)
 * x_t = row token_idx[offsets[b]+j] of X (bf16, row stride ldx elements), or
 * row offsets[b]+j when token_idx is NULL.  fp32 accumulation of exact bf16
 * products on the tcgen05 tensor cores.  n_prev may be NULL (= 0; H is then
 * overwritten, not read).  When n == 0 H[b] is left untouched.  n_prev is NOT
 * updated (forge_counts_add does that).  C must be a multiple of 8.
 * `status` (device int32, may be NULL) receives FORGE_ERR_TIMEOUT if a bounded
 * wait inside the kernel ran out, FORGE_ERR_INVALID if a bounds check failed.
 * Replaces GPTQ.update, forge/gptq.py:62-80 (H.addmm_ at :76-79).
 * Bounds: n_rows = rows of X, list_len = entries of token_idx (ignored when token_idx is NULL).  offsets lives in
 * device memory, so the kernel checks it: a slot whose claim offsets[b] .. offsets[b+1] does not fit in the token
 * list (in X, when the rows are contiguous) is skipped untouched, and a list entry that is not a row of X
 * contributes zeros; either way the status word becomes FORGE_ERR_INVALID and no out-of-bounds read happens.
 */
int forge_hessian_grouped(const void *X_bf16, int64_t n_rows, int64_t ldx, int64_t C, const int32_t *token_idx,
                          int64_t list_len, const int64_t *offsets, int nb, float *H, const int64_t *n_prev,
                          int flags, int32_t *status, void *stream);

/* Self-test of the bounded device-side wait used by every tensor-core kernel: a one-CTA kernel waits on a barrier
 * nothing arrives on for at most budget_cycles (<= 2e9), gives up, writes FORGE_ERR_TIMEOUT to *status (device int32)
 * and returns normally.  No counterpart in the reference (it has no device-side waits). */
int forge_selftest_bounded_wait(int32_t *status, int64_t budget_cycles, void *stream);

/* Diagnostic: cycles[0] (device int64) = clock cycles one thread needs to issue and complete `iters` back-to-back
 * tcgen05.mma kind::tf32 M128 x N x K8 (N = 64, 128 or 256; operands in shared memory — zeros, or pseudo-random values
 * with pattern != 0 —, accumulator in tensor memory), measured on SM 0 while every SM runs the same loop.  cycles / iters is the issue ceiling of the instruction
 * the solver and the Cholesky are built from; the benchmark reports its kernels against it.  The only wait in the
 * kernel is bounded (status = FORGE_ERR_TIMEOUT if it runs out).  No counterpart in the reference. */
int forge_selftest_mma_rate(int N, int iters, int pattern, int64_t *cycles, int32_t *status, void *stream);

/* n_prev[b] += offsets[b+1]-offsets[b]  (GPTQ.update's num_samples.add_, forge/gptq.py:80) */
int forge_counts_add(int64_t *n_prev, const int64_t *offsets, int nb, void *stream);

/* ---- A3: Hessian preparation ---------------------------------------------
 * forge_hessian_scan: for each b, invalid[b] = (n_samples[b]==0) or any NaN in
 * H[b]  (n_samples may be NULL = "has samples"); diag[b,c] = 1 if invalid or
 * H[b,c,c]==0 else H[b,c,c]; pruned[b,c] = !invalid && H[b,c,c]==0.
 * The caller sorts diag (descending) to get the activation order.
 * Replaces the checks of GPTQ._prep, forge/gptq.py:96-103. */
int forge_hessian_scan(const float *H, int nb, int64_t C, const int64_t *n_samples, float *diag,
                       uint8_t *pruned, int32_t *invalid, void *stream);

/* W[b,:,c] = 0 for every column c pruned in Hessian slot u_map[b] (u_map NULL = b); in place.
 * Replaces `self.W[:, self.pruned_ids] = 0`, forge/gptq.py:91,115,124. */
int forge_weight_apply_pruned(void *W, int w_dtype, int nb, int64_t R, int64_t C, const uint8_t *pruned,
                              const int32_t *u_map, void *stream);

/* wzero[b,c] = 1 iff column c of W[b] is all zero.
 * Replaces `self.W.clone().eq(0).all(dim=0)`, forge/gptq.py:145. */
int forge_weight_zero_cols(const void *W, int w_dtype, int nb, int64_t R, int64_t C, uint8_t *wzero,
                           void *stream);

/* forge_hessian_gather_damp: builds, per Hessian b, the matrix the factorisation consumes.
 *   H'  = I if invalid[b] else H[b] with pruned rows/cols zeroed and their diagonal set to 1
 *   Hp[i,j] = H'[perm[i], perm[j]]                       (perm NULL = identity)
 *   if wzero[b,i] or wzero[b,j]: Hp[i,j] = (i==j)        (indexed by POSITION i, as the reference does)
 *   damp = rel_damp * mean(diag Hp);  Hp[i,i] += damp
 *   A[b, C-1-i, C-1-j] = Hp[i,j]                         (index-reversed copy)
 * Hp_out (optional, [nb,C,C]) receives Hp itself; damp_out [nb] (required) receives damp.
 * A must not alias H.
 * Replaces the gather of GPTQ._prep (forge/gptq.py:117) and the damping of
 * GPTQ._h_factor (forge/gptq.py:145-154). */
int forge_hessian_gather_damp(const float *H, int nb, int64_t C, const int32_t *perm,
                              const uint8_t *pruned, const uint8_t *wzero, const int32_t *invalid,
                              float rel_damp, float *A, float *Hp_out, float *damp_out, void *stream);

/* ---- A4: batched Cholesky -> unit-diagonal upper factor of the inverse ---
 * A [nb,C,C] is the index-reversed damped Hessian from forge_hessian_gather_damp and is destroyed.
 * On return U[b] (fp32 [C,C]) is upper triangular with unit diagonal, U = diag(T)^-1 T where
 * T^T T = Hp^-1 (T upper, the reference's cholesky(cholesky_inverse(cholesky(Hp))), upper=True),
 * udiag[b,c] = T[c,c], and info[b] = 0, or > 0 when a pivot was not positive: then U[b] = I and
 * udiag = 1 (the reference's issue_non_invertible fallback).  With zero_lower != 0 the strict lower
 * triangle of U is zero-filled, otherwise it holds scratch values.
 * ws: forge_chol_workspace_bytes(nb, C) bytes.
 * Replaces GPTQ._h_factor, forge/gptq.py:156-177. */
int64_t forge_chol_workspace_bytes(int nb, int64_t C);
/* Inversion-free variant: factor only.  With J Hp J = L L^T (A = J Hp J on entry), V = J L J is upper with
 * Hp = V V^T and Vt = V diag(V)^-1 is the inverse of the reference's unit factor U.  On return the strict upper
 * triangle of A[b] holds -Vt, the diagonal 1 (the lower triangle is scratch), udiag[b,c] = 1 / V[c,c] (equal to
 * the diagonal of the reference's un-normalised factor), info as below.  A[b] is then the `U` operand of
 * forge_gptq_solve_batched with form = 1: x_t = w_t + sum_{s<t} (w_s - deq_s) Vt[s,t] is the reference's
 * recurrence x_t = w_t - sum_{s<t} err_s U[s,t] with err = (w - deq) Vt substituted.  Half the flops of
 * forge_chol_inv_upper_batched.  ws: forge_chol_workspace_bytes(nb, C). */
int forge_chol_factor_batched(float *A, int nb, int64_t C, float *udiag, int32_t *info, void *ws, void *stream);
int forge_chol_inv_upper_batched(float *A, int nb, int64_t C, float *U, float *udiag, int32_t *info,
                                 int zero_lower, void *ws, void *stream);

/* Allocation-free variant for ONE matrix; it has no counterpart in the reference.
 * Same result as forge_chol_inv_upper_batched(A, 1, C, ...), but the workspace is a 3 MiB array that
 * lives inside the library on every GPU that loads it, for callers that cannot obtain device memory
 * when they need a factorisation: a layer driver that has already given all of HBM to its Hessian
 * batches and must redo one expert (info > 0) with a larger damping, or a host application whose memory
 * manager forbids cudaMalloc (which would also stall its other streams).
 * C <= forge_noalloc_max_c() (4096), else FORGE_ERR_UNSUPPORTED.  The first call on a device looks up the
 * array's address (cudaGetSymbolAddress): make that call outside of stream capture, and make it early — the CUDA
 * runtime loads the library's code lazily, so the 3 MiB array itself is created on a device by that first call;
 * a warm-up call at start-up, while device memory is still free, guarantees it exists when memory has run out.  All calls on a device
 * share the array, so calls that overlap on the GPU (different streams) race; calls on one stream are safe,
 * and nothing in the array needs clearing between calls. */
int64_t forge_noalloc_max_c(void);
int forge_chol_inv_upper_noalloc(float *A, int64_t C, float *U, float *udiag, int32_t *info,
                                 int zero_lower, void *stream);

/* ---- A5/A6: per-group scale / zero grid -----------------------------------
 * W [nb*R, C] (bf16 or fp32, row-major, groups of gs consecutive columns, the last one zero padded).
 * scales,qzeros [nb*R*G] fp32.  symmetric: s = 2/maxq*max|w| + 1e-12, q0 = (maxq+1)/2;  else
 * s = (max-min)/maxq + 1e-12, q0 = clamp(rint(-min/s)).  With n_cand > 0 the L^norm error of every
 * shrink factor candidates[p] is evaluated and the first best (s, q0) is kept.  gs in {32,64,128}.
 * Replaces kernels.build_group_meta_packed (forge/backend/cuda/quant_grid.cu:42-99,186-224) and
 * kernels.mse_scale_groups_packed (quant_grid.cu:101-183,227-287), called from forge/gptq.py:181-227. */
int forge_quant_grid(const void *W, int w_dtype, int64_t rows, int64_t C, int gs, int bits, int symmetric,
                     const float *candidates, int n_cand, float norm, float *scales, float *qzeros,
                     void *stream);
/* MSE refinement only, on scales/qzeros computed earlier (in place). */
int forge_quant_grid_mse(const void *W, int w_dtype, int64_t rows, int64_t C, int gs, int bits,
                         int symmetric, const float *candidates, int n_cand, float norm,
                         float *scales, float *qzeros, void *stream);

/* ---- A7-A9: fused column solver -------------------------------------------
 * forge_gptq_solve_cr is the reference's operator: Wt [C,R] fp32 (columns already permuted), U [C,C]
 * unit-diagonal upper, scales/qzeros per ELEMENT [C,R]; writes codes q [C,R] uint8, overwrites Wt with
 * the de-quantised weights; sparse14 != 0 selects the SparseGPT 1:4 variant (uinv [C] = 1/diag of the
 * un-normalised factor; M [ceil(C/32),R] uint32 keep-mask).  ws: forge_solve_workspace_bytes(1,R,C).
 * `status` (device int32, may be NULL) receives FORGE_ERR_TIMEOUT if a bounded wait of the tensor-core
 * build ran out.  With R % 4 == 0 and C % 4 == 0 the lazy update runs on tcgen05 (TF32 x3 split, fp32
 * accumulate in TMEM), otherwise on the FMA pipe; FORGE_SOLVER_IMPL=simt in the environment forces the latter.
 * Replaces kernels.gptq_solver (forge/backend/cuda/solver.cu:99-154) and kernels.sparsegptq14_solver
 * (forge/backend/cuda/solver_sparsegptq14.cu:142-200). */
int64_t forge_solve_workspace_bytes(int nb, int64_t R, int64_t C);
int forge_gptq_solve_cr(float *Wt, const float *U, const float *uinv, const float *scales,
                        const float *qzeros, int bits, int64_t R, int64_t C, int sparse14,
                        uint8_t *q, uint32_t *M, void *ws, int32_t *status, void *stream);

/* forge_gptq_solve_batched is the batched fast path: nb weights W[b] [R,C] (bf16 or fp32) in ORIGINAL
 * column order, solved against U[u_map[b]] (u_map NULL = b) with per-GROUP scales/qzeros [nb,R,G]
 * (group of a column = original index / gs, as forge/gptq.py:251-252 expands them), perm [nu,C] per
 * Hessian slot (NULL = identity; nu = number of slots), udiag [nu,C] from the factorisation (sparse14).  Outputs codes qweight [nb,R,C] uint8 in ORIGINAL
 * column order (forge/gptq.py:139) and, for sparse14, M [nb, ceil(C/32), R] in PERMUTED order like the
 * reference.  ws: forge_solve_workspace_bytes(nb,R,C).  form = 0: U is the unit upper factor of the inverse
 * (forge_chol_inv_upper_batched) and the column errors x - deq are propagated, as in the reference;
 * form = 1: U is the output of forge_chol_factor_batched and w - deq is propagated (same recurrence without
 * the triangular inverse; needs R % 4 == 0 and C % 4 == 0).  Replaces the glue of GPTQ.quantize/_solver,
 * forge/gptq.py:129-139,231-276, together with the two solvers above.
 * usplit (may be NULL): the tensor-core operand pieces of U prepared once per Hessian slot by forge_solve_split_u
 * (forge_solve_split_u_bytes(nu, C) bytes).  With it the solver's row strips fetch U with bulk copies instead of each
 * re-splitting the same rows; gate and up of an expert, which share U, share the pieces too.  Needs R, C % 4 == 0. */
int64_t forge_solve_split_u_bytes(int nu, int64_t C);
int forge_solve_split_u(const float *U, int nu, int64_t C, void *usplit, void *stream);
int forge_gptq_solve_batched(const void *W, int w_dtype, int nb, int64_t R, int64_t C, const float *U,
                             const float *udiag, const int32_t *u_map, const int32_t *perm, int nu,
                             const float *scales, const float *qzeros, int gs, int bits, int sparse14,
                             int form, const void *usplit, uint8_t *qweight, uint32_t *M, void *ws, int32_t *status,
                             void *stream);

/* ---- checkpoint weight materialisation on the device (callers of the path) -----
 * Packed int4 ("pack-quantized", e.g. Kimi-K2): packed int32 [O, I/8] + scales fp32 [O, I/gs] -> dense [O, I]
 * (bf16 or fp32): out = fp32(nibble) * scale (or * 1/scale when scale_is_inv); nibbles are two's-complement int4 when
 * symmetric, unsigned otherwise.  Replaces _apply_block_scale, forge/utils/io.py:722-808 (CPU torch there). */
int forge_int4_packed_dequant(const int32_t *packed, const float *scales, int64_t O, int64_t I, int gs,
                              int symmetric, int scale_is_inv, void *out, int out_dtype, void *stream);

/* MXFP4 (gpt-oss): blocks u8 [rows, NB, 16] (32 E2M1 codes each, low nibble first) + E8M0 scales u8 [rows, NB]
 * -> dense, TRANSPOSED like the reference: out [NB*32, rows] (bf16 or fp32); scale = 2^(e-127), 2^-23 for e == 0.
 * Replaces _dequant_mxfp4_blocks_to_fp / _e8m0_to_scale_fp32, forge/utils/io.py:505-531. */
int forge_mxfp4_dequant(const uint8_t *blocks, const uint8_t *scales, int64_t rows, int64_t NB, void *out,
                        int out_dtype, void *stream);

/* ---- A12: de-quantise codes ------------------------------------------------
 * out[r,c] = dtype( (q[r,c] - qzeros[r,c/gs]) * scales[r,c/gs] )   (fp32 arithmetic)
 * Replaces dequantize_forge_full, forge/utils/engine.py:72-97. */
int forge_dequantize(const uint8_t *q, const float *scales, const float *qzeros, int64_t rows, int64_t C,
                     int gs, void *out, int out_dtype, void *stream);

/* ---- acceptance quantity: layer reconstruction loss ---------------------------
 * loss[b] = || X_b W[b]^T - X_b What[b]^T ||_F^2 with What = (q - qzeros) * scales (per group of gs input
 * columns), X_b the rows of X that slot x_map[b] (x_map NULL = b) lists through token_idx / offsets exactly as in
 * forge_hessian_grouped.  W [nb,R,C] bf16 or fp32, q [nb,R,C] uint8, scales/qzeros [nb,R,G] fp32, loss [nb] double
 * (overwritten).  fp32 dot products, squares summed in double.  A check, not a hot kernel.
 * Replaces the per-layer relative-error evaluation of the driver, quant.py:491-496 (dequantize_forge_full,
 * forge/utils/engine.py:72-97, followed by a forward). */
int forge_recon_loss(const void *W, int w_dtype, const uint8_t *q, const float *scales, const float *qzeros, int gs,
                     int nb, int64_t R, int64_t C, const void *X_bf16, int64_t n_rows, int64_t ldx,
                     const int32_t *token_idx, int64_t list_len, const int64_t *offsets, const int32_t *x_map,
                     double *loss, int32_t *status, void *stream);

/* ---- A11: dense int4 "pack-quantized" layout -------------------------------
 * packed[r, j] = sum_{i<8} uint8(int8(q[r,8j+i]) - int8(zero[r,(8j+i)/gs]) + 8) << 4i   (int32 wrap;
 * columns past C contribute 0) — bit-exact with compressed_tensors.pack_to_int32 as called by
 * pack_weight, pack_quantized.py:279-313.  packed is [rows, ceil(C/8)] int32. */
int forge_pack_int4(const uint8_t *q, const float *qzeros, int64_t rows, int64_t C, int gs,
                    int32_t *packed, void *stream);

/* ---- A10: sparse 1:4 + int4 "Wpair" layout ----------------------------------
 * q [R,C] uint8 (original layout), M [G32,R] uint32, scales32 [G32,R] fp32 (one scale per 32 columns)
 * -> out [G2=ceil(G32/2), R, 2] uint64:  bf16(scale)<<48 | idx16<<32 | eight 4-bit codes.
 * Replaces kernels.pack_sparsegptq14_to_u64x2, forge/backend/cuda/bitpacking_sparsegptq14.cu:58-175. */
int forge_pack_sparse14(const uint8_t *q, const uint32_t *M, const float *scales32, int64_t R, int64_t C,
                        uint64_t *out, void *stream);
/* The same for nb matrices in one launch: q [nb,R,C], M [nb,ceil(C/32),R], scales32 [nb,ceil(C/32),R] -> out
 * [nb,G2,R,2] (a layer's experts; the reference calls its packer once per Linear, quant.py:438-447). */
int forge_pack_sparse14_batched(const uint8_t *q, const uint32_t *M, const float *scales32, int nb, int64_t R, int64_t C,
                                uint64_t *out, void *stream);

/* ---- inference over the Wpair layout ------------------------------------------
 * Y[n, r] = bf16( sum_c X[n, c] * What[r, c] ), What decoded on the fly from wpair [ceil(C/64), R, 2] uint64
 * (the output of forge_pack_sparse14): per 32-channel half  scale * sum_{i<8} X[n, base + 4 i + pos_i] * (code_i - 8),
 * fp32 fused multiply-adds in that order, one rounding at the end.  X bf16 [N, ldx >= C], Y bf16 [N, R]; no padding
 * of N, R or C is required.  Bit-identical to kernels.sparsegptq14_gemm
 * (moe_proj_unstructured_sparse14_int4symq_gemm, forge/backend/cuda/sparse14_gemm.cu:49-140, :282-374), which it
 * replaces. */
int forge_sparse14_gemm(const uint64_t *wpair, const void *X_bf16, int64_t ldx, int64_t N, int64_t R, int64_t C,
                        void *Y_bf16, void *stream);

/* Grouped forms for a mixture-of-experts layer.  The routed rows are sorted by expert: permuted positions
 * [offsets[e], offsets[e+1]) (int64, device) belong to expert e; `active` (int32 [n_active], device) lists the experts to
 * run; w13 / w2 hold all experts' packets, [E, ceil(C/64), R, 2] uint64.  `token_idx` (int32 [N], device) maps a permuted
 * position to its row of X [x_rows, ldx]; NULL means X is already in permuted order.  Claims beyond N and rows outside X
 * are clipped / read as zeros.
 *   forge_sparse14_moe_w13_swiglu: R = 2 I with the gate rows first;  X2[m, i] = bf16( silu(g) * u ), g and u the fp32 sums
 *     of rows i and I + i, silu(g) = g / (1 + expf(-g)); X2 bf16 [N, I].  Interface and arithmetic of
 *     kernels.sparsegptq14_grouped_gemm_w13 (usp14w4a16sym_sm80_fused_moe_w13_gemm,
 *     forge/backend/cuda/fused_moe_usp14w4a16_gemm.cu:398-439, :722-723, :1028-1084).
 *   forge_sparse14_moe_w2: Y[m, r] = bf16( sum ), bit-identical to forge_sparse14_gemm run per expert; Y bf16 [N, R].
 *     Replaces kernels.sparsegptq14_grouped_gemm_w2 (:1086-1140). */
int forge_sparse14_moe_w13_swiglu(const uint64_t *w13, const void *X_bf16, int64_t ldx, int64_t x_rows,
                                  const int32_t *token_idx, const int64_t *offsets, const int32_t *active, int n_active,
                                  int64_t N, int64_t R, int64_t C, void *X2_bf16, void *stream);
int forge_sparse14_moe_w2(const uint64_t *w2, const void *X2_bf16, int64_t ldx, int64_t x_rows, const int32_t *token_idx,
                          const int64_t *offsets, const int32_t *active, int n_active, int64_t N, int64_t R, int64_t C,
                          void *Y_bf16, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FORGE_B200_H */
