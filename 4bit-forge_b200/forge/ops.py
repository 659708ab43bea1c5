"""Torch-tensor wrappers over the C ABI.  PyTorch supplies device memory and the stream; every
computation happens in libforge_b200.so.  Shapes follow include/forge_b200.h."""
from __future__ import annotations

import torch

from . import _abi
from ._abi import call, ptr, stream_ptr, dtype_code, query


def _dev(t):
    return t.device


def fp8_block_dequant(w_fp8: torch.Tensor, scale_inv: torch.Tensor, out=None) -> torch.Tensor:
    """bf16( fp32(w_fp8) * scale_inv[tile] ) — forge/utils/io.py:533-563, :864-874 on the device."""
    O, I = w_fp8.shape
    nO, nI = scale_inv.shape
    w8 = w_fp8.contiguous().view(torch.uint8)
    if out is None:
        out = torch.empty((O, I), dtype=torch.bfloat16, device=_dev(w_fp8))
    assert out.dtype == torch.bfloat16 and out.shape == (O, I) and out.is_contiguous()
    call("forge_fp8_block_dequant", ptr(w8), ptr(scale_inv.to(torch.float32).contiguous()), ptr(out), O, I, nO, nI,
         stream_ptr())
    return out


def int4_packed_dequant(packed: torch.Tensor, scales: torch.Tensor, shape, symmetric: bool = True,
                        scale_is_inv: bool = False, dtype=torch.bfloat16) -> torch.Tensor:
    """Packed int32 [O, I/8] + per-group scales [O, I/gs] -> dense [O, I] — forge/utils/io.py:722-808 on the device."""
    O, I = int(shape[0]), int(shape[1])
    sc = scales.to(torch.float32).contiguous()
    assert (O * I) % sc.numel() == 0
    gs = (O * I) // sc.numel()
    out = torch.empty((O, I), dtype=dtype, device=_dev(packed))
    code = _abi.BF16 if dtype == torch.bfloat16 else _abi.F32
    assert dtype in (torch.float32, torch.bfloat16)
    call("forge_int4_packed_dequant", ptr(packed.to(torch.int32).contiguous()), ptr(sc), O, I, gs, int(symmetric),
         int(scale_is_inv), ptr(out), code, stream_ptr())
    return out


def mxfp4_dequant(blocks_u8: torch.Tensor, scales_u8: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """blocks [..., rows, NB, 16] u8 + scales [..., rows, NB] u8 -> [..., NB*32, rows] — forge/utils/io.py:505-531 on the
    device (the transpose of the last two dimensions included)."""
    lead = blocks_u8.shape[:-3]
    rows, NB = int(blocks_u8.shape[-3]), int(blocks_u8.shape[-2])
    b = blocks_u8.contiguous().view(-1, rows, NB, 16)
    s = scales_u8.contiguous().view(-1, rows, NB)
    out = torch.empty((b.shape[0], NB * 32, rows), dtype=dtype, device=_dev(blocks_u8))
    code = _abi.BF16 if dtype == torch.bfloat16 else _abi.F32
    assert dtype in (torch.float32, torch.bfloat16)
    for k in range(b.shape[0]):
        call("forge_mxfp4_dequant", ptr(b[k]), ptr(s[k]), rows, NB, ptr(out[k]), code, stream_ptr())
    return out.view(*lead, NB * 32, rows)


def route_topk(logits: torch.Tensor, top_k: int, mode: str = "softmax", n_groups: int = 1, topk_groups: int = 1,
               bias=None, want_weights: bool = False):
    """Router logits [T,E] fp32 -> expert ids int32 [T,k] in descending score order (forge_route_topk).
    mode: "softmax", "sigmoid" or "sigmoid_group" (DeepSeek-V3 group-limited selection)."""
    T, E = logits.shape
    lg = logits.to(torch.float32).contiguous()
    dev = _dev(lg)
    ids = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    w = torch.empty((T, top_k), dtype=torch.float32, device=dev) if want_weights else None
    b = None if bias is None else bias.to(torch.float32).contiguous()
    call("forge_route_topk", ptr(lg), ptr(b), T, E, int(top_k), _abi.ROUTE_MODES[mode], int(n_groups), int(topk_groups),
         ptr(ids), ptr(w), stream_ptr())
    return (ids, w) if want_weights else ids


def route_build_lists(topk_ids, e_begin: int, e_count: int, dense_tail: int = 0, n_tokens: int = 0):
    """topk_ids [T,k] int32 -> (counts int32 [n], offsets int64 [n+1], token_lists int32 [T*k + dense_tail*T]) for the
    routed experts [e_begin, e_begin+e_count) followed by dense_tail slots that see every token; n = e_count +
    dense_tail.  With e_count == 0 topk_ids may be None and n_tokens gives T."""
    if topk_ids is not None:
        T, k = topk_ids.shape
        ids = topk_ids.to(torch.int32).contiguous()
        dev = _dev(ids)
    else:
        T, k, ids = int(n_tokens), 1, None
        dev = torch.device("cuda", torch.cuda.current_device())
    n = e_count + dense_tail
    counts = torch.empty(n, dtype=torch.int32, device=dev)
    offsets = torch.empty(n + 1, dtype=torch.int64, device=dev)
    lists = torch.empty(max((T * k if e_count else 0) + dense_tail * T, 1), dtype=torch.int32, device=dev)
    call("forge_route_build_lists", ptr(ids), T, k, e_begin, e_count, dense_tail, ptr(counts), ptr(offsets), ptr(lists),
         stream_ptr())
    return counts, offsets, lists


def expert_swiglu_grouped(X, token_idx, offsets, Wg, Wu, out_rows: int, out=None, simt: bool = False, status=None):
    """Down-projection calibration input of every slot, packed by slot: bf16(silu(x Wg^T) * (x Wu^T)) with the
    block forward's bf16 roundings (forge_expert_swiglu_grouped).  X bf16 [T, ldx], Wg/Wu bf16 [nb, I, H]."""
    assert X.dtype == torch.bfloat16 and Wg.dtype == torch.bfloat16 and Wu.dtype == torch.bfloat16
    nb, I, H = Wg.shape
    assert offsets.dtype == torch.int64 and offsets.numel() == nb + 1
    if out is None:
        out = torch.empty((max(out_rows, 1), I), dtype=torch.bfloat16, device=_dev(X))
    list_len = 0 if token_idx is None else token_idx.numel()
    call("forge_expert_swiglu_grouped", ptr(X), X.shape[0], X.stride(0), H, I, ptr(token_idx), list_len, ptr(offsets), nb,
         ptr(Wg), ptr(Wu), ptr(out), out.shape[0], _abi.FWD_SIMT if simt else 0, ptr(status), stream_ptr())
    return out


def recon_loss(W, q, scales, qzeros, gs: int, X, token_idx, offsets, x_map=None, status=None):
    """|| X_b W[b]^T - X_b What[b]^T ||_F^2 per matrix (forge_recon_loss) -> float64 [nb].  W [nb,R,C], q [nb,R,C] u8,
    scales/qzeros [nb,R,G]; X bf16 rows listed per slot like hessian_grouped."""
    nb, R, C = W.shape
    loss = torch.empty(nb, dtype=torch.float64, device=_dev(W))
    list_len = 0 if token_idx is None else token_idx.numel()
    call("forge_recon_loss", ptr(W), dtype_code(W), ptr(q), ptr(scales), ptr(qzeros), int(gs), nb, R, C, ptr(X), X.shape[0],
         X.stride(0), ptr(token_idx), list_len, ptr(offsets), ptr(x_map), ptr(loss), ptr(status), stream_ptr())
    return loss


def hessian_grouped(X: torch.Tensor, C: int, token_idx, offsets: torch.Tensor, H: torch.Tensor, n_prev=None,
                    mirror: bool = True, simt: bool = False, status=None):
    """H[b] = beta*H[b] + alpha * X_b^T X_b (see forge_hessian_grouped).  X bf16 [T, ldx>=C]; H fp32 [nb,C,C]."""
    assert X.dtype == torch.bfloat16 and X.dim() == 2 and H.dtype == torch.float32
    nb = H.shape[0]
    assert offsets.dtype == torch.int64 and offsets.numel() == nb + 1
    flags = (_abi.HESS_MIRROR if mirror else 0) | (_abi.HESS_SIMT if simt else 0)
    own_status = status is None
    if own_status:
        status = torch.zeros(1, dtype=torch.int32, device=_dev(X))
    list_len = 0 if token_idx is None else token_idx.numel()
    call("forge_hessian_grouped", ptr(X), X.shape[0], X.stride(0), C, ptr(token_idx), list_len, ptr(offsets), nb, ptr(H),
         ptr(n_prev), flags, ptr(status), stream_ptr())
    return status


def counts_add(n_prev: torch.Tensor, offsets: torch.Tensor):
    call("forge_counts_add", ptr(n_prev), ptr(offsets), n_prev.numel(), stream_ptr())


def hessian_scan(H: torch.Tensor, n_samples=None):
    nb, C, _ = H.shape
    dev = _dev(H)
    diag = torch.empty((nb, C), dtype=torch.float32, device=dev)
    pruned = torch.empty((nb, C), dtype=torch.uint8, device=dev)
    invalid = torch.empty(nb, dtype=torch.int32, device=dev)
    call("forge_hessian_scan", ptr(H), nb, C, ptr(n_samples), ptr(diag), ptr(pruned), ptr(invalid), stream_ptr())
    return diag, pruned, invalid


def weight_apply_pruned(W: torch.Tensor, pruned: torch.Tensor, u_map=None):
    nb, R, C = W.shape
    call("forge_weight_apply_pruned", ptr(W), dtype_code(W), nb, R, C, ptr(pruned), ptr(u_map), stream_ptr())


def weight_zero_cols(W: torch.Tensor) -> torch.Tensor:
    nb, R, C = W.shape
    wz = torch.empty((nb, C), dtype=torch.uint8, device=_dev(W))
    call("forge_weight_zero_cols", ptr(W), dtype_code(W), nb, R, C, ptr(wz), stream_ptr())
    return wz


def hessian_gather_damp(H, perm, pruned, wzero, invalid, rel_damp: float, A=None, want_hp: bool = False):
    nb, C, _ = H.shape
    dev = _dev(H)
    if A is None:
        A = torch.empty_like(H)
    Hp = torch.empty_like(H) if want_hp else None
    damp = torch.empty(nb, dtype=torch.float32, device=dev)
    call("forge_hessian_gather_damp", ptr(H), nb, C, ptr(perm), ptr(pruned), ptr(wzero), ptr(invalid), float(rel_damp),
         ptr(A), ptr(Hp), ptr(damp), stream_ptr())
    return A, Hp, damp


def chol_inv_upper(A: torch.Tensor, U=None, zero_lower: bool = True):
    """A [nb,C,C] (index-reversed damped Hessian, destroyed) -> (U, udiag, info)."""
    nb, C, _ = A.shape
    dev = _dev(A)
    if U is None:
        U = torch.empty_like(A)
    udiag = torch.empty((nb, C), dtype=torch.float32, device=dev)
    info = torch.empty(nb, dtype=torch.int32, device=dev)
    ws = torch.empty(query("forge_chol_workspace_bytes", nb, C), dtype=torch.uint8, device=dev)
    call("forge_chol_inv_upper_batched", ptr(A), nb, C, ptr(U), ptr(udiag), ptr(info), int(zero_lower), ptr(ws),
         stream_ptr())
    return U, udiag, info


def chol_factor(A: torch.Tensor):
    """Inversion-free form: A [nb,C,C] (index-reversed damped Hessian) is overwritten; its upper triangle then
    holds -Vt (see forge_chol_factor_batched).  Returns (A, udiag, info)."""
    nb, C, _ = A.shape
    dev = _dev(A)
    udiag = torch.empty((nb, C), dtype=torch.float32, device=dev)
    info = torch.empty(nb, dtype=torch.int32, device=dev)
    ws = torch.empty(query("forge_chol_workspace_bytes", nb, C), dtype=torch.uint8, device=dev)
    call("forge_chol_factor_batched", ptr(A), nb, C, ptr(udiag), ptr(info), ptr(ws), stream_ptr())
    return A, udiag, info


def quant_grid(W: torch.Tensor, gs: int, bits: int, symmetric: bool, candidates=None, norm: float = 2.4):
    """W [rows, C] (bf16/fp32) -> (scales, qzeros) fp32 [rows*G]; candidates given = MSE search fused in."""
    rows, C = W.shape
    G = (C + gs - 1) // gs
    dev = _dev(W)
    scales = torch.empty(rows * G, dtype=torch.float32, device=dev)
    qzeros = torch.empty(rows * G, dtype=torch.float32, device=dev)
    n_cand = 0 if candidates is None else candidates.numel()
    call("forge_quant_grid", ptr(W), dtype_code(W), rows, C, gs, bits, int(bool(symmetric)), ptr(candidates), n_cand,
         float(norm), ptr(scales), ptr(qzeros), stream_ptr())
    return scales, qzeros


def quant_grid_mse(W, gs, bits, symmetric, candidates, norm, scales, qzeros):
    rows, C = W.shape
    call("forge_quant_grid_mse", ptr(W), dtype_code(W), rows, C, gs, bits, int(bool(symmetric)), ptr(candidates),
         candidates.numel(), float(norm), ptr(scales), ptr(qzeros), stream_ptr())
    return scales, qzeros


def gptq_solve_cr(Wt, U, scales_el, qzeros_el, bits: int, uinv=None, status=None):
    """Reference operator layout: Wt [C,R] fp32 (mutated -> dequantised), per-element scales [C,R]."""
    C, R = Wt.shape
    dev = _dev(Wt)
    q = torch.empty((C, R), dtype=torch.uint8, device=dev)
    sparse = uinv is not None
    M = torch.zeros(((C + 31) // 32, R), dtype=torch.int32, device=dev) if sparse else None
    ws = torch.empty(query("forge_solve_workspace_bytes", 1, R, C), dtype=torch.uint8, device=dev)
    call("forge_gptq_solve_cr", ptr(Wt), ptr(U), ptr(uinv), ptr(scales_el), ptr(qzeros_el), bits, R, C, int(sparse),
         ptr(q), ptr(M), ptr(ws), ptr(status), stream_ptr())
    return (q, M) if sparse else q


def solve_split_u(U: torch.Tensor, out=None):
    """Tensor-core operand pieces of U [nu,C,C] for gptq_solve_batched(usplit=...) (forge_solve_split_u); None when
    the shape does not take the tensor-core path (C not a multiple of 4).  out: callable nbytes -> uint8 buffer, or
    None (a fresh tensor)."""
    nu, C, _ = U.shape
    nbytes = query("forge_solve_split_u_bytes", nu, C)
    if nbytes == 0:
        return None
    out = torch.empty(nbytes, dtype=torch.uint8, device=_dev(U)) if out is None else out(nbytes)
    call("forge_solve_split_u", ptr(U), nu, C, ptr(out), stream_ptr())
    return out


def gptq_solve_batched(W, U, scales, qzeros, gs: int, bits: int, perm=None, u_map=None, udiag=None,
                       sparse14: bool = False, ws=None, status=None, form: int = 0, usplit=None):
    """W [nb,R,C] original order; U [nu,C,C]; scales/qzeros [nb*R*G] -> qweight [nb,R,C] (+ M [nb,G32,R])."""
    nb, R, C = W.shape
    dev = _dev(W)
    nu = U.shape[0]
    q = torch.empty((nb, R, C), dtype=torch.uint8, device=dev)
    M = torch.zeros((nb, (C + 31) // 32, R), dtype=torch.int32, device=dev) if sparse14 else None
    if ws is None:
        ws = torch.empty(query("forge_solve_workspace_bytes", nb, R, C), dtype=torch.uint8, device=dev)
    elif callable(ws):
        ws = ws(query("forge_solve_workspace_bytes", nb, R, C))
    call("forge_gptq_solve_batched", ptr(W), dtype_code(W), nb, R, C, ptr(U), ptr(udiag), ptr(u_map), ptr(perm), nu,
         ptr(scales), ptr(qzeros), gs, bits, int(sparse14), int(form), ptr(usplit if (R % 4 == 0 and C % 4 == 0) else None),
         ptr(q), ptr(M), ptr(ws), ptr(status), stream_ptr())
    return (q, M) if sparse14 else q


def dequantize(q, scales, qzeros, gs: int, dtype=torch.float32):
    """(q - q0) * s in fp32 -> dtype; q [..., C] uint8, scales/qzeros flat per (row, group)."""
    C = q.shape[-1]
    rows = q.numel() // C
    out = torch.empty(q.shape, dtype=dtype, device=_dev(q))
    code = _abi.BF16 if dtype == torch.bfloat16 else _abi.F32
    assert dtype in (torch.float32, torch.bfloat16)
    call("forge_dequantize", ptr(q), ptr(scales), ptr(qzeros), rows, C, gs, ptr(out), code, stream_ptr())
    return out


def pack_int4(q, qzeros, gs: int):
    """weight_packed int32 [..., ceil(C/8)] of the compressed-tensors pack-quantized format."""
    C = q.shape[-1]
    rows = q.numel() // C
    out = torch.empty((*q.shape[:-1], (C + 7) // 8), dtype=torch.int32, device=_dev(q))
    call("forge_pack_int4", ptr(q), ptr(qzeros), rows, C, gs, ptr(out), stream_ptr())
    return out


def pack_sparse14(q_rc, M, scales32):
    """q [R,C] u8, M [G32,R], scales32 [G32,R] fp32 -> Wpair int64 bit pattern [G2,R,2]."""
    R, C = q_rc.shape
    G32 = (C + 31) // 32
    out = torch.empty(((G32 + 1) // 2, R, 2), dtype=torch.int64, device=_dev(q_rc))
    call("forge_pack_sparse14", ptr(q_rc), ptr(M), ptr(scales32), R, C, ptr(out), stream_ptr())
    return out


def pack_sparse14_batched(q, M, scales32):
    """q [nb,R,C] u8, M [nb,G32,R], scales32 [nb,G32,R] fp32 -> Wpair int64 bit patterns [nb,G2,R,2], one launch."""
    nb, R, C = q.shape
    G32 = (C + 31) // 32
    assert M.shape == (nb, G32, R) and scales32.shape == (nb, G32, R)
    out = torch.empty((nb, (G32 + 1) // 2, R, 2), dtype=torch.int64, device=_dev(q))
    call("forge_pack_sparse14_batched", ptr(q), ptr(M), ptr(scales32), nb, R, C, ptr(out), stream_ptr())
    return out


def sparse14_gemm(wpair: torch.Tensor, X: torch.Tensor) -> torch.Tensor:
    """Y = X @ What^T with What decoded from the Wpair words [G2, R, 2] (forge_sparse14_gemm).  X bf16 [N, C]."""
    assert X.dtype == torch.bfloat16 and X.dim() == 2 and wpair.dim() == 3 and wpair.shape[2] == 2
    G2, R, _ = wpair.shape
    N, C = X.shape
    if G2 != (C + 63) // 64:
        raise RuntimeError(f"Wpair G2 mismatch: got {G2} expected {(C + 63) // 64}")
    X = X.contiguous()
    Y = torch.empty((N, R), dtype=torch.bfloat16, device=_dev(X))
    call("forge_sparse14_gemm", ptr(wpair.contiguous()), ptr(X), X.stride(0), N, R, C, ptr(Y), stream_ptr())
    return Y


def _sparse14_moe(entry: str, W: torch.Tensor, X: torch.Tensor, offsets: torch.Tensor, active: torch.Tensor,
                  token_idx, n_out: int, swiglu: bool) -> torch.Tensor:
    assert X.dtype == torch.bfloat16 and X.dim() == 2 and W.dim() == 4 and W.shape[3] == 2
    E, G2, R, _ = W.shape
    C = X.shape[1]
    if G2 != (C + 63) // 64:
        raise RuntimeError(f"Wpair G2 mismatch: got {G2} expected {(C + 63) // 64}")
    if offsets.numel() != E + 1:
        raise RuntimeError("offsets must hold E + 1 entries")
    X = X.contiguous()
    offsets = offsets.to(torch.int64).contiguous()
    active = active.to(torch.int32).contiguous()
    if token_idx is not None:
        token_idx = token_idx.to(torch.int32).contiguous()
        assert token_idx.numel() >= n_out
    out = torch.zeros((n_out, R // 2 if swiglu else R), dtype=torch.bfloat16, device=_dev(X))
    call(entry, ptr(W.contiguous()), ptr(X), X.stride(0), X.shape[0], ptr(token_idx), ptr(offsets), ptr(active),
         int(active.numel()), n_out, R, C, ptr(out), stream_ptr())
    return out


def sparse14_moe_w13_swiglu(W13, X, offsets, active, token_idx=None, n_out=None) -> torch.Tensor:
    """X2[m, :] = silu(gate) * up of the expert that owns permuted position m (forge_sparse14_moe_w13_swiglu).
    W13 [E, G2, 2I, 2] Wpair words, X bf16 [rows, H]; rows of inactive experts stay zero."""
    return _sparse14_moe("forge_sparse14_moe_w13_swiglu", W13, X, offsets, active, token_idx,
                         X.shape[0] if n_out is None else int(n_out), True)


def sparse14_moe_w2(W2, X2, offsets, active, token_idx=None, n_out=None) -> torch.Tensor:
    """Y[m, :] = X2[m, :] @ What_e^T for the expert e that owns permuted position m (forge_sparse14_moe_w2)."""
    return _sparse14_moe("forge_sparse14_moe_w2", W2, X2, offsets, active, token_idx,
                         X2.shape[0] if n_out is None else int(n_out), False)


def mma_issue_cycles(N: int = 128, iters: int = 2000, pattern: bool = True) -> float:
    """Cycles per tcgen05.mma kind::tf32 M128 x N x K8 when one thread issues them back to back on every SM
    (forge_selftest_mma_rate): the issue ceiling of the solver's and the factorisation's MMA shape on this GPU."""
    dev = torch.device("cuda", torch.cuda.current_device())
    cyc = torch.zeros(1, dtype=torch.int64, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    call("forge_selftest_mma_rate", int(N), int(iters), int(bool(pattern)), ptr(cyc), ptr(st), stream_ptr())
    vals = torch.cat([cyc, st.to(torch.int64)]).tolist()      # one host read
    if vals[1] != 0:
        raise RuntimeError(f"forge_selftest_mma_rate: status {vals[1]}")
    return vals[0] / float(iters)
