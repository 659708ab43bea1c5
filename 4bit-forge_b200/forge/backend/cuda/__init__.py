"""`kernels`: the reference's extension-module surface (forge/backend/cuda/kernels.cpp:92-150) re-created
over the sm_100a C ABI.  Function names, argument order, in-place behaviour and return values follow the
pybind module; the per-expert inference GEMM over the Wpair layout is here too, the fused MoE inference GEMMs and the
Babai solver are not part of the solver path and are absent.

Like the reference stub (forge/backend/cuda/__init__.py:74-87) every call raises RuntimeError when CUDA
or the library is unavailable: there is no CPU fallback.
"""
from __future__ import annotations

import torch

from ... import ops

__all__ = ["kernels"]


class _Kernels:
    @staticmethod
    def build_group_meta_packed(X, bits, symmetric):
        """quant_grid.cu:186-224 — X [R*G, gs] -> (scales, qzeros) fp32 [R*G]."""
        X = X.contiguous()
        RG, gs = X.shape
        return ops.quant_grid(X.view(RG, gs), int(gs), int(bits), bool(symmetric))

    @staticmethod
    def mse_scale_groups_packed(X, scales, qzeros, candidates, norm, bits, symmetric):
        """quant_grid.cu:227-287 — refines scales/qzeros in place and returns them."""
        X = X.contiguous()
        RG, gs = X.shape
        if gs not in (32, 64, 128):
            raise RuntimeError(f"Unsupported group_size={gs} (expected 32/64/128)")
        return ops.quant_grid_mse(X, int(gs), int(bits), bool(symmetric),
                                  candidates.to(torch.float32).contiguous(), float(norm), scales, qzeros)

    @staticmethod
    def gptq_solver(W, U, scales, qzeros, bits):
        """solver.cu:99-154 — W [C,R] fp32 is overwritten with the de-quantised weights; returns u8 [C,R]."""
        if not W.is_contiguous():
            raise RuntimeError("gptq_solver: W must be contiguous (it is updated in place)")
        return ops.gptq_solve_cr(W, U.contiguous(), scales.contiguous(), qzeros.contiguous(), int(bits))

    @staticmethod
    def sparsegptq14_solver(W, U, scales, qzeros, bits):
        """solver_sparsegptq14.cu:142-200 — U is row-normalised in place; returns (u8 [C,R], u32 [C/32,R])."""
        if not (W.is_contiguous() and U.is_contiguous()):
            raise RuntimeError("sparsegptq14_solver: W and U must be contiguous (both are updated in place)")
        uinv = U.diagonal().reciprocal().contiguous()
        U.mul_(uinv.unsqueeze(1))
        q, M = ops.gptq_solve_cr(W, U, scales.contiguous(), qzeros.contiguous(), int(bits), uinv=uinv)
        return q, M.view(torch.uint32)

    @staticmethod
    def pack_sparsegptq14_to_u64x2(qweight_rc, M, scales):
        """bitpacking_sparsegptq14.cu:110-175 — -> uint64 [G2,R,2]."""
        if qweight_rc.dim() != 2:
            raise RuntimeError("qweight_rc must be [R, C]")
        if M.dim() != 2:
            raise RuntimeError("M must be [G32, R]")
        if scales.dim() != 2:
            raise RuntimeError("scales must be [G32, R]")
        R, C = qweight_rc.shape
        G32 = (C + 31) // 32
        if M.shape[1] != R or scales.shape[1] != R:
            raise RuntimeError("M / scales second dim must equal R")
        if M.shape[0] != G32 or scales.shape[0] != G32:
            raise RuntimeError(f"M first dim (G32) mismatch: got {M.shape[0]} expected {G32}")
        Mi = M.contiguous()
        if Mi.dtype != torch.int32:
            Mi = Mi.view(torch.int32)
        out = ops.pack_sparse14(qweight_rc.to(torch.uint8).contiguous(), Mi,
                                scales.to(torch.float32).contiguous())
        return out.view(torch.uint64)


    @staticmethod
    def sparsegptq14_gemm(qW2S1u64, X):
        """sparse14_gemm.cu:282-374 — Wpair [G2, R, 2] uint64, X bf16 [N, C] -> Y bf16 [N, R]."""
        if not (qW2S1u64.dim() == 3 and qW2S1u64.size(2) == 2):
            raise RuntimeError("qW2S1u64 must be [G2, R, 2]")
        if X.dim() != 2:
            raise RuntimeError("X must be [N, C]")
        if X.dtype != torch.bfloat16:
            raise RuntimeError("X must be bfloat16")
        w = qW2S1u64.contiguous()
        if w.dtype != torch.int64:
            w = w.view(torch.int64)
        return ops.sparse14_gemm(w, X)

    @staticmethod
    def _grouped_args(W, X, offsets, U):
        if not (W.dim() == 4 and W.size(3) == 2):
            raise RuntimeError("W must be [E, G2, R, 2]")
        if X.dim() != 2 or X.dtype != torch.bfloat16:
            raise RuntimeError("X must be bfloat16 [N, C]")
        w = W.contiguous()
        return (w if w.dtype == torch.int64 else w.view(torch.int64)), X, offsets, U

    @staticmethod
    def sparsegptq14_grouped_gemm_w13(W13, X, offsets, U):
        """fused_moe_usp14w4a16_gemm.cu:1028-1084 — W13 [E, G2, 2I, 2] uint64, X bf16 [N, H] sorted by expert,
        offsets int64 [E+1], U int32 active expert ids -> X2 bf16 [N, I] = silu(gate) * up."""
        return ops.sparse14_moe_w13_swiglu(*_Kernels._grouped_args(W13, X, offsets, U))

    @staticmethod
    def sparsegptq14_grouped_gemm_w2(W2, X2, offsets, U):
        """fused_moe_usp14w4a16_gemm.cu:1086-1140 — W2 [E, G2, H, 2] uint64, X2 bf16 [N, I] sorted by expert -> Y bf16
        [N, H]."""
        return ops.sparse14_moe_w2(*_Kernels._grouped_args(W2, X2, offsets, U))


kernels = _Kernels()
