"""Inference over the packed sparse 1:4 + int4 experts: the runtime of the reference's sparse14_gemm.py:23-65
(Sparse14MoERuntime) on the grouped kernels.

The reference sorts the (token, slot) pairs by expert with vLLM's moe_permute, copies the hidden states into that
order and loops over experts and 256-row chunks with two per-expert GEMM calls and a torch SwiGLU between them.  Here
the sort is the routing-list kernel of the quantisation path, the permuted copy is replaced by a gather inside the
first kernel, and each projection pair is ONE launch over all experts (forge_sparse14_moe_w13_swiglu,
forge_sparse14_moe_w2).  Nothing is read back on the way.
"""
from __future__ import annotations

import torch

from . import ops


class Sparse14MoERuntime:
    """Same constructor and forward signature as sparse14_gemm.py:23-31.  w13_packed [E, G2(H), 2I, 2] and w2_packed
    [E, G2(I), H, 2] are the stacked outputs of the Wpair packer (uint64 bit patterns)."""

    def __init__(self, w13_packed, w2_packed, intermediate_size, num_experts, chunk_m=256):
        self.w13_packed = self._words(w13_packed)
        self.w2_packed = self._words(w2_packed)
        self.intermediate_size = int(intermediate_size)
        self.num_experts = int(num_experts)
        self.chunk_m = int(chunk_m)          # kept for signature compatibility; the grouped kernels need no chunking
        if self.w13_packed.shape[0] != self.num_experts or self.w2_packed.shape[0] != self.num_experts:
            raise RuntimeError("packed weights must be stacked over the experts")
        if self.w13_packed.shape[2] != 2 * self.intermediate_size:
            raise RuntimeError("w13_packed must hold 2 * intermediate_size rows (gate rows first)")
        self._active = torch.arange(self.num_experts, dtype=torch.int32, device=self.w13_packed.device)

    @staticmethod
    def _words(w):
        if not (w.dim() == 4 and w.shape[3] == 2):
            raise RuntimeError("packed weights must be [E, G2, R, 2]")
        w = w.contiguous()
        return w if w.dtype == torch.int64 else w.view(torch.int64)

    @torch.no_grad()
    def forward(self, hidden_states, topk_ids, topk_weights):
        """hidden_states bf16 [T, H], topk_ids [T, K], topk_weights [T, K] -> bf16 [T, H]: sum over the K slots of
        weight * down(silu(gate(x)) * up(x)) of the slot's expert (sparse14_gemm.py:32-65)."""
        T, H = hidden_states.shape
        K = topk_ids.shape[1]
        with torch.cuda.device(hidden_states.device):
            ids = topk_ids.to(torch.int32).contiguous()
            _, offsets, lists = ops.route_build_lists(ids, 0, self.num_experts)
            n = T * K
            a2 = ops.sparse14_moe_w13_swiglu(self.w13_packed, hidden_states, offsets, self._active, token_idx=lists,
                                             n_out=n)
            out_perm = ops.sparse14_moe_w2(self.w2_packed, a2, offsets, self._active, n_out=n)
            # weighted un-permute: the router weight of (token, expert) for every permuted position, fp32 sum, one
            # rounding
            tok = lists[:n].to(torch.int64)
            pos = torch.arange(n, device=hidden_states.device)
            expert = torch.searchsorted(offsets[1:].contiguous(), pos, right=True).clamp_(max=self.num_experts - 1)
            w = (topk_weights[tok].float() * (ids[tok].to(torch.int64) == expert[:, None])).sum(1)
            out = torch.zeros((T, H), dtype=torch.float32, device=hidden_states.device)
            out.index_add_(0, tok, out_perm.float() * w[:, None])
        return out.to(hidden_states.dtype)
