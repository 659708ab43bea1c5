"""Layer-level batched GPTQ / SparseGPT for one MoE layer.

The reference quantises one nn.Linear at a time: a forward hook per expert Linear feeds GPTQ.update, then
every handle runs quantize() on its own (quant.py:355-512).  Here the whole layer is one batched pass
over the experts a rank owns:

  routing lists -> grouped tcgen05 Hessian of the layer input (shared by gate and up, the reference's
  --owner_gptq_handles mode) -> expert forward for the down-projection input -> its Hessian ->
  scan / permutation / damping -> batched Cholesky -> scale grid -> fused column solver -> packing.

Everything stays on the device; the host reads back the per-expert token offsets once (to slice the
expert forward) and one flag (whether gate and up have the same all-zero columns).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


@dataclass
class MoEQuantConfig:
    bits: int = 4
    group_size: int = 128
    symmetric: bool = True
    quantization_scale: str = "absmax"     # or "mse"
    quantization_order: str = "default"    # or "activation"
    rel_damp: float = 0.01
    algorithm: str = "gptq"                # or "sparsegptq"
    pack: bool = True
    mse_grid: int = 100
    mse_max_shrink: float = 0.2
    mse_norm: float = 2.4
    expert_chunk: int = 0                  # experts factorised/solved per pass (0 = all at once)
    inversion_free: bool = True            # solve from the Cholesky factor itself, without the triangular inverse


def swiglu_expert_forward(X, token_lists, offsets_host, Wg, Wu):
    """Down-projection calibration input of every expert, packed by expert: bf16(silu(x Wg^T) * (x Wu^T)).
    Library bf16 GEMMs (fp32 accumulate), exactly what the HF MoE block computes before down_proj.
    The routed rows are gathered once for all experts and the activation runs once over the packed buffer,
    so an expert costs two GEMM launches and nothing else."""
    total = int(offsets_host[-1])
    I = Wg.shape[1]
    if total == 0:
        return torch.empty((1, I), dtype=torch.bfloat16, device=X.device)
    Xg = X.index_select(0, token_lists[:total].long())
    gate = torch.empty((total, I), dtype=torch.bfloat16, device=X.device)
    up = torch.empty((total, I), dtype=torch.bfloat16, device=X.device)
    for e in range(Wg.shape[0]):
        a, b = int(offsets_host[e]), int(offsets_host[e + 1])
        if b == a:
            continue
        torch.mm(Xg[a:b], Wg[e].T, out=gate[a:b])
        torch.mm(Xg[a:b], Wu[e].T, out=up[a:b])
    del Xg
    return torch.nn.functional.silu(gate, inplace=True).mul_(up)


class MoELayerQuantizer:
    """Quantise the experts [e_begin, e_begin + n_local) of one MoE layer on the current CUDA device."""

    def __init__(self, cfg: MoEQuantConfig):
        self.cfg = cfg
        self.inversion_free = False
        self._status = None

    # ---- one family of matrices sharing per-slot Hessians -------------------------------------
    def _factor(self, H, n_samples, Ws):
        """H [nu,C,C] (consumed: overwritten by U).  Ws: list of weight batches [nu,R,C] that share H.
        Returns (U, udiag, perm32, info, per-batch wzero handling done)."""
        cfg = self.cfg
        nu, C, _ = H.shape
        diag, pruned, invalid = ops.hessian_scan(H, n_samples)
        if cfg.quantization_order == "activation":
            perm32 = torch.argsort(diag, dim=1, descending=True).to(torch.int32).contiguous()
        else:
            perm32 = None
        for W in Ws:
            ops.weight_apply_pruned(W, pruned)
        wz = [ops.weight_zero_cols(W) for W in Ws]
        shared = all(torch.equal(wz[0], w) for w in wz[1:])
        outs = []
        groups = [wz[0]] if shared else wz
        for gi, wzero in enumerate(groups):
            last = gi == len(groups) - 1
            A, _, _ = ops.hessian_gather_damp(H, perm32, pruned, wzero, invalid, cfg.rel_damp)
            if self.inversion_free:
                # factor only: the solver works from the scaled reverse-Cholesky factor (form = 1)
                U, udiag, info = ops.chol_factor(A)
            else:
                # the last group may overwrite H with U; earlier groups need H intact
                U, udiag, info = ops.chol_inv_upper(A, U=H if last else None, zero_lower=False)
                del A
            outs.append((U, udiag, info))
        if shared:
            outs = outs * len(Ws)
        return outs, perm32

    def _solve_family(self, H, n_samples, Ws):
        cfg = self.cfg
        sparse = cfg.algorithm == "sparsegptq"
        cand = None
        if cfg.quantization_scale == "mse":
            cand = torch.linspace(1.0, cfg.mse_max_shrink, cfg.mse_grid, dtype=torch.float32, device=H.device)
        # the inversion-free form needs 16-byte rows in the solver's work layout
        # (dense GPTQ only: the 1:4 mask choice of SparseGPT is a near-tie argmax and reacts to the different
        # rounding of that form, so the sparse path keeps the reference's form)
        self.inversion_free = (bool(cfg.inversion_free) and not sparse
                               and all(W.shape[1] % 4 == 0 and W.shape[2] % 4 == 0 for W in Ws))
        factors, perm32 = self._factor(H, n_samples, Ws)
        results = []
        for W, (U, udiag, info) in zip(Ws, factors):
            nb, R, C = W.shape
            scales, qzeros = ops.quant_grid(W.view(nb * R, C), cfg.group_size, cfg.bits, cfg.symmetric, cand,
                                            cfg.mse_norm)
            out = ops.gptq_solve_batched(W, U, scales, qzeros, cfg.group_size, cfg.bits, perm=perm32,
                                         udiag=udiag if sparse else None, sparse14=sparse, status=self._status,
                                         form=1 if self.inversion_free else 0)
            q, M = out if sparse else (out, None)
            G = (C + cfg.group_size - 1) // cfg.group_size
            res = {"qweight": q, "scales": scales.view(nb, R, G), "qzeros": qzeros.view(nb, R, G), "info": info,
                   "perm": perm32}
            if sparse:
                res["M"] = M
            if cfg.pack:
                res.update(self._pack(q, res["scales"], res["qzeros"], M))
            results.append(res)
        return results

    def _pack(self, q, scales, qzeros, M):
        cfg = self.cfg
        nb, R, C = q.shape
        if cfg.algorithm == "sparsegptq":
            # one scale per 32 columns: a group scale repeated gs/32 times (quant.py:438-440 assumes gs == 32)
            rep = cfg.group_size // 32
            G32 = (C + 31) // 32
            packed = []
            for b in range(nb):
                s32 = scales[b].repeat_interleave(rep, dim=1)[:, :G32].transpose(0, 1).contiguous()
                packed.append(ops.pack_sparse14(q[b], M[b], s32))
            return {"wpair": torch.stack(packed)}
        return {"weight_packed": ops.pack_int4(q, qzeros.reshape(-1), cfg.group_size),
                "weight_scale": scales.to(torch.float16)}

    # ---- the layer ----------------------------------------------------------------------------------
    @torch.no_grad()
    def quantize_experts(self, X: torch.Tensor, topk_ids: Optional[torch.Tensor], Wg: torch.Tensor,
                         Wu: torch.Tensor, Wd: torch.Tensor, e_begin: int = 0, dense_tail: int = 0):
        """X [T,Hd] bf16; topk_ids [T,k] int32 (global expert ids); Wg/Wu [n,I,Hd], Wd [n,Hd,I] hold the experts
        this rank owns: first the routed experts e_begin.., then `dense_tail` experts that see every token
        (shared experts).  The weight tensors are updated in place only where a dead input channel forces a
        column to zero.  Returns {"gate": .., "up": .., "down": .., "counts": ..} with per-matrix results."""
        cfg = self.cfg
        n_local = Wg.shape[0]
        n_routed = n_local - dense_tail
        T, Hd = X.shape
        I = Wg.shape[1]
        dev = X.device
        # ---- routing lists for the local experts
        parts_counts, parts_lists = [], []
        if n_routed > 0:
            counts, offsets, lists = ops.route_build_lists(topk_ids, e_begin, n_routed)
            parts_counts.append(counts.to(torch.int64))
            total_routed = offsets[-1:]
        else:
            lists = torch.empty(0, dtype=torch.int32, device=dev)
            total_routed = torch.zeros(1, dtype=torch.int64, device=dev)
        if dense_tail > 0:
            parts_counts.append(torch.full((dense_tail,), T, dtype=torch.int64, device=dev))
        counts64 = torch.cat(parts_counts)
        offsets = torch.zeros(n_local + 1, dtype=torch.int64, device=dev)
        offsets[1:] = torch.cumsum(counts64, 0)
        offsets_host = offsets.cpu()
        n_routed_tok = int(offsets_host[n_routed])
        if dense_tail > 0:
            ar = torch.arange(T, dtype=torch.int32, device=dev)
            lists = torch.cat([lists[:n_routed_tok]] + [ar] * dense_tail)
        lists = lists.contiguous()
        # ---- down-projection inputs (packed by expert)
        act = swiglu_expert_forward(X, lists, offsets_host, Wg, Wu)

        chunk = cfg.expert_chunk if cfg.expert_chunk > 0 else n_local
        res = {"gate": [], "up": [], "down": []}
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._status = status
        for c0 in range(0, n_local, chunk):
            c1 = min(n_local, c0 + chunk)
            nb = c1 - c0
            offs = offsets[c0:c1 + 1].contiguous()
            n_samples = counts64[c0:c1].contiguous()
            H1 = torch.empty((nb, Hd, Hd), dtype=torch.float32, device=dev)
            ops.hessian_grouped(X, Hd, lists, offs, H1, mirror=True, status=status)
            g, u = self._solve_family(H1, n_samples, [Wg[c0:c1], Wu[c0:c1]])
            del H1
            H2 = torch.empty((nb, I, I), dtype=torch.float32, device=dev)
            ops.hessian_grouped(act, I, None, offs, H2, mirror=True, status=status)
            (d,) = self._solve_family(H2, n_samples, [Wd[c0:c1]])
            del H2
            res["gate"].append(g)
            res["up"].append(u)
            res["down"].append(d)
        out = {k: _cat_results(v) for k, v in res.items()}
        out["counts"] = counts64
        out["status"] = status
        return out


def _cat_results(parts):
    if len(parts) == 1:
        return parts[0]
    out = {}
    for k in parts[0]:
        vals = [p[k] for p in parts]
        out[k] = None if vals[0] is None else torch.cat(vals, 0)
    return out
