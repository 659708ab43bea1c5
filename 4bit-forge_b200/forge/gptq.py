"""GPTQ handle with the reference's interface (forge/gptq.py:10-276) over the sm_100a engine.

Same constructor, public methods (`update`, `quantize`, `reset`, `_is_owner`), attributes (`layer`, `H`,
`num_samples`, `perm`, `perm_inv`, `pruned_ids`, `issue_non_invertible`) and return values.  What differs
is where the work happens:

* `update` runs the tcgen05 Hessian kernel on bf16 activations (fp32 accumulation) and never syncs the
  host; the reference upcasts to fp32, calls addmm_ and reads `num_samples.item()` every call.
* `_prep` / `_h_factor` use the scan + gather/damp kernels and the batched Cholesky (batch of one) and do not
  read anything back either: the NaN / empty / not-positive-definite fall-backs of the reference
  (forge/gptq.py:96-98, :172-175) happen inside the kernels.  `quantize()` ends with ONE host read, of the
  status word of the bounded waits and bounds checks; `issue_non_invertible` reads the factorisation's info
  flag when (and only when) a caller looks at it.
* `quantize` feeds the fused column solver with per-group scales and the permutation directly instead
  of expanding two [C,R] fp32 tensors (forge/gptq.py:251-252); `_solver` keeps the reference's
  expanded-operand form for callers that use it.

Activations are taken in bf16, the calibration dtype of the models the reference targets; other dtypes
are rounded to bf16 first.
"""
from __future__ import annotations

import uuid

import torch
import torch.nn as nn
from torch import Tensor

from forge import ops
from forge.backend.cuda import kernels


class GPTQ(object):
    def __init__(self,
                 layer: nn.Module,
                 bits: int = 4,
                 group_size: int = 128,
                 symmetric: bool = False,
                 quantization_scale: str = "mse",
                 quantization_order: str = "activation",
                 rel_damp: float = 1e-2,
                 algorithm: str = "gptq",
                 owner=None,
                 device=None):
        self.layer = layer
        self.W = self.layer.weight.clone()  # (R, C)
        self.device = device if device is not None else self.W.device
        self.H = None
        self.num_samples = torch.zeros((), device=self.device, dtype=torch.int64)
        self.bits = bits
        self.group_size = group_size
        self.symmetric = symmetric
        self.quantization_scale = quantization_scale
        self.quantization_order = quantization_order
        self.rel_damp = rel_damp
        if algorithm not in ("gptq", "sparsegptq"):
            raise RuntimeError(f"algorithm={algorithm!r} is not part of the solver path (gptq / sparsegptq)")
        self.algorithm = algorithm
        self.owner = owner if owner is not None else self

        self.perm = None
        self.pruned_ids = None
        self.prepared = False
        self.perm_inv = None
        self._info = None
        self._issue_override = None
        self._status = None
        self._invalid = None
        self.id = uuid.uuid4()

    # the reference sets this attribute in _h_factor after reading info.item() (forge/gptq.py:172-175); here the
    # flag stays on the device until somebody asks
    @property
    def issue_non_invertible(self):
        if self._issue_override is not None:
            return self._issue_override
        return self._info is not None and int(self._info.item()) > 0

    @issue_non_invertible.setter
    def issue_non_invertible(self, value):
        self._issue_override = bool(value)

    def _is_owner(self):
        return self.id == self.owner.id

    @torch.no_grad()
    def reset(self):
        self.W = self.layer.weight.clone()
        self.H = None
        self.num_samples = torch.zeros((), device=self.device, dtype=torch.int64)
        self.prepared = False
        self.perm = None
        self.pruned_ids = None
        self.perm_inv = None
        self._status = None
        self._info = None
        self._issue_override = None
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------ Hessian (forge/gptq.py:62-80)
    @torch.no_grad()
    def update(self, X: Tensor):
        if not self._is_owner():
            return
        o = self.owner
        C = int(o.W.shape[-1])
        X = X.reshape(-1, X.shape[-1])
        n = int(X.shape[0])
        if n == 0:
            return
        X = X.to(device=o.device, dtype=torch.bfloat16).contiguous()
        if o.H is None:
            o.H = torch.empty((C, C), device=o.device, dtype=torch.float32)  # beta = 0: overwritten, not read
        offsets = torch.tensor([0, n], dtype=torch.int64).to(o.device, non_blocking=True)
        if o._status is None:
            o._status = torch.zeros(1, dtype=torch.int32, device=o.device)
        ops.hessian_grouped(X, C, None, offsets, o.H.view(1, C, C), n_prev=o.num_samples.view(1), mirror=True,
                            simt=(C % 8 != 0) or (X.stride(0) % 8 != 0), status=o._status)
        ops.counts_add(o.num_samples.view(1), offsets)

    # ------------------------------------------------------------------ prep (forge/gptq.py:83-126)
    def _copy_from_owner(self):
        o = self.owner
        self.H = o.H.clone()
        self.pruned_ids = o.pruned_ids.clone()
        self.perm = o.perm.clone()
        self.perm_inv = o.perm_inv.clone()
        self._zero_pruned(self)
        self.num_samples = o.num_samples.clone()
        self.prepared = True

    @staticmethod
    def _zero_pruned(h):
        R, C = h.W.shape
        if h.W.dtype not in (torch.float32, torch.bfloat16):
            h.W = h.W.to(torch.float32)
        h.W = h.W.contiguous()
        ops.weight_apply_pruned(h.W.view(1, R, C), h.pruned_ids.to(torch.uint8).view(1, C).contiguous())

    @torch.no_grad()
    def _prep(self):
        if self._is_owner() and self.prepared:
            return
        if (not self._is_owner()) and self.owner.prepared and (not self.prepared):
            self._copy_from_owner()
            return
        o = self.owner
        C = int(o.W.shape[-1])
        if o.H is None:
            o.H = torch.eye(C, device=o.device, dtype=torch.float32)
            n_samples = torch.zeros(1, dtype=torch.int64, device=o.device)
        else:
            n_samples = o.num_samples.view(1)
        diag, pruned, invalid = ops.hessian_scan(o.H.view(1, C, C), n_samples)
        o.pruned_ids = pruned.view(C).to(torch.bool)
        if o.quantization_order == "activation":
            o.perm = torch.argsort(diag.view(C), descending=True)
        else:
            o.perm = torch.arange(C, device=o.device)
        o.perm_inv = torch.argsort(o.perm)
        self._zero_pruned(o)
        # H <- H'[perm][:, perm] with the empty / NaN / dead-column fix-ups folded in
        _, Hp, _ = ops.hessian_gather_damp(o.H.view(1, C, C), o.perm.to(torch.int32).view(1, C).contiguous(), pruned,
                                           None, invalid, 0.0, want_hp=True)
        o.H = Hp.view(C, C)
        o.prepared = True
        if (not self._is_owner()) and (not self.prepared):
            self._copy_from_owner()

    # ------------------------------------------------------------------ quantize (forge/gptq.py:129-139)
    @torch.no_grad()
    def quantize(self):
        self._prep()
        scales, qzeros = self._quant_grid()
        A = self._h_factor()
        R, C = self.W.shape
        perm32 = self.perm.to(torch.int32).view(1, C).contiguous()
        sparse = self.algorithm == "sparsegptq"
        # when the factorisation failed the kernel has already written U = I, udiag = 1 (the reference's fall-back)
        U = self._U_norm
        st = self.owner._status
        if st is None:
            st = torch.zeros(1, dtype=torch.int32, device=self.W.device)
        out = ops.gptq_solve_batched(self.W.view(1, R, C), U.view(1, C, C), scales, qzeros, int(self.group_size),
                                     int(self.bits), perm=perm32,
                                     udiag=self._udiag.view(1, C) if sparse else None, sparse14=sparse, status=st)
        code = int(st.item())       # the one host read of quantize()
        if code != 0:
            raise RuntimeError("forge.gptq: " + ("a bounded device-side wait ran out (FORGE_ERR_TIMEOUT)" if code == 3
                                                else f"a kernel reported status {code}") + "; the codes are not valid")
        if sparse:
            q, M = out
            return q.view(R, C), scales, qzeros, M.view((C + 31) // 32, R).view(torch.uint32)
        return out.view(R, C), scales, qzeros

    # ------------------------------------------------------------------ factor (forge/gptq.py:142-177)
    @torch.no_grad()
    def _h_factor(self):
        R, C = self.W.shape
        wzero = ops.weight_zero_cols(self.W.view(1, R, C))
        # damp in place like the reference (H[zero_cols] fix + H[i,i] += damp), and build the reversed copy
        A, Hp, _ = ops.hessian_gather_damp(self.H.view(1, C, C), None, None, wzero, None, float(self.rel_damp),
                                           want_hp=True)
        self.H = Hp.view(C, C)
        U, udiag, info = ops.chol_inv_upper(A, zero_lower=True)
        U = U.view(C, C)
        self._udiag = udiag.view(C)
        self._U_norm = U
        self._info = info
        self._issue_override = None
        if self.algorithm == "sparsegptq":
            # the reference returns the un-normalised factor here (:165-170); after a failed factorisation the kernel
            # left U = I and udiag = 1, so this is the identity then, like the reference's fall-back
            return U * self._udiag[:, None]
        return U

    # ------------------------------------------------------------------ grid (forge/gptq.py:181-227)
    @torch.no_grad()
    def _quant_grid(self, max_shrink: float = 0.2, n_grid: int = 100, norm: float = 2.4):
        if self.W.dtype not in (torch.float32, torch.bfloat16):
            self.W = self.W.to(torch.float32)
        W = self.W.contiguous()
        R, C = W.shape
        G = (C + self.group_size - 1) // self.group_size
        cand = None
        if self.quantization_scale == "mse":
            cand = torch.linspace(1.0, max_shrink, n_grid, dtype=torch.float32, device=W.device)
        scales, qzeros = ops.quant_grid(W, int(self.group_size), int(self.bits), bool(self.symmetric), cand, float(norm))
        self.G = int(G)
        return scales, qzeros

    # ------------------------------------------------------------------ solver (forge/gptq.py:231-276)
    @torch.no_grad()
    def _solver(self, A, W, scales, qzeros):
        """Reference operand form: W [C,R] already permuted, per-group meta expanded to [C,R]."""
        C, R = W.shape
        s_el = scales.clone().view(R, self.G).repeat_interleave(self.group_size, dim=1)[:, :C].transpose(-2, -1)[self.perm].contiguous()
        z_el = qzeros.clone().view(R, self.G).repeat_interleave(self.group_size, dim=1)[:, :C].transpose(-2, -1)[self.perm].contiguous()
        Wf = W.to(torch.float32).contiguous()
        if self.algorithm == "gptq":
            return kernels.gptq_solver(Wf, A, s_el, z_el, self.bits)
        return kernels.sparsegptq14_solver(Wf, A.contiguous(), s_el, z_el, self.bits)
