"""CPU oracle: a restatement of the reference GPTQ / SparseGPT path.

TEST INFRASTRUCTURE ONLY.  Imported by tests/, the smoke check and the
benchmark's CPU-baseline leg as the checker / reported baseline.  The shipped
package never imports it.

The Python half of the reference (Hessian running mean, column pruning,
activation ordering, damped Cholesky -> upper Cholesky of the inverse) is
restated with the same torch calls in the same order; tests/golden holds
outputs of the reference's own code for it (made by tests/golden/make_golden.py
with the reference importable), so that half is pinned.  The CUDA-only half
(scale grid, column solver, packers) is restated in oracle/forge_oracle.c and
pinned against outputs of the reference's own kernels, compiled for sm_100a
from the reference checkout (oracle/ref_build.py) and run on a B200
(tests/golden/make_golden_gpu.py -> tests/golden/ref_kernels_b200.npz).

Citations are paths inside the reference project.
"""
from __future__ import annotations

import ctypes
import math
import os
import sys

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))


def _load_build():
    """oracle/build.py by path (a plain `import build` could pick up another build.py on sys.path)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("forge_oracle_build", os.path.join(_HERE, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_build = _load_build()

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build()
        L = ctypes.CDLL(path)
        L.fo_num_threads.restype = ctypes.c_int
        L.fo_mse_grid.restype = ctypes.c_int
        _lib = L
    return _lib


def _p(t: torch.Tensor):
    assert t.is_contiguous() and t.device.type == "cpu"
    return ctypes.c_void_p(t.data_ptr())


# --------------------------------------------------------------------------- #
# CUDA-only half (C restatement)
# --------------------------------------------------------------------------- #
def build_group_meta_packed(X: torch.Tensor, bits: int, symmetric: bool):
    """kernels.build_group_meta_packed, forge/backend/cuda/quant_grid.cu:186-224."""
    X = X.to(torch.float32).contiguous()
    RG, gs = X.shape
    scales = torch.empty(RG, dtype=torch.float32)
    qzeros = torch.empty(RG, dtype=torch.float32)
    lib().fo_absmax_grid(_p(X), ctypes.c_int64(RG), ctypes.c_int64(gs), int(bits), int(bool(symmetric)),
                         _p(scales), _p(qzeros))
    return scales, qzeros


def mse_scale_groups_packed(X, scales, qzeros, candidates, norm, bits, symmetric):
    """kernels.mse_scale_groups_packed, forge/backend/cuda/quant_grid.cu:227-287 (in place + returned)."""
    X = X.to(torch.float32).contiguous()
    RG, gs = X.shape
    candidates = candidates.to(torch.float32).contiguous()
    rc = lib().fo_mse_grid(_p(X), _p(scales), _p(qzeros), _p(candidates), ctypes.c_int64(RG),
                           ctypes.c_int64(gs), ctypes.c_int64(candidates.numel()), int(bits),
                           ctypes.c_float(float(norm)), int(bool(symmetric)))
    if rc != 0:
        raise RuntimeError(f"Unsupported group_size={gs} (expected 32/64/128)")
    return scales, qzeros


def gptq_solver(W, U, scales, qzeros, bits, block: int = 32):
    """kernels.gptq_solver, forge/backend/cuda/solver.cu:99-154.  W [C,R] is mutated to the dequantised weights."""
    assert W.dtype == torch.float32 and W.is_contiguous()
    C, R = W.shape
    U = U.contiguous()
    scales = scales.contiguous()
    qzeros = qzeros.contiguous()
    q = torch.empty((C, R), dtype=torch.uint8)
    lib().fo_gptq_solve(_p(W), _p(U), None, _p(scales), _p(qzeros), int(bits), ctypes.c_int64(R),
                        ctypes.c_int64(C), int(block), 0, _p(q), None)
    return q


def sparsegptq14_solver(W, U, scales, qzeros, bits):
    """kernels.sparsegptq14_solver, forge/backend/cuda/solver_sparsegptq14.cu:142-200.
    U is normalised in place by its diagonal like the reference (:154-155)."""
    assert W.dtype == torch.float32 and W.is_contiguous()
    C, R = W.shape
    assert U.is_contiguous()
    uinv = U.diagonal().reciprocal().contiguous()
    U.mul_(uinv.unsqueeze(1))
    scales = scales.contiguous()
    qzeros = qzeros.contiguous()
    q = torch.empty((C, R), dtype=torch.uint8)
    M = torch.zeros(((C + 31) // 32, R), dtype=torch.int32)
    lib().fo_gptq_solve(_p(W), _p(U), _p(uinv), _p(scales), _p(qzeros), int(bits), ctypes.c_int64(R),
                        ctypes.c_int64(C), 32, 1, _p(q), _p(M))
    return q, M.view(torch.uint32) if hasattr(torch, "uint32") else M


def pack_sparsegptq14_to_u64x2(qweight_rc, M, scales):
    """kernels.pack_sparsegptq14_to_u64x2, forge/backend/cuda/bitpacking_sparsegptq14.cu:110-175.
    qweight_rc [R,C] u8, M [G32,R] u32, scales [G32,R] f32 -> [G2,R,2] u64 (returned as int64 bit pattern)."""
    R, C = qweight_rc.shape
    q_cr = qweight_rc.transpose(0, 1).contiguous()
    G32 = (C + 31) // 32
    assert M.shape == (G32, R) and scales.shape == (G32, R)
    Mi = M.contiguous().view(torch.int32) if M.dtype != torch.int32 else M.contiguous()
    scales = scales.to(torch.float32).contiguous()
    G2 = (G32 + 1) // 2
    out = torch.empty((G2, R, 2), dtype=torch.int64)
    lib().fo_pack_sparse14(_p(q_cr), _p(Mi), _p(scales), ctypes.c_int64(C), ctypes.c_int64(R),
                           ctypes.c_int64(G32), _p(out))
    return out


def sparsegptq14_gemm(wpair: torch.Tensor, X: torch.Tensor) -> torch.Tensor:
    """kernels.sparsegptq14_gemm, forge/backend/cuda/sparse14_gemm.cu:49-140, :282-374.  wpair [G2,R,2] (uint64 bit
    pattern as int64), X bf16 [N,C] -> Y bf16 [N,R]."""
    G2, R, _ = wpair.shape
    N, C = X.shape
    assert G2 == (C + 63) // 64
    w = wpair.contiguous().view(torch.int64)
    xb = X.contiguous().view(torch.int16)
    y = torch.empty((N, R), dtype=torch.int16)
    lib().fo_sparse14_gemm(_p(w), _p(xb), ctypes.c_int64(N), ctypes.c_int64(R), ctypes.c_int64(C), _p(y))
    return y.view(torch.bfloat16)


def pack_int4(qweight_rc, zeros_rg, group_size):
    """weight_packed of pack_quantized.py:279-313 via compressed_tensors.pack_to_int32 semantics."""
    q = qweight_rc.to(torch.uint8).contiguous()
    R, C = q.shape
    z = zeros_rg.to(torch.float32).contiguous()
    out = torch.empty((R, (C + 7) // 8), dtype=torch.int32)
    lib().fo_pack_int4(_p(q), _p(z), ctypes.c_int64(R), ctypes.c_int64(C), ctypes.c_int64(group_size), _p(out))
    return out


def pack_weight(weight: dict, bits: int, sym: bool, group_size=None) -> dict:
    """pack_quantized.py:279-313 restated with the installed compressed_tensors.pack_to_int32 when it is
    importable, else the C restatement (they are checked against each other in the tests)."""
    qweight, scale, zero = weight["qweight"], weight["scale"], weight["zero"]
    group_size = int(group_size or qweight.shape[-1])
    zero_rep = zero.repeat_interleave(group_size, dim=-1).to(torch.int8)[..., : qweight.shape[-1]]
    q_shift = qweight.to(torch.int8) - zero_rep
    try:
        from compressed_tensors.compressors import pack_to_int32
        q_packed = pack_to_int32(q_shift, bits)
    except Exception:  # pragma: no cover
        q_packed = pack_int4(qweight, zero, group_size)
    out = {"weight_packed": q_packed,
           "weight_shape": torch.tensor(qweight.shape, dtype=torch.int64),
           "weight_scale": scale}
    if not sym:
        out["weight_zero_point"] = zero
    return out


# --------------------------------------------------------------------------- #
# Python half (torch restatement of forge/gptq.py)
# --------------------------------------------------------------------------- #
class _W:
    def __init__(self, w):
        self.weight = w


class OracleGPTQ:
    """forge/gptq.py:10-276 on CPU.  Same constructor, attributes and return values."""

    def __init__(self, layer, bits=4, group_size=128, symmetric=False, quantization_scale="mse",
                 quantization_order="activation", rel_damp=1e-2, algorithm="gptq", owner=None, device=None,
                 solver_block=32, kernels=None):
        if isinstance(layer, torch.Tensor):
            layer = _W(layer)
        self.layer = layer
        self.W = layer.weight.clone()
        self.device = device or "cpu"
        self.H = None
        self.num_samples = 0
        self.bits, self.group_size, self.symmetric = bits, group_size, symmetric
        self.quantization_scale, self.quantization_order = quantization_scale, quantization_order
        self.rel_damp, self.algorithm = rel_damp, algorithm
        self.perm = self.perm_inv = self.pruned_ids = None
        self.prepared = False
        self.issue_non_invertible = False
        self.solver_block = solver_block
        # the five kernel operators: the C oracle by default; the reference's own CUDA kernels (oracle/_ref) when the
        # class runs on a GPU as the same-device baseline of the benchmark
        self.k = kernels

    def _op(self, name):
        return getattr(self.k, name) if self.k is not None else globals()[name]

    @torch.no_grad()
    def update(self, X):
        """forge/gptq.py:62-80."""
        X = X.reshape(-1, X.shape[-1]).to(torch.float32)
        n = int(X.shape[0])
        if n == 0:
            return
        total = self.num_samples + n
        alpha = 2.0 / total
        if self.H is None:
            self.H = X.T @ (alpha * X)
        beta = self.num_samples / total
        self.H.addmm_(X.transpose(-2, -1), X, alpha=alpha, beta=beta)
        self.num_samples = total

    @torch.no_grad()
    def _prep(self):
        """forge/gptq.py:83-126 (owner path)."""
        if self.prepared:
            return
        C = int(self.W.shape[-1])
        if self.H is None or self.num_samples == 0 or torch.isnan(self.H).any().item():
            self.H = torch.eye(C, dtype=torch.float32, device=self.W.device)
        self.pruned_ids = torch.diag(self.H) == 0
        self.H[self.pruned_ids, :] = 0
        self.H[:, self.pruned_ids] = 0
        self.H[self.pruned_ids, self.pruned_ids] = 1
        if self.quantization_order == "activation":
            self.perm = torch.argsort(self.H.diag(), descending=True)
        else:
            self.perm = torch.arange(C, device=self.W.device)
        self.perm_inv = torch.argsort(self.perm)
        self.W[:, self.pruned_ids] = 0
        self.prepared = True
        self.H = self.H[self.perm][:, self.perm]

    @torch.no_grad()
    def _h_factor(self):
        """forge/gptq.py:142-177."""
        H = self.H
        C = self.W.shape[-1]
        zero_cols = self.W.clone().eq(0).all(dim=0)
        if zero_cols.any():
            H[zero_cols, :] = 0
            H[:, zero_cols] = 0
            H[zero_cols, zero_cols] = 1.0
        diag = torch.diag(H)
        damp = float(self.rel_damp) * diag.mean()
        H[range(C), range(C)] += damp
        H, info = torch.linalg.cholesky_ex(H, upper=False)
        H = torch.cholesky_inverse(H, upper=False)
        H, info2 = torch.linalg.cholesky_ex(H, upper=True)
        info = info + info2
        if self.algorithm == "gptq":
            H.div_(H.diag()[:, None])
        if info.item() > 0:
            self.issue_non_invertible = True
            H = torch.eye(C, dtype=torch.float32, device=self.W.device)
        return H

    @torch.no_grad()
    def _quant_grid(self, max_shrink=0.2, n_grid=100, norm=2.4):
        """forge/gptq.py:181-227."""
        W = self.W.clone()
        R, C = W.shape
        G = (C + self.group_size - 1) // self.group_size
        pad = G * self.group_size - C
        if pad:
            W = torch.nn.functional.pad(W, (0, pad))
        Wg = W.reshape(R * G, self.group_size).to(torch.float32).contiguous()
        scales, qzeros = self._op("build_group_meta_packed")(Wg, self.bits, self.symmetric)
        if self.quantization_scale == "mse":
            p = torch.linspace(1.0, max_shrink, n_grid, dtype=torch.float32, device=Wg.device)
            scales, qzeros = self._op("mse_scale_groups_packed")(Wg, scales, qzeros, p, float(norm), self.bits,
                                                                 self.symmetric)
        self.G = int(G)
        return scales, qzeros

    @torch.no_grad()
    def _expand(self, t, R, C):
        """forge/gptq.py:251-252: per-group -> per-element [C,R] in permuted order."""
        return t.clone().view(R, self.G).repeat_interleave(self.group_size, dim=1)[:, :C].transpose(-2, -1)[self.perm].contiguous()

    @torch.no_grad()
    def quantize(self):
        """forge/gptq.py:129-139."""
        self._prep()
        scales, qzeros = self._quant_grid()
        A = self._h_factor().contiguous()
        W = self.W.clone().transpose(-2, -1)[self.perm].to(torch.float32).contiguous()
        C, R = W.shape
        s_el, z_el = self._expand(scales, R, C), self._expand(qzeros, R, C)
        if self.algorithm == "sparsegptq":
            q, M = self._op("sparsegptq14_solver")(W, A, s_el, z_el, self.bits)
            self.W_deq_perm = W
            return q[self.perm_inv].transpose(-2, -1).contiguous(), scales, qzeros, M
        if self.k is not None:
            q = self.k.gptq_solver(W, A, s_el, z_el, self.bits)
        else:
            q = gptq_solver(W, A, s_el, z_el, self.bits, block=self.solver_block)
        self.W_deq_perm = W
        return q[self.perm_inv].transpose(-2, -1).contiguous(), scales, qzeros


def dequantize_forge_full(dtype, qweight, scales, qzeros, group_size):
    """forge/utils/engine.py:72-97."""
    R, C = qweight.shape
    G = (C + group_size - 1) // group_size
    s = scales.reshape(-1).view(R, G).repeat_interleave(group_size, dim=1)[:, :C]
    z = qzeros.reshape(-1).view(R, G).repeat_interleave(group_size, dim=1)[:, :C]
    w = (qweight.to(torch.float32) - z.to(torch.float32)) * s.to(torch.float32)
    return w.to(dtype)


def fp8_block_dequant(w_fp8: torch.Tensor, scale_inv: torch.Tensor, dtype=torch.bfloat16):
    """forge/utils/io.py:533-563 and the fp8 branch :864-874:  bf16( fp32(W_fp8) * scale_inv[tile] )."""
    w = w_fp8.to(torch.float32)
    O, I = w.shape
    nO, nI = scale_inv.shape
    assert I % nI == 0
    si = I // nI
    cd = lambda a, b: (a + b - 1) // b
    so = si if cd(O, si) == nO else cd(O, nO)
    rows = torch.arange(O) // so
    cols = torch.arange(I) // si
    return (w * scale_inv.to(torch.float32)[rows][:, cols]).to(dtype)


def recon_loss(W: torch.Tensor, What: torch.Tensor, X: torch.Tensor) -> float:
    """|| X W^T - X What^T ||_F^2 in fp64 on the CPU (the acceptance quantity)."""
    D = (W.to(torch.float64) - What.to(torch.float64))
    Y = X.to(torch.float64) @ D.T
    return float((Y * Y).sum())


def swiglu_down_input(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor) -> torch.Tensor:
    """Down-projection calibration input of one expert: bf16( silu(x Wg^T) * (x Wu^T) ), the projections
    taken in bf16 with fp32 accumulation and rounded to bf16 before the activation (HF MoE block forward,
    which the reference hooks at quant.py:398-406)."""
    g = (x.to(torch.float32) @ wg.to(torch.float32).T).to(torch.bfloat16)
    u = (x.to(torch.float32) @ wu.to(torch.float32).T).to(torch.bfloat16)
    return (torch.nn.functional.silu(g.to(torch.float32)).to(torch.bfloat16) * u)


# --------------------------------------------------------------------------- #
# checkpoint weight materialisation (forge/utils/io.py)
# --------------------------------------------------------------------------- #
_MXFP4_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def int4_packed_dequant(packed: torch.Tensor, scales: torch.Tensor, shape, symmetric=True, scale_is_inv=False):
    """_apply_block_scale, forge/utils/io.py:722-808 (bits = 4, scales [O, I/gs]) in numpy: fp32 [O, I]."""
    O, I = int(shape[0]), int(shape[1])
    w = packed.numpy().astype(np.int64) & 0xFFFFFFFF
    sf = scales.to(torch.float32).numpy()
    if scale_is_inv:
        sf = (np.float32(1.0) / sf).astype(np.float32)
    gs = (O * I) // sf.size
    u = np.stack([(w >> (4 * i)) & 0xF for i in range(8)], axis=-1).reshape(O, I).astype(np.int32)
    if symmetric:
        u = np.where(u >= 8, u - 16, u)
    return torch.from_numpy(u.astype(np.float32) * np.repeat(sf.reshape(O, I // gs), gs, axis=1))


def mxfp4_dequant(blocks_u8: torch.Tensor, scales_u8: torch.Tensor):
    """_dequant_mxfp4_blocks_to_fp with _e8m0_to_scale_fp32, forge/utils/io.py:505-531 in numpy: fp32
    [..., NB*32, rows] (the reference's transpose of the last two dimensions included)."""
    b = blocks_u8.numpy().astype(np.uint8)
    codes = np.stack([b & 0x0F, (b >> 4) & 0x0F], axis=-1).reshape(*b.shape[:-1], 32)
    vals = _MXFP4_MAG[codes & 7]
    vals = np.where((codes & 8) != 0, -vals, vals)
    e = scales_u8.numpy().astype(np.int32)
    with np.errstate(over="ignore"):
        sc = np.where(e == 0, np.float32(2.0 ** -23), np.power(np.float32(2.0), (e - 127).astype(np.float32))).astype(np.float32)
    out = (vals * sc[..., None]).astype(np.float32).reshape(*vals.shape[:-2], vals.shape[-2] * 32)
    return torch.from_numpy(np.ascontiguousarray(np.swapaxes(out, -1, -2)))


def wpair_to_dense(wpair: torch.Tensor, C: int) -> torch.Tensor:
    """The weights a Wpair tensor [G2,R,2] encodes, fp32 [R,C] (exact: bf16 scale times an integer in [-8, 7]); word
    layout of bitpacking_sparsegptq14.cu:58-107 as consumed by sparse14_gemm.cu:96-131."""
    G2, R, _ = wpair.shape
    w = wpair.contiguous().view(torch.int64)
    out = torch.zeros((R, G2 * 64), dtype=torch.float32)
    rows = torch.arange(R)
    for g2 in range(G2):
        for half in range(2):
            u = w[g2, :, half]
            qw = u & 0xFFFFFFFF
            idx = (u >> 32) & 0xFFFF
            sc_bits = ((u >> 48) & 0xFFFF).to(torch.int32) << 16
            scale = sc_bits.view(torch.float32)
            for i in range(8):
                ch = g2 * 64 + half * 32 + 4 * i + ((idx >> (2 * i)) & 3)
                val = (((qw >> (4 * i)) & 0xF).to(torch.float32) - 8.0) * scale
                out[rows, ch] = val
    return out[:, :C].contiguous()


def sparse14_grouped_w13(W13, X, offsets, active):
    """usp14w4a16sym_sm80_fused_moe_w13_gemm's contract (fused_moe_usp14w4a16_gemm.cu:398-439, :722-723, :1028-1084):
    X rows sorted by expert, gate rows then up rows, X2 = bf16(silu(g) * u) from unrounded sums.  The sums are taken
    in fp64 here (the tensor-core summation order of that kernel is unspecified)."""
    E, G2, R, _ = W13.shape
    N, C = X.shape
    I = R // 2
    X2 = torch.zeros((N, I), dtype=torch.bfloat16)
    for e in [int(a) for a in active]:
        s, t = int(offsets[e]), int(offsets[e + 1])
        if t <= s:
            continue
        Wd = wpair_to_dense(W13[e], C).double()
        y = X[s:t].double() @ Wd.T
        g, u = y[:, :I], y[:, I:]
        X2[s:t] = ((g / (1.0 + torch.exp(-g))) * u).to(torch.bfloat16)
    return X2


def sparse14_moe_runtime_forward(w13, w2, hidden_states, topk_ids, topk_weights, chunk_m=256):
    """Sparse14MoERuntime.forward, sparse14_gemm.py:32-65, with the permutation written out (stable sort of the
    (token, slot) pairs by expert = moe_permute) and the weighted un-permute as an fp32 sum rounded once."""
    T, H = hidden_states.shape
    K = topk_ids.shape[1]
    E = w13.shape[0]
    I = w13.shape[2] // 2
    flat = topk_ids.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    tok = order // K
    hs_perm = hidden_states[tok]
    counts = torch.bincount(flat, minlength=E)
    offs = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)])
    out_perm = torch.zeros((T * K, H), dtype=hidden_states.dtype)
    for e in range(E):
        s0, t0 = int(offs[e]), int(offs[e + 1])
        for s in range(s0, t0, chunk_m):
            t = min(s + chunk_m, t0)
            y13 = sparsegptq14_gemm(w13[e], hs_perm[s:t])
            gate, up = y13.split(I, dim=1)
            a2 = torch.nn.functional.silu(gate) * up
            out_perm[s:t] = sparsegptq14_gemm(w2[e], a2.contiguous())
    wts = topk_weights.reshape(-1)[order].float()
    out = torch.zeros((T, H), dtype=torch.float32)
    out.index_add_(0, tok, out_perm.float() * wts[:, None])
    return out.to(hidden_states.dtype)
