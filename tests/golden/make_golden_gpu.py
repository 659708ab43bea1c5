"""Golden vectors from the reference's OWN CUDA kernels, run on a B200.

    python oracle/ref_build.py <reference checkout>        # on the build machine: oracle/_ref/forge_ref_kernels.so
    python tests/golden/make_golden_gpu.py [out dir]       # on a GPU machine: writes ref_kernels_b200.npz (solver-path
                                                           # kernels) and ref_sparse14_gemm_b200.npz (inference GEMM
                                                           # over the Wpair layout) into tests/golden/ (or out dir)

Every case stores its inputs (small) next to the reference's outputs, so that the CPU tests can replay the oracle on
exactly the same numbers without the reference and without a GPU.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import ref_build  # noqa: E402


def cases(ref, dev):
    out = {}
    g = torch.Generator().manual_seed(2024)
    # ---- scale grid (A5 / A6): 96 groups of 128 and 64 groups of 32, with outliers, an all-zero group, a constant group
    for tag, gs, n in (("g128", 128, 96), ("g32", 32, 64)):
        X = torch.randn(n, gs, generator=g) * 0.02
        X[::7] *= torch.where(torch.rand(X[::7].shape, generator=g) < 0.03, 12.0, 1.0)
        X[3] = 0.0
        X[5] = 0.0123
        out[f"grid_{tag}_X"] = X
        for sym in (False, True):
            s, z = ref.build_group_meta_packed(X.to(dev), 4, sym)
            out[f"grid_{tag}_sym{int(sym)}_scales"], out[f"grid_{tag}_sym{int(sym)}_qzeros"] = s.cpu(), z.cpu()
            cand = torch.linspace(1.0, 0.2, 100)
            s2, z2 = ref.mse_scale_groups_packed(X.to(dev), s.clone(), z.clone(), cand.to(dev), 2.4, 4, sym)
            out[f"mse_{tag}_sym{int(sym)}_scales"], out[f"mse_{tag}_sym{int(sym)}_qzeros"] = s2.cpu(), z2.cpu()
    # ---- solvers (A8 / A9): C = 160 (five 32-column blocks), R = 96, group size 32, asymmetric grid for gptq
    C, R, gs = 160, 96, 32
    W = torch.randn(R, C, generator=g) * 0.02
    A = torch.randn(C, 4 * C, generator=g)
    H = A @ A.T / (4 * C) + 0.05 * torch.eye(C)
    Hinv = torch.linalg.inv(H.double())
    Uraw = torch.linalg.cholesky(Hinv, upper=True).float()
    Unorm = Uraw / Uraw.diag()[:, None]
    for sym, name in ((False, "gptq"), (True, "sparse")):
        s, z = ref.build_group_meta_packed(W.reshape(-1, gs).contiguous().to(dev), 4, sym)
        G = C // gs
        s_el = s.cpu().view(R, G).repeat_interleave(gs, 1).T.contiguous()       # [C, R]
        z_el = z.cpu().view(R, G).repeat_interleave(gs, 1).T.contiguous()
        Wt = W.T.contiguous()
        out[f"{name}_Wt"], out[f"{name}_s"], out[f"{name}_z"] = Wt, s_el, z_el
        if name == "gptq":
            out["gptq_U"] = Unorm
            q = ref.gptq_solver(Wt.clone().to(dev), Unorm.to(dev), s_el.to(dev), z_el.to(dev), 4)
            out["gptq_q"] = q.cpu()
        else:
            out["sparse_U"] = Uraw
            q, M = ref.sparsegptq14_solver(Wt.clone().to(dev), Uraw.clone().to(dev), s_el.to(dev), z_el.to(dev), 4)
            out["sparse_q"], out["sparse_M"] = q.cpu(), M.cpu().view(torch.int32)
            # ---- packer (A10) on the solver's own output, one scale per 32 columns
            qrc = q.cpu().T.contiguous()
            s32 = s.cpu().view(R, G).T.contiguous()                              # [G32, R]
            wp = ref.pack_sparsegptq14_to_u64x2(qrc.to(dev), M, s32.to(dev))
            out["pack_q_rc"], out["pack_scales"] = qrc, s32
            out["pack_wpair"] = wp.cpu().view(torch.int64)
    return out


def gemm_cases(ref, dev):
    """kernels.sparsegptq14_gemm (forge/backend/cuda/sparse14_gemm.cu) on Wpair words made by the reference's own
    packer: C a multiple of 64 and not, R not a multiple of the CTA's 128 rows, token counts around every tile size of
    the launcher's heuristic (1, 2, 3, 4 tokens per CTA)."""
    out = {}
    g = torch.Generator().manual_seed(4242)
    for tag, (R, C, Ns) in {"c256": (130, 256, (1, 5)), "c160": (96, 160, (3, 70, 300)), "c320": (40, 320, (800,))}.items():
        G32 = (C + 31) // 32
        q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
        pos = torch.randint(0, 4, (G32, R, 8), generator=g)                       # surviving channel of each group
        keep = (torch.rand(G32, R, 8, generator=g) > 0.1)                         # a few groups fully pruned
        M = ((keep.long() << (4 * torch.arange(8) + pos)).sum(-1)).to(torch.int64)
        M = (M & 0xFFFFFFFF).to(torch.int32)
        s32 = (torch.rand(G32, R, generator=g) * 0.01 + 1e-3).float()
        wp = ref.pack_sparsegptq14_to_u64x2(q.to(dev), M.to(dev).view(torch.uint32), s32.to(dev))
        out[f"{tag}_wpair"] = wp.cpu().view(torch.int64)
        for N in Ns:
            X = (torch.randn(N, C, generator=g) * 0.7).to(torch.bfloat16)
            Y = ref.sparsegptq14_gemm(wp, X.to(dev))
            out[f"{tag}_X{N}"] = X.view(torch.int16)
            out[f"{tag}_Y{N}"] = Y.cpu().contiguous().view(torch.int16)
    return out


def main():
    ref = ref_build.load_built()
    if ref is None:
        raise SystemExit("oracle/_ref/forge_ref_kernels.so is missing: run oracle/ref_build.py first")
    dev = torch.device("cuda")
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden")
    os.makedirs(out_dir, exist_ok=True)
    for name, fn in (("ref_kernels_b200.npz", cases), ("ref_sparse14_gemm_b200.npz", gemm_cases)):
        arrays = {k: v.numpy() for k, v in fn(ref, dev).items()}
        path = os.path.join(out_dir, name)
        np.savez_compressed(path, **arrays)
        print(path, os.path.getsize(path), "bytes;", torch.cuda.get_device_name(0))


if __name__ == "__main__":
    main()
