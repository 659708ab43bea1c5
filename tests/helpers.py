"""Shared helpers for the parity tests."""
import numpy as np
import torch


def bf16_from_bits(arr) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.bfloat16)


def golden_case(golden, name):
    pre = name + "/"
    return {k[len(pre):]: v for k, v in golden.items() if k.startswith(pre)}


def case_inputs(c):
    seed, R, C, act, sparse = [int(v) for v in c["meta"]]
    W = bf16_from_bits(c["W_bits"]).view(R, C)
    Xs = [bf16_from_bits(c[f"X{b}_bits"]).view(-1, C) for b in range(int(c["n_batches"]))]
    return dict(R=R, C=C, order="activation" if act else "default",
                algorithm="sparsegptq" if sparse else "gptq", W=W, Xs=Xs, rel_damp=float(c["rel_damp"]))


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def random_spd(C, seed, cond=1e3):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(4 * C, C, generator=g) * torch.exp(torch.randn(C, generator=g))
    H = (X.T @ X) * (2.0 / (4 * C))
    return H.float()
