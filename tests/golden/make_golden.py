"""Generate golden vectors from the reference's own Python code (CPU only).

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

Imports forge.gptq.GPTQ from the reference checkout given on PYTHONPATH (its CUDA extension resolves
to a raising stub without a GPU, which is fine: only the torch half is exercised) and records, for
small seeded inputs, the Hessian after update(), the permutation and permuted Hessian after _prep(),
and the factor returned by _h_factor().  The arrays land in tests/golden/gptq_python_half.npz; the
inputs are stored too so that the checked code sees identical bits.

The reference's scale grid, column solver and packers exist only as CUDA kernels and cannot be run
here, so no golden vectors exist for them.
"""
import os
import sys

import numpy as np
import torch

from forge.gptq import GPTQ  # the reference's class (PYTHONPATH)

HERE = os.path.dirname(os.path.abspath(__file__))


class Layer:
    def __init__(self, w):
        self.weight = w


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().copy()


def make_case(seed, R, C, n_batches, order, algorithm, dead_col=None, zero_w_col=None, rel_damp=1e-2):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16)
    if zero_w_col is not None:
        W[:, zero_w_col] = 0
    ch = torch.exp(torch.randn(C, generator=g))
    Xs = []
    for b in range(n_batches):
        n = 48 + 16 * b
        X = (torch.randn(n, C, generator=g) * ch).to(torch.bfloat16)
        if dead_col is not None:
            X[:, dead_col] = 0
        Xs.append(X)
    h = GPTQ(Layer(W), bits=4, group_size=32, symmetric=True, quantization_scale="absmax",
             quantization_order=order, rel_damp=rel_damp, algorithm=algorithm, device="cpu")
    for X in Xs:
        h.update(X)
    H_acc = h.H.clone()
    n_samples = int(h.num_samples.item())
    h._prep()
    H_prep = h.H.clone()
    perm = h.perm.clone()
    pruned = h.pruned_ids.clone()
    W_prep = h.W.clone()
    h.issue_non_invertible = False
    U = h._h_factor().clone()
    out = {
        "W_bits": bf16_bits(W), "H_acc": H_acc.numpy(), "H_prep": H_prep.numpy(), "perm": perm.numpy(),
        "pruned": pruned.numpy(), "W_prep_bits": bf16_bits(W_prep), "U": U.numpy(),
        "n_samples": np.int64(n_samples), "n_batches": np.int64(n_batches),
        "non_invertible": np.int64(int(h.issue_non_invertible)),
        "meta": np.array([seed, R, C, 1 if order == "activation" else 0, 1 if algorithm == "sparsegptq" else 0]),
        "rel_damp": np.float64(rel_damp),
    }
    for b, X in enumerate(Xs):
        out[f"X{b}_bits"] = bf16_bits(X)
    return out


def main():
    cases = {
        "plain": make_case(1, 24, 64, 1, "default", "gptq"),
        "actorder_multibatch": make_case(2, 16, 96, 3, "activation", "gptq"),
        "deadcol_zerow": make_case(3, 16, 64, 2, "activation", "gptq", dead_col=5, zero_w_col=9),
        "sparse_unnormalised": make_case(4, 16, 64, 1, "default", "sparsegptq"),
    }
    # empty Hessian -> identity (forge/gptq.py:96-98)
    h = GPTQ(Layer((torch.ones(4, 32) * 0.01).to(torch.bfloat16)), group_size=32, symmetric=True,
             quantization_scale="absmax", quantization_order="activation", device="cpu")
    h._prep()
    cases["empty"] = {"H_prep": h.H.numpy().copy(), "perm": h.perm.numpy().copy()}
    flat = {}
    for name, d in cases.items():
        for k, v in d.items():
            flat[f"{name}/{k}"] = v
    np.savez_compressed(os.path.join(HERE, "gptq_python_half.npz"), **flat)
    print("wrote", len(flat), "arrays")


if __name__ == "__main__":
    main()
