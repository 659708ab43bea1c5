"""The oracle's torch half against outputs of the reference's own Python code (tests/golden)."""
import numpy as np
import pytest
import torch

import ref_port as O
from helpers import golden_case, case_inputs

CASES = ["plain", "actorder_multibatch", "deadcol_zerow", "sparse_unnormalised"]


@pytest.mark.parametrize("name", CASES)
def test_python_half_matches_reference(golden, name):
    c = golden_case(golden, name)
    inp = case_inputs(c)
    h = O.OracleGPTQ(inp["W"], bits=4, group_size=32, symmetric=True, quantization_scale="absmax",
                     quantization_order=inp["order"], rel_damp=inp["rel_damp"], algorithm=inp["algorithm"])
    for X in inp["Xs"]:
        h.update(X)
    assert h.num_samples == int(c["n_samples"])
    np.testing.assert_array_equal(h.H.numpy(), c["H_acc"])          # same torch ops, same order: bit-exact
    h._prep()
    np.testing.assert_array_equal(h.perm.numpy(), c["perm"])
    np.testing.assert_array_equal(h.pruned_ids.numpy(), c["pruned"])
    np.testing.assert_array_equal(h.H.numpy(), c["H_prep"])
    U = h._h_factor()
    np.testing.assert_array_equal(U.numpy(), c["U"])
    assert int(h.issue_non_invertible) == int(c["non_invertible"])


def test_empty_hessian_is_identity(golden):
    c = golden_case(golden, "empty")
    h = O.OracleGPTQ((torch.ones(4, 32) * 0.01).to(torch.bfloat16), group_size=32, symmetric=True,
                     quantization_scale="absmax", quantization_order="activation")
    h._prep()
    np.testing.assert_array_equal(h.H.numpy(), c["H_prep"])
    np.testing.assert_array_equal(h.perm.numpy(), c["perm"])


def test_reversed_cholesky_identity(golden):
    """The factorisation the CUDA path uses (one Cholesky of the index-reversed matrix + one triangular
    inverse) gives the reference's three-step factor, here in float64 on a golden Hessian."""
    c = golden_case(golden, "actorder_multibatch")
    H = torch.from_numpy(c["H_prep"]).double()
    C = H.shape[0]
    H[range(C), range(C)] += 0.01 * H.diag().mean()
    L = torch.linalg.cholesky(H)
    T = torch.linalg.cholesky(torch.cholesky_inverse(L), upper=True)
    U_ref = T / T.diag()[:, None]
    Lr = torch.linalg.cholesky(torch.flip(H, (0, 1)))
    Minv = torch.linalg.solve_triangular(Lr, torch.eye(C, dtype=torch.float64), upper=False)
    U_alt = torch.flip(Lr.diag()[:, None] * Minv, (0, 1))
    assert float((U_ref - U_alt).abs().max()) < 1e-9
    udiag = torch.flip(1.0 / Lr.diag(), (0,))
    assert float((udiag - T.diag()).abs().max() / T.diag().abs().max()) < 1e-9
