"""The materialisation rules of the oracle against the reference's own Python functions
(tests/golden/io_materialise.npz, made by tests/golden/make_golden_io.py from forge/utils/io.py of the reference)."""
import os

import numpy as np
import pytest
import torch

import ref_port as O

PATH = os.path.join(os.path.dirname(__file__), "golden", "io_materialise.npz")


@pytest.fixture(scope="module")
def gold():
    z = np.load(PATH)
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("inv", [False, True])
def test_int4_packed_dequant_bit_exact(gold, sym, inv):
    w = O.int4_packed_dequant(gold["int4_packed"], gold["int4_scales"], gold[f"int4_out_sym{int(sym)}_inv{int(inv)}"].shape,
                              symmetric=sym, scale_is_inv=inv)
    assert torch.equal(w, gold[f"int4_out_sym{int(sym)}_inv{int(inv)}"])


def test_mxfp4_dequant_bit_exact(gold):
    w = O.mxfp4_dequant(gold["mx_blocks"], gold["mx_scales"])
    assert w.shape == gold["mx_out"].shape
    assert torch.equal(w, gold["mx_out"])
