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


@pytest.mark.parametrize("tag", ["sq", "ragged", "tall"])
def test_fp8_block_dequant_bit_exact(gold, tag):
    """O.fp8_block_dequant against _apply_block_scale_inv_2d + the bf16 cast of the reference (forge/utils/io.py:533-563,
    :864-874), run on the CPU by make_golden_io.py."""
    w8 = gold[f"fp8_{tag}_w"].view(torch.float8_e4m3fn)
    got = O.fp8_block_dequant(w8, gold[f"fp8_{tag}_sinv"])
    assert torch.equal(got.view(torch.int16), gold[f"fp8_{tag}_out_bits"])
