"""The CPU oracle against the reference's own CUDA kernels.

tests/golden/ref_kernels_b200.npz holds inputs and outputs of the reference's kernels (quant_grid.cu, solver.cu,
solver_sparsegptq14.cu, bitpacking_sparsegptq14.cu) compiled from the reference checkout for sm_100a and run on a
B200 by tests/golden/make_golden_gpu.py.  These tests replay the oracle on the stored inputs: this is what pins
oracle/forge_oracle.c.
"""
import os

import numpy as np
import pytest
import torch

import ref_port as O

PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_kernels_b200.npz")


@pytest.fixture(scope="module")
def ref():
    z = np.load(PATH)
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize("tag", ["g128", "g32"])
@pytest.mark.parametrize("sym", [False, True])
def test_minmax_grid_bit_exact(ref, tag, sym):
    s, z = O.build_group_meta_packed(ref[f"grid_{tag}_X"], 4, sym)
    assert torch.equal(s, ref[f"grid_{tag}_sym{int(sym)}_scales"])
    assert torch.equal(z, ref[f"grid_{tag}_sym{int(sym)}_qzeros"])


@pytest.mark.parametrize("tag", ["g128", "g32"])
@pytest.mark.parametrize("sym", [False, True])
def test_mse_search_picks_the_same_candidates(ref, tag, sym):
    """The kernel evaluates |e|^2.4 with the hardware's approximate lg2 / ex2, the oracle with logf / expf; on these
    vectors no group is close enough to a tie for that to matter: the chosen scales and zeros are identical."""
    X = ref[f"grid_{tag}_X"]
    s0, z0 = ref[f"grid_{tag}_sym{int(sym)}_scales"], ref[f"grid_{tag}_sym{int(sym)}_qzeros"]
    cand = torch.linspace(1.0, 0.2, 100)
    s, z = O.mse_scale_groups_packed(X, s0.clone(), z0.clone(), cand, 2.4, 4, sym)
    assert torch.equal(s, ref[f"mse_{tag}_sym{int(sym)}_scales"])
    assert torch.equal(z, ref[f"mse_{tag}_sym{int(sym)}_qzeros"])
    assert float((s < s0).float().mean()) > 0.3          # the search did shrink scales


def test_gptq_solver_codes(ref):
    q = O.gptq_solver(ref["gptq_Wt"].clone().contiguous(), ref["gptq_U"].contiguous(), ref["gptq_s"], ref["gptq_z"], 4)
    assert torch.equal(q, ref["gptq_q"])


def test_sparse_solver_codes_and_mask(ref):
    q, M = O.sparsegptq14_solver(ref["sparse_Wt"].clone().contiguous(), ref["sparse_U"].clone().contiguous(), ref["sparse_s"], ref["sparse_z"], 4)
    Mi = M.view(torch.int32) if M.dtype != torch.int32 else M
    assert torch.equal(Mi, ref["sparse_M"])
    assert torch.equal(q, ref["sparse_q"])


def test_sparse_packer_bit_exact(ref):
    M = ref["sparse_M"]
    wp = O.pack_sparsegptq14_to_u64x2(ref["pack_q_rc"], M, ref["pack_scales"])
    assert torch.equal(wp.view(torch.int64), ref["pack_wpair"])


GEMM_PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_sparse14_gemm_b200.npz")


@pytest.mark.skipif(not os.path.exists(GEMM_PATH), reason="inference-GEMM vectors not generated yet")
@pytest.mark.parametrize("tag,N", [("c256", 1), ("c256", 5), ("c160", 3), ("c160", 70), ("c160", 300), ("c320", 800)])
def test_sparse14_gemm_bit_exact(tag, N):
    """O.sparsegptq14_gemm against the reference's inference kernel over the Wpair layout (sparse14_gemm.cu), run on a
    B200 by make_golden_gpu.py: identical bf16 outputs."""
    z = np.load(GEMM_PATH)
    wp = torch.from_numpy(z[f"{tag}_wpair"])
    X = torch.from_numpy(z[f"{tag}_X{N}"]).view(torch.bfloat16)
    Y = O.sparsegptq14_gemm(wp, X)
    assert torch.equal(Y.view(torch.int16), torch.from_numpy(z[f"{tag}_Y{N}"]))


def test_sparse14_gemm_equals_dense_product_of_the_decoded_weights():
    """Independent of any stored vector: decode the Wpair words to a dense matrix and multiply in float64."""
    g = torch.Generator().manual_seed(9)
    R, C, N = 50, 192, 7
    q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
    pos = torch.randint(0, 4, (C // 32, R, 8), generator=g)
    M = ((1 << (4 * torch.arange(8) + pos)).sum(-1)).to(torch.int32)
    s32 = (torch.rand(C // 32, R, generator=g) * 0.01 + 1e-3).float()
    wp = O.pack_sparsegptq14_to_u64x2(q, M, s32)
    X = torch.randn(N, C, generator=g).to(torch.bfloat16)
    Y = O.sparsegptq14_gemm(wp, X).double()
    keep = torch.zeros(R, C, dtype=torch.bool)
    for gI in range(C // 32):
        for i in range(8):
            keep[torch.arange(R), gI * 32 + 4 * i + pos[gI, :, i]] = True
    s_bf = s32.to(torch.bfloat16).double().T.repeat_interleave(32, 1)            # the packed scale is bf16
    What = (q.double() - 8.0) * s_bf * keep
    ref = X.double() @ What.T
    assert float((Y - ref).abs().max()) <= 0.01 * float(ref.abs().max()) + 1e-6


def test_wpair_decode_and_grouped_restatements_agree_with_the_pinned_gemm():
    """O.wpair_to_dense, O.sparse14_grouped_w13 and O.sparse14_moe_runtime_forward (the checkers of the grouped MoE
    kernels) against O.sparsegptq14_gemm, which the reference's own kernel pins above."""
    g = torch.Generator().manual_seed(11)
    E, H, I, T, K = 3, 128, 64, 10, 2

    def stack(R, C, seed):
        out = []
        for e in range(E):
            ge = torch.Generator().manual_seed(seed + e)
            q = torch.randint(0, 16, (R, C), generator=ge, dtype=torch.uint8)
            pos = torch.randint(0, 4, (C // 32, R, 8), generator=ge)
            M = ((1 << (4 * torch.arange(8) + pos)).sum(-1)).to(torch.int32)
            s32 = (torch.rand(C // 32, R, generator=ge) * 0.01 + 1e-3).float()
            out.append(O.pack_sparsegptq14_to_u64x2(q, M, s32).view(torch.int64))
        return torch.stack(out)

    w13, w2 = stack(2 * I, H, 1), stack(H, I, 5)
    X = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dense = O.wpair_to_dense(w13[1], H)
    y = O.sparsegptq14_gemm(w13[1], X).double()
    ref = X.double() @ dense.double().T
    assert float((y - ref).abs().max()) <= 0.01 * float(ref.abs().max()) + 1e-6
    # grouped W13: two experts' row ranges, the third inactive
    offsets = torch.tensor([0, 4, 4, 10])
    X2 = O.sparse14_grouped_w13(w13, X, offsets, torch.tensor([0, 2]))
    gu = O.sparsegptq14_gemm(w13[2], X[4:10]).float()
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert float((X2[4:10].float() - want).norm() / want.norm()) < 2e-2
    assert not X2[4:4].any()
    # runtime: top-1 routing with unit weights reduces to one expert's two GEMMs per token
    ids = torch.randint(0, E, (T, 1), generator=g)
    out = O.sparse14_moe_runtime_forward(w13, w2, X, ids, torch.ones(T, 1))
    for t in range(T):
        e = int(ids[t, 0])
        y13 = O.sparsegptq14_gemm(w13[e], X[t:t + 1])
        a2 = torch.nn.functional.silu(y13[:, :I]) * y13[:, I:]
        assert torch.equal(O.sparsegptq14_gemm(w2[e], a2.contiguous()).view(torch.int16), out[t:t + 1].view(torch.int16))
