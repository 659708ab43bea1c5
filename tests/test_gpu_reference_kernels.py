"""The engine against the reference's OWN CUDA kernels, both running on the GPU on the same inputs.

oracle/_ref/forge_ref_kernels.so is built from the reference checkout's .cu files by oracle/ref_build.py (test
infrastructure; it is not part of the product and nothing under the package loads it).  The five functions are the
solver-path operators of the reference's pybind module (forge/backend/cuda/kernels.cpp:92-150); the engine side
goes through the same-named wrappers of forge.backend.cuda.kernels, i.e. through the C ABI.
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import ref_build  # noqa: E402


@pytest.fixture(scope="module")
def ref():
    mod = ref_build.load_built()
    if mod is None:
        pytest.skip("oracle/_ref/forge_ref_kernels.so not built (needs the reference checkout at build time)")
    return mod


def _weights(rows, C, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    W = torch.randn(rows, C, generator=g) * 0.02
    if outliers:
        W = torch.where(torch.rand(rows, C, generator=g) < 0.002, W * 15.0, W)
    return W.to(DEV)


@pytest.mark.parametrize("gs", [32, 64, 128])
@pytest.mark.parametrize("sym", [False, True])
def test_minmax_and_mse_grid_bit_exact(ref, gs, sym):
    from forge.backend.cuda import kernels
    X = _weights(4096, gs, 100 + gs).contiguous()
    s_ref, z_ref = ref.build_group_meta_packed(X, 4, sym)
    s, z = kernels.build_group_meta_packed(X, 4, sym)
    assert torch.equal(s, s_ref) and torch.equal(z, z_ref)
    cand = torch.linspace(1.0, 0.2, 100, device=DEV)
    s2_ref, z2_ref = ref.mse_scale_groups_packed(X, s_ref.clone(), z_ref.clone(), cand, 2.4, 4, sym)
    s2, z2 = kernels.mse_scale_groups_packed(X, s.clone(), z.clone(), cand, 2.4, 4, sym)
    assert torch.equal(s2, s2_ref) and torch.equal(z2, z2_ref)      # same approximate lg2 / ex2, same summation order


def _factor(C, seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(C, 4 * C, generator=g, dtype=torch.float64)
    H = A @ A.T / (4 * C) + 0.05 * torch.eye(C, dtype=torch.float64)
    U = torch.linalg.cholesky(torch.linalg.inv(H), upper=True).float()
    return U


def _element_meta(ref, W, gs, sym):
    R, C = W.shape
    s, z = ref.build_group_meta_packed(W.reshape(-1, gs).contiguous(), 4, sym)
    G = C // gs
    exp = lambda t: t.view(R, G).repeat_interleave(gs, 1).T.contiguous()
    return exp(s), exp(z), s, z


@pytest.mark.parametrize("R,C", [(256, 512), (96, 160)])
@pytest.mark.parametrize("impl", ["tensor", "simt"])
def test_gptq_solver_against_reference_kernel(ref, R, C, impl, monkeypatch):
    from forge.backend.cuda import kernels
    if impl == "simt":
        monkeypatch.setenv("FORGE_SOLVER_IMPL", "simt")
    W = _weights(R, C, 7 + C, outliers=False)
    U = _factor(C, 3 + C)
    U = (U / U.diag()[:, None]).contiguous().to(DEV)
    s_el, z_el, _, _ = _element_meta(ref, W, 32, False)
    Wt = W.T.contiguous()
    W_ref, W_eng = Wt.clone(), Wt.clone()
    q_ref = ref.gptq_solver(W_ref, U, s_el, z_el, 4)
    q = kernels.gptq_solver(W_eng, U, s_el, z_el, 4)
    agree = float((q == q_ref).float().mean())
    # all-FMA build: same arithmetic up to the summation order of the lazy update; tensor-core build: TF32 x3 products
    assert agree >= (0.9995 if impl == "simt" else 0.995), agree
    # both overwrite W with the de-quantised weights
    same = q == q_ref
    assert torch.equal(W_eng[same], W_ref[same])


def test_sparse_solver_and_packer_against_reference_kernels(ref):
    from forge.backend.cuda import kernels
    R, C = 192, 256
    W = _weights(R, C, 77, outliers=False)
    U = _factor(C, 78).contiguous().to(DEV)                      # un-normalised: the operator divides by the diagonal
    s_el, z_el, s, _ = _element_meta(ref, W, 32, True)
    Wt = W.T.contiguous()
    q_ref, M_ref = ref.sparsegptq14_solver(Wt.clone(), U.clone(), s_el, z_el, 4)
    q, M = kernels.sparsegptq14_solver(Wt.clone(), U.clone(), s_el, z_el, 4)
    Mi, Mr = M.view(torch.int32), M_ref.view(torch.int32)
    nib = lambda m: torch.stack([(m >> (4 * i)) & 0xF for i in range(8)], -1)
    # >= 99.5 % of the 1-of-4 choices and of the codes agree; whole 32-column mask words on >= 99 %
    assert float((nib(Mi) == nib(Mr)).float().mean()) >= 0.995
    assert float((Mi == Mr).float().mean()) >= 0.99
    assert float((q == q_ref).float().mean()) >= 0.995
    # the packer is integer work: bit-exact on identical inputs
    s32 = s.view(R, C // 32).T.contiguous()
    qrc = q_ref.T.contiguous()
    wp_ref = ref.pack_sparsegptq14_to_u64x2(qrc, M_ref, s32)
    wp = kernels.pack_sparsegptq14_to_u64x2(qrc, M_ref, s32)
    assert torch.equal(wp.view(torch.int64), wp_ref.view(torch.int64))


def _random_wpair(ref, R, C, seed):
    g = torch.Generator().manual_seed(seed)
    G32 = (C + 31) // 32
    q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
    pos = torch.randint(0, 4, (G32, R, 8), generator=g)
    keep = torch.rand(G32, R, 8, generator=g) > 0.1
    M = ((keep.long() << (4 * torch.arange(8) + pos)).sum(-1) & 0xFFFFFFFF).to(torch.int32)
    s32 = (torch.rand(G32, R, generator=g) * 0.01 + 1e-3).float()
    return ref.pack_sparsegptq14_to_u64x2(q.to(DEV), M.to(DEV).view(torch.uint32), s32.to(DEV))


@pytest.mark.parametrize("R,C,N", [(130, 256, 1), (96, 160, 3), (96, 160, 70), (1536, 3072, 1), (1536, 3072, 8),
                                   (3072, 1536, 37), (40, 1088, 800)])
def test_inference_gemm_over_wpair_bit_exact(ref, R, C, N):
    """forge_sparse14_gemm against the reference's inference kernel (forge/backend/cuda/sparse14_gemm.cu) on the same
    packed words: identical bf16 outputs, for every token tile of either launcher, ragged R and C included."""
    from forge.backend.cuda import kernels
    import ref_port as O
    wp = _random_wpair(ref, R, C, R + C + N)
    g = torch.Generator().manual_seed(N)
    X = (torch.randn(N, C, generator=g) * 0.7).to(torch.bfloat16).to(DEV)
    Y_ref = ref.sparsegptq14_gemm(wp, X)
    Y = kernels.sparsegptq14_gemm(wp, X)
    assert Y.shape == (N, R) and torch.equal(Y.view(torch.int16), Y_ref.contiguous().view(torch.int16))
    if R * C <= 64 * 1024:
        Yo = O.sparsegptq14_gemm(wp.cpu().view(torch.int64), X.cpu())
        assert torch.equal(Yo.view(torch.int16), Y.cpu().view(torch.int16))


def test_packed_sparse_layer_is_consumed_end_to_end():
    """SparseGPT 1:4 + int4 through forge.moe, then the packed Wpair words through the inference GEMM: the product
    equals X times the de-quantised, masked weights (the bf16 scale of the packed layout is the only difference)."""
    from forge import synth, moe, ops
    shape = synth.LayerShape("s", 4, 0, 256, 128, 2048, 2)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=91).to(DEV)
    ids = synth.route(shape, shape.tokens, seed=91).to(DEV)
    Wg, Wu, Wd = [w.to(DEV) for w in synth.expert_weights(shape, range(4), seed=91)]
    cfg = moe.MoEQuantConfig(bits=4, group_size=32, symmetric=True, algorithm="sparsegptq", rel_damp=0.01)
    out = moe.MoELayerQuantizer(cfg).quantize_experts(X, ids, Wg, Wu, Wd)
    e = 1
    xin = X[:64].contiguous()
    Y = ops.sparse14_gemm(out["gate"]["wpair"][e], xin).float()
    r = out["gate"]
    What = ops.dequantize(r["qweight"][e], r["scales"][e].contiguous(), r["qzeros"][e].contiguous(), 32, torch.float32)
    Mi = r["M"][e].view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    keep = ((Mi.unsqueeze(-1) >> torch.arange(32, device=DEV)) & 1).permute(1, 0, 2).reshape(What.shape[0], -1).float()
    ref_y = xin.float() @ (What * keep[:, :What.shape[1]]).T
    assert float((Y - ref_y).norm() / ref_y.norm()) < 1e-2


def _random_moe_wpair(E, R, C, seed):
    """Stacked Wpair words [E, G2, R, 2] from the engine's own packer (bit-exact with the reference's, see above)."""
    from forge.backend.cuda import kernels
    out = []
    for e in range(E):
        g = torch.Generator().manual_seed(seed + e)
        G32 = (C + 31) // 32
        q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
        pos = torch.randint(0, 4, (G32, R, 8), generator=g)
        keep = torch.rand(G32, R, 8, generator=g) > 0.1
        M = ((keep.long() << (4 * torch.arange(8) + pos)).sum(-1) & 0xFFFFFFFF).to(torch.int32)
        s32 = (torch.rand(G32, R, generator=g) * 0.01 + 1e-3).float()
        out.append(kernels.pack_sparsegptq14_to_u64x2(q.to(DEV), M.to(DEV).view(torch.uint32), s32.to(DEV)).view(torch.int64))
    return torch.stack(out).contiguous()


def _bf16_ulps(a, b):
    """Distance in bf16 steps between two bf16 tensors (sign-magnitude bit patterns mapped to a line)."""
    def line(t):
        v = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(v < 0, -(v & 0x7FFF), v)
    return (line(a) - line(b)).abs()


@pytest.mark.parametrize("E,H,I,counts", [(4, 256, 128, [5, 0, 17, 8]), (6, 160, 96, [1, 2, 3, 40, 0, 9]),
                                          (3, 1536, 256, [300, 7, 64])])
def test_grouped_moe_gemms_over_wpair(E, H, I, counts):
    """The grouped W13+SwiGLU and W2 kernels (interfaces of fused_moe_usp14w4a16_gemm.cu:1028-1140) on rows sorted by
    expert: W2 bit-identical to the per-expert inference GEMM (itself bit-identical to the reference's kernel), W13
    within one bf16 step of silu(g)*u from fp64 sums of the decoded weights; inactive experts' rows stay zero; the
    gather by token index gives the same bytes as a permuted copy."""
    from forge.backend.cuda import kernels
    from forge import ops
    import ref_port as O
    w13 = _random_moe_wpair(E, 2 * I, H, 100 * E + H)
    w2 = _random_moe_wpair(E, H, I, 200 * E + I)
    N = sum(counts)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int64, device=DEV)
    g = torch.Generator().manual_seed(N)
    X = (torch.randn(N, H, generator=g) * 0.7).to(torch.bfloat16).to(DEV)
    active = torch.tensor([e for e in range(E) if e != 1], dtype=torch.int32, device=DEV)
    X2 = kernels.sparsegptq14_grouped_gemm_w13(w13, X, offsets, active)
    assert X2.shape == (N, I)
    X2o = O.sparse14_grouped_w13(w13.cpu(), X.cpu(), offsets.cpu(), active.cpu())
    d = _bf16_ulps(X2.cpu(), X2o)
    assert float((d == 0).float().mean()) >= 0.99
    # the rest: one bf16 step apart, or a near-cancelled sum whose fp32 error is small against the output's scale
    err = (X2.cpu().float() - X2o.float()).abs()
    assert bool(((d <= 1) | (err <= 1e-4 * X2o.float().abs().mean())).all())
    s1, t1 = int(offsets[1]), int(offsets[2])
    assert not X2[s1:t1].any()
    Y = kernels.sparsegptq14_grouped_gemm_w2(w2, X2, offsets, active)
    assert Y.shape == (N, H)
    for e in range(E):
        s, t = int(offsets[e]), int(offsets[e + 1])
        if t == s:
            continue
        if e == 1:
            assert not Y[s:t].any()
            continue
        Ye = kernels.sparsegptq14_gemm(w2[e], X2[s:t].contiguous())
        assert torch.equal(Ye.view(torch.int16), Y[s:t].view(torch.int16))
    # gather fused into the load: X in token order + a position -> token list
    perm = torch.randperm(N, generator=g).to(DEV)
    Xtok = torch.empty_like(X)
    Xtok[perm] = X
    X2g = ops.sparse14_moe_w13_swiglu(w13, Xtok, offsets, active, token_idx=perm.to(torch.int32), n_out=N)
    assert torch.equal(X2g.view(torch.int16), X2.view(torch.int16))


def test_sparse14_moe_runtime_matches_reference_runtime():
    """forge.inference.Sparse14MoERuntime against the restated Sparse14MoERuntime.forward of the reference
    (sparse14_gemm.py:32-65: per-expert GEMM, bf16 SwiGLU in torch, per-expert GEMM, weighted un-permute).  The grouped
    W13 kernel rounds once where the reference rounds gate and up first, hence a tolerance."""
    from forge import inference
    import ref_port as O
    E, H, I, T, K = 8, 256, 128, 96, 2
    w13 = _random_moe_wpair(E, 2 * I, H, 7)
    w2 = _random_moe_wpair(E, H, I, 9)
    g = torch.Generator().manual_seed(3)
    X = (torch.randn(T, H, generator=g) * 0.7).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    wts, ids = torch.topk(torch.softmax(logits, -1), K, dim=-1)
    rt = inference.Sparse14MoERuntime(w13, w2, I, E)
    out = rt.forward(X.to(DEV), ids.to(torch.int32).to(DEV), wts.to(DEV))
    ref_out = O.sparse14_moe_runtime_forward(w13.cpu(), w2.cpu(), X, ids, wts)
    assert out.shape == (T, H)
    rel = float((out.cpu().float() - ref_out.float()).norm() / ref_out.float().norm())
    assert rel < 1e-2, rel
