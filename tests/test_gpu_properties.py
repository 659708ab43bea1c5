"""Size-independent properties at the full shapes of the benchmark configurations, and failure handling.

The oracle is too slow for a 7168-wide matrix, so at full size the kernels are checked through properties the
domain offers: pack -> unpack round trips, symmetry / trace identities of the Hessian, linearity of the running
mean, the factor identity U^-1 U^-T = H, and idempotence of the solver on already-quantised weights.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    from forge import ops
    return ops


def test_bounded_wait_reports_timeout_without_hanging():
    """A wait that nothing satisfies runs out after its budget and the kernel returns a status; the context stays
    usable (the next launch works)."""
    from forge import _abi
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    _abi.call("forge_selftest_bounded_wait", _abi.ptr(st), 2_000_000, _abi.stream_ptr())   # ~1 ms
    torch.cuda.synchronize()
    assert int(st.item()) == _abi.ERR_TIMEOUT
    x = torch.ones(8, device=DEV)
    assert float(x.sum()) == 8.0


@pytest.mark.parametrize("R,C", [(2048, 7168), (7168, 2048), (768, 2048)])
def test_pack_int4_roundtrip_full_size(R, C):
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(1)
    q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8, device=DEV)
    z = torch.full((R * (C // 128),), 8.0, device=DEV)
    packed = ops.pack_int4(q, z, 128)
    assert packed.shape == (R, C // 8) and packed.dtype == torch.int32
    shifts = torch.arange(8, device=DEV, dtype=torch.int32) * 4
    un = ((packed.unsqueeze(-1) >> shifts) & 0xF).reshape(R, C).to(torch.uint8)
    assert torch.equal(un, q)


@pytest.mark.parametrize("R,C", [(1536, 3072), (3072, 1536)])
def test_pack_sparse14_roundtrip_full_size(R, C):
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(2)
    q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8, device=DEV)
    G32 = C // 32
    keep = torch.randint(0, 4, (G32, 8, R), generator=g, device=DEV)
    M64 = (torch.ones_like(keep) << (keep + (torch.arange(8, device=DEV) * 4).view(1, 8, 1))).sum(1)
    M = (M64 & 0xFFFFFFFF).to(torch.int64)
    M32 = torch.where(M >= 2 ** 31, M - 2 ** 32, M).to(torch.int32)
    sc = torch.rand(G32, R, generator=g, device=DEV) * 0.01 + 1e-4
    out = ops.pack_sparse14(q, M32, sc)                     # [G2, R, 2] int64 bit patterns
    words = out.permute(0, 2, 1).reshape(-1, R)[:G32]       # word of group gid at [gid, r]
    codes = torch.stack([(words >> (4 * i)) & 0xF for i in range(8)], 1)          # [G32, 8, R]
    idx = torch.stack([(words >> (32 + 2 * i)) & 0x3 for i in range(8)], 1)
    assert torch.equal(idx, keep)
    cols = (torch.arange(G32, device=DEV).view(-1, 1, 1) * 32 + torch.arange(8, device=DEV).view(1, 8, 1) * 4 + keep)
    want = q.T[cols, torch.arange(R, device=DEV).view(1, 1, R)]
    assert torch.equal(codes.to(torch.uint8), want)
    sbits = ((words >> 48) & 0xFFFF).to(torch.int32)
    assert torch.equal(sbits, (sc.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF))


def test_hessian_identities_full_width():
    """C = 7168 (DeepSeek / Kimi hidden size): symmetry, trace = 2/n * ||X||_F^2, and the running mean over two
    batches equals the one-shot Hessian of their concatenation."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(3)
    C, n1, n2 = 7168, 1500, 700
    X = (torch.randn(n1 + n2, C, generator=g, device=DEV) * 0.5).to(torch.bfloat16)
    H = torch.empty((1, C, C), device=DEV)
    st = ops.hessian_grouped(X, C, None, torch.tensor([0, n1 + n2], device=DEV), H, mirror=True)
    assert int(st.item()) == 0
    assert torch.equal(H[0], H[0].T)
    tr = 2.0 / (n1 + n2) * float((X.double() ** 2).sum())
    assert abs(float(H[0].diagonal().double().sum()) - tr) <= 1e-5 * tr
    H2 = torch.empty((1, C, C), device=DEV)
    n_prev = torch.zeros(1, dtype=torch.int64, device=DEV)
    o1 = torch.tensor([0, n1], device=DEV)
    ops.hessian_grouped(X[:n1], C, None, o1, H2, n_prev=n_prev, mirror=True, status=st)
    ops.counts_add(n_prev, o1)
    ops.hessian_grouped(X[n1:].contiguous(), C, None, torch.tensor([0, n2], device=DEV), H2, n_prev=n_prev,
                        mirror=True, status=st)
    assert int(st.item()) == 0
    assert float((H2 - H).norm() / H.norm()) < 1e-5
    # a random 64x64 block against fp32 torch
    ref = 2.0 / (n1 + n2) * (X[:, 3000:3064].float().T @ X[:, 5000:5064].float())
    assert float((H[0, 3000:3064, 5000:5064] - ref).norm() / ref.norm()) < 1e-4


@pytest.mark.parametrize("C", [2048, 3072, 4352])
def test_factor_identities_full_size(C):
    """U is unit upper triangular and U^-1 U^-T reproduces the damped Hessian up to the diagonal scaling;
    the inversion-free factor is the inverse of it."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(4)
    X = torch.randn(4 * C, C, generator=g, device=DEV) * torch.exp(0.5 * torch.randn(C, generator=g, device=DEV))
    H = (2.0 / (4 * C)) * (X.T @ X)
    H.diagonal().add_(0.01 * H.diagonal().mean())
    A = torch.flip(H, (0, 1)).contiguous().view(1, C, C)
    U, udiag, info = ops.chol_inv_upper(A.clone(), zero_lower=True)
    assert int(info[0]) == 0
    assert float(torch.tril(U[0], -1).abs().max()) == 0.0
    assert torch.equal(U[0].diagonal(), torch.ones(C, device=DEV))
    T = (U[0] * udiag[0][:, None]).double()                   # un-normalised factor, T^T T = H^-1
    resid = T.T @ T @ H.double() - torch.eye(C, device=DEV, dtype=torch.float64)
    assert float(resid.abs().max()) < 5e-3
    V, ud1, info1 = ops.chol_factor(A.clone())
    assert int(info1[0]) == 0
    Vt = torch.eye(C, device=DEV, dtype=torch.float64) - torch.triu(V[0].double(), 1)
    assert float((Vt @ U[0].double() - torch.eye(C, device=DEV, dtype=torch.float64)).abs().max()) < 5e-3


def test_solver_is_idempotent_on_quantised_weights():
    """Weights that already lie on the grid are reproduced exactly (zero error, nothing to propagate), at the
    gate shape of the benchmark layer."""
    ops = _ops()
    g = torch.Generator(device=DEV).manual_seed(5)
    nb, R, C, gs = 2, 768, 2048, 128
    W = (torch.randn(nb, R, C, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    s, z = ops.quant_grid(W.view(nb * R, C), gs, 4, True)
    U = torch.triu(torch.randn(nb, C, C, generator=g, device=DEV) * 0.01, 1) + torch.eye(C, device=DEV)
    q1 = ops.gptq_solve_batched(W, U, s, z, gs, 4)
    Wq = ops.dequantize(q1, s, z, gs, torch.float32)           # on-grid weights, fp32 (exactly (q - 8) * s)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    q2 = ops.gptq_solve_batched(Wq, U, s, z, gs, 4, status=st)
    assert int(st.item()) == 0
    assert float((q2 == q1).float().mean()) >= 0.9999


def test_hessian_error_does_not_grow_with_the_token_count():
    """The tensor core adds to its fp32 accumulator with truncation, so one long accumulation drifts (3e-4 relative
    after 65536 tokens).  The kernel accumulates at most 4096 tokens per pass and adds the passes in fp32: the error
    against float64 stays at the level of an fp32 sum for a shared expert's token count as for a cold expert's, well
    inside the 1e-4 the Hessian is allowed."""
    from forge import synth
    ops = _ops()
    C = 1024
    errs = {}
    for T in (2048, 65536):
        X = synth.student_t_activations(T, C, seed=5, device=DEV)
        H = torch.zeros((1, C, C), dtype=torch.float32, device=DEV)
        offs = torch.tensor([0, T], dtype=torch.int64, device=DEV)
        ops.hessian_grouped(X, C, None, offs, H)
        Xd = X.double()
        H64 = (2.0 / T) * (Xd.T @ Xd)
        errs[T] = float((H[0].double() - H64).norm() / H64.norm())
        assert torch.equal(H[0], H[0].T)                       # the mirror image follows the same additions
    assert errs[2048] <= 2e-5 and errs[65536] <= 3e-5, errs


def test_running_mean_over_batches_that_need_several_accumulation_passes():
    """Two updates of 6000 and 9000 tokens (two and three accumulation passes each) in the running-mean form equal the
    Hessian of the 15000 tokens at once, and both match float64; token lists with a gather, two slots of unequal
    length."""
    from forge import synth
    ops = _ops()
    C, T = 512, 15000
    X = synth.student_t_activations(T, C, seed=9, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(9)
    perm = torch.randperm(T, generator=g, device=DEV).to(torch.int32)
    # slot 0 sees tokens perm[:6000] then perm[6000:15000]; slot 1 sees the first 100 tokens once
    H = torch.zeros((2, C, C), dtype=torch.float32, device=DEV)
    lists1 = torch.cat([perm[:6000], torch.arange(100, device=DEV, dtype=torch.int32)]).contiguous()
    offs1 = torch.tensor([0, 6000, 6100], dtype=torch.int64, device=DEV)
    ops.hessian_grouped(X, C, lists1, offs1, H)
    n_prev = torch.tensor([6000, 100], dtype=torch.int64, device=DEV)
    lists2 = perm[6000:].contiguous()
    offs2 = torch.tensor([0, 9000, 9000], dtype=torch.int64, device=DEV)
    ops.hessian_grouped(X, C, lists2, offs2, H, n_prev=n_prev)
    Xd = X.double()
    H0 = (2.0 / T) * (Xd.T @ Xd)
    H1 = (2.0 / 100) * (Xd[:100].T @ Xd[:100])
    assert float((H[0].double() - H0).norm() / H0.norm()) < 3e-5
    assert float((H[1].double() - H1).norm() / H1.norm()) < 3e-5
    assert torch.equal(H[0], H[0].T) and torch.equal(H[1], H[1].T)
    one = torch.zeros((1, C, C), dtype=torch.float32, device=DEV)
    ops.hessian_grouped(X, C, perm.contiguous(), torch.tensor([0, T], dtype=torch.int64, device=DEV), one)
    assert float((H[0] - one[0]).norm() / one[0].norm()) < 2e-5



def test_mma_issue_rate_diagnostic():
    """forge_selftest_mma_rate: the back-to-back cost of the solver's MMA shape, a plausible number of cycles, and the
    wider shape costs more."""
    ops = _ops()
    c128 = ops.mma_issue_cycles(128, 1000)
    c256 = ops.mma_issue_cycles(256, 1000)
    assert 40.0 < c128 < 400.0 and c128 < c256 < 2.5 * c128, (c128, c256)
