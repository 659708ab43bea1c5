"""The C restatement of the CUDA-only kernels against independent restatements (plain torch / Python loops)
and against the installed compressed_tensors packer."""
import math

import numpy as np
import pytest
import torch

import ref_port as O


def _groups(seed, RG, gs, scale=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(RG, gs, generator=g) * scale).to(torch.bfloat16).float()


@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("gs", [32, 64, 128, 48])
def test_absmax_grid_formula(sym, gs):
    X = _groups(1, 37, gs)
    s, z = O.build_group_meta_packed(X, 4, sym)
    mn, mx = X.min(1).values, X.max(1).values
    if sym:
        s_ref = torch.tensor([np.float32(math.fma(np.float32(2.0 / 15.0), float(a), 1e-12)) if hasattr(math, "fma") else 0
                              for a in torch.maximum(mn.abs(), mx.abs())]) if hasattr(math, "fma") else None
        s2 = (2.0 / 15.0) * torch.maximum(mn.abs(), mx.abs()) + 1e-12
        assert torch.allclose(s, s2, rtol=1e-6, atol=0)
        assert torch.all(z == 8.0)
    else:
        s2 = (mx - mn) / 15.0 + 1e-12
        assert torch.equal(s, s2)
        assert torch.equal(z, torch.clamp(torch.round(-mn / s2), 0, 15))


def test_mse_grid_against_python_loop():
    X = _groups(2, 6, 32)
    cand = torch.linspace(1.0, 0.2, 100, dtype=torch.float32)
    for sym in (True, False):
        s0, z0 = O.build_group_meta_packed(X, 4, sym)
        s, z = O.mse_scale_groups_packed(X, s0.clone(), z0.clone(), cand, 2.4, 4, sym)
        for g in range(X.shape[0]):
            best = (np.float32(3.4e38), s0[g].item(), z0[g].item())
            xmin = np.float32(0.0) if sym else -(np.float32(s0[g]) * np.float32(z0[g]))
            for p in cand.numpy():
                sc = np.float32(s0[g]) * np.float32(p)
                rcp = np.float32(1.0) / (sc + np.float32(1e-12))
                q0 = np.float32(z0[g]) if sym else np.clip(np.rint(-xmin * rcp), 0, 15).astype(np.float32)
                v = X[g].numpy()
                q = np.clip(np.rint(v.astype(np.float64) * rcp + q0), 0, 15).astype(np.float32)
                diff = np.maximum(np.abs((q - q0).astype(np.float64) * sc - v), 1e-20)
                loss = float(np.sum(np.exp(np.log(diff) * 2.4)))
                if loss < best[0] * (1 - 1e-6):
                    best = (loss, float(sc), float(q0))
            # the independent loop works in float64, so only demand that the chosen scale is (near) optimal
            assert abs(s[g].item() - best[1]) <= 0.0101 * s0[g].item() + 1e-12
            assert 0.2 * s0[g].item() - 1e-7 <= s[g].item() <= s0[g].item() + 1e-7


def test_mse_rejects_other_group_sizes():
    X = _groups(3, 4, 48)
    s, z = O.build_group_meta_packed(X, 4, True)
    with pytest.raises(RuntimeError):
        O.mse_scale_groups_packed(X, s, z, torch.linspace(1, 0.2, 10), 2.4, 4, True)


def _naive_gptq(W, U, S, Z, maxq=15):
    """Column-at-a-time GPTQ in float64 with immediate propagation: the mathematical definition."""
    W = W.double().clone()
    C, R = W.shape
    Q = torch.zeros((C, R), dtype=torch.uint8)
    for t in range(C):
        s, z = S[t].double(), Z[t].double()
        q = torch.clamp(torch.round(W[t] / (s + 1e-12) + z), 0, maxq)
        deq = (q - z) * s
        err = W[t] - deq
        Q[t] = q.to(torch.uint8)
        W[t] = deq
        if t + 1 < C:
            W[t + 1:] -= U[t, t + 1:].double()[:, None] * err[None, :]
    return Q, W


@pytest.mark.parametrize("block", [32, 128])
def test_solver_matches_definition(block):
    from helpers import random_spd
    C, R = 96, 40
    g = torch.Generator().manual_seed(5)
    Wt = (torch.randn(C, R, generator=g) * 0.02).float()
    H = random_spd(C, 6)
    H[range(C), range(C)] += 0.01 * H.diag().mean()
    T = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    U = (T / T.diag()[:, None]).contiguous()
    S = torch.full((C, R), 0.01) + torch.rand(C, R, generator=g) * 0.002
    Z = torch.full((C, R), 8.0)
    Wc = Wt.clone()
    q = O.gptq_solver(Wc, U, S, Z, 4, block=block)
    qn, Wn = _naive_gptq(Wt, U, S, Z)
    assert float((q == qn).float().mean()) > 0.995
    assert torch.allclose(Wc.double(), Wn, atol=2e-2)


def test_sparse_solver_keeps_one_of_four():
    from helpers import random_spd
    C, R = 64, 24
    g = torch.Generator().manual_seed(7)
    Wt = (torch.randn(C, R, generator=g) * 0.02).float()
    H = random_spd(C, 8)
    H[range(C), range(C)] += 0.01 * H.diag().mean()
    T = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True).contiguous()
    S = torch.full((C, R), 0.01)
    Z = torch.full((C, R), 8.0)
    Wc = Wt.clone()
    q, M = O.sparsegptq14_solver(Wc, T.clone(), S, Z, 4)
    Mi = M.view(torch.int32).numpy().astype(np.uint32)
    for gidx in range(C // 32):
        for r in range(R):
            m = int(Mi[gidx, r])
            for i in range(8):
                assert bin((m >> (4 * i)) & 0xF).count("1") == 1
                for c in range(4):
                    col = gidx * 32 + 4 * i + c
                    if not (m >> (4 * i + c)) & 1:
                        assert q[col, r] == 0 and Wc[col, r] == 0.0


def test_pack_int4_matches_compressed_tensors():
    ct = pytest.importorskip("compressed_tensors.compressors")
    g = torch.Generator().manual_seed(9)
    for (R, C, gs, sym) in [(8, 64, 32, True), (5, 100, 32, False), (3, 24, 8, False)]:
        q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
        G = (C + gs - 1) // gs
        zero = torch.full((R, G), 8.0) if sym else torch.randint(0, 16, (R, G), generator=g).float()
        ref = O.pack_weight({"qweight": q, "scale": torch.ones(R, G), "zero": zero}, 4, sym, gs)["weight_packed"]
        mine = O.pack_int4(q, zero, gs)
        assert torch.equal(ref, mine)
    # known answer from the packer itself: values -8..-1 -> 0x76543210
    v = torch.arange(-8, 0, dtype=torch.int8).view(1, 8)
    assert int(ct.pack_to_int32(v, 4)[0, 0]) == 0x76543210
    assert int(O.pack_int4((v + 8).to(torch.uint8), torch.full((1, 1), 8.0), 8)[0, 0]) == 0x76543210


def test_pack_sparse14_layout():
    R, C = 6, 96  # G32 = 3 -> odd tail word must be zero
    g = torch.Generator().manual_seed(11)
    q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
    keep = torch.randint(0, 4, (C // 4, R), generator=g)
    M = torch.zeros((3, R), dtype=torch.int64)
    for grp in range(C // 4):
        for r in range(R):
            M[grp // 8, r] |= 1 << (4 * (grp % 8) + int(keep[grp, r]))
    M32 = M.to(torch.int32) if int(M.max()) < 2 ** 31 else torch.from_numpy(M.numpy().astype(np.uint32).view(np.int32))
    M32 = torch.from_numpy(M.numpy().astype(np.uint32).view(np.int32).copy())
    sc = torch.rand(3, R, generator=g) * 0.01 + 0.001
    out = O.pack_sparsegptq14_to_u64x2(q, M32, sc).numpy().view(np.uint64)
    assert out.shape == (2, R, 2)
    for gid in range(3):
        for r in range(R):
            w = int(out[gid // 2, r, gid % 2])
            sbits = (w >> 48) & 0xFFFF
            assert sbits == int(sc[gid, r].to(torch.bfloat16).view(torch.int16)) & 0xFFFF
            for i in range(8):
                c = int(keep[gid * 8 + i, r])
                assert (w >> (32 + 2 * i)) & 3 == c
                assert (w >> (4 * i)) & 0xF == int(q[r, gid * 32 + 4 * i + c])
    assert np.all(out[1, :, 1] == 0)


def test_fp8_block_dequant_rule():
    g = torch.Generator().manual_seed(13)
    O_, I_ = 200, 256
    w = (torch.randn(O_, I_, generator=g)).to(torch.float8_e4m3fn)
    sinv = torch.rand(2, 2, generator=g) + 0.5
    out = O.fp8_block_dequant(w, sinv)
    assert out.dtype == torch.bfloat16
    assert out[130, 200] == (w[130, 200].float() * sinv[1, 1]).to(torch.bfloat16)
    assert out[5, 5] == (w[5, 5].float() * sinv[0, 0]).to(torch.bfloat16)
