"""Parity of the layer-level path (forge.moe) with the CPU oracle on the RECIPES the benchmark configurations use,
at scaled-down shapes: codes >= 99.5 % per matrix, reconstruction loss within 1 % per expert, packed bytes bit-exact
given the codes; plus the device kernels that only the layer path uses (router top-k, grouped expert forward,
reconstruction loss)."""
import pytest
import torch

import ref_port as O
from helpers import rel_fro

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _oracle_matrix(Wm, xin, kw, perm=None, grid=None):
    """The oracle on one Linear.  perm: the engine's activation order (argsort of near-tied diagonals is unspecified,
    ordering noise is not counted as error).  grid: (scales, qzeros) to solve with instead of the oracle's own search
    (used where the MSE search, which runs on approximate hardware lg2/ex2 in the kernels, picked another candidate
    for a few groups: the codes are then compared on every group, given the same grid)."""
    ho = O.OracleGPTQ(Wm, **kw)
    ho.update(xin)
    ho._prep()
    if perm is not None:
        ho.H = ho.H[ho.perm_inv][:, ho.perm_inv]
        ho.perm = perm.cpu().long()
        ho.perm_inv = torch.argsort(ho.perm)
        ho.H = ho.H[ho.perm][:, ho.perm]
    own = ho._quant_grid()
    if grid is not None:
        ho._quant_grid = lambda *a, **k: (grid[0].clone(), grid[1].clone())
    return ho, ho.quantize(), own


def _token_lists(ids, n_routed, T, n_tail):
    return [torch.nonzero((ids == e).any(1)).flatten() for e in range(n_routed)] + [torch.arange(T)] * n_tail


def _check_layer(out, lists, X, Ws, acts, kw, gs, mse=False, min_codes=0.995, sparse=False):
    """Per expert and matrix: scales, codes, reconstruction loss against the oracle."""
    worst = 1.0
    for e in range(len(lists)):
        xe = X[lists[e]]
        for name, Wm, xin in (("gate", Ws[0][e], xe), ("up", Ws[1][e], xe), ("down", Ws[2][e], acts[e])):
            res = out[name]
            perm = res["perm"][e] if res["perm"] is not None else None
            s_eng, z_eng = res["scales"][e].reshape(-1).cpu(), res["qzeros"][e].reshape(-1).cpu()
            ho, o, own = _oracle_matrix(Wm, xin, kw, perm, grid=(s_eng, z_eng) if mse else None)
            if mse:
                assert float((s_eng == own[0]).float().mean()) >= 0.99, (name, e)
            else:
                assert torch.equal(s_eng, o[1]) and torch.equal(z_eng, o[2]), (name, e)
            assert int(res["info"][e]) == 0
            q_eng = res["qweight"][e].cpu()
            agree = float((q_eng == o[0]).float().mean())
            worst = min(worst, agree)
            assert agree >= min_codes, (name, e, agree)
            if xin.shape[0] == 0:
                continue
            if sparse:
                keep_e = _keep_mask(res["M"][e].cpu(), ho.perm)
                keep_o = _keep_mask(o[3], ho.perm)
                What_e = O.dequantize_forge_full(torch.float32, q_eng, s_eng, z_eng, gs) * keep_e
                What_o = O.dequantize_forge_full(torch.float32, o[0], o[1], o[2], gs) * keep_o
            else:
                What_e = O.dequantize_forge_full(torch.float32, q_eng, s_eng, z_eng, gs)
                What_o = O.dequantize_forge_full(torch.float32, o[0], o[1], o[2], gs)
            le, lo = O.recon_loss(ho.W, What_e, xin), O.recon_loss(ho.W, What_o, xin)
            assert abs(le - lo) <= 0.01 * lo, (name, e, le, lo)
    return worst


def _keep_mask(M, perm):
    """[R, C] 0/1 mask in ORIGINAL column order from the solver's M [C/32, R] (bit t of word g = permuted column
    32 g + t is kept)."""
    M = M.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    G32, R = M.shape
    bits = ((M.unsqueeze(-1) >> torch.arange(32)) & 1).permute(1, 0, 2).reshape(R, G32 * 32).float()   # permuted order
    out = torch.zeros_like(bits)
    out[:, perm] = bits[:, :perm.numel()]
    return out


def _engine_acts(out, lists):
    offs = out["routing"]["offsets"].cpu()
    act = out["routing"]["act"].cpu()
    return [act[int(offs[e]):int(offs[e + 1])] for e in range(len(lists))]


# ---------------------------------------------------------------------------------------------- recipes
def test_recipe_asym_mse_g128_inversion_free():
    """Qwen3-30B-A3B recipe: softmax top-k routing, W4 asymmetric g128, MSE scale search, inversion-free solve."""
    from forge import synth, moe
    shape = synth.LayerShape("q", 8, 0, 512, 256, 4096, 2)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=31)
    ids = synth.route(shape, shape.tokens, seed=31)
    Wg, Wu, Wd = synth.expert_weights(shape, range(8), seed=31)
    cfg = moe.MoEQuantConfig(bits=4, group_size=128, symmetric=False, quantization_scale="mse",
                             quantization_order="default", rel_damp=0.01, algorithm="gptq", inversion_free=True)
    qz = moe.MoELayerQuantizer(cfg)
    Wd_ = [w.to(DEV) for w in (Wg, Wu, Wd)]
    out = qz.quantize_experts(X.to(DEV), ids.to(DEV), *Wd_)
    assert qz._form([Wd_[0]]) == 1
    lists = _token_lists(ids, 8, shape.tokens, 0)
    acts = _engine_acts(out, lists)
    kw = dict(bits=4, group_size=128, symmetric=False, quantization_scale="mse", quantization_order="default",
              rel_damp=0.01, algorithm="gptq")
    _check_layer(out, lists, X, (Wg, Wu, Wd), acts, kw, 128, mse=True)
    # device-side reconstruction loss against the fp64 host evaluation
    dl = qz.reconstruction_loss(out, X.to(DEV), *Wd_)
    for name, Wm in (("gate", Wg), ("up", Wu), ("down", Wd)):
        for e in (0, 5):
            xin = acts[e] if name == "down" else X[lists[e]]
            What = O.dequantize_forge_full(torch.float32, out[name]["qweight"][e].cpu(), out[name]["scales"][e].cpu(),
                                           out[name]["qzeros"][e].cpu(), 128)
            ref = O.recon_loss(Wm[e], What, xin)
            assert abs(float(dl[name][e]) - ref) <= 1e-3 * ref, (name, e, float(dl[name][e]), ref)


def test_recipe_fp8_sigmoid_group_actorder_through_host_api():
    """DeepSeek-V3 recipe: sigmoid group-limited routing (device kernel), fp8 e4m3 weights + 128x128 block scales
    de-quantised on the device, W4 symmetric g128, activation order, one shared expert, through
    quantize_experts_host."""
    from forge import synth, moe, ops
    shape = synth.LayerShape("d", 16, 1, 512, 256, 4096, 4, "sigmoid_group", 4, 2, True)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=41)
    logits = synth.router_logits(shape, shape.tokens, seed=41)
    ids_t = synth.route(shape, shape.tokens, seed=41, logits=logits)
    ids = ops.route_topk(logits.to(DEV), shape.top_k, "sigmoid_group", shape.n_groups, shape.topk_groups)
    same = (ids.cpu() == ids_t).all(1).float().mean()
    assert float(same) >= 0.999, float(same)      # the rest are score ties at the last place of fp32
    ids_h = ids.cpu()
    W = synth.expert_weights(shape, range(17), seed=41)
    enc = [[synth.fp8_block_encode(w) for w in Wm] for Wm in W]
    host_w = [torch.stack([q for q, _ in e]).pin_memory() for e in enc]
    host_s = [torch.stack([s for _, s in e]).float().pin_memory() for e in enc]
    Wdq = [torch.stack([O.fp8_block_dequant(q, s) for q, s in e]) for e in enc]     # what the oracle quantises
    cfg = moe.MoEQuantConfig(bits=4, group_size=128, symmetric=True, quantization_scale="absmax",
                             quantization_order="activation", rel_damp=0.01, algorithm="gptq")
    qz = moe.MoELayerQuantizer(cfg)
    out, host = qz.quantize_experts_host(X.pin_memory(), ids_h.pin_memory(), *host_w, e_begin=0, dense_tail=1,
                                         fp8_scale_inv=host_s)
    lists = _token_lists(ids_h, 16, shape.tokens, 1)
    assert out["counts"].tolist() == [len(l) for l in lists]
    acts = _engine_acts(out, lists)
    for e in (0, 16):   # the engine's activations are the block forward's
        if len(lists[e]):
            assert rel_fro(acts[e].float(), O.swiglu_down_input(X[lists[e]], Wdq[0][e], Wdq[1][e]).float()) < 2e-2
    kw = dict(bits=4, group_size=128, symmetric=True, quantization_scale="absmax", quantization_order="activation",
              rel_damp=0.01, algorithm="gptq")
    _check_layer(out, lists, X, Wdq, acts, kw, 128)
    for nm in ("gate", "up", "down"):
        pk = torch.stack([O.pack_int4(out[nm]["qweight"][e].cpu(), out[nm]["qzeros"][e].cpu(), 128) for e in range(17)])
        assert torch.equal(host[f"{nm}.weight_packed"], pk)


def test_recipe_sparse14_g128_repeated_scale():
    """MiniMax-M2 recipe: SparseGPT 1:4 + W4 symmetric at group size 128; the Wpair layout takes one scale per 32
    columns, i.e. each group scale four times."""
    from forge import synth, moe
    shape = synth.LayerShape("m", 8, 0, 512, 256, 4096, 2, outlier_frac=0.001)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=51)
    ids = synth.route(shape, shape.tokens, seed=51)
    Wg, Wu, Wd = synth.expert_weights(shape, range(8), seed=51)
    cfg = moe.MoEQuantConfig(bits=4, group_size=128, symmetric=True, quantization_scale="absmax",
                             quantization_order="default", rel_damp=0.01, algorithm="sparsegptq")
    qz = moe.MoELayerQuantizer(cfg)
    out = qz.quantize_experts(X.to(DEV), ids.to(DEV), Wg.to(DEV), Wu.to(DEV), Wd.to(DEV))
    lists = _token_lists(ids, 8, shape.tokens, 0)
    acts = _engine_acts(out, lists)
    kw = dict(bits=4, group_size=128, symmetric=True, quantization_scale="absmax", quantization_order="default",
              rel_damp=0.01, algorithm="sparsegptq")
    worst = _check_layer(out, lists, X, (Wg, Wu, Wd), acts, kw, 128, min_codes=0.995, sparse=True)
    print("sparse g128: worst code agreement", worst)
    for nm, Wm in (("gate", Wg), ("up", Wu), ("down", Wd)):
        C = Wm.shape[2]
        for e in range(8):
            s32 = out[nm]["scales"][e].cpu().repeat_interleave(4, 1)[:, :C // 32].T.contiguous()
            wp = O.pack_sparsegptq14_to_u64x2(out[nm]["qweight"][e].cpu(), out[nm]["M"][e].cpu(), s32)
            assert torch.equal(out[nm]["wpair"][e].cpu(), wp), (nm, e)


def test_recipe_sharded_slices_equal_the_unsharded_layer():
    """Kimi-K2 recipe (routed + one shared expert, placed by load): the slices two logical ranks compute through
    balance_experts / placement_tables, run one after the other on this GPU, are bit-identical to the unsharded run."""
    from forge import synth, moe, dist as fdist
    shape = synth.LayerShape("k", 12, 1, 256, 128, 3072, 2)
    E, T = shape.n_experts, shape.tokens
    X = synth.student_t_activations(T, shape.hidden, seed=61).to(DEV)
    ids = synth.route(shape, T, seed=61)
    W = synth.expert_weights(shape, range(E + 1), seed=61)
    cfg = moe.MoEQuantConfig(bits=4, group_size=128, symmetric=True, quantization_scale="absmax", rel_damp=0.01)
    full = moe.MoELayerQuantizer(cfg).quantize_experts(X, ids.to(DEV), *[w.to(DEV) for w in W], e_begin=0, dense_tail=1)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E)
    owned = fdist.balance_experts(counts.tolist(), 2, 1, T, fixed_cost_tokens=2000.0)
    table, spans = fdist.placement_tables(owned, E)
    ids_r = table[ids.long()].to(torch.int32).to(DEV)
    seen = []
    for r in range(2):
        mine = owned[r]
        e0, n_r = spans[r]
        part = moe.MoELayerQuantizer(cfg).quantize_experts(X, ids_r, *[w[mine].to(DEV) for w in W], e_begin=e0,
                                                           dense_tail=len(mine) - n_r)
        for j, e in enumerate(mine):
            seen.append(e)
            for nm in ("gate", "up", "down"):
                for key in ("qweight", "scales", "weight_packed"):
                    assert torch.equal(part[nm][key][j], full[nm][key][e]), (r, e, nm, key)
    assert sorted(seen) == list(range(E + 1))


def test_merged_and_separate_gate_up_launches_give_identical_codes():
    from forge import synth, moe
    shape = synth.LayerShape("g", 6, 0, 256, 128, 2048, 2)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=71).to(DEV)
    ids = synth.route(shape, shape.tokens, seed=71).to(DEV)
    W = synth.expert_weights(shape, range(6), seed=71)
    outs = []
    for merge in (True, False):
        cfg = moe.MoEQuantConfig(bits=4, group_size=128, symmetric=True, rel_damp=0.01, merge_gate_up=merge)
        outs.append(moe.MoELayerQuantizer(cfg).quantize_experts(X, ids, *[w.to(DEV) for w in W]))
    for nm in ("gate", "up", "down"):
        assert torch.equal(outs[0][nm]["qweight"], outs[1][nm]["qweight"])
    assert moe.MoELayerQuantizer.merge_pays(128, 768, 148) in (True, False)


def test_gate_and_up_with_different_zero_columns_get_separate_factors():
    """An input column that is all zero in up_proj only: the shared factor is not valid for up (forge/gptq.py:145-149
    zeroes that row and column of ITS Hessian), the device flag says so and the layer is redone per matrix."""
    from forge import synth, moe
    shape = synth.LayerShape("z", 4, 0, 256, 128, 2048, 2)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=81)
    ids = synth.route(shape, shape.tokens, seed=81)
    Wg, Wu, Wd = synth.expert_weights(shape, range(4), seed=81)
    Wu[2][:, 17] = 0
    cfg = moe.MoEQuantConfig(bits=4, group_size=64, symmetric=True, rel_damp=0.01)
    out = moe.MoELayerQuantizer(cfg).quantize_experts(X.to(DEV), ids.to(DEV), Wg.to(DEV), Wu.to(DEV), Wd.to(DEV))
    lists = _token_lists(ids, 4, shape.tokens, 0)
    kw = dict(bits=4, group_size=64, symmetric=True, quantization_scale="absmax", quantization_order="default",
              rel_damp=0.01, algorithm="gptq")
    for nm, Wm in (("gate", Wg), ("up", Wu)):
        _, o, _ = _oracle_matrix(Wm[2], X[lists[2]], kw)
        assert float((out[nm]["qweight"][2].cpu() == o[0]).float().mean()) >= 0.995, nm


# ---------------------------------------------------------------------------------------------- kernels
@pytest.mark.parametrize("mode,E,k,ng,tg", [("softmax", 128, 8, 1, 1), ("sigmoid", 64, 6, 1, 1),
                                             ("sigmoid_group", 256, 8, 8, 4), ("sigmoid_group", 48, 4, 4, 2),
                                             ("softmax", 100, 3, 1, 1)])
def test_route_topk_matches_torch(mode, E, k, ng, tg):
    from forge import ops, synth
    shape = synth.LayerShape("r", E, 0, 8, 8, 5000, k, "softmax" if mode != "sigmoid_group" else "sigmoid_group", ng, tg)
    logits = synth.router_logits(shape, 5000, seed=3).to(DEV)
    if mode == "sigmoid":
        want = torch.sigmoid(logits).topk(k, dim=-1).indices.to(torch.int32)
    else:
        want = synth.route(shape, 5000, seed=3, device=DEV, logits=logits)
    got, w = ops.route_topk(logits, k, mode, ng, tg, want_weights=True)
    rows_equal = (got == want).all(1)
    assert float(rows_equal.float().mean()) >= 0.999
    # where a row differs, it is a tie (or a last-place difference of the score) and the chosen sets still score alike
    sc = torch.softmax(logits, -1) if mode == "softmax" else torch.sigmoid(logits)
    assert torch.allclose(sc.gather(1, got.long()).sum(1), sc.gather(1, want.long()).sum(1), rtol=1e-5, atol=1e-6)
    assert torch.allclose(w, sc.gather(1, got.long()), rtol=1e-5, atol=1e-7)
    assert bool((got[:, :-1] != got[:, 1:]).all()) and int(got.min()) >= 0 and int(got.max()) < E


@pytest.mark.parametrize("H,I,counts", [(64, 32, [5, 0, 130]), (512, 256, [300, 129, 1, 64]), (320, 136, [200, 77]),
                                        (2048, 768, [1000])])
def test_expert_forward_matches_block_forward(H, I, counts):
    """forge_expert_swiglu_grouped (tcgen05, gather fused) against the plain-FMA kernel and the oracle's restatement of
    the HF block forward."""
    from forge import ops
    g = torch.Generator().manual_seed(H + I)
    T = 1500
    X = (torch.randn(T, H, generator=g) * torch.exp(0.5 * torch.randn(H, generator=g))).to(torch.bfloat16)
    nb = len(counts)
    Wg = (torch.randn(nb, I, H, generator=g) * 0.05).to(torch.bfloat16)
    Wu = (torch.randn(nb, I, H, generator=g) * 0.05).to(torch.bfloat16)
    lists = [torch.randperm(T, generator=g)[:c].sort().values.to(torch.int32) for c in counts]
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int64)
    total = int(offsets[-1])
    tl = torch.cat(lists).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    args = (X.to(DEV), tl, offsets.to(DEV), Wg.to(DEV), Wu.to(DEV), total + 7)
    out_tc = ops.expert_swiglu_grouped(*args, status=status)
    out_fma = ops.expert_swiglu_grouped(*args, simt=True, status=status)
    assert int(status.item()) == 0
    # against the FMA kernel: same roundings, only the summation order differs -> a few last-place bf16 differences
    assert rel_fro(out_tc[:total].float().cpu(), out_fma[:total].float().cpu()) < 4e-3
    for b in range(nb):
        if counts[b] == 0:
            continue
        ref = O.swiglu_down_input(X[lists[b].long()], Wg[b], Wu[b]).float()
        got = out_tc[int(offsets[b]):int(offsets[b + 1])].float().cpu()
        assert rel_fro(got, ref) < 4e-3, b
    # contiguous rows (no token list): rows offsets[b] .. of X itself
    offs2 = torch.tensor([0, 100, 100, 356], dtype=torch.int64)
    out2 = ops.expert_swiglu_grouped(X.to(DEV), None, offs2.to(DEV), Wg[:3].to(DEV) if nb >= 3 else Wg[:1].repeat(3, 1, 1).to(DEV),
                                     Wu[:3].to(DEV) if nb >= 3 else Wu[:1].repeat(3, 1, 1).to(DEV), 356, status=status)
    wg3 = Wg[:3] if nb >= 3 else Wg[:1].repeat(3, 1, 1)
    wu3 = Wu[:3] if nb >= 3 else Wu[:1].repeat(3, 1, 1)
    assert rel_fro(out2[100:356].float().cpu(), O.swiglu_down_input(X[100:356], wg3[2], wu3[2]).float()) < 4e-3


def test_bounds_checks_skip_bad_claims_and_report_them():
    """Offsets that claim more rows than the token list holds, and a list entry that is not a row of X: the kernels
    skip the slot / treat the row as zeros and raise FORGE_ERR_INVALID in the status word; nothing out of bounds is read."""
    from forge import ops, _abi
    g = torch.Generator().manual_seed(2)
    C, T = 128, 256
    X = torch.randn(T, C, generator=g).to(torch.bfloat16).to(DEV)
    tl = torch.arange(200, dtype=torch.int32, device=DEV)
    H = torch.full((2, C, C), 7.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    offsets = torch.tensor([0, 100, 3000], dtype=torch.int64, device=DEV)     # slot 1 claims 2900 rows of a 200-entry list
    ops.hessian_grouped(X, C, tl, offsets, H, status=status)
    assert int(status.item()) == _abi.ERR_INVALID
    assert bool((H[1] == 7.0).all())                                          # skipped untouched
    ref = (X[:100].float().T @ X[:100].float()) * (2.0 / 100)
    assert rel_fro(H[0].cpu(), ref.cpu()) < 1e-4                              # the good slot is still right
    status.zero_()
    tl2 = tl.clone()
    tl2[5] = T + 40                                                           # not a row of X
    tl2[6] = -3
    H2 = torch.empty((1, C, C), device=DEV)
    ops.hessian_grouped(X, C, tl2, torch.tensor([0, 100], dtype=torch.int64, device=DEV), H2, status=status)
    assert int(status.item()) == _abi.ERR_INVALID
    keep = [i for i in range(100) if i not in (5, 6)]
    ref2 = (X[keep].float().T @ X[keep].float()) * (2.0 / 100)
    assert rel_fro(H2[0].cpu(), ref2.cpu()) < 1e-4
    # the expert forward applies the same checks
    status.zero_()
    Wg = torch.randn(2, 64, C, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((210, 64), 3.0, dtype=torch.bfloat16, device=DEV)
    ops.expert_swiglu_grouped(X, tl, offsets, Wg, Wg, 210, out=out, status=status)
    assert int(status.item()) == _abi.ERR_INVALID
    assert bool((out[100:].float() == 3.0).all())


@pytest.mark.parametrize("nb,R,C,sparse", [(3, 256, 640, False), (40, 1024, 256, False), (3, 128, 384, True)])
def test_presplit_factor_pieces_give_identical_codes(nb, R, C, sparse):
    """forge_solve_split_u + bulk copies of the operand pieces against the solver splitting U itself: the same values
    reach the same MMAs in the same order, so the codes are identical.  (3 x 2 strips: the deep ring; 40 x 8 strips:
    the shallow ring, three CTAs per SM.)"""
    from forge import ops
    from helpers import random_spd
    g = torch.Generator().manual_seed(nb + C)
    W = (torch.randn(nb, R, C, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    nu = min(nb, 3)
    H = torch.stack([random_spd(C, 10 + i) for i in range(nu)]).to(DEV)
    A, _, _ = ops.hessian_gather_damp(H, None, None, None, None, 0.01)
    U, udiag, info = ops.chol_inv_upper(A, zero_lower=False) if sparse else ops.chol_factor(A)
    assert int(info.abs().sum()) == 0
    u_map = (torch.arange(nb, dtype=torch.int32) % nu).to(DEV)
    s, z = ops.quant_grid(W.view(nb * R, C), 128, 4, True)
    kw = dict(perm=None, u_map=u_map, udiag=udiag if sparse else None, sparse14=sparse, form=0 if sparse else 1)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = ops.gptq_solve_batched(W, U, s, z, 128, 4, status=status, **kw)
    b = ops.gptq_solve_batched(W, U, s, z, 128, 4, status=status, usplit=ops.solve_split_u(U), **kw)
    assert int(status.item()) == 0
    if sparse:
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    else:
        assert torch.equal(a, b)


def test_full_width_expert_matches_the_oracle():
    """The benchmark recipe (W4 symmetric g128, activation order, inversion-free solve) at the FULL hidden size of the
    DeepSeek-V3 / Kimi-K2 shapes, 7168, against the oracle: one expert with 8192 tokens, gate / up [512, 7168], down
    [7168, 512].  At this width the Hessian goes through every level of the blocked factorisation (outer blocks of 512,
    block inverse, the multiplication for the rows behind a block, 256 x 256 update tiles) and the solver through its
    wide-matrix build (56 column blocks, errors through tensor memory)."""
    from forge import synth, moe
    shape = synth.LayerShape("w", 1, 0, 7168, 512, 8192, 1)
    X = synth.student_t_activations(shape.tokens, shape.hidden, seed=77)
    ids = torch.zeros((shape.tokens, 1), dtype=torch.int32)
    Wg, Wu, Wd = synth.expert_weights(shape, range(1), seed=77)
    cfg = moe.MoEQuantConfig(bits=4, group_size=128, symmetric=True, quantization_scale="absmax",
                             quantization_order="activation", rel_damp=0.01, algorithm="gptq")
    qz = moe.MoELayerQuantizer(cfg)
    Wdev = [w.to(DEV) for w in (Wg, Wu, Wd)]
    out = qz.quantize_experts(X.to(DEV), ids.to(DEV), *Wdev)
    assert qz._form([Wdev[0]]) == 1
    lists = _token_lists(ids, 1, shape.tokens, 0)
    acts = _engine_acts(out, lists)
    kw = dict(bits=4, group_size=128, symmetric=True, quantization_scale="absmax", quantization_order="activation",
              rel_damp=0.01, algorithm="gptq")
    worst = _check_layer(out, lists, X, (Wg, Wu, Wd), acts, kw, 128)
    assert worst >= 0.995
