"""Host-side pieces that need no GPU: synthetic layers, routing model, fp8 block encoding."""
import torch

import ref_port as O
from forge import synth


def test_expert_weights_independent_of_sharding():
    shape = synth.LayerShape("t", 6, 0, 32, 16, 64, 2)
    Wg, Wu, Wd = synth.expert_weights(shape, range(6), seed=5)
    Wg2, _, Wd2 = synth.expert_weights(shape, [4, 5], seed=5)
    assert torch.equal(Wg[4:].view(torch.int16), Wg2.view(torch.int16))
    assert torch.equal(Wd[4:].view(torch.int16), Wd2.view(torch.int16))
    assert Wg.shape == (6, 16, 32) and Wd.shape == (6, 32, 16)


def test_router_topk_shapes_and_skew():
    for router, groups in (("softmax", (1, 1)), ("sigmoid_group", (4, 2))):
        shape = synth.LayerShape("t", 32, 0, 16, 8, 2048, 4, router, *groups)
        ids = synth.route(shape, 2048, seed=2)
        assert ids.shape == (2048, 4) and ids.dtype == torch.int32
        assert int(ids.min()) >= 0 and int(ids.max()) < 32
        # top-k never repeats an expert for one token
        assert all(len(set(row.tolist())) == 4 for row in ids[:64])
        counts = torch.bincount(ids.reshape(-1).long(), minlength=32)
        assert counts.max() > 2 * counts.float().mean()  # Zipf bias makes some experts hot


def test_fp8_block_roundtrip_through_oracle():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(200, 256, generator=g) * 0.02
    q, sinv = synth.fp8_block_encode(w)
    assert q.dtype == torch.float8_e4m3fn and sinv.shape == (2, 2)
    back = O.fp8_block_dequant(q, sinv).float()
    assert float((back - w).abs().max()) < 0.07 * float(w.abs().max())


def test_activation_model_is_heavy_tailed():
    X = synth.student_t_activations(4096, 64, seed=4).float()
    k = ((X - X.mean(0)) ** 4).mean(0) / (X.var(0) ** 2)
    assert float(k.median()) > 4.0  # well above the Gaussian kurtosis of 3


def test_checkpoint_layouts(tmp_path):
    """Keys, shapes and dtypes of the block tensors match what the reference's writers emit
    (pack_quantized.py:279-313 for dense W4, quant.py:615-622 for the stacked Wpair tensors)."""
    import torch
    from safetensors.torch import load_file
    from forge import checkpoint
    n, I, H, gs = 3, 64, 128, 32
    g = torch.Generator().manual_seed(0)

    def fam(R, C):
        return {"qweight": torch.randint(0, 16, (n, R, C), generator=g, dtype=torch.uint8),
                "weight_packed": torch.randint(-2 ** 31, 2 ** 31 - 1, (n, R, C // 8), generator=g, dtype=torch.int32),
                "weight_scale": torch.rand(n, R, C // gs, generator=g).to(torch.float16),
                "qzeros": torch.randint(0, 16, (n, R, C // gs), generator=g).float(),
                "wpair": torch.randint(0, 2 ** 62, (n, (C // 32 + 1) // 2, R, 2), generator=g, dtype=torch.int64)}

    out = {"gate": fam(I, H), "up": fam(I, H), "down": fam(H, I)}
    t = checkpoint.dense_block_tensors(out, "model.layers.3.", n_routed=2, symmetric=False)
    assert len(t) == 3 * n * 4
    k = "model.layers.3.mlp.experts.1.down_proj"
    assert t[k + ".weight_packed"].shape == (H, I // 8) and t[k + ".weight_packed"].dtype == torch.int32
    assert t[k + ".weight_shape"].tolist() == [H, I] and t[k + ".weight_shape"].dtype == torch.int64
    assert t[k + ".weight_scale"].shape == (H, I // gs) and t[k + ".weight_scale"].dtype == torch.float16
    assert t[k + ".weight_zero_point"].dtype == torch.uint8
    assert "model.layers.3.mlp.shared_experts.gate_proj.weight_packed" in t          # the one shared expert
    assert not any("weight_zero_point" in key for key in
                   checkpoint.dense_block_tensors(out, "p.", n_routed=3, symmetric=True))
    s = checkpoint.sparse_block_tensors(out, "model.layers.3.")
    w13 = s["model.layers.3.mlp.experts.gate_up_proj.w13_weight"]
    assert w13.shape == (n, (H // 32 + 1) // 2, 2 * I, 2)
    assert torch.equal(w13[:, :, :I], out["gate"]["wpair"]) and torch.equal(w13[:, :, I:], out["up"]["wpair"])
    assert s["model.layers.3.mlp.experts.down_proj.w2_weight"].shape == (n, (I // 32 + 1) // 2, H, 2)
    wm = checkpoint.write_block_shard(str(tmp_path / "block_003.safetensors"), {**t, **s})
    back = load_file(str(tmp_path / "block_003.safetensors"))
    assert set(wm) == set(back) and all(v == "block_003.safetensors" for v in wm.values())
    assert torch.equal(back[k + ".weight_packed"], t[k + ".weight_packed"])
    cfg = checkpoint.quantization_config(4, 128, symmetric=False)
    assert cfg["format"] == "pack-quantized" and cfg["config_groups"]["group_0"]["weights"]["symmetric"] is False


def test_writers_driver_dict_index_and_resume(tmp_path):
    """quantized_weight.pt with the driver's keys (quant.py:498-511), the incrementally rewritten index
    (forge/utils/io.py:630-672), dropped dense expert keys, resume by existing shard, gather re-ordering."""
    import json
    import torch
    from safetensors.torch import load_file
    from forge import checkpoint
    g = torch.Generator().manual_seed(1)
    R, C, gs = 8, 64, 32
    q = torch.randint(0, 16, (R, C), generator=g, dtype=torch.uint8)
    s, z = torch.rand(R * C // gs, generator=g), torch.randint(0, 16, (R * C // gs,), generator=g).float()
    res = {"mlp.experts.0.gate_proj": (q, s, z), "mlp.experts.0.gate_proj.info": torch.tensor(0)}
    paths = checkpoint.write_linear_results(str(tmp_path / "save"), 3, res, gs, 4)
    assert paths == [str(tmp_path / "save" / "block.3" / "mlp.experts.0.gate_proj" / "quantized_weight.pt")]
    d = torch.load(paths[0])
    assert set(d) == {"qweight", "scales", "qzeros", "group_size", "bits", "shape"}
    assert d["qweight"].dtype == torch.int8 and d["scales"].dtype == torch.float32 and d["qzeros"].dtype == torch.int32
    assert d["shape"] == (R, C) and d["group_size"] == gs and d["bits"] == 4 and torch.equal(d["qweight"], q.to(torch.int8))
    assert checkpoint.write_linear_results(str(tmp_path / "save"), 3, res, gs, 4) == []          # resume: kept
    assert torch.load(checkpoint.write_run_metadata(str(tmp_path / "save"), 4, gs, True))["quantize_only_experts"] is True

    n, I, H = 2, 32, 64
    fam = lambda R_, C_: {"qweight": torch.zeros(n, R_, C_, dtype=torch.uint8),
                          "weight_packed": torch.randint(0, 99, (n, R_, C_ // 8), generator=g, dtype=torch.int32),
                          "weight_scale": torch.rand(n, R_, C_ // gs, generator=g).to(torch.float16),
                          "qzeros": torch.full((n, R_, C_ // gs), 8.0)}
    out = {"gate": fam(I, H), "up": fam(I, H), "down": fam(H, I)}
    prefix = "model.layers.5."
    base = {"metadata": {"total_size": 1}, "weight_map": {
        f"{prefix}mlp.experts.0.gate_proj.weight": "a.safetensors", f"{prefix}mlp.experts.1.down_proj.weight_scale_inv": "a.safetensors",
        f"{prefix}mlp.shared_experts.gate_proj.weight": "a.safetensors", f"{prefix}self_attn.q_proj.weight": "a.safetensors",
        "model.layers.6.mlp.experts.0.gate_proj.weight": "b.safetensors"}}
    w = checkpoint.IncrementalIndexWriter(str(tmp_path / "base"), str(tmp_path / "out"), base)
    assert not w.block_done(5)
    path = checkpoint.write_moe_block(w, 5, prefix, out, n_routed=n, symmetric=True, sparse=False)
    assert path.endswith("block_005.safetensors") and w.block_done(5)
    idx = json.load(open(tmp_path / "out" / "model.safetensors.index.json"))
    wm = idx["weight_map"]
    assert wm[f"{prefix}mlp.experts.1.down_proj.weight_packed"] == "block_005.safetensors"
    assert f"{prefix}mlp.experts.0.gate_proj.weight" not in wm and f"{prefix}mlp.experts.1.down_proj.weight_scale_inv" not in wm
    assert wm[f"{prefix}mlp.shared_experts.gate_proj.weight"] == "a.safetensors"       # shared experts are never dropped
    assert wm[f"{prefix}self_attn.q_proj.weight"] == "a.safetensors" and "model.layers.6.mlp.experts.0.gate_proj.weight" in wm
    back = load_file(path)
    assert torch.equal(back[f"{prefix}mlp.experts.1.gate_proj.weight_packed"], out["gate"]["weight_packed"][1])
    assert checkpoint.write_moe_block(w, 5, prefix, out, n_routed=n, symmetric=True, sparse=False) is None   # resume
    w2 = checkpoint.IncrementalIndexWriter(str(tmp_path / "base"), str(tmp_path / "out"), base)               # rerun
    assert w2.block_done(5) and f"{prefix}mlp.experts.0.gate_proj.weight" not in w2.weight_map
    assert w2.weight_map[f"{prefix}mlp.experts.0.up_proj.weight_packed"] == "block_005.safetensors"

    owned = [[0, 3], [1, 2, 4]]
    gathered = {"x": [torch.tensor([[0.], [3.]]), torch.tensor([[1.], [2.], [4.]])]}
    assert checkpoint.reorder_gathered(gathered, owned)["x"].flatten().tolist() == [0., 1., 2., 3., 4.]
