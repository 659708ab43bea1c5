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
