"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark configurations.

No model checkpoint or calibration set is available offline; these generators stand in for them:
weights ~ N(0, 0.02) (optionally a few input columns x20, or 0.1 % entries x10), activations = per-channel
scale exp(N(0,1)) times Student-t(nu=4) entries, router logits N(0,1) plus a Zipf(s=1.1) per-expert bias.
Every expert's weights depend only on (seed, expert id), so a sharded run sees the same layer as a
single-GPU run.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class LayerShape:
    name: str
    n_experts: int
    n_shared: int
    hidden: int
    inter: int
    tokens: int
    top_k: int
    router: str = "softmax"       # or "sigmoid_group"
    n_groups: int = 1
    topk_groups: int = 1
    fp8_weights: bool = False
    outlier_frac: float = 0.0


CONFIGS = {
    "qwen3_30b_a3b": LayerShape("qwen3_30b_a3b", 128, 0, 2048, 768, 65536, 8),
    "deepseek_v3": LayerShape("deepseek_v3", 256, 1, 7168, 2048, 131072, 8, "sigmoid_group", 8, 4, True),
    "minimax_m2": LayerShape("minimax_m2", 256, 0, 3072, 1536, 65536, 8, outlier_frac=0.001),
    "kimi_k2": LayerShape("kimi_k2", 384, 1, 7168, 2048, 262144, 8),
}


def student_t_activations(T, C, seed, device="cpu", nu=4, chunk=8192):
    g = torch.Generator(device=device).manual_seed(seed)
    ch = torch.exp(torch.randn(C, generator=g, device=device))
    out = torch.empty((T, C), dtype=torch.bfloat16, device=device)
    for t0 in range(0, T, chunk):
        t1 = min(T, t0 + chunk)
        z = torch.randn(t1 - t0, C, generator=g, device=device)
        chi = torch.zeros_like(z)
        for _ in range(nu):
            chi += torch.randn(t1 - t0, C, generator=g, device=device) ** 2
        out[t0:t1] = (z / torch.sqrt(chi / nu) * ch).to(torch.bfloat16)
    return out


def zipf_bias(n_experts, seed, s=1.1, device="cpu"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    ranks = torch.randperm(n_experts, generator=g).float() + 1.0
    w = ranks.pow(-s)
    return torch.log(w / w.sum() * n_experts).to(device)


def router_logits(shape: LayerShape, T, seed, device="cpu"):
    """Router logits [T,E] fp32: N(0,1) plus the Zipf(1.1) per-expert bias."""
    g = torch.Generator(device=device).manual_seed(seed + 17)
    E = shape.n_experts
    return torch.randn(T, E, generator=g, device=device) + zipf_bias(E, seed + 18, device=device)


def route(shape: LayerShape, T, seed, device="cpu", logits=None):
    """Top-k expert ids [T,k] int32 for the layer's router type, in torch (the statement the device kernel
    forge_route_topk is checked against)."""
    E = shape.n_experts
    if logits is None:
        logits = router_logits(shape, T, seed, device)
    if shape.router == "softmax":
        scores = torch.softmax(logits, dim=-1)
        ids = scores.topk(shape.top_k, dim=-1).indices
    else:
        scores = torch.sigmoid(logits)
        grp = scores.view(T, shape.n_groups, E // shape.n_groups)
        gscore = grp.topk(2, dim=-1).values.sum(-1)
        keep = gscore.topk(shape.topk_groups, dim=-1).indices
        mask = torch.zeros(T, shape.n_groups, dtype=torch.bool, device=device)
        mask.scatter_(1, keep, True)
        masked = grp.masked_fill(~mask.unsqueeze(-1), float("-inf")).view(T, E)
        ids = masked.topk(shape.top_k, dim=-1).indices
    return ids.to(torch.int32).contiguous()


def expert_weights(shape: LayerShape, expert_ids, seed, device="cpu"):
    """(Wg [n,I,H], Wu [n,I,H], Wd [n,H,I]) bf16 for the listed expert ids."""
    H, I = shape.hidden, shape.inter
    n = len(expert_ids)
    Wg = torch.empty((n, I, H), dtype=torch.bfloat16, device=device)
    Wu = torch.empty((n, I, H), dtype=torch.bfloat16, device=device)
    Wd = torch.empty((n, H, I), dtype=torch.bfloat16, device=device)
    for i, e in enumerate(expert_ids):
        g = torch.Generator(device=device).manual_seed(seed * 100003 + int(e))
        for dst, shp in ((Wg, (I, H)), (Wu, (I, H)), (Wd, (H, I))):
            w = torch.randn(shp, generator=g, device=device) * 0.02
            if shape.outlier_frac > 0:
                m = torch.rand(shp, generator=g, device=device) < shape.outlier_frac
                w = torch.where(m, w * 10.0, w)
            dst[i] = w.to(torch.bfloat16)
    return Wg, Wu, Wd


def fp8_block_encode(w: torch.Tensor, block: int = 128):
    """Encode to e4m3 with fp32 128x128 block scales (scale = amax/448), DeepSeek-V3 checkpoint style.
    Returns (w_fp8, scale_inv) with  w ~ fp32(w_fp8) * scale_inv[tile]."""
    O, I = w.shape
    nO, nI = (O + block - 1) // block, (I + block - 1) // block
    wp = torch.zeros((nO * block, nI * block), dtype=torch.float32, device=w.device)
    wp[:O, :I] = w.to(torch.float32)
    tiles = wp.view(nO, block, nI, block)
    amax = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale_inv = (amax / 448.0).to(torch.float32)
    q = (tiles / scale_inv[:, None, :, None]).view(nO * block, nI * block)[:O, :I]
    return q.to(torch.float8_e4m3fn).contiguous(), scale_inv.contiguous()


def dense_linear_case(seed=1, R=768, C=2048, T=4096, device="cpu"):
    """Single dense Linear: W ~ N(0,0.02) with 8 input columns x20; heavy-tailed X."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = torch.randn(R, C, generator=g, device=device) * 0.02
    cols = torch.randperm(C, generator=g, device=device)[:8]
    W[:, cols] *= 20.0
    X = student_t_activations(T, C, seed + 1, device=device)
    return W.to(torch.bfloat16), X
