"""Layer-level calibration capture for one MoE block.

The reference driver (quant.py:344-406) creates one GPTQ handle per expert Linear, registers one forward hook per
Linear (or one fused-experts hook, forge/utils/engine.py:210-258), runs the block forward so that every hook
feeds `GPTQ.update`, and then calls `quantize()` handle by handle (quant.py:412-512).  That is 3 x n_experts
Hessian updates, host synchronisations and factorisations of batch one.

Here the same block is quantised in one batched pass: the caller hands over the block input X (what the hooks of
gate_proj / up_proj would have seen before the gather), the router's top-k choice, and the expert modules; the
weights are stacked, `forge.moe.MoELayerQuantizer` does the work, and the result comes back keyed by the
reference's layer names with exactly the tuples `GPTQ.quantize()` returns, so the code that consumes them
(quant.py:417-511: casts, dequantised write-back, packing) stays as it is.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from .moe import MoELayerQuantizer, MoEQuantConfig


def topk_from_logits(router_logits: torch.Tensor, top_k: int, scoring: str = "softmax") -> torch.Tensor:
    """Router logits [T, E] -> chosen expert ids int32 [T, top_k] (softmax or sigmoid scores, plain top-k).
    Models with grouped or bias-corrected selection pass their own ids instead."""
    if scoring == "softmax":
        scores = torch.softmax(router_logits.float(), dim=-1)
    elif scoring == "sigmoid":
        scores = torch.sigmoid(router_logits.float())
    else:
        raise ValueError(f"unknown scoring {scoring!r}")
    return torch.topk(scores, top_k, dim=-1).indices.to(torch.int32)


def _stack(mods, name):
    return torch.stack([getattr(m, name).weight.detach() for m in mods]).to(torch.bfloat16).contiguous()


@torch.no_grad()
def quantize_moe_block(experts: Sequence[torch.nn.Module], X: torch.Tensor, topk_ids: torch.Tensor,
                       cfg: MoEQuantConfig, shared_experts: Sequence[torch.nn.Module] = (),
                       prefix: str = "mlp.experts", shared_prefix: str = "mlp.shared_experts",
                       proj_names: Tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj"),
                       quantizer: Optional[MoELayerQuantizer] = None) -> Dict[str, tuple]:
    """experts[e] / shared_experts[j]: modules with three Linear children named `proj_names` (SwiGLU:
    down(silu(gate(x)) * up(x))).  X [T, H] (any float dtype, rounded to bf16), topk_ids [T, k].

    Returns {"<prefix>.<e>.<proj>": (qweight u8 [R,C], scales f32 [R*G], qzeros f32 [R*G][, M u32 [C/32,R]])} —
    the return value of the reference's GPTQ.quantize() for that Linear (forge/gptq.py:129-139) — plus
    "<name>.info" entries (0 = factorised, > 0 = fell back to the identity Hessian like forge/gptq.py:156-170)."""
    gname, uname, dname = proj_names
    mods = list(experts) + list(shared_experts)
    Wg, Wu, Wd = _stack(mods, gname), _stack(mods, uname), _stack(mods, dname)
    dev = Wg.device
    qz = quantizer or MoELayerQuantizer(cfg)
    Xb = X.reshape(-1, X.shape[-1]).to(device=dev, dtype=torch.bfloat16).contiguous()
    ids = topk_ids.reshape(Xb.shape[0], -1).to(device=dev, dtype=torch.int32).contiguous()
    out = qz.quantize_experts(Xb, ids, Wg, Wu, Wd, e_begin=0, dense_tail=len(shared_experts))
    sparse = cfg.algorithm == "sparsegptq"
    result: Dict[str, tuple] = {}
    for i in range(len(mods)):
        base = f"{prefix}.{i}" if i < len(experts) else (
            shared_prefix if len(shared_experts) == 1 else f"{shared_prefix}.{i - len(experts)}")
        for fam, proj in (("gate", gname), ("up", uname), ("down", dname)):
            r = out[fam]
            tup = (r["qweight"][i], r["scales"][i].reshape(-1), r["qzeros"][i].reshape(-1))
            if sparse:
                tup = tup + (r["M"][i],)
            result[f"{base}.{proj}"] = tup
            result[f"{base}.{proj}.info"] = r["info"][i]
    return result
