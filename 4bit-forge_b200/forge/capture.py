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


# ---------------------------------------------------------------------------------------------------------------
# The driver's flow around the batched pass (quant.py:344-417, :489-496, :670-680): obtain X and the router's choice
# from the block's own forward, quantise, write the de-quantised weights back, and run the block again so that the
# NEXT block calibrates on the outputs of the quantised one (sequential activation update).
# ---------------------------------------------------------------------------------------------------------------
class MoEBlockCapture:
    """Two hooks instead of one per expert Linear: a forward pre-hook on the MoE module records its input (what every
    gate_proj / up_proj hook of the reference would have seen, before the per-expert gather), a forward hook on the
    router records its output.  Routers that return logits [T, E] (an nn.Linear gate, e.g. Qwen3-MoE) are turned
    into ids by forge_route_topk with the given scoring; routers that return (indices, weights) (DeepSeek-V3 style
    gate modules) hand over their indices as they are.  Use as a context manager around the calibration forward."""

    def __init__(self, moe_module: torch.nn.Module, router: torch.nn.Module, top_k: int, scoring: str = "softmax",
                 n_groups: int = 1, topk_groups: int = 1):
        self.moe_module, self.router = moe_module, router
        self.top_k, self.scoring, self.n_groups, self.topk_groups = top_k, scoring, n_groups, topk_groups
        self._x, self._ids, self._hooks = [], [], []

    def _pre(self, mod, args, kwargs=None):
        hs = args[0] if args else kwargs["hidden_states"]
        self._x.append(hs.detach().reshape(-1, hs.shape[-1]).to(torch.bfloat16))

    def _router(self, mod, args, out):
        from . import ops
        if isinstance(out, (tuple, list)):
            idx = next(t for t in out if torch.is_tensor(t) and not t.is_floating_point())
            self._ids.append(idx.detach().reshape(-1, idx.shape[-1]).to(torch.int32))
        else:
            lg = out.detach().reshape(-1, out.shape[-1]).float()
            self._ids.append(ops.route_topk(lg, self.top_k, self.scoring, self.n_groups, self.topk_groups))

    def __enter__(self):
        self._hooks = [self.moe_module.register_forward_pre_hook(self._pre),
                       self.router.register_forward_hook(self._router)]
        return self

    def __exit__(self, *exc):
        for h in self._hooks:
            h.remove()
        self._hooks = []
        return False

    @property
    def X(self) -> torch.Tensor:
        return torch.cat(self._x, 0)

    @property
    def topk_ids(self) -> torch.Tensor:
        return torch.cat(self._ids, 0)


@torch.no_grad()
def write_back_dequantized(experts: Sequence[torch.nn.Module], results: Dict[str, tuple], group_size: int,
                           shared_experts: Sequence[torch.nn.Module] = (), prefix: str = "mlp.experts",
                           shared_prefix: str = "mlp.shared_experts",
                           proj_names: Tuple[str, str, str] = ("gate_proj", "up_proj", "down_proj")) -> None:
    """layer.weight <- (q - q0) * s in the layer's dtype for every quantised Linear, what the driver does after each
    handle's quantize() (quant.py:491-496 with dequantize_forge_full, forge/utils/engine.py:72-97), so that the rest
    of the calibration sees the quantised layer."""
    from . import ops
    mods = list(experts) + list(shared_experts)
    for i, m in enumerate(mods):
        base = f"{prefix}.{i}" if i < len(experts) else (
            shared_prefix if len(shared_experts) == 1 else f"{shared_prefix}.{i - len(experts)}")
        for proj in proj_names:
            tup = results[f"{base}.{proj}"]
            lin = getattr(m, proj)
            w = ops.dequantize(tup[0], tup[1].contiguous(), tup[2].contiguous(), group_size, torch.float32)
            if len(tup) > 3:      # SparseGPT: the pruned weights are zero, whatever their code says
                w = w * _keep_mask(tup[3], w.shape[1])
            lin.weight.copy_(w.to(lin.weight.dtype))


def _keep_mask(M: torch.Tensor, C: int) -> torch.Tensor:
    """[R, C] 0/1 from the solver's keep mask M [ceil(C/32), R] (bit t of word g: column 32 g + t is kept)."""
    Mi = M.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    bits = (Mi.unsqueeze(-1) >> torch.arange(32, device=M.device)) & 1        # [G32, R, 32]
    return bits.permute(1, 0, 2).reshape(Mi.shape[1], -1)[:, :C].to(torch.float32)


@torch.no_grad()
def forward_batches(block: torch.nn.Module, X: list, batch: int = 1, act_update: bool = False, **block_kwargs):
    """The calibration forward of the driver (forge/utils/engine.py:100-130): the cached block inputs X[i] ([1, S, H]
    each) go through the block `batch` at a time; with act_update the entries of X are replaced by the block's
    outputs — after write_back_dequantized that is the sequential activation update of quant.py:678-679."""
    dev = next(block.parameters()).device
    for s in range(0, len(X), batch):
        e = min(len(X), s + batch)
        x = torch.cat([X[i] for i in range(s, e)], dim=0).to(dev, non_blocking=True)
        out = block(x, **block_kwargs)
        out = out[0] if isinstance(out, (tuple, list)) else out
        if act_update:
            for j in range(e - s):
                X[s + j] = out[j:j + 1].to(X[s + j].device).contiguous()
    return X if act_update else None


@torch.no_grad()
def calibrate_and_quantize_block(block: torch.nn.Module, X: list, cfg: MoEQuantConfig, top_k: int,
                                 scoring: str = "softmax", n_groups: int = 1, topk_groups: int = 1, batch: int = 1,
                                 moe_attr: str = "mlp", experts_attr: str = "experts", router_attr: str = "gate",
                                 shared_attr: str = "shared_experts", update_activations: bool = True,
                                 quantizer: Optional[MoELayerQuantizer] = None, **block_kwargs) -> Dict[str, tuple]:
    """One transformer block of the driver's loop (quant.py:344-417, :489-496, :670-680) with the batched engine:
    calibration forward with two hooks -> one batched quantisation of all experts -> de-quantised weights written
    back -> (update_activations) the block is run again and X is replaced by its outputs for the next block.
    Returns the per-Linear results keyed like the reference's handles."""
    moe_mod = getattr(block, moe_attr)
    experts = list(getattr(moe_mod, experts_attr))
    shared = getattr(moe_mod, shared_attr, None)
    shared = [] if shared is None else (list(shared) if isinstance(shared, (list, torch.nn.ModuleList)) else [shared])
    with MoEBlockCapture(moe_mod, getattr(moe_mod, router_attr), top_k, scoring, n_groups, topk_groups) as cap:
        forward_batches(block, X, batch, False, **block_kwargs)
    pre = f"{moe_attr}.{experts_attr}"
    spre = f"{moe_attr}.{shared_attr}"
    results = quantize_moe_block(experts, cap.X, cap.topk_ids, cfg, shared, prefix=pre, shared_prefix=spre,
                                 quantizer=quantizer)
    write_back_dequantized(experts, results, cfg.group_size, shared, prefix=pre, shared_prefix=spre)
    if update_activations:
        forward_batches(block, X, batch, True, **block_kwargs)
    return results
