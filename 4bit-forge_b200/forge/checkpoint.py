"""Checkpoint tensors of one quantised MoE block, in the layouts the reference's writers produce.

Dense W4: the compressed-tensors "pack-quantized" entries of `pack_weight` (pack_quantized.py:279-313) per Linear —
`weight_packed` int32 [R, C/8], `weight_shape` int64 [2], `weight_scale` [R, G] fp16, `weight_zero_point` [R, G]
(asymmetric only) — under the model's own parameter names, so that the reference's scales/qzeros <-> scale/zero
renaming step between quant.py:501-511 and pack_quantized.py is not needed.  Sparse 1:4: the two stacked Wpair
tensors `...mlp.experts.gate_up_proj.w13_weight` [E, G2, 2I, 2] (gate rows then up rows) and
`...mlp.experts.down_proj.w2_weight` [E, G2, H, 2] (quant.py:615-622).

Host logic over the result dict of `forge.moe.MoELayerQuantizer.quantize_experts` (device or host tensors).
"""
from __future__ import annotations

from typing import Any, Dict

import torch


def dense_block_tensors(out: Dict[str, Any], prefix: str, n_routed: int, symmetric: bool,
                        shared_name: str = "shared_experts") -> Dict[str, torch.Tensor]:
    """out: result of quantize_experts with cfg.pack = True (dense).  Experts [0, n_routed) are the routed ones,
    the rest shared experts.  prefix e.g. "model.layers.3." (with the trailing dot, like quant.py's `prefix`)."""
    tensors: Dict[str, torch.Tensor] = {}
    n = out["gate"]["weight_packed"].shape[0]
    for fam, proj in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")):
        r = out[fam]
        R, CP = r["weight_packed"].shape[1:]
        shape = torch.tensor([R, r["qweight"].shape[2]], dtype=torch.int64)
        for i in range(n):
            if i < n_routed:
                base = f"{prefix}mlp.experts.{i}.{proj}"
            else:
                j = i - n_routed
                base = f"{prefix}mlp.{shared_name}.{proj}" if n - n_routed == 1 else f"{prefix}mlp.{shared_name}.{j}.{proj}"
            tensors[f"{base}.weight_packed"] = r["weight_packed"][i].contiguous()
            tensors[f"{base}.weight_shape"] = shape.clone()
            tensors[f"{base}.weight_scale"] = r["weight_scale"][i].to(torch.float16).contiguous()
            if not symmetric:
                tensors[f"{base}.weight_zero_point"] = r["qzeros"][i].to(torch.uint8).contiguous()
    return tensors


def sparse_block_tensors(out: Dict[str, Any], prefix: str) -> Dict[str, torch.Tensor]:
    """out: result of quantize_experts with algorithm = "sparsegptq" and cfg.pack = True: Wpair words
    [E, G2, R, 2] per matrix.  Gate and up are stacked along R like the driver does (quant.py:464, 615-622)."""
    w13 = torch.cat([out["gate"]["wpair"], out["up"]["wpair"]], dim=2).contiguous()
    w2 = out["down"]["wpair"].contiguous()
    return {f"{prefix}mlp.experts.gate_up_proj.w13_weight": w13, f"{prefix}mlp.experts.down_proj.w2_weight": w2}


def quantization_config(bits: int, group_size: int, symmetric: bool, only_routed_experts: bool = True) -> Dict[str, Any]:
    """The `quantization_config` entry of config.json for the dense format (pack_quantized.py:316-346); `symmetric`
    states what was actually done (the reference writes True whatever --sym was)."""
    ignore = ["lm_head"]
    if only_routed_experts:
        ignore += ["re:.*self_attn.*", "re:.*shared_experts.*", "re:.*mlp\\.(gate|up|gate_up|down)_proj.*"]
    return {
        "config_groups": {"group_0": {
            "input_activations": None, "output_activations": None, "targets": ["Linear"],
            "weights": {"actorder": None, "block_structure": None, "dynamic": False, "group_size": int(group_size),
                        "num_bits": int(bits), "observer": "minmax", "observer_kwargs": {}, "strategy": "group",
                        "symmetric": bool(symmetric), "type": "int"}}},
        "format": "pack-quantized", "ignore": ignore, "kv_cache_scheme": None,
        "quant_method": "compressed-tensors", "quantization_status": "compressed",
    }


def write_block_shard(path: str, tensors: Dict[str, torch.Tensor]) -> Dict[str, str]:
    """Write one block's tensors as a safetensors shard; returns the weight_map entries {key: file name}."""
    import os
    from safetensors.torch import save_file
    save_file({k: v.detach().cpu().contiguous() for k, v in tensors.items()}, path)
    name = os.path.basename(path)
    return {k: name for k in tensors}
