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


# ---------------------------------------------------------------------------------------------------------------
# Writers.  The reference driver saves, per quantised Linear, a `quantized_weight.pt` dict (quant.py:498-511) that
# pack_quantized.py later repacks, and, on the sparse path, one safetensors shard per transformer block plus an
# index that is rewritten after every block (forge/utils/io.py:630-672, quant.py:615-666); a rerun skips the blocks
# whose shard already exists.  The same three pieces follow, fed from the batched result instead of one handle at a
# time.
# ---------------------------------------------------------------------------------------------------------------
def linear_result_dict(qweight, scales, qzeros, group_size: int, bits: int, shape) -> Dict[str, Any]:
    """The per-Linear dict of the reference driver, same keys, dtypes and meaning (quant.py:498-511): `qweight` int8
    (codes before the nibble shift), `scales` fp32, `qzeros` int32, flat per (row, group) like GPTQ.quantize()."""
    return {"qweight": qweight.to(torch.int8).cpu(), "scales": scales.reshape(-1).to(torch.float32).cpu(),
            "qzeros": qzeros.reshape(-1).to(torch.int32).cpu(), "group_size": int(group_size), "bits": int(bits),
            "shape": tuple(int(v) for v in shape)}


def write_linear_results(save_dir: str, block_id: int, results: Dict[str, tuple], group_size: int, bits: int,
                         skip_existing: bool = True):
    """results: {"<layer name>": (qweight [R,C], scales, qzeros[, M])} as forge.capture.quantize_moe_block returns
    them (entries ending in ".info" are ignored).  Writes save_dir/block.<id>/<layer name>/quantized_weight.pt, the
    layout pack_quantized.py reads.  Returns the paths written; existing files are kept when skip_existing."""
    import os
    written = []
    for name, tup in results.items():
        if name.endswith(".info"):
            continue
        out_dir = os.path.join(save_dir, f"block.{block_id}", name)
        path = os.path.join(out_dir, "quantized_weight.pt")
        if skip_existing and os.path.exists(path):
            continue
        os.makedirs(out_dir, exist_ok=True)
        q, s, z = tup[0], tup[1], tup[2]
        tmp = path + ".tmp"
        torch.save(linear_result_dict(q, s, z, group_size, bits, q.shape), tmp)
        os.replace(tmp, path)       # a file that exists is complete
        written.append(path)
    return written


def write_run_metadata(save_dir: str, bits: int, group_size: int, quantize_only_experts: bool) -> str:
    """metadata.pt at the root of the save directory (quant.py:690-698)."""
    import os
    os.makedirs(save_dir, exist_ok=True)
    path = os.path.join(save_dir, "metadata.pt")
    torch.save({"bits": int(bits), "group_size": int(group_size), "quantize_only_experts": bool(quantize_only_experts)},
               path)
    return path


class IncrementalIndexWriter:
    """model.safetensors.index.json of the output checkpoint, rewritten after every block
    (forge/utils/io.py:630-672).  Starts from the base checkpoint's index; `write_block_shard` writes one shard with
    a block's tensors, points their keys at it, removes the keys the block no longer has (the dense expert weights
    the packed tensors replace; shared experts are never dropped) and flushes the index.  Shard and index are
    written to a temporary name and renamed, so a shard that exists is complete and `block_done` can be trusted by
    a rerun (resume = skip the blocks whose shard exists)."""

    def __init__(self, base_model_dir: str, out_dir: str, base_index: Dict[str, Any]):
        from pathlib import Path
        self.base_model_dir = Path(base_model_dir)
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.index_path = self.out_dir / "model.safetensors.index.json"
        self.metadata = dict(base_index.get("metadata", {}))
        self.weight_map = dict(base_index["weight_map"])
        if self.index_path.exists():        # a rerun continues from the index the earlier run left
            import json
            with self.index_path.open() as f:
                prev = json.load(f)
            self.weight_map.update({k: v for k, v in prev.get("weight_map", {}).items()
                                    if (self.out_dir / v).exists()})
            for k in [k for k in self.weight_map if k not in prev.get("weight_map", {})]:
                # keys an earlier run dropped stay dropped if the block that dropped them is on disk
                blk = _block_of_key(k)
                if blk is not None and self.block_done(blk):
                    del self.weight_map[k]

    @staticmethod
    def shard_name(block_id: int) -> str:
        return f"block_{block_id:03d}.safetensors"

    def block_done(self, block_id: int) -> bool:
        return (self.out_dir / self.shard_name(block_id)).exists()

    def flush(self) -> None:
        import json
        import os
        tmp = str(self.index_path) + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"metadata": self.metadata, "weight_map": self.weight_map}, f, indent=2, sort_keys=True)
        os.replace(tmp, self.index_path)

    def write_block_shard(self, block_id: int, prefix: str, tensors: Dict[str, torch.Tensor], shard_name: str = None,
                          drop_keys=()) -> str:
        import os
        from safetensors.torch import save_file
        shard_name = shard_name or self.shard_name(block_id)
        path = self.out_dir / shard_name
        tmp = str(path) + ".tmp"
        save_file({k: v.detach().cpu().contiguous() for k, v in tensors.items()}, tmp)
        os.replace(tmp, path)
        for k in tensors:
            self.weight_map[k] = shard_name
        for k in drop_keys:
            if k in self.weight_map and "shared_experts" not in k and k not in tensors:
                del self.weight_map[k]
        self.flush()
        return str(path)


def _block_of_key(key: str):
    import re
    m = re.search(r"\.layers\.(\d+)\.", key)
    return int(m.group(1)) if m else None


def routed_expert_weight_keys(weight_map, prefix: str):
    """Keys of the block's dense routed-expert tensors, which the packed tensors replace (quant.py:640-647)."""
    import re
    pat = re.compile(rf"^{re.escape(prefix)}mlp\.experts\.\d+\.(gate_proj|up_proj|down_proj)\."
                     r"(weight|weight_scale_inv|weight_inv_scale|bias|bias_scale|bias_scale_inv|bias_inv_scale)$")
    return {k for k in weight_map if pat.match(k)}


def reorder_gathered(gathered: Dict[str, list], owned) -> Dict[str, torch.Tensor]:
    """Rank 0's view after the gather ({key: [tensor of rank 0, rank 1, ...]}, each holding that rank's experts in
    the order of owned[r]) -> {key: one tensor in global expert order}."""
    order = [e for ids in owned for e in ids]
    inv = torch.empty(len(order), dtype=torch.int64)
    inv[torch.tensor(order)] = torch.arange(len(order))
    return {k: torch.cat([p.cpu() for p in parts], 0)[inv] for k, parts in gathered.items()}


def write_moe_block(writer: IncrementalIndexWriter, block_id: int, prefix: str, out: Dict[str, Any], n_routed: int,
                    symmetric: bool, sparse: bool, skip_existing: bool = True):
    """One block of the output checkpoint from a quantize_experts result (or the re-ordered gather of all ranks on
    rank 0, as {"gate": {...}, "up": {...}, "down": {...}}).  Returns the shard path, or None when the shard was
    already there (resume)."""
    if skip_existing and writer.block_done(block_id):
        return None
    tensors = sparse_block_tensors(out, prefix) if sparse else dense_block_tensors(out, prefix, n_routed, symmetric)
    drop = routed_expert_weight_keys(writer.weight_map, prefix)
    return writer.write_block_shard(block_id, prefix, tensors, drop_keys=drop)
