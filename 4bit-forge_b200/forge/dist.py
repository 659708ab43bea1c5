"""Expert-parallel plumbing: one process per GPU, experts sharded across ranks.

The path has exactly one exchange step in and one out: rank 0 broadcasts the layer input and the routing
table, every rank accumulates and solves its own expert slice with no further communication (experts are
independent once routed), and the packed weights are gathered on rank 0 for the checkpoint.  The reference
is single-GPU (quant.py:116 `rank = 0 #TODO multigpu`), so this layer is new.  Works over NCCL (GPU) and
gloo (CPU tests of the host logic).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist


def shard_experts(n_experts: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous split; the first (n_experts % world) ranks take one extra expert."""
    base, rem = divmod(n_experts, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shared_expert_owner(topk_ids: torch.Tensor, n_experts: int, world: int) -> int:
    """Rank with the fewest routed tokens (ties -> lowest rank); every rank computes the same answer."""
    counts = torch.bincount(topk_ids.reshape(-1).long(), minlength=n_experts)
    loads = []
    for r in range(world):
        b, e = shard_experts(n_experts, world, r)
        loads.append(int(counts[b:e].sum()))
    return min(range(world), key=lambda r: (loads[r], r))


def broadcast_inputs(X: torch.Tensor, topk_ids: torch.Tensor, src: int = 0, chunks: int = 1):
    """Broadcast the calibration input [T,H] and the routing table [T,k] from `src` (in place)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return X, topk_ids
    dist.broadcast(topk_ids, src=src)
    if chunks <= 1:
        dist.broadcast(X, src=src)
    else:
        for part in X.chunk(chunks, dim=0):
            dist.broadcast(part, src=src)
    return X, topk_ids


def gather_to_rank0(local: Dict[str, torch.Tensor], shapes_of_rank) -> Dict[str, List[torch.Tensor]]:
    """Gather same-keyed tensors of every rank on rank 0 with point-to-point copies (slices may differ in
    size, which a plain gather collective does not allow).  `shapes_of_rank(r)` -> {key: (shape, dtype)}.
    Returns {key: [tensor of rank 0, rank 1, ...]} on rank 0 and {} elsewhere."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return {k: [v] for k, v in local.items()}
    world, rank = dist.get_world_size(), dist.get_rank()
    keys = sorted(local)
    if rank == 0:
        out = {k: [local[k]] for k in keys}
        reqs = []
        for r in range(1, world):
            meta = shapes_of_rank(r)
            for k in keys:
                shape, dtype = meta[k]
                buf = torch.empty(shape, dtype=dtype, device=local[k].device)
                out[k].append(buf)
                if buf.numel():
                    reqs.append(dist.irecv(_as_bytes(buf), src=r))
        for q in reqs:
            q.wait()
        return out
    reqs = [dist.isend(_as_bytes(local[k].contiguous()), dst=0) for k in keys if local[k].numel()]
    for q in reqs:
        q.wait()
    return {}


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8) if t.dtype not in (torch.uint8,) else t
