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


def balance_experts(token_counts, world: int, n_shared: int = 0, n_tokens: int = 0,
                    fixed_cost_tokens: float = 15000.0) -> List[List[int]]:
    """Placement by load instead of by index: longest-processing-time-first over the cost
    `fixed_cost_tokens + routed tokens` of each expert (the factorisation, scale search and solve of an expert
    cost the same whatever its traffic; the Hessian and the expert forward grow with its tokens: with a skewed
    router a contiguous split leaves the rank that holds the popular experts far behind the others).
    Shared experts (ids n_experts .. n_experts + n_shared - 1) see every token.  Deterministic: every rank
    computes the same placement from the same counts.  Returns the expert ids of each rank, ascending."""
    counts = [int(c) for c in token_counts]
    E = len(counts)
    cost = [(fixed_cost_tokens + c, e) for e, c in enumerate(counts)]
    cost += [(fixed_cost_tokens + n_tokens, E + j) for j in range(n_shared)]
    loads = [0.0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for c, e in sorted(cost, key=lambda t: (-t[0], t[1])):
        r = min(range(world), key=lambda q: (loads[q], q))
        loads[r] += c
        owned[r].append(e)
    return [sorted(o) for o in owned]


def placement_tables(owned: List[List[int]], n_experts: int):
    """For a placement of the ROUTED experts (ids < n_experts; shared experts are not routed): a table
    old id -> new id under which every rank's routed experts are one contiguous range, and that range
    (begin, count) per rank.  Renumbering the routing table through it lets the contiguous-range kernels serve
    any placement."""
    table = torch.empty(n_experts, dtype=torch.int64)
    spans = []
    nxt = 0
    for ids in owned:
        routed = [e for e in ids if e < n_experts]
        for e in routed:
            table[e] = nxt
            nxt += 1
        spans.append((nxt - len(routed), len(routed)))
    assert nxt == n_experts, "placement must cover every routed expert exactly once"
    return table, spans


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
