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
    """Broadcast the calibration input [T,H] and the routing table [T,k] from `src` (in place).

    With chunks > 1 the rows of X travel as `chunks` separate asynchronous broadcasts and the call returns
    (X, topk_ids, ready) at once: ready = [(row_end, wait)], one entry per chunk in row order, where wait() makes
    the CURRENT CUDA stream wait for that chunk (it blocks the host only on gloo).  The caller hands `ready` to
    MoELayerQuantizer.quantize_experts(x_chunks=...), which accumulates the Hessians of chunk i while chunk i+1 is
    still in flight.  With chunks <= 1 everything is broadcast before returning and ready is None."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return (X, topk_ids) if chunks <= 1 else (X, topk_ids, None)
    dist.broadcast(topk_ids, src=src)
    if chunks <= 1:
        dist.broadcast(X, src=src)
        return X, topk_ids
    ready = []
    T = X.shape[0]
    bounds = [T * (i + 1) // chunks for i in range(chunks)]
    t0 = 0
    for t1 in bounds:
        if t1 > t0:
            work = dist.broadcast(X[t0:t1], src=src, async_op=True)
            ready.append((t1, work.wait))
        t0 = t1
    return X, topk_ids, ready


def agree_ok(ok: bool, what: str = "step") -> None:
    """Every rank reports whether its part of the step succeeded; if any rank failed, ALL ranks raise.  Call it
    (from a try / except around the local work) before a collective that would otherwise wait for a rank that has
    already given up.  A rank that died without reaching this call ends the all-reduce with the process group's
    timeout error, which is finite, instead of hanging the others."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        if not ok:
            raise RuntimeError(f"forge.dist: the local {what} failed")
        return
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    flag = torch.tensor([0 if ok else 1], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.SUM)
    bad = int(flag.item())
    if bad:
        raise RuntimeError(f"forge.dist: {bad} rank(s) failed their {what}"
                           + ("" if ok else " (this rank among them)") + "; nothing was gathered")


class GatherPlan:
    """One exchange per step for the packed results: every rank serialises its tensors into ONE byte buffer (padded
    to the largest rank's size) and a single gather collective delivers all of them to rank 0.  Slices differ in
    size between ranks (experts are placed by load), which is why the buffers are padded; layouts are computed
    once from `shapes_of_rank(r) -> {key: (shape, dtype)}`, and the send / receive buffers are allocated once and
    reused by every step."""

    ALIGN = 256

    def __init__(self, shapes_of_rank, device, world=None, rank=None):
        live = dist.is_available() and dist.is_initialized()
        self.world = world if world is not None else (dist.get_world_size() if live else 1)
        self.rank = rank if rank is not None else (dist.get_rank() if live else 0)
        self.device = torch.device(device)
        self.layouts = []
        for r in range(self.world):
            meta = shapes_of_rank(r)
            lay, off = {}, 0
            for k in sorted(meta):
                shape, dtype = meta[k]
                nbytes = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
                lay[k] = (off, nbytes, tuple(shape), dtype)
                off += (nbytes + self.ALIGN - 1) // self.ALIGN * self.ALIGN
            self.layouts.append((lay, off))
        self.max_bytes = max(max(off for _, off in self.layouts), self.ALIGN)
        self.send = torch.empty(self.max_bytes, dtype=torch.uint8, device=self.device)
        self.recv = None
        if self.rank == 0 and self.world > 1:
            self.recv = [torch.empty(self.max_bytes, dtype=torch.uint8, device=self.device) for _ in range(self.world)]

    def _views(self, buf, r):
        lay, _ = self.layouts[r]
        return {k: buf[off:off + nbytes].view(dtype).view(shape) for k, (off, nbytes, shape, dtype) in lay.items()}

    def pack(self, local: Dict[str, torch.Tensor]) -> None:
        lay, _ = self.layouts[self.rank]
        assert sorted(local) == sorted(lay), "result keys differ from the plan"
        for k, (off, nbytes, shape, dtype) in lay.items():
            t = local[k]
            assert tuple(t.shape) == shape and t.dtype == dtype, (k, tuple(t.shape), shape, t.dtype, dtype)
            if nbytes:
                self.send[off:off + nbytes].view(dtype).view(shape).copy_(t)

    def run(self, local: Dict[str, torch.Tensor]) -> Dict[str, List[torch.Tensor]]:
        """Returns {key: [tensor of rank 0, rank 1, ...]} on rank 0 (views into the plan's buffers, valid until the
        next run) and {} elsewhere."""
        if self.world == 1:
            return {k: [v] for k, v in local.items()}
        self.pack(local)
        dist.gather(self.send, gather_list=self.recv if self.rank == 0 else None, dst=0)
        if self.rank != 0:
            return {}
        per_rank = [self._views(self.recv[r], r) for r in range(self.world)]
        return {k: [per_rank[r][k] for r in range(self.world)] for k in per_rank[0]}


def gather_to_rank0(local: Dict[str, torch.Tensor], shapes_of_rank, plan: "GatherPlan" = None):
    """Gather same-keyed tensors of every rank on rank 0 in one collective (see GatherPlan; pass a plan built once
    outside the step to reuse its buffers).  Returns {key: [tensor of rank 0, rank 1, ...]} on rank 0, {} elsewhere."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return {k: [v] for k, v in local.items()}
    if plan is None:
        plan = GatherPlan(shapes_of_rank, next(iter(local.values())).device)
    return plan.run(local)
