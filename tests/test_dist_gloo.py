"""Expert-parallel host logic with world_size-2 gloo ranks on the CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from forge import dist as fdist
from forge import synth


def test_shard_experts_partitions_everything():
    for E in (1, 7, 128, 257, 385):
        for world in (1, 2, 4, 8):
            spans = [fdist.shard_experts(E, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == E
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert fdist.shard_experts(384, 8, 3) == (144, 192)  # 48 experts per GPU


def test_shared_expert_goes_to_least_loaded_rank():
    ids = torch.tensor([[0, 1], [0, 1], [2, 3], [0, 2]], dtype=torch.int32)
    # experts 0-1 -> rank 0 (5 tokens), experts 2-3 -> rank 1 (3 tokens)
    assert fdist.shared_expert_owner(ids, 4, 2) == 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fail_rank):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        E, T, Hd = 5, 64, 16
        if rank == 0:
            X = synth.student_t_activations(T, Hd, seed=3)
            ids = synth.route(synth.LayerShape("t", E, 0, Hd, 8, T, 2), T, seed=3)
        else:
            X = torch.zeros((T, Hd), dtype=torch.bfloat16)
            ids = torch.zeros((T, 2), dtype=torch.int32)
        X, ids, ready = fdist.broadcast_inputs(X, ids, src=0, chunks=4)
        assert [t1 for t1, _ in ready] == [16, 32, 48, 64]
        for _, wait in ready:
            wait()
        X_ref = synth.student_t_activations(T, Hd, seed=3)
        assert torch.equal(X.view(torch.int16), X_ref.view(torch.int16))
        b, e = fdist.shard_experts(E, world, rank)
        # every rank "packs" its slice: value = expert id, so the gathered result is checkable
        local = {"packed": torch.stack([torch.full((3, 2), i, dtype=torch.int32) for i in range(b, e)]),
                 "scale": torch.arange(b, e, dtype=torch.float16)}

        def shapes(r):
            bb, ee = fdist.shard_experts(E, world, r)
            return {"packed": ((ee - bb, 3, 2), torch.int32), "scale": ((ee - bb,), torch.float16)}

        # a rank whose local work raised: every rank learns of it BEFORE the gather and raises, nobody waits forever
        ok = True
        try:
            if rank == fail_rank:
                raise RuntimeError("injected: this rank's solve failed on the host")
        except RuntimeError:
            ok = False
        if fail_rank >= 0:
            try:
                fdist.agree_ok(ok, "solve")
            except RuntimeError as exc:
                assert "rank(s) failed" in str(exc)
                assert ("this rank among them" in str(exc)) == (rank == fail_rank)
                return
            raise AssertionError("agree_ok did not raise although a rank failed")
        fdist.agree_ok(ok, "solve")
        plan = fdist.GatherPlan(shapes, "cpu")
        for _ in range(2):      # the plan's buffers are reused by every step
            got = fdist.gather_to_rank0(local, shapes, plan)
        if rank == 0:
            packed = torch.cat(got["packed"])
            assert packed.shape == (E, 3, 2)
            assert torch.equal(packed[:, 0, 0], torch.arange(E, dtype=torch.int32))
            assert torch.equal(torch.cat(got["scale"]), torch.arange(E, dtype=torch.float16))
        else:
            assert got == {}
        assert fdist.shared_expert_owner(ids, E, world) in range(world)
    finally:
        dist.destroy_process_group()


def test_broadcast_and_gather_two_ranks():
    port = _free_port()
    mp.spawn(_worker, args=(2, port, -1), nprocs=2, join=True)


def test_a_rank_that_fails_on_the_host_stops_every_rank_before_the_gather():
    port = _free_port()
    mp.spawn(_worker, args=(2, port, 1), nprocs=2, join=True)


def test_gather_plan_layout_is_padded_and_aligned():
    shapes = lambda r: {"a": ((r + 1, 3), torch.int32), "b": ((2 * r,), torch.float16)}
    plan = fdist.GatherPlan(shapes, "cpu", world=3, rank=0)
    assert plan.max_bytes % 256 == 0 and plan.max_bytes >= 3 * 3 * 4 + 4 * 2
    for r in range(3):
        lay, total = plan.layouts[r]
        assert total <= plan.max_bytes and all(off % 256 == 0 for off, *_ in lay.values())


def test_balanced_placement_covers_all_and_evens_out_load():
    from forge import dist as fdist
    import torch
    g = torch.Generator().manual_seed(0)
    E, world, T = 128, 8, 65536
    counts = (torch.rand(E, generator=g) ** 6 * 60000).long() + 20      # a few hot experts, many cold ones
    owned = fdist.balance_experts(counts.tolist(), world, n_shared=1, n_tokens=T)
    flat = sorted(e for o in owned for e in o)
    assert flat == list(range(E + 1))                                     # every expert once, the shared one included
    cost = lambda ids: sum(15000.0 + (T if e >= E else int(counts[e])) for e in ids)
    loads = [cost(o) for o in owned]
    contiguous = [cost(range(*fdist.shard_experts(E, world, r))) for r in range(world)]
    assert max(loads) <= 1.05 * (sum(loads) / world) or max(loads) == max(15000.0 + T, 15000.0 + int(counts.max()))
    assert max(loads) < max(contiguous)
    table, spans = fdist.placement_tables(owned, E)
    assert sorted(table.tolist()) == list(range(E))
    for r, (b, n) in enumerate(spans):
        routed = [e for e in owned[r] if e < E]
        assert [int(table[e]) for e in routed] == list(range(b, b + n))     # contiguous, in ascending id order
    assert fdist.balance_experts(counts.tolist(), world, 1, T) == owned   # deterministic
