"""Benchmark: experts GPTQ'd per second for one MoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl ours|reference]

A step is one full pass of the solver path over one synthetic MoE layer: (broadcast) -> routing lists ->
per-expert Hessians of the layer input and of the down-projection input (incl. the expert forward that
produces it) -> scan / permutation / damping -> batched Cholesky -> scale grid -> fused column solver ->
packing -> (gather).  Experts are sharded over the ranks; the layer is fixed, so scaling is strong.
Rank 0 prints one JSON line.  `--impl reference` times the CPU restatement of the reference path
(oracle/) on the host cores over a bounded sample of the same workload.
"""
import argparse
import gc
import json
import os

# the layer is processed in passes of a few tens of GB whose buffers come and go on two streams: growable segments
# keep the caching allocator from stranding that memory in fixed-size blocks
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (os.path.join(ROOT, "4bit-forge_b200"), os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

METRIC = "experts_gptq_per_sec_per_moe_layer"
UNIT = "experts/s"

# DRAM bytes of forge_gptq_solve_batched per expert (gate + up + down launches), from ncu captures of small cuts of
# the same matrix shapes (the full layers are too large to capture; traffic is per expert, so it scales with the
# expert count).  The summaries and their commands are under profiles/.
SOLVER_TRAFFIC_PER_EXPERT = {"deepseek_v3": 4.97e9}    # 84.5 GB over the 3 launches of a 17-expert cut

# quantisation recipe per benchmark configuration
RECIPES = {
    "qwen3_30b_a3b": dict(symmetric=False, quantization_scale="mse", quantization_order="default", algorithm="gptq"),
    "deepseek_v3": dict(symmetric=True, quantization_scale="absmax", quantization_order="activation", algorithm="gptq"),
    "minimax_m2": dict(symmetric=True, quantization_scale="absmax", quantization_order="default", algorithm="sparsegptq"),
    "kimi_k2": dict(symmetric=True, quantization_scale="absmax", quantization_order="default", algorithm="gptq"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="deepseek_v3", choices=sorted(RECIPES))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override the calibration token count (smaller runs)")
    ap.add_argument("--experts", type=int, default=0, help="override the routed expert count (smaller runs)")
    ap.add_argument("--expert-chunk", type=int, default=0, help="experts per pass (0: chosen from the free memory)")
    ap.add_argument("--bcast-chunks", type=int, default=2,
                    help="row chunks of the X broadcast (N > 1): the Hessian of chunk i overlaps the transfer of chunk i+1")
    ap.add_argument("--placement", default="lpt", choices=["lpt", "contiguous"],
                    help="experts to ranks: by load (routed tokens, longest first) or contiguous index ranges")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def layer_shape(args):
    from forge import synth
    import dataclasses
    shape = synth.CONFIGS[args.config]
    if args.tokens:
        shape = dataclasses.replace(shape, tokens=args.tokens)
    if args.experts:
        shape = dataclasses.replace(shape, n_experts=args.experts)
    return shape


def workload_name(shape, recipe):
    return (f"{shape.name}: {shape.n_experts}+{shape.n_shared} experts, hidden {shape.hidden}, inter {shape.inter}, "
            f"{shape.tokens} tokens top-{shape.top_k}, W4 g128 "
            f"{'sym' if recipe['symmetric'] else 'asym'} {recipe['quantization_scale']} {recipe['algorithm']}"
            f"{' act-order' if recipe['quantization_order'] == 'activation' else ''}")


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(shape, recipe, n_tokens_list, seed=0):
    """Oracle (reference restatement) on the host cores for the listed per-expert token counts; full matrix
    shapes, gate/up share one Hessian (the reference's --owner_gptq_handles mode) but are factorised per
    handle as the reference does.  Returns seconds."""
    import ref_port as O
    from forge import synth
    torch.set_num_threads(os.cpu_count() or 1)
    kw = dict(bits=4, group_size=128, rel_damp=0.01, **recipe)
    t_total = 0.0
    for i, n in enumerate(n_tokens_list):
        Wg, Wu, Wd = synth.expert_weights(shape, [i], seed=seed + 1)
        x = synth.student_t_activations(max(n, 1), shape.hidden, seed=seed + 2 + i)[:n]
        t0 = time.perf_counter()
        hg = O.OracleGPTQ(Wg[0], **kw)
        hg.update(x)
        hu = O.OracleGPTQ(Wu[0], **kw)
        hu.H, hu.num_samples = hg.H.clone() if hg.H is not None else None, hg.num_samples
        act = O.swiglu_down_input(x, Wg[0], Wu[0])
        hd = O.OracleGPTQ(Wd[0], **kw)
        hd.update(act)
        for h in (hg, hu, hd):
            out = h.quantize()
            if recipe["algorithm"] == "sparsegptq":
                G32 = h.W.shape[1] // 32
                O.pack_sparsegptq14_to_u64x2(out[0], out[3], out[1].view(-1, h.G).repeat_interleave(4, 1)[:, :G32].T.contiguous())
            else:
                O.pack_int4(out[0], out[2].view(-1, h.G), 128)
        t_total += time.perf_counter() - t0
    return t_total


def reference_gpu_sample(shape, recipe, n_tokens_list, dev, seed=0):
    """The reference's algorithm with the reference's OWN CUDA kernels (oracle/_ref, compiled for sm_100a from the
    reference checkout) and torch for its Python half, on this GPU: one handle per Linear, one update and one
    quantize() each, as its driver does.  Returns (seconds, launches are not ours) or None when the library was not
    built.  A same-device baseline beside the CPU one; none of this engine's kernels run here."""
    import ref_build
    import ref_port as O
    from forge import synth
    ref = ref_build.load_built()
    if ref is None:
        return None
    kw = dict(bits=4, group_size=128, rel_damp=0.01, kernels=ref, **recipe)
    work = []
    for i, n in enumerate(n_tokens_list):
        Wg, Wu, Wd = synth.expert_weights(shape, [i], seed=seed + 1, device=dev)
        x = synth.student_t_activations(max(n, 1), shape.hidden, seed=seed + 2 + i, device=dev)[:n]
        work.append((Wg[0], Wu[0], Wd[0], x))

    def one_pass():
        for Wg, Wu, Wd, x in work:
            hg, hu = O.OracleGPTQ(Wg, **kw), O.OracleGPTQ(Wu, **kw)
            hg.update(x)
            hu.update(x)
            hd = O.OracleGPTQ(Wd, **kw)
            hd.update(O.swiglu_down_input(x, Wg, Wu))
            for h in (hg, hu, hd):
                h.quantize()

    one_pass()                                  # warm-up (cuSOLVER handles, kernel load)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    one_pass()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3


def fixed_cost_in_tokens(Hd, I, recipe):
    """What an expert costs whatever its traffic (factorisation, scale search, column solve), in units of one routed
    token's cost (its share of the two Hessians and of the expert forward): the exchange rate of the placement.  From
    the rates the kernels reach on one GPU: solver and factorisation ~1.1e14 algorithmic flop/s (R C^2 per matrix,
    C^3/3 per Hessian; the triangular inverse of the SparseGPT path doubles the latter), the MSE search ~5.5e12
    element-candidates/s, Hessian and expert forward ~1e15 flop/s.  19 600 tokens at hidden 7168 / inter 2048, 12 600
    at 2048 / 768 with the MSE search."""
    solve = (2.0 * I * Hd * Hd + Hd * I * I) / 1.1e14
    factor = (Hd ** 3 + I ** 3) / 3.0 / 1.1e14 * (2.0 if recipe["algorithm"] == "sparsegptq" else 1.0)
    search = (300.0 * Hd * I / 5.5e12) if recipe["quantization_scale"] == "mse" else 0.0
    per_token = 2.0 * (Hd * Hd + I * I) / 1.0e15 + 4.0 * Hd * I / 1.0e15
    return (solve + factor + search) / per_token


def run_reference(args, rank, world):
    if rank != 0:
        return
    shape = layer_shape(args)
    recipe = RECIPES[args.config]
    mean_tokens = max(1, shape.tokens * shape.top_k // shape.n_experts)
    import ref_port as O
    O.lib()
    for _ in range(args.warmup):
        cpu_sample(shape, recipe, [mean_tokens])
    t = 0.0
    for _ in range(args.steps):
        t += cpu_sample(shape, recipe, [mean_tokens])
    value = args.steps / t
    cores = os.cpu_count() or 1
    sample = f"per step: 1 expert (3 matrices, full shape) with the mean routed token count {mean_tokens}; extrapolated to experts/s"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(shape, recipe), "inputs": "larger than L2 / CPU resident"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
class PhaseTimer:
    """Wraps forge._abi.call with CUDA events to attribute device time to each C-ABI entry point."""

    def __init__(self):
        self.records = []
        self.enabled = False

    def install(self):
        from forge import _abi, ops
        orig = _abi.call
        timer = self

        def timed_call(name, *a):
            if not timer.enabled:
                return orig(name, *a)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = orig(name, *a)
            e1.record()
            timer.records.append((name, e0, e1))
            return rc
        _abi.call = timed_call
        ops.call = timed_call

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, e0, e1 in self.records:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out


def pick_expert_chunk(n_local, Hd, I, free_bytes, sparse):
    """Experts factorised / solved per pass so that the per-pass working set fits the free memory: three fp32 [Hd,Hd]
    matrices (Hessian, its factor copy, the factor's tensor-core operand pieces) plus the solver's work buffers of
    a weight batch (fp32 transposed weights + codes)."""
    per_expert = 3 * Hd * Hd * 4 + I * Hd * 8 + (1 << 20)
    fit = max(1, int(0.5 * free_bytes // per_expert))
    if fit >= n_local:
        return 0
    passes = -(-n_local // fit)
    return -(-n_local // passes)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from forge import _abi, synth, moe, ops, dist as fdist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    _abi.load_library()
    shape = layer_shape(args)
    recipe = RECIPES[args.config]
    E = shape.n_experts
    e0, e1 = fdist.shard_experts(E, world, rank)
    route_args = (shape.top_k, shape.router, shape.n_groups, shape.topk_groups)

    # ---- inputs resident in HBM: X and the router logits on rank 0, each rank's own expert weights
    T, Hd, I = shape.tokens, shape.hidden, shape.inter
    if rank == 0:
        X = synth.student_t_activations(T, Hd, seed=11, device=dev)
        logits = synth.router_logits(shape, T, seed=11, device=dev)
    else:
        X = torch.empty((T, Hd), dtype=torch.bfloat16, device=dev)
        logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    if world > 1:
        dist.broadcast(logits, src=0)  # only to decide the placement; the timed step broadcasts again
    # placement is decided from the routing statistics before the timed region (like the shared expert's owner)
    ids_host = ops.route_topk(logits, *route_args).cpu()
    remap = None
    if args.placement == "lpt" and world > 1:
        counts_all = torch.bincount(ids_host.reshape(-1).long(), minlength=E)
        owned = fdist.balance_experts(counts_all.tolist(), world, shape.n_shared, T,
                                      fixed_cost_tokens=fixed_cost_in_tokens(Hd, I, recipe))
        table, spans = fdist.placement_tables(owned, E)
        remap = table.to(dev)
        my_ids = owned[rank]
        e0, n_r = spans[rank]
        e1 = e0 + n_r
        n_tail = len(my_ids) - n_r
        n_local_of = [len(o) for o in owned]
    else:
        owner = fdist.shared_expert_owner(ids_host, E, world) if shape.n_shared else -1
        n_tail = shape.n_shared if rank == owner else 0
        my_ids = list(range(e0, e1)) + [E + j for j in range(n_tail)]
        n_local_of = []
        for r in range(world):
            b, e = fdist.shard_experts(E, world, r)
            n_local_of.append((e - b) + (shape.n_shared if r == owner else 0))
    n_loc = len(my_ids)
    Wg, Wu, Wd = synth.expert_weights(shape, my_ids, seed=12, device=dev)
    fp8 = None
    if shape.fp8_weights:
        # the checkpoint form: e4m3 weights [n,R,C] + fp32 block scales [n,R/128,C/128]; de-quantised inside the step
        enc = [[synth.fp8_block_encode(w) for w in Wm] for Wm in (Wg, Wu, Wd)]
        fp8 = [(torch.stack([q8 for q8, _ in e_]), torch.stack([sv for _, sv in e_]).float().contiguous()) for e_ in enc]
        del enc
    sparse = recipe["algorithm"] == "sparsegptq"
    torch.cuda.empty_cache()
    chunk = args.expert_chunk or pick_expert_chunk(n_loc, Hd, I, torch.cuda.mem_get_info()[0], sparse)
    cfg = moe.MoEQuantConfig(bits=4, group_size=128, rel_damp=0.01, expert_chunk=chunk, keep_codes=False, **recipe)
    qz = moe.MoELayerQuantizer(cfg)

    def shapes_of_rank(r):
        n = n_local_of[r]
        meta = {}
        for nm, (R, C) in (("gate", (I, Hd)), ("up", (I, Hd)), ("down", (Hd, I))):
            if sparse:
                meta[f"{nm}.wpair"] = ((n, (C // 32 + 1) // 2, R, 2), torch.int64)
            else:
                meta[f"{nm}.weight_packed"] = ((n, R, C // 8), torch.int32)
                meta[f"{nm}.weight_scale"] = ((n, R, C // 128), torch.float16)
                if not cfg.symmetric:
                    meta[f"{nm}.weight_zero_point"] = ((n, R, C // 128), torch.uint8)
        return meta

    plan = fdist.GatherPlan(shapes_of_rank, dev) if world > 1 else None   # buffers allocated once, outside the step

    def local_results(out):
        local = {}
        for nm in ("gate", "up", "down"):
            r = out[nm]
            if sparse:
                local[f"{nm}.wpair"] = r["wpair"]
            else:
                local[f"{nm}.weight_packed"] = r["weight_packed"]
                local[f"{nm}.weight_scale"] = r["weight_scale"]
                if not cfg.symmetric:
                    local[f"{nm}.weight_zero_point"] = r["qzeros"].to(torch.uint8)
        return local

    def route_local(lg):
        ids = ops.route_topk(lg, *route_args)
        if remap is not None:
            ids = remap[ids.long()].to(torch.int32)      # renumber: this rank's experts become one contiguous range
        return ids

    def dequant_weights():
        if fp8 is not None:
            for Wm, (q8, sinv) in zip((Wg, Wu, Wd), fp8):
                n, R, C = q8.shape
                ops.fp8_block_dequant(q8.view(n * R, C), sinv.view(-1, sinv.shape[-1]), out=Wm.view(n * R, C))

    def step(quantizer=None):
        """One layer: broadcast -> route -> (fp8 -> bf16) -> Hessians / factor / search / solve / pack -> gather."""
        x_chunks = None
        if world > 1:
            dist.broadcast(logits, src=0)
            ids = route_local(logits)
            x_chunks = _bcast_x()
        else:
            ids = route_local(logits)
        dequant_weights()
        ok, out, err = True, None, None
        try:
            out = (quantizer or qz).quantize_experts(X, ids, Wg, Wu, Wd, e_begin=e0, dense_tail=n_tail,
                                                     x_chunks=x_chunks)
        except RuntimeError as exc:     # a rank that failed says so before the gather; nobody waits for it
            ok, err = False, exc
        if world > 1:
            fdist.agree_ok(ok, "solve")
        elif not ok:
            raise err
        gathered = plan.run(local_results(out)) if world > 1 else None
        return out, gathered

    def _bcast_x():
        ready = []
        t0 = 0
        for i in range(args.bcast_chunks):
            t1 = T * (i + 1) // args.bcast_chunks
            if t1 > t0:
                ready.append((t1, dist.broadcast(X[t0:t1], src=0, async_op=True).wait))
            t0 = t1
        return ready

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(vals):
        if world > 1:
            t = torch.tensor(vals, dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return [float(v) for v in t.tolist()]
        return list(vals)

    def timed(fn, steps):
        """Total device time of `steps` calls (barrier + synchronize on both sides, max over ranks) and the per-step
        device times (events between the steps, max over ranks per step)."""
        # the steps are queued from Python: a collection of the cyclic garbage collector in the middle of a step
        # (hundreds of ms with this many live tensors) would leave the GPU waiting for the host
        gc.collect()
        gc.disable()
        barrier()
        torch.cuda.synchronize()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        evs[0].record()
        for i in range(steps):
            fn()
            evs[i + 1].record()
        torch.cuda.synchronize()
        barrier()
        gc.enable()
        total = max_over_ranks([evs[0].elapsed_time(evs[-1])])[0]
        per_step = max_over_ranks([evs[i].elapsed_time(evs[i + 1]) for i in range(steps)])
        return total, per_step

    def mem(tag):
        if os.environ.get("BENCH_DEBUG_MEM"):
            print(f"[mem] {tag}: allocated {torch.cuda.memory_allocated() / 2**30:.1f} GiB, peak "
                  f"{torch.cuda.max_memory_allocated() / 2**30:.1f} GiB, reserved "
                  f"{torch.cuda.memory_reserved() / 2**30:.1f} GiB, chunk {chunk}", file=sys.stderr, flush=True)

    mem("inputs ready")
    # ---- device-resident timing
    for _ in range(max(args.warmup, 1)):
        out, _ = step()     # every step checks the status word (quantize_experts raises on a non-zero status)
    torch.cuda.synchronize()
    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
    n0 = _abi.query("forge_launch_count")
    ms, per_step = timed(step, args.steps)
    launches = _abi.query("forge_launch_count") - n0
    clk = clocks.stop() if rank == 0 else None
    n_total = E + shape.n_shared
    value = n_total * args.steps / (ms / 1e3)

    # ---- per-entry-point device time of one more step (rank 0's slice) and the roofline of the top kernel
    # (streams not overlapped in this one step, so that every entry point's events bracket its own kernels only)
    qz_serial = moe.MoELayerQuantizer(moe.MoEQuantConfig(**{**cfg.__dict__, "overlap_streams": False}))
    qz_serial._arena = qz._arena        # the same work buffers: a second set would not fit beside the first
    pt = PhaseTimer()
    pt.install()
    pt.enabled = True
    out, _ = step(qz_serial)
    phases = pt.summary()
    pt.enabled = False
    counts = out["counts"].cpu().double()
    del out
    # every rank's own kernel time in that step (sum over its entry points): how even the placement is
    phase_sums = [float(sum(phases.values()))]
    if world > 1:
        t = torch.zeros(world, dtype=torch.float64, device=dev)
        t[rank] = phase_sums[0]
        dist.all_reduce(t)
        phase_sums = [round(float(v), 3) for v in t.tolist()]
    barrier()
    mem("after the device-resident phases")

    # ---- end to end: host buffers in, packed results out (pinned memory, copies inside the timed region).
    # The call a user makes: MoELayerQuantizer.quantize_experts_host — weights (fp8 + block scales where the
    # checkpoint is fp8) and activations come from pinned host memory, packed results land in pinned host memory;
    # its copies run on their own streams beside the kernels.
    e2e = None
    if not args.no_e2e:
        hX = X.cpu().pin_memory() if rank == 0 else None
        hlog = logits.cpu().pin_memory() if rank == 0 else None
        if fp8 is not None:
            hW = [q8.cpu().pin_memory() for q8, _ in fp8]
            hS = [sv.cpu().pin_memory() for _, sv in fp8]
        else:
            hW = [w.cpu().pin_memory() for w in (Wg, Wu, Wd)]
            hS = None
        # the device-resident copies of the weights are not part of this path: free them
        del Wg, Wu, Wd
        fp8 = None
        torch.cuda.empty_cache()
        mem("device-resident weights freed")
        bytes_in = sum(w.numel() * w.element_size() for w in hW) + sum(t.numel() * 4 for t in (hS or []))
        if rank == 0:
            bytes_in += hX.numel() * 2 + hlog.numel() * 4
        host_out = {}
        d2h = [0]

        def step_e2e():
            if rank == 0:
                X.copy_(hX, non_blocking=True)
                logits.copy_(hlog, non_blocking=True)
            x_chunks = None
            if world > 1:
                dist.broadcast(logits, src=0)
                x_chunks = _bcast_x()
            ids = route_local(logits)
            ok, res, err = True, None, None
            try:
                if world == 1:
                    res = qz.quantize_experts_host(X, ids, hW[0], hW[1], hW[2], e_begin=e0, dense_tail=n_tail,
                                                   fp8_scale_inv=hS)
                else:
                    for _, wait in x_chunks:
                        wait()
                    res = qz.quantize_experts_host(X, ids, hW[0], hW[1], hW[2], e_begin=e0, dense_tail=n_tail,
                                                   fp8_scale_inv=hS, ship_results=False)
            except RuntimeError as exc:
                ok, err = False, exc
            if world == 1:
                if not ok:
                    raise err
                d2h[0] = sum(v.numel() * v.element_size() for v in res[1].values())
                return
            fdist.agree_ok(ok, "solve")
            gathered = plan.run(local_results(res[0]))
            if rank == 0:
                tot = 0
                for k, parts in gathered.items():
                    for j, p in enumerate(parts):
                        key = (k, j)
                        if key not in host_out:
                            host_out[key] = torch.empty(p.shape, dtype=p.dtype).pin_memory()
                        host_out[key].copy_(p, non_blocking=True)
                        tot += p.numel() * p.element_size()
                d2h[0] = tot
            torch.cuda.current_stream().synchronize()

        for _ in range(min(args.warmup, 2)):
            step_e2e()
        ms_e2e, per_e2e = timed(step_e2e, args.steps)
        h2d_total = bytes_in
        if world > 1:
            t = torch.tensor([float(bytes_in)], dtype=torch.float64, device=dev)
            dist.all_reduce(t)
            h2d_total = int(t.item())
        med = sorted(per_e2e)[len(per_e2e) // 2]
        e2e = {"value": n_total / (med / 1e3), "unit": UNIT, "h2d_bytes_per_step": int(h2d_total),
               "d2h_bytes_per_step": int(d2h[0]), "ms_per_step": med, "statistic": "median of the per-step device times",
               "ms_per_step_mean": ms_e2e / args.steps, "ms_per_step_min": min(per_e2e), "ms_per_step_max": max(per_e2e)}

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak, hbm_src = (peaks.get("hbm_gbs"), "measured") if peaks.get("hbm_gbs") else (6650.0, "fallback")
    tf_peak, tf_src = ((peaks.get("bf16_tflops_sustained"), "measured sustained") if peaks.get("bf16_tflops_sustained")
                       else (1400.0, "fallback sustained"))
    hess_flops = float((2.0 * counts * (Hd * Hd + I * I)).sum())
    fwd_flops = float((2.0 * counts * (2.0 * I * Hd)).sum())
    # the kernel computes only the 256x256 tiles on or above the diagonal: flops it actually executes
    def _tri(c):
        nt = (c + 255) // 256
        return nt * (nt + 1) // 2 * 256 * 256
    hess_exec_flops = float((2.0 * counts * (_tri(Hd) + _tri(I))).sum())
    elems = n_loc * 3 * I * Hd
    alg_bytes = {
        "forge_quant_grid": elems * 2 + 8 * elems / 128,
        "forge_chol_inv_upper_batched": n_loc * (2 * Hd * Hd + I * I) * 4 * 2,
        "forge_chol_factor_batched": n_loc * (Hd * Hd + I * I) * 4 * 2,
        "forge_hessian_gather_damp": n_loc * (Hd * Hd + I * I) * 4 * 2,
        "forge_hessian_scan": n_loc * (Hd * Hd + I * I) * 4,
        "forge_pack_int4": elems * 1.5,
        "forge_fp8_block_dequant": elems * 3.0,
    }
    top = max(phases, key=phases.get) if phases else None
    roofline = None
    if top is not None:
        t_s = phases[top] / 1e3
        if top in ("forge_hessian_grouped", "forge_expert_swiglu_grouped"):
            ach = (hess_flops if top == "forge_hessian_grouped" else fwd_flops) / t_s / 1e12
            roofline = {"kernel": top, "bound": "tensor", "achieved": ach, "peak": tf_peak, "unit": "TFLOP/s",
                        "frac": ach / tf_peak, "traffic": None, "peak_source": tf_src}
        elif top in ("forge_gptq_solve_batched", "forge_chol_factor_batched", "forge_chol_inv_upper_batched"):
            # fp32 algorithms run on the tensor pipe as TF32 x3 (three MMAs per product keep fp32 fidelity):
            # `achieved` counts the algorithm's own flops; `executed_tf32_tflops` is what the pipe does for them.
            # No TF32 peak is measured on this pool: half the measured bf16 peak stands in for it.
            if top == "forge_gptq_solve_batched":
                flops = n_loc * (2.0 * I * Hd * Hd + 1.0 * Hd * I * I)       # R C^2 per matrix (error propagation)
            else:
                inv = 3.0 if top == "forge_chol_inv_upper_batched" else 1.0    # + triangular inverse (2/3 n^3 more)
                flops = n_loc * inv * (Hd ** 3 + I ** 3) / 3.0
            ach = flops / t_s / 1e12
            # DRAM bytes of the solver per expert, from ncu captures of small cuts of the same shapes (profiles/),
            # scaled by the experts of this rank; shapes without a capture: null
            per_expert = SOLVER_TRAFFIC_PER_EXPERT.get(args.config) if top == "forge_gptq_solve_batched" else None
            roofline = {"kernel": top, "bound": "tensor", "achieved": ach, "peak": tf_peak, "unit": "TFLOP/s",
                        "frac": ach / tf_peak, "traffic": per_expert * n_loc if per_expert else None,
                        "peak_source": tf_src,
                        "executed_tf32_tflops": 3.0 * ach, "tf32_peak_assumed": tf_peak / 2.0,
                        "executed_frac_of_tf32_peak": 3.0 * ach / (tf_peak / 2.0),
                        "note": "fp32 algorithm as TF32 x3 on tcgen05; the column loop between the MMAs is a serial "
                                "dependency chain per weight row"}
            if top == "forge_gptq_solve_batched":
                # The solver's MMAs are M128 x N128 x K8 kind::tf32 (a 128-column block per accumulator).  The library's
                # diagnostic measures what one such MMA costs when a thread issues them back to back on every SM (64
                # cycles on this pool's B200s = 4096 flop/cycle/SM): the ceiling of any kernel built from this
                # instruction shape, taken at the SM clock seen during the timed region.
                mhz = (clk or {}).get("sm_mhz") or 1965.0
                try:
                    cyc = ops.mma_issue_cycles(128, 2000)      # measured on this GPU, now
                except RuntimeError:
                    cyc = 64.0                                 # the figure of this pool's B200s
                roofline["tf32_m128n128k8_cycles_per_mma"] = cyc
                floor = 2.0 * 128 * 128 * 8 / cyc * 148 * mhz * 1e6 / 1e12
                roofline["tf32_m128n128k8_issue_peak_tflops"] = floor
                roofline["executed_frac_of_issue_peak"] = 3.0 * ach / floor
        else:
            ab = alg_bytes.get(top) or 0.0
            ach = ab / t_s / 1e9
            roofline = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                        "frac": ach / hbm_peak, "traffic": None, "peak_source": hbm_src,
                        "note": "algorithmic bytes over the entry point's device time"}
        if recipe["quantization_scale"] == "mse" and phases.get("forge_quant_grid"):
            # the shrink-factor search costs 2 MUFU operations (lg2, ex2) per element-candidate it evaluates; its
            # ceiling is the special-function pipe (16 lanes/clk/SM), not HBM.  The kernel prunes candidates exactly
            # (partial loss above a finished candidate's loss), so the ALGORITHMIC rate below can exceed that ceiling:
            # the executed share is in the ncu summary of the kernel (XU pipe utilisation).
            sm_hz = (clk or {}).get("sm_mhz") or 1965.0
            mufu_peak = 16.0 * 148 * sm_hz * 1e6
            ec = 100.0 * elems
            t_g = phases["forge_quant_grid"] / 1e3
            roofline["scale_search"] = {"algorithmic_element_candidates_per_s": ec / t_g,
                                        "algorithmic_mufu_ops_per_s": 2 * ec / t_g,
                                        "peak_mufu_ops_per_s": mufu_peak,
                                        "algorithmic_over_peak": 2 * ec / t_g / mufu_peak,
                                        "pruned": True}
        t_h = phases.get("forge_hessian_grouped", 0.0) / 1e3
        roofline["hessian_tflops"] = hess_flops / t_h / 1e12 if t_h > 0 else None
        roofline["hessian_frac_of_bf16_peak"] = (hess_flops / t_h / 1e12 / tf_peak) if t_h > 0 else None
        roofline["hessian_executed_tflops"] = hess_exec_flops / t_h / 1e12 if t_h > 0 else None
        roofline["hessian_executed_frac_of_bf16_peak"] = (hess_exec_flops / t_h / 1e12 / tf_peak) if t_h > 0 else None
        t_f = phases.get("forge_expert_swiglu_grouped", 0.0) / 1e3
        roofline["expert_forward_tflops"] = fwd_flops / t_f / 1e12 if t_f > 0 else None
        # HBM-bound entry points: algorithmic bytes over their device time, against the measured copy bandwidth
        roofline["hbm_kernels"] = {k: {"GB/s": round(alg_bytes[k] / (phases[k] / 1e3) / 1e9, 1),
                                       "frac": round(alg_bytes[k] / (phases[k] / 1e3) / 1e9 / hbm_peak, 3)}
                                   for k in alg_bytes if phases.get(k)}

    cpu_base = None
    if rank == 0 and not args.no_cpu_baseline:
        c = sorted(int(v) for v in counts.tolist()[: max(1, e1 - e0)])
        hot, cold = c[-1], c[0]
        secs = cpu_sample(shape, recipe, [hot, cold])
        cpu_base = {"value": 2.0 / secs, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                    "sample": f"2 experts at full matrix shape: hottest ({hot} tokens) and coldest ({cold} tokens) "
                              f"of rank 0's slice; experts/s extrapolated from their mean time"}

    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and recipe["algorithm"] == "gptq":
        c = sorted(int(v) for v in counts.tolist()[: max(1, e1 - e0)])
        try:
            secs = reference_gpu_sample(shape, recipe, [c[-1], c[0]], dev)
        except Exception as exc:   # a baseline leg must never take the measurement down with it
            secs = None
            print(f"reference_same_gpu leg skipped: {exc}", file=sys.stderr)
        if secs is not None:
            ref_gpu = {"value": 2.0 / secs, "unit": UNIT, "kind": "reference kernels recompiled for sm_100a + torch, "
                       "per-Linear handles on this GPU", "sample": f"2 experts at full matrix shape: hottest ({c[-1]} "
                       f"tokens) and coldest ({c[0]} tokens); experts/s extrapolated from their mean time"}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16 inputs / f32 accumulate and solve", "data": "synthetic",
                "config": {"workload": workload_name(shape, recipe), "parallelism": f"ep{world}",
                           "placement": args.placement if world > 1 else "single", "expert_chunk": chunk,
                           "l2": "inputs larger than L2 (X, weights and Hessians >> 126 MB)"},
                "clocks": clk, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
                "cpu_baseline": cpu_base, "reference_same_gpu": ref_gpu,
                "ms_per_step_median": sorted(per_step)[len(per_step) // 2],
                "phases_ms_rank0": {k: round(v, 3) for k, v in sorted(phases.items(), key=lambda kv: -kv[1])},
                "kernel_ms_by_rank": phase_sums}
        print(json.dumps(line), flush=True)


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
