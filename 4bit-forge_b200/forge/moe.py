"""Layer-level batched GPTQ / SparseGPT for one MoE layer.

The reference quantises one nn.Linear at a time: a forward hook per expert Linear feeds GPTQ.update, then
every handle runs quantize() on its own (quant.py:355-512).  Here the whole layer is one batched pass
over the experts a rank owns:

  routing lists -> grouped tcgen05 Hessian of the layer input (shared by gate and up, the reference's
  --owner_gptq_handles mode) -> expert forward for the down-projection input -> its Hessian ->
  scan / permutation / damping -> batched Cholesky -> scale grid -> fused column solver -> packing.

Everything stays on the device; the host reads back the per-expert token offsets once (to slice the
expert forward) and one flag (whether gate and up have the same all-zero columns).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


@dataclass
class MoEQuantConfig:
    bits: int = 4
    group_size: int = 128
    symmetric: bool = True
    quantization_scale: str = "absmax"     # or "mse"
    quantization_order: str = "default"    # or "activation"
    rel_damp: float = 0.01
    algorithm: str = "gptq"                # or "sparsegptq"
    pack: bool = True
    mse_grid: int = 100
    mse_max_shrink: float = 0.2
    mse_norm: float = 2.4
    expert_chunk: int = 0                  # experts factorised/solved per pass (0 = all at once)
    inversion_free: bool = True            # solve from the Cholesky factor itself, without the triangular inverse
    overlap_streams: bool = True           # scale search on a second stream beside the (latency-bound) factorisation


def swiglu_expert_forward(X, token_lists, offsets_host, Wg, Wu):
    """Down-projection calibration input of every expert, packed by expert: bf16(silu(x Wg^T) * (x Wu^T)).
    Library bf16 GEMMs (fp32 accumulate), exactly what the HF MoE block computes before down_proj.
    The routed rows are gathered once for all experts and the activation runs once over the packed buffer,
    so an expert costs two GEMM launches and nothing else."""
    total = int(offsets_host[-1])
    I = Wg.shape[1]
    if total == 0:
        return torch.empty((1, I), dtype=torch.bfloat16, device=X.device)
    Xg = X.index_select(0, token_lists[:total].long())
    gate = torch.empty((total, I), dtype=torch.bfloat16, device=X.device)
    up = torch.empty((total, I), dtype=torch.bfloat16, device=X.device)
    for e in range(Wg.shape[0]):
        a, b = int(offsets_host[e]), int(offsets_host[e + 1])
        if b == a:
            continue
        torch.mm(Xg[a:b], Wg[e].T, out=gate[a:b])
        torch.mm(Xg[a:b], Wu[e].T, out=up[a:b])
    del Xg
    return torch.nn.functional.silu(gate, inplace=True).mul_(up)


class MoELayerQuantizer:
    """Quantise the experts [e_begin, e_begin + n_local) of one MoE layer on the current CUDA device."""

    def __init__(self, cfg: MoEQuantConfig):
        self.cfg = cfg
        self.inversion_free = False
        self._status = None
        self._side = None          # second compute stream (scale search), created on first use
        self._h2d = None           # copy streams of quantize_experts_host
        self._d2h = None
        self._host_out = {}

    def _side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(priority=-1)
        return self._side

    # ---- one family of matrices sharing per-slot Hessians -------------------------------------
    def _factor(self, H, perm32, pruned, invalid, Ws, wz):
        """H [nu,C,C] (consumed: overwritten by U).  Ws: list of weight batches [nu,R,C] that share H; wz: their
        all-zero-column masks.  Returns one (U, udiag, info) per weight batch."""
        cfg = self.cfg
        shared = all(torch.equal(wz[0], w) for w in wz[1:])      # the one host read of this step
        outs = []
        groups = [wz[0]] if shared else wz
        for gi, wzero in enumerate(groups):
            last = gi == len(groups) - 1
            A, _, _ = ops.hessian_gather_damp(H, perm32, pruned, wzero, invalid, cfg.rel_damp)
            if self.inversion_free:
                # factor only: the solver works from the scaled reverse-Cholesky factor (form = 1)
                U, udiag, info = ops.chol_factor(A)
            else:
                # the last group may overwrite H with U; earlier groups need H intact
                U, udiag, info = ops.chol_inv_upper(A, U=H if last else None, zero_lower=False)
                del A
            outs.append((U, udiag, info))
        if shared:
            outs = outs * len(Ws)
        return outs

    def _solve_family(self, H, n_samples, Ws, names=(), gates=None, between=None):
        """Everything after the Hessian for the weight batches Ws that share it.  names[i]: input name to wait for
        (gates.need) before Ws[i] is touched.  between(): extra work for the main stream while the factorisation
        runs beside it (the expert forward)."""
        cfg = self.cfg
        sparse = cfg.algorithm == "sparsegptq"
        cand = None
        if cfg.quantization_scale == "mse":
            cand = torch.linspace(1.0, cfg.mse_max_shrink, cfg.mse_grid, dtype=torch.float32, device=H.device)
        # the inversion-free form needs 16-byte rows in the solver's work layout
        # (dense GPTQ only: the 1:4 mask choice of SparseGPT is a near-tie argmax and reacts to the different
        # rounding of that form, so the sparse path keeps the reference's form)
        self.inversion_free = (bool(cfg.inversion_free) and not sparse
                               and all(W.shape[1] % 4 == 0 and W.shape[2] % 4 == 0 for W in Ws))
        nu, C, _ = H.shape
        diag, pruned, invalid = ops.hessian_scan(H, n_samples)
        if cfg.quantization_order == "activation":
            perm32 = torch.argsort(diag, dim=1, descending=True).to(torch.int32).contiguous()
        else:
            perm32 = None

        def grid_of(W):
            nb, R, Cw = W.shape
            return ops.quant_grid(W.view(nb * R, Cw), cfg.group_size, cfg.bits, cfg.symmetric, cand, cfg.mse_norm)

        # The scale grids depend on the weights only (after the dead channels are zeroed), the factorisation on the
        # Hessian and on which weight columns are all zero.  The factorisation is a chain of small latency-bound
        # launches: it runs on a high-priority second stream, beside the scale search (special-function bound, many
        # short CTAs) and the expert forward on the main stream, and the solver waits for both.
        main = torch.cuda.current_stream()
        fork = cfg.overlap_streams
        grids = []
        for i, W in enumerate(Ws):
            if gates is not None and i < len(names):
                gates.need(names[i])
            ops.weight_apply_pruned(W, pruned)
            if gates is not None and i < len(Ws) - 1:
                grids.append(grid_of(W))      # overlaps the arrival of the next weight batch
        if fork:
            # host order matters: the main stream's work is queued BEFORE the one host read of the factorisation
            # (are the zero-column masks equal?), so the GPU never waits for the host, and the factorisation's
            # launches are queued right after that read, at high priority
            side = self._side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                wz = [ops.weight_zero_cols(W) for W in Ws]
            for W in Ws[len(grids):]:
                grids.append(grid_of(W))
            if between is not None:
                between()
            with torch.cuda.stream(side):
                factors = self._factor(H, perm32, pruned, invalid, Ws, wz)
            for t in [H, pruned, invalid] + ([perm32] if perm32 is not None else []) + list(Ws):
                t.record_stream(side)
            main.wait_stream(side)
            for U, udiag, info in factors:
                for t in (U, udiag, info):
                    t.record_stream(main)
        else:
            wz = [ops.weight_zero_cols(W) for W in Ws]
            factors = self._factor(H, perm32, pruned, invalid, Ws, wz)
            for W in Ws[len(grids):]:
                grids.append(grid_of(W))
            if between is not None:
                between()
        results = []
        merged = self._solve_merged(Ws, factors, grids, perm32) if len(Ws) == 2 and not sparse else None
        for i, (W, (U, udiag, info), (scales, qzeros)) in enumerate(zip(Ws, factors, grids)):
            nb, R, C = W.shape
            if merged is not None:
                out = merged[i * nb:(i + 1) * nb]
            else:
                out = ops.gptq_solve_batched(W, U, scales, qzeros, cfg.group_size, cfg.bits, perm=perm32,
                                             udiag=udiag if sparse else None, sparse14=sparse, status=self._status,
                                             form=1 if self.inversion_free else 0)
            q, M = out if sparse else (out, None)
            G = (C + cfg.group_size - 1) // cfg.group_size
            res = {"qweight": q, "scales": scales.view(nb, R, G), "qzeros": qzeros.view(nb, R, G), "info": info,
                   "perm": perm32}
            if sparse:
                res["M"] = M
            if cfg.pack:
                res.update(self._pack(q, res["scales"], res["qzeros"], M))
            results.append(res)
        return results

    def _solve_merged(self, Ws, factors, grids, perm32):
        """Two weight batches that share one factor (gate and up) in ONE solver launch, when that fills the GPU
        better: the solver runs one CTA per 128 weight rows, three CTAs per SM, all of equal length, so a launch
        whose last wave is nearly empty wastes most of a wave; together the two batches waste it once, not twice.
        Returns the codes [2 nb, R, C] or None (not worth it / not applicable)."""
        cfg = self.cfg
        (U0, _, _), (U1, _, _) = factors
        W0, W1 = Ws
        if U0 is not U1 or W0.shape != W1.shape:
            return None
        nb, R, C = W0.shape
        slots = 3 * torch.cuda.get_device_properties(W0.device).multi_processor_count
        waves = nb * ((R + 127) // 128) / slots
        if not (0.0 < waves - int(waves) < 0.35):
            return None
        W = torch.cat([W0, W1], 0)
        scales = torch.cat([grids[0][0], grids[1][0]])
        qzeros = torch.cat([grids[0][1], grids[1][1]])
        u_map = torch.arange(nb, dtype=torch.int32, device=W.device).repeat(2)
        return ops.gptq_solve_batched(W, U0, scales, qzeros, cfg.group_size, cfg.bits, perm=perm32, u_map=u_map,
                                      status=self._status, form=1 if self.inversion_free else 0)

    def _pack(self, q, scales, qzeros, M):
        cfg = self.cfg
        nb, R, C = q.shape
        if cfg.algorithm == "sparsegptq":
            # one scale per 32 columns: a group scale repeated gs/32 times (quant.py:438-440 assumes gs == 32)
            rep = cfg.group_size // 32
            G32 = (C + 31) // 32
            packed = []
            for b in range(nb):
                s32 = scales[b].repeat_interleave(rep, dim=1)[:, :G32].transpose(0, 1).contiguous()
                packed.append(ops.pack_sparse14(q[b], M[b], s32))
            return {"wpair": torch.stack(packed)}
        return {"weight_packed": ops.pack_int4(q, qzeros.reshape(-1), cfg.group_size),
                "weight_scale": scales.to(torch.float16)}

    # ---- the layer ----------------------------------------------------------------------------------
    @torch.no_grad()
    def quantize_experts(self, X: torch.Tensor, topk_ids: Optional[torch.Tensor], Wg: torch.Tensor,
                         Wu: torch.Tensor, Wd: torch.Tensor, e_begin: int = 0, dense_tail: int = 0, _gates=None):
        """X [T,Hd] bf16; topk_ids [T,k] int32 (global expert ids); Wg/Wu [n,I,Hd], Wd [n,Hd,I] hold the experts
        this rank owns: first the routed experts e_begin.., then `dense_tail` experts that see every token
        (shared experts).  The weight tensors are updated in place only where a dead input channel forces a
        column to zero.  Returns {"gate": .., "up": .., "down": .., "counts": ..} with per-matrix results.

        `_gates` (internal, see quantize_experts_host): object whose need(name) makes the current stream wait until
        the named input ("gate", "up", "down") has arrived, and whose done(name, results) is told when a family's
        results exist."""
        cfg = self.cfg
        n_local = Wg.shape[0]
        n_routed = n_local - dense_tail
        T, Hd = X.shape
        I = Wg.shape[1]
        dev = X.device
        # ---- routing lists for the local experts
        parts_counts, parts_lists = [], []
        if n_routed > 0:
            counts, offsets, lists = ops.route_build_lists(topk_ids, e_begin, n_routed)
            parts_counts.append(counts.to(torch.int64))
        else:
            lists = torch.empty(0, dtype=torch.int32, device=dev)
        if dense_tail > 0:
            parts_counts.append(torch.full((dense_tail,), T, dtype=torch.int64, device=dev))
        counts64 = torch.cat(parts_counts)
        offsets = torch.zeros(n_local + 1, dtype=torch.int64, device=dev)
        offsets[1:] = torch.cumsum(counts64, 0)
        offsets_host = offsets.cpu()
        n_routed_tok = int(offsets_host[n_routed])
        if dense_tail > 0:
            ar = torch.arange(T, dtype=torch.int32, device=dev)
            lists = torch.cat([lists[:n_routed_tok]] + [ar] * dense_tail)
        lists = lists.contiguous()

        chunk = cfg.expert_chunk if cfg.expert_chunk > 0 else n_local
        res = {"gate": [], "up": [], "down": []}
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._status = status
        act = None
        for c0 in range(0, n_local, chunk):
            c1 = min(n_local, c0 + chunk)
            nb = c1 - c0
            offs = offsets[c0:c1 + 1].contiguous()
            n_samples = counts64[c0:c1].contiguous()
            # the layer-input Hessians need no weights: they run while the weights may still be on their way
            H1 = torch.empty((nb, Hd, Hd), dtype=torch.float32, device=dev)
            ops.hessian_grouped(X, Hd, lists, offs, H1, mirror=True, status=status)
            def forward():
                # down-projection inputs of all local experts (packed by expert); zeroing dead input channels in the
                # weights before does not change them (those channels are zero in every routed row)
                nonlocal act
                if act is None:
                    act = swiglu_expert_forward(X, lists, offsets_host, Wg, Wu)

            g, u = self._solve_family(H1, n_samples, [Wg[c0:c1], Wu[c0:c1]], ("gate", "up"), _gates, forward)
            del H1
            if _gates is not None:
                _gates.done("gate_up", (g, u))
            H2 = torch.empty((nb, I, I), dtype=torch.float32, device=dev)
            ops.hessian_grouped(act, I, None, offs, H2, mirror=True, status=status)
            (d,) = self._solve_family(H2, n_samples, [Wd[c0:c1]], ("down",), _gates)
            del H2
            res["gate"].append(g)
            res["up"].append(u)
            res["down"].append(d)
        out = {k: _cat_results(v) for k, v in res.items()}
        out["counts"] = counts64
        out["status"] = status
        return out

    # ---- the same layer from host memory ---------------------------------------------------------------
    _HOST_KEYS = {"gptq": ("weight_packed", "weight_scale", "qzeros"), "sparsegptq": ("wpair",)}

    @torch.no_grad()
    def quantize_experts_host(self, X, topk_ids, Wg_host, Wu_host, Wd_host, e_begin: int = 0, dense_tail: int = 0,
                              device=None, ship_results: bool = True, fp8_scale_inv=None):
        """quantize_experts for weights that live in (pinned) host memory, results delivered to pinned host memory.

        X / topk_ids may be host or device tensors.  Copies run on their own streams and overlap the kernels:
        the layer-input Hessians start as soon as X has arrived, while gate / up are still being uploaded; down is
        uploaded during the gate / up solve; the packed gate / up results travel back during the down solve.
        Requires expert_chunk == 0 (one pass).  Returns (out, host) where `host` maps "gate.weight_packed" etc. to
        pinned host tensors, valid after the call returns (it synchronises the copy streams); with
        ship_results=False nothing is copied back (the caller gathers on the device) and `host` is empty.

        fp8 checkpoints (DeepSeek-V3): pass the e4m3 weights [n,R,C] and fp8_scale_inv = (sg, su, sd), host fp32
        block scales [n, R/128, C/128]; half the bytes cross PCIe and the bf16 weights are materialised on the
        device (forge/utils/io.py:533-563 of the reference does this on the CPU).  R must be a multiple of 128."""
        cfg = self.cfg
        if cfg.expert_chunk:
            raise ValueError("quantize_experts_host runs the layer in one pass: set expert_chunk = 0")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        main = torch.cuda.current_stream()
        if self._h2d is None:
            self._h2d, self._d2h = torch.cuda.Stream(), torch.cuda.Stream()
        h2d, d2h = self._h2d, self._d2h
        keys = self._HOST_KEYS["sparsegptq" if cfg.algorithm == "sparsegptq" else "gptq"]
        host = {}
        me = self

        def to_device(t, stream_needed):
            if t.is_cuda:
                return t, None
            d = torch.empty(t.shape, dtype=t.dtype, device=dev)      # allocated on the main stream
            return d, t

        Xd, Xh = to_device(X, True)
        idd, idh = to_device(topk_ids, True)
        hosts = (Wg_host, Wu_host, Wd_host)
        fp8 = fp8_scale_inv is not None
        Wg, Wu, Wd = (torch.empty(w.shape, dtype=torch.bfloat16, device=dev) for w in hosts)
        if fp8:
            if any(w.shape[1] % 128 for w in hosts):
                raise ValueError("fp8 block scales need R to be a multiple of 128")
            raw = [torch.empty(w.shape, dtype=torch.uint8, device=dev) for w in hosts]
            sinv = [torch.empty(t.shape, dtype=torch.float32, device=dev) for t in fp8_scale_inv]
            src = [w.view(torch.uint8) for w in hosts]
        else:
            raw, sinv, src = [Wg, Wu, Wd], [None] * 3, list(hosts)
        h2d.wait_stream(main)
        events = {}
        with torch.cuda.stream(h2d):
            if Xh is not None:
                Xd.copy_(Xh, non_blocking=True)
            if idh is not None:
                idd.copy_(idh, non_blocking=True)
            events["x"] = h2d.record_event()
            for j in (0, 1, 2):
                raw[j].copy_(src[j], non_blocking=True)
                if fp8:
                    sinv[j].copy_(fp8_scale_inv[j], non_blocking=True)
                events[("gate", "up", "down")[j]] = h2d.record_event()
        for t in [Xd, idd] + raw + [t for t in sinv if t is not None]:
            t.record_stream(h2d)

        def materialise(js):
            if fp8:
                for j in js:
                    n, R, C = raw[j].shape
                    ops.fp8_block_dequant(raw[j].view(n * R, C), sinv[j].view(-1, sinv[j].shape[-1]),
                                          out=(Wg, Wu, Wd)[j].view(n * R, C))

        def ship(prefix, r):
            # device -> pinned host on the return stream, after the kernels that produced r
            if not ship_results:
                return
            d2h.wait_stream(main)
            with torch.cuda.stream(d2h):
                for k in keys:
                    v = r.get(k)
                    if v is None:
                        continue
                    if k == "qzeros":
                        if cfg.symmetric:
                            continue
                        v = v.to(torch.uint8)
                        name = f"{prefix}.weight_zero_point"
                    else:
                        name = f"{prefix}.{k}"
                    buf = me._host_out.get(name)
                    if buf is None or buf.shape != v.shape or buf.dtype != v.dtype:
                        buf = torch.empty(v.shape, dtype=v.dtype).pin_memory()
                        me._host_out[name] = buf
                    buf.copy_(v, non_blocking=True)
                    v.record_stream(d2h)
                    host[name] = buf

        class Gates:
            def need(self, name):
                torch.cuda.current_stream().wait_event(events[name])
                materialise((("gate", "up", "down").index(name),))

            def done(self, name, results):
                g, u = results
                ship("gate", g)
                ship("up", u)

        main.wait_event(events["x"])
        out = self.quantize_experts(Xd, idd, Wg, Wu, Wd, e_begin=e_begin, dense_tail=dense_tail, _gates=Gates())
        ship("down", out["down"])
        d2h.synchronize()
        return out, host


def _cat_results(parts):
    if len(parts) == 1:
        return parts[0]
    out = {}
    for k in parts[0]:
        vals = [p[k] for p in parts]
        out[k] = None if vals[0] is None else torch.cat(vals, 0)
    return out
