"""Layer-level batched GPTQ / SparseGPT for one MoE layer.

The reference quantises one nn.Linear at a time: a forward hook per expert Linear feeds GPTQ.update, then
every handle runs quantize() on its own (quant.py:355-512).  Here the whole layer is one batched pass
over the experts a rank owns:

  routing lists -> grouped tcgen05 Hessian of the layer input (shared by gate and up, the reference's
  --owner_gptq_handles mode) -> expert forward for the down-projection input -> its Hessian ->
  scan / permutation / damping -> batched Cholesky -> scale grid -> fused column solver -> packing.

Everything stays on the device and nothing is read back while the step is being queued: routing lists, the
expert forward and the factorisation take their sizes from device-side offsets.  The host reads ONE small tensor
when all launches are queued (the status word of the bounded waits and bounds checks, and whether gate and up
turned out to have different all-zero columns, in which case the layer is redone with separate factors).
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
    merge_gate_up: Optional[bool] = None   # gate and up in one solver launch (None: when the last wave would be thin)
    keep_codes: bool = True                # keep the unpacked uint8 codes in the result (tests, write-back)
    presplit_factor: bool = True           # split each factor into tensor-core operand pieces once, for all row strips


def swiglu_expert_forward(X, token_lists, offsets, Wg, Wu, out_rows, status=None):
    """Down-projection calibration input of every expert, packed by expert: bf16(silu(x Wg^T) * (x Wu^T)) with
    the bf16 roundings of the HF MoE block forward — one grouped tcgen05 launch (forge_expert_swiglu_grouped);
    `offsets` stays on the device, `out_rows` is the capacity of the packed output."""
    return ops.expert_swiglu_grouped(X, token_lists, offsets, Wg, Wu, out_rows, status=status)


class MoELayerQuantizer:
    """Quantise the experts [e_begin, e_begin + n_local) of one MoE layer on the device that holds X."""

    def __init__(self, cfg: MoEQuantConfig):
        self.cfg = cfg
        self._status = None
        self._mismatch = None      # device flag: gate and up of some expert have different all-zero columns
        self._side = None          # second compute stream (factorisation), created on first use
        self._h2d = None           # copy streams of quantize_experts_host
        self._d2h = None
        self._host_out = {}
        self._arena = {}           # the large per-pass work buffers, kept across passes and steps

    def _buf(self, name, nbytes, device):
        """A named work buffer of at least nbytes (uint8), allocated once and reused by every pass and every step:
        Hessians, factor copy, operand pieces and solver workspace are tens of GB that would otherwise go through
        the caching allocator several times per step, on two streams.  Reuse is safe because each pass orders its
        two streams explicitly (the factorisation's stream waits for the main one when it starts, and the main one
        waits for it before the solve)."""
        buf = self._arena.get(name)
        if buf is None or buf.numel() < nbytes or buf.device != device:
            self._arena.pop(name, None)
            buf = None
            buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
            self._arena[name] = buf
        return buf[:int(nbytes)]

    def _buf_f32(self, name, shape, device):
        n = 1
        for v in shape:
            n *= int(v)
        return self._buf(name, 4 * n, device).view(torch.float32).view(*shape)

    def release_buffers(self):
        """Drop the cached work buffers (they are re-created on the next call)."""
        self._arena.clear()

    def _side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(priority=-1)
        return self._side

    def _form(self, Ws) -> int:
        """1 = inversion-free solve (dense GPTQ, 16-byte rows in the solver's work layout), 0 = the reference's.
        The 1:4 mask choice of SparseGPT is a near-tie argmax and reacts to the different rounding of form 1, so
        the sparse path keeps the reference's form."""
        cfg = self.cfg
        ok = (bool(cfg.inversion_free) and cfg.algorithm != "sparsegptq"
              and all(W.shape[1] % 4 == 0 and W.shape[2] % 4 == 0 for W in Ws))
        return 1 if ok else 0

    # ---- one family of matrices sharing per-slot Hessians -------------------------------------
    def _factor(self, H, perm32, pruned, invalid, Ws, wz, form, separate):
        """H [nu,C,C] (consumed: overwritten by U).  Ws: list of weight batches [nu,R,C] that share H; wz: their
        all-zero-column masks.  Returns one (U, udiag, info) per weight batch.

        The factor depends on which weight columns are all zero (forge/gptq.py:145-149).  Gate and up normally
        agree on that (dead input channels are zeroed in both), so ONE factor serves both and a device-side flag
        records whether some expert disagreed; quantize_experts reads the flag once, when everything is queued,
        and redoes the layer with `separate` factors in that rare case."""
        cfg = self.cfg
        outs = []
        if not separate and len(wz) > 1:
            differ = torch.zeros((), dtype=torch.bool, device=H.device)
            for w in wz[1:]:
                differ = differ | (wz[0] != w).any()
            self._mismatch = differ if self._mismatch is None else (self._mismatch | differ)
        groups = wz if separate else [wz[0]]
        for gi, wzero in enumerate(groups):
            last = gi == len(groups) - 1
            A = None
            if form == 1 and len(groups) == 1:
                A = self._buf_f32("factor", H.shape, H.device)
            A, _, _ = ops.hessian_gather_damp(H, perm32, pruned, wzero, invalid, cfg.rel_damp, A=A)
            if form == 1:
                # factor only: the solver works from the scaled reverse-Cholesky factor
                U, udiag, info = ops.chol_factor(A)
            else:
                # the last group may overwrite H with U; earlier groups need H intact
                U, udiag, info = ops.chol_inv_upper(A, U=H if last else None, zero_lower=False)
                del A
            outs.append((U, udiag, info))
        if not separate:
            outs = outs * len(Ws)
        return outs

    def _solve_family(self, Hbox, n_samples, Ws, names=(), gates=None, between=None, separate=False):
        """Everything after the Hessian for the weight batches Ws that share it.  Hbox: one-element list holding the
        Hessian batch; the list is emptied as soon as the factorisation is queued, so that the Hessians' memory is
        free again during the solve (the inversion-free form factors a copy).  names[i]: input name to wait for
        (gates.need) before Ws[i] is touched.  between(): extra work for the main stream while the factorisation
        runs beside it (the expert forward)."""
        cfg = self.cfg
        H = Hbox[0]
        sparse = cfg.algorithm == "sparsegptq"
        cand = None
        if cfg.quantization_scale == "mse":
            cand = torch.linspace(1.0, cfg.mse_max_shrink, cfg.mse_grid, dtype=torch.float32, device=H.device)
        form = self._form(Ws)
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
            side = self._side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                wz = [ops.weight_zero_cols(W) for W in Ws]
                factors = self._factor(H, perm32, pruned, invalid, Ws, wz, form, separate)
            for W in Ws[len(grids):]:
                grids.append(grid_of(W))
            if between is not None:
                between()
            for t in [H, pruned, invalid] + ([perm32] if perm32 is not None else []) + list(Ws):
                t.record_stream(side)
            Hbox.clear()
            del H
            main.wait_stream(side)
            for U, udiag, info in factors:
                for t in (U, udiag, info):
                    t.record_stream(main)
        else:
            wz = [ops.weight_zero_cols(W) for W in Ws]
            factors = self._factor(H, perm32, pruned, invalid, Ws, wz, form, separate)
            Hbox.clear()
            del H
            for W in Ws[len(grids):]:
                grids.append(grid_of(W))
            if between is not None:
                between()
        results = []
        # tensor-core operand pieces of each distinct factor, split once for all row strips (and for gate and up)
        splits = {}
        for U, _, _ in factors:
            if id(U) not in splits:
                splits[id(U)] = (ops.solve_split_u(U, out=(lambda n, d=U.device: self._buf("pieces", n, d))
                                                   if len(factors) == 1 or factors[0][0] is factors[-1][0] else None)
                                 if cfg.presplit_factor else None)
        merged = (self._solve_merged(Ws, factors, grids, perm32, form, splits) if len(Ws) == 2 and not sparse else None)
        for i, (W, (U, udiag, info), (scales, qzeros)) in enumerate(zip(Ws, factors, grids)):
            nb, R, C = W.shape
            if merged is not None:
                out = merged[i * nb:(i + 1) * nb]
            else:
                out = ops.gptq_solve_batched(W, U, scales, qzeros, cfg.group_size, cfg.bits, perm=perm32,
                                             udiag=udiag if sparse else None, sparse14=sparse, status=self._status,
                                             form=form, usplit=splits[id(U)],
                                             ws=lambda n, d=W.device: self._buf("solve", n, d))
            q, M = out if sparse else (out, None)
            G = (C + cfg.group_size - 1) // cfg.group_size
            res = {"qweight": q, "scales": scales.view(nb, R, G), "qzeros": qzeros.view(nb, R, G), "info": info,
                   "perm": perm32}
            if sparse:
                res["M"] = M
            if cfg.pack:
                res.update(self._pack(q, res["scales"], res["qzeros"], M))
                if not cfg.keep_codes:
                    res["qweight"] = None
            results.append(res)
        return results

    @staticmethod
    def merge_pays(nb: int, R: int, sm_count: int) -> bool:
        """The solver runs one CTA per 128 weight rows, three CTAs per SM, all of equal length; a launch whose last
        wave is nearly empty wastes most of a wave, and gate and up together waste it once instead of twice."""
        waves = nb * ((R + 127) // 128) / (3.0 * sm_count)
        return 0.0 < waves - int(waves) < 0.35

    def _solve_merged(self, Ws, factors, grids, perm32, form, splits):
        """Two weight batches that share one factor (gate and up) in ONE solver launch.  Same arithmetic per
        matrix, so the codes are identical to two launches; only the launch shape differs.
        Returns the codes [2 nb, R, C] or None (not worth it / not applicable)."""
        cfg = self.cfg
        (U0, _, _), (U1, _, _) = factors
        W0, W1 = Ws
        if U0 is not U1 or W0.shape != W1.shape:
            return None
        nb, R, C = W0.shape
        want = cfg.merge_gate_up
        if want is None:
            want = self.merge_pays(nb, R, torch.cuda.get_device_properties(W0.device).multi_processor_count)
        if not want:
            return None
        W = torch.cat([W0, W1], 0)
        scales = torch.cat([grids[0][0], grids[1][0]])
        qzeros = torch.cat([grids[0][1], grids[1][1]])
        u_map = torch.arange(nb, dtype=torch.int32, device=W.device).repeat(2)
        return ops.gptq_solve_batched(W, U0, scales, qzeros, cfg.group_size, cfg.bits, perm=perm32, u_map=u_map,
                                      status=self._status, form=form, usplit=splits[id(U0)],
                                      ws=lambda n, d=W.device: self._buf("solve", n, d))

    def _pack(self, q, scales, qzeros, M):
        cfg = self.cfg
        nb, R, C = q.shape
        if cfg.algorithm == "sparsegptq":
            # one scale per 32 columns: a group scale repeated gs/32 times (quant.py:438-440 assumes gs == 32)
            rep = cfg.group_size // 32
            G32 = (C + 31) // 32
            s32 = scales.reshape(nb, R, -1).repeat_interleave(rep, dim=2)[:, :, :G32].transpose(1, 2).contiguous()
            return {"wpair": ops.pack_sparse14_batched(q.contiguous(), M.contiguous(), s32)}
        return {"weight_packed": ops.pack_int4(q, qzeros.reshape(-1), cfg.group_size),
                "weight_scale": scales.to(torch.float16)}

    # ---- the layer ----------------------------------------------------------------------------------
    @torch.no_grad()
    def quantize_experts(self, X: torch.Tensor, topk_ids: Optional[torch.Tensor], Wg: torch.Tensor,
                         Wu: torch.Tensor, Wd: torch.Tensor, e_begin: int = 0, dense_tail: int = 0, _gates=None,
                         check: bool = True, x_chunks=None):
        """X [T,Hd] bf16; topk_ids [T,k] int32 (global expert ids); Wg/Wu [n,I,Hd], Wd [n,Hd,I] hold the experts
        this rank owns: first the routed experts e_begin.., then `dense_tail` experts that see every token
        (shared experts).  The weight tensors are updated in place only where a dead input channel forces a
        column to zero.  Returns {"gate": .., "up": .., "down": .., "counts": .., "status": ..} with per-matrix
        results.  With check=True (default) the call ends with one host read of the status word and raises
        RuntimeError if a bounded wait ran out or a bounds check failed; check=False leaves that read to the
        caller (out["status"], out["mismatch"]).

        x_chunks (expert-parallel runs): [(row_end, wait)] as returned by forge.dist.broadcast_inputs(chunks > 1) —
        the rows of X arrive chunk by chunk; wait() makes the current stream wait for a chunk.  The layer-input
        Hessians are then accumulated chunk by chunk in the running-mean form of GPTQ.update (forge/gptq.py:62-80:
        H <- n_prev/N H + 2/N X_c^T X_c), so the Hessian of chunk i runs while chunk i+1 is still in flight.

        `_gates` (internal, see quantize_experts_host): object whose need(name) makes the current stream wait until
        the named input ("gate", "up", "down") has arrived, and whose done(results, c0, n) is told when the results
        of the experts [c0, c0 + chunk) of a family exist."""
        with torch.cuda.device(X.device):
            out = self._quantize_experts(X, topk_ids, Wg, Wu, Wd, e_begin, dense_tail, _gates, separate=False,
                                         x_chunks=x_chunks)
            if check and _gates is None:
                out = self._finish(out, lambda: self._quantize_experts(X, topk_ids, Wg, Wu, Wd, e_begin, dense_tail,
                                                                        None, separate=True))
        return out

    def _finish(self, out, redo):
        """The one host read of a step: status word + gate/up zero-column disagreement."""
        flags = torch.stack([out["status"].view(()).to(torch.int32),
                             out["mismatch"].view(()).to(torch.int32)]).cpu()
        status, mismatch = int(flags[0]), int(flags[1])
        if status != 0:
            what = {1: "a bounds check failed (FORGE_ERR_INVALID)", 3: "a bounded device-side wait ran out "
                    "(FORGE_ERR_TIMEOUT)"}.get(status, f"status {status}")
            raise RuntimeError(f"forge.moe: {what}; the results of this step are not valid")
        if mismatch:
            out = redo()
            status = int(out["status"].item())
            if status != 0:
                raise RuntimeError(f"forge.moe: status {status} in the separate-factor pass")
        return out

    def _chunked_input_hessians(self, X, topk_ids, e_begin, n_routed, dense_tail, x_chunks, status):
        """Layer-input Hessians of all local slots, accumulated over the row chunks of X as they arrive."""
        T, Hd = X.shape
        n_local = n_routed + dense_tail
        H1 = self._buf_f32("hessian", (n_local, Hd, Hd), X.device)
        n_prev = torch.zeros(n_local, dtype=torch.int64, device=X.device)
        t0 = 0
        for t1, wait in x_chunks:
            wait()
            if t1 > t0:
                ids_c = topk_ids[t0:t1] if n_routed > 0 else None
                _, offs_c, lists_c = ops.route_build_lists(ids_c, e_begin, n_routed, dense_tail, n_tokens=t1 - t0)
                ops.hessian_grouped(X[t0:t1], Hd, lists_c, offs_c, H1, n_prev=n_prev, mirror=True, status=status)
                ops.counts_add(n_prev, offs_c)
            t0 = t1
        return H1

    def _quantize_experts(self, X, topk_ids, Wg, Wu, Wd, e_begin, dense_tail, _gates, separate, x_chunks=None):
        cfg = self.cfg
        n_local = Wg.shape[0]
        n_routed = n_local - dense_tail
        T, Hd = X.shape
        I = Wg.shape[1]
        dev = X.device
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        H1_all = None
        if x_chunks:
            if cfg.expert_chunk and cfg.expert_chunk < n_local:
                for _, wait in x_chunks:     # expert chunking and row chunking do not combine: take X whole
                    wait()
            else:
                H1_all = self._chunked_input_hessians(X, topk_ids, e_begin, n_routed, dense_tail, x_chunks, status)
        # ---- routing lists for the local slots: routed experts, then the dense tail (every token)
        counts, offsets, lists = ops.route_build_lists(topk_ids if n_routed > 0 else None, e_begin, n_routed,
                                                       dense_tail, n_tokens=T)
        counts64 = counts.to(torch.int64)
        k = topk_ids.shape[1] if (topk_ids is not None and n_routed > 0) else 0
        act_rows = T * k + dense_tail * T      # capacity of the packed activations; the true size stays on the device

        chunk = cfg.expert_chunk if cfg.expert_chunk > 0 else n_local
        res = {"gate": [], "up": [], "down": []}
        self._status = status
        self._mismatch = None
        act = None
        for c0 in range(0, n_local, chunk):
            c1 = min(n_local, c0 + chunk)
            nb = c1 - c0
            offs = offsets[c0:c1 + 1]
            n_samples = counts64[c0:c1]
            # the layer-input Hessians need no weights: they run while the weights may still be on their way
            if H1_all is not None:
                H1, H1_all = H1_all, None
            else:
                H1 = self._buf_f32("hessian", (nb, Hd, Hd), dev)
                ops.hessian_grouped(X, Hd, lists, offs, H1, mirror=True, status=status)

            def forward():
                # down-projection inputs of all local experts (packed by expert); zeroing dead input channels in the
                # weights before does not change them (those channels are zero in every routed row)
                nonlocal act
                if act is None:
                    act = swiglu_expert_forward(X, lists, offsets, Wg, Wu, act_rows, status=status)

            Hbox = [H1]
            del H1
            g, u = self._solve_family(Hbox, n_samples, [Wg[c0:c1], Wu[c0:c1]], ("gate", "up"), _gates, forward, separate)
            if _gates is not None:
                _gates.done({"gate": g, "up": u}, c0, n_local)
            H2 = self._buf_f32("hessian", (nb, I, I), dev)
            ops.hessian_grouped(act, I, None, offs, H2, mirror=True, status=status)
            Hbox = [H2]
            del H2
            (d,) = self._solve_family(Hbox, n_samples, [Wd[c0:c1]], ("down",), _gates)
            if _gates is not None:
                _gates.done({"down": d}, c0, n_local)
            res["gate"].append(g)
            res["up"].append(u)
            res["down"].append(d)
        out = {k_: _cat_results(v) for k_, v in res.items()}
        out["counts"] = counts64
        out["status"] = status
        out["mismatch"] = self._mismatch if self._mismatch is not None else torch.zeros((), dtype=torch.bool, device=dev)
        out["routing"] = {"lists": lists, "offsets": offsets, "act": act}
        return out

    @torch.no_grad()
    def reconstruction_loss(self, out, X, Wg, Wu, Wd):
        """|| X W^T - X What^T ||_F^2 of every matrix of a quantize_experts result, on the device
        (forge_recon_loss): {"gate": f64 [n], "up": f64 [n], "down": f64 [n]}.  Wg/Wu/Wd are the weights as
        quantize_experts left them; the down projection is evaluated on the activations the step produced."""
        gs = self.cfg.group_size
        r = out["routing"]
        losses = {}
        for name, W, Xin, lst in (("gate", Wg, X, r["lists"]), ("up", Wu, X, r["lists"]), ("down", Wd, r["act"], None)):
            o = out[name]
            losses[name] = ops.recon_loss(W, o["qweight"], o["scales"].contiguous(), o["qzeros"].contiguous(), gs, Xin,
                                          lst, r["offsets"], status=out["status"])
        return losses

    # ---- the same layer from host memory ---------------------------------------------------------------
    _HOST_KEYS = {"gptq": ("weight_packed", "weight_scale", "qzeros"), "sparsegptq": ("wpair",)}

    @torch.no_grad()
    def quantize_experts_host(self, X, topk_ids, Wg_host, Wu_host, Wd_host, e_begin: int = 0, dense_tail: int = 0,
                              device=None, ship_results: bool = True, fp8_scale_inv=None):
        """quantize_experts for weights that live in (pinned) host memory, results delivered to pinned host memory.

        X / topk_ids may be host or device tensors.  Copies run on their own streams and overlap the kernels:
        the layer-input Hessians start as soon as X has arrived, while gate / up are still being uploaded; down is
        uploaded during the gate / up solve; the packed gate / up results travel back during the down solve.
        Returns (out, host) where `host` maps "gate.weight_packed" etc. to
        pinned host tensors.  They are complete when the call returns (it synchronises the copy streams and checks
        the status word: RuntimeError if a bounded wait ran out or a bounds check failed) and they are the
        quantizer's own cached buffers: the NEXT call on this quantizer with the same shapes overwrites them, so a
        caller that keeps a layer's results while the next layer runs (an asynchronous checkpoint writer) must copy
        them or use a second quantizer.  With ship_results=False nothing is copied back (the caller gathers on the
        device) and `host` is empty.

        fp8 checkpoints (DeepSeek-V3): pass the e4m3 weights [n,R,C] and fp8_scale_inv = (sg, su, sd), host fp32
        block scales [n, R/128, C/128]; half the bytes cross PCIe and the bf16 weights are materialised on the
        device (forge/utils/io.py:533-563 of the reference does this on the CPU).  R must be a multiple of 128."""
        cfg = self.cfg
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        for t in (X, topk_ids):
            if t.is_cuda and t.device != dev:
                raise ValueError(f"quantize_experts_host: input on {t.device}, but the layer runs on {dev}")
        with torch.cuda.device(dev):
            return self._quantize_experts_host(X, topk_ids, Wg_host, Wu_host, Wd_host, e_begin, dense_tail, dev,
                                               ship_results, fp8_scale_inv)

    def _quantize_experts_host(self, X, topk_ids, Wg_host, Wu_host, Wd_host, e_begin, dense_tail, dev, ship_results,
                               fp8_scale_inv):
        cfg = self.cfg
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

        def ship(prefix, r, c0=0, n_total=None):
            # device -> pinned host on the return stream, after the kernels that produced r; r holds the experts
            # [c0, c0 + len) of n_total, the pinned buffers hold all of them
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
                    full = (n_total if n_total is not None else v.shape[0],) + tuple(v.shape[1:])
                    buf = me._host_out.get(name)
                    if buf is None or tuple(buf.shape) != full or buf.dtype != v.dtype:
                        buf = torch.empty(full, dtype=v.dtype).pin_memory()
                        me._host_out[name] = buf
                    buf[c0:c0 + v.shape[0]].copy_(v, non_blocking=True)
                    v.record_stream(d2h)
                    host[name] = buf

        arrived = set()

        def need(name):
            if name in arrived:
                return
            arrived.add(name)
            torch.cuda.current_stream().wait_event(events[name])
            materialise((("gate", "up", "down").index(name),))

        def done(results, c0, n_total):
            for nm, r in results.items():
                ship(nm, r, c0, n_total)

        gates = _Gates(need, done)
        main.wait_event(events["x"])
        out = self._quantize_experts(Xd, idd, Wg, Wu, Wd, e_begin, dense_tail, gates, separate=False)

        def redo():
            # gate and up disagree on their all-zero columns: same layer again with one factor per matrix
            # (every input is on the device by now; nothing overlaps in this rare pass)
            o = self._quantize_experts(Xd, idd, Wg, Wu, Wd, e_begin, dense_tail, None, separate=True)
            for nm in ("gate", "up", "down"):
                ship(nm, o[nm])
            return o

        out = self._finish(out, redo)
        d2h.synchronize()
        gates.need = gates.done = None      # the closures hold this call's device buffers: drop them now
        return out, host


class _Gates:
    """need(name) / done(results, c0, n) callbacks of quantize_experts_host.  A module-level class on purpose: a class
    defined inside the call would be a reference cycle, and the tens of GB of device buffers its closures reach
    would stay allocated until Python's cycle collector happens to run."""

    def __init__(self, need, done):
        self.need, self.done = need, done


def _cat_results(parts):
    if len(parts) == 1:
        return parts[0]
    out = {}
    for k in parts[0]:
        vals = [p[k] for p in parts]
        out[k] = None if vals[0] is None else torch.cat(vals, 0)
    return out
