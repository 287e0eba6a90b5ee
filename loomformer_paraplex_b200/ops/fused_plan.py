"""Fused execution plan: hand-written forward and backward over whole temporal chunks.

The composed plan (``models/loomformer.py``) leaves differentiation to autograd, one node per
PyTorch op.  Here the whole training step is a fixed sequence of fat kernels:

* forward of a chunk = L x { QKV GEMM, RoPE + cache write, dual-context attention, out-proj GEMM,
  depth read, readout GEMM, add+LayerNorm, depth K/V GEMM, depth read, readout GEMM, up-projection
  GEMMs (real / gate / segmented imaginary), fused Paraplex core + Tria step, down GEMM, add+LayerNorm,
  depth K/V GEMM } followed by the temporal endpoint (+PolARM);
* backward walks the chunks in reverse and the layers of each chunk in reverse, accumulating weight
  gradients straight into the flat fp32 gradient buffer, key/value gradients into per-layer fp32
  cache-gradient buffers and depth-history gradients into one history-gradient buffer.

Nothing in the sequence depends on host-side values (no ``.item()``), so a whole optimizer step can
be captured in one CUDA graph.  The kernels come from a *kernel set*: ``CudaKernels`` (sm_100a) on a
B200, ``TorchKernels`` (``ops/twins.py``) elsewhere, which lets this file be verified on a CPU
against autograd of the composed plan.

Structure of the reference being replaced: ``loomformer.py:3544-3635`` (block), ``3686-3766`` (chunk
stack), ``3788-3893`` (chunked forward); its per-op ``autograd.Function`` wrappers and the Tria
replay tape (``tria.py:279-709``) have no counterpart because carriers are stored, not replayed.
"""
from __future__ import annotations

import dataclasses
import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..utils.tracing import span

from ..config import FANIN_GAIN
from .twins import TorchKernels


def make_kernels(device: torch.device):
    if device.type == "cuda":
        from .kernels import CudaKernels
        return CudaKernels()
    return TorchKernels()


class FusedPlan:
    def __init__(self, model, kernels=None, flat=None, compute_dtype: Optional[torch.dtype] = None,
                 pad_hidden: Optional[bool] = None) -> None:
        """``pad_hidden``: run the Paraplex FFN with every head's hidden sector rounded up to a multiple of 8
        neurons (None = do so on a GPU exactly when the sector width is not one already).  A transplanted SmolLM2
        has 171 neurons per head: its [M, H] activations would have rows that start off a 16-byte boundary, which
        neither TMA nor the vectorised kernels take.  The padded neurons have zero weights in and out, so they
        change neither the loss nor any gradient (``_refresh_padded`` / ``_unpad_grads``)."""
        self.model, self.d_true = model, model.d
        dev = model.emb.weight.device
        self.K = kernels if kernels is not None else make_kernels(dev)
        self.flat = flat
        self.adt = compute_dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        d = model.d
        if pad_hidden is None:
            pad_hidden = dev.type == "cuda" and d.hpq % 8 != 0
        self._hpad: Dict[int, Tuple[torch.Tensor, int]] = {}      # id(param) -> (param, axis that indexes neurons)
        self._wp: Dict[int, torch.Tensor] = {}                    # padded values (compute dtype; fp32 for vectors)
        self._gp: Dict[int, torch.Tensor] = {}                    # padded fp32 gradients of the current run
        if pad_hidden and d.hpq % 8 != 0:
            hpq_p = (d.hpq + 7) // 8 * 8
            self.d = dataclasses.replace(d, hidden=d.qh * hpq_p, hpq=hpq_p)
            for blk in model.blocks:
                f = blk.ffn
                rows = [f.w1_real.weight, f.w1_real.bias, f.w1_imag, f.w1_imag_bias, f.w1_imag_trace]
                if f.gate_proj is not None:
                    rows += [f.gate_proj.weight, f.gate_proj.bias]
                for q in rows:
                    self._hpad[id(q)] = (q, 0)
                self._hpad[id(f.w2.weight)] = (f.w2.weight, 1)
        else:
            self.d = d
        # The depth-read branch of a sublayer (read + readout GEMM) runs on a second stream beside the branch it does
        # not depend on (attention, resp. the real up-projection), forked and joined inside the cell; in the backward
        # a slot's gradient is formed beside the attention backward of the layer above.  LOOM_OVERLAP=0 keeps
        # everything on one stream.  Measured on one B200: 176.4 -> 173.8 ms per step (113M model, 16 x 2048).
        self._overlap = dev.type == "cuda" and os.environ.get("LOOM_OVERLAP", "1") != "0"
        self._side = None
        self._wcache: Dict[int, torch.Tensor] = {}
        self._consts: Dict[tuple, torch.Tensor] = {}
        self._fetched: set = set()
        self.anchor_sync = None        # optional callable(sumsq [L], count) for cross-rank anchor statistics

    # ------------------------------------------------------------------ parameter access
    def bind(self, flat) -> None:
        self.flat = flat
        self._wcache.clear()

    # sharded weights: ``gather_spec(param)`` (set by the engine in sharded data-parallel mode) says where the owners'
    # copies live; the first linear layer of a run that consumes such a weight fetches it inside its GEMM
    gather_spec = None

    def lin(self, x, p, bias=None, out=None):
        """``x @ p^T (+ bias)`` with ``p`` a parameter (not a weight tensor), fetching sharded weights on first use."""
        spec = None
        if self.gather_spec is not None and id(p) not in self._fetched:
            self._fetched.add(id(p))
            spec = self.gather_spec(p)
        if spec is None:
            return self.K.linear(x, self.w(p), bias, out=out)
        if id(p) in self._hpad:
            raise NotImplementedError("row-sharded weights and padded hidden sectors are not combined; use the "
                                      "replicated or fused-step gradient modes for this model shape")
        return self.K.linear(x, self.w(p), bias, gather=spec, out=out)

    # ------------------------------------------------------------------ padded hidden sectors
    def _sector_view(self, t: torch.Tensor, axis: int, width: int) -> torch.Tensor:
        """View of ``t`` with the neuron axis split into (heads, width)."""
        qh = self.d.qh
        if axis == 0:
            return t.view(qh, width, *t.shape[1:])
        return t.view(t.shape[0], qh, width)

    def _refresh_padded(self) -> None:
        """Copy the current values of the neuron-indexed FFN parameters into their padded buffers (pads stay zero)."""
        hp, hpp = self.d_true.hpq, self.d.hpq
        for key, (p, axis) in self._hpad.items():
            src = self._w_plain(p) if p.dim() == 2 else p.data
            buf = self._wp.get(key)
            if buf is None:
                shape = list(p.shape)
                shape[axis] = self.d.hidden
                buf = self._wp[key] = torch.zeros(shape, dtype=src.dtype if p.dim() == 2 else torch.float32,
                                                  device=p.device)
            dst = self._sector_view(buf, axis, hpp)
            (dst[:, :hp] if axis == 0 else dst[:, :, :hp]).copy_(self._sector_view(src, axis, hp))
        self._gp.clear()

    def _unpad_grads(self) -> None:
        """Add the real neurons' share of every padded gradient into the parameter's own gradient."""
        hp, hpp = self.d_true.hpq, self.d.hpq
        for key, gp in self._gp.items():
            p, axis = self._hpad[key]
            src = self._sector_view(gp, axis, hpp)
            self._sector_view(FusedPlan._g_plain(p), axis, hp).add_(src[:, :hp] if axis == 0 else src[:, :, :hp])
        self._gp.clear()

    def _unpad_neurons(self, t: torch.Tensor, axis: int) -> torch.Tensor:
        """Drop the padded neurons of an activation-like tensor whose ``axis`` indexes (padded) hidden neurons."""
        if not self._hpad:
            return t
        hp, hpp, qh = self.d_true.hpq, self.d.hpq, self.d.qh
        shape = list(t.shape)
        v = t.reshape(*shape[:axis], qh, hpp, *shape[axis + 1:]).narrow(axis + 1, 0, hp)
        return v.reshape(*shape[:axis], qh * hp, *shape[axis + 1:])

    def _pad_neurons(self, t: torch.Tensor, axis: int) -> torch.Tensor:
        """Inverse of :meth:`_unpad_neurons` with zeros in the padded positions."""
        if not self._hpad:
            return t
        hp, hpp, qh = self.d_true.hpq, self.d.hpq, self.d.qh
        shape = list(t.shape)
        out = torch.zeros(*shape[:axis], qh, hpp, *shape[axis + 1:], dtype=t.dtype, device=t.device)
        out.narrow(axis + 1, 0, hp).copy_(t.reshape(*shape[:axis], qh, hp, *shape[axis + 1:]))
        return out.reshape(*shape[:axis], qh * hpp, *shape[axis + 1:])

    def v(self, p: torch.Tensor) -> torch.Tensor:
        """A neuron-indexed vector parameter (bias, trace weight) in fp32, padded when the plan pads."""
        return self._wp[id(p)] if id(p) in self._hpad else p.data

    def w(self, p: torch.Tensor) -> torch.Tensor:
        """Weight in the compute dtype (bf16 shadow on a GPU, the fp32 parameter itself on a CPU); the padded copy for
        a neuron-indexed FFN weight when the plan pads."""
        if id(p) in self._hpad:
            return self._wp[id(p)]
        return self._w_plain(p)

    def _w_plain(self, p: torch.Tensor) -> torch.Tensor:
        if self.adt == torch.float32:
            return p.data
        if self.flat is not None and self.flat.shadow is not None:
            key = id(p)
            v = self._wcache.get(key)
            if v is None:
                v = self.flat.shadow_of(p)
                self._wcache[key] = v
            return v
        return p.data.to(self.adt)

    def _const(self, values: tuple, dev) -> torch.Tensor:
        """Small integer constants as a cached device tensor (no host-to-device copy once a shape has been seen,
        which keeps the step free of pageable copies and therefore capturable in a CUDA graph)."""
        key = (values, str(dev))
        t = self._consts.get(key)
        if t is None:
            t = self._consts[key] = torch.tensor(values, device=dev)
        return t

    def g(self, p: torch.Tensor) -> torch.Tensor:
        """fp32 gradient accumulator of ``p`` (for a padded FFN parameter: this run's padded accumulator, folded into
        the parameter's own gradient by :meth:`_unpad_grads`)."""
        key = id(p)
        if key in self._hpad:
            gp = self._gp.get(key)
            if gp is None:
                gp = self._gp[key] = torch.zeros(self._wp[key].shape, dtype=torch.float32, device=p.device)
            return gp
        return FusedPlan._g_plain(p)

    @staticmethod
    def _g_plain(p: torch.Tensor) -> torch.Tensor:
        if p.grad is None:
            p.grad = torch.zeros_like(p.data, dtype=torch.float32)
        return p.grad

    # ------------------------------------------------------------------ public entry points
    def forward(self, model, idx, attn_mask, position_ids):
        if attn_mask is not None or torch.is_grad_enabled():
            # arbitrary masks and autograd-through-logits go through the composed plan
            if model.d.tria and model.d.tria_temporal and not model.ablation:
                return model._forward_chunked(idx, attn_mask, position_ids)
            return model._forward_flat(idx, attn_mask, position_ids)
        return self.run(idx, None, position_ids, None, want_grad=False)[1]

    def loss(self, model, x, y, attn_mask, position_ids, ignore_index, segment_ids=None):
        if attn_mask is not None or model.ablation:
            raise NotImplementedError("the fused plan takes segment_ids, not dense masks")
        return _FusedLoss.apply(self, x, y, position_ids, segment_ids, ignore_index, self._hook())

    def _hook(self) -> torch.Tensor:
        # a differentiable dummy so autograd calls _FusedLoss.backward
        return torch.zeros((), device=self.model.emb.weight.device, requires_grad=True)

    # ------------------------------------------------------------------ the step
    def run(self, idx, y, position_ids, seg, want_grad: bool, ignore_index: int = -100, grad_scale: float = 1.0,
            return_state: bool = False, cuts=None):
        """Forward (and, with ``want_grad``, backward into ``param.grad``).  Returns (loss, logits); with
        ``return_state`` (inference) additionally the caches a decoder needs to continue the sequences."""
        m, d, K = self.model, self.d, self.K
        B, T = idx.shape
        dev = idx.device
        self._fetched.clear()
        if self._hpad:
            self._refresh_padded()
        if position_ids is None:
            position_ids = torch.arange(T, device=dev).view(1, T).expand(B, T)
        chunked = d.tria and d.tria_temporal and not m.ablation
        if chunked:
            reset, fire, cuts = m.fire_plan(idx, position_ids, last_may_fire=return_state, cuts=cuts)
        else:
            reset, fire, cuts = m._doc_reset(position_ids), None, []
        cut_set = set(cuts)
        stops = cuts + ([T - 1] if not cuts or cuts[-1] != T - 1 else [])
        training = m.training and want_grad
        # activation checkpointing per temporal chunk (reference: loomformer.py:3720-3749): the forward keeps only what
        # crosses chunk boundaries; the backward sweep rebuilds each chunk's tape right before it is consumed
        ckpt = bool(d.grad_checkpointing and want_grad and not return_state)
        emb_w = self.w(m.emb.weight)
        h_emb = emb_w[idx]                                              # [B,T,N]
        cos_all, sin_all = m.rope_cos[position_ids], m.rope_sin[position_ids]     # [B,T,HD] fp32
        tok_reset = position_ids.eq(0)
        L = d.layers
        kc = [torch.zeros(B, T, d.kvh, d.hd, dtype=self.adt, device=dev) for _ in range(L)]
        vc = [torch.zeros(B, T, d.kvh, d.hd, dtype=self.adt, device=dev) for _ in range(L)]
        self._step = self._step_constants(dev, want_grad)
        if want_grad:       # accumulators the cells ask for: sum beta^2 (1), d trace [B,H], and per chunk d seed [B,H,9]
            n_chunks = len(stops)
            K.begin_step(n_chunks * L * (64 + B * d.hidden + 64) + n_chunks * (B * d.hidden * 9 + 64), dev)
        traces: Optional[List[torch.Tensor]] = None
        temporal = None
        tapes, h_parts, keys, key_valid, key_pos = [], [], [], [], []
        s = 0
        for bp in stops:
            e = min(bp + 1, T)
            if e <= s:
                continue
            seed, seed_valid = None, None
            if chunked and temporal is not None:
                seed, seed_valid = temporal, fire[:, s - 1] & ~reset[:, s]
            with span(f"chunk_fwd[{s}:{e}]"):
                # one packed copy per chunk; every layer's RoPE kernels (forward and backward) read it
                tape = self._chunk_forward(h_emb[:, s:e], cos_all[:, s:e].contiguous(), sin_all[:, s:e].contiguous(),
                                           tok_reset[:, s:e], seg,
                                           s, e, kc, vc, traces, seed, seed_valid, training, want_grad)
            traces_in, traces = traces, tape["trace_out"]
            tape.update(s=s, e=e, seed=seed, seed_valid=seed_valid, temporal_in=temporal, fired=None,
                        has_endpoint=False, key_index=None)
            if chunked:
                local_reset = reset[:, s:e].clone()
                if seed_valid is not None:
                    local_reset[:, 0] |= seed_valid
                tape["local_reset"] = local_reset
                if e != T or (e - 1) in cut_set or return_state:
                    fired = fire[:, e - 1] if (e - 1) in cut_set else None
                    temporal, tape["t_aux"] = K.temporal_fwd(tape["depth"], B, e - s, d.hidden, local_reset, temporal,
                                                             fired, m.d_polarm_beta)
                    tape["has_endpoint"], tape["fired"] = True, fired
                    if fired is not None:
                        tape["key_index"] = len(keys)
                        keys.append(temporal); key_valid.append(fired); key_pos.append(e - 1)
            h_parts.append(tape["h_out"].view(B, e - s, d.n))
            if not want_grad:
                tape = {"s": s, "e": e}
            elif ckpt:
                keep = ("s", "e", "seed", "seed_valid", "temporal_in", "fired", "has_endpoint", "key_index",
                        "local_reset", "t_aux")
                light = {k: tape[k] for k in keep if k in tape}
                light["traces_in"] = traces_in
                light["anchors"] = [t["core"]["anchor"] for t in tape["layers"]]
                tape = light
            tapes.append(tape)
            s = e
        h = torch.cat(h_parts, dim=1) if len(h_parts) > 1 else h_parts[0]
        m.last_tria_fire_mask = fire
        # ---- sparse readout of the boundary keys
        ro = None
        if keys:
            ro = self._readout_forward(h, self._unpad_neurons(torch.stack(keys, 1), 2), torch.stack(key_valid, 1),
                                       self._const(tuple(key_pos), dev), seg)
            h = ro["h_out"]
        hn = K.rms_norm_fwd(h, m.ln_final.weight) if m.ln_final is not None else h
        logits = self.lin(hn.reshape(B * T, d.n), m.head.weight).view(B, T, d.vocab)
        if return_state:
            if self._hpad:                       # a decoder continues with the model's own hidden width
                traces = None if traces is None else [self._unpad_neurons(t, 1) for t in traces]
                temporal = None if temporal is None else self._unpad_neurons(temporal, 1)
            state = {"kc": kc, "vc": vc, "traces": traces, "temporal": temporal, "n_keys": len(keys),
                     "pending": fire[:, T - 1] if (chunked and fire is not None) else None}
            if temporal is None and chunked:
                state["pending"] = None
            if ro is not None:
                Kn = len(keys)
                state["ca_k"], state["ca_v"], state["ca_valid"] = ro["k"], ro["v"], torch.stack(key_valid, 1)
            if chunked and state["pending"] is None:
                state["pending"] = torch.zeros(B, dtype=torch.bool, device=dev)
            return None, logits, state
        if y is None:
            return None, logits
        loss, dlogits = K.ce_fwd_bwd(logits.view(B * T, d.vocab), y.reshape(-1), ignore_index,
                                     grad_scale if want_grad else None)
        if not want_grad:
            return loss, logits
        # =============================================================== backward
        hn2 = hn.reshape(B * T, d.n)
        K.linear_wgrad(dlogits, hn2, self.g(m.head.weight))
        dh = K.linear_dgrad(dlogits, self.w(m.head.weight)).view(B, T, d.n)
        del dlogits, logits
        if m.ln_final is not None:
            dh = K.rms_norm_bwd(dh, h, m.ln_final.weight, self.g(m.ln_final.weight))
        dkeys = None
        if ro is not None:
            dh, dkeys = self._readout_backward(ro, dh)
            dkeys = self._pad_neurons(dkeys, 2)
        dkc = [K.alloc_kv_grad(d, B, T, dev) for _ in range(L)]
        dvc = [K.alloc_kv_grad(d, B, T, dev) for _ in range(L)]
        d_emb = torch.empty(B, T, d.n, dtype=self.adt, device=dev)
        dtraces: Optional[List[Optional[torch.Tensor]]] = None
        dtemporal = None                      # gradient w.r.t. the temporal state entering the NEXT chunk
        for tape in reversed(tapes):
            s, e = tape["s"], tape["e"]
            if ckpt:
                with span(f"chunk_recompute[{s}:{e}]"):
                    full = self._chunk_forward(h_emb[:, s:e], cos_all[:, s:e].contiguous(),
                                               sin_all[:, s:e].contiguous(), tok_reset[:, s:e], seg, s, e, kc, vc,
                                               tape["traces_in"], tape["seed"], tape["seed_valid"], False, True,
                                               anchors=tape["anchors"])
                full.update({k: v for k, v in tape.items() if k not in ("traces_in", "anchors")})
                tape = full
            ddepth = None
            if tape["has_endpoint"]:
                dstate = dtemporal
                if tape["key_index"] is not None and dkeys is not None:
                    gk = dkeys[:, tape["key_index"]]
                    dstate = gk if dstate is None else dstate + gk
                if dstate is not None:
                    ddepth, dprev = K.temporal_bwd(dstate, tape["depth"], B, e - s, d.hidden, tape["local_reset"],
                                                   tape["temporal_in"], tape["fired"], m.d_polarm_beta, tape["t_aux"])
                    dtemporal = dprev
                else:
                    dtemporal = None
            else:
                dtemporal = None
            with span(f"chunk_bwd[{s}:{e}]"):
                dx, dtraces, dseed = self._chunk_backward(tape, dh[:, s:e], ddepth, dtraces, kc, vc, dkc, dvc, seg)
            d_emb[:, s:e] = dx.view(B, e - s, d.n)
            if dseed is not None:
                dtemporal = dseed if dtemporal is None else dtemporal + dseed
            tape.clear()
        K.flush_wgrads()           # also joins the weight-gradient stream: with tied embeddings the head's weight
        #                            gradient and the embedding rows below share one buffer
        self.g(m.emb.weight).index_add_(0, idx.reshape(-1), d_emb.view(B * T, d.n).float())
        self._step_constants_bwd()
        if self._hpad:
            self._unpad_grads()
        return loss, None

    # ------------------------------------------------------------------ per-step constants
    def _step_constants(self, dev, want_grad: bool) -> Dict[str, object]:
        """Quantities that depend on parameters only, not on the chunk: the identity-gate strength and the carrier
        read-out weights of every layer and the depth-attention queries.  They are evaluated once per step instead
        of once per (layer, chunk) cell, and the gradients the cells produce for them are summed in two small
        buffers whose chain rule runs once, after the last chunk (:meth:`_step_constants_bwd`)."""
        m, d = self.model, self.d
        L = d.layers
        use_tria = d.tria and not m.ablation
        alpha, gate_w = [], []
        for bi, blk in enumerate(m.blocks):
            ffn = blk.ffn
            alpha.append(ffn.identity_gate.alpha().detach() if ffn.identity_gate is not None else None)
            gate_w.append(ffn.gate_selector.weights().detach() if (use_tria and bi != L - 1) else None)
        st: Dict[str, object] = {"alpha": alpha, "gate_w": gate_w,
                                 "q_all": torch.stack([self._depth_query(sub) for sub in range(2 * L)]).contiguous()}
        if want_grad:
            st["gsc"] = torch.zeros(L, 10, dtype=torch.float32, device=dev)      # [d alpha | d gate_w(9)] per layer
            st["gq"] = torch.zeros(2 * L, d.qh, d.hd, dtype=torch.float32, device=dev)
        return st

    def _step_constants_bwd(self) -> None:
        m, st = self.model, self._step
        gsc = st["gsc"]
        for bi, blk in enumerate(m.blocks):
            ffn = blk.ffn
            ig = ffn.identity_gate
            if ig is not None and ig.raw_alpha.requires_grad:
                self.g(ig.raw_alpha).add_((gsc[bi, 0] * ig.alpha_max * (1.0 - torch.tanh(ig.raw_alpha.data) ** 2))
                                          .reshape(ig.raw_alpha.shape))
            if st["gate_w"][bi] is not None and ffn.gate_selector.logits.requires_grad:
                w9 = st["gate_w"][bi].float()
                gw9 = gsc[bi, 1:10]
                self.g(ffn.gate_selector.logits).add_((w9 * (gw9 - (gw9 * w9).sum())).reshape(
                    ffn.gate_selector.logits.shape))
        for sub in range(st["gq"].shape[0]):
            self._depth_query_bwd(sub, st["gq"][sub])

    # ------------------------------------------------------------------ depth-attention helpers
    def _project_state(self, x2d, slot, hist_k, hist_v, tape_layer, key):
        """K/V projection of a residual-stream state into history slot ``slot``."""
        m, d, K = self.model, self.d, self.K
        M = x2d.shape[0]
        if not d.depth_qkv_rms:
            # hist_k[slot] and hist_v[slot] are the two halves of one packed [M, 2N] block
            assert hist_k.stride(1) == 2 * d.n and hist_v.storage_offset() == hist_k.storage_offset() + d.n
            self.lin(x2d, m.depth_attn.kv_weight, out=hist_k[slot].as_strided((M, 2 * d.n), (2 * d.n, 1)))
            return
        kv = self.lin(x2d, m.depth_attn.kv_weight)
        k, v = kv[:, :d.n].view(M, d.qh, d.hd), kv[:, d.n:].view(M, d.qh, d.hd)
        tape_layer[key + "_kv_raw"] = kv
        hist_k[slot] = K.fixed_rms_fwd(k, FANIN_GAIN)
        hist_v[slot] = K.fixed_rms_fwd(v, FANIN_GAIN * d.deepnorm_beta)

    def _slot_grad(self, slot, dstate, hist_k, hist_v, tape_layer, key, M):
        """Gradient of history slot ``slot`` w.r.t. the K/V projection output, rows [dK | dV], formed in one pass over
        every sublayer that read the slot (all of them must have been staged)."""
        d, K = self.d, self.K
        dkv = K.dread_slot_bwd(d, slot, dstate["q"], hist_k, hist_v, dstate["dm"], dstate["lse"], dstate["dd"],
                               dstate["gq"])                              # [M, 2, QH, HD]: rows [dK | dV]
        if d.depth_qkv_rms:
            kv = tape_layer[key + "_kv_raw"]
            dk = K.fixed_rms_bwd(dkv[:, 0], kv[:, :d.n].view(M, d.qh, d.hd), FANIN_GAIN)
            dv = K.fixed_rms_bwd(dkv[:, 1], kv[:, d.n:].view(M, d.qh, d.hd), FANIN_GAIN * d.deepnorm_beta)
            dkv = torch.cat((dk.reshape(M, d.n), dv.reshape(M, d.n)), -1)
        return dkv.reshape(M, 2 * d.n).to(self.adt)

    def _project_state_bwd(self, x2d, slot, dstate, hist_k, hist_v, tape_layer, key, dkv=None):
        """Backward of :meth:`_project_state`: accumulates the weight gradient and returns the data-gradient term as a
        segment ``(dkv, W)`` for :meth:`linear_dgrad_multi` (the caller folds it into one launch with the other
        products that end in the same tensor).  ``dkv``: the slot's gradient if it has been formed already
        (:meth:`_slot_grad` on the second stream)."""
        m, K = self.model, self.K
        if dkv is None:
            dkv = self._slot_grad(slot, dstate, hist_k, hist_v, tape_layer, key, x2d.shape[0])
        K.linear_wgrad(dkv, x2d, self.g(m.depth_attn.kv_weight))
        return (dkv, self.w(m.depth_attn.kv_weight))

    def _depth_query(self, sub):
        da, d = self.model.depth_attn, self.d
        q = da.q_params.data[sub].float()
        if d.depth_qkv_rms:
            q = self.K.fixed_rms_fwd(q, d.fanin_std(d.hd))
        return q

    def _depth_query_bwd(self, sub, gq):
        da, d = self.model.depth_attn, self.d
        if d.depth_qkv_rms:
            gq = self.K.fixed_rms_bwd(gq, da.q_params.data[sub].float(), d.fanin_std(d.hd))
        self.g(da.q_params)[sub].add_(gq)

    def _readout_w(self, sub):
        da = self.model.depth_attn
        return self.w(da.w_o_weight)[sub] if da.w_o is None else self.w(da.w_o.weight)

    def _readout_lin(self, x, sub):
        da = self.model.depth_attn
        return self.K.linear(x, self.w(da.w_o_weight)[sub]) if da.w_o is None else self.lin(x, da.w_o.weight)

    def _readout_g(self, sub):
        da = self.model.depth_attn
        return self.g(da.w_o_weight)[sub] if da.w_o is None else self.g(da.w_o.weight)

    # ------------------------------------------------------------------ chunk forward
    def _chunk_forward(self, h_emb, cos, sin, tok_reset, seg, s, e, kc, vc, traces_in, seed, seed_valid,
                       training, want_grad, anchors=None):
        """``anchors``: per-layer running radii recorded by an earlier pass over this chunk; given them, the pass
        rebuilds the chunk's tape without touching the running statistics (activation checkpointing)."""
        m, d, K = self.model, self.d, self.K
        B, Tc, N = h_emb.shape
        M = B * Tc
        dev = h_emb.device
        L = d.layers
        S = 2 * L
        # depth history: slot rows are the [K | V] rows of the projection GEMM, so the GEMM stores straight into its slot
        hist = torch.empty(S, M, 2, d.qh, d.hd, dtype=self.adt, device=dev)
        hist_k, hist_v = hist[:, :, 0], hist[:, :, 1]
        h = h_emb.reshape(M, N).contiguous()
        tape = {"layers": [], "hist_k": hist_k, "hist_v": hist_v, "h_emb": h, "cos": cos, "sin": sin, "B": B,
                "emb_l": {}}
        reset_flat = tok_reset.reshape(M)
        c_prev, p_in = None, None
        trace_out = []
        use_tria = d.tria and not m.ablation
        overlap = self._overlap and self.gather_spec is None
        if overlap:
            if self._side is None:
                self._side = torch.cuda.Stream(device=dev)
            side, main = self._side, torch.cuda.current_stream(dev)

        def depth_branch(sub_):
            mm, lse_ = K.dread_fwd(d, self._step["q_all"][sub_], hist_k, hist_v, sub_ + 1)
            return mm, lse_, self._readout_lin(mm.reshape(M, N), sub_)

        # the projection of a state into its history slot is needed first by the depth read of the next sublayer, so it
        # travels with that read: on the second stream both run beside the main stream's GEMMs
        proj = (h, 0, tape["emb_l"], "emb")
        for bi, blk in enumerate(m.blocks):
            last = bi == L - 1
            t: Dict[str, object] = {"h_in": h}
            sub = 2 * bi
            if overlap:                     # depth read 2bi needs only the history: fork it beside attention
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    self._project_state(proj[0], proj[1], hist_k, hist_v, proj[2], proj[3])
                    m1, t["lse1"], s1 = depth_branch(sub)
            else:
                self._project_state(proj[0], proj[1], hist_k, hist_v, proj[2], proj[3])
            # --- attention
            qkc = torch.empty(M, 3, d.qh, d.hd, dtype=self.adt, device=dev)     # sectors: rotated Q, A@K, A@V
            if self.gather_spec is None:    # projection, rotation and cache write as one launch
                K.qkv_rope(d, h, self.w(blk.attn.qkv_weight), cos, sin, qkc, kc[bi], vc[bi], s)
            else:                           # a sharded weight is fetched by its GEMM on first use
                qkv = self.lin(h, blk.attn.qkv_weight).view(B, Tc, -1)
                K.rope_store(d, qkv, cos, sin, qkc, kc[bi], vc[bi], s)
            t["lse"] = K.attn_fwd(d, qkc, kc[bi], vc[bi], s, e, seg)
            t["qkc"] = qkc
            a = self.lin(qkc[:, 2].reshape(M, N), blk.attn.o.weight)
            # --- depth read 2bi, residual, LN
            if overlap:
                main.wait_stream(side)
            else:
                m1, t["lse1"], s1 = depth_branch(sub)
            m1 = m1.reshape(M, N)
            u, t["x1"], t["mean1"], t["rstd1"] = K.add_ln_fwd(s1, a, blk.ln_attn.weight.data, blk.ln_attn.bias.data,
                                                              d.branch_rms_cap)
            t["m1"], t["u"] = m1, u
            if d.branch_rms_cap is not None:
                t["s1"], t["a"] = s1, a
            if overlap:                     # depth read 2bi+1 beside the real (and gate) up-projection
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    self._project_state(u, sub + 1, hist_k, hist_v, t, "u")
                    m2, t["lse2"], s2 = depth_branch(sub + 1)
            else:
                self._project_state(u, sub + 1, hist_k, hist_v, t, "u")
                m2, t["lse2"], s2 = depth_branch(sub + 1)
            t["m2"] = m2
            # --- Paraplex FFN
            ffn = blk.ffn
            x_real = self.lin(u, ffn.w1_real.weight)
            gate_lin = self.lin(u, ffn.gate_proj.weight, self.v(ffn.gate_proj.bias)) if ffn.gate_proj is not None else None
            if overlap:
                main.wait_stream(side)
            beta_lin = K.imag_fwd(d, qkc, u, m2, self.w(ffn.w1_imag))
            alpha_gate = self._step["alpha"][bi] if p_in is not None else None
            gate_w = self._step["gate_w"][bi]
            anchor = None
            core_in = {"x_real": x_real, "p_in": p_in, "alpha_gate": alpha_gate, "b_real": self.v(ffn.w1_real.bias),
                       "gate_lin": gate_lin, "beta_lin": beta_lin, "b_imag": self.v(ffn.w1_imag_bias),
                       "w_trace": self.v(ffn.w1_imag_trace), "trace_in": None if traces_in is None else traces_in[bi],
                       "reset": reset_flat, "c_prev": c_prev, "seed": seed if bi == 0 else None,
                       "seed_valid": seed_valid if bi == 0 else None, "gate_w": gate_w,
                       "axis": (bi % 3) if use_tria else None, "tria_alpha": m.tria_alpha, "B": B}
            out = K.ffn_core_fwd(d, x_real, p_in, alpha_gate, core_in["b_real"], gate_lin, beta_lin, core_in["b_imag"],
                                 core_in["w_trace"], core_in["trace_in"], reset_flat, None, c_prev, core_in["seed"],
                                 core_in["seed_valid"], gate_w, core_in["axis"], m.tria_alpha, B)
            if d.phase_secant:
                if anchors is not None:
                    anchor = anchors[bi]
                elif training:
                    anchor = K.anchor_update(out["beta_sq_sum"], float(M * self.d_true.hidden), ffn.beta_anchor,
                                             ffn.beta_anchor_decay)
                else:
                    anchor = ffn.beta_anchor.detach().clone()
            core_in["anchor"] = anchor
            t["core"] = core_in
            o = out["o"]
            t["o"] = o
            trace_out.append(out["trace_out"])
            c_prev, p_in = out["c"], out["p_out"]
            f = self.lin(o, ffn.w2.weight, ffn.w2.bias.data)
            h, t["x2"], t["mean2"], t["rstd2"] = K.add_ln_fwd(s2, f, blk.ln_ffn.weight.data, blk.ln_ffn.bias.data,
                                                              d.branch_rms_cap)
            if d.branch_rms_cap is not None:
                t["s2"], t["f"] = s2, f
            t["h_out"] = h
            proj = (h, sub + 2, t, "h")     # taken up by the next block (the last block's state has no slot)
            tape["layers"].append(t)
        tape["h_out"] = h
        tape["depth"] = c_prev
        tape["trace_out"] = trace_out
        return tape

    # ------------------------------------------------------------------ chunk backward
    def _chunk_backward(self, tape, dh_out, ddepth, dtraces_out, kc, vc, dkc, dvc, seg):
        """Reverse pass over the layers of one chunk.

        dh_out [B,Tc,N]: gradient of the chunk's final hidden states; ddepth [B,Tc,H,9] or None: gradient of
        the last layer's carriers (from the temporal endpoint); dtraces_out: per-layer gradient of the phase
        trace handed to the next chunk.  Returns (d h_emb [M,N], per-layer d trace_in, d seed)."""
        m, d, K = self.model, self.d, self.K
        B, s, e = tape["B"], tape["s"], tape["e"]
        Tc = e - s
        M, N, L = B * Tc, d.n, d.layers
        dev = dh_out.device
        hist_k, hist_v = tape["hist_k"], tape["hist_v"]
        # depth attention: every sublayer's read gradient is staged; a slot's gradient is formed when the sweep reaches
        # the layer that produced the slot (by then all of its readers have been staged)
        S = 2 * L
        dst = {"q": self._step["q_all"],
               "dm": torch.empty(S, M, d.qh, d.hd, dtype=self.adt, device=dev),
               "lse": torch.empty(S, M, d.qh, dtype=torch.float32, device=dev),
               "dd": torch.empty(S, M, d.qh, dtype=torch.float32, device=dev),
               "gq": self._step["gq"]}                                  # summed over chunks; applied once per step
        dh = dh_out.reshape(M, N).to(self.adt)
        dc = ddepth                      # carrier-layout gradient (opaque to the plan)
        dp_out = None
        dseed = None
        dtraces_in: List[Optional[torch.Tensor]] = [None] * L
        cap = d.branch_rms_cap
        # with the second stream: once sublayer 2bi has been staged, every reader of history slot 2bi is known, so the
        # slot's gradient is formed beside this layer's attention backward and picked up by the layer below
        overlap = self._overlap and self.gather_spec is None and self._side is not None
        if overlap:
            side, main = self._side, torch.cuda.current_stream(dev)
        pending = None
        dh_seg = None                    # (d qkv, W_qkv) of the layer above: its product is the other half of dh
        for bi in range(L - 1, -1, -1):
            blk, t = m.blocks[bi], tape["layers"][bi]
            ffn = blk.ffn
            last = bi == L - 1
            sub = 2 * bi
            if not last:
                if pending is not None:
                    main.wait_stream(side)
                # d h_out = d qkv @ W_qkv (layer above) + d[K|V] @ W_kv (this state's history slot): one launch
                dh = K.linear_dgrad_multi([dh_seg, self._project_state_bwd(t["h_out"], sub + 2, dst, hist_k, hist_v, t, "h",
                                                                            dkv=pending)])
                pending = None
            # --- LN2 and the two addends
            ds2, df = K.add_ln_bwd(dh, t["x2"], t["mean2"], t["rstd2"], blk.ln_ffn.weight.data,
                                   self.g(blk.ln_ffn.weight), self.g(blk.ln_ffn.bias), cap, t.get("s2"), t.get("f"))
            # --- w2
            K.linear_wgrad(df, t["o"], self.g(ffn.w2.weight))
            K.colsum_add(df, self.g(ffn.w2.bias))
            do = K.linear_dgrad(df, self.w(ffn.w2.weight))
            # --- Paraplex core + Tria
            core = t["core"]
            core["g_b_real"], core["g_b_imag"] = self.g(ffn.w1_real.bias), self.g(ffn.w1_imag_bias)
            core["g_w_trace"] = self.g(ffn.w1_imag_trace)
            core["gsc_acc"] = self._step["gsc"][bi]     # d alpha_gate and d gate_w are summed here across chunks
            gr = K.ffn_core_bwd(d, core, do, dc, dp_out, None if dtraces_out is None else dtraces_out[bi])
            dx_real, dbeta = gr["d_x_real"].to(self.adt), gr["d_beta_lin"].to(self.adt)
            dtraces_in[bi] = gr.get("d_trace_in")
            dc, dp_out = gr.get("d_c_prev"), gr.get("d_p_in")
            if gr.get("d_seed") is not None:
                dseed = gr["d_seed"]
            if gr.get("d_b_real") is not None:          # the native kernel accumulates these itself
                core["g_b_real"].add_(gr["d_b_real"])
                core["g_b_imag"].add_(gr["d_b_imag"])
                core["g_w_trace"].add_(gr["d_w_trace"])
            u = t["u"]
            # d u collects four products (real up-projection, gate projection, the shared sector of the imaginary
            # projection, this state's history slot); they leave as one launch once the last of them is known
            K.linear_wgrad(dx_real, u, self.g(ffn.w1_real.weight))
            du_segs = [(dx_real, self.w(ffn.w1_real.weight))]
            if ffn.gate_proj is not None:
                dgl = gr["d_gate_lin"].to(self.adt)
                K.linear_wgrad(dgl, u, self.g(ffn.gate_proj.weight))
                K.colsum_add(dgl, self.g(ffn.gate_proj.bias))
                du_segs.append((dgl, self.w(ffn.gate_proj.weight)))
            dqkc, _, dm2_i, u_seg = K.imag_bwd(d, dbeta, t["qkc"], u, t["m2"], self.w(ffn.w1_imag), self.g(ffn.w1_imag),
                                               defer_u=True)
            du_segs.append(u_seg)
            # --- depth read 2bi+1 (its output feeds the readout GEMM and the imaginary projection)
            K.linear_wgrad(ds2, t["m2"].reshape(M, N), self._readout_g(sub + 1))
            K.dread_stage(d, K.linear_dgrad(ds2, self._readout_w(sub + 1)).view(M, d.qh, d.hd), dm2_i, t["m2"], t["lse2"],
                          dst, sub + 1)
            du_segs.append(self._project_state_bwd(u, sub + 1, dst, hist_k, hist_v, t, "u"))
            du = K.linear_dgrad_multi(du_segs)
            # --- LN1
            ds1, da = K.add_ln_bwd(du, t["x1"], t["mean1"], t["rstd1"], blk.ln_attn.weight.data,
                                   self.g(blk.ln_attn.weight), self.g(blk.ln_attn.bias), cap, t.get("s1"), t.get("a"))
            K.linear_wgrad(ds1, t["m1"], self._readout_g(sub))
            K.dread_stage(d, K.linear_dgrad(ds1, self._readout_w(sub)).view(M, d.qh, d.hd), None,
                          t["m1"].view(M, d.qh, d.hd), t["lse1"], dst, sub)
            if overlap:
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    below = (tape["layers"][bi - 1], "h") if bi > 0 else (tape["emb_l"], "emb")
                    pending = self._slot_grad(sub, dst, hist_k, hist_v, below[0], below[1], M)
            # --- attention
            qkc = t["qkc"]
            K.linear_wgrad(da, qkc[:, 2].reshape(M, N), self.g(blk.attn.o.weight))
            K.linear_dgrad(da, self.w(blk.attn.o.weight), out=dqkc.view(M, 3, N)[:, 2], accumulate=True)
            dq_attn = K.attn_bwd(d, dqkc, qkc, kc[bi], vc[bi], t["lse"], s, e, seg, dkc[bi], dvc[bi])
            dqkv = K.rope_bwd(d, dq_attn.reshape(B, Tc, d.qh, d.hd), dqkc, dkc[bi], dvc[bi], s, e, tape["cos"],
                              tape["sin"], self.adt).view(M, -1)
            K.linear_wgrad(dqkv, t["h_in"], self.g(blk.attn.qkv_weight))
            dh_seg = (dqkv, self.w(blk.attn.qkv_weight))
        if pending is not None:
            main.wait_stream(side)
        dh = K.linear_dgrad_multi([dh_seg, self._project_state_bwd(tape["h_emb"], 0, dst, hist_k, hist_v, tape["emb_l"],
                                                                    "emb", dkv=pending)])
        return dh, dtraces_in, dseed

    # ------------------------------------------------------------------ readout
    def _readout_forward(self, h, doc_keys, valid, key_pos, seg):
        """doc_keys [B,Kn,H,9] fp32 -> pooled 9-vectors -> keys [B,Kn,N]; masked cross-attention added to h."""
        m, d, K = self.model, self.d, self.K
        agg, fca = m.tria_agg, m.tria_final_ca
        B, T, N = h.shape
        Kn = key_pos.numel()
        score_w = agg.score_w().detach().float()
        pooled = K.slot_pool_fwd(doc_keys, score_w)                                   # [B,Kn,9] fp32
        z = torch.addmm(agg.reader.proj.bias.data, pooled.view(B * Kn, 9), agg.reader.proj.weight.data.t())
        a = torch.addmm(agg.up.bias.data, z, agg.up.weight.data.t()).to(self.adt)     # [B*Kn,N]
        q = self.lin(h.reshape(B * T, N), fca.w_qk.weight).view(B, T, N)
        k = self.lin(a, fca.w_qk.weight).view(B, Kn, N)
        v = self.lin(a, fca.w_v.weight).view(B, Kn, N)
        allowed = key_pos.view(1, 1, Kn) <= torch.arange(T, device=h.device).view(1, T, 1)
        allowed = allowed & valid[:, None, :]
        if seg is not None:
            allowed = allowed & (seg.unsqueeze(-1) == seg[:, key_pos].unsqueeze(1))
        out = K.cross_attn_fwd(q, k, v, allowed, fca.scale)
        gamma = fca.gamma().detach()
        h_out = (h.float() + gamma * out.float()).to(h.dtype)
        return {"h": h, "h_out": h_out, "doc_keys": doc_keys, "score_w": score_w, "pooled": pooled, "z": z, "a": a,
                "q": q, "k": k, "v": v, "allowed": allowed, "out": out, "gamma": gamma}

    def _readout_backward(self, ro, dh_out):
        m, d, K = self.model, self.d, self.K
        agg, fca = m.tria_agg, m.tria_final_ca
        h = ro["h"]
        B, T, N = h.shape
        Kn = ro["k"].shape[1]
        gamma = ro["gamma"]
        dgamma = (dh_out.float() * ro["out"].float()).sum()
        self.g(fca.raw_gamma).add_(dgamma * fca.gamma_max * (1.0 - torch.tanh(fca.raw_gamma.data) ** 2))
        dout = (dh_out.float() * gamma).to(self.adt)
        dq, dk, dv = K.cross_attn_bwd(dout, ro["q"], ro["k"], ro["v"], ro["allowed"], fca.scale)
        dq, dk, dv = dq.to(self.adt).reshape(B * T, N), dk.to(self.adt).reshape(B * Kn, N), dv.to(self.adt).reshape(B * Kn, N)
        a = ro["a"]
        K.linear_wgrad(dq, h.reshape(B * T, N), self.g(fca.w_qk.weight))
        K.linear_wgrad(dk, a, self.g(fca.w_qk.weight))
        K.linear_wgrad(dv, a, self.g(fca.w_v.weight))
        dh = dh_out + K.linear_dgrad(dq, self.w(fca.w_qk.weight)).view(B, T, N)
        da = (K.linear_dgrad(dk, self.w(fca.w_qk.weight)) + K.linear_dgrad(dv, self.w(fca.w_v.weight))).float()
        # tiny fp32 tail: up (32->N) and proj (9->32)
        self.g(agg.up.weight).add_(da.t() @ ro["z"]); self.g(agg.up.bias).add_(da.sum(0))
        dz = da @ agg.up.weight.data
        pooled = ro["pooled"].view(B * Kn, 9)
        self.g(agg.reader.proj.weight).add_(dz.t() @ pooled); self.g(agg.reader.proj.bias).add_(dz.sum(0))
        dpooled = (dz @ agg.reader.proj.weight.data).view(B, Kn, 9)
        dkeys, dscore = K.slot_pool_bwd(dpooled, ro["doc_keys"], ro["score_w"])
        # score_w = normalize(key_proj^T query) * softplus(logit_scale_raw): differentiate the 9-vector by autograd
        with torch.enable_grad():
            kp = agg.reader.key_proj.weight.detach().requires_grad_(True)
            qy = agg.pool.query.detach().requires_grad_(True)
            ls = agg.pool.logit_scale_raw.detach().requires_grad_(True)
            w9 = torch.nn.functional.normalize(torch.mv(kp.t(), qy), dim=0, eps=1e-6) * torch.nn.functional.softplus(ls)
            g_kp, g_q, g_ls = torch.autograd.grad(w9, [kp, qy, ls], dscore.to(w9.dtype))
        self.g(agg.reader.key_proj.weight).add_(g_kp)
        self.g(agg.pool.query).add_(g_q)
        self.g(agg.pool.logit_scale_raw).add_(g_ls)
        return dh, dkeys


class _FusedLoss(torch.autograd.Function):
    """Loss node of the fused plan: forward and backward both run in ``forward`` (gradients are written
    straight into ``param.grad``); ``backward`` only checks the incoming scale."""

    @staticmethod
    def forward(ctx, plan, x, y, position_ids, seg, ignore_index, hook):
        with torch.no_grad():
            loss, _ = plan.run(x, y, position_ids, seg, want_grad=True, ignore_index=ignore_index,
                               grad_scale=plan.pending_scale if hasattr(plan, "pending_scale") else 1.0)
        return loss

    @staticmethod
    def backward(ctx, g):
        return (None,) * 7
