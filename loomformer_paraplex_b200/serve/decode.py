"""Graph-replayed incremental decoding.

``DecodeEngine`` keeps every piece of per-sequence state in preallocated device tensors (KV caches, per-layer phase
traces, the Tria temporal carrier, the sparse final cross-attention key cache) and advances all sequences of a batch
by one token per call.  The step contains no host-side control flow -- the shared position, the fire decision, the
conditional key append and the greedy/top-k choice are all device-side -- so it is captured once in a CUDA graph and
replayed per token.  The reference decodes with a Python loop of ~25 launches per layer plus several ``.item()``
synchronisations per token and prefills token by token (reference ``loomformer.py:3951-4091``, ``loomchat.py:338-380``).

Prefill runs the prompt through the chunked fused forward once and converts its caches into decode state.
"""
from __future__ import annotations

import math
import dataclasses
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ..config import FANIN_GAIN
from ..ops import reference as R


def check_request(prompt_len: int, max_new: int, max_len: int) -> None:
    """Refuse, on the host, a request whose positions would leave the KV cache / RoPE table of ``max_len`` rows."""
    if prompt_len < 1:
        raise ValueError("empty prompt")
    if max_new < 1:
        raise ValueError(f"max_new={max_new} must be at least 1")
    if prompt_len + max_new - 1 > max_len:
        raise ValueError(f"prompt of {prompt_len} tokens + {max_new} new tokens needs {prompt_len + max_new - 1} "
                         f"positions; this engine holds max_len={max_len}")


class DecodeEngine:
    def __init__(self, model, batch: int, max_len: Optional[int] = None, use_graph: bool = True,
                 dtype: Optional[torch.dtype] = None) -> None:
        self.m, self.d = model, model.d
        d = self.d
        self.B = int(batch)
        self.S = int(max_len or d.seq_len)
        if self.S < 1 or self.S > int(d.seq_len):
            raise ValueError(f"max_len={self.S} is outside 1..seq_len={int(d.seq_len)} (the RoPE table and the "
                             "position grid end there)")
        self._host_pos = 0          # host mirror of the device-side position: bounds are refused before any launch
        dev = model.emb.weight.device
        self.dev = dev
        self.dt = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        self.use_graph = bool(use_graph and dev.type == "cuda")
        B, S, L = self.B, self.S, d.layers
        z = lambda *s, dtype=None: torch.zeros(*s, dtype=dtype or self.dt, device=dev)
        self.kc, self.vc = z(L, B, S, d.kvh, d.hd), z(L, B, S, d.kvh, d.hd)
        self.trace = z(L, B, d.hidden, dtype=torch.float32)
        self.carry = z(B, d.hidden, 3, 3, dtype=torch.float32)
        self.have_carry = z(1, dtype=torch.bool)
        self.pending = z(B, dtype=torch.bool)
        # boundary keys: one per hard window boundary; any token can fire when the model has a carry token
        W = max(1, int(model.tria_window or 1))
        self.ca_cap = S if model.carry_token_id is not None else S // W + 1
        self.ca_k, self.ca_v = z(B, self.ca_cap, d.n), z(B, self.ca_cap, d.n)
        self.ca_valid = z(B, self.ca_cap, dtype=torch.bool)
        self.ca_len = z(1, dtype=torch.long)
        self.pos = z(1, dtype=torch.long)
        self.tok_in = z(B, dtype=torch.long)
        self.logits = z(B, d.vocab, dtype=torch.float32)
        self.next_tok = z(B, dtype=torch.long)
        self._graph = None
        self._w = {}
        # native KV-cache attention (bf16 on CUDA): positions are split over enough blocks to fill the GPU
        self._native_attn = False
        if dev.type == "cuda" and self.dt == torch.bfloat16 and d.hd % 8 == 0 and d.group <= 8:
            from ..ops import native
            if native.available():
                self._native_attn = True
                # position slices per (sequence, KV head): 128 positions each (one tile of the tensor-core kernel) while
                # that needs no more than 64 slices, else about four blocks per SM with at least 64 positions each (the
                # merge of the slices by the last block grows with their number)
                self._ns = -(-S // 128)
                if self._ns > 64:
                    self._ns = max(1, min(16, -(-592 // (B * d.kvh)), -(-S // 64)))
                n_ws = B * d.kvh * self._ns * (2 * d.group + 2 * d.group * d.hd) + B * d.kvh
                self._attn_ws = torch.zeros(n_ws, dtype=torch.float32, device=dev)     # partial states | ticket counters
                from ..ops.kernels import status_word
                self._status = status_word(dev)        # set by a bounded wait that gave up; read by check_status
        # fused kernels of the training plan reused at one token per sequence (fewer, larger launches per layer).  A
        # hidden sector that is not a multiple of 8 neurons wide (a SmolLM2 transplant has 171 per head) is padded
        # with inert neurons inside the FFN part of the step, exactly as the training plan does; the engine's own
        # state (trace, carry) keeps the model's width.
        self._dk = d if d.hpq % 8 == 0 else dataclasses.replace(d, hidden=d.qh * ((d.hpq + 7) // 8 * 8),
                                                                hpq=(d.hpq + 7) // 8 * 8)
        self._wpad = {}
        self._fused = bool(self._native_attn and d.activation == "pvpowlu" and d.hd <= 128
                           and d.n % 8 == 0 and d.n <= 1024 and not model.ablation
                           and os.environ.get("LOOM_DECODE_FUSED", "1") != "0")
        if self._fused:
            from ..ops.kernels import CudaKernels
            self._K = CudaKernels(defer_wgrad=False)
            # depth history: a slot's row is the [K | V] row of the projection GEMM, which stores straight into it
            self._hist = z(2 * L, B, 2, d.qh, d.hd)
            self._hk, self._hv = self._hist[:, :, 0], self._hist[:, :, 1]
            self._qkc = z(B, 3, d.qh, d.hd)
            self._rope_cos = model.rope_cos.detach().float().reshape(-1, d.hd).contiguous()
            self._rope_sin = model.rope_sin.detach().float().reshape(-1, d.hd).contiguous()
            # per-step flags, scratch that every step overwrites
            self._fire, self._reset, self._row_reset, self._seed_valid = (z(B, dtype=torch.bool) for _ in range(4))
            self._allowed = z(B, self.ca_cap, dtype=torch.uint8)
            self._any = z(1, dtype=torch.long)
            self._trace_new = z(L, B, self._dk.hidden, dtype=torch.float32)
            self._bsq = z(1, dtype=torch.float32)
        self.refresh_weights()

    # ------------------------------------------------------------------ weights in the compute dtype
    def refresh_weights(self) -> None:
        self._w = {id(p): p.detach().to(self.dt) for p in self.m.parameters()}
        self._wpad = {}
        if getattr(self, "_fused", False) and self._dk is not self.d:
            for blk in self.m.blocks:
                f = blk.ffn
                rows = [f.w1_real.weight, f.w1_real.bias, f.w1_imag, f.w1_imag_bias, f.w1_imag_trace]
                if f.gate_proj is not None:
                    rows += [f.gate_proj.weight, f.gate_proj.bias]
                for q in rows:
                    src = q.detach().to(self.dt if q.dim() == 2 else torch.float32)
                    self._wpad[id(q)] = self._pad(src, 0)
                self._wpad[id(f.w2.weight)] = self._pad(f.w2.weight.detach().to(self.dt), 1)
        if getattr(self, "_fused", False):
            # parameter-derived constants of the step (softmaxes, tanh gains, normalised depth queries): evaluated once
            # per weight refresh instead of once per token
            m, da = self.m, self.m.depth_attn
            c = {"query": [da.query(sub).detach().float().contiguous() for sub in range(2 * self.d.layers)],
                 "gate_w": [None if getattr(b.ffn, "gate_selector", None) is None
                            else b.ffn.gate_selector.weights().detach().float().contiguous() for b in m.blocks],
                 "alpha": [None if b.ffn.identity_gate is None else b.ffn.identity_gate.alpha().detach().float().reshape(1)
                           for b in m.blocks]}
            if self.d.tria:
                agg, fca = m.tria_agg, m.tria_final_ca
                c["score_w"] = agg.score_w().detach().float().contiguous()
                c["proj_wT"] = agg.reader.proj.weight.detach().float().t().contiguous()
                c["proj_b"] = agg.reader.proj.bias.detach().float()
                c["up_wT"] = agg.up.weight.detach().float().t().contiguous()
                c["up_b"] = agg.up.bias.detach().float()
                c["gamma"] = float(fca.gamma().detach())
            self._const = c
        self._graph = None

    def _pad(self, t: torch.Tensor, axis: int) -> torch.Tensor:
        """Zero-padded copy of ``t`` whose ``axis`` indexes hidden neurons (heads x sector): sector width d.hpq ->
        the kernels' width."""
        d, dk = self.d, self._dk
        if dk is d:
            return t
        shape = list(t.shape)
        out = torch.zeros(*shape[:axis], d.qh, dk.hpq, *shape[axis + 1:], dtype=t.dtype, device=t.device)
        out.narrow(axis + 1, 0, d.hpq).copy_(t.reshape(*shape[:axis], d.qh, d.hpq, *shape[axis + 1:]))
        return out.reshape(*shape[:axis], dk.hidden, *shape[axis + 1:])

    def _unpad(self, t: torch.Tensor, axis: int) -> torch.Tensor:
        d, dk = self.d, self._dk
        if dk is d:
            return t
        shape = list(t.shape)
        v = t.reshape(*shape[:axis], d.qh, dk.hpq, *shape[axis + 1:]).narrow(axis + 1, 0, d.hpq)
        return v.reshape(*shape[:axis], d.hidden, *shape[axis + 1:])

    def wk(self, p):
        """Weight as the fused kernels want it: the padded copy for a neuron-indexed FFN parameter (2-D in the compute
        dtype, vectors in fp32), the compute-dtype copy otherwise."""
        v = self._wpad.get(id(p))
        return v if v is not None else self._w[id(p)]

    def w(self, p):
        return self._w[id(p)]

    def invalidate(self) -> None:
        """Drop the captured graph: call after changing a hyper-parameter that the step bakes in as a constant
        (temporal window, carrier alpha, PolARM beta) or after ``refresh_weights`` replaced the weight copies."""
        self._graph = None

    # ------------------------------------------------------------------ state management
    def reset(self) -> None:
        if self.m.carry_token_id is not None and self.ca_cap < self.S:
            # the model was given a carry token after this engine was built: any token may now append a boundary key
            z = lambda *shape, dtype=self.dt: torch.zeros(*shape, dtype=dtype, device=self.dev)
            self.ca_cap = self.S
            self.ca_k, self.ca_v = z(self.B, self.S, self.d.n), z(self.B, self.S, self.d.n)
            self.ca_valid = z(self.B, self.S, dtype=torch.bool)
            if self._fused:
                self._allowed = z(self.B, self.S, dtype=torch.uint8)
            self._graph = None
        for t in (self.kc, self.vc, self.trace, self.carry, self.ca_k, self.ca_v):
            t.zero_()
        self.have_carry.zero_(); self.pending.zero_(); self.ca_valid.zero_(); self.ca_len.zero_(); self.pos.zero_()
        self._host_pos = 0

    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """Ingest ``prompt`` [B, T0] (equal lengths) and return the logits of its last position [B, V]."""
        B, T0 = prompt.shape
        if B != self.B:
            raise ValueError(f"prompt batch {B} does not match the engine's batch {self.B}")
        if T0 < 1 or T0 > self.S:
            raise ValueError(f"prompt length {T0} is outside 1..max_len={self.S}")
        self.reset()
        plan = self.m._opset(self.m.emb.weight)
        if plan is not None and not self.m.ablation:
            _, logits, st = plan.run(prompt, None, None, None, want_grad=False, return_state=True)
            L = self.d.layers
            for l in range(L):
                self.kc[l, :, :T0] = st["kc"][l][:, :T0]
                self.vc[l, :, :T0] = st["vc"][l][:, :T0]
                self.trace[l] = st["traces"][l].float()
            if st["temporal"] is not None:
                self.carry.copy_(st["temporal"].view(B, self.d.hidden, 3, 3))
                self.have_carry.fill_(True)
                self.pending.copy_(st["pending"])
            n = st["n_keys"]
            if n:
                self.ca_k[:, :n], self.ca_v[:, :n] = st["ca_k"], st["ca_v"]
                self.ca_valid[:, :n] = st["ca_valid"]
            self.ca_len.fill_(n)
            self.pos.fill_(T0)
            self._host_pos = T0
            return logits[:, -1].float()
        out = None
        for t in range(T0):
            out = self.step(prompt[:, t])
        return out

    # ------------------------------------------------------------------ one token
    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """Feed ``tokens`` [B] at the current position; returns logits [B, V] (a view that the next call overwrites).
        Raises ``ValueError`` on the host, before anything is launched, when the cache is full."""
        if self._host_pos >= self.S:
            raise ValueError(f"decode position {self._host_pos} would pass max_len={self.S}: the KV cache and the "
                             "RoPE table end there")
        self._host_pos += 1
        self.tok_in.copy_(tokens)
        if not self.use_graph:
            self._step_impl()
            return self.logits
        if self._graph is None:
            # warm-up on a side stream (allocator / lazy init), with state restored afterwards
            snap = [t.clone() for t in self._state()]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._step_impl()
            torch.cuda.current_stream().wait_stream(s)
            for t, c in zip(self._state(), snap):
                t.copy_(c)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._step_impl()
            for t, c in zip(self._state(), snap):
                t.copy_(c)
        self._graph.replay()
        return self.logits

    def _state(self):
        return [self.kc, self.vc, self.trace, self.carry, self.have_carry, self.pending, self.ca_k, self.ca_v,
                self.ca_valid, self.ca_len, self.pos]

    def _lin(self, x, p, bias=None):
        y = F.linear(x, self.w(p))
        return y if bias is None else y + self.w(bias)

    def _step_impl(self) -> None:
        if self._fused:
            return self._step_fused()
        return self._step_composed()

    # ------------------------------------------------------------------ one token with the fused kernels
    def _step_fused(self) -> None:
        """Same arithmetic as :meth:`_step_composed` with the training plan's kernels at M = batch rows.  The step is
        bound by the number of dependent launches, so everything that waits for the same producer leaves in one launch:
        the linear layers of a layer are four multi-segment launches (QKV + depth K/V of the incoming stream; attention
        output + first depth readout; real / gate projections + depth K/V of the normalised stream; the per-head
        imaginary projection + second depth readout) and the down projection, RoPE and the cache append are one kernel,
        attention (with its merge) one, the Paraplex core with the Tria step one."""
        m, d, K, dk = self.m, self.d, self._K, self._dk
        B, S = self.B, self.S
        pos, cst = self.pos, self._const
        from ..ops import native
        ext = native.ext()
        bf = dict(dtype=self.dt, device=self.dev)
        ext.decode_step_flags(pos, self.tok_in, self.pending, self.have_carry, self._fire, self._reset, self._row_reset,
                              self._seed_valid, int(m.tria_window or 0), int(d.seq_len), bool(m.tria_hard_fire_enabled),
                              -1 if m.carry_token_id is None else int(m.carry_token_id), bool(d.tria_temporal))
        native.count()
        h = self.w(m.emb.weight)[self.tok_in]
        da = m.depth_attn
        hk, hv, qkc = self._hk, self._hv, self._qkc
        small = B <= 128          # products of up to 128 rows have a multi-segment kernel (16: CUDA cores, 128: tcgen05)
        after = []

        def project_seg(x, slot):
            """Segment that projects ``x`` into history slot ``slot`` ([K | V] row, written in place)."""
            if not d.depth_qkv_rms:
                return ([x], self.w(da.kv_weight), None, self._hist[slot].view(B, 2 * d.n))
            kv = torch.empty(B, 2 * d.n, **bf)

            def norm():
                k, v = kv[:, :d.n].view(B, d.qh, d.hd), kv[:, d.n:].view(B, d.qh, d.hd)
                hk[slot].copy_(K.fixed_rms_fwd(k, FANIN_GAIN)); hv[slot].copy_(K.fixed_rms_fwd(v, FANIN_GAIN * d.deepnorm_beta))
            after.append(norm)
            return ([x], self.w(da.kv_weight), None, kv)

        def multi(segs):
            K.linear_multi(segs, static_weights=True)
            while after:
                after.pop()()

        def w_o(sub):
            return self.w(da.w_o_weight)[sub] if da.w_o is None else self.w(da.w_o.weight)

        cap = d.branch_rms_cap if (d.branch_rms_cap is not None and m.decode_applies_rms_cap) else None
        use_tria = d.tria
        padded = dk is not d
        vec = (lambda q: self.wk(q)) if padded else (lambda q: q.data)
        c_planes, p_in = None, None
        fork = os.environ.get("LOOM_DECODE_FORK", "1") != "0"     # second stream for the branch that needs only the history
        if fork:
            if getattr(self, "_side", None) is None:
                self._side = torch.cuda.Stream()
            side, main = self._side, torch.cuda.current_stream()
        for bi, blk in enumerate(m.blocks):
            last = bi == d.layers - 1
            sub = 2 * bi
            ffn = blk.ffn
            qkv = torch.empty(B, d.n + 2 * d.kv_dim, **bf)
            multi([([h], self.w(blk.attn.qkv_weight), None, qkv), project_seg(h, sub)])
            if fork:        # the first depth read needs only the history: it runs beside RoPE and attention
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    mm_a, _ = K.dread_fwd(d, cst["query"][sub], hk, hv, sub + 1)
            # RoPE of Q and K at the device-side position, rotated Q into the attention operand, K / V appended
            ext.decode_rope_store(qkv, self._rope_cos, self._rope_sin, pos, qkc[:, 0].view(B, d.n), self.kc[bi],
                                  self.vc[bi], d.qh, d.kvh, d.hd)
            ext.decode_attn(qkc[:, 0], self.kc[bi], self.vc[bi], pos, qkc[:, 2], qkc[:, 1], self._attn_ws, B, S,
                            d.qh, d.kvh, d.hd, self._ns, self._status)
            native.count(2)
            if fork:
                main.wait_stream(side)
            else:
                mm_a, _ = K.dread_fwd(d, cst["query"][sub], hk, hv, sub + 1)
            attn_out, skip = torch.empty(B, d.n, **bf), torch.empty(B, d.n, **bf)
            multi([([qkc[:, 2].reshape(B, d.n)], self.w(blk.attn.o.weight), None, attn_out),
                   ([mm_a.view(B, d.n)], w_o(sub), None, skip)])
            u = K.add_ln_fwd(skip, attn_out, blk.ln_attn.weight.data, blk.ln_attn.bias.data, cap)[0]
            wx = torch.empty(B, dk.hidden, **bf)
            segs = [project_seg(u, sub + 1), ([u], self.wk(ffn.w1_real.weight), None, wx)]
            gate_lin = None
            if ffn.gate_proj is not None:
                gate_lin = torch.empty(B, dk.hidden, **bf)
                segs.append(([u], self.wk(ffn.gate_proj.weight), self.wk(ffn.gate_proj.bias), gate_lin))
            multi(segs)
            d_sel, _ = K.dread_fwd(d, cst["query"][sub + 1], hk, hv, sub + 2)
            skip2 = torch.empty(B, d.n, **bf)
            read2 = ([d_sel.view(B, d.n)], w_o(sub + 1), None, skip2)
            if small:
                # the per-head operand [q | k-context | context | u | depth read] of the imaginary projection is gathered
                # from its pieces by the kernel; one segment per head
                beta_lin = torch.empty(B, dk.hidden, **bf)
                w3 = self.wk(ffn.w1_imag).view(d.qh, dk.hpq, d.imag_in)
                b3 = beta_lin.view(B, d.qh, dk.hpq)
                segs = [read2]
                for g in range(d.qh):
                    if d.open_sectors:
                        pieces = [qkc[:, 0, g], qkc[:, 1].reshape(B, d.n), qkc[:, 2].reshape(B, d.n), u, d_sel.view(B, d.n)]
                    else:
                        pieces = [qkc[:, 0, g], qkc[:, 1, g], qkc[:, 2, g], u, d_sel[:, g]]
                    segs.append((pieces, w3[g], None, b3[:, g]))
                multi(segs)
            else:
                multi([read2])
                beta_lin = K.imag_fwd(dk, qkc, u, d_sel, self.wk(ffn.w1_imag))
            tria_here = use_tria
            core = K.ffn_core_fwd(
                dk, wx, p_in if ffn.identity_gate is not None else None,
                cst["alpha"][bi], vec(ffn.w1_real.bias), gate_lin, beta_lin,
                vec(ffn.w1_imag_bias), vec(ffn.w1_imag_trace), self._pad(self.trace[bi], 1), self._row_reset, None,
                c_planes if bi > 0 else None,
                self._pad(self.carry.view(B, d.hidden, 9), 1) if (tria_here and bi == 0) else None,
                self._seed_valid if (tria_here and bi == 0) else None,
                cst["gate_w"][bi] if (tria_here and not last) else None,
                (bi % 3) if tria_here else None, m.tria_alpha if tria_here else 0.0, B,
                trace_out=self._trace_new[bi], bsq=self._bsq)
            if tria_here:
                c_planes = core["c"]
                p_in = None if last else core["p_out"]
            a_t = None
            if last and fork:
                # the temporal endpoint and the boundary key need only the last layer's carriers: they (and the trace
                # hand-over) run beside the last down projection and its add + LayerNorm
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    self.trace.copy_(self._unpad(self._trace_new, 2))
                    if use_tria:
                        a_t = self._boundary_key(c_planes)
            f = torch.empty(B, d.n, **bf)
            multi([([core["o"]], self.wk(ffn.w2.weight), ffn.w2.bias.data, f)])
            h = K.add_ln_fwd(skip2, f, blk.ln_ffn.weight.data, blk.ln_ffn.bias.data, cap)[0]
        if fork:
            main.wait_stream(side)
        else:
            self.trace.copy_(self._unpad(self._trace_new, 2))
            if use_tria:
                a_t = self._boundary_key(c_planes)
        self._finish_fused(h, a_t)

    def _boundary_key(self, c_planes) -> torch.Tensor:
        """Temporal endpoint of this token's carriers (the training plan's ``temporal_fwd`` at a chunk of one token), new
        carried state, and the pooled boundary-key vector ``[B, N]`` (slot pool, reader projection, up projection)."""
        m, d, K, dk = self.m, self.d, self._K, self._dk
        B, cst = self.B, self._const
        state = self._pad(self.carry.view(B, d.hidden, 9), 1)
        doc, _ = K.temporal_fwd(c_planes, B, 1, dk.hidden, self._reset.view(B, 1), state, self._fire, float(m.d_polarm_beta))
        doc = self._unpad(doc, 1)                                              # [B,H,9] fp32
        self.carry.copy_(doc.reshape(B, d.hidden, 3, 3))
        pooled = K.slot_pool_fwd(self.carry.view(B, 1, d.hidden, 9), cst["score_w"])   # [B,1,9]
        z = torch.addmm(cst["proj_b"], pooled.view(B, 9), cst["proj_wT"])
        return torch.addmm(cst["up_b"], z, cst["up_wT"]).to(self.dt)

    def _finish_fused(self, h, a_t) -> None:
        """Boundary-key append, final cross attention (the training plan's masked cross-attention kernel), head."""
        m, d, K, dk = self.m, self.d, self._K, self._dk
        B, cst = self.B, self._const
        from ..ops import native
        ext = native.ext()
        bf = dict(dtype=self.dt, device=self.dev)
        if a_t is not None:
            fca = m.tria_final_ca
            newk, newv, qv = (torch.empty(B, d.n, **bf) for _ in range(3))
            K.linear_multi([([a_t], self.w(fca.w_qk.weight), None, newk), ([a_t], self.w(fca.w_v.weight), None, newv),
                            ([h], self.w(fca.w_qk.weight), None, qv)], static_weights=True)
            ext.decode_ca_append(newk, newv, self._fire, self.ca_k, self.ca_v, self.ca_valid, self.ca_len, self._allowed,
                                 self._any, self.pending, self.have_carry)
            native.count()
            self.ca_len.add_(self._any)
            out = K.cross_attn_fwd(qv.view(B, 1, d.n), self.ca_k, self.ca_v, self._allowed.view(B, 1, self.ca_cap), fca.scale)
            h = torch.add(h, out.view(B, d.n), alpha=cst["gamma"])
        hn = K.rms_norm_fwd(h, m.ln_final.weight.data) if m.ln_final is not None else h
        K.linear_small(hn, self.w(m.head.weight), None, out=self.logits)
        self.next_tok.copy_(self.logits.argmax(-1))
        self.pos.add_(1)

    def _step_composed(self) -> None:
        m, d = self.m, self.d
        B, S, dt = self.B, self.S, self.dt
        pos = self.pos                                   # [1]
        h = self.w(m.emb.weight)[self.tok_in]            # [B, N]
        cos = m.rope_cos.index_select(0, pos).to(dt).view(1, 1, d.hd)
        sin = m.rope_sin.index_select(0, pos).to(dt).view(1, 1, d.hd)
        key_ok = (torch.arange(S, device=self.dev) <= pos).view(1, 1, S)
        da = m.depth_attn
        scale = 1.0 / math.sqrt(d.hd)

        def project(x):
            kv = self._lin(x, da.kv_weight)
            k, v = kv[:, :d.n].view(B, d.qh, d.hd), kv[:, d.n:].view(B, d.qh, d.hd)
            if d.depth_qkv_rms:
                k, v = R.fixed_rms(k, FANIN_GAIN), R.fixed_rms(v, FANIN_GAIN * d.deepnorm_beta)
            return k, v

        hist_k, hist_v = [], []
        k0, v0 = project(h)
        hist_k.append(k0); hist_v.append(v0)

        def read(sub):
            q = da.query(sub).to(dt)
            hk, hv = torch.stack(hist_k), torch.stack(hist_v)          # [n,B,QH,HD]
            wts = torch.softmax((hk.float() * q.float()).sum(-1) * scale, dim=0)
            mm = (wts.unsqueeze(-1) * hv.float()).sum(0).to(dt)
            return F.linear(mm.reshape(B, d.n), self.w(da.w_o_weight)[sub] if da.w_o is None else self.w(da.w_o.weight)), mm

        cap = (lambda t: R.capped_rms(t, d.branch_rms_cap)) if (d.branch_rms_cap is not None and m.decode_applies_rms_cap) else (lambda t: t)
        is_bos = pos.eq(0)
        seed_valid = self.pending & ~is_bos & self.have_carry
        carry_c, p_in = None, None
        use_tria = d.tria and not m.ablation
        for bi, blk in enumerate(m.blocks):
            last = bi == d.layers - 1
            qkv = self._lin(h, blk.attn.qkv_weight)
            q = R.apply_rope(qkv[:, :d.n].view(B, d.qh, d.hd), cos, sin)
            k = R.apply_rope(qkv[:, d.n:d.n + d.kv_dim].view(B, d.kvh, d.hd), cos, sin)
            v = qkv[:, d.n + d.kv_dim:].view(B, d.kvh, d.hd)
            self.kc[bi].index_copy_(1, pos, k.unsqueeze(1))
            self.vc[bi].index_copy_(1, pos, v.unsqueeze(1))
            if self._native_attn:
                from ..ops import native
                q = q.contiguous()
                c, k_ctx = torch.empty_like(q), torch.empty_like(q)
                native.ext().decode_attn(q, self.kc[bi], self.vc[bi], pos, c, k_ctx, self._attn_ws, B, S, d.qh, d.kvh,
                                         d.hd, self._ns, self._status)
                native.count(2 if self._ns > 1 else 1)
            else:
                kk = self.kc[bi].view(B, S, d.kvh, 1, d.hd).expand(B, S, d.kvh, d.group, d.hd).reshape(B, S, d.qh, d.hd)
                vv = self.vc[bi].view(B, S, d.kvh, 1, d.hd).expand(B, S, d.kvh, d.group, d.hd).reshape(B, S, d.qh, d.hd)
                sc = torch.einsum("bhd,bshd->bhs", q.float(), kk.float()) * scale
                a = torch.softmax(sc.masked_fill(~key_ok, float("-inf")), dim=-1)
                k_ctx = torch.einsum("bhs,bshd->bhd", a, kk.float()).to(dt)
                c = torch.einsum("bhs,bshd->bhd", a, vv.float()).to(dt)
            attn_out = self._lin(c.reshape(B, d.n), blk.attn.o.weight)
            sub = 2 * bi
            skip, _ = read(sub)
            u = F.layer_norm((cap(skip) + cap(attn_out)).float(), (d.n,), blk.ln_attn.weight, blk.ln_attn.bias).to(dt)
            ku, vu = project(u)
            hist_k.append(ku); hist_v.append(vu)
            skip2, d_sel = read(sub + 1)
            ffn = blk.ffn
            wx = self._lin(u, ffn.w1_real.weight)
            if ffn.identity_gate is not None and p_in is not None:
                r = wx * (1.0 + ffn.identity_gate.alpha().to(dt) * p_in) + self.w(ffn.w1_real.bias)
            else:
                r = wx + self.w(ffn.w1_real.bias)
            gsrc = self._lin(u, ffn.gate_proj.weight, ffn.gate_proj.bias) if ffn.gate_proj is not None else r
            w3 = self.w(ffn.w1_imag).view(d.qh, d.hpq, d.imag_in)
            if d.open_sectors:
                shared = torch.cat((k_ctx.reshape(B, d.n), c.reshape(B, d.n), u, d_sel.reshape(B, d.n)), -1)
                a_in = torch.cat((q, shared.unsqueeze(1).expand(B, d.qh, 4 * d.n)), -1)
            else:
                a_in = torch.cat((q, k_ctx, c, u.unsqueeze(1).expand(B, d.qh, d.n), d_sel), -1)
            beta = (torch.einsum("bgk,ghk->bgh", a_in, w3).reshape(B, d.hidden).float() + ffn.w1_imag_bias)
            s0 = torch.sin(R.HALF_PI * beta * torch.rsqrt(1.0 + beta * beta))
            prev = torch.where(is_bos, torch.zeros_like(self.trace[bi]), self.trace[bi])
            zz = s0 + prev * ffn.w1_imag_trace
            i_sq = zz * torch.rsqrt(1.0 + zz * zz)
            self.trace[bi].copy_(s0)
            amp = F.softplus(gsrc.float())
            rf = r.float()
            if m.ablation:
                p_act = rf + amp
            else:
                p_act = rf + amp * i_sq
            o = (p_act * R.powlu_gate(amp, d.powlu_m)) if d.activation == "pvpowlu" else (
                F.gelu(p_act) if d.activation == "gelu" else R.powlu(p_act, d.powlu_m))
            if use_tria:
                t3 = R.build_tria(rf, i_sq, o, m.tria_alpha, bi % 3)                      # [B,H,3,3]
                if bi == 0:
                    pre = torch.where(seed_valid[:, None, None, None], torch.matmul(t3, self.carry), t3)
                else:
                    pre = torch.matmul(t3, carry_c)
                carry_c = R.normalize9(pre)
                p_in = None if last else (carry_c.reshape(B, d.hidden, 9) * ffn.gate_selector.weights()).sum(-1).to(dt)
            f = self._lin(o.to(dt), ffn.w2.weight, ffn.w2.bias)
            h = F.layer_norm((cap(skip2) + cap(f)).float(), (d.n,), blk.ln_ffn.weight, blk.ln_ffn.bias).to(dt)
            if not last:
                kh, vh = project(h)
                hist_k.append(kh); hist_v.append(vh)
        self._finish_step(h, carry_c if use_tria else None, is_bos)

    def _finish_step(self, h, carry_c, is_bos) -> None:
        """Temporal endpoint, boundary-key append, final cross attention, head."""
        m, d = self.m, self.d
        B, S, dt = self.B, self.S, self.dt
        pos = self.pos
        use_tria = carry_c is not None
        if use_tria:
            reset_now = self.pending | is_bos | (not d.tria_temporal) | ~self.have_carry
            cont = R.normalize9(torch.matmul(carry_c, self.carry))
            doc = torch.where(reset_now[:, None, None, None], carry_c, cont)
            W = m.tria_window
            hard = ((pos + 1) % W == 0) & (pos + 1 < d.seq_len) & bool(m.tria_hard_fire_enabled)
            fire = hard.expand(B)
            if m.carry_token_id is not None:
                fire = fire | self.tok_in.eq(int(m.carry_token_id))
            doc = torch.where(fire[:, None, None, None], R.polarm(doc, m.d_polarm_beta), doc)
            fca, agg = m.tria_final_ca, m.tria_agg
            a_t = agg(doc.unsqueeze(1)).to(dt)[:, 0]                                   # [B,N]
            any_fire = fire.any()
            slot = self.ca_len.clamp(max=self.ca_cap - 1)
            newk, newv = self._lin(a_t, fca.w_qk.weight), self._lin(a_t, fca.w_v.weight)
            oldk, oldv = self.ca_k.index_select(1, slot), self.ca_v.index_select(1, slot)
            oldm = self.ca_valid.index_select(1, slot)
            self.ca_k.index_copy_(1, slot, torch.where(any_fire, newk.unsqueeze(1), oldk))
            self.ca_v.index_copy_(1, slot, torch.where(any_fire, newv.unsqueeze(1), oldv))
            self.ca_valid.index_copy_(1, slot, torch.where(any_fire, fire.unsqueeze(1), oldm))
            self.ca_len.add_(any_fire.long())
            allowed = self.ca_valid & (torch.arange(self.ca_cap, device=self.dev).view(1, -1) < self.ca_len)
            qv = self._lin(h, fca.w_qk.weight)
            out = R.masked_cross_attention(qv.float().unsqueeze(1), self.ca_k.float(), self.ca_v.float(),
                                           allowed.unsqueeze(1), fca.scale)[:, 0]
            h = (h.float() + fca.gamma() * out).to(dt)
            self.carry.copy_(doc)
            self.pending.copy_(fire)
            self.have_carry.fill_(True)
        hn = m.ln_final(h) if m.ln_final is not None else h
        self.logits.copy_(F.linear(hn.to(dt), self.w(m.head.weight)).float())
        self.next_tok.copy_(self.logits.argmax(-1))
        self.pos.add_(1)

    # ------------------------------------------------------------------ convenience
    def check_request(self, prompt_len: int, max_new: int) -> None:
        """Host-side admission check: the last generated token is fed at position ``prompt_len + max_new - 2``."""
        check_request(prompt_len, max_new, self.S)

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new: int) -> torch.Tensor:
        """Greedy continuation of an equal-length prompt batch; returns ``[B, max_new]`` token ids."""
        self.check_request(int(prompt.shape[1]), int(max_new))
        logits = self.prefill(prompt)
        tok = logits.argmax(-1)
        out = [tok]
        for _ in range(max_new - 1):
            self.step(tok)
            tok = self.next_tok.clone()
            out.append(tok)
        return torch.stack(out, dim=1)
