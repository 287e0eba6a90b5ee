"""LoomFormer model: embeddings -> L blocks (GQA + DepthAttn + Paraplex FFN + Tria) -> readout.

Execution plans
---------------
``forward``  training / scoring.  With Tria on, the sequence is cut at *fire boundaries*
             (every ``W`` tokens and at every ``<CARRY>`` column) and the whole block stack is
             run chunk by chunk, because layer 0 of chunk ``k+1`` is seeded with the temporal
             endpoint built from the last-layer carriers of chunk ``k``
             (reference ``loomformer.py:3788-3893``).
``_forward_flat``  one pass over the full sequence; legal when Tria is off, and used by the
             start-up calibration and the analysis tools (reference ``3895-3949``).
``step``     token-by-token decoding with fixed-size recurrent state plus KV caches
             (reference ``3951-4091``).
``prefill``  batched prompt ingestion that returns a decode state (not in the reference, whose
             prefill is token-by-token).

The math of each block lives in :meth:`Model._block`; the operator implementations come from an
``OpSet`` (``ops/opset.py``): pure PyTorch on CPU, fused sm_100a kernels on a B200.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint

from ..config import Config, Dims, resolve
from ..ops import reference as R
from . import rope as rope_mod
from .modules import Block, DepthAttn, RMSNorm, SharedTriaReader, TriaAggregator, TriaFinalCrossAttention


# ----------------------------------------------------------------------------- state containers
@dataclass
class LayerCache:
    k: Optional[torch.Tensor] = None            # [B, S, KVH, HD] preallocated
    v: Optional[torch.Tensor] = None
    phase_trace: Optional[torch.Tensor] = None  # [B, H]
    cache_len: int = 0


@dataclass
class TriaCACache:
    k: Optional[torch.Tensor] = None            # [B, S, N]
    v: Optional[torch.Tensor] = None
    carry_key_mask: Optional[torch.Tensor] = None  # [B, S] bool
    cache_len: int = 0


@dataclass
class TriaTemporalState:
    carry: Optional[torch.Tensor] = None           # [B, H, 3, 3]
    refeed_pending: Optional[torch.Tensor] = None  # [B] bool


@dataclass
class ChunkLayerState:
    """Per-layer state that crosses chunk boundaries during a chunked forward."""
    k_chunks: tuple = ()
    v_chunks: tuple = ()
    phase_trace: Optional[torch.Tensor] = None


_ckpt_anchor_tls: dict = {}


class Model(nn.Module):
    def __init__(self, cfg: Config, ablation: bool = False, dims: Optional[Dims] = None) -> None:
        super().__init__()
        self.cfg = cfg
        self.d = d = dims if dims is not None else resolve(cfg)
        self.ablation = bool(ablation)
        self.carry_token_id: Optional[int] = None
        self.emb = nn.Embedding(d.vocab, d.n)
        self.blocks = nn.ModuleList([Block(d, ablation=ablation) for _ in range(d.layers)])
        self.depth_attn = DepthAttn(d)
        self.head = nn.Linear(d.n, d.vocab, bias=False)
        if d.tied:
            self.head.weight = self.emb.weight
        self.ln_final = RMSNorm(d.n) if d.final_norm else None
        if d.tria:
            self.tria_agg: Optional[TriaAggregator] = TriaAggregator(SharedTriaReader(k=32), d.n)
            self.tria_final_ca: Optional[TriaFinalCrossAttention] = TriaFinalCrossAttention(
                d.n, gamma_max=d.tria_gamma_max, raw_gamma_init=d.tria_raw_gamma_init)
            # Block 0 never sees an incoming gate value and the last block never emits one.
            self.blocks[0].ffn.identity_gate.raw_alpha.requires_grad_(False)
            self.blocks[-1].ffn.gate_selector.logits.requires_grad_(False)
        else:
            self.tria_agg = None
            self.tria_final_ca = None
        with torch.no_grad():
            nn.init.normal_(self.emb.weight, mean=0.0, std=d.fanin_std(d.n))
        cos, sin = rope_mod.build_tables(d)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)
        # introspection surface used by the analysis tools
        self.tria_hard_fire_enabled = True
        self.capture_tria_depth_carry = False
        self.last_tria_depth_carry: Optional[torch.Tensor] = None
        self.last_tria_document_carry: Optional[torch.Tensor] = None
        self.last_tria_document_carry_stats: Optional[dict] = None
        self.last_tria_fire_mask: Optional[torch.Tensor] = None
        # decode applies the residual-branch RMS cap like training does; set False to mimic the
        # reference, whose ``step`` skips it.
        self.decode_applies_rms_cap = True
        self.ops = None   # lazily bound OpSet (see ops/opset.py)

    # ------------------------------------------------------------------ helpers
    @property
    def tria_alpha(self) -> float:
        return float(self.cfg.tria_carrier_alpha)

    @property
    def tria_window(self) -> int:
        return int(self.cfg.tria_temporal_window or self.d.seq_len)

    def _opset(self, x: torch.Tensor):
        from ..ops.opset import select_opset
        return select_opset(self, x)

    def _head_in(self, x: torch.Tensor) -> torch.Tensor:
        return self.head(self.ln_final(x) if self.ln_final is not None else x)

    def _rope(self, position_ids: torch.Tensor, dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        if position_ids.dim() == 1:
            position_ids = position_ids.unsqueeze(0)
        return (self.rope_cos[position_ids].to(dtype).unsqueeze(2),
                self.rope_sin[position_ids].to(dtype).unsqueeze(2))

    def _cap(self, x: torch.Tensor) -> torch.Tensor:
        cap = self.d.branch_rms_cap
        return x if cap is None else R.capped_rms(x, cap)

    @staticmethod
    def _doc_reset(position_ids: torch.Tensor) -> torch.Tensor:
        reset = position_ids.eq(0)
        reset[:, 0].fill_(True)          # fill_ takes the scalar as a kernel argument (no host-to-device copy)
        return reset

    # ------------------------------------------------------------------ attention (composed plan)
    def _attend(self, block: Block, z: torch.Tensor, past_k: Sequence[torch.Tensor],
                past_v: Sequence[torch.Tensor], position_ids: torch.Tensor, allowed: torch.Tensor):
        """QKV projection, RoPE, dual-context attention of this chunk against ``past + new`` keys."""
        d = self.d
        B, T, _ = z.shape
        q, k, v = F.linear(z, block.attn.qkv_weight).split((d.n, d.kv_dim, d.kv_dim), dim=-1)
        cos, sin = self._rope(position_ids, q.dtype)
        q = R.apply_rope(q.view(B, T, d.qh, d.hd), cos, sin)
        k = R.apply_rope(k.view(B, T, d.kvh, d.hd), cos, sin)
        v = v.view(B, T, d.kvh, d.hd)
        k_all = torch.cat((*past_k, k), dim=1) if past_k else k
        v_all = torch.cat((*past_v, v), dim=1) if past_v else v
        k_ctx, c = R.dual_context_attention(q, k_all, v_all, allowed, d.group)
        return block.attn.o(c.reshape(B, T, d.n)), q, k_ctx, c, k, v

    # ------------------------------------------------------------------ FFN (composed plan)
    def _ffn(self, block: Block, u, q, k_ctx, c, d_sel, trace, reset, p_in, anchor_override=None):
        d, ffn = self.d, block.ffn
        wx = F.linear(u, ffn.w1_real.weight)
        if ffn.identity_gate is not None:
            r = ffn.identity_gate(wx, ffn.w1_real.bias, p_in)
        else:
            r = wx + ffn.w1_real.bias
        gate_src = ffn.gate_proj(u) if ffn.gate_proj is not None else r
        if self.ablation:
            amp = F.softplus(gate_src)
            p = r + amp
            out = p * R.powlu_gate(amp, d.powlu_m) if d.activation == "pvpowlu" else (
                F.gelu(p) if d.activation == "gelu" else R.powlu(p, d.powlu_m))
            return ffn.w2(out), torch.ones(u.shape[0], d.hidden, device=u.device, dtype=u.dtype), None
        beta_lin = ffn.beta_linear(u, q, k_ctx, c, d_sel)
        anchor = None
        if d.phase_secant:
            if ffn.training and anchor_override is None:
                ffn.update_anchor(beta_lin + ffn.w1_imag_bias)
            anchor = ffn.beta_anchor if anchor_override is None else anchor_override
        out, i_sq, next_trace = R.paraplex_core(
            r, gate_src, beta_lin, ffn.w1_imag_bias, ffn.w1_imag_trace, trace, reset, anchor,
            floor=d.phase_floor, m=d.powlu_m, activation=d.activation)
        return ffn.w2(out), next_trace, (r, i_sq, out)

    # ------------------------------------------------------------------ one block
    def _block(self, bi: int, block: Block, h, hist_k: List[torch.Tensor], hist_v: List[torch.Tensor],
               attn_pack, position_ids, trace, carry_prev, p_in, seed, seed_valid, apply_cap=True,
               anchor_override=None):
        d, da = self.d, self.depth_attn
        attn_out, q, k_ctx, c = attn_pack
        B, T = h.shape[:2]
        last = bi == d.layers - 1
        sub = 2 * bi

        def read(s: int):
            m = R.depth_read(da.query(s).to(hist_k[0].dtype), torch.stack(hist_k), torch.stack(hist_v))
            return F.linear(m.reshape(B, T, d.n), da.readout_weight(s)), m

        cap = self._cap if apply_cap else (lambda t: t)
        skip, _ = read(sub)
        u = block.ln_attn(cap(skip) + cap(attn_out))
        k_i, v_i = da.project(u)
        hist_k, hist_v = [*hist_k, k_i], [*hist_v, v_i]
        skip, d_sel = read(sub + 1)
        reset = position_ids.eq(0) if position_ids is not None else None
        ffn_out, next_trace, rio = self._ffn(block, u, q, k_ctx, c, d_sel, trace, reset, p_in, anchor_override)
        carry_new, p_out = carry_prev, None
        if d.tria and not self.ablation:
            r, i_sq, o = rio
            gate_w = None if last else block.ffn.gate_selector.weights()
            axis = bi % 3
            if bi == 0:
                carry_new, p_out = R.tria_compose(r, i_sq, o, self.tria_alpha, axis, seed=seed,
                                                  seed_valid=seed_valid, gate_w=gate_w)
            else:
                carry_new, p_out = R.tria_compose(r, i_sq, o, self.tria_alpha, axis, prev=carry_prev,
                                                  gate_w=gate_w)
        h = block.ln_ffn(cap(skip) + cap(ffn_out))
        if not last:
            k_i, v_i = da.project(h)
            hist_k, hist_v = [*hist_k, k_i], [*hist_v, v_i]
        return h, hist_k, hist_v, next_trace, carry_new, p_out

    # ------------------------------------------------------------------ chunk stack (composed plan)
    def _run_chunk_stack_impl(self, h_emb, position_ids, allowed, layer_states, seed, seed_valid,
                              anchor_overrides=None):
        k0, v0 = self.depth_attn.project(h_emb)
        hist_k, hist_v = [k0], [v0]
        h, carry, p = h_emb, None, None
        new_k, new_v, traces = [], [], []
        for bi, block in enumerate(self.blocks):
            ls = layer_states[bi]
            attn_out, q, k_ctx, c, k_new, v_new = self._attend(block, h, ls.k_chunks, ls.v_chunks,
                                                               position_ids, allowed)
            ov = None if anchor_overrides is None else anchor_overrides[bi]
            h, hist_k, hist_v, tr, carry, p = self._block(
                bi, block, h, hist_k, hist_v, (attn_out, q, k_ctx, c), position_ids,
                ls.phase_trace, carry, p, seed, seed_valid, anchor_override=ov)
            new_k.append(k_new); new_v.append(v_new); traces.append(tr)
        return (h, carry, *new_k, *new_v, *traces)

    def _run_chunk_stack(self, h_emb, position_ids, allowed, layer_states, seed, seed_valid):
        """Run all blocks over one temporal chunk.  Returns ``(h, last_layer_carry, new_layer_states)``."""
        L = self.d.layers
        if self.d.grad_checkpointing and self.training and torch.is_grad_enabled():
            # The first pass updates each layer's anchor EMA once and evaluates the phase slope with
            # the updated value; the recompute must reuse exactly that value and leave the EMA alone.
            holder: dict = {}

            def body(h_emb_, pos_, allowed_, seed_, seed_valid_):
                return self._run_chunk_stack_impl(h_emb_, pos_, allowed_, layer_states, seed_, seed_valid_,
                                                  holder.get("snap"))
            flat = torch.utils.checkpoint.checkpoint(body, h_emb, position_ids, allowed, seed, seed_valid,
                                                     use_reentrant=False)
            holder["snap"] = [b.ffn.beta_anchor.detach().clone() for b in self.blocks]
        else:
            flat = self._run_chunk_stack_impl(h_emb, position_ids, allowed, layer_states, seed, seed_valid)
        h, carry = flat[0], flat[1]
        ks, vs, trs = flat[2:2 + L], flat[2 + L:2 + 2 * L], flat[2 + 2 * L:2 + 3 * L]
        states = [ChunkLayerState(layer_states[i].k_chunks + (ks[i],), layer_states[i].v_chunks + (vs[i],), trs[i])
                  for i in range(L)]
        return h, carry, states

    # ------------------------------------------------------------------ fire plan
    def fire_plan(self, idx: torch.Tensor, position_ids: torch.Tensor, last_may_fire: bool = False, cuts=None):
        """Reset mask, fire mask and the sorted list of cut columns for a chunked forward.

        A row fires at column ``i`` when ``(i+1) % W == 0`` (never at the last column, and not when
        column ``i+1`` starts a new document) or when token ``i`` is ``<CARRY>``.  Chunks are cut at
        the union over the batch of firing columns.
        """
        B, T = idx.shape
        W = self.tria_window
        reset = self._doc_reset(position_ids)
        if self.carry_token_id is not None:
            explicit = idx.eq(int(self.carry_token_id))
        else:
            explicit = torch.zeros(B, T, dtype=torch.bool, device=idx.device)
        if self.tria_hard_fire_enabled:
            ar = torch.arange(T, device=idx.device)
            grid = (ar + 1).remainder(W).eq(0)
            # A training sequence never fires at its last index.  A prompt that will be continued by the decoder
            # does (the decoder's rule: fire when the next position starts a new window and still fits).
            last_fires = bool(last_may_fire and T < self.d.seq_len and T % W == 0)      # known on the host
            if not last_fires:
                grid = grid & ar.ne(T - 1)          # device-side: a scalar store would be a host-to-device copy
        else:
            grid = torch.zeros(T, dtype=torch.bool, device=idx.device)
            last_fires = False
        next_reset = torch.zeros_like(reset)
        next_reset[:, :-1] = reset[:, 1:]
        fire = (grid.view(1, T) & ~next_reset) | explicit
        if cuts is not None:
            cuts = list(cuts)                       # the caller already knows them (no device read-back here)
        elif self.carry_token_id is None:
            cuts = list(range(W - 1, T - 1, W)) if self.tria_hard_fire_enabled else []
            if last_fires:
                cuts.append(T - 1)
        else:
            cuts = (grid | explicit.any(dim=0)).nonzero().flatten().tolist()
        return reset, fire, cuts

    # ------------------------------------------------------------------ forward
    def forward(self, idx: torch.Tensor, attn_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, T = idx.shape
        if T > self.d.seq_len:
            raise ValueError(f"input length {T} exceeds configured seq_len {self.d.seq_len}")
        if position_ids is None:
            position_ids = torch.arange(T, device=idx.device).view(1, T).expand(B, T)
        else:
            position_ids = position_ids.to(device=idx.device, dtype=torch.long)
        ops = self._opset(self.emb.weight)
        if ops is not None and attn_mask is None and not torch.is_grad_enabled() and not self.ablation:
            return ops.run(idx, None, position_ids, None, want_grad=False)[1].float()
        if self.d.tria and self.d.tria_temporal and not self.ablation:
            return self._forward_chunked(idx, attn_mask, position_ids)
        return self._forward_flat(idx, attn_mask, position_ids)

    def _forward_chunked(self, idx, attn_mask, position_ids) -> torch.Tensor:
        B, T = idx.shape
        h_emb = self.emb(idx)
        reset, fire, cuts = self.fire_plan(idx, position_ids)
        cut_set = set(cuts)
        causal = torch.ones(T, T, dtype=torch.bool, device=idx.device).tril()
        states = [ChunkLayerState() for _ in self.blocks]
        h_parts, keys, key_depth, key_valid, key_pos = [], [], [], [], []
        temporal = None
        s = 0
        for bp in cuts + ([T - 1] if not cuts or cuts[-1] != T - 1 else []):
            e = min(bp + 1, T)
            if e <= s:
                continue
            allowed = causal[s:e, :e].view(1, 1, e - s, e)
            if attn_mask is not None:
                allowed = allowed & attn_mask[:, :, s:e, :e]
            seed, seed_valid = None, None
            if temporal is not None:
                seed, seed_valid = temporal, fire[:, s - 1] & ~reset[:, s]
            h_c, depth_c, states = self._run_chunk_stack(h_emb[:, s:e], position_ids[:, s:e], allowed,
                                                         states, seed, seed_valid)
            local_reset = reset[:, s:e].clone()
            if seed_valid is not None:
                local_reset[:, 0] |= seed_valid
            # The tail chunk's endpoint feeds nothing (it never fires and has no successor).
            if e != T or (e - 1) in cut_set:
                temporal = R.temporal_endpoint(depth_c, local_reset, temporal)
            h_parts.append(h_c)
            if (e - 1) in cut_set:
                fired = fire[:, e - 1]
                fixed = R.polarm(temporal, self.d_polarm_beta)
                temporal = torch.where(fired[:, None, None, None], fixed, temporal)
                keys.append(temporal); key_depth.append(depth_c[:, -1]); key_valid.append(fired); key_pos.append(e - 1)
            s = e
        if s != T:
            raise RuntimeError(f"chunk boundaries stopped at {s}, expected {T}")
        h = torch.cat(h_parts, dim=1)
        self.last_tria_fire_mask = fire
        self.last_tria_document_carry_stats = None
        self.last_tria_depth_carry = self.last_tria_document_carry = None
        if not keys:
            return self._head_in(h)
        doc_keys, valid = torch.stack(keys, dim=1), torch.stack(key_valid, dim=1)
        pos = torch.tensor(key_pos, device=idx.device, dtype=torch.long)
        if self.capture_tria_depth_carry:
            self.last_tria_depth_carry = torch.stack(key_depth, dim=1).detach()
            self.last_tria_document_carry = doc_keys.detach()
        h = self._final_readout(h, doc_keys, valid, pos, attn_mask)
        return self._head_in(h)

    @property
    def d_polarm_beta(self) -> float:
        return float(self.cfg.tria_polarm_beta)

    def _final_readout(self, h, doc_keys, valid, key_pos, attn_mask):
        """Aggregate boundary carriers to keys and cross-attend: key allowed iff its position <= t,
        it fired in this row, and the packing mask lets token t see that position."""
        B, T = h.shape[:2]
        K = key_pos.numel()
        a = self.tria_agg(doc_keys)
        allowed = key_pos.view(1, 1, K) <= torch.arange(T, device=h.device).view(1, T, 1)
        allowed = allowed & valid[:, None, :]
        if attn_mask is not None:
            m3 = attn_mask.squeeze(1) if attn_mask.dim() == 4 else attn_mask
            allowed = allowed & torch.gather(m3.expand(B, T, T), 2, key_pos.view(1, 1, K).expand(B, T, K))
        return self.tria_final_ca(a, h, allowed)

    def _forward_flat(self, idx, attn_mask=None, position_ids=None) -> torch.Tensor:
        B, T = idx.shape
        if position_ids is None:
            position_ids = torch.arange(T, device=idx.device).view(1, T).expand(B, T)
        h = self.emb(idx)
        allowed = torch.ones(T, T, dtype=torch.bool, device=idx.device).tril().view(1, 1, T, T)
        if attn_mask is not None:
            allowed = attn_mask
        k0, v0 = self.depth_attn.project(h)
        hist_k, hist_v, carry, p = [k0], [v0], None, None
        for bi, block in enumerate(self.blocks):
            attn_out, q, k_ctx, c, _, _ = self._attend(block, h, (), (), position_ids, allowed)
            h, hist_k, hist_v, _, carry, p = self._block(
                bi, block, h, hist_k, hist_v, (attn_out, q, k_ctx, c), position_ids, None, carry, p, None, None)
        self.last_tria_depth_carry = None
        self.last_tria_document_carry_stats = None
        self.last_tria_fire_mask = None
        if carry is not None:
            if self.capture_tria_depth_carry:
                self.last_tria_depth_carry = carry.detach()
            reset = self._doc_reset(position_ids)
            doc = R.temporal_scan(carry, reset) if self.d.tria_temporal else carry
            hard = (position_ids + 1) % self.tria_window == 0
            nxt = torch.zeros_like(hard)
            if T > 1:
                nxt[:, :-1] = reset[:, 1:]
            key_mask = hard & ~nxt
            self.last_tria_fire_mask = key_mask
            with torch.no_grad():
                self.last_tria_document_carry_stats = {
                    "max_abs": float(doc.detach().abs().amax()), "reset_count": int(reset.sum()),
                    "fire_count": int(key_mask.sum())}
            active = key_mask.any(dim=0).nonzero().flatten()
            if active.numel():
                h = self._final_readout(h, doc.index_select(1, active).to(h.dtype),
                                        key_mask.index_select(1, active), active, attn_mask)
        return self._head_in(h)

    # ------------------------------------------------------------------ incremental decoding
    @torch.no_grad()
    def step(self, idx_t: torch.Tensor, pos_t: int, states):
        """Advance every sequence of the batch by one token at shared position ``pos_t``.

        ``states`` is ``None`` or the tuple returned by the previous call
        ``(layer_caches, final_ca_cache, temporal_state)``; ``pos_t == 0`` restarts everything.
        Returns ``(logits [B,V], states)``.
        """
        ops = self._opset(self.emb.weight)
        if ops is not None and hasattr(ops, "step"):
            return ops.step(self, idx_t, pos_t, states)
        return self._step_composed(idx_t, pos_t, states)

    def _step_composed(self, idx_t, pos_t, states):
        d = self.d
        bos = pos_t == 0
        caches = ca = ts = None
        if states is not None and not bos:
            caches, ca = states[0], states[1]
            ts = states[2] if len(states) > 2 else None
        caches = caches or [LayerCache() for _ in range(d.layers)]
        ca = ca or TriaCACache()
        ts = ts or TriaTemporalState()
        B = idx_t.shape[0]
        dev = idx_t.device
        h = self.emb(idx_t).view(B, 1, d.n)
        pos = torch.full((1, 1), int(pos_t), device=dev, dtype=torch.long)
        k0, v0 = self.depth_attn.project(h)
        hist_k, hist_v = [k0], [v0]
        pending = torch.zeros(B, dtype=torch.bool, device=dev) if ts.refeed_pending is None else ts.refeed_pending.to(dev)
        seed_valid = pending & (not bos)
        seed = ts.carry
        carry = p = None
        new_caches = []
        for bi, (block, cache) in enumerate(zip(self.blocks, caches)):
            if cache.cache_len >= d.seq_len:
                raise ValueError(f"generation exceeded seq_len={d.seq_len}; no wraparound support")
            if cache.k is None:
                cache.k = h.new_zeros(B, d.seq_len, d.kvh, d.hd)
                cache.v = h.new_zeros(B, d.seq_len, d.kvh, d.hd)
            n_past = cache.cache_len
            allowed = torch.ones(1, 1, 1, n_past + 1, dtype=torch.bool, device=dev)
            attn_out, q, k_ctx, c, k_new, v_new = self._attend(
                block, h, (cache.k[:, :n_past],) if n_past else (), (cache.v[:, :n_past],) if n_past else (),
                pos, allowed)
            cache.k[:, n_past] = k_new[:, 0]
            cache.v[:, n_past] = v_new[:, 0]
            h, hist_k, hist_v, tr, carry, p = self._block(
                bi, block, h, hist_k, hist_v, (attn_out, q, k_ctx, c), None, cache.phase_trace, carry, p,
                seed.to(h.dtype) if (seed is not None) else None, seed_valid,
                apply_cap=self.decode_applies_rms_cap)
            new_caches.append(LayerCache(cache.k, cache.v, tr, n_past + 1))
        self.last_tria_document_carry_stats = None
        if carry is not None:
            depth_t = carry[:, 0]
            reset_now = pending | bos | (not d.tria_temporal)
            if ts.carry is None:
                doc_t = depth_t
            else:
                cont = R.normalize9(torch.matmul(depth_t, ts.carry.to(device=dev, dtype=depth_t.dtype)))
                doc_t = torch.where(reset_now[:, None, None, None], depth_t, cont)
            hard = bool(self.tria_hard_fire_enabled and pos_t + 1 < d.seq_len
                        and (pos_t + 1) % self.tria_window == 0)
            if self.carry_token_id is not None:
                explicit = idx_t.view(-1).eq(int(self.carry_token_id))
            else:
                explicit = torch.zeros(B, dtype=torch.bool, device=dev)
            fire = explicit | hard
            if hard or (self.carry_token_id is not None and bool(explicit.any())):
                doc_t = torch.where(fire[:, None, None, None], R.polarm(doc_t, self.d_polarm_beta), doc_t)
            h, ca = self._final_ca_step(doc_t, h, ca, fire)
            ts = TriaTemporalState(carry=doc_t, refeed_pending=fire)
        return self._head_in(h[:, -1, :]), (new_caches, ca, ts)

    def _final_ca_step(self, doc_t, h, ca: TriaCACache, fire: torch.Tensor):
        d, fca = self.d, self.tria_final_ca
        B = h.shape[0]
        if ca.k is None:
            ca = TriaCACache(h.new_zeros(B, d.seq_len, d.n), h.new_zeros(B, d.seq_len, d.n),
                             torch.zeros(B, d.seq_len, dtype=torch.bool, device=h.device), 0)
        n = int(ca.cache_len)
        if bool(fire.any()):
            a_t = self.tria_agg(doc_t.unsqueeze(1)).to(h.dtype)
            ca.k[:, n] = fca.w_qk(a_t)[:, 0]
            ca.v[:, n] = fca.w_v(a_t)[:, 0]
            ca.carry_key_mask[:, n] = fire
            n += 1
        ca = TriaCACache(ca.k, ca.v, ca.carry_key_mask, n)
        if n == 0:
            return h, ca
        out = R.masked_cross_attention(fca.w_qk(h), ca.k[:, :n], ca.v[:, :n], ca.carry_key_mask[:, None, :n], fca.scale)
        return h + fca.gamma().to(out.dtype) * out, ca

    @torch.no_grad()
    def prefill(self, idx: torch.Tensor):
        """Ingest an equal-length prompt batch in one chunked pass and return
        ``(logits of the last position [B,V], states)`` ready for :meth:`step` at ``pos = T``.

        Equivalent to calling :meth:`step` for positions ``0..T-1`` (tested), but runs the prompt
        through the chunked training plan so the work is batched over tokens.
        """
        ops = self._opset(self.emb.weight)
        if ops is not None and hasattr(ops, "prefill"):
            return ops.prefill(self, idx)
        states, logits = None, None
        for t in range(idx.shape[1]):
            logits, states = self._step_composed(idx[:, t], t, states)
        return logits, states

    # ------------------------------------------------------------------ misc
    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())
