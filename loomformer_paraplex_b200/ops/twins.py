"""PyTorch twins of the fused sm_100a kernels.

Every kernel the fused execution plan launches has a twin here with the *same signature and the
same saved-tensor contract*, written with ordinary PyTorch ops.  The twins serve two purposes:

* the fused plan (hand-written forward and backward over whole temporal chunks) can be run and
  checked on a CPU against plain autograd of the composed model;
* each CUDA kernel is unit-tested on a B200 against its twin evaluated in fp32.

Backward twins recompute the forward under autograd and differentiate it, which keeps them
obviously consistent with ``ops/reference.py``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import reference as R


def _f(x):
    return x.float() if x is not None else None


class TorchKernels:
    """Reference implementation of the kernel interface (any device, any float dtype)."""

    name = "torch"

    # ------------------------------------------------------------------ GEMMs
    def linear(self, x, w, bias=None, out_dtype=None, out=None):
        """``x @ w^T (+ bias)``; with ``out`` the product is written into that buffer and the buffer returned."""
        y = F.linear(x, w.to(x.dtype))
        if bias is not None:
            y = y + bias.to(y.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y if out_dtype is None else y.to(out_dtype)

    def linear_small(self, x, w, bias=None, out=None, out_dtype=None):
        y = F.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
        if out_dtype is not None:
            y = y.to(out_dtype)
        if out is None:
            return y
        out.copy_(y)
        return out

    def linear_multi(self, segs, static_weights=False):
        """Several independent ``out = cat(pieces, -1) @ w^T (+ bias)`` products that wait for the same producers;
        ``segs``: ``(pieces, w, bias or None, out)`` with ``out`` a ``[M, N]`` view that is written in place."""
        for pieces, w, bias, out in segs:
            x = pieces[0] if len(pieces) == 1 else torch.cat(list(pieces), -1)
            out.copy_(F.linear(x.float(), w.float(), None if bias is None else bias.float()))

    def linear_dgrad(self, dy, w, out=None, accumulate=False):
        r = dy @ w.to(dy.dtype)
        if out is None:
            return r
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r)
        return out

    def linear_dgrad_multi(self, segs):
        """``sum_i dy_i @ w_i`` over segments ``(dy_i [M, K_i], w_i [K_i, N])``; a segment ``(None, value)`` contributes
        an already formed ``[M, N]`` term.  The native kernel set runs all products as one launch."""
        acc = None
        for dy, w in segs:
            r = w if dy is None else dy @ w.to(dy.dtype)
            acc = r if acc is None else acc + r.to(acc.dtype)
        return acc

    def linear_wgrad(self, dy, x, gw):
        gw.add_((dy.reshape(-1, dy.shape[-1]).float().t() @ x.reshape(-1, x.shape[-1]).float()).view_as(gw))

    def colsum_add(self, dy, gb):
        gb.add_(dy.reshape(-1, dy.shape[-1]).float().sum(0))

    # ------------------------------------------------------------------ imaginary projection
    @staticmethod
    def _imag_operand(d, qkc, u, m2):
        """Per-head operand [M, QH, IMAG_IN] in the storage order of ``w1_imag``."""
        M = u.shape[0]
        q, kc, c = qkc[:, 0], qkc[:, 1], qkc[:, 2]
        if d.open_sectors:
            shared = torch.cat((kc.reshape(M, d.n), c.reshape(M, d.n), u, m2.reshape(M, d.n)), -1)
            return torch.cat((q, shared.unsqueeze(1).expand(M, d.qh, 4 * d.n)), -1)
        return torch.cat((q, kc, c, u.unsqueeze(1).expand(M, d.qh, d.n), m2), -1)

    def imag_fwd(self, d, qkc, u, m2, w_imag):
        a = self._imag_operand(d, qkc, u, m2)
        w = w_imag.view(d.qh, d.hpq, d.imag_in).to(a.dtype)
        return torch.einsum("mgk,ghk->mgh", a, w).reshape(u.shape[0], d.hidden)

    def imag_bwd(self, d, dbeta, qkc, u, m2, w_imag, gw_imag, du_acc=None, defer_u=False):
        """Returns (dqkc, du, dm2) and accumulates the weight gradient into ``gw_imag`` (fp32); ``du`` includes
        ``du_acc`` when that is given.  ``defer_u``: do not form the gradient of ``u`` here; return it as a fourth
        element, a segment for :meth:`linear_dgrad_multi`, so the caller can fold it into one launch with the other
        products that end in the same tensor."""
        dqkc, du, dm2 = self._imag_bwd(d, dbeta, qkc, u, m2, w_imag, gw_imag)
        if defer_u:
            return dqkc, None, dm2, (None, du)
        return dqkc, (du if du_acc is None else du_acc + du.to(du_acc.dtype)), dm2

    def _imag_bwd(self, d, dbeta, qkc, u, m2, w_imag, gw_imag):
        M = u.shape[0]
        a = self._imag_operand(d, qkc, u, m2)
        w = w_imag.view(d.qh, d.hpq, d.imag_in).to(a.dtype)
        db = dbeta.view(M, d.qh, d.hpq)
        gw_imag.add_(torch.einsum("mgh,mgk->ghk", db.float(), a.float()).reshape_as(gw_imag))
        da = torch.einsum("mgh,ghk->mgk", db, w)
        hd, n = d.hd, d.n
        dqkc = torch.zeros_like(qkc)
        if d.open_sectors:
            dqkc[:, 0] = da[..., :hd]
            sh = da[..., hd:].sum(1)
            dqkc[:, 1] = sh[:, :n].view(M, d.qh, hd)
            dqkc[:, 2] = sh[:, n:2 * n].view(M, d.qh, hd)
            return dqkc, sh[:, 2 * n:3 * n], sh[:, 3 * n:].reshape(M, d.qh, hd)
        dqkc[:, 0], dqkc[:, 1], dqkc[:, 2] = da[..., :hd], da[..., hd:2 * hd], da[..., 2 * hd:3 * hd]
        return dqkc, da[..., 3 * hd:3 * hd + n].sum(1), da[..., 3 * hd + n:]

    # ------------------------------------------------------------------ rope + cache
    def rope_store(self, d, qkv, cos, sin, qkc, kcache, vcache, s):
        """qkv [B,Tc,N+2KV]; cos/sin [B,Tc,HD]; writes rotated q into qkc[:,0] and k,v into the
        caches at rows [s, s+Tc)."""
        B, Tc, _ = qkv.shape
        q, k, v = qkv.split((d.n, d.kv_dim, d.kv_dim), -1)
        c, s_ = cos.unsqueeze(2).to(qkv.dtype), sin.unsqueeze(2).to(qkv.dtype)
        qkc.view(B, Tc, 3, d.qh, d.hd)[:, :, 0] = R.apply_rope(q.view(B, Tc, d.qh, d.hd), c, s_)
        kcache[:, s:s + Tc] = R.apply_rope(k.view(B, Tc, d.kvh, d.hd), c, s_)
        vcache[:, s:s + Tc] = v.view(B, Tc, d.kvh, d.hd)

    def qkv_rope(self, d, x, w, cos, sin, qkc, kcache, vcache, s):
        """[Q | K | V] projection of ``x`` [B*Tc, N] followed by :meth:`rope_store`: rotated Q into ``qkc[:, 0]``, rotated
        K and V into the caches at rows [s, s+Tc)."""
        B, Tc = cos.shape[:2]
        self.rope_store(d, self.linear(x, w).view(B, Tc, -1), cos, sin, qkc, kcache, vcache, s)

    def rope_bwd(self, d, dq_attn, dqkc, dkc, dvc, s, e, cos, sin, out_dtype):
        """Inverse rotation of the q / k gradients and packing into d(qkv) [B,Tc,N+2KV].  The q gradient is the
        attention part plus sector 0 of ``dqkc``; k/v gradients are rows [s,e) of the fp32 cache gradients."""
        B, Tc = dq_attn.shape[:2]
        dq = dq_attn.float() + dqkc[:, 0].reshape(B, Tc, d.qh, d.hd).float()
        dk, dv = dkc[:, s:e], dvc[:, s:e]
        c, s_ = cos.unsqueeze(2).float(), sin.unsqueeze(2).float()

        def inv(g):
            g = g.float()
            return g * c - R.rotate_half(g * s_)
        return torch.cat((inv(dq).reshape(B, Tc, d.n), inv(dk).reshape(B, Tc, d.kv_dim),
                          dv.float().reshape(B, Tc, d.kv_dim)), -1).to(out_dtype)

    # ------------------------------------------------------------------ attention
    @staticmethod
    def _allowed(Tc, s, e, seg, device):
        qpos = torch.arange(s, e, device=device).view(1, 1, Tc, 1)
        kpos = torch.arange(e, device=device).view(1, 1, 1, e)
        ok = kpos <= qpos
        if seg is not None:
            ok = ok & (seg[:, None, s:e, None] == seg[:, None, None, :e])
        return ok

    def alloc_kv_grad(self, d, B, T, device):
        """fp32 accumulator for key/value gradients of one layer's cache."""
        return torch.zeros(B, T, d.kvh, d.hd, dtype=torch.float32, device=device)

    def attn_fwd(self, d, qkc, kcache, vcache, s, e, seg):
        """Dual-context attention of the chunk's queries against cache rows [0,e).  Fills
        qkc[:,1] (A@K) and qkc[:,2] (A@V); returns log-sum-exp [B,QH,Tc] (fp32)."""
        B, Tc = kcache.shape[0], e - s
        v5 = qkc.view(B, Tc, 3, d.qh, d.hd)
        q = v5[:, :, 0].transpose(1, 2).float()
        k = kcache[:, :e].repeat_interleave(d.group, 2).transpose(1, 2).float()
        v = vcache[:, :e].repeat_interleave(d.group, 2).transpose(1, 2).float()
        sc = (q @ k.transpose(-1, -2)) / math.sqrt(d.hd)
        sc = sc.masked_fill(~self._allowed(Tc, s, e, seg, q.device), float("-inf"))
        lse = torch.logsumexp(sc, -1)
        p = torch.exp(sc - lse.unsqueeze(-1))
        v5[:, :, 1] = (p @ k).transpose(1, 2).to(qkc.dtype)
        v5[:, :, 2] = (p @ v).transpose(1, 2).to(qkc.dtype)
        return lse

    def attn_bwd(self, d, dqkc, qkc, kcache, vcache, lse, s, e, seg, dkcache, dvcache):
        """Returns dq [B,Tc,QH,HD] (attention part only) and accumulates the key/value gradients of
        cache rows [0,e) into the fp32 buffers ``dkcache`` / ``dvcache``."""
        B, Tc = kcache.shape[0], e - s
        v5, g5 = qkc.view(B, Tc, 3, d.qh, d.hd), dqkc.view(B, Tc, 3, d.qh, d.hd)
        q = v5[:, :, 0].transpose(1, 2).float()
        k = kcache[:, :e].repeat_interleave(d.group, 2).transpose(1, 2).float()
        v = vcache[:, :e].repeat_interleave(d.group, 2).transpose(1, 2).float()
        dok, dov = g5[:, :, 1].transpose(1, 2).float(), g5[:, :, 2].transpose(1, 2).float()
        ok_, ov_ = v5[:, :, 1].transpose(1, 2).float(), v5[:, :, 2].transpose(1, 2).float()
        scale = 1.0 / math.sqrt(d.hd)
        sc = (q @ k.transpose(-1, -2)) * scale
        sc = sc.masked_fill(~self._allowed(Tc, s, e, seg, q.device), float("-inf"))
        p = torch.exp(sc - lse.unsqueeze(-1))
        dp = dov @ v.transpose(-1, -2) + dok @ k.transpose(-1, -2)
        delta = (dov * ov_).sum(-1, keepdim=True) + (dok * ok_).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = (ds @ k).transpose(1, 2)
        dk = ds.transpose(-1, -2) @ q + p.transpose(-1, -2) @ dok           # [B,QH,e,HD]
        dv = p.transpose(-1, -2) @ dov
        dkcache[:, :e].add_(dk.view(B, d.kvh, d.group, e, d.hd).sum(2).transpose(1, 2))
        dvcache[:, :e].add_(dv.view(B, d.kvh, d.group, e, d.hd).sum(2).transpose(1, 2))
        return dq.to(qkc.dtype)

    # ------------------------------------------------------------------ depth attention
    def dread_fwd(self, d, q_row, hist_k, hist_v, n):
        """q_row [QH,HD] fp32; hist_* [S,M,QH,HD]; uses states [0,n).  Returns (m [M,QH,HD], lse [M,QH])."""
        k, v = hist_k[:n].float(), hist_v[:n].float()
        sc = (k * q_row.float()).sum(-1) / math.sqrt(d.hd)
        lse = torch.logsumexp(sc, 0)
        w = torch.exp(sc - lse)
        return (w.unsqueeze(-1) * v).sum(0).to(hist_v.dtype), lse

    def dread_bwd(self, d, dm, m, lse, q_row, hist_k, hist_v, n, dhist_k, dhist_v, gq):
        """Accumulates into dhist_k/dhist_v [S,M,QH,HD] (fp32) and gq [QH,HD] (fp32)."""
        k, v, dmf = hist_k[:n].float(), hist_v[:n].float(), dm.float()
        inv = 1.0 / math.sqrt(d.hd)
        w = torch.exp((k * q_row.float()).sum(-1) * inv - lse)
        dw = (v * dmf).sum(-1) - (dmf * m.float()).sum(-1)
        dsc = w * dw * inv
        dhist_v[:n].add_(w.unsqueeze(-1) * dmf)
        dhist_k[:n].add_(dsc.unsqueeze(-1) * q_row.float())
        gq.add_((dsc.unsqueeze(-1) * k).sum((0, 1)))

    def dread_stage(self, d, a, b, m, lse, dst, sub):
        """Stage sublayer ``sub``'s read gradient: ``dm[sub] = a (+ b)``, ``dd[sub] = <dm, m>``, ``lse[sub] = lse``."""
        dm = a if b is None else a + b
        dst["dm"][sub] = dm.to(dst["dm"].dtype)
        dst["dd"][sub] = (dst["dm"][sub].float() * m.float()).sum(-1)
        dst["lse"][sub] = lse

    def dread_slot_bwd(self, d, slot, q_all, hist_k, hist_v, dm_all, lse_all, dd_all, gq_all):
        """Gradient of history slot ``slot`` summed over the sublayers ``slot..S-1`` that read it -> [M,2,QH,HD]
        (index 0: dK, index 1: dV, i.e. rows [dK | dV] as the K/V projection's gradient wants them); adds those
        sublayers' query gradients into ``gq_all``."""
        inv = 1.0 / math.sqrt(d.hd)
        k, v = hist_k[slot].float(), hist_v[slot].float()
        q, dmf = q_all[slot:].float(), dm_all[slot:].float()
        w = torch.exp(torch.einsum("mgh,ngh->nmg", k, q) * inv - lse_all[slot:])
        dsc = w * ((dmf * v).sum(-1) - dd_all[slot:]) * inv
        gq_all[slot:].add_(torch.einsum("nmg,mgh->ngh", dsc, k))
        dk = torch.einsum("nmg,ngh->mgh", dsc, q)
        dv = (w.unsqueeze(-1) * dmf).sum(0)
        return torch.stack((dk, dv), 1).to(hist_k.dtype)

    def fixed_rms_fwd(self, x, target):
        return R.fixed_rms(x, target)

    def fixed_rms_bwd(self, dy, x, target, eps=1e-6):
        xf, g = x.float(), dy.float()
        r = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
        return (target * r * (g - xf * r * r * (g * xf).mean(-1, keepdim=True)))

    def anchor_update(self, beta_sq_sum, n_el, anchor, decay):
        """In-place running radius ``anchor <- decay * anchor + (1 - decay) * max(sqrt(beta_sq_sum / n_el), 1e-4)``;
        returns a snapshot of the updated value (reference: loomformer.py:2866-2872, the beta-anchor EMA)."""
        rad = (beta_sq_sum / n_el).sqrt().clamp_min(1e-4)
        anchor.mul_(decay).add_(rad.to(anchor.dtype), alpha=1.0 - decay)
        return anchor.detach().clone()

    def zeros(self, *shape, device=None):
        """fp32 zeros; a kernel set may carve them out of one buffer cleared once per step (:meth:`begin_step`)."""
        return torch.zeros(*shape, dtype=torch.float32, device=device)

    def begin_step(self, zero_floats: int, device) -> None:
        """Called at the start of a step with an upper bound on the fp32 zeros the step will ask for."""

    def flush_wgrads(self) -> None:
        """Issue any weight-gradient products that a kernel set queued for grouping (nothing is queued here)."""

    # ------------------------------------------------------------------ add + (cap) + LayerNorm
    def add_ln_fwd(self, a, b, w, bias, cap, eps=1e-5):
        """y = LN(cap(a) + cap(b)).  Returns (y, x, mean, rstd) with x the pre-norm sum."""
        if cap is not None:
            a, b = R.capped_rms(a, cap), R.capped_rms(b, cap)
        x = a + b
        xf = x.float()
        mean = xf.mean(-1, keepdim=True)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + eps)
        y = ((xf - mean) * rstd * w.float() + bias.float()).to(x.dtype)
        return y, x, mean.squeeze(-1), rstd.squeeze(-1)

    def add_ln_bwd(self, dy, x, mean, rstd, w, gw, gb, cap, a, b):
        """Returns (da, db); LayerNorm weight/bias gradients are accumulated into gw, gb (fp32)."""
        g, xf = dy.float(), x.float()
        xh = (xf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1)
        gw.add_((g * xh).sum(0)); gb.add_(g.sum(0))
        gx = g * w.float()
        dx = rstd.unsqueeze(-1) * (gx - gx.mean(-1, keepdim=True) - xh * (gx * xh).mean(-1, keepdim=True))
        if cap is None:
            dx = dx.to(dy.dtype)
            return dx, dx
        outs = []
        for t in (a, b):
            tf = t.float()
            rms = torch.sqrt(tf.square().mean(-1, keepdim=True) + 1e-6)
            sc = (cap / rms).clamp(max=1.0)
            shrink = (cap / rms) < 1.0
            corr = tf * (dx * tf).mean(-1, keepdim=True) / (rms * rms)
            outs.append(torch.where(shrink, sc * (dx - corr), dx).to(dy.dtype))
        return outs[0], outs[1]

    # ------------------------------------------------------------------ paraplex core + tria step
    def ffn_core_fwd(self, d, x_real, p_in, alpha_gate, b_real, gate_lin, beta_lin, b_imag, w_trace, trace_in,
                     reset, anchor, c_prev, seed, seed_valid, gate_w, axis, tria_alpha, B, trace_out=None, bsq=None):
        """Gate, bias, phase, trace, softplus, PvPowLU and the Tria depth step in one pass.
        ``trace_out`` / ``bsq``: caller-owned fp32 buffers for the new trace ``[B,H]`` (not ``trace_in``) and the
        squared-phase sum (inference paths that run every token pass persistent ones).

        x_real/gate_lin/beta_lin: [M,H] (gate_lin None = self-referential gate); p_in [M,H] or None;
        trace_in [B,H] or None; reset [M] bool or None; c_prev [M,H,9] or None; seed [B,H,9].
        Returns dict(r, gsrc, o, i, trace_out [B,H], c [M,H,9] or None, p_out [M,H] or None, beta_sq_sum).
        """
        M, H = x_real.shape
        Tc = M // B
        r = x_real * (1.0 + alpha_gate.to(x_real.dtype) * p_in) + b_real.to(x_real.dtype) if p_in is not None \
            else x_real + b_real.to(x_real.dtype)
        gsrc = r if gate_lin is None else gate_lin
        o, i_sq, tr = R.paraplex_core(
            r.view(B, Tc, H), gsrc.view(B, Tc, H), beta_lin.view(B, Tc, H), b_imag.to(r.dtype), w_trace.to(r.dtype),
            trace_in, None if reset is None else reset.view(B, Tc), anchor, floor=d.phase_floor, m=d.powlu_m,
            activation=d.activation)
        out = {"r": r, "gsrc": gsrc, "o": o.reshape(M, H), "i": i_sq.reshape(M, H), "trace_out": tr,
               "beta_sq_sum": (beta_lin.float() + b_imag.float()).square().sum(), "c": None, "p_out": None}
        if axis is not None:
            c, p = R.tria_compose(
                r.view(B, Tc, H), i_sq, o, tria_alpha, axis,
                prev=None if c_prev is None else c_prev.view(B, Tc, H, 3, 3),
                seed=None if seed is None else seed.view(B, H, 3, 3), seed_valid=seed_valid, gate_w=gate_w)
            out["c"] = c.reshape(M, H, 9)
            out["p_out"] = None if p is None else p.reshape(M, H)
        if trace_out is not None:
            trace_out.copy_(out["trace_out"])
            out["trace_out"] = trace_out
        return out

    def ffn_core_bwd(self, d, saved, do, dc, dp_out, dtrace_out):
        """Differentiates :meth:`ffn_core_fwd`.  ``saved`` holds its inputs.  Returns a dict of gradients:
        dx_real, dp_in, dgate_lin, dbeta_lin, dtrace_in, dc_prev, dseed, and the parameter gradients
        (d_alpha_gate, d_b_real, d_b_imag, d_w_trace, d_gate_w)."""
        names = ["x_real", "p_in", "alpha_gate", "b_real", "gate_lin", "beta_lin", "b_imag", "w_trace", "trace_in",
                 "c_prev", "seed", "gate_w"]
        leaves = {}
        for k in names:
            t = saved.get(k)
            leaves[k] = None if t is None else t.detach().float().requires_grad_(True)
        with torch.enable_grad():
            out = self.ffn_core_fwd(d, leaves["x_real"], leaves["p_in"], leaves["alpha_gate"], leaves["b_real"],
                                    leaves["gate_lin"], leaves["beta_lin"], leaves["b_imag"], leaves["w_trace"],
                                    leaves["trace_in"], saved.get("reset"), saved.get("anchor"), leaves["c_prev"],
                                    leaves["seed"], saved.get("seed_valid"), leaves["gate_w"], saved.get("axis"),
                                    saved.get("tria_alpha"), saved["B"])
            outs, grads = [], []
            for t, g in ((out["o"], do), (out["c"], dc), (out["p_out"], dp_out), (out["trace_out"], dtrace_out)):
                if t is not None and g is not None and t.requires_grad:
                    outs.append(t); grads.append(g.float().reshape(t.shape))
            ins = [(k, v) for k, v in leaves.items() if v is not None]
            res = torch.autograd.grad(outs, [v for _, v in ins], grads, allow_unused=True)
        gr = {"d_" + k: g for (k, _), g in zip(ins, res)}
        acc = saved.get("gsc_acc")           # [10]: d alpha_gate, then d gate_w -- summed across the step's chunks
        if acc is not None:
            if gr.get("d_alpha_gate") is not None:
                acc[0] += gr.pop("d_alpha_gate").reshape(())
            if gr.get("d_gate_w") is not None:
                acc[1:10] += gr.pop("d_gate_w").reshape(9)
        return gr

    # ------------------------------------------------------------------ temporal endpoint (+ PolARM)
    def temporal_fwd(self, depth, B, Tc, H, reset, state, fired, polarm_beta):
        """depth: last-layer carriers of the chunk in this kernel set's carrier layout (here [M,H,9]);
        reset [B,Tc]; state [B,H,9] fp32 or None; fired [B] bool or None (PolARM applied to fired rows).
        Returns (new fp32 state [B,H,9], aux for the backward pass)."""
        return self._temporal(depth.reshape(B, Tc, H, 9), reset, state, fired, polarm_beta), None

    def _temporal(self, depth, reset, state, fired, polarm_beta):
        B, Tc, H, _ = depth.shape
        st = R.temporal_endpoint(depth.view(B, Tc, H, 3, 3), reset, None if state is None else state.view(B, H, 3, 3))
        if fired is not None:
            st = torch.where(fired[:, None, None, None], R.polarm(st, polarm_beta), st)
        return st.reshape(B, H, 9)

    def temporal_bwd(self, dstate_out, depth, B, Tc, H, reset, state, fired, polarm_beta, aux):
        dl = depth.detach().float().reshape(B, Tc, H, 9).requires_grad_(True)
        sl = None if state is None else state.detach().float().requires_grad_(True)
        with torch.enable_grad():
            out = self._temporal(dl, reset, sl, fired, polarm_beta)
            ins = [dl] + ([sl] if sl is not None else [])
            res = torch.autograd.grad(out, ins, dstate_out.float().reshape(out.shape), allow_unused=True)
        return res[0].reshape(B * Tc, H, 9), (res[1] if sl is not None else None)

    # ------------------------------------------------------------------ readout
    def slot_pool_fwd(self, keys, score_w):
        return R.slot_pool(keys.view(*keys.shape[:3], 3, 3).float(), score_w.float())

    def slot_pool_bwd(self, dpooled, keys, score_w):
        kl = keys.detach().float().requires_grad_(True)
        wl = score_w.detach().float().requires_grad_(True)
        with torch.enable_grad():
            out = R.slot_pool(kl.view(*kl.shape[:3], 3, 3), wl)
            gk, gw = torch.autograd.grad(out, [kl, wl], dpooled.float())
        return gk, gw

    def cross_attn_fwd(self, q, k, v, allowed, scale):
        return R.masked_cross_attention(q.float(), k.float(), v.float(), allowed, scale).to(q.dtype)

    def cross_attn_bwd(self, dout, q, k, v, allowed, scale):
        ls = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
        with torch.enable_grad():
            out = R.masked_cross_attention(ls[0], ls[1], ls[2], allowed, scale)
            return torch.autograd.grad(out, ls, dout.float())

    # ------------------------------------------------------------------ loss
    def ce_fwd_bwd(self, logits, targets, ignore_index, grad_scale):
        """Mean CE over non-ignored targets (fp32 math).  Returns (loss, dlogits in logits' dtype)."""
        lf = logits.float()
        valid = targets.ne(ignore_index)
        n = valid.sum().clamp(min=1)
        lse = torch.logsumexp(lf, -1)
        tgt = targets.clamp(min=0)
        nll = (lse - lf.gather(-1, tgt.unsqueeze(-1)).squeeze(-1)) * valid
        loss = nll.sum() / n
        if grad_scale is None:
            return loss, None
        p = torch.exp(lf - lse.unsqueeze(-1))
        p.scatter_add_(-1, tgt.unsqueeze(-1), -torch.ones_like(lse).unsqueeze(-1))
        return loss, (p * (valid.unsqueeze(-1) * (grad_scale / n))).to(logits.dtype)

    def rms_norm_fwd(self, x, w, eps=1e-6):
        return R.rms_norm(x, w.to(x.dtype) if x.dtype != torch.float32 else w, eps)

    def rms_norm_bwd(self, dy, x, w, gw, eps=1e-6):
        xf, g = x.float(), dy.float()
        r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        gw.add_((g * xf * r).reshape(-1, xf.shape[-1]).sum(0))
        gx = g * w.float()
        return (r * (gx - xf * r * r * (gx * xf).mean(-1, keepdim=True))).to(dy.dtype)
