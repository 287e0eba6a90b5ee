"""Flat-buffer optimizer state for one-launch multi-tensor updates.

All parameters of a model are re-homed into ONE fp32 buffer (each tensor padded to a multiple of
``BLOCK`` elements); ``param.data`` and ``param.grad`` become views of the parameter / gradient
buffers.  Consequences:

* gradient synchronisation is a collective over one contiguous range (or a few ranges), and the
  fused reduce-scatter + update + all-gather kernel works on plain pointers;
* AdamW and ATOM update every tensor in one pass; per-tensor hyper-parameters (learning-rate
  multiplier, weight decay, frozen flag) are stored per ``BLOCK``;
* the global gradient norm, the clip coefficient and the finite check are device-side scalars, so
  a training step needs no host synchronisation;
* a bf16 shadow of the parameters (what the tensor-core kernels read) is refreshed by the update.

The update rules themselves are AdamW (``torch.optim.AdamW`` semantics, betas (0.9, 0.999),
eps 1e-8) and ATOM (reference ``atom/atom.py:157-248`` kernel semantics: per-block trust and
commit gating, decoupled weight decay always applied, per-block EMA statistics).  ATOM's block
grid restarts at every tensor, which the per-tensor padding reproduces exactly.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

BLOCK = 256


@dataclass
class Segment:
    name: str
    param: nn.Parameter
    offset: int          # element offset into the flat buffers (multiple of BLOCK)
    numel: int
    padded: int
    trainable: bool
    lr_mult: float = 1.0
    weight_decay: float = 0.0


class FlatParams:
    """Owns the flat parameter / gradient / bf16-shadow buffers of a model."""

    def __init__(self, model: nn.Module, want_bf16_shadow: bool = False, alloc=None) -> None:
        """``alloc(name, numel, dtype, device)`` may supply the backing storage (e.g. peer-mapped symmetric
        memory for the fused NVLink gradient step); the default is ordinary device memory."""
        seen: Dict[int, str] = {}
        self.segments: List[Segment] = []
        off = 0
        for name, p in model.named_parameters():
            if id(p) in seen:
                continue
            seen[id(p)] = name
            padded = -(-p.numel() // BLOCK) * BLOCK
            self.segments.append(Segment(name, p, off, p.numel(), padded, bool(p.requires_grad)))
            off += padded
        self.total = off
        dev = self.segments[0].param.device
        self.device = dev
        mk = alloc or (lambda name, n, dt, d: torch.zeros(n, dtype=dt, device=d))
        self.params = mk("params", off, torch.float32, dev)
        self.grads = mk("grads", off, torch.float32, dev)
        self.shadow = mk("shadow", off, torch.bfloat16, dev) if want_bf16_shadow else None
        for s in self.segments:
            view = self.params[s.offset:s.offset + s.numel].view_as(s.param)
            view.copy_(s.param.data)
            s.param.data = view
            if s.trainable:
                s.param.grad = self.grads[s.offset:s.offset + s.numel].view_as(s.param)
        self.by_name = {s.name: s for s in self.segments}
        self.refresh_shadow()

    @property
    def nblk(self) -> int:
        return self.total // BLOCK

    def refresh_shadow(self) -> None:
        if self.shadow is not None:
            self.shadow.copy_(self.params)

    def shadow_of(self, p: nn.Parameter) -> torch.Tensor:
        s = next(x for x in self.segments if x.param is p)
        return self.shadow[s.offset:s.offset + s.numel].view_as(p)

    def zero_grad(self) -> None:
        self.grads.zero_()

    def reattach_grads(self) -> None:
        """Re-point ``param.grad`` at the flat gradient buffer (after something set it to None)."""
        for s in self.segments:
            if s.trainable:
                s.param.grad = self.grads[s.offset:s.offset + s.numel].view_as(s.param)

    def block_vector(self, fn) -> torch.Tensor:
        """Per-block fp32 vector filled with ``fn(segment)``."""
        out = torch.empty(self.nblk, dtype=torch.float32)
        for s in self.segments:
            out[s.offset // BLOCK:(s.offset + s.padded) // BLOCK] = float(fn(s))
        return out.to(self.device)

    def block_counts(self) -> torch.Tensor:
        out = torch.zeros(self.nblk, dtype=torch.float32)
        for s in self.segments:
            b0 = s.offset // BLOCK
            full, rem = divmod(s.numel, BLOCK)
            out[b0:b0 + full] = BLOCK
            if rem:
                out[b0 + full] = rem
        return out.to(self.device)


class FlatOptimizer:
    """AdamW / ATOM over :class:`FlatParams`.  ``lr`` is set per step via :meth:`set_lr`."""

    def __init__(self, flat: FlatParams, kind: str = "adamw", lr: float = 1e-3, weight_decay: float = 0.01,
                 betas: Tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, grad_clip: float = 0.0,
                 no_decay: Iterable[str] = (), lr_mults: Optional[Dict[str, float]] = None) -> None:
        kind = str(kind or "adamw").strip().lower()
        if kind not in ("adamw", "atom"):
            raise ValueError(f"unknown optimizer={kind!r}; expected 'adamw' or 'atom'")
        self.flat, self.kind = flat, kind
        self.base_lr, self.lr = float(lr), float(lr)
        self.betas, self.eps = (float(betas[0]), float(betas[1])), float(eps)
        self.grad_clip = float(grad_clip or 0.0)
        no_decay = set(no_decay)
        lr_mults = lr_mults or {}
        for s in flat.segments:
            s.weight_decay = 0.0 if s.name in no_decay else float(weight_decay)
            s.lr_mult = float(lr_mults.get(s.name, 1.0))
        dev = flat.device
        self.lr_mult_blk = flat.block_vector(lambda s: s.lr_mult if s.trainable else 0.0)
        self.wd_blk = flat.block_vector(lambda s: s.weight_decay if s.trainable else 0.0)
        self.active_blk = flat.block_vector(lambda s: 1.0 if s.trainable else 0.0)
        self.cnt_blk = flat.block_counts() * self.active_blk
        self.m = torch.zeros_like(flat.params)
        self.v = torch.zeros_like(flat.params)
        self.step_count = 0
        # device scalars: [grad_norm, clip_coef, finite(1/0), sticky count of skipped updates]
        self.stats = torch.zeros(4, dtype=torch.float32, device=dev)
        if kind == "atom":
            self.meta_scale = max(1, min(8, int(os.getenv("ATOM_META_SCALE", "1"))))
            if self.meta_scale != 1:
                raise ValueError("the flat ATOM layout is built for ATOM_META_SCALE=1 (256-element blocks)")
            self.trust_min, self.trust_max = 0.90, 1.90
            self.bootstrap_steps, self.bootstrap_gain = 20 * self.meta_scale, 2.4
            self.proxy_ema, self.pnode = 0.0, 0.65
            self.gprev_blk = torch.zeros(flat.nblk, dtype=torch.float32, device=dev)
            self.pnode_blk = torch.full((flat.nblk,), self.pnode, dtype=torch.float32, device=dev)
            self.trust_blk = torch.full((flat.nblk,), 1.25, dtype=torch.float32, device=dev)
            self.atom_out = torch.zeros(3, dtype=torch.float32, device=dev)   # proxy, commits, count
            self.last_stats: Dict[str, float] = {}

    # ------------------------------------------------------------------ knobs
    def set_lr(self, lr: float) -> None:
        self.lr = float(lr)

    # ------------------------------------------------------------------ norm / clip
    def compute_clip(self) -> None:
        """grad norm -> ``stats[0]``, clip coefficient -> ``stats[1]``, finite flag -> ``stats[2]``."""
        norm = torch.linalg.vector_norm(self.flat.grads)
        self.stats[0] = norm
        if self.grad_clip > 0:
            self.stats[1] = (self.grad_clip / (norm + 1e-6)).clamp(max=1.0)
        else:
            self.stats[1] = 1.0
        self.stats[2] = torch.isfinite(norm).float()
        self.stats[3] += 1.0 - self.stats[2]

    def grads_finite(self) -> bool:
        return bool(self.stats[2].item() > 0.5)

    def skipped_updates(self) -> int:
        """Updates skipped on the device so far (non-finite gradient norm, or a kernel that gave up a bounded wait);
        one host sync, meant for log cadence."""
        return int(self.stats[3].item())

    # ------------------------------------------------------------------ update
    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        from ..ops import native
        if self.flat.device.type == "cuda" and native.available():
            native.optimizer_step(self)
        else:
            self.compute_clip()
            self._step_torch()

    @torch.no_grad()
    def _step_torch(self) -> None:
        f = self.flat
        t = self.step_count
        b1, b2 = self.betas
        ok = self.stats[2]
        g = (f.grads * self.stats[1]).view(-1, BLOCK)
        g = torch.where(ok > 0.5, g, torch.zeros_like(g))
        p, m, v = f.params.view(-1, BLOCK), self.m.view(-1, BLOCK), self.v.view(-1, BLOCK)
        act = (self.active_blk * ok).view(-1, 1)
        lr = (self.lr * self.lr_mult_blk).view(-1, 1)
        wd = self.wd_blk.view(-1, 1)
        bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
        m_new = m + (1.0 - b1) * (g - m)
        v_new = v + (1.0 - b2) * (g * g - v)
        m.copy_(torch.where(act > 0, m_new, m))
        v.copy_(torch.where(act > 0, v_new, v))
        if self.kind == "adamw":
            upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
            p_new = p * (1.0 - lr * wd) - lr * upd
            p.copy_(torch.where(act > 0, p_new, p))
        else:
            self.trust_blk.copy_(self.trust_min + self.pnode_blk * (self.trust_max - self.trust_min))
            if t <= self.bootstrap_steps:
                self.trust_blk.clamp_(min=self.bootstrap_gain)
            trust, gprev, pnode = self.trust_blk.view(-1, 1), self.gprev_blk.view(-1, 1), self.pnode_blk.view(-1, 1)
            v_hat = v / max(bc2, 1e-12)
            base = (m / max(bc1, 1e-12)) / (v_hat.sqrt() + self.eps)
            delta = -lr * base * (1.0 + trust)
            pred = -((g + 0.35 * (g - gprev)) * delta) - 0.5 * v_hat * delta * delta
            commit = ((pred > 0) & (pnode >= 0.5)).float() * act
            delta = delta * commit - lr * wd * p
            p.copy_(torch.where(act > 0, p + delta, p))
            cnt = self.cnt_blk.clamp(min=1.0)
            live = self.cnt_blk > 0
            csum = commit.sum(1)
            self.gprev_blk.copy_(torch.where(live, g.sum(1) / cnt, self.gprev_blk))
            pn = (0.95 * self.pnode_blk + 0.05 * (0.5 + 0.5 * csum / cnt)).clamp(0.01, 0.99)
            self.pnode_blk.copy_(torch.where(live, pn, self.pnode_blk))
            self.atom_out[0] = -(g * delta * act).sum()
            self.atom_out[1] = csum.sum()
            self.atom_out[2] = self.cnt_blk.sum()
        f.refresh_shadow()

    def atom_refresh_stats(self) -> Dict[str, float]:
        """Pull ATOM's global statistics to the host (one sync; call at log cadence)."""
        if self.kind != "atom":
            return {}
        out = self.atom_out
        if getattr(self, "stats_shard_local", False):
            # the fused NVLink step runs ATOM on this rank's block range only: its three sums are partial
            import torch.distributed as dist
            out = self.atom_out.clone()
            dist.all_reduce(out)
        proxy, commits, count = (float(x) for x in out.tolist())
        if count > 0:
            pm, cf = proxy / count, commits / count
            live = self.cnt_blk > 0
            trust_mean = float(self.trust_blk[live].mean()) if bool(live.any()) else 0.0
            self.proxy_ema = 0.98 * self.proxy_ema + 0.02 * pm
            self.pnode = float(min(0.99, max(0.01, 0.95 * self.pnode + 0.05 * (0.5 + 0.5 * cf))))
            self.last_stats = {"params_tensors": float(sum(1 for s in self.flat.segments if s.trainable)),
                               "trust_mean": trust_mean, "commit_frac": cf, "impact_proxy_mean": pm,
                               "pnode": self.pnode}
        return self.last_stats

    # ------------------------------------------------------------------ torch-format state dicts
    def _groups(self) -> List[Tuple[Tuple[float, float], List[Segment]]]:
        groups: Dict[Tuple[float, float], List[Segment]] = {}
        for s in self.flat.segments:
            if s.trainable:
                groups.setdefault((s.weight_decay, s.lr_mult), []).append(s)
        return list(groups.items())

    def state_dict(self) -> dict:
        """Per-parameter state in the ``torch.optim`` layout (AdamW: ``step/exp_avg/exp_avg_sq``;
        ATOM: ``step/m/v/gprev_blk/pnode_blk/trust_blk`` + ``atom_meta``), grouped by
        ``(weight_decay, lr_mult)`` in model parameter order like the reference trainer."""
        state, groups, idx = {}, [], 0
        shard = getattr(self, "shard", None)        # sharded mode keeps compact moments: rebuild the full arrays
        full_m = self.m if shard is None else shard.expand(self.m)
        full_v = self.v if shard is None else shard.expand(self.v)
        for (wd, mult), segs in self._groups():
            ids = []
            for s in segs:
                sl = slice(s.offset, s.offset + s.numel)
                bs = slice(s.offset // BLOCK, (s.offset + s.padded) // BLOCK)
                if self.kind == "adamw":
                    st = {"step": torch.tensor(float(self.step_count)),
                          "exp_avg": full_m[sl].view_as(s.param).clone(),
                          "exp_avg_sq": full_v[sl].view_as(s.param).clone()}
                else:
                    st = {"step": torch.tensor(self.step_count, dtype=torch.int64),
                          "m": full_m[sl].view_as(s.param).clone(), "v": full_v[sl].view_as(s.param).clone(),
                          "gprev_blk": self.gprev_blk[bs].clone(), "pnode_blk": self.pnode_blk[bs].clone(),
                          "trust_blk": self.trust_blk[bs].clone()}
                if self.step_count > 0:
                    state[idx] = st
                ids.append(idx)
                idx += 1
            g = {"lr": self.lr * mult, "betas": self.betas, "eps": self.eps, "weight_decay": wd,
                 "lr_mult": mult, "params": ids}
            groups.append(g)
        out = {"state": state, "param_groups": groups}
        if self.kind == "atom":
            out["atom_meta"] = {"step": self.step_count, "proxy_ema": self.proxy_ema, "pnode": self.pnode,
                                "last_stats": dict(self.last_stats), "meta_scale": 1}
        return out

    def load_state_dict(self, sd: dict) -> None:
        order = [s for _, segs in self._groups() for s in segs]
        n_saved = sum(len(g["params"]) for g in sd.get("param_groups", []))
        if n_saved != len(order):
            raise ValueError("optimizer checkpoint is incompatible with the active trainable parameter groups; "
                             "keep train_lr/freeze settings unchanged or start without --resume")
        steps = []
        shard = getattr(self, "shard", None)
        if shard is not None:                       # load into full arrays, then keep this rank's blocks
            self.m = torch.zeros(self.flat.total, dtype=torch.float32, device=self.flat.device)
            self.v = torch.zeros_like(self.m)
        for idx, s in enumerate(order):
            st = sd["state"].get(idx, sd["state"].get(str(idx)))
            if st is None:
                continue
            sl = slice(s.offset, s.offset + s.numel)
            bs = slice(s.offset // BLOCK, (s.offset + s.padded) // BLOCK)
            m = st.get("m", st.get("exp_avg"))
            v = st.get("v", st.get("exp_avg_sq"))
            if m is not None:
                self.m[sl].copy_(m.reshape(-1))
            if v is not None:
                self.v[sl].copy_(v.reshape(-1))
            if self.kind == "atom":
                for key, buf in (("gprev_blk", self.gprev_blk), ("pnode_blk", self.pnode_blk),
                                 ("trust_blk", self.trust_blk)):
                    if key in st and st[key].numel() == buf[bs].numel():
                        buf[bs].copy_(st[key].reshape(-1).float())
            if "step" in st:
                steps.append(int(float(st["step"])))
        self.step_count = max(steps) if steps else 0
        if shard is not None:
            self.m, self.v = shard.compact(self.m), shard.compact(self.v)
        meta = sd.get("atom_meta")
        if meta is not None and self.kind == "atom":
            self.step_count = int(meta.get("step", self.step_count))
            self.proxy_ema = float(meta.get("proxy_ema", self.proxy_ema))
            self.pnode = float(meta.get("pnode", self.pnode))
            self.last_stats = dict(meta.get("last_stats", {}))
