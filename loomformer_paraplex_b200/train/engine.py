"""Training engine: the public "one optimizer step" API.

``TrainEngine.step(batch)`` takes a ``[B, T+1]`` token batch (host pinned memory or device),
copies it to the device, runs forward + fp32 cross-entropy + backward for each micro-batch,
synchronises gradients across ranks, clips by global norm, applies the optimizer and returns the
mean loss as a device scalar.  Nothing inside synchronises with the host; callers decide when
to read the loss.

It replaces the body of the reference's training loop (``loomformer.py:5064-5170``): seeds, LR
schedule, parameter groups by ``(weight_decay, lr_mult)``, gradient accumulation with the
collective skipped on non-final micro-batches, fp32 CE, global-norm clip and the non-finite
guards (one fused finite flag instead of a host sync per parameter).
"""
from __future__ import annotations

import contextlib
import os
import math
import re
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..config import Config
from ..optim.flat import FlatOptimizer, FlatParams
from ..parallel import dist as pdist
from ..parallel.ddp import GradSync
from .schedule import lr_at


def train_lr_overrides(model, cfg: Config) -> Dict[str, float]:
    """Apply ``cfg.train_lr`` (freeze flags + absolute per-tensor learning rates, matched by name with
    the ``blocks.N.`` prefix stripped; first match wins) and return ``{param_name: lr_mult}``."""
    entries = cfg.train_lr or []
    out: Dict[str, float] = {}
    if not entries:
        return out
    strip = re.compile(r"^blocks\.\d+\.")
    matched = 0
    for name, p in model.named_parameters():
        canon = strip.sub("", name)
        for e in entries:
            if e.get("name") == canon:
                p.requires_grad_(bool(e.get("train", True)))
                if "lr" in e:
                    out[name] = float(e["lr"]) / float(cfg.lr)
                matched += 1
                break
    total = sum(1 for _ in model.parameters())
    pdist.rank0_print(f"[loomcloner] train_lr: {matched}/{total} parameters matched an override "
                      f"({len(entries)} entries, {sum(1 for e in entries if not e.get('train', True))} frozen)")
    return out


class TrainEngine:
    def __init__(self, cfg: Config, model, device: torch.device, *, optimizer: Optional[str] = None,
                 grad_sync: str = "collective", anchor_mode: str = "mean", loss_mask_ignore: int = -100,
                 train_lr: bool = True, cuda_graph: Optional[bool] = None) -> None:
        self.cfg, self.model, self.device = cfg, model, device
        self.accum = max(1, int(cfg.grad_accum_steps or 1))
        self.amp = cfg.amp_dtype if device.type == "cuda" else "fp32"
        lr_mults = train_lr_overrides(model, cfg) if train_lr else {}
        self.symm = None
        alloc = None
        self.opt_name = str(optimizer or cfg.optimizer or "adamw").lower()
        if grad_sync == "fsdp" and self.opt_name != "adamw":
            # the sharded update exists for AdamW; ATOM keeps its per-block state replicated and runs in the fused
            # NVLink step (reduce-scatter, ATOM on the own slice, parameter push), which is what is selected instead
            if not pdist.initialized() or pdist.rank() == 0:
                print(f"[engine] grad_sync='fsdp' implements AdamW; optimizer {self.opt_name!r} uses the replicated "
                      "fused step (grad_sync='p2p')", flush=True)
            grad_sync = "p2p"
        self.grad_sync = grad_sync
        if grad_sync in ("p2p", "fsdp") and pdist.initialized() and device.type == "cuda":
            from ..parallel.symm import SymmetricBuffers
            self.symm = SymmetricBuffers()
            alloc = self.symm.alloc
        self.flat = FlatParams(model, want_bf16_shadow=(device.type == "cuda"), alloc=alloc)
        no_decay = {"tria_agg.pool.logit_scale_raw"}
        self.opt = FlatOptimizer(self.flat, self.opt_name, lr=cfg.lr, weight_decay=cfg.weight_decay,
                                 grad_clip=cfg.grad_clip, no_decay=no_decay, lr_mults=lr_mults)
        self.sync = GradSync(self.flat, model, backend=grad_sync, anchor_mode=anchor_mode, symm=self.symm)
        self.sync.attach_optimizer(self.opt)
        self.plan = model._opset(model.emb.weight) if not model.ablation else None   # fused plan on CUDA
        if self.plan is not None:
            self.plan.bind(self.flat)
            if self.sync.shard is not None:
                self.plan.gather_spec = self.sync.gather_spec
        # Whole forward+backward of a micro-batch as one CUDA graph: the fused plan issues several thousand launches per
        # step and the host cannot enqueue them as fast as a B200 retires them.  On by default on CUDA, off with
        # LOOM_CUDA_GRAPH=0 or ``cfg.graph: false`` given explicitly through ``cuda_graph``.
        if cuda_graph is None:
            cuda_graph = os.environ.get("LOOM_CUDA_GRAPH", "1") != "0"
        self.use_graph = bool(cuda_graph and device.type == "cuda" and self.plan is not None)
        self._graphs: Dict[tuple, dict] = {}
        self.step_idx = 0           # completed optimizer steps
        self.ignore_index = loss_mask_ignore
        self.last_fire_count = torch.zeros((), dtype=torch.long, device=device)
        self._skipped_seen = 0

    # ------------------------------------------------------------------ pieces
    def _autocast(self):
        if self.device.type != "cuda" or self.amp in ("fp32", "off"):
            return contextlib.nullcontext()
        return torch.autocast("cuda", dtype=torch.bfloat16 if self.amp == "bf16" else torch.float16)

    def loss_fn(self, x, y, attn_mask=None, position_ids=None) -> torch.Tensor:
        with self._autocast():
            logits = self.model(x, attn_mask=attn_mask, position_ids=position_ids)
        return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), y.reshape(-1),
                               ignore_index=self.ignore_index)

    def to_device(self, batch: torch.Tensor) -> torch.Tensor:
        return batch.to(self.device, non_blocking=True) if batch.device != self.device else batch

    # ------------------------------------------------------------------ graph-replayed micro-batch
    GRAPH_WARMUP = 2        # eager runs per shape before capture (lazy kernel attributes, allocator, constant caches)

    def _graphed_micro(self, x, y, position_ids, segment_ids, scale: float) -> torch.Tensor:
        """Forward + backward of one micro-batch (gradients accumulate into the flat buffer).  The first runs of a
        shape are eager; then the launch sequence is captured once and replayed with the inputs copied into the
        graph's static buffers.  Chunk boundaries are part of the graph, so a batch whose ``<CARRY>`` columns differ
        gets its own graph (their positions are read back once per step only when the tokenizer has that token)."""
        from ..ops import native
        m = self.model
        cuts = None
        if m.carry_token_id is not None and m.d.tria and m.d.tria_temporal:
            pos = position_ids if position_ids is not None else \
                torch.arange(x.shape[1], device=x.device).view(1, -1).expand(x.shape[0], -1)
            cuts = tuple(m.fire_plan(x, pos)[2])
        key = (tuple(x.shape), position_ids is not None, segment_ids is not None, cuts, float(scale))
        ent = self._graphs.setdefault(key, {"runs": 0, "graph": None})
        if ent["graph"] is None and ent["runs"] < self.GRAPH_WARMUP:
            ent["runs"] += 1
            with torch.no_grad():
                loss, _ = self.plan.run(x, y, position_ids, segment_ids, want_grad=True, ignore_index=self.ignore_index,
                                        grad_scale=scale, cuts=cuts)
            return loss
        if ent["graph"] is None:
            ent["x"], ent["y"] = x.clone(), y.clone()
            ent["pos"] = None if position_ids is None else position_ids.clone()
            ent["seg"] = None if segment_ids is None else segment_ids.clone()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = native.launches()
            with torch.no_grad(), torch.cuda.graph(g):
                ent["loss"], _ = self.plan.run(ent["x"], ent["y"], ent["pos"], ent["seg"], want_grad=True,
                                               ignore_index=self.ignore_index, grad_scale=scale, cuts=cuts)
                ent["fire"] = m.last_tria_fire_mask
            ent["launches"] = native.launches() - before
            ent["graph"] = g
        ent["x"].copy_(x); ent["y"].copy_(y)
        if ent["pos"] is not None:
            ent["pos"].copy_(position_ids)
        if ent["seg"] is not None:
            ent["seg"].copy_(segment_ids)
        ent["graph"].replay()
        native.count(ent["launches"])
        m.last_tria_fire_mask = ent["fire"]
        return ent["loss"].clone()

    # ------------------------------------------------------------------ one optimizer step
    def step(self, batch, targets: Optional[torch.Tensor] = None, attn_mask=None, position_ids=None,
             segment_ids=None) -> torch.Tensor:
        """``batch`` is ``[B, T+1]`` tokens (inputs ``[:, :-1]``, targets ``[:, 1:]``) or, with explicit
        ``targets``, ``[B, T]`` inputs.  With ``grad_accum_steps > 1`` pass a list of micro-batches."""
        micro = batch if isinstance(batch, (list, tuple)) else [batch]
        self.model.train()
        self.flat.zero_grad()
        total = None
        for mb in micro:
            if isinstance(mb, dict):     # a packed micro-batch carrying its own targets and reset state
                x, y = self.to_device(mb["x"]), self.to_device(mb["y"])
                position_ids, segment_ids = mb.get("position_ids"), mb.get("segment_ids")
            elif targets is None:
                mb = self.to_device(mb)
                x, y = mb[:, :-1], mb[:, 1:]
            else:
                x, y = self.to_device(mb), self.to_device(targets)
            mask_i = attn_mask
            if self.plan is not None and attn_mask is None:
                scale = 1.0 / float(len(micro))
                if self.use_graph:
                    loss = self._graphed_micro(x, y, position_ids, segment_ids, scale)
                else:
                    with torch.no_grad():
                        loss, _ = self.plan.run(x, y, position_ids, segment_ids, want_grad=True,
                                                ignore_index=self.ignore_index, grad_scale=scale)
            else:
                if segment_ids is not None and mask_i is None:
                    T = x.shape[1]
                    mask_i = ((segment_ids[:, :, None] == segment_ids[:, None, :])
                              & torch.ones(T, T, dtype=torch.bool, device=x.device).tril()).unsqueeze(1)
                loss = self.loss_fn(x, y, mask_i, position_ids)
                (loss / float(len(micro))).backward()
            fm = self.model.last_tria_fire_mask
            if fm is not None:
                self.last_fire_count += fm.sum()
            total = loss.detach() if total is None else total + loss.detach()
        self.opt.set_lr(lr_at(self.cfg, self.step_idx))
        if self.sync.backend in ("p2p", "fsdp"):
            self.sync.fused_step(self.opt)
        else:
            self.sync.all_reduce_grads()
            self.opt.step()
        self.sync.sync_anchors()
        self.step_idx += 1
        return total / float(len(micro))

    def complete_master(self) -> None:
        """Sharded mode: make this rank's fp32 parameters complete again (collective; call on every rank before a
        checkpoint, an export, or anything else that reads ``model.state_dict()``)."""
        if self.sync.shard is not None:
            self.sync.shard.gather_master()

    def checkpoint_view(self):
        """Object whose ``state_dict()`` is the optimizer state to save.  In sharded mode this completes the fp32
        master parameters and assembles the full moments (collectives: call on every rank)."""
        self.check_device_status()                  # never checkpoint the result of a step whose waits timed out
        if self.sync.shard is None:
            self.sync.gather_optimizer_state(self.opt)        # no-op unless the fused NVLink step owns the update
            return self.opt
        self.complete_master()
        sd = self.opt.state_dict()

        class _Frozen:
            def state_dict(self_inner):
                return sd
        return _Frozen()

    def check_device_status(self) -> None:
        """Raise if a kernel gave up a bounded wait since the last check (status word of this device)."""
        from ..ops import kernels
        if kernels.has_status_word(self.device):
            kernels.check_status(self.device)

    def check_finite(self, loss: torch.Tensor) -> None:
        """Host-side guard (one sync): raise if a kernel gave up a bounded wait, if the loss or the last gradient norm
        was not finite, or if any update since the previous check was skipped on the device."""
        self.check_device_status()
        lv = float(loss)
        if not math.isfinite(lv):
            raise RuntimeError(f"non-finite training loss: loss={lv:.9g} optimizer={self.opt_name} step={self.step_idx}")
        if not self.opt.grads_finite():
            raise RuntimeError("non-finite gradient detected before optimizer step: "
                               f"optimizer={self.opt_name} step={self.step_idx} (update was skipped on device)")
        skipped = self.opt.skipped_updates()
        if skipped > self._skipped_seen:
            n = skipped - self._skipped_seen
            self._skipped_seen = skipped
            raise RuntimeError(f"{n} optimizer update(s) since the last check were skipped on the device "
                               f"(non-finite gradients or a timed-out wait): optimizer={self.opt_name} "
                               f"step={self.step_idx}")
