"""Data-parallel gradient synchronisation over the flat gradient buffer.

Back ends
---------
``collective``  ``torch.distributed.all_reduce`` (NCCL on GPUs, gloo on CPU) over one contiguous
                fp32 range -- the measured baseline.
``p2p``         the fused sm_100a kernel (``ops/csrc/comm.cu``): every rank reduces its shard by
                reading the peers' gradient buffers over NVLink, applies clip + AdamW/ATOM to the
                shard in the same pass, and writes the refreshed fp32/bf16 parameters into every
                peer's buffers -- reduce-scatter, optimizer and all-gather in one launch.

The reference wraps its model in ``torch.nn.parallel.DistributedDataParallel`` with 64 MiB
buckets (``loomformer.py:4783-4792``) and re-broadcasts every module buffer from rank 0 before
each forward; here buffers that matter (the per-layer phase anchors) are synchronised
explicitly and only they.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import dist as pdist


class GradSync:
    def __init__(self, flat, model, backend: str = "collective", anchor_mode: str = "mean", symm=None) -> None:
        self.flat, self.model = flat, model
        self.world = dist.get_world_size() if pdist.initialized() else 1
        self.backend = backend if self.world > 1 else "none"
        self.anchor_mode = anchor_mode
        self.symm = symm
        self._anchors: Optional[List[torch.Tensor]] = None
        self.shard = None
        if self.backend in ("p2p", "fsdp"):
            if symm is None or flat.shadow is None:
                raise RuntimeError(f"grad_sync={self.backend!r} needs symmetric flat buffers on CUDA")
            dev = flat.device
            # words 0..63: flags of the exchange; from word 64 on, 64 words per rank for the phase radii
            self.sync_words = symm.alloc("sync", 64 + 64 * 8, torch.int32, dev)
            self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            self.use_multimem = False
            self.fused_anchors = None
            blocks = list(getattr(model, "blocks", []))
            if blocks and len(blocks) <= 64 and all(hasattr(b.ffn, "beta_anchor") for b in blocks):
                # the per-layer running radii become views of one array, so the fused step can average them across
                # ranks in the kernel that already exchanges the shard norms (no separate collective per step)
                arr = torch.stack([b.ffn.beta_anchor.detach().float().reshape(()) for b in blocks]).contiguous()
                for i, b in enumerate(blocks):
                    b.ffn.beta_anchor = arr[i]
                self.fused_anchors = arr
        if self.world > 1:
            self.broadcast_parameters()
        if self.backend == "fsdp":
            from .fsdp import ShardPlan
            tied = getattr(model, "head", None) is not None and getattr(model.head, "weight", None) is model.emb.weight
            self.shard = ShardPlan(flat, model, self.world, dist.get_rank(), tied_head=tied)

    def attach_optimizer(self, opt) -> None:
        """Sharded mode: the optimizer keeps Adam moments only for the blocks this rank owns."""
        # fused NVLink step with ATOM: each rank's [proxy, commits, count] sums cover its own block range only
        opt.stats_shard_local = bool(self.backend == "p2p" and self.world > 1 and opt.kind == "atom")
        if self.shard is not None and getattr(opt, "shard", None) is None:
            opt.m, opt.v = self.shard.compact(opt.m), self.shard.compact(opt.v)
            opt.shard = self.shard

    def gather_spec(self, p):
        """``(peer pointers of the weight's bf16 copy, rank)`` when ``p`` is a sharded weight that the next consuming
        GEMM has to fetch from its owners, else ``None``."""
        if self.shard is None or id(p) not in self.shard.gathered:
            return None
        seg = next(s for s in self.flat.segments if s.param is p)
        return [base + seg.offset * 2 for base in self.symm.peer_ptrs("shadow")], self.shard.rank

    def fused_step(self, opt) -> None:
        """Reduce-scatter + clip + AdamW on the own shard + all-gather in three launches over peer memory."""
        from ..ops import kernels, native
        f, s = self.flat, self.symm
        if opt.kind != "adamw":
            if self.shard is not None:
                raise NotImplementedError("sharded mode implements AdamW; use grad_sync='p2p' or 'collective' for ATOM")
            opt.step_count += 1
            hyper = kernels.upload_hyper(opt)
            native.ext().p2p_grad_step_atom(self.world, dist.get_rank(), f.nblk, s.peer_ptrs("grads"), s.peer_ptrs("params"),
                                            s.peer_ptrs("shadow"), s.peer_ptrs("sync"), opt.m, opt.v, opt.lr_mult_blk,
                                            opt.wd_blk, hyper, opt.stats, self.sumsq, opt.grad_clip,
                                            kernels.status_word(f.device), opt.cnt_blk, opt.gprev_blk, opt.pnode_blk,
                                            opt.trust_blk, opt.atom_out, self.fused_anchors, self.anchor_mode == "rank0")
            native.count(5)
            return
        opt.step_count += 1
        hyper = kernels.upload_hyper(opt)
        mc = s.multicast_ptr("grads") if self.use_multimem else 0
        sh = self.shard
        native.ext().p2p_grad_step(self.world, dist.get_rank(), f.nblk, s.peer_ptrs("grads"), s.peer_ptrs("params"),
                                   s.peer_ptrs("shadow"), s.peer_ptrs("sync"), mc, opt.m, opt.v, opt.lr_mult_blk,
                                   opt.wd_blk, opt.active_blk, hyper, opt.stats, self.sumsq, opt.grad_clip,
                                   kernels.status_word(f.device), None if sh is None else sh.owner_blk,
                                   None if sh is None else sh.slot_blk, None if sh is None else sh.replicate_blk,
                                   self.fused_anchors, self.anchor_mode == "rank0")
        native.count(3)

    def own_block_range(self):
        """Contiguous block range this rank updates in the replicated fused step (matches comm.cu)."""
        per = -(-self.flat.nblk // self.world)
        r = dist.get_rank()
        return min(per * r, self.flat.nblk), min(per * (r + 1), self.flat.nblk)

    def gather_optimizer_state(self, opt) -> None:
        """Fused-step mode: moments and per-block ATOM statistics are current only on the rank that owns a block;
        make them complete on every rank (collective) before a checkpoint."""
        if self.backend != "p2p" or self.world <= 1:
            return
        lo, hi = self.own_block_range()
        def gather(t, per_block):
            unit = 1 if per_block else 256
            keep = torch.zeros_like(t)
            keep[lo * unit:hi * unit] = t[lo * unit:hi * unit]
            dist.all_reduce(keep)
            t.copy_(keep)
        gather(opt.m, False); gather(opt.v, False)
        if opt.kind == "atom":
            for t in (opt.gprev_blk, opt.pnode_blk, opt.trust_blk):
                gather(t, True)

    def broadcast_parameters(self) -> None:
        """Every rank starts from rank 0's weights and buffers (what DDP does at construction)."""
        dist.broadcast(self.flat.params, src=0)
        self.flat.refresh_shadow()
        for b in self.model.buffers():
            if b.is_floating_point() and b.numel() == 1:
                dist.broadcast(b, src=0)

    def all_reduce_grads(self) -> None:
        if self.backend == "none":
            return
        g = self.flat.grads
        dist.all_reduce(g)
        g.mul_(1.0 / self.world)

    def sync_anchors(self) -> None:
        """Keep each layer's phase-anchor EMA identical on all ranks.

        ``mean``: average of the ranks' updated anchors (every rank's data contributes);
        ``rank0``: rank 0's value wins, which is what the reference's per-forward buffer
        broadcast amounts to (use it to match a reference loss curve).
        """
        if self.world <= 1:
            return
        if self.backend in ("p2p", "fsdp") and self.fused_anchors is not None:
            return                                   # done inside the fused step's norm exchange
        if self._anchors is None:
            self._anchors = [b.ffn.beta_anchor for b in self.model.blocks]
        packed = torch.stack([a.detach().float() for a in self._anchors])
        if self.anchor_mode == "rank0":
            dist.broadcast(packed, src=0)
        else:
            dist.all_reduce(packed)
            packed.mul_(1.0 / self.world)
        for a, v in zip(self._anchors, packed.unbind(0)):
            a.copy_(v)
