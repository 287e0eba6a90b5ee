"""Sharded data parallelism over the flat parameter buffers (ZeRO-style full sharding of the optimizer state and of
weight ownership).

Every 256-element block of the flat parameter space has exactly one owner rank.  The owner holds the block's Adam
moments (compact arrays: only owned blocks exist), reduces the block's gradient from all ranks, updates it, and keeps
the refreshed fp32 master and bf16 value.  Two kinds of blocks:

* **GEMM weights** (rows of the big linear layers) are owned in runs of 64 rows, contiguous per rank.  Their new
  values are NOT pushed to the other ranks.  Instead the first GEMM of the next step that consumes the weight fetches
  each 64-row block from its owner -- TMA loads from the owner's memory inside the GEMM kernel -- and completes the
  local bf16 copy as a side effect (``ops/csrc/gemm.cu``, ``GATHER``).  The parameter all-gather is thus fused into
  the first consuming GEMM and overlaps its math tile by tile.
* **Everything else** (biases, norms, gates, carriers' small matrices, embeddings) is a few percent of the bytes; the
  owner stores the refreshed values straight into every rank's buffers, as in the replicated fused step.

The reference has no sharded mode at all (its only strategy is DistributedDataParallel,
``loomformer.py:4783-4792``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..optim.flat import BLOCK

# parameters that reach the tensor cores as the plain K-major B operand of a linear layer
GATHERED_SUFFIXES = ("attn.qkv_weight", "attn.o.weight", "ffn.w1_real.weight", "ffn.gate_proj.weight", "ffn.w2.weight",
                     "depth_attn.kv_weight", "depth_attn.w_o.weight", "head.weight", "tria_final_ca.w_qk.weight",
                     "tria_final_ca.w_v.weight")


def row_block_owner(rows: int, world: int) -> Tuple[int, List[int]]:
    """Ownership of a ``rows``-row weight in runs of 64 rows: (blocks per rank, owner of each 64-row block)."""
    nb = -(-rows // 64)
    per = -(-nb // world)
    return per, [min(b // per, world - 1) for b in range(nb)]


class ShardPlan:
    def __init__(self, flat, model, world: int, rank: int, tied_head: bool = False) -> None:
        self.flat, self.world, self.rank = flat, int(world), int(rank)
        nblk = flat.nblk
        owner = torch.empty(nblk, dtype=torch.uint8)
        repl = torch.ones(nblk, dtype=torch.uint8)
        self.gathered: Dict[int, str] = {}                 # id(param) -> name, for weights fetched on use
        small: List[Tuple[int, int]] = []
        # a hidden sector that is not a multiple of 8 neurons wide makes the execution plan work on padded copies of
        # the neuron-indexed FFN weights, which it rebuilds from complete local values: those stay replicated
        padded_ffn = getattr(getattr(model, "d", None), "hpq", 8) % 8 != 0
        ffn_suffixes = ("ffn.w1_real.weight", "ffn.gate_proj.weight", "ffn.w2.weight")
        for s in flat.segments:
            b0, b1 = s.offset // BLOCK, (s.offset + s.padded) // BLOCK
            p = s.param
            ok = (p.dim() == 2 and s.name.endswith(GATHERED_SUFFIXES) and p.shape[0] >= 64 * world
                  and (64 * p.shape[1]) % BLOCK == 0 and (p.shape[1] * 2) % 16 == 0
                  and not (tied_head and s.name in ("head.weight", "emb.weight"))
                  and not (padded_ffn and s.name.endswith(ffn_suffixes)))
            if ok:
                _, blocks = row_block_owner(p.shape[0], world)
                per64 = 64 * p.shape[1] // BLOCK           # flat blocks per 64-row block
                for j in range(b0, b1):
                    owner[j] = blocks[min((j - b0) // per64, len(blocks) - 1)]
                repl[b0:b1] = 0
                self.gathered[id(p)] = s.name
            else:
                small.append((b0, b1))
        # replicated tensors: spread their blocks over the ranks in contiguous runs
        n_small = sum(b1 - b0 for b0, b1 in small)
        per = max(1, -(-n_small // world))
        k = 0
        for b0, b1 in small:
            for j in range(b0, b1):
                owner[j] = min(k // per, world - 1)
                k += 1
        mine = owner.eq(self.rank)
        slot = torch.full((nblk,), -1, dtype=torch.int32)
        slot[mine] = torch.arange(int(mine.sum()), dtype=torch.int32)
        dev = flat.device
        self.owner_blk, self.replicate_blk, self.slot_blk = owner.to(dev), repl.to(dev), slot.to(dev)
        self.owned_blocks = int(mine.sum())
        self.owned_index = mine.nonzero().flatten().to(dev)          # block ids owned by this rank, ascending
        self.gather_bytes = sum(s.numel * 2 for s in flat.segments if id(s.param) in self.gathered)

    # ------------------------------------------------------------------ compact <-> full moment arrays
    def compact(self, full: torch.Tensor) -> torch.Tensor:
        return full.view(-1, BLOCK)[self.owned_index].reshape(-1).contiguous()

    def expand(self, compact: torch.Tensor, reduce: bool = True) -> torch.Tensor:
        """Full-size array from the ranks' compact shards (an all-reduce of disjoint supports)."""
        full = torch.zeros(self.flat.total, dtype=compact.dtype, device=compact.device)
        full.view(-1, BLOCK)[self.owned_index] = compact.view(-1, BLOCK)
        if reduce and self.world > 1:
            dist.all_reduce(full)
        return full

    def gather_master(self) -> None:
        """Make this rank's fp32 parameter buffer complete (owners hold the truth for sharded weights); used before
        checkpoints and evaluation through the fp32 module path."""
        if self.world <= 1:
            return
        p = self.flat.params
        mask = self.owner_blk.eq(self.rank).view(-1, 1)
        mine = torch.where(mask, p.view(-1, BLOCK), torch.zeros_like(p.view(-1, BLOCK)))
        dist.all_reduce(mine)
        p.view(-1, BLOCK).copy_(mine)
