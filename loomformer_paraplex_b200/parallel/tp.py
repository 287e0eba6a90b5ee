"""Tensor parallelism building blocks: the two GEMMs of a column-parallel / row-parallel layer pair with their
collectives inside the kernels.

``column_parallel``  ``Y_local = all_gather_rows(X) @ W_local^T``.  ``X`` is row-sharded (sequence parallel): rank r
                     holds rows ``[r*M/W, (r+1)*M/W)`` in a peer-mapped buffer.  The GEMM's producer warp fetches every
                     128-row tile of ``X`` from the rank that holds it with a TMA load from that peer's memory, so the
                     all-gather is the operand fetch and overlaps the tensor-core work tile by tile.
``row_parallel``     ``Y_shard = reduce_scatter_rows(O_local @ W_local^T)``.  Each rank multiplies its slice of the
                     hidden dimension and the epilogue adds every fp32 output tile straight into the buffer of the rank
                     that owns those rows (16-byte stores over NVLink into the owner's per-sender slot; the owner
                     sums its slots): the scatter of the reduce-scatter is the epilogue, and the sum is deterministic.

Both are bracketed by a bounded cross-rank barrier on peer-mapped flag words.  For the Paraplex FFN the column-parallel
weights are ``W_real``, ``W_imag`` and ``gate_proj`` split over hidden units (whole heads per rank, so the phase sectors
stay local; the per-neuron Tria carriers and phase traces shard with them) and the row-parallel weight is ``W2``.  The
reference has no tensor parallelism."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels, native
from .symm import SymmetricBuffers


class TensorParallel:
    def __init__(self, symm: Optional[SymmetricBuffers] = None, device: Optional[torch.device] = None) -> None:
        self.symm = symm or SymmetricBuffers()
        self.world, self.rank = self.symm.world, self.symm.rank
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.symm.alloc("tp_flags", 64, torch.int32, self.device)
        self.epoch = 0
        self._bufs = {}

    # ------------------------------------------------------------------ plumbing
    def barrier(self, code: int = 501) -> None:
        """Every rank's earlier work on this stream is visible to every other rank afterwards (bounded wait)."""
        self.epoch += 1
        native.ext().tp_barrier(self.symm.peer_ptrs("tp_flags"), self.rank, self.epoch,
                                kernels.status_word(self.device), code)
        native.count()

    def buffer(self, name: str, shape, dtype) -> torch.Tensor:
        """A peer-mapped buffer of the given shape (allocated once per name; every rank must ask for the same)."""
        key = (name, tuple(shape), dtype)
        if key not in self._bufs:
            n = 1
            for s in shape:
                n *= int(s)
            self._bufs[key] = self.symm.alloc(f"tp_{name}", n, dtype, self.device).view(*shape)
        return self._bufs[key]

    # ------------------------------------------------------------------ the two fused GEMMs
    def column_parallel(self, name: str, x_rows: torch.Tensor, w_local: torch.Tensor, M: int,
                        bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x_rows`` [M/W, K] bf16 (this rank's rows) -> ``[M, N_local]`` bf16."""
        W, K = self.world, x_rows.shape[1]
        per = M // W
        assert M % W == 0 and per % 128 == 0, "rows per rank must be a multiple of the 128-row tile"
        xs = self.buffer(name, (M, K), torch.bfloat16)
        xs[self.rank * per:(self.rank + 1) * per].copy_(x_rows)
        self.barrier(502)                                   # every rank's rows are in place
        y = torch.empty(M, w_local.shape[0], dtype=torch.bfloat16, device=x_rows.device)
        kernels.gemm([xs], [K], w_local, y, M=M, N=w_local.shape[0], bias=None if bias is None else bias.float().contiguous(),
                     a_peer_ptrs=self.symm.peer_ptrs(f"tp_{name}"), a_rows_per_rank=per)
        self.barrier(503)                                   # nobody overwrites its rows while others still read them
        return y

    def row_parallel(self, name: str, o_local: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
        """``o_local`` [M, H_local] bf16, ``w_local`` [N, H_local] bf16 -> this rank's rows of the summed product,
        ``[M/W, N]`` fp32."""
        W = self.world
        M, Hl = o_local.shape
        N = w_local.shape[0]
        per = M // W
        assert M % W == 0
        stage = self.buffer(name, (W, per, N), torch.float32)
        self.barrier(504)                                   # every owner has consumed what the last call left there
        kernels.gemm([o_local], [Hl], w_local, stage[0], M=M, N=N, rs_out_ptrs=self.symm.peer_ptrs(f"tp_{name}"),
                     rs_rows_per_rank=per, rs_rank=self.rank)
        self.barrier(505)                                   # every rank's partial products have landed
        return stage.sum(0)
