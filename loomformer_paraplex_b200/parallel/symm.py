"""Symmetric (peer-mapped) device buffers.

``SymmetricBuffers`` allocates tensors whose backing memory every rank of the group can address
directly over NVLink (``torch.distributed._symmetric_memory``: CUDA VMM allocations whose handles are
exchanged through the process group's store), and exposes the raw peer pointers that the fused
communication kernels take.  An NVSwitch multicast mapping is reported when the driver provides one.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class SymmetricBuffers:
    def __init__(self, group=None) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        self._sm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.handles: Dict[str, object] = {}
        self.tensors: Dict[str, torch.Tensor] = {}

    def alloc(self, name: str, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        t = self._sm.empty(numel, dtype=dtype, device=device)
        t.zero_()
        hdl = self._sm.rendezvous(t, self.group)
        self.handles[name], self.tensors[name] = hdl, t
        return t

    def peer_ptrs(self, name: str) -> List[int]:
        return [int(p) for p in self.handles[name].buffer_ptrs]

    def multicast_ptr(self, name: str) -> int:
        hdl = self.handles[name]
        try:
            return int(hdl.multicast_ptr) if hdl.has_multicast_support(hdl.device.type, hdl.device.index) else 0
        except Exception:
            try:
                return int(hdl.multicast_ptr)
            except Exception:
                return 0

    def barrier(self, name: str) -> None:
        self.handles[name].barrier()
