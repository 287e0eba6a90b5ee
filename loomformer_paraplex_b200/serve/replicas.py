"""Data-parallel serving: one independent model replica per device, requests spread over them.

Each replica is a process that owns one device, loads the checkpoint (or ``.aio`` archive) once, keeps a
:class:`DecodeEngine` with its CUDA graph, and serves ``generate`` requests from its own queue.  The front end hands
requests to the replicas round-robin and collects results in submission order.  Replicas never talk to each other,
so throughput scales with the number of devices (the reference serves with one process and batch 1,
``loomchat.py:338-380`` there)."""
from __future__ import annotations

import itertools
import queue
from typing import Dict, List, Optional, Sequence

import torch
import torch.multiprocessing as mp


def _load(path: str, device: torch.device):
    if str(path).lower().endswith(".aio"):
        from .chat import load_aio
        model, tok, *_ = load_aio(path, device)
        return model, tok
    from .runtime import load_model
    model, _, tok, _ = load_model(path, device)
    return model, tok


def _replica_main(index: int, device: str, path: str, batch: int, max_len: Optional[int], inbox, outbox) -> None:
    torch.set_num_threads(max(1, torch.get_num_threads() // 2))
    dev = torch.device(device)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    try:
        model, _ = _load(path, dev)
        from .decode import DecodeEngine
        eng = DecodeEngine(model, batch=batch, max_len=max_len, use_graph=(dev.type == "cuda"))
        outbox.put(("ready", index, None))
    except Exception as e:                                   # report and leave: the pool raises on start-up
        outbox.put(("error", index, repr(e)))
        return
    while True:
        msg = inbox.get()
        if msg is None:
            return
        rid, prompts, max_new = msg
        try:
            eng.check_request(len(prompts[0]), int(max_new))     # refuse on the host, before touching the device
            rows = torch.tensor(prompts, dtype=torch.long, device=dev)
            n = rows.shape[0]
            if n < batch:                                   # pad the batch with copies of the first row
                rows = torch.cat((rows, rows[:1].expand(batch - n, -1)), 0)
            out = eng.generate(rows, max_new)[:n].tolist()
            outbox.put(("done", rid, out))
        except Exception as e:
            outbox.put(("fail", rid, repr(e)))


class ReplicaPool:
    """``ReplicaPool(path, devices=["cuda:0", ...], batch=64)``; ``generate(prompts, max_new)`` takes equal-length
    token-id prompts, cuts them into per-replica batches and returns the continuations in order."""

    def __init__(self, path: str, devices: Sequence[str], batch: int = 1, max_len: Optional[int] = None,
                 start_timeout: float = 600.0) -> None:
        self.ctx = mp.get_context("spawn")
        self.batch = int(batch)
        self.max_len = max_len          # None: the replicas use the model's seq_len and check there
        self.outbox = self.ctx.Queue()
        self.inboxes, self.procs = [], []
        for i, dev in enumerate(devices):
            q = self.ctx.Queue()
            p = self.ctx.Process(target=_replica_main, args=(i, str(dev), path, self.batch, max_len, q, self.outbox),
                                 daemon=True)
            p.start()
            self.inboxes.append(q)
            self.procs.append(p)
        ready = 0
        while ready < len(self.procs):
            try:
                kind, idx, info = self.outbox.get(timeout=start_timeout)
            except queue.Empty:
                self.close()
                raise RuntimeError("a replica did not come up in time")
            if kind == "error":
                self.close()
                raise RuntimeError(f"replica {idx} failed to start: {info}")
            ready += 1
        self._rr = itertools.cycle(range(len(self.procs)))
        self._next_id = 0

    def generate(self, prompts: List[List[int]], max_new: int, timeout: float = 600.0) -> List[List[int]]:
        if not prompts:
            return []
        if len({len(p) for p in prompts}) != 1:
            raise ValueError("prompts of one call must have equal length (pad or bucket them first)")
        if self.max_len is not None:
            from .decode import check_request
            check_request(len(prompts[0]), int(max_new), int(self.max_len))
        pending: Dict[int, int] = {}
        for lo in range(0, len(prompts), self.batch):
            rid = self._next_id
            self._next_id += 1
            self.inboxes[next(self._rr)].put((rid, prompts[lo:lo + self.batch], int(max_new)))
            pending[rid] = lo
        out: List[Optional[List[int]]] = [None] * len(prompts)
        while pending:
            try:
                kind, rid, payload = self.outbox.get(timeout=timeout)
            except queue.Empty:
                raise RuntimeError("a replica stopped answering")      # failure detection on the host side
            if kind == "fail":
                raise RuntimeError(f"request {rid} failed on its replica: {payload}")
            lo = pending.pop(rid)
            for j, row in enumerate(payload):
                out[lo + j] = row
        return out          # type: ignore[return-value]

    def close(self) -> None:
        for q in self.inboxes:
            try:
                q.put(None)
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()

    def __enter__(self) -> "ReplicaPool":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
