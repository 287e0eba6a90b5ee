"""Process-group bootstrap and the small host-side collectives the trainer needs.

One process per GPU; NCCL on CUDA, gloo on CPU (the reference only supports NCCL and refuses to
start a multi-rank job without CUDA, ``loomformer.py:146-195``).  All helpers degrade to the
single-process answer when no group is initialised.
"""
from __future__ import annotations

import datetime
import os
import subprocess
import sys
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def rank() -> int:
    return int(os.environ.get("RANK", "0"))


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def is_main() -> bool:
    return rank() == 0


def initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def rank0_print(*args, **kw) -> None:
    if is_main():
        print(*args, **kw)


def parse_cuda_list(pref: str) -> Optional[List[int]]:
    """``"cuda:0,cuda:1"`` / ``"0, 1"`` -> ``[0, 1]``; ``None`` for a scalar selector."""
    raw = str(pref or "").strip().lower().replace(" ", "")
    if "," not in raw:
        return None
    out: List[int] = []
    for part in raw.split(","):
        part = part[5:] if part.startswith("cuda:") else part
        if not part.isdigit():
            raise ValueError(f"bad CUDA device list {pref!r}; expected e.g. cuda:0,cuda:1")
        out.append(int(part))
    if len(set(out)) != len(out):
        raise ValueError(f"duplicate CUDA device in {pref!r}")
    return out


def auto_omp_threads(nproc: int) -> int:
    return 1 if nproc <= 0 else max(1, min(8, (os.cpu_count() or 1) // nproc))


def maybe_self_launch(device_pref: Optional[str], script: str, argv: List[str]) -> None:
    """``--device cudas`` or a comma list re-executes the script under ``torch.distributed.run``
    with one worker per selected GPU and exits with the launcher's return code."""
    pref = str(device_pref or "").strip().lower()
    subset = parse_cuda_list(pref)
    if not (pref == "cudas" or subset is not None) or "WORLD_SIZE" in os.environ:
        return
    if not torch.cuda.is_available():
        raise RuntimeError(f"--device {pref or 'cudas'} requested but CUDA is unavailable")
    env = os.environ.copy()
    if subset is None:
        n = torch.cuda.device_count()
    else:
        if len(subset) < 2:
            raise RuntimeError(f"--device {pref!r} selects fewer than 2 CUDA devices")
        parent = [x.strip() for x in env.get("CUDA_VISIBLE_DEVICES", "").split(",") if x.strip()]
        if parent and all(0 <= i < len(parent) for i in subset):
            env["CUDA_VISIBLE_DEVICES"] = ",".join(parent[i] for i in subset)
        else:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(i) for i in subset)
        n = len(subset)
    if n < 2:
        raise RuntimeError(f"--device {pref or 'cudas'} requested but fewer than 2 CUDA GPUs are visible")
    env.setdefault("OMP_NUM_THREADS", str(auto_omp_threads(n)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc_per_node", str(n), script] + list(argv)
    print("[ddp] launching:", " ".join(cmd), flush=True)
    raise SystemExit(subprocess.call(cmd, env=env))


def init(device_pref: Optional[str] = None, timeout_s: float = 600.0) -> Tuple[torch.device, int, int]:
    """Join the process group described by the torchrun environment (if any).

    Returns ``(device, world_size, rank)``.
    """
    pref = str(device_pref or "").strip().lower()
    ws, rk, lr = world_size(), rank(), local_rank()
    use_cuda = torch.cuda.is_available() and not pref.startswith("cpu")
    if ws > 1:
        if not initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("OMP_NUM_THREADS", str(auto_omp_threads(ws)))
            if use_cuda:
                torch.cuda.set_device(lr)
                dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=timeout_s),
                                        device_id=torch.device("cuda", lr))
            else:
                dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=timeout_s))
        dev = torch.device("cuda", lr) if use_cuda else torch.device("cpu")
        return dev, ws, rk
    if pref in ("", "none"):
        dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    elif pref == "cudas":
        dev = torch.device("cuda:0")
    else:
        subset = parse_cuda_list(pref)
        dev = torch.device(f"cuda:{subset[0]}") if subset is not None else torch.device(pref)
    if dev.type == "cuda":
        dev = torch.device("cuda", dev.index if dev.index is not None else torch.cuda.current_device())
        torch.cuda.set_device(dev)
    return dev, 1, 0


def barrier() -> None:
    if not initialized():
        return
    if dist.get_backend() == "nccl":
        dist.barrier(device_ids=[local_rank()])
    else:
        dist.barrier()


def mean_float(value: float, device: torch.device) -> float:
    if not initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float32, device=device)
    dist.all_reduce(t)
    return float(t.item()) / dist.get_world_size()


def sum_int(value: int, device: torch.device) -> int:
    if not initialized():
        return int(value)
    t = torch.tensor([int(value)], dtype=torch.long, device=device)
    dist.all_reduce(t)
    return int(t.item())


def max_float(value: float, device: torch.device) -> float:
    if not initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def broadcast_int(value: int, device: torch.device, src: int = 0) -> int:
    if not initialized():
        return int(value)
    t = torch.tensor([int(value)], dtype=torch.int32, device=device)
    dist.broadcast(t, src=src)
    return int(t.item())


def shutdown() -> None:
    if initialized():
        dist.destroy_process_group()


class StepControl:
    """Rank 0's per-step decisions (interrupt, run-point key, wall-clock stop) made collective.

    Saving a checkpoint is a collective in the fused and sharded gradient modes, so every rank must reach the same
    decision at the same step.  Only rank 0 watches the keyboard and its clock counts; before each step it publishes
    a small bit set and every rank acts on that value, never on its own flags.  The value travels through the job's
    key-value store (a host round trip; no device synchronisation, so the launch queue keeps running ahead) and falls
    back to a one-int broadcast when no store is reachable.  Single-process runs return the local bits unchanged.
    """
    INTERRUPT, RUNPOINT, STOP = 1, 2, 4

    def __init__(self, device: torch.device, prefix: str = "loom/ctl", use_store: bool = True) -> None:
        self.device, self.prefix = device, prefix
        self.store = None
        self._n = 0
        if initialized() and use_store:
            try:
                from torch.distributed import distributed_c10d as c10d
                self.store = c10d._get_default_store()
            except Exception:
                self.store = None

    def agree(self, local_bits: int) -> int:
        """Call on every rank, once per step, in the same order.  Returns rank 0's ``local_bits``."""
        if not initialized():
            return int(local_bits)
        self._n += 1
        if self.store is None:
            return broadcast_int(int(local_bits) if is_main() else 0, self.device)
        key = f"{self.prefix}/{self._n}"
        if is_main():
            self.store.set(key, str(int(local_bits)))
            if self._n > 64:                       # keep the store small: every rank has long read this one
                try:
                    self.store.delete_key(f"{self.prefix}/{self._n - 64}")
                except Exception:
                    pass
            return int(local_bits)
        return int(self.store.get(key).decode())
