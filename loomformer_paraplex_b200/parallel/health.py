"""Host-side failure detection for multi-rank runs.

A rank can disappear between steps (crash, pre-emption, operator kill).  The survivors must learn of it on the host,
before their next launch, instead of sitting in a collective:

* :class:`Heartbeat` -- every rank stamps a counter into the job's key-value store (the one ``torch.distributed``
  rendezvoused on) from a background thread; :meth:`Heartbeat.check` raises :class:`PeerLost` when a peer's stamp stops
  advancing for longer than ``max_silence`` seconds.  The training loops call it once per step, before launching.
* :class:`StepWatchdog` -- a host timer armed around each step; if the step does not come back within the limit (a
  peer died inside a collective, a kernel gave up a bounded wait and the status word is pending) the callback fires,
  by default dumping a message and raising in the main thread through ``_thread.interrupt_main``.
* device-side waits on peer flags are bounded (``ops/csrc/comm.cu``, ``sm100.cuh``): they record a code in the status
  word and return; ``ops.kernels.check_status`` turns that into a host exception after the step.

Recovery is restart-from-run-point: the trainers write run-points periodically and resume deterministically
(optimizer state, step, token count, data fast-forward).  The reference has none of this
(``torchrun --standalone``, no health checks; reference ``loomformer.py:52-195``)."""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, ranks: List[int], silence: float) -> None:
        super().__init__(f"rank(s) {ranks} stopped reporting for {silence:.1f}s; stop launching and restart from the "
                         f"last run-point")
        self.ranks = ranks


def default_store():
    from torch.distributed import distributed_c10d as c10d
    return c10d._get_default_store()


class Heartbeat:
    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, interval: float = 0.5,
                 max_silence: float = 5.0, prefix: str = "loom/hb") -> None:
        self.store = store if store is not None else default_store()
        self.rank = dist.get_rank() if rank is None else int(rank)
        self.world = dist.get_world_size() if world is None else int(world)
        self.interval, self.max_silence, self.prefix = float(interval), float(max_silence), prefix
        self._stop = threading.Event()
        self._seen: Dict[int, tuple] = {}            # rank -> (last counter value, host time when it last changed)
        self._count = 0
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def _beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:
                return                                   # the store went away with the job

    def check(self) -> None:
        """Raise :class:`PeerLost` if some peer's counter has not moved for ``max_silence`` seconds."""
        now = time.monotonic()
        lost = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = self.store.get(self._key(r)).decode() if self._has(r) else None
            except Exception:
                val = None
            last = self._seen.get(r)
            if last is None or (val is not None and val != last[0]):
                self._seen[r] = (val, now)
            elif now - last[1] > self.max_silence:
                lost.append(r)
        if lost:
            raise PeerLost(lost, self.max_silence)

    def _has(self, r: int) -> bool:
        try:
            return bool(self.store.check([self._key(r)]))
        except Exception:
            return True

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2 * self.interval + 1.0)


class StepWatchdog:
    """``with watchdog.step():`` arms a timer; if the block takes longer than ``limit`` seconds ``on_timeout`` runs in
    the timer thread (default: interrupt the main thread, which surfaces as ``KeyboardInterrupt`` there)."""

    def __init__(self, limit: float, on_timeout: Optional[Callable[[float], None]] = None) -> None:
        self.limit = float(limit)
        self.on_timeout = on_timeout or self._interrupt
        self.fired = False

    @staticmethod
    def _interrupt(limit: float) -> None:
        import _thread
        import sys
        print(f"[watchdog] step exceeded {limit:.0f}s -- interrupting", file=sys.stderr, flush=True)
        _thread.interrupt_main()

    def step(self):
        wd = self

        class _Armed:
            def __enter__(self_inner):
                wd.fired = False
                self_inner.t = threading.Timer(wd.limit, wd._fire)
                self_inner.t.daemon = True
                self_inner.t.start()
                return wd

            def __exit__(self_inner, *exc):
                self_inner.t.cancel()
                return False
        return _Armed()

    def _fire(self) -> None:
        self.fired = True
        self.on_timeout(self.limit)
