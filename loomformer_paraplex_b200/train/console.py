"""Console interaction of the trainer: graceful Ctrl-C (first press finishes the step and asks whether to save,
second press restores the default handler) and an ``s`` key watcher that requests an asynchronous run-point
(reference ``loomformer.py:4526-4657``).  Only rank 0 touches the terminal."""
from __future__ import annotations

import signal
import sys
import threading
from typing import Optional

from ..parallel import dist as pdist


class GracefulInterrupt:
    def __init__(self) -> None:
        self.requested, self._hits, self._prev = False, 0, None

    def _on_sigint(self, signum, frame) -> None:
        self._hits += 1
        if self._hits >= 2 and callable(self._prev):
            signal.signal(signal.SIGINT, self._prev)
            self._prev(signum, frame)
            return
        self.requested = True

    def __enter__(self):
        try:
            self._prev = signal.getsignal(signal.SIGINT)
            signal.signal(signal.SIGINT, self._on_sigint)
        except ValueError:          # not the main thread
            self._prev = None
        return self

    def __exit__(self, *exc) -> None:
        if self._prev is not None:
            signal.signal(signal.SIGINT, self._prev)


class RunpointWatcher:
    def __init__(self) -> None:
        self._flag, self._stop = threading.Event(), threading.Event()
        self._saved, self._thread, self._active = None, None, False

    def _loop(self) -> None:
        import select
        while not self._stop.is_set():
            try:
                ready, _, _ = select.select([sys.stdin], [], [], 0.05)
                if not ready:
                    continue
                ch = sys.stdin.read(1)
            except Exception:
                return
            if not ch:
                return
            if ch.lower() == "s":
                self._flag.set()

    def _raw_mode(self) -> bool:
        try:
            import termios
            import tty
            tty.setcbreak(sys.stdin.fileno())
            attrs = termios.tcgetattr(sys.stdin)
            attrs[3] &= ~termios.ECHO
            termios.tcsetattr(sys.stdin, termios.TCSADRAIN, attrs)
            return True
        except Exception:
            return False

    def _restore(self) -> None:
        if self._saved is not None:
            try:
                import termios
                termios.tcsetattr(sys.stdin, termios.TCSADRAIN, self._saved)
            except Exception:
                pass

    def _start(self) -> None:
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def __enter__(self):
        if not pdist.is_main():
            return self
        try:
            import termios
            if not sys.stdin.isatty():
                return self
            self._saved = termios.tcgetattr(sys.stdin)
        except Exception:
            return self
        if self._raw_mode():
            self._active = True
            self._start()
        return self

    def pause(self) -> None:
        if self._active:
            self._stop.set()
            if self._thread is not None:
                self._thread.join(timeout=0.5)
            self._restore()

    def resume(self) -> None:
        if self._active and self._raw_mode():
            self._start()

    def consume(self) -> bool:
        if self._flag.is_set():
            self._flag.clear()
            return True
        return False

    def __exit__(self, *exc) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=0.5)
        self._restore()
        self._active = False
