"""Host-side failure detection: a stall watchdog and a heartbeat-based rank monitor.

* ``StallWatchdog`` is the in-process thread the reference's stress tests start to find hangs
  (tests/test_dispatch_grads_stress.py:53-174): if ``heartbeat()`` is not called for ``timeout_s``
  it dumps every Python thread's stack and the kernel wait channel of every OS thread, then calls
  ``on_stall``.
* ``RankMonitor`` lets ranks learn ON THE HOST that a peer is gone before they launch the next
  collective kernel: every rank stamps a key in a ``torch.distributed`` store; a rank whose stamp
  is older than the limit is reported dead.  (Device-side waits are bounded as well and report
  through ``Buffer.check_status``; this covers the case where nothing was launched yet.)
"""
from __future__ import annotations

import faulthandler
import glob
import io
import os
import sys
import threading
import time
from typing import Callable, List, Optional


class StallWatchdog:
    def __init__(self, timeout_s: float, on_stall: Optional[Callable[[str], None]] = None,
                 stream=None, poll_s: float = 0.05):
        self.timeout_s = float(timeout_s)
        self.on_stall = on_stall
        self.stream = stream if stream is not None else sys.stderr
        self.poll_s = poll_s
        self._last = time.monotonic()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.stalls = 0

    def heartbeat(self) -> None:
        self._last = time.monotonic()

    def _report(self) -> str:
        buf = io.StringIO()
        buf.write(f"[streamep watchdog] no heartbeat for {self.timeout_s:.1f}s in pid {os.getpid()}\n")
        try:
            tmp = os.tmpfile() if hasattr(os, "tmpfile") else None
        except OSError:
            tmp = None
        import tempfile
        with tempfile.TemporaryFile(mode="w+") as f:
            faulthandler.dump_traceback(file=f, all_threads=True)
            f.seek(0)
            buf.write(f.read())
        for path in sorted(glob.glob("/proc/self/task/*/wchan")):
            try:
                with open(path) as f:
                    buf.write(f"{path.split('/')[4]}: wchan={f.read().strip() or '-'}\n")
            except OSError:
                pass
        _ = tmp
        return buf.getvalue()

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            if time.monotonic() - self._last > self.timeout_s:
                self.stalls += 1
                text = self._report()
                try:
                    self.stream.write(text)
                    self.stream.flush()
                except (OSError, ValueError):
                    pass
                if self.on_stall is not None:
                    self.on_stall(text)
                self._last = time.monotonic()

    def start(self) -> "StallWatchdog":
        self._thread = threading.Thread(target=self._run, name="streamep-watchdog", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()


class RankMonitor:
    """Liveness of the ranks of a group through a key-value store (``dist.TCPStore``,
    ``dist.FileStore``, or the store of the default process group)."""

    def __init__(self, store, rank: int, world_size: int, prefix: str = "streamep/hb", period_s: float = 0.2):
        self.store, self.rank, self.world_size, self.prefix, self.period_s = store, rank, world_size, prefix, period_s
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.beat()

    def beat(self) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", repr(time.time()))

    def start(self) -> "RankMonitor":
        def run():
            while not self._stop.wait(self.period_s):
                try:
                    self.beat()
                except Exception:  # noqa: BLE001  (store gone: the job is ending)
                    return
        self._thread = threading.Thread(target=run, name="streamep-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def mark_leaving(self) -> None:
        """Announce an orderly exit between steps (no kernels in flight)."""
        self.stop()
        self.store.set(f"{self.prefix}/{self.rank}", "left")

    def dead_ranks(self, limit_s: float = 2.0) -> List[int]:
        now = time.time()
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"{self.prefix}/{r}").decode()
            except Exception:  # noqa: BLE001
                dead.append(r)
                continue
            if v == "left" or now - float(v) > limit_s:
                dead.append(r)
        return dead

    def assert_all_alive(self, limit_s: float = 2.0) -> None:
        from ..errors import StreamEPError
        dead = self.dead_ranks(limit_s)
        if dead:
            raise StreamEPError(f"rank(s) {dead} stopped sending heartbeats: not launching the next collective")
