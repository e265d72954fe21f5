"""Host-side failure detection between the processes of a run.

Every process keeps a counter in a small TCP key-value store (rank 0 serves it, on its own port) and bumps it from a
background thread; before each optimizer step a process looks at the others' counters and failure notices. A peer that
posted a notice (it caught an exception and is leaving) or whose counter has not moved for ``timeout_s`` is reported as
``PeerFailure`` BEFORE this process enters the step's collectives, so the survivors leave between steps with none of
their kernels or collectives in flight instead of waiting inside a collective for a process that is gone. Counters,
not clocks, are compared, so hosts need no common time. Nothing here touches a GPU.

(The reference has no watchdog beyond NCCL's own and polls only for SIGTERM, src/pretrain/train/loop.py:1087-1106; this
module is the host-side detector that a box of shared GPUs calls for.)
"""
from __future__ import annotations

import datetime
import threading
import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__("process %d is gone: %s" % (rank, reason))
        self.rank, self.reason = rank, reason


class Heartbeat:
    def __init__(self, rank: int, world: int, host: str, port: int, interval_s: float = 0.5, timeout_s: float = 10.0,
                 connect_timeout_s: float = 60.0):
        self.rank, self.world, self.interval_s, self.timeout_s = rank, world, interval_s, timeout_s
        self.store = dist.TCPStore(host, port, world, rank == 0, timeout=datetime.timedelta(seconds=connect_timeout_s),
                                   wait_for_workers=False)
        self._stop = threading.Event()
        self._count = 0
        self._seen: dict[int, tuple[int, float]] = {}  # peer -> (last counter value, local time it changed)
        self._beat()
        self._thread = threading.Thread(target=self._run, name="otb-heartbeat", daemon=True)
        self._thread.start()

    def _beat(self) -> None:
        self._count += 1
        self.store.set("hb/%d" % self.rank, str(self._count))

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self._beat()
            except Exception:  # the store is gone: the run is ending
                return

    def report_failure(self, reason: str) -> None:
        """Tell the others that this process is leaving because of ``reason`` (call from an exception handler)."""
        try:
            self.store.set("failed/%d" % self.rank, reason[:2000])
        except Exception:
            pass

    def check(self) -> None:
        """Raise ``PeerFailure`` if a peer posted a failure notice or stopped beating; call between steps."""
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check(["failed/%d" % r]):
                raise PeerFailure(r, self.store.get("failed/%d" % r).decode(errors="replace"))
            if not self.store.check(["hb/%d" % r]):
                first = self._seen.setdefault(r, (0, now))
                if now - first[1] > self.timeout_s:
                    raise PeerFailure(r, "never reported in within %.1f s" % self.timeout_s)
                continue
            value = int(self.store.get("hb/%d" % r))
            last = self._seen.get(r)
            if last is None or last[0] != value:
                self._seen[r] = (value, now)
            elif now - last[1] > self.timeout_s:
                raise PeerFailure(r, "no heartbeat for %.1f s" % (now - last[1]))

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2 * self.interval_s + 1.0)
