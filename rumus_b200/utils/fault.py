"""Failure detection and host-side fault injection.

The reference has none: a rank that dies leaves its peers blocked forever in
``Condvar::wait_while`` (rumus-distributed/src/collective.rs:64-66).  Here:

* every device-side wait is bounded and reports through a status word; ``check_device_status``
  turns a non-zero word into ``DeviceWaitTimeout`` on the host, with the context still usable;
* ``Heartbeat`` publishes a per-rank timestamp in the process group's key-value store from a
  background thread; ``check_peers`` — called between steps, before the next launch — raises
  ``PeerLost`` naming the ranks whose heartbeat is stale, so no kernel is launched that would wait
  for a dead peer;
* ``FaultInjector`` creates failures on the HOST only (delay a rank, make a rank leave between
  steps, stop its heartbeat); nothing here faults, traps or hangs a GPU.
"""
from __future__ import annotations

import os
import threading
import time
from typing import List, Optional

from ..ops import native


class PeerLost(RuntimeError):
    def __init__(self, ranks: List[int]):
        super().__init__(f"ranks {ranks} stopped sending heartbeats")
        self.ranks = ranks


def check_device_status(where: str = "") -> None:
    """Raise ``native.DeviceWaitTimeout`` if a bounded device-side wait ran out since the last check."""
    native.raise_on_status(where)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, timeout_s: float = 2.0,
                 prefix: str = "rb_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._beat()

    def _beat(self):
        self.store.set(f"{self.prefix}/{self.rank}", repr(time.time()))

    def _run(self):
        while not self._stop.wait(self.interval_s):
            if not self._paused.is_set():
                try:
                    self._beat()
                except Exception:
                    return

    def start(self) -> "Heartbeat":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()

    def pause(self) -> None:
        """Fault injection: keep running but stop publishing."""
        self._paused.set()

    def stale_peers(self) -> List[int]:
        now, out = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                t = float(self.store.get(f"{self.prefix}/{r}").decode())
            except Exception:
                out.append(r)
                continue
            if now - t > self.timeout_s:
                out.append(r)
        return out

    def check_peers(self) -> None:
        s = self.stale_peers()
        if s:
            raise PeerLost(s)


class FaultInjector:
    """``RB_FAULT`` = comma separated ``kind:rank:arg`` items, e.g. ``exit:1:3`` (rank 1 leaves
    after step 3), ``delay:0:0.5`` (rank 0 sleeps 0.5 s before every step), ``mute:1:2`` (rank 1
    stops its heartbeat after step 2)."""

    def __init__(self, rank: int, spec: Optional[str] = None):
        self.rank = rank
        self.items = []
        for item in (spec if spec is not None else os.environ.get("RB_FAULT", "")).split(","):
            if item.strip():
                kind, r, arg = item.split(":")
                if int(r) == rank:
                    self.items.append((kind, float(arg)))

    def before_step(self, step: int, heartbeat: Optional[Heartbeat] = None) -> bool:
        """Returns False when this rank should leave the job now (between steps)."""
        for kind, arg in self.items:
            if kind == "delay":
                time.sleep(arg)
            elif kind == "mute" and heartbeat is not None and step >= int(arg):
                heartbeat.pause()
            elif kind == "exit" and step >= int(arg):
                if heartbeat is not None:
                    heartbeat.stop()
                return False
        return True
