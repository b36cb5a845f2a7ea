"""Failure detection on the host: heartbeats in the rendezvous store and a coordinated abort.

Every rank runs a daemon thread that writes a monotonically increasing beat under its key in a
``torch.distributed`` store (TCPStore / FileStore) and checks the beats of all other ranks. A
rank whose beat has not moved for ``timeout`` seconds is reported dead: the watchdog sets an
abort key so that every surviving rank sees it before its next step (``check()`` raises
:class:`PeerFailure`), after which the job restarts from the last complete checkpoint. Device
side, every kernel wait in this package is bounded and reports through a status word, so a
missing peer surfaces as an error code rather than a hung GPU.

The reference relies on the cluster scheduler restarting the whole gang
(k8s/qwen35_eval_jobset.yaml:84-100) and has no in-process detection.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional


class PeerFailure(RuntimeError):
    def __init__(self, dead: List[int], reason: str = ""):
        super().__init__(f"ranks {dead} stopped responding{(': ' + reason) if reason else ''}")
        self.dead = dead


class Watchdog:
    def __init__(self, store, rank: int, world: int, interval: float = 1.0, timeout: float = 10.0,
                 on_failure: Optional[Callable[[List[int]], None]] = None, prefix: str = "b200_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.on_failure, self.prefix = interval, timeout, on_failure, prefix
        self._beat = 0
        self._stop = threading.Event()
        self._dead: List[int] = []
        self._seen = {r: (None, time.monotonic()) for r in range(world)}
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def start(self):
        self.store.set(self._key(self.rank), "0")
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=self.interval * 4)

    def _get(self, key):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def _run(self):
        while not self._stop.is_set():
            self._beat += 1
            try:
                self.store.set(self._key(self.rank), str(self._beat))
            except Exception:
                pass
            now = time.monotonic()
            dead = []
            for r in range(self.world):
                if r == self.rank:
                    continue
                v = self._get(self._key(r))
                last_v, last_t = self._seen[r]
                if v is not None and v != last_v:
                    self._seen[r] = (v, now)
                elif now - last_t > self.timeout:
                    dead.append(r)
            if self._get(f"{self.prefix}/abort") is not None and not dead:
                dead = [int(x) for x in self._get(f"{self.prefix}/abort").split(",") if x]
            if dead and not self._dead:
                self._dead = dead
                try:
                    self.store.set(f"{self.prefix}/abort", ",".join(str(d) for d in dead))
                except Exception:
                    pass
                if self.on_failure is not None:
                    self.on_failure(dead)
            self._stop.wait(self.interval)

    def check(self):
        """Call between steps: raises :class:`PeerFailure` once a peer is known to be gone."""
        if self._dead:
            raise PeerFailure(self._dead)

    @property
    def dead_ranks(self) -> List[int]:
        return list(self._dead)
