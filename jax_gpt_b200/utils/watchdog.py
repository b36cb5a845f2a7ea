"""Failure detection on the host: heartbeats in the rendezvous store and a coordinated abort.

Every rank runs a daemon thread that writes a monotonically increasing beat under its key in a
``torch.distributed`` store (TCPStore / FileStore) and checks the beats of all other ranks. A
rank whose beat was seen and then has not moved for ``timeout`` seconds is reported dead (one that was never
seen gets the longer ``startup_grace``; one that wrote its done key on a clean exit is not reported): the watchdog sets an
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
    """``timeout`` bounds the silence of a peer that HAS been seen beating; a peer that has not written its first
    beat yet (slow import, CUDA initialisation, launcher skew) is given the separate, longer ``startup_grace``.
    ``stop()`` writes a done key, so a rank that finishes cleanly is not mistaken for a dead one."""

    def __init__(self, store, rank: int, world: int, interval: float = 1.0, timeout: float = 10.0,
                 on_failure: Optional[Callable[[List[int]], None]] = None, prefix: str = "b200_hb",
                 startup_grace: float = 300.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.on_failure, self.prefix = interval, timeout, on_failure, prefix
        self.startup_grace = startup_grace
        self._beat = 0
        self._stop = threading.Event()
        self._dead: List[int] = []
        self._t0 = time.monotonic()
        self._seen = {r: (None, None) for r in range(world)}      # rank -> (last beat value, when it last moved)
        self._done: set = set()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def _done_key(self, r):
        return f"{self.prefix}/done/{r}"

    def start(self):
        self.store.set(self._key(self.rank), "0")
        self._thread.start()
        return self

    def stop(self):
        """Clean exit: peers that read the done key stop expecting beats from this rank."""
        try:
            self.store.set(self._done_key(self.rank), "1")
        except Exception:
            pass
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=self.interval * 4)

    def _get(self, key):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def peers_seen(self) -> List[int]:
        """Ranks whose first beat this rank has observed (or that finished cleanly)."""
        return sorted(r for r in range(self.world)
                      if r != self.rank and (self._seen[r][0] is not None or r in self._done))

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
                if r == self.rank or r in self._done:
                    continue
                v = self._get(self._key(r))
                last_v, last_t = self._seen[r]
                if v is not None and v != last_v:
                    self._seen[r] = (v, now)
                    continue
                if self._get(self._done_key(r)) is not None:
                    self._done.add(r)
                elif last_t is None:
                    if now - self._t0 > self.startup_grace:        # never seen at all
                        dead.append(r)
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
