"""Host-side failure detection for multi-rank jobs; nothing here touches a GPU.

* :class:`StepWatchdog` — a thread with a per-step deadline.  The training loop calls ``beat()`` once per step; when
  no beat arrives within the deadline the watchdog dumps every Python thread's stack and the last known state, and
  exits the process with code 124 so that the launcher tears the job down.  The reference has no in-process hang
  detection (a dead peer leaves the others in cudaStreamSynchronize, training/distributed.cpp:157-199) and relies
  on its launcher; this is the in-process half of that.
* :class:`Heartbeat` — ranks publish a counter in the job's key-value store and read their peers' before each step.
  A peer whose counter stops, or that posted a failure, is reported *before* the next collective is launched, so no
  kernel waits on a rank that is gone.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time
from typing import Callable, Dict, List, Optional

EXIT_WATCHDOG = 124


class StepWatchdog:
    def __init__(self, deadline_s: float, describe: Optional[Callable[[], str]] = None, on_expire: Optional[Callable[[str], None]] = None,
                 first_step_factor: float = 4.0, stream=None):
        """``on_expire`` replaces the default action (dump + ``os._exit(124)``); tests pass a recorder."""
        if deadline_s <= 0:
            raise ValueError("watchdog deadline must be positive")
        self.deadline, self.describe, self.on_expire = float(deadline_s), describe, on_expire
        self.first_factor = max(1.0, first_step_factor)       # the first step compiles, captures graphs, opens shards
        self.stream = stream or sys.stderr
        self._last = time.monotonic()
        self._beats = 0
        self._paused = 0
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self.expired = False

    def start(self) -> "StepWatchdog":
        if self._thread is None:
            self._last = time.monotonic()
            self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
            self._thread.start()
        return self

    def beat(self) -> None:
        with self._lock:
            self._last = time.monotonic()
            self._beats += 1

    def hold(self) -> None:
        """Suspend the deadline for a phase with no step cadence (evaluation, checkpoint capture)."""
        with self._lock:
            self._paused = 1

    def release(self) -> None:
        with self._lock:
            if self._paused:
                self._paused = 0
                self._last = time.monotonic()

    def pause(self):
        """``with wd.pause():`` = hold() ... release()."""
        wd = self

        class _P:
            def __enter__(self):
                wd.hold()

            def __exit__(self, *a):
                wd.release()
        return _P()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None

    def _run(self):
        poll = min(1.0, self.deadline / 4.0)
        while not self._stop.wait(poll):
            with self._lock:
                idle = time.monotonic() - self._last
                limit = self.deadline * (self.first_factor if self._beats == 0 else 1.0)
                paused = self._paused > 0
            if paused or idle <= limit:
                continue
            self.expired = True
            msg = "[watchdog] no step finished for %.1f s (deadline %.1f s, %d steps done)" % (idle, limit, self._beats)
            if self.describe is not None:
                try:
                    msg += "\n[watchdog] state: " + self.describe()
                except Exception as e:                       # never let the report itself hide the hang
                    msg += "\n[watchdog] state unavailable: %r" % (e,)
            if self.on_expire is not None:
                self.on_expire(msg)
                return
            print(msg, file=self.stream, flush=True)
            try:
                faulthandler.dump_traceback(file=self.stream, all_threads=True)
            except Exception:
                pass
            os._exit(EXIT_WATCHDOG)


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, why: str):
        super().__init__("rank %d: %s" % (rank, why))
        self.rank, self.why = rank, why


class Heartbeat:
    """Liveness through a key-value store with ``set``/``get``/``add`` (torch.distributed's TCPStore, FileStore or
    HashStore).  ``check()`` raises :class:`PeerFailure` when a peer posted a failure, left, or made no progress for
    ``stale_s`` seconds."""

    def __init__(self, store, rank: int, world: int, stale_s: float = 60.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.stale, self.prefix = store, rank, world, float(stale_s), prefix
        self._seen: Dict[int, int] = {}
        self._when: Dict[int, float] = {}
        self._count = 0
        self.store.set(self._k(rank, "n"), "0")
        self.store.set(self._k(rank, "state"), "alive")

    def _k(self, rank: int, what: str) -> str:
        return "%s/%d/%s" % (self.prefix, rank, what)

    def beat(self) -> None:
        self._count += 1
        self.store.set(self._k(self.rank, "n"), str(self._count))

    def fail(self, why: str) -> None:
        self.store.set(self._k(self.rank, "state"), "failed:" + why[:200])

    def leave(self) -> None:
        """A rank that leaves between steps, with nothing of its own in flight, says so first."""
        self.store.set(self._k(self.rank, "state"), "left")

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            v = self.store.get(key)
        except Exception:
            return None
        return v.decode() if isinstance(v, (bytes, bytearray)) else str(v)

    def peers(self) -> List[dict]:
        out = []
        for r in range(self.world):
            out.append({"rank": r, "state": self._get(self._k(r, "state")), "beats": self._get(self._k(r, "n"))})
        return out

    def check(self) -> None:
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            state = self._get(self._k(r, "state"))
            if state is None:
                continue                                     # not joined yet: the rendezvous timeout covers that
            if state.startswith("failed:"):
                raise PeerFailure(r, state[7:] or "failed")
            if state == "left":
                raise PeerFailure(r, "left the job")
            n = int(self._get(self._k(r, "n")) or 0)
            if self._seen.get(r) != n:
                self._seen[r], self._when[r] = n, now
            elif now - self._when.get(r, now) > self.stale:
                raise PeerFailure(r, "no heartbeat for %.0f s (stuck at step %d)" % (now - self._when[r], n))
