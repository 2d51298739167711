"""Host-side membership: who is still in the job.

The reference sets ``MPI.ERRORS_RETURN`` and accepts an ``err_handler`` that it
never calls (allreducer.py:173-174,202,212; gtopk_trainer.py:42-44).  Here a
rank that leaves between two iterations says so in the job's key-value store,
and every rank looks at the store before it launches the next exchange, so a
departure is noticed on the host in well under a second instead of through a
device-side wait running out.  A rank that dies without saying goodbye is
caught by its heartbeat going stale, and, as the last resort, by the bounded
waits of the exchange itself.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional

import torch.distributed as dist


class PeerLeft(RuntimeError):
    """One or more ranks left the job (or stopped beating).  ``planned`` is set
    when every survivor learns of the departure at the same iteration (the
    leaver announced it ahead of time), which is what re-forming a smaller job
    needs."""

    def __init__(self, ranks: List[int], why: str, planned: bool = False):
        super().__init__("ranks %s %s" % (ranks, why))
        self.ranks = ranks
        self.planned = planned


def default_store():
    """The key-value store behind the default process group, or None."""
    if not dist.is_initialized():
        return None
    try:
        from torch.distributed.distributed_c10d import _get_default_store
        return dist.PrefixStore("gtopk_membership/", _get_default_store())
    except Exception:  # a build without that accessor: no membership service
        return None


class Membership:
    def __init__(self, store, rank: int, world: int, stale_after_s: float = 60.0, check_every: int = 10):
        self.store, self.rank, self.world = store, rank, world
        self.stale_after_s, self.check_every = stale_after_s, max(int(check_every), 1)
        self._calls = 0
        self._left_sent = False
        self._leave_at: Optional[int] = None
        self._planned: dict = {}
        self._dropped: set = set()
        if store is not None:
            self.beat(0)

    @classmethod
    def for_default_group(cls, **kw) -> Optional["Membership"]:
        store = default_store()
        if store is None or dist.get_world_size() < 2:
            return None
        return cls(store, dist.get_rank(), dist.get_world_size(), **kw)

    # -- this rank --------------------------------------------------------------------------
    def beat(self, step: int) -> None:
        self.store.set("hb/%d" % self.rank, "%d:%.3f" % (step, time.time()))

    def leave(self) -> None:
        """Announce an orderly departure (call between iterations, nothing in flight)."""
        if not self._left_sent and self.store is not None:
            try:
                self.store.set("left/%d" % self.rank, "1")
            except Exception:
                pass  # the store's host may already be gone at shutdown
            self._left_sent = True

    def announce_leave(self, step: int) -> int:
        """Planned departure: this rank keeps working up to, and not including,
        the returned iteration.  That iteration is the second next check point
        of the survivors, so each of them reads the announcement at the check
        point in between and all of them drop this rank at the same iteration."""
        ce = self.check_every
        at = (step // ce + 2) * ce
        self.store.set("leave_at/%d" % self.rank, str(at))
        self._leave_at = at
        return at

    # -- the others ---------------------------------------------------------------------------
    def departed(self) -> List[int]:
        return [q for q in range(self.world) if q != self.rank and self.store.check(["left/%d" % q])]

    def planned(self) -> dict:
        """{rank: iteration} of the announced departures seen so far."""
        for q in range(self.world):
            if q != self.rank and q not in self._planned and self.store.check(["leave_at/%d" % q]):
                self._planned[q] = int(self.store.get("leave_at/%d" % q).decode())
        return self._planned

    def stale(self, now: Optional[float] = None) -> List[int]:
        now = time.time() if now is None else now
        out = []
        for q in range(self.world):
            if q == self.rank or not self.store.check(["hb/%d" % q]):
                continue
            stamp = float(self.store.get("hb/%d" % q).decode().split(":")[1])
            if now - stamp > self.stale_after_s:
                out.append(q)
        return out

    def check(self, step: int, force: bool = False) -> None:
        """Called at the top of an iteration, before anything is launched.
        Every ``check_every`` calls: beat, then raise PeerLeft if somebody left
        or went silent."""
        self._calls += 1
        due = sorted(q for q, at in self._planned.items() if step >= at)
        if due:  # announced earlier, effective now: the same on every survivor
            for q in due:
                del self._planned[q]
            self._dropped.update(due)
            raise PeerLeft(due, "left the job as announced", planned=True)
        if not force and step % self.check_every:
            return
        self.beat(step)
        self.planned()
        gone = [q for q in self.departed() if q not in self._dropped]
        if gone:
            raise PeerLeft(gone, "left the job")
        silent = self.stale()
        if silent:
            raise PeerLeft(silent, "stopped sending heartbeats")


class StreamWatchdog:
    """Host thread that watches the device work of the last iteration.

    After an iteration has been enqueued the trainer records an event behind it
    and calls ``arm(event)``; the thread polls ``event.query()`` and, if the
    event has not completed ``limit_s`` seconds later, calls ``on_stall(seconds)``
    once.  Every device-side wait of the exchange is bounded, so the event does
    complete eventually; the watchdog reports a stream that is stuck for another
    reason (a peer process stopped inside a library collective, a wedged
    driver call) while the Python thread sits in a blocking read.

    ``pause()`` / ``resume()`` bracket CUDA-graph capture: a query from another
    thread during a global-mode capture would invalidate the capture, so while
    paused the thread makes no CUDA call at all (``pause`` returns only after a
    query in flight has finished).
    """

    def __init__(self, limit_s: float, on_stall: Callable[[float], None], poll_s: float = 0.25):
        self.limit_s, self.poll_s, self.on_stall = float(limit_s), float(poll_s), on_stall
        self._lock = threading.Lock()
        self._event = None
        self._armed_at = 0.0
        self._paused = False
        self._stop = threading.Event()
        self.stalls = 0
        self._thread = threading.Thread(target=self._run, name="gtopk-watchdog", daemon=True)
        self._thread.start()

    def arm(self, event) -> None:
        with self._lock:
            if not self._paused:
                self._event, self._armed_at = event, time.monotonic()

    def disarm(self) -> None:
        with self._lock:
            self._event = None

    def pause(self) -> None:
        with self._lock:
            self._paused, self._event = True, None

    def resume(self) -> None:
        with self._lock:
            self._paused = False

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2.0)

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            fire = None
            with self._lock:
                if self._paused or self._event is None:
                    continue
                if self._event.query():
                    self._event = None
                    continue
                waited = time.monotonic() - self._armed_at
                if waited > self.limit_s:
                    self._event = None
                    self.stalls += 1
                    fire = waited
            if fire is not None:
                try:
                    self.on_stall(fire)
                except Exception:  # a reporting problem must not end the thread
                    pass
