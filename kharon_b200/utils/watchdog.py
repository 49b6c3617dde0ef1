"""Rank liveness over the job's TCP store.

Every rank runs a daemon thread that bumps ``hb/<rank>`` in the ``torch.distributed`` store;
``dead_ranks()`` lists peers whose counter has not moved for ``timeout_s``.  A training loop
checks it between steps (before launching kernels that wait on peers) and raises
``RankFailure`` instead of entering a collective that could never complete.  The reference has
no failure detection: a dead rank leaves the others blocked inside NCCL (src/parallel/comms.cu:7-14
only prints and exits on local errors).  Faults are only ever observed or injected on the
host; nothing here touches the GPU.
"""
from __future__ import annotations

import threading
import time

import torch.distributed as dist


class RankFailure(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 10.0, store=None):
        self.rank, self.world = rank, world
        self.interval, self.timeout = interval_s, timeout_s
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self._stop = threading.Event()
        self._seen = {}        # rank -> (counter, time it last changed)
        self._lock = threading.Lock()
        self.store.add("hb/%d" % rank, 1)
        self._t = threading.Thread(target=self._beat, daemon=True)
        self._t.start()

    def _beat(self):
        while not self._stop.wait(self.interval):
            try:
                self.store.add("hb/%d" % self.rank, 1)
                self._poll()          # keep "last seen moving" current, so that one later query is enough
            except Exception:
                return

    def stop(self):
        self._stop.set()

    def _poll(self):
        """Read the peers' counters; returns the ranks whose counter has not moved for ``timeout`` seconds
        (or whose key cannot be read)."""
        now = time.monotonic()
        dead = []
        with self._lock:
            for r in range(self.world):
                if r == self.rank:
                    continue
                try:
                    c = self.store.add("hb/%d" % r, 0)
                except Exception:
                    dead.append(r)
                    continue
                last = self._seen.get(r)
                if last is None or last[0] != c:
                    self._seen[r] = (c, now)
                elif now - last[1] > self.timeout:
                    dead.append(r)
        return dead

    def dead_ranks(self):
        return self._poll()

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure("ranks %s stopped sending heartbeats" % dead)


class CollectiveTimeout(RuntimeError):
    pass


def abort_group(group=None):
    """Best effort: tear the communicator of ``group`` down so that kernels of a collective that can no
    longer complete leave the stream (NCCL: ncclCommAbort through the process group; other backends have
    nothing to abort).  Never raises."""
    try:
        pg = group if group is not None else dist.distributed_c10d._get_default_group()
        backend = pg._get_backend(__import__("torch").device("cuda")) if dist.get_backend(pg) == "nccl" else None
        if backend is not None and hasattr(backend, "abort"):
            backend.abort()
            return True
    except Exception:
        pass
    return False


def guarded(work, heartbeat=None, timeout_s=60.0, group=None, poll_s=0.02, what="collective"):
    """Wait for an asynchronous collective (``async_op=True`` work handle, or a list of them) the way a
    job that must not hang waits: poll its completion from the host, and between polls look at the
    peers' heartbeats.  A peer that died turns into ``RankFailure`` within the heartbeat time-out, a
    collective that does not finish within ``timeout_s`` into ``CollectiveTimeout``; in both cases the
    communicator is aborted first (the reference's NCCL_CK only prints and exits on a local error and
    blocks forever on a remote one, src/parallel/comms.cu:7-14)."""
    works = list(work) if isinstance(work, (list, tuple)) else [work]
    t0 = time.monotonic()
    while True:
        if all(w.is_completed() for w in works):
            for w in works:
                w.wait()            # surfaces an asynchronous error of the collective as an exception
            return
        if heartbeat is not None:
            dead = heartbeat.dead_ranks()
            if dead:
                abort_group(group)
                raise RankFailure("%s cannot complete: ranks %s stopped sending heartbeats" % (what, dead))
        if time.monotonic() - t0 > timeout_s:
            abort_group(group)
            raise CollectiveTimeout("%s did not complete within %.0f s" % (what, timeout_s))
        time.sleep(poll_s)
