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
        self.store.add("hb/%d" % rank, 1)
        self._t = threading.Thread(target=self._beat, daemon=True)
        self._t.start()

    def _beat(self):
        while not self._stop.wait(self.interval):
            try:
                self.store.add("hb/%d" % self.rank, 1)
            except Exception:
                return

    def stop(self):
        self._stop.set()

    def dead_ranks(self):
        now = time.monotonic()
        dead = []
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

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure("ranks %s stopped sending heartbeats" % dead)
