"""3-D process mesh over ``torch.distributed``: tensor x pipeline x data parallel.

Rank order matches the reference so that per-rank checkpoint files stay interchangeable
(src/parallel/comms.cu:79-96):  ``rank = dp_rank * (pp * tp) + stage * tp + tp_rank`` -- TP
innermost, so a TP group is a run of adjacent GPUs.  Process groups:

* ``tp_group``   ranks that share (dp_rank, stage)
* ``dp_group``   ranks that share (stage, tp_rank)
* ``tie_group``  first and last stage of one pipeline (same dp_rank, tp_rank); carries the
                 gradient exchange that keeps the embedding and the head tied
* ``pp_group``   all stages of one pipeline (same dp_rank, tp_rank), group rank = stage; used to
  exchange the addresses of the stage mailboxes
* pipeline neighbours are ``rank -/+ tp`` on the world group (src/pp_train.c:27)

One process per GPU; bootstrap is the TCP store of ``torchrun`` (the reference used MPI only
to broadcast the NCCL id, comms.cu:17-29).  Backend ``nccl`` on GPUs, ``gloo`` on CPU ranks.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class Coord:
    rank: int
    world: int
    tp: int
    pp: int
    dp: int

    @property
    def tp_rank(self):
        return self.rank % self.tp

    @property
    def stage(self):
        return (self.rank // self.tp) % self.pp

    @property
    def dp_rank(self):
        return self.rank // (self.tp * self.pp)

    @property
    def first(self):
        return self.stage == 0

    @property
    def last(self):
        return self.stage == self.pp - 1

    @property
    def prev_rank(self):
        return self.rank - self.tp

    @property
    def next_rank(self):
        return self.rank + self.tp


def rank_of(dp_rank, stage, tp_rank, tp, pp):
    return dp_rank * (pp * tp) + stage * tp + tp_rank


class Mesh:
    """Holds the coordinate of this process and its process groups.  ``Mesh.single()`` is the
    degenerate one-process mesh that needs no process group at all."""

    def __init__(self, tp=1, pp=None, dp=1, timeout_s=600):
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        if pp is None:
            pp = self.world // (tp * dp)
        if tp * pp * dp != self.world:
            raise ValueError("mesh %dx%dx%d does not cover %d ranks" % (tp, pp, dp, self.world))
        self.c = Coord(self.rank, self.world, tp, pp, dp)
        self.tp_group = self.dp_group = self.tie_group = self.pp_group = None
        to = datetime.timedelta(seconds=timeout_s)
        # every rank must create every group, in the same order
        for d in range(dp):
            for s in range(pp):
                ranks = [rank_of(d, s, t, tp, pp) for t in range(tp)]
                g = dist.new_group(ranks, timeout=to) if tp > 1 else None
                if self.rank in ranks:
                    self.tp_group = g
        for s in range(pp):
            for t in range(tp):
                ranks = [rank_of(d, s, t, tp, pp) for d in range(dp)]
                g = dist.new_group(ranks, timeout=to) if dp > 1 else None
                if self.rank in ranks:
                    self.dp_group = g
        if pp > 1:
            for d in range(dp):
                for t in range(tp):
                    ranks = [rank_of(d, 0, t, tp, pp), rank_of(d, pp - 1, t, tp, pp)]
                    g = dist.new_group(ranks, timeout=to)
                    if self.rank in ranks:
                        self.tie_group = g
            for d in range(dp):         # all stages of one pipeline, group rank = stage
                for t in range(tp):
                    ranks = [rank_of(d, s, t, tp, pp) for s in range(pp)]
                    g = dist.new_group(ranks, timeout=to)
                    if self.rank in ranks:
                        self.pp_group = g

    @classmethod
    def single(cls):
        m = cls.__new__(cls)
        m.world, m.rank = 1, 0
        m.c = Coord(0, 1, 1, 1, 1)
        m.tp_group = m.dp_group = m.tie_group = m.pp_group = None
        return m

    def describe(self):
        c = self.c
        return "tp%d x pp%d x dp%d (rank %d = dp%d/stage%d/tp%d)" % (c.tp, c.pp, c.dp, c.rank, c.dp_rank, c.stage,
                                                                   c.tp_rank)


def init_distributed(device_type=None, timeout_s=600):
    """Join the job described by the torchrun environment.  Returns (rank, world, device).  The
    collective / store time-out is ``timeout_s`` seconds unless KHARON_DIST_TIMEOUT_S overrides it."""
    timeout_s = int(os.environ.get("KHARON_DIST_TIMEOUT_S", timeout_s))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() if device_type is None else device_type == "cuda"
    if use_cuda:
        torch.cuda.set_device(local % torch.cuda.device_count())
        device = torch.device("cuda", local % torch.cuda.device_count())
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, device
