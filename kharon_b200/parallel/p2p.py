"""Pipeline-stage message transports for schedules whose sends must not wait for the receiver.

``Mailbox``      product path on GPUs: every stage owns, in symmetric (peer-mapped) memory, one
                 slot per micro-batch and direction; the sender's ``kh_p2p_put`` kernel stores the
                 message straight into the receiver's slot over NVLink and raises the slot's
                 counter, the receiver's ``kh_p2p_wait`` kernel (bounded) sits in stream order in
                 front of the first consumer.  All calls are ordinary native launches with constant
                 arguments, so they are recorded in launch plans together with the compute.
``DistMailbox``  the same interface on ``torch.distributed`` isend/irecv for CPU ranks (gloo), where
                 an isend returns at once and completes in the background.

The reference exchanges these messages with blocking NCCL send/recv pairs on the compute stream
(src/parallel/comms.cu:58-74); that path is kept as the baseline transport of the engine.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops

WAIT_LIMIT_MS = 20000      # first-step set-up on a peer (plan recording, buffer exchange) can take seconds


class Mailbox:
    def __init__(self, mesh, device, n_slots, rows, cols, dtype=torch.bfloat16):
        from .fused import _symm_alloc
        c = mesh.c
        self.stage, self.P, self.n = c.stage, c.pp, n_slots
        self.rows, self.cols, self.dtype = rows, cols, dtype
        es = torch.empty(0, dtype=dtype).element_size()
        self.msg = (rows * cols * es + 255) // 256 * 256
        self.off_grad = n_slots * self.msg
        self.off_flag = 2 * n_slots * self.msg
        total = self.off_flag + 2 * n_slots * 4 + 256
        self.buf, self.h = _symm_alloc(total, device, mesh.pp_group)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.h.barrier()
        self.base = [int(p) for p in self.h.buffer_ptrs]          # index = stage
        # local words: put state [sent, ticket] per (direction, slot), expected count per (direction, slot)
        self.put_state = torch.zeros(2, n_slots, 2, dtype=torch.int32, device=device)
        self.expected = torch.zeros(2, n_slots, dtype=torch.int32, device=device)

    def _view(self, off):
        es = torch.empty(0, dtype=self.dtype).element_size()
        return self.buf[off:off + self.rows * self.cols * es].view(self.dtype).view(self.rows, self.cols)

    def act_in(self, i):
        return self._view(i * self.msg)

    def grad_in(self, i):
        return self._view(self.off_grad + i * self.msg)

    def _put(self, direction, i, src, peer):
        assert src.is_contiguous()
        dst = self.base[peer] + (self.off_grad if direction else 0) + i * self.msg
        flag = self.base[peer] + self.off_flag + 4 * (direction * self.n + i)
        ops.p2p_put(src, dst, flag, self.put_state[direction, i])

    def _wait(self, direction, i):
        flag = self.base[self.stage] + self.off_flag + 4 * (direction * self.n + i)
        ops.p2p_wait(flag, self.expected[direction, i], WAIT_LIMIT_MS)

    def send_act(self, i, src):
        self._put(0, i, src, self.stage + 1)

    def send_grad(self, i, src):
        self._put(1, i, src, self.stage - 1)

    def wait_act(self, i):
        self._wait(0, i)

    def wait_grad(self, i):
        self._wait(1, i)

    def finish(self):
        pass


class DistMailbox:
    def __init__(self, mesh, device, n_slots, rows, cols, dtype=torch.bfloat16):
        c = mesh.c
        self.prev, self.next = c.prev_rank, c.next_rank
        self.acts = [torch.empty(rows, cols, dtype=dtype, device=device) for _ in range(n_slots)]
        self.grads = [torch.empty(rows, cols, dtype=dtype, device=device) for _ in range(n_slots)]
        self.pending = []

    def act_in(self, i):
        return self.acts[i]

    def grad_in(self, i):
        return self.grads[i]

    def send_act(self, i, src):
        self.pending.append(dist.isend(src.clone(), self.next, tag=i))

    def send_grad(self, i, src):
        self.pending.append(dist.isend(src.clone(), self.prev, tag=4096 + i))

    def wait_act(self, i):
        dist.irecv(self.acts[i], self.prev, tag=i).wait()

    def wait_grad(self, i):
        dist.irecv(self.grads[i], self.next, tag=4096 + i).wait()

    def finish(self):
        for w in self.pending:
            w.wait()
        self.pending.clear()
