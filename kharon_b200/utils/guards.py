"""Guard-band canaries for device buffers (debug aid standing in for compute-sanitizer, which is not
available on the build pool).  ``GuardedAlloc`` hands out tensors that sit between two 256-byte
bands filled with a known pattern; ``check()`` lists the buffers whose bands were overwritten, i.e.
out-of-bounds writes by a kernel.  Enable for a model with ``models.gpt.set_allocator(GuardedAlloc())``
before constructing it."""
from __future__ import annotations

import torch

GUARD = 256
PATTERN = 0xA5


class GuardedAlloc:
    def __init__(self):
        self.bufs = []          # (name, raw uint8 tensor, payload bytes)

    def empty(self, shape, dtype, device, name=""):
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        pad = (-nbytes) % 256
        raw = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device=device)
        self.bufs.append((name or "buf%d" % len(self.bufs), raw, nbytes))
        return raw[GUARD:GUARD + nbytes].view(dtype).view(*shape)

    def zeros(self, shape, dtype, device, name=""):
        t = self.empty(shape, dtype, device, name)
        t.zero_()
        return t

    def check(self):
        """Names of buffers with a damaged guard band (empty list = clean)."""
        bad = []
        for name, raw, nbytes in self.bufs:
            tail = raw[GUARD + nbytes:]
            if not (bool((raw[:GUARD] == PATTERN).all()) and bool((tail == PATTERN).all())):
                bad.append(name)
        return bad
