"""ZeRO-1 optimizer step fused into one kernel over NVLink peer memory (``csrc/comm/zero1.cu``).

The gradient arena and the bf16 compute copy of every data-parallel rank are allocated in
symmetric memory (``alloc`` is handed to ``ParamStore``); ``step`` launches the kernel that
reduce-scatters the gradients, applies AdamW to this rank's slice, pushes the bf16 weights to all
ranks and clears the gradients.  The NCCL reduce-scatter / all-gather path in ``TrainEngine`` is
the baseline it replaces.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native, ops
from .fused import _symm_alloc


class ZeroFused:
    def __init__(self, mesh, device):
        self.group = mesh.dp_group
        self.dp, self.rank = mesh.c.dp, mesh.c.dp_rank
        self.device = torch.device(device)
        self.ptrs = {}
        self.handles = []
        self.epoch = 0
        self.grid = 0

    def alloc(self, kind, n, dtype):
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        buf, h = _symm_alloc(nbytes, self.device, self.group)
        buf.zero_()
        self.handles.append((buf, h))
        self.ptrs[kind] = [int(p) for p in h.buffer_ptrs]
        return buf.view(dtype)

    def finalize(self):
        buf, h = _symm_alloc(256, self.device, self.group)
        buf.zero_()
        self.handles.append((buf, h))
        self.ptrs["ctr"] = [int(p) for p in h.buffer_ptrs]
        torch.cuda.synchronize(self.device)
        h.barrier()
        U = C.c_uint64 * self.dp
        self.c_g = U(*self.ptrs["g"])
        self.c_wb = U(*self.ptrs["wb"]) if "wb" in self.ptrs else None
        self.c_ctr = U(*self.ptrs["ctr"])
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # every CTA must be resident (the exit barrier spans the grid): the launch is cooperative and
        # the grid is capped by what the occupancy query says the device can hold
        lib = _native.cuda()
        fit = int(lib.kh_zero1_max_grid()) if hasattr(lib, "kh_zero1_max_grid") else 2 * sms
        self.grid = max(1, min(2 * sms, fit))

    def step(self, ps, shard, step_no, o):
        self.epoch += 1
        bc1 = 1.0 - o["beta1"] ** step_no
        bc2 = 1.0 - o["beta2"] ** step_no
        rc = _native.cuda().kh_zero1_step(self.c_g, self.c_wb, self.c_ctr, ps.w.data_ptr(), ps.m.data_ptr(),
                                          ps.v.data_ptr(), shard, self.dp, self.rank, o["lr"], o["beta1"], o["beta2"],
                                          o["eps"], o["wd"], bc1, bc2, self.epoch, self.grid,
                                          torch.cuda.current_stream().cuda_stream)
        ops._chk(rc)
