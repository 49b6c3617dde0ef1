"""CHRN fixture files (src/core/refio.c:5-72): ``"CHRN"``, i32 version, 6xi32 config, 5xf32
optimizer settings, then records ``{i32 name_len, name, i32 ndim, dims, i32 dtype, raw}``
terminated by ``name_len == -1``.  dtype 0 = f32, 1 = i32.  The writer is Python (fixtures come
from the PyTorch oracle), the reader is the native one.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np
import torch

from .. import _native


class Writer:
    def __init__(self, path, cfg, opt):
        self.f = open(path, "wb")
        self.f.write(b"CHRN")
        self.f.write(struct.pack("<i", 1))
        self.f.write(struct.pack("<6i", *[int(c) for c in cfg]))
        self.f.write(struct.pack("<5f", *[float(o) for o in opt]))

    def put(self, name: str, t):
        if not torch.is_tensor(t):
            t = torch.tensor(float(t), dtype=torch.float32)
        t = t.detach().cpu()
        if t.dtype in (torch.int64, torch.int32):
            arr, dt = t.to(torch.int32).numpy(), 1
        else:
            arr, dt = t.to(torch.float32).numpy(), 0
        nb = name.encode()
        self.f.write(struct.pack("<i", len(nb)))
        self.f.write(nb)
        self.f.write(struct.pack("<i", arr.ndim))
        for s in arr.shape:
            self.f.write(struct.pack("<i", s))
        self.f.write(struct.pack("<i", dt))
        self.f.write(np.ascontiguousarray(arr).tobytes())

    def close(self):
        self.f.write(struct.pack("<i", -1))
        self.f.close()


def load(path):
    """Returns (cfg list, opt list, {name: tensor})."""
    lib = _native.rt()
    h = lib.kh_ref_load(str(path).encode())
    if not h:
        raise _native.NativeError(lib.kh_last_error().decode())
    try:
        cfg = (C.c_int32 * 6)()
        opt = (C.c_float * 5)()
        lib.kh_ref_header(h, cfg, opt)
        out = {}
        for i in range(lib.kh_ref_count(h)):
            name = lib.kh_ref_name(h, i).decode()
            nd = lib.kh_ref_ndim(h, i)
            dims = (C.c_int32 * 4)()
            lib.kh_ref_dims(h, i, dims)
            shape = [dims[k] for k in range(nd)]
            n = int(np.prod(shape)) if nd else 1
            dt = np.int32 if lib.kh_ref_dtype(h, i) == 1 else np.float32
            buf = (C.c_char * (n * 4)).from_address(lib.kh_ref_data(h, i))
            arr = np.frombuffer(buf, dtype=dt, count=n).copy().reshape(shape)
            out[name] = torch.from_numpy(arr)
        return list(cfg), list(opt), out
    finally:
        lib.kh_ref_free(h)
