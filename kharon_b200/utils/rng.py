"""xorshift64* stream and the samplers built on it (native: csrc/runtime/kharon_rt.cpp).

The state is a single u64, which is what the CKP1 header stores, so a resumed run draws the
same batches as an uninterrupted one.  Mirrors src/core/rng.h:7-22 of the reference.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .. import _native


class Rng:
    def __init__(self, seed: int = 0):
        self._s = C.c_uint64(0)
        _native.rt().kh_rng_seed(C.byref(self._s), seed)

    @property
    def state(self) -> int:
        return int(self._s.value)

    @state.setter
    def state(self, v: int):
        self._s.value = int(v) & 0xFFFFFFFFFFFFFFFF

    def u32(self) -> int:
        return int(_native.rt().kh_rng_u32(C.byref(self._s)))

    def batch(self, n: int, vocab: int):
        """n input ids then n target ids, each uniform in [0, vocab) (int32 CPU tensors)."""
        idx = torch.empty(n, dtype=torch.int32)
        tgt = torch.empty(n, dtype=torch.int32)
        _native.rt().kh_rng_batch(C.byref(self._s), idx.data_ptr(), tgt.data_ptr(), n, vocab)
        return idx, tgt

    def batch_into(self, idx: torch.Tensor, tgt: torch.Tensor, vocab: int):
        _native.rt().kh_rng_batch(C.byref(self._s), idx.data_ptr(), tgt.data_ptr(), idx.numel(), vocab)

    def normal(self, n: int, std: float) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float32)
        _native.rt().kh_fill_normal(C.byref(self._s), out.data_ptr(), n, std)
        return out

    def normal_block(self, rows, cols, r0, r1, c0, c1, std, keep=True):
        """Advance the stream by a full [rows, cols] matrix; return block [r0:r1, c0:c1] or None."""
        out = torch.empty((r1 - r0, c1 - c0), dtype=torch.float32) if keep else None
        _native.rt().kh_fill_normal_block(C.byref(self._s), out.data_ptr() if keep else None, rows, cols, r0, r1,
                                          c0, c1, std)
        return out


class ByteData:
    """Whole byte corpus in RAM; a batch is B random windows of T+1 bytes (src/core/data.c:6-30)."""

    def __init__(self, path: str, B: int, T: int, seed: int):
        self._h = _native.rt().kh_data_open(str(path).encode(), T)
        if not self._h:
            raise _native.NativeError(_native.rt().kh_last_error().decode())
        self.B, self.T = B, T
        self.rng = Rng(seed)
        self.vocab = 256

    def next_into(self, idx: torch.Tensor, tgt: torch.Tensor):
        _native.rt().kh_data_next(self._h, C.byref(self.rng._s), self.B, idx.data_ptr(), tgt.data_ptr())

    def close(self):
        if self._h:
            _native.rt().kh_data_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SyntheticData:
    """Uniform random token ids from a seed (rng_batch, src/core/rng.h:19-22)."""

    def __init__(self, vocab: int, B: int, T: int, seed: int):
        self.vocab, self.B, self.T = vocab, B, T
        self.rng = Rng(seed)

    def next_into(self, idx: torch.Tensor, tgt: torch.Tensor):
        self.rng.batch_into(idx, tgt, self.vocab)

    def close(self):
        pass
