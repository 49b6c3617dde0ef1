"""ctypes bindings to the two native libraries (host runtime, CUDA kernels).

``rt()`` returns the host runtime (built on demand with g++; needs no GPU).  ``cuda()``
returns the CUDA kernel library; on a machine with a GPU a missing library is a hard
error -- no operation silently falls back to PyTorch there.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from . import _build

_lock = threading.Lock()
_rt = None
_cuda = None

i32, i64, u32, u64, f32 = C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float
vp, cp = C.c_void_p, C.c_char_p
P = C.POINTER


class NativeError(RuntimeError):
    pass


def _sig(lib, name, res, *args):
    fn = getattr(lib, name)
    fn.restype = res
    fn.argtypes = list(args)
    return fn


def rt():
    global _rt
    if _rt is not None:
        return _rt
    with _lock:
        if _rt is not None:
            return _rt
        path = _build.build_runtime()
        lib = C.CDLL(str(path))
        _sig(lib, "kh_last_error", cp)
        _sig(lib, "kh_rng_seed", None, P(u64), u64)
        _sig(lib, "kh_rng_u32", u32, P(u64))
        _sig(lib, "kh_rng_batch", None, P(u64), vp, vp, i64, i32)
        _sig(lib, "kh_fill_normal", None, P(u64), vp, i64, f32)
        _sig(lib, "kh_fill_normal_block", None, P(u64), vp, i64, i64, i64, i64, i64, i64, f32)
        _sig(lib, "kh_layout_params", i32, P(i32), i32, i32, i32, P(i64), P(i64), i32, P(i64))
        _sig(lib, "kh_data_open", vp, cp, i32)
        _sig(lib, "kh_data_size", i64, vp)
        _sig(lib, "kh_data_next", None, vp, P(u64), i32, vp, vp)
        _sig(lib, "kh_data_close", None, vp)
        _sig(lib, "kh_ckpt_save", i32, cp, P(i32), i32, u64, u64, u64, vp, vp, vp)
        _sig(lib, "kh_ckpt_peek", i32, cp, P(i32), P(i32), P(u64), P(u64), P(u64))
        _sig(lib, "kh_ckpt_load", i32, cp, P(i32), u64, u64, P(i32), P(u64), vp, vp, vp)
        _sig(lib, "kh_ref_load", vp, cp)
        _sig(lib, "kh_ref_free", None, vp)
        _sig(lib, "kh_ref_header", None, vp, P(i32), P(f32))
        _sig(lib, "kh_ref_count", i32, vp)
        _sig(lib, "kh_ref_name", cp, vp, i32)
        _sig(lib, "kh_ref_ndim", i32, vp, i32)
        _sig(lib, "kh_ref_dims", None, vp, i32, P(i32))
        _sig(lib, "kh_ref_dtype", i32, vp, i32)
        _sig(lib, "kh_ref_data", vp, vp, i32)
        _sig(lib, "kh_ref_find", i32, vp, cp)
        _sig(lib, "kh_grpo_advantages", None, vp, i32, i32, f32, vp)
        _sig(lib, "kh_grpo_coef", None, vp, vp, vp, i32, i32, i32, i32, f32, vp)
        _sig(lib, "kh_pp_schedule", i32, i32, i32, i32, vp, i32)
        _sig(lib, "kh_pp_num_slots", i32, i32, i32, i32)
        _sig(lib, "kh_pp_schedule_deferred", i32, i32, i32, i32, i32, i32, vp, i32)
        _sig(lib, "kh_eng_create", vp, i32, i32, i32, i32)
        _sig(lib, "kh_eng_free", None, vp)
        _sig(lib, "kh_eng_reset", None, vp)
        _sig(lib, "kh_eng_add", i32, vp, vp, i32, i32)
        _sig(lib, "kh_eng_fork", i32, vp, i32, i32, i32, vp)
        _sig(lib, "kh_eng_push", i32, vp, i32, i32)
        _sig(lib, "kh_eng_set_eos", None, vp, i32)
        _sig(lib, "kh_eng_plan", i32, vp, i32, i32, vp, vp, vp, vp, vp, vp, P(i32), P(i32), vp, i32, P(i32))
        _sig(lib, "kh_eng_commit", i32, vp, vp, i32)
        _sig(lib, "kh_eng_seq_len", i32, vp, i32)
        _sig(lib, "kh_eng_seq_tokens", i32, vp, i32, vp, i32)
        _sig(lib, "kh_eng_seq_done", i32, vp, i32)
        _sig(lib, "kh_eng_release", None, vp, i32)
        _sig(lib, "kh_eng_stats", None, vp, P(i64))
        _sig(lib, "kh_eng_blocks_in_use", i32, vp)
        _sig(lib, "kh_eng_block_ref", i32, vp, i32)
        _rt = lib
        return lib


def rt_check(rc: int) -> int:
    """Raise NativeError carrying the runtime's message when ``rc`` is negative."""
    if rc < 0:
        raise NativeError(rt().kh_last_error().decode())
    return rc


def cuda_lib_path() -> Path:
    return _build.LIB / "libkharon_cuda.so"


def cuda():
    """The CUDA kernel library.  Built on demand when nvcc is present; raises otherwise."""
    global _cuda
    if _cuda is not None:
        return _cuda
    with _lock:
        if _cuda is not None:
            return _cuda
        path = cuda_lib_path()
        if not path.exists():
            path = _build.build_cuda()
        lib = C.CDLL(str(path))
        from .ops import _sigs
        _sigs.declare(lib)
        _cuda = lib
        return lib
