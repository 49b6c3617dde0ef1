"""CKP1 checkpoint files, byte-compatible with the reference (src/core/ckpt.c:25-68):

``"CKP1" | cfg 6xi32 | step i32 | rng u64 | pb u64 | ob u64 | params[pb] | m[ob] | v[ob]``

``pb`` is the byte size of the 256-byte-aligned fp32 parameter arena; ``ob`` equals ``pb``
or, under ZeRO-1, the byte size of this rank's moment shard.  Multi-rank runs write one file
per rank named ``<prefix>.r<rank>`` (src/pp_train.c:102).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native


def _cfg_arr(cfg):
    return (C.c_int32 * 6)(*[int(x) for x in cfg])


def _host(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu").contiguous()


def save(path, cfg, step: int, rng_state: int, params: torch.Tensor, m: torch.Tensor, v: torch.Tensor):
    p, mm, vv = _host(params), _host(m), _host(v)
    pb = p.numel() * p.element_size()
    ob = mm.numel() * mm.element_size()
    assert vv.numel() == mm.numel()
    _native.rt_check(_native.rt().kh_ckpt_save(str(path).encode(), _cfg_arr(cfg), int(step), int(rng_state), pb, ob,
                                               p.data_ptr(), mm.data_ptr(), vv.data_ptr()))


def peek(path):
    cfg = (C.c_int32 * 6)()
    step = C.c_int32()
    rng, pb, ob = C.c_uint64(), C.c_uint64(), C.c_uint64()
    _native.rt_check(_native.rt().kh_ckpt_peek(str(path).encode(), cfg, C.byref(step), C.byref(rng), C.byref(pb),
                                               C.byref(ob)))
    return dict(cfg=list(cfg), step=step.value, rng=rng.value, pb=pb.value, ob=ob.value)


def load(path, cfg, params: torch.Tensor, m: torch.Tensor, v: torch.Tensor):
    """Validates the header, then fills the three buffers in place.  Returns (step, rng)."""
    pb = params.numel() * params.element_size()
    ob = m.numel() * m.element_size()
    hp = torch.empty(params.numel(), dtype=params.dtype)
    hm = torch.empty(m.numel(), dtype=m.dtype)
    hv = torch.empty(v.numel(), dtype=v.dtype)
    step = C.c_int32()
    rng = C.c_uint64()
    _native.rt_check(_native.rt().kh_ckpt_load(str(path).encode(), _cfg_arr(cfg), pb, ob, C.byref(step),
                                               C.byref(rng), hp.data_ptr(), hm.data_ptr(), hv.data_ptr()))
    params.copy_(hp.view_as(params))
    m.copy_(hm.view_as(m))
    v.copy_(hv.view_as(v))
    return step.value, rng.value
