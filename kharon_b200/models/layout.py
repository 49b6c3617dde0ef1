"""Model configuration and flat parameter storage.

Parameters live in flat arenas whose tensor offsets come from the native layout routine
(256-byte aligned bump allocation in the order of src/core/gpt.c:18-42 of the reference), so
the fp32 arena is, byte for byte, the ``params`` block of a CKP1 checkpoint.  Arenas:

* ``w``   fp32 master weights        * ``g``  fp32 gradients (accumulated across micro-batches)
* ``wb``  compute copy (bf16; aliases ``w`` when the model computes in fp32)
* ``m``, ``v``  AdamW moments (full-size, or one ZeRO-1 shard)
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _native

LAYER_FIELDS = ["ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "ln2_w", "ln2_b", "fc_w", "fc_b",
                "fcproj_w", "fcproj_b"]


@dataclass(frozen=True)
class Config:
    n_layer: int
    d_model: int
    n_head: int
    vocab: int
    seq: int
    batch: int

    def as_list(self):
        return [self.n_layer, self.d_model, self.n_head, self.vocab, self.seq, self.batch]

    @property
    def head_dim(self):
        return self.d_model // self.n_head


def n_params(cfg: Config, has_head=False) -> int:
    d = cfg.d_model
    per = 4 * d + 3 * d * d + 3 * d + d * d + d + 4 * d * d + 4 * d + 4 * d * d + d
    return cfg.vocab * d + cfg.seq * d + cfg.n_layer * per + 2 * d + (cfg.vocab * d if has_head else 0)


def matmul_params(cfg: Config) -> int:
    """Parameters that take part in a GEMM per token (the MFU numerator uses 6x this)."""
    return 12 * cfg.n_layer * cfg.d_model ** 2 + cfg.vocab * cfg.d_model


def param_names(n_layer: int, has_head: bool):
    names = ["wte", "wpe"]
    for l in range(n_layer):
        names += ["l%d.%s" % (l, f) for f in LAYER_FIELDS]
    names += ["lnf_w", "lnf_b"]
    if has_head:
        names.append("head_w")
    return names


def param_shapes(cfg: Config, tp: int, has_head: bool):
    d, V, S = cfg.d_model, cfg.vocab, cfg.seq
    qo, pi, fo = 3 * d // tp, d // tp, 4 * d // tp
    layer = {"ln1_w": (d,), "ln1_b": (d,), "qkv_w": (qo, d), "qkv_b": (qo,), "proj_w": (d, pi), "proj_b": (d,),
             "ln2_w": (d,), "ln2_b": (d,), "fc_w": (fo, d), "fc_b": (fo,), "fcproj_w": (d, fo), "fcproj_b": (d,)}
    shapes = {"wte": (V, d), "wpe": (S, d)}
    for l in range(cfg.n_layer):
        for f in LAYER_FIELDS:
            shapes["l%d.%s" % (l, f)] = layer[f]
    shapes["lnf_w"] = (d,)
    shapes["lnf_b"] = (d,)
    if has_head:
        shapes["head_w"] = (V, d)
    return shapes


def layout(cfg: Config, tp: int, has_head: bool, elem_size: int):
    """(names, byte offsets, element counts, total bytes) of one arena."""
    names = param_names(cfg.n_layer, has_head)
    n = len(names)
    offs = (C.c_int64 * n)()
    nums = (C.c_int64 * n)()
    total = C.c_int64()
    cfg_arr = (C.c_int32 * 6)(*cfg.as_list())
    got = _native.rt_check(_native.rt().kh_layout_params(cfg_arr, tp, int(has_head), elem_size, offs, nums, n,
                                                         C.byref(total)))
    assert got == n
    return names, list(offs), list(nums), int(total.value)


class ParamStore:
    """Flat arenas plus named views.  ``compute_dtype`` is torch.bfloat16 or torch.float32."""

    def __init__(self, cfg: Config, device, compute_dtype=torch.bfloat16, tp=1, has_head=False, pad_to=1, alloc=None):
        self.cfg, self.tp, self.has_head = cfg, tp, has_head
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        names, offs4, nums, total4 = layout(cfg, tp, has_head, 4)
        self.names = names
        self.shapes = param_shapes(cfg, tp, has_head)
        self.param_bytes = total4                  # == pb of the checkpoint
        self.n_flat = total4 // 4                  # AdamW sweeps the alignment gaps too (kept at zero)
        # ZeRO-1 pads the flat length to a multiple of the data-parallel size
        self.n_padded = (self.n_flat + pad_to - 1) // pad_to * pad_to
        z = dict(device=self.device)
        # ``alloc(kind, n, dtype)`` lets the parallel layer place the gradient arena and the compute
        # copy in symmetric (peer-mapped) memory; it must return zero-filled storage
        mk = alloc if alloc is not None else (lambda kind, n, dt: torch.zeros(n, dtype=dt, **z))
        self.w = torch.zeros(self.n_padded, dtype=torch.float32, **z)
        self.g = mk("g", self.n_padded, torch.float32)
        self.offsets = {n: o // 4 for n, o in zip(names, offs4)}
        self.numels = dict(zip(names, nums))
        if compute_dtype == torch.float32:
            self.wb = self.w
        else:
            # same element offsets as the fp32 arena: one fused optimizer pass emits wb[i] from w[i]
            self.wb = mk("wb", self.n_padded, compute_dtype)
        self.p = {n: self._view(self.w, n) for n in names}     # fp32 master views
        self.grad = {n: self._view(self.g, n) for n in names}  # fp32 gradient views
        self.c = {n: self._view(self.wb, n) for n in names}    # compute-dtype views
        self.m = None
        self.v = None

    def _view(self, flat, name):
        o, n = self.offsets[name], self.numels[name]
        return flat[o:o + n].view(self.shapes[name])

    def alloc_moments(self, n=None):
        n = self.n_padded if n is None else n
        self.m = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(n, dtype=torch.float32, device=self.device)

    def sync_compute_copy(self):
        """Refresh the compute-dtype copy from the fp32 master (after init / load; the
        optimizer keeps it current afterwards)."""
        if self.wb is not self.w:
            from .. import ops
            ops.cast_f32_bf16(self.w, self.wb)
