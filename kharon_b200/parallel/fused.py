"""Fused tensor-parallel GEMM + collective (the product path; NCCL all-reduce is the baseline).

``FusedTP`` owns the symmetric (peer-mapped) staging buffers and arrival counters that the
``kh_gemm_comm`` kernel needs and exposes

* ``gemm_ar``  partial GEMM on every rank, summed across the TP group inside the kernel: every rank
               pushes each partial tile to every peer and reduces every tile itself (one-shot
               all-reduce: (tp - 1) x M x N bf16 out per rank, the traffic of reduce-scatter +
               all-gather only at tp = 2), bias / residual added in the reduction;
* ``gemm_rs``  same, but each rank keeps only its row shard (GEMM -> reduce-scatter);
* ``ag_gemm``  all-gather -> GEMM: the A operand is the concatenation of per-rank row shards
               that live in symmetric memory and are read tile by tile with TMA.

Buffers come from ``torch.distributed._symmetric_memory`` (allocation and address exchange
only); all data movement is issued from inside the kernel.  The call counter of a buffer set
is a device word that the kernel advances itself (identical on all ranks because every rank
issues the same sequence of calls), so a fused product is an ordinary native call: it can be
recorded in a launch plan and captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native, ops

MODE_AR, MODE_RS = 0, 1


_alloc_seq = {}      # per process group: allocations rendezvoused on it so far (identical on its ranks)
_alloc_total = 0     # symmetric allocations of this process, over all groups


def align_allocation_counts(mesh, device):
    """The symmetric-memory rendezvous pairs the buffers of a group's ranks by each process's running
    allocation number, so two ranks can only rendezvous when they have made the same number of symmetric
    allocations before -- over ALL groups.  Pipeline stages differ there (only the last stage owns the
    head's buffers, contexts are created at first use), so before a rendezvous that spans stages every
    rank pads its count to the maximum of the job with small allocations on its TP group (whose ranks
    share a stage and therefore a count).  Collective over the world; raises instead of letting a
    mismatched rendezvous run into the store time-out."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return
    t = torch.tensor([_alloc_total, -_alloc_total], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mx, mn = int(t[0]), -int(t[1])
    if mx == mn:
        return
    if mesh.tp_group is None:
        raise RuntimeError("symmetric allocation counts differ between ranks (%d..%d) and there is no TP group to pad on"
                           % (mn, mx))
    keep = []
    while _alloc_total < mx:
        keep.append(_symm_alloc(16, device, mesh.tp_group))
    _pads.extend(keep)
    t = torch.tensor([_alloc_total, -_alloc_total], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if int(t[0]) != -int(t[1]):
        raise RuntimeError("symmetric allocation counts still differ after padding (%d..%d)" % (-int(t[1]), int(t[0])))


_pads = []


def _symm_alloc(nbytes, device, group):
    """A peer-mapped buffer of ``nbytes`` bytes and its rendezvous handle.

    Before the buffer is handed out all ranks of the group drain their GPUs and meet in a device
    barrier, stamp the buffer with (allocation number, rank) and read the peers' stamps through the
    mapped addresses.  The drain matters when a process drops one set of buffers and builds another
    (tests, notebooks): a peer whose GPU still runs the last kernels of the old set writes into
    memory that this rank has already released and may just have received again.  Without it about
    one run in four of such a sequence trained on corrupted weights or gradients; with it none of
    eleven did.  The stamps turn a handle that pairs the buffer with anything but the peers'
    buffers of the same allocation into an error."""
    import torch.distributed._symmetric_memory as symm_mem
    global _alloc_total
    _alloc_total += 1
    t = symm_mem.empty(max(nbytes, 16), dtype=torch.uint8, device=device)
    name = group.group_name if hasattr(group, "group_name") else group
    h = symm_mem.rendezvous(t, name)
    seq = _alloc_seq[name] = _alloc_seq.get(name, 0) + 1
    stamp = lambda r: (seq << 40) + (int(nbytes) << 8) + r + 1
    t[:8].view(torch.int64).fill_(stamp(h.rank))
    torch.cuda.synchronize(device)
    h.barrier()
    for r in range(h.world_size):
        try:
            got = int(h.get_buffer(r, (1,), torch.int64).item())
        except (AttributeError, TypeError, NotImplementedError):
            break           # this build exposes no typed view of a peer buffer: keep the drain + barrier only
        if got != stamp(r):
            raise RuntimeError("symmetric allocation #%d (%d bytes, group %s): the address mapped for rank %d holds stamp "
                               "%#x, expected %#x" % (seq, nbytes, name, r, got, stamp(r)))
    torch.cuda.synchronize(device)
    h.barrier()
    t[:8].zero_()
    return t, h


class _Ctx:
    """Staging + counters for one (M, N, mode) shape."""

    def __init__(self, M, N, tp, rank, device, group, mode=0):
        self.M, self.N, self.tp, self.rank = M, N, tp, rank
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        # the all-gather form (mode 2) reduces nothing: no partial-tile staging
        self.slot_bytes = tp * M * N * 2 if mode != 2 else 0
        self.flag_bytes = tp * tiles * 4 * 4          # one counter per (source rank, tile, 64-column chunk)
        total = 2 * self.slot_bytes + self.flag_bytes + 256
        self.buf, self.h = _symm_alloc(total, device, group)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.h.barrier()
        base = [int(p) for p in self.h.buffer_ptrs]
        self.flags = [b + 2 * self.slot_bytes for b in base]
        self.ready = [b + 2 * self.slot_bytes + self.flag_bytes for b in base]
        U = C.c_uint64 * tp
        self.c_stage = U(*base)                  # parity-0 bases; parity 1 follows at slot_bytes
        self.c_flags = U(*self.flags)
        self.c_ready = U(*self.ready)
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)    # [calls completed, CTAs finished]
        self.gathers = 0


class SymRows:
    """A [rows, cols] bf16 matrix whose row block r (``rows / tp`` rows) is produced by TP rank r and read
    by all ranks: the operand of the all-gather -> GEMM kernel.  ``t`` is this rank's full-size buffer in
    symmetric memory; the rank writes its own block (``mine``), ``ag_gemm_sym`` fills in the others, so
    afterwards ``t`` is the complete gathered matrix (kept for the weight-gradient products)."""

    def __init__(self, t, shard_ptrs, rank, tp):
        self.t, self.ptrs, self.rank, self.tp = t, shard_ptrs, rank, tp
        self.rs = t.shape[0] // tp

    @property
    def mine(self):
        return self.t[self.rank * self.rs:(self.rank + 1) * self.rs]


class FusedTP:
    #: sequence-parallel operands come from symmetric memory and are moved by the kernels themselves
    emulated = False

    def __init__(self, mesh, device):
        self.group = mesh.tp_group
        self.tp, self.rank = mesh.c.tp, mesh.c.tp_rank
        self.device = torch.device(device)
        self.ctx = {}
        self._vp = {}
        self.max_ctas = 0

    def _get(self, M, N, mode, K=0):
        key = (M, N, mode, K)
        c = self.ctx.get(key)
        if c is None:
            c = self.ctx[key] = _Ctx(M, N, self.tp, self.rank, self.device, self.group, mode)
        return c

    def symmetric_rows(self, rows, cols, dtype=torch.bfloat16):
        """A [rows, cols] tensor in symmetric memory plus the peers' addresses of it (for ag_gemm)."""
        t, h = _symm_alloc(rows * cols * 2, self.device, self.group)
        return t.view(dtype).view(rows, cols), [int(p) for p in h.buffer_ptrs], h

    def sym_rows(self, rows, cols, count=1, slots=1):
        """``count`` x ``slots`` SymRows of [rows, cols] carved from ONE symmetric allocation.  The ``slots``
        matrices of one group are contiguous ([slots * rows, cols], slot-major), so that a product over
        several micro-batch slots can read them as one operand.  Returns (list of lists, slab tensor)."""
        per = rows * cols * 2
        buf, h = _symm_alloc(count * slots * per, self.device, self.group)
        self._slabs = getattr(self, "_slabs", []) + [(buf, h)]
        base = [int(p) for p in h.buffer_ptrs]
        rs = rows // self.tp
        out = []
        for i in range(count):
            grp = []
            for j in range(slots):
                off = (i * slots + j) * per
                t = buf[off:off + per].view(torch.bfloat16).view(rows, cols)
                grp.append(SymRows(t, [b + off + r * rs * cols * 2 for r, b in enumerate(base)], self.rank, self.tp))
            out.append(grp)
        slab = buf[:count * slots * per].view(torch.bfloat16).view(count, slots * rows, cols)
        return out, slab

    def ag_gemm_sym(self, sym, b, out, *, b_mn=False, epi=0, bias=None, aux=None):
        """out = epilogue(gathered(sym) @ op(b)); leaves the gathered matrix in ``sym.t``."""
        K = sym.t.shape[1]
        return self.ag_gemm(sym.ptrs, K, sym.rs, b, out, b_mn=b_mn, K=K, epi=epi, bias=bias, aux=aux, gather_buf=sym.t)

    def all_gather_rows(self, sym):
        """Complete ``sym.t`` from the ranks' own row blocks without a following product (NCCL all-gather;
        used once per micro-batch in front of the replicated embedding backward)."""
        ops.plan_call(dist.all_gather_into_tensor, sym.t, sym.mine, self.group)

    def vp_combine(self, stats, tgt, gmax, gsum, rowloss):
        """Vocabulary-parallel softmax statistics: push this rank's per-row (max, sum exp, target logit)
        ``stats [R, 3]`` to the peers, wait for theirs and write the global ``gmax``, ``gsum`` and the
        row losses -- one kernel (``csrc/comm/vp_combine.cu``), an ordinary recordable native call."""
        R = stats.shape[0]
        c = self._vp.get(R)
        if c is None:
            nblk = (R + 255) // 256
            data = 2 * self.tp * R * 3 * 4
            buf, h = _symm_alloc(data + self.tp * nblk * 4, self.device, self.group)
            buf.zero_()
            torch.cuda.synchronize(self.device)
            h.barrier()
            base = [int(p) for p in h.buffer_ptrs]
            U = C.c_uint64 * self.tp
            c = self._vp[R] = (buf, h, U(*base), U(*[b + data for b in base]),
                               torch.zeros(2, dtype=torch.int32, device=self.device))
        ops._call(_native.cuda().kh_vp_combine, 1, stats.data_ptr(), c[2], c[3], c[4].data_ptr(), tgt.data_ptr(),
                  gmax.data_ptr(), gsum.data_ptr(), rowloss.data_ptr(), R, self.tp, self.rank, ops._stream())

    def _gemm(self, a, b, out, a_mn, b_mn, mode, bias, resid):
        if a_mn:
            K, M = a.shape
        else:
            M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        c = self._get(M, N, mode)
        ptr = (C.c_uint64 * 1)(a.data_ptr())
        ops._call(_native.cuda().kh_gemm_comm, 1, ptr, a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn),
                  out.data_ptr(), out.stride(0), M, N, K, mode, 0, self.tp, self.rank, c.c_stage, c.c_flags,
                  c.c_ready, 0, 0, c.epoch.data_ptr(), None, None, ops._p(bias), ops._p(resid),
                  resid.stride(0) if resid is not None else 0, 0, None, 0, self.max_ctas, ops._stream())
        return out

    def gemm_ar(self, a, b, out, *, a_mn=False, b_mn=False, bias=None, resid=None):
        """out[M,N] = sum over TP ranks of op(a) @ op(b) (+ bias + resid), identical on all ranks."""
        return self._gemm(a, b, out, a_mn, b_mn, MODE_AR, bias, resid)

    def gemm_rs(self, a, b, out, *, a_mn=False, b_mn=False, bias=None, resid=None):
        """out[M/tp,N] = this rank's row block of the summed product (+ bias + resid rows)."""
        return self._gemm(a, b, out, a_mn, b_mn, MODE_RS, bias, resid)

    def ag_gemm(self, shard_ptrs, lda, rows_per_rank, b, out, *, b_mn=False, K=None, epi=0, bias=None, aux=None,
                gather_buf=None):
        """out[M,N] = epilogue(concat_r(shard_r)[M,K] @ op(b)): ``shard_ptrs`` are the tp peer addresses of
        the row shards ([M/tp, K] each, symmetric memory).  Local product only -- no reduction.  Epilogues
        (``ops.EPI_*``): none, bias, bias + GELU (``aux`` receives the pre-activation), dGELU (``aux`` is the
        pre-activation).  ``gather_buf`` [M, K]: where the remote rows land (default: a buffer owned by the
        context); when the shards are row blocks of per-rank [M, K] buffers in symmetric memory, passing this
        rank's buffer leaves the complete gathered operand behind for later use (weight gradients).

        A rank's shard may be rewritten once a LATER collective that needs every rank's contribution has
        completed on this rank (the peers' copies of the shard precede their contribution); rewriting it
        earlier races with the peers' copier CTAs."""
        M = rows_per_rank * self.tp
        N = b.shape[1] if b_mn else b.shape[0]
        K = K if K is not None else (b.shape[0] if b_mn else b.shape[1])
        ptrs = (C.c_uint64 * self.tp)(*shard_ptrs)
        ops.plan_call(self._launch_ag, ptrs, lda, b, b_mn, out, M, N, K, epi, bias, aux, gather_buf)
        return out

    def _launch_ag(self, ptrs, lda, b, b_mn, out, M, N, K, epi=0, bias=None, aux=None, gather_buf=None):
        # gather mode uses a context of its own: its "reduction" is local-only (no staging)
        c = self._get(M, N, 2, K)
        c.gathers += 1
        if getattr(c, "gbuf_k", None) != K:      # per-block delivery counters (+ default landing buffer)
            c.gbuf = None
            c.blk_ready = torch.zeros((M + 127) // 128, dtype=torch.int32, device=self.device)
            c.epoch.zero_()
            c.gbuf_k = K
        if gather_buf is None:
            if c.gbuf is None:
                c.gbuf = torch.empty(M, K, dtype=torch.bfloat16, device=self.device)
            gather_buf = c.gbuf
        lib = _native.cuda()
        rc = lib.kh_gemm_comm(ptrs, lda, 0, b.data_ptr(), b.stride(0), int(b_mn), out.data_ptr(), out.stride(0),
                              M, N, K, 2, 1, self.tp, self.rank, c.c_stage, c.c_flags, c.c_ready,
                              0, c.gathers, c.epoch.data_ptr(), gather_buf.data_ptr(), c.blk_ready.data_ptr(),
                              ops._p(bias), None, 0, epi, ops._p(aux), aux.stride(0) if aux is not None else 0,
                              self.max_ctas, torch.cuda.current_stream().cuda_stream)
        ops._chk(rc)
        ops.launch_count += 1


def install(model, mesh):
    """Route the model's row-parallel products (and the conjugate input-gradient products)
    through the fused GEMM + all-reduce kernel."""
    f = FusedTP(mesh, model.device)
    model.fused_tp = f
    return f


def make(mesh, device):
    """The fused operators for ``device``: the NVLink kernels on a GPU, the collective-based evaluation
    of the same interface elsewhere."""
    return FusedTP(mesh, device) if torch.device(device).type == "cuda" else FusedTPEmu(mesh, device)


class FusedTPEmu:
    """The FusedTP interface evaluated with ``torch.distributed`` collectives and the operator layer:
    the execution path of CPU ranks (gloo) and the oracle of the fused kernels in multi-rank tests.
    Partial products are rounded to the storage dtype before they are summed, as the kernels do."""
    emulated = True

    def __init__(self, mesh, device):
        self.group = mesh.tp_group
        self.tp, self.rank = mesh.c.tp, mesh.c.tp_rank
        self.device = torch.device(device)

    def sym_rows(self, rows, cols, count=1, slots=1, dtype=torch.bfloat16):
        slab = torch.zeros(count, slots * rows, cols, dtype=dtype, device=self.device)
        out = [[SymRows(slab[i, j * rows:(j + 1) * rows], None, self.rank, self.tp) for j in range(slots)]
               for i in range(count)]
        return out, slab

    def _partial(self, a, b, a_mn, b_mn):
        M = a.shape[1] if a_mn else a.shape[0]
        N = b.shape[1] if b_mn else b.shape[0]
        part = torch.empty(M, N, dtype=a.dtype, device=a.device)
        ops.gemm(a, b, part, a_mn=a_mn, b_mn=b_mn)
        full = part.float()
        dist.all_reduce(full, group=self.group)
        return full

    def gemm_ar(self, a, b, out, *, a_mn=False, b_mn=False, bias=None, resid=None):
        full = self._partial(a, b, a_mn, b_mn)
        if bias is not None:
            full = full + bias.float()
        if resid is not None:
            full = full + resid.float()
        out.copy_(full)
        return out

    def gemm_rs(self, a, b, out, *, a_mn=False, b_mn=False, bias=None, resid=None):
        full = self._partial(a, b, a_mn, b_mn)
        rs = full.shape[0] // self.tp
        mine = full[self.rank * rs:(self.rank + 1) * rs]
        if bias is not None:
            mine = mine + bias.float()
        if resid is not None:
            mine = mine + resid.float()
        out.copy_(mine)
        return out

    def all_gather_rows(self, sym):
        parts = [torch.empty_like(sym.mine) for _ in range(self.tp)]
        dist.all_gather(parts, sym.mine.contiguous(), group=self.group)
        for r, t in enumerate(parts):
            if r != self.rank:
                sym.t[r * sym.rs:(r + 1) * sym.rs].copy_(t)

    def ag_gemm_sym(self, sym, b, out, *, b_mn=False, epi=0, bias=None, aux=None):
        self.all_gather_rows(sym)
        ops.gemm(sym.t, b, out, b_mn=b_mn, epi=epi, bias=bias, aux=aux)
        return out
