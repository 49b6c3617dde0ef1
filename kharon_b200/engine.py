"""Training engine: one optimizer step of a GPT on a tensor x pipeline x data-parallel mesh.

``TrainEngine.train_step(idx, tgt)`` is the public call a user makes: it takes the step's
token ids for this data-parallel replica ([M * mbatch * seq] int32, normally in pinned host
memory), copies them to the device, runs the micro-batches through the 1F1B schedule,
reduces gradients, applies AdamW and returns the loss as a device tensor (``float(...)`` /
``engine.loss()`` is the only device->host read).

What runs where (reference: src/pp_train.c:108-116):

* pipeline   the C++ schedule generator emits the 1F1B op list for this stage; sends and
             receives are NCCL point-to-point (``batch_isend_irecv`` so that a send and its
             matching receive are one group, the deadlock-free form of comms.cu:68-74).
* tensor     the model's ``tp_allreduce`` seam: NCCL all-reduce (baseline) or the fused
             in-kernel NVLink path of ``parallel.fused`` when enabled.
* data       ZeRO-1: gradients are reduce-scattered (average), AdamW updates this rank's
             slice of the flat arena and emits the bf16 copy of that slice, and only the bf16
             compute copy is all-gathered.  The fp32 master outside the rank's slice is
             refreshed only when a checkpoint is written (src/core/adamw.c:21-58 kept the fp32
             master replicated and gathered 4 bytes per parameter every step).
* tied head  with more than one stage the last stage owns a copy of the embedding matrix;
             the two copies receive the sum of both gradients each step and therefore stay
             identical.
"""
from __future__ import annotations

import ctypes as C
import time

import torch
import torch.distributed as dist

from . import _native, ops
from .models import GPT, Config
from .parallel.mesh import Mesh

PP_RECV_ACT, PP_SEND_ACT, PP_RECV_GRAD, PP_SEND_GRAD, PP_FWD, PP_BWD, PP_SEND_ACT_RECV_GRAD, PP_SEND_GRAD_RECV_ACT, PP_FLUSH_DW = range(9)


def pp_schedule(stage: int, n_stages: int, n_micro: int):
    """1F1B op list [(op, a0, a1)] of one stage from the native generator."""
    cap = 8 * (n_micro + n_stages) + 16
    buf = (C.c_int32 * (3 * cap))()
    n = _native.rt_check(_native.rt().kh_pp_schedule(stage, n_stages, n_micro, buf, cap))
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


def pp_schedule_deferred(stage: int, n_stages: int, n_micro: int, extra: int = 1, mid: bool = True):
    """Op list for non-blocking sends with deferred weight gradients (see kh_pp_schedule_deferred)."""
    cap = 8 * (n_micro + n_stages) + 16
    buf = (C.c_int32 * (3 * cap))()
    n = _native.rt_check(_native.rt().kh_pp_schedule_deferred(stage, n_stages, n_micro, extra, int(mid), buf, cap))
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


def pp_num_slots(stage: int, n_stages: int, n_micro: int) -> int:
    return int(_native.rt().kh_pp_num_slots(stage, n_stages, n_micro))


def stage_split(layers: int, pp: int, d_model: int, vocab: int, spec=None):
    """Layers per pipeline stage.  ``spec``: None/"even" (the reference's L/P, src/pp_train.c:73-76), a
    list or "a,b,..." string, or "auto": the last stage also runs the head GEMMs and the loss, whose
    cost in units of one transformer layer is about 3*V*d / (3*12*d^2) = V / (12 d); "auto" moves that
    many layers (rounded down) from the last stage to the earlier ones so that 1F1B stages take equal time."""
    if pp == 1:
        return [layers]
    if spec is None or spec == "even":
        if layers % pp:
            raise ValueError("layers (%d) must divide evenly over %d pipeline stages" % (layers, pp))
        return [layers // pp] * pp
    if isinstance(spec, str) and spec != "auto":
        spec = [int(x) for x in spec.split(",")]
    if spec == "auto":
        head = vocab / (12.0 * d_model)                     # head + loss cost in layer units
        per = (layers + head) / pp
        last = max(1, int(round(per - head)))
        rest = layers - last
        base, extra = divmod(rest, pp - 1)
        spec = [base + (1 if i < extra else 0) for i in range(pp - 1)] + [last]
    spec = list(spec)
    if len(spec) != pp or sum(spec) != layers or min(spec) < 1:
        raise ValueError("pipeline split %s does not cover %d layers on %d stages" % (spec, layers, pp))
    return spec


class TrainEngine:
    def __init__(self, layers, d_model, heads, vocab, seq, mbatch, n_micro, mesh: Mesh | None = None, device="cuda",
                 dtype=torch.bfloat16, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, untied_head=False,
                 fuse_microbatches=False, seed=1337, init="host", fused_comm=False, trace=False, heartbeat=None, pp_split=None, vocab_parallel=True,
                 defer_dw=None, eager_p2p=None, bucket_optimizer=True, sp=None, pp_fuse=1):
        from .utils.trace import Tracer
        self.mesh = mesh or Mesh.single()
        # The in-kernel collectives move bf16 activations / weights; an fp32 model (the oracle
        # configuration) takes the NCCL path, which also gathers fp32 parameters under ZeRO-1.
        fused_comm = bool(fused_comm and dtype == torch.bfloat16)
        self.tracer = Tracer(enabled=bool(trace))     # per-phase CUDA-event timeline (forward / backward / p2p / optimizer)
        self.heartbeat = heartbeat                     # utils.watchdog.Heartbeat: peers are checked before every step
        self.p2p_timeout_s = 120.0                     # guarded NCCL / gloo point-to-point waits (with a heartbeat)
        c = self.mesh.c
        self.device = torch.device(device)
        self.stage_layers = stage_split(layers, c.pp, d_model, vocab // (c.tp if vocab_parallel else 1), pp_split)
        self.total_layers = layers
        self.n_micro = n_micro
        self.fused_mb = bool(fuse_microbatches and c.pp == 1)
        if self.fused_mb:            # one pass over M x mbatch sequences: identical math, larger GEMMs
            mbatch, n_micro = mbatch * n_micro, 1
        # Pipeline meshes: ``pp_fuse`` consecutive micro-batches travel through the stages as one (identical
        # math: the loss is a mean over tokens and gradients add).  Halving the number of micro-batches grows
        # the 1F1B bubble from (P-1)/(M+P-1) to (P-1)/(M/2+P-1), but every kernel and every fused collective
        # of a stage runs on twice the rows; the deferred weight-gradient pass fills the larger bubble.
        self.pp_fuse = 1
        if c.pp > 1 and pp_fuse and pp_fuse > 1 and n_micro % pp_fuse == 0 and n_micro // pp_fuse >= c.pp:
            self.pp_fuse = int(pp_fuse)
            mbatch, n_micro = mbatch * self.pp_fuse, n_micro // self.pp_fuse
        self.M, self.mbatch, self.seq = n_micro, mbatch, seq
        self.opt = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, wd=wd)
        nl = self.stage_layers[c.stage]
        layer0 = sum(self.stage_layers[:c.stage])
        self.cfg = Config(nl, d_model, heads, vocab, seq, mbatch)
        self.n_slots = pp_num_slots(c.stage, c.pp, n_micro)
        # Deferred weight gradients (default under pipeline parallelism): every micro-batch keeps its
        # own activation slot, backward stores the layers' output gradients, and one pass after the
        # schedule forms all weight/bias gradients over M x R rows.
        self.defer_dw = bool(c.pp > 1 and n_micro > 1) if defer_dw is None else bool(defer_dw and not self.fused_mb)
        if self.defer_dw:
            self.n_slots = n_micro
        self.zero_fused = None
        if c.dp > 1 and fused_comm and self.device.type == "cuda":
            from .parallel.zero_fused import ZeroFused
            self.zero_fused = ZeroFused(self.mesh, self.device)
        # Sequence parallelism over the TP group (all-gather -> GEMM, GEMM -> reduce-scatter, LayerNorm and
        # residual stream on row shards, activations between the blocks 1/tp the size); needs micro-batches
        # that split into whole sequences per rank.  CPU ranks evaluate the same layer with collectives.
        # Measured on B200 (1.2B model, TP2): the replicated form with the fused GEMM + all-reduce is the
        # faster one at both 16384 and 2048 rows per product (83.9 vs 88.3 ms and 62.4 vs 71.1 ms per step:
        # the gather in front of every column-parallel product costs more than the halved LayerNorm work
        # and reduce-scatter traffic save), so sequence parallelism is opt-in.
        if sp is None:
            sp = False
        self.sp = bool(sp and c.tp > 1 and mbatch % c.tp == 0)
        self.sp_ops = None
        if self.sp:
            from .parallel import fused as fused_mod
            self.sp_ops = fused_mod.make(self.mesh, self.device)
        self.model = GPT(self.cfg, self.device, dtype, tp=c.tp, tp_rank=c.tp_rank, first=c.first, last=c.last,
                         untied_head=untied_head, n_slots=self.n_slots, dp=c.dp,
                         alloc=self.zero_fused.alloc if self.zero_fused else None, defer_dw=self.defer_dw,
                         sp=self.sp_ops)
        if init == "device":
            self.model.init_weights_device(seed)
        else:
            self.model.init_weights(seed, layer0=layer0, total_layers=layers)
        self.schedule = pp_schedule(c.stage, c.pp, n_micro)
        R = mbatch * seq
        if self.sp:
            R //= c.tp          # stages exchange row shards: TP rank r of a stage talks to TP rank r of the next
        dev = self.device
        # Message transport between stages.  With deferred weight gradients and a transport whose
        # sends do not wait for the receiver (mailboxes in peer memory on GPUs, gloo isend on CPU
        # ranks) the stage runs the deeper-warm-up schedule that hides half of the weight-gradient
        # pass; blocking NCCL send/recv keeps the 1F1B order and appends one pass at the end.
        self.box = None
        if self.defer_dw and c.pp > 1 and eager_p2p is not False:
            from .parallel import p2p
            if self.device.type == "cuda" and fused_comm:
                from .parallel import fused as fused_mod
                fused_mod.align_allocation_counts(self.mesh, dev)      # the mailbox rendezvous spans stages
                self.box = p2p.Mailbox(self.mesh, dev, n_micro, R, d_model, dtype)
            elif dist.get_backend() == "gloo":
                self.box = p2p.DistMailbox(self.mesh, dev, n_micro, R, d_model, dtype)
        if self.box is not None:
            self.schedule = pp_schedule_deferred(c.stage, c.pp, n_micro)
        elif self.defer_dw:
            self.schedule = self.schedule + [(PP_FLUSH_DW, 0, n_micro)]
        self.tok_dev = torch.zeros(n_micro * mbatch * seq, dtype=torch.int32, device=dev)
        self.tgt_dev = torch.zeros(n_micro * mbatch * seq, dtype=torch.int32, device=dev)
        if c.pp > 1:
            self.recv_act = [torch.empty(R, d_model, dtype=dtype, device=dev) for _ in range(2)]
            self.recv_grad = [torch.empty(R, d_model, dtype=dtype, device=dev) for _ in range(2)]
        # ---- tensor parallel seam
        self.fused = None
        if c.tp > 1:
            grp = self.mesh.tp_group
            self.model.tp_allreduce = lambda t: dist.all_reduce(t, group=grp)
            if self.sp_ops is not None:
                self.fused = self.model.fused_tp = self.sp_ops
            elif fused_comm and self.device.type == "cuda":
                from .parallel import fused as fused_mod
                self.fused = fused_mod.install(self.model, self.mesh)
            if c.last and vocab_parallel:
                from .parallel.mesh import rank_of
                self.model.enable_vocab_parallel(grp, [rank_of(c.dp_rank, c.stage, t, c.tp, c.pp) for t in range(c.tp)])
        # ---- ZeRO-1
        ps = self.model.params
        self.zero = c.dp > 1
        if self.zero:
            self.shard = ps.n_padded // c.dp
            self.lo = c.dp_rank * self.shard
            ps.alloc_moments(self.shard)
            self.g_shard = None if self.zero_fused else torch.zeros(self.shard, dtype=torch.float32, device=dev)
            if self.zero_fused:
                self.zero_fused.finalize()
        # Optimizer buckets: without ZeRO, a layer's AdamW range is launched on a side stream as soon as the
        # layer's gradients are final, i.e. under the backward pass of the layers below it (memory-bound
        # work next to compute-bound work); the rest of the arena follows after the last backward.
        # (under sequence parallelism the LayerNorm gradients are only complete after their exchange at the
        # end of the step, so the layers are not updated early there)
        self.bucketed = bool(not self.zero and not self.sp and self.device.type == "cuda" and dtype == torch.bfloat16
                             and bucket_optimizer)
        self._opt_pending = False
        if self.bucketed:
            self.opt_stream = torch.cuda.Stream(self.device)
            self.opt_events = [torch.cuda.Event() for _ in range(nl)]
            self.opt_done = torch.cuda.Event()
        self.plans = {}
        # launch plans replay native calls only; the fp32 oracle path also runs PyTorch operators
        self.use_plans = self.device.type == "cuda" and dtype == torch.bfloat16
        # host -> device input staging (see _upload)
        self._par = 0
        if self.device.type == "cuda":
            self.copy_stream = torch.cuda.Stream(self.device)
            self.stage = [[torch.zeros_like(self.tok_dev), torch.zeros_like(self.tgt_dev)] for _ in range(2)]
            self.stage_free = [None, None]

    # ------------------------------------------------------------------ helpers
    @property
    def tokens_per_step(self):
        """Tokens this replica consumes per step."""
        return self.M * self.mbatch * self.seq

    def _p2p(self, ops_):
        if not ops_:
            return
        works = dist.batch_isend_irecv(ops_)
        if self.heartbeat is not None:      # a dead neighbour becomes an exception instead of a blocked rank
            from .utils.watchdog import guarded
            guarded(works, self.heartbeat, timeout_s=self.p2p_timeout_s, what="pipeline send/recv")
            return
        for w in works:
            w.wait()

    def _stage_input(self, mb):
        R = self.mbatch * self.seq
        s = self.model.slots[mb % self.n_slots]
        ops.plan_call(s.tok.copy_, self.tok_dev[mb * R:(mb + 1) * R])
        ops.plan_call(s.tgt.copy_, self.tgt_dev[mb * R:(mb + 1) * R])

    def _compute(self, key, fn):
        """Run one forward/backward of the schedule.  On a GPU the first execution records the
        exact native calls (buffers are static per micro-batch slot) and later steps replay them,
        which removes the per-launch Python marshalling from the critical path."""
        if not self.use_plans:
            return fn()
        hit = self.plans.get(key)
        if hit is not None:
            hit[0].replay()
            return hit[1]
        plan = ops.LaunchPlan()
        with plan.record():
            out = fn()
        self.plans[key] = (plan, out)
        return out

    def _upload(self, idx, tgt):
        """Bring the step's token ids onto the device.  Host tensors go through a copy stream into one
        of two staging buffers and the call returns only when that copy has completed, so the caller
        may overwrite its (pinned) host buffers right away even while the GPU is still busy with the
        previous step; the compute stream then moves the staged ids into place in stream order."""
        idx, tgt = idx.reshape(-1), tgt.reshape(-1)
        if self.device.type != "cuda" or idx.is_cuda:
            self.tok_dev.copy_(idx, non_blocking=True)
            self.tgt_dev.copy_(tgt, non_blocking=True)
            return
        self._par ^= 1
        par = self._par
        cur = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.copy_stream):
            if self.stage_free[par] is not None:
                self.copy_stream.wait_event(self.stage_free[par])    # its previous reader has finished
            self.stage[par][0].copy_(idx, non_blocking=True)
            self.stage[par][1].copy_(tgt, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        done.synchronize()
        cur.wait_event(done)
        self.tok_dev.copy_(self.stage[par][0], non_blocking=True)
        self.tgt_dev.copy_(self.stage[par][1], non_blocking=True)
        free = torch.cuda.Event()
        free.record(cur)
        self.stage_free[par] = free

    # ------------------------------------------------------------------ one step
    def train_step(self, idx, tgt):
        """idx/tgt: int32 [M * mbatch * seq] for this replica (host or device)."""
        m, c = self.model, self.mesh.c
        if self.heartbeat is not None:
            self.heartbeat.check()      # raises RankFailure before any kernel that would wait on a dead peer
        tr = self.tracer
        with tr.range("upload"):
            self._upload(idx, tgt)
        M = self.M
        inv = 1.0 / M
        cur_act = cur_grad = None
        out_act = {}
        in_grad = {}
        n_loss = 0
        box = self.box
        for op, a0, a1 in self.schedule:
            if self.defer_dw and op in (PP_FWD, PP_BWD):
                a1 = a0                 # one slot per micro-batch
            if op == PP_FLUSH_DW:
                m.on_layer_grads = self._adamw_layer if (self.bucketed and a1 == M) else None
                with tr.range("weight gradients"):
                    self._compute(("W", a0, a1), lambda: m.flush_dw(a0, a1))
                m.on_layer_grads = None
                continue
            if box is not None and op not in (PP_FWD, PP_BWD):
                with tr.range("pipeline p2p"):
                    if op == PP_RECV_ACT:
                        self._compute(("RA", a0), lambda: box.wait_act(a0))
                    elif op == PP_SEND_ACT:
                        self._compute(("SA", a0), lambda: box.send_act(a0, out_act.pop(a0)))
                    elif op == PP_RECV_GRAD:
                        self._compute(("RG", a0), lambda: box.wait_grad(a0))
                    elif op == PP_SEND_GRAD:
                        self._compute(("SG", a0), lambda: box.send_grad(a0, in_grad.pop(a0)))
                continue
            if box is not None:
                cur_act = None if c.first else box.act_in(a0)
                cur_grad = None if c.last else box.grad_in(a0)
            if op == PP_FWD:
                with tr.range("forward"):
                    out_act[a0] = self._compute(("F", a0, a1), lambda: (
                        self._stage_input(a0), m.forward(slot=a1, x_in=cur_act, compute_loss=False))[1])
                continue
            if op == PP_BWD:
                dxo = None if c.last else cur_grad
                first_loss = n_loss == 0
                # the last micro-batch's backward completes the gradients layer by layer
                m.on_layer_grads = self._adamw_layer if (self.bucketed and not self.defer_dw and n_loss == M - 1) else None
                with tr.range("backward"):
                    in_grad[a0] = self._compute(("B", a0, a1), lambda: m.backward(
                        slot=a1, dx_out=dxo, inv_mb=inv, loss_scale=inv, accumulate_loss=not first_loss))
                m.on_layer_grads = None
                n_loss += 1
                continue
            with tr.range("pipeline p2p"):
                if op == PP_RECV_ACT:
                    cur_act = self.recv_act[a0 & 1]
                    self._p2p([dist.P2POp(dist.irecv, cur_act, c.prev_rank)])
                elif op == PP_SEND_ACT:
                    self._p2p([dist.P2POp(dist.isend, out_act.pop(a0), c.next_rank)])
                elif op == PP_RECV_GRAD:
                    cur_grad = self.recv_grad[a0 & 1]
                    self._p2p([dist.P2POp(dist.irecv, cur_grad, c.next_rank)])
                elif op == PP_SEND_GRAD:
                    self._p2p([dist.P2POp(dist.isend, in_grad.pop(a0), c.prev_rank)])
                elif op == PP_SEND_ACT_RECV_GRAD:     # a0 = micro-batch sent, a1 = micro-batch whose grad arrives
                    cur_grad = self.recv_grad[a1 & 1]
                    self._p2p([dist.P2POp(dist.isend, out_act.pop(a0), c.next_rank),
                               dist.P2POp(dist.irecv, cur_grad, c.next_rank)])
                elif op == PP_SEND_GRAD_RECV_ACT:     # a0 = micro-batch whose grad is sent, a1 = next activation
                    cur_act = self.recv_act[a1 & 1]
                    self._p2p([dist.P2POp(dist.isend, in_grad.pop(a0), c.prev_rank),
                               dist.P2POp(dist.irecv, cur_act, c.prev_rank)])
        if box is not None:
            box.finish()
        with tr.range("optimizer"):
            m.sync_head_grad()
            self._tie_embedding_grads()
            self._sync_sp_grads()
            self.optimizer_step()
        return m.loss_acc

    def _sync_sp_grads(self):
        """Sequence parallelism: LayerNorm gains / biases saw only this rank's rows; sum their gradients
        over the TP group (one packed all-reduce of a few hundred KB per step)."""
        if not self.sp:
            return
        gs = self.model.sp_partial_grads()
        if getattr(self, "_sp_pack", None) is None:
            self._sp_pack = torch.empty(sum(g.numel() for g in gs), dtype=torch.float32, device=self.device)
            self._sp_views = list(self._sp_pack.split([g.numel() for g in gs]))
        torch._foreach_copy_(self._sp_views, gs)
        dist.all_reduce(self._sp_pack, group=self.mesh.tp_group)
        torch._foreach_copy_(gs, self._sp_views)

    def _tie_embedding_grads(self):
        m = self.model
        if self.mesh.c.pp > 1 and not m.untied_head and self.mesh.tie_group is not None:
            g = m.params.grad["wte"] if m.first else m.params.grad["head_w"]
            dist.all_reduce(g, group=self.mesh.tie_group)

    def _adamw_layer(self, l):
        """AdamW over layer l's range on the optimizer stream, ordered after everything the compute stream
        has issued so far (the layer's last gradient kernel)."""
        m, o = self.model, self.opt
        if not self._opt_pending:          # first bucket of the step
            m.step += 1
            self._opt_pending = True
        cur = torch.cuda.current_stream(self.device)
        ev = self.opt_events[l]
        ev.record(cur)
        self.opt_stream.wait_event(ev)
        lo, hi = m.layer_range(l)
        with torch.cuda.stream(self.opt_stream):
            m.adamw_step(o["lr"], o["beta1"], o["beta2"], o["eps"], o["wd"], lo=lo, hi=hi, advance=False)

    def optimizer_step(self):
        m, ps, o = self.model, self.model.params, self.opt
        if not self.zero:
            if self._opt_pending:
                # the layers were updated under the backward pass; what is left: embeddings, final norm, head
                self._opt_pending = False
                lo0, _ = m.layer_range(0)
                _, hi1 = m.layer_range(m.cfg.n_layer - 1)
                m.adamw_step(o["lr"], o["beta1"], o["beta2"], o["eps"], o["wd"], lo=0, hi=lo0, advance=False)
                m.adamw_step(o["lr"], o["beta1"], o["beta2"], o["eps"], o["wd"], lo=hi1, hi=ps.w.numel(), advance=False)
                self.opt_done.record(self.opt_stream)
                torch.cuda.current_stream(self.device).wait_event(self.opt_done)
                return
            m.adamw_step(o["lr"], o["beta1"], o["beta2"], o["eps"], o["wd"])
            return
        grp = self.mesh.dp_group
        if self.zero_fused is not None:
            m.step += 1
            self.zero_fused.step(ps, self.shard, m.step, o)
            return
        if dist.get_backend(grp) == "nccl":
            dist.reduce_scatter_tensor(self.g_shard, ps.g, op=dist.ReduceOp.AVG, group=grp)
        else:   # CPU ranks (gloo) have no reduce-scatter / AVG: same result via all-reduce
            dist.all_reduce(ps.g, group=grp)
            self.g_shard.copy_(ps.g[self.lo:self.lo + self.shard] / self.mesh.c.dp)
        m.step += 1
        lo, hi = self.lo, self.lo + self.shard
        wb = None if ps.wb is ps.w else ps.wb[lo:hi]
        ops.adamw(ps.w[lo:hi], self.g_shard, ps.m, ps.v, wb, lr=o["lr"], beta1=o["beta1"], beta2=o["beta2"],
                  eps=o["eps"], wd=o["wd"], step=m.step, grad_scale=1.0, zero_grad=False)
        ps.g.zero_()
        # only the compute copy travels; the fp32 master stays sharded
        tgt_full = ps.wb if ps.wb is not ps.w else ps.w
        dist.all_gather_into_tensor(tgt_full, tgt_full[lo:hi], group=grp)

    def loss(self) -> float:
        """Mean loss of the last step (valid on the last pipeline stage).  Reading it synchronises
        with the device, so this is also where a bounded wait that ran out during the step (a peer
        that never delivered a partial tile, a mailbox message or its gradients) turns into an
        exception instead of a silently wrong step."""
        v = float(self.model.loss_acc.item())
        if self.device.type == "cuda":
            ops.check_device_status()
        return v

    # ------------------------------------------------------------------ checkpoint
    def gather_master(self):
        """Rebuild the full fp32 master on every rank of the data-parallel group (ZeRO-1 keeps
        only this rank's slice current between checkpoints)."""
        if self.zero:
            ps = self.model.params
            dist.all_gather_into_tensor(ps.w, ps.w[self.lo:self.lo + self.shard].clone(), group=self.mesh.dp_group)

    def ckpt_path(self, prefix):
        return prefix if self.mesh.world == 1 else "%s.r%d" % (prefix, self.mesh.rank)

    def save(self, prefix, rng_state=0):
        """One CKP1 file per rank (``<prefix>.r<rank>`` on more than one rank): the rank's full
        fp32 parameter arena plus its moments -- under ZeRO-1 only its shard of them."""
        self.gather_master()
        ps = self.model.params
        self.model.save(self.ckpt_path(prefix), rng_state, moments=(ps.m, ps.v) if self.zero else None)

    def load(self, prefix):
        ps = self.model.params
        rng = self.model.load(self.ckpt_path(prefix), moments=(ps.m, ps.v) if self.zero else None)
        return rng

    def memory_report(self):
        out = {"params_arena_mb": self.model.params.param_bytes / 1e6,
               "optimizer_state_mb": 2 * self.model.params.m.numel() * 4 / 1e6}
        if self.device.type == "cuda":
            out["cuda_allocated_gb"] = torch.cuda.memory_allocated(self.device) / 1e9
        return out
