"""Pre-norm GELU GPT with explicit forward and backward passes (no autograd tape).

Architecture = the PyTorch model of the reference's tests/gen_reference.py:59-118: learned
absolute positions, fused qkv projection, causal attention, tanh-GELU MLP of width 4d,
LayerNorm eps 1e-5, weight-tied head, mean cross-entropy.  The op order follows the
reference's gpt.c (forward :399-438, backward :493-543, TP :443-485/:569-625, pipeline
stage :665-772) but every elementwise step is folded into a GEMM epilogue or a fused kernel:

  forward / layer   LN -> GEMM(+bias) -> flash attention -> GEMM(+bias+residual)
                    -> LN -> GEMM(+bias, GELU) -> GEMM(+bias+residual)
  backward / layer  GEMM(dW+=, db+=), GEMM(dX * gelu'), GEMM(dW+=, db+=), GEMM(dX),
                    LN-bwd(+residual grad), GEMM(dW+=, db+=), GEMM(dX), flash-bwd,
                    GEMM(dW+=, db+=), GEMM(dX), LN-bwd(+residual grad)
                    (bias gradients are column sums taken inside the weight-gradient products)

The same code runs in three modes: bf16 on a B200 (native kernels), bf16 on CPU (emulated,
for the CPU test tier) and fp32 on CPU (the numerical oracle).

Tensor parallelism (Megatron): qkv/fc are column-parallel, proj/fcproj row-parallel.  The
partial sums of the row-parallel products and of the two input-gradient products are summed
by ``tp_allreduce`` -- a callback installed by the parallel layer (None = single rank), the
same seam the reference uses (model.h:88-89).  Rank 0 of the TP group folds bias+residual
into its partial product so the sum needs no extra pass.

Sequence parallelism (``sp``, with tp > 1): between the blocks' products the activations live as row
shards [R / tp, d] -- residual stream, LayerNorm, bias and residual adds run on a rank's own rows
only.  A column-parallel product gathers its LayerNorm'd input inside the kernel (all-gather ->
GEMM), a row-parallel product leaves each rank its own rows of the sum (GEMM -> reduce-scatter);
backward uses the conjugates (all-gather -> GEMM for the input gradients of the row-parallel layers,
GEMM -> reduce-scatter for those of the column-parallel ones).  These replace the four all-reduces
per layer and micro-batch of the reference (src/core/gpt.c:687,693,746,761).  LayerNorm gains and
biases see only a rank's rows, so their gradients are summed over the TP group once per step.

Pipeline parallelism: a stage owns ``n_layer`` consecutive layers; ``first`` embeds,
``last`` applies the final norm, head and loss.  Activations are stashed per ``slot`` so
that several micro-batches can be in flight (1F1B).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .layout import Config, ParamStore, LAYER_FIELDS


def _pad64(n):
    return (n + 63) // 64 * 64


_ALLOCATOR = None


def set_allocator(alloc):
    """Route activation / scratch allocations of models constructed afterwards through ``alloc``
    (``utils.guards.GuardedAlloc`` adds canary bands around every buffer); None restores torch.empty."""
    global _ALLOCATOR
    _ALLOCATOR = alloc


def _buf(shape, dtype, dev):
    if _ALLOCATOR is not None:
        return _ALLOCATOR.empty(shape, dtype, dev)
    return torch.empty(*shape, dtype=dtype, device=dev)


class _SlotGroup:
    """Buffers that the deferred weight-gradient pass reads across ALL micro-batches of a step: per
    layer the four GEMM inputs (ln1, att, ln2, act) and the four output gradients (d_out, d_pre,
    d_mid, d_qkv), each one [n_slots * R, width] tensor of which slot i owns rows [i*R, (i+1)*R).
    One product over n_slots * R rows then replaces n_slots products over R rows."""
    WIDTHS = ("ln1", "att", "ln2", "act", "d_out", "d_pre", "d_mid", "d_qkv")

    SYM = ("ln1", "ln2", "d_out", "d_mid")      # gathered across the TP group under sequence parallelism

    def __init__(self, cfg: Config, tp, dev, dt, n, sp=None):
        R, d = cfg.batch * cfg.seq, cfg.d_model
        dl, fo = d // tp, 4 * d // tp
        w = dict(ln1=d, att=dl, ln2=d, act=fo, d_out=d, d_pre=fo, d_mid=d, d_qkv=3 * dl)
        self.n, self.R = n, R
        names = [k for k in self.WIDTHS if not (sp is not None and k in self.SYM)]
        self.layers = [{k: _buf((n * R, w[k]), dt, dev) for k in names} for _ in range(cfg.n_layer)]
        self.sym = None
        if sp is not None:
            # the four [n * R, d] operands per layer that peers read: one symmetric slab
            syms, slab = sp.sym_rows(R, d, count=4 * cfg.n_layer, slots=n) if not sp.emulated else \
                sp.sym_rows(R, d, count=4 * cfg.n_layer, slots=n, dtype=dt)
            self.sym = [{k: syms[4 * l + i] for i, k in enumerate(self.SYM)} for l in range(cfg.n_layer)]
            for l in range(cfg.n_layer):
                for i, k in enumerate(self.SYM):
                    self.layers[l][k] = slab[4 * l + i]

    def view(self, l, name, i):
        return self.layers[l][name][i * self.R:(i + 1) * self.R]

    def rows(self, l, name, lo, hi):
        return self.layers[l][name][lo * self.R:hi * self.R]


class _Slot:
    """Activation stash of one in-flight micro-batch."""

    def __init__(self, cfg: Config, tp, dev, dt, first, last, Vp, group=None, index=0, sp=None, sp_syms=None):
        R, d = cfg.batch * cfg.seq, cfg.d_model
        dl, fo, Hl = d // tp, 4 * d // tp, cfg.n_head // tp
        Rs = R // tp if sp is not None else R          # rows of the residual stream this rank holds
        e = lambda *s: _buf(s, dt, dev)
        f = lambda *s: _buf(s, torch.float32, dev)
        self.x = [e(Rs, d) for _ in range(cfg.n_layer + 1)]   # residual stream: x[l] enters layer l
        self.layers = []
        for l in range(cfg.n_layer):
            g = (lambda name, *shp: group.view(l, name, index)) if group is not None else (lambda name, *shp: e(*shp))
            a = dict(
                ln1=g("ln1", R, d) if sp is None or group is not None else None, mean1=f(Rs), rstd1=f(Rs),
                qkv=e(R, 3 * dl), att=g("att", R, dl),
                lse=f(cfg.batch, Hl, cfg.seq), xmid=e(Rs, d),
                ln2=g("ln2", R, d) if sp is None or group is not None else None, mean2=f(Rs), rstd2=f(Rs),
                pre=e(R, fo), act=g("act", R, fo))
            if group is not None:
                for k in ("d_out", "d_pre", "d_mid", "d_qkv"):
                    a[k] = group.view(l, k, index)
            if sp is not None:
                # gathered operands as SymRows: from the slot group (deferred weight gradients) or this slot's own
                if group is not None:
                    for k in _SlotGroup.SYM:
                        a["sym_" + k] = group.sym[l][k][index]
                else:
                    a["sym_ln1"], a["sym_ln2"] = sp_syms[2 * l][0], sp_syms[2 * l + 1][0]
                    a["ln1"], a["ln2"] = a["sym_ln1"].t, a["sym_ln2"].t
            self.layers.append(a)
        self.tok = torch.zeros(R, dtype=torch.int32, device=dev)
        self.tgt = torch.zeros(R, dtype=torch.int32, device=dev)
        if last:
            if sp is not None:
                self.sym_lnf = sp_syms[-1][0]
                self.lnf, self.meanf, self.rstdf = self.sym_lnf.t, f(Rs), f(Rs)
            else:
                self.lnf, self.meanf, self.rstdf = e(R, d), f(R), f(R)
            self.logits = torch.zeros(R, Vp, dtype=dt, device=dev)
            self.rowloss = f(R)
            self.prob = f(R)
            if tp > 1:      # vocabulary-parallel head: per-rank softmax statistics and their combination
                self.stats = f(R, 3)
                self.stats_all = f(tp, R, 3)
                self.gmax, self.gsum = f(R), f(R)


class GPT:
    def __init__(self, cfg: Config, device="cpu", dtype=torch.bfloat16, tp=1, tp_rank=0, first=True, last=True,
                 untied_head=False, n_slots=1, dp=1, alloc=None, defer_dw=False, sp=None):
        """``sp``: the fused tensor-parallel operators (parallel.fused.FusedTP or FusedTPEmu) to run the
        layers sequence-parallel with; None keeps every activation replicated over the TP group."""
        assert cfg.d_model % cfg.n_head == 0 and cfg.n_head % tp == 0
        assert sp is None or (tp > 1 and cfg.batch % tp == 0), "sequence parallelism splits whole sequences over tp > 1 ranks"
        self.cfg, self.tp, self.tp_rank = cfg, tp, tp_rank
        self.sp = sp
        self.first, self.last = first, last
        self.device, self.dtype = torch.device(device), dtype
        # a separate head matrix exists on the last stage of a multi-stage pipeline (tied to the
        # first stage's wte by a gradient exchange) or when an untied head is requested
        self.has_head = last and (untied_head or not first)
        self.untied_head = untied_head
        self.params = ParamStore(cfg, device, dtype, tp, self.has_head, pad_to=4 * dp if dp > 1 else 1, alloc=alloc)
        self.params.alloc_moments()
        self.step = 0
        self.Vp = _pad64(cfg.vocab)
        # deferred weight gradients: backward only stores each layer's output gradients; flush_dw()
        # forms all weight and bias gradients of the step in one pass over every micro-batch
        self.group = _SlotGroup(cfg, tp, self.device, dtype, n_slots, sp) if defer_dw else None
        R, d = cfg.batch * cfg.seq, cfg.d_model
        dl, fo = d // tp, 4 * d // tp
        e = lambda *s: _buf(s, dtype, self.device)
        Rs = R // tp if sp is not None else R
        sp_syms = [None] * n_slots
        self.sym_dx = None
        if sp is not None:
            # per slot: LayerNorm outputs of every layer (unless the slot group holds them) and of the final
            # norm; shared: two gathered gradient buffers (outside the slot group) and the stage-input gradient
            kw = {} if not sp.emulated else dict(dtype=dtype)
            # (the final norm's buffer is allocated on every stage: ranks that later rendezvous on a group
            # spanning stages must have made the same sequence of symmetric allocations)
            per_slot = (0 if defer_dw else 2 * cfg.n_layer) + 1
            syms, _ = sp.sym_rows(R, d, count=per_slot * n_slots, **kw)
            sp_syms = [syms[i * per_slot:(i + 1) * per_slot] for i in range(n_slots)]
            (self.sym_dx, _) = sp.sym_rows(R, d, count=3, **kw)
            self.sym_dx = [g[0] for g in self.sym_dx]
        self.slots = [_Slot(cfg, tp, self.device, dtype, first, last, self.Vp, self.group, i, sp, sp_syms[i])
                      for i in range(n_slots)]
        # backward scratch, shared by all layers and slots
        self.s_dx = [e(Rs, d), e(Rs, d)]
        self.s_dln = e(Rs, d)
        self.s_dln_full = e(R, d) if sp is not None and last else None
        self.s_dpre = e(R, fo)
        self.s_datt = e(R, dl)
        self.s_dqkv = e(R, 3 * dl)
        self.s_delta = torch.empty(cfg.batch, cfg.n_head // tp, cfg.seq, dtype=torch.float32, device=self.device)
        self.s_lnpart = torch.zeros(ops.layernorm_bwd_scratch_elems(Rs, d) if self.device.type == "cuda" else 2 * d,
                                    dtype=torch.float32, device=self.device)
        self.s_table = torch.empty(2 * cfg.vocab, dtype=torch.int32, device=self.device)
        self.loss_acc = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.tp_allreduce = None      # callable(tensor) summing in place over the TP group
        # callable(layer) invoked as soon as every gradient of that layer is final for the step (last
        # micro-batch's backward, or the last deferred weight-gradient pass): the engine starts the
        # layer's optimizer bucket there, under the backward of the layers below
        self.on_layer_grads = None
        self.skip_loss = False
        # fused tensor-parallel operators (installed by parallel.tp when available)
        self.fused_tp = None
        # vocabulary-parallel head (enable_vocab_parallel): this rank's rows [v0, v1) of the head matrix
        self.vp_group = None
        self.v0, self.v1 = 0, cfg.vocab

    # ------------------------------------------------------------------ parameters
    def L(self, l, name):
        return self.params.c["l%d.%s" % (l, name)]

    def G(self, l, name):
        return self.params.grad["l%d.%s" % (l, name)]

    def init_weights(self, seed: int, layer0: int = 0, total_layers: int | None = None):
        """GPT-2 init N(0, 0.02) from the host xorshift stream, drawn in the global order of the
        whole model so that any TP x PP sharding reassembles to the single-GPU weights
        (src/core/gpt.c:247-264, :301-323, :638-663)."""
        from ..utils.rng import Rng
        cfg, tp, r = self.cfg, self.tp, self.tp_rank
        d, V, S = cfg.d_model, cfg.vocab, cfg.seq
        ff, dl, fo = 4 * d, d // tp, 4 * d // tp
        total = cfg.n_layer if total_layers is None else total_layers
        st = Rng(seed)
        P = self.params.p

        def put(name, t):
            P[name].copy_(t.view(P[name].shape))

        wte = st.normal_block(V, d, 0, V, 0, d, 0.02, keep=self.first or (self.has_head and not self.untied_head))
        if self.first:
            put("wte", wte)
        if self.has_head and not self.untied_head:
            put("head_w", wte)
        wpe = st.normal_block(S, d, 0, S, 0, d, 0.02, keep=self.first)
        if self.first:
            put("wpe", wpe)
        for gl in range(total):
            own = layer0 <= gl < layer0 + cfg.n_layer
            pre = "l%d." % (gl - layer0)
            if own:
                for n in ("ln1_w", "ln2_w"):
                    P[pre + n].fill_(1.0)
                for n in ("ln1_b", "ln2_b", "qkv_b", "proj_b", "fc_b", "fcproj_b"):
                    P[pre + n].zero_()
            # qkv: dl rows from each of the q, k, v thirds
            parts = [st.normal_block(d, d, r * dl, (r + 1) * dl, 0, d, 0.02, keep=own) for _ in range(3)]
            if own:
                put(pre + "qkv_w", torch.cat(parts, 0))
            t = st.normal_block(d, d, 0, d, r * dl, (r + 1) * dl, 0.02, keep=own)
            if own:
                put(pre + "proj_w", t)
            t = st.normal_block(ff, d, r * fo, (r + 1) * fo, 0, d, 0.02, keep=own)
            if own:
                put(pre + "fc_w", t)
            t = st.normal_block(d, ff, 0, d, r * fo, (r + 1) * fo, 0.02, keep=own)
            if own:
                put(pre + "fcproj_w", t)
        if self.has_head and self.untied_head:
            put("head_w", st.normal_block(V, d, 0, V, 0, d, 0.02))
        P["lnf_w"].fill_(1.0)
        P["lnf_b"].zero_()
        self.params.sync_compute_copy()

    def init_weights_device(self, seed: int):
        """N(0, 0.02) drawn on the device (fast start-up for benchmarks; not stream-compatible
        with ``init_weights``).  Replicated tensors use the same generator state on every rank."""
        g = torch.Generator(device=self.device)
        P = self.params.p
        for name in self.params.names:
            t = P[name]
            base = name.split(".")[-1]
            sharded = base in ("qkv_w", "proj_w", "fc_w", "fcproj_w")
            g.manual_seed(seed * 1000003 + (hash(name) % 65536) * 31 + (self.tp_rank if sharded else 0))
            if base.endswith("_b"):
                t.zero_()
            elif base in ("ln1_w", "ln2_w", "lnf_w"):
                t.fill_(1.0)
            else:
                t.normal_(0.0, 0.02, generator=g)
        self.params.sync_compute_copy()

    def load_ref(self, tensors: dict):
        """Load weights from a CHRN fixture (names of tests/gen_reference.py:131-141)."""
        P = self.params.p
        P["wte"].copy_(tensors["wte"])
        P["wpe"].copy_(tensors["wpe"])
        ren = {"ln1_w": "ln1.w", "ln1_b": "ln1.b", "qkv_w": "qkv.w", "qkv_b": "qkv.b", "proj_w": "proj.w",
               "proj_b": "proj.b", "ln2_w": "ln2.w", "ln2_b": "ln2.b", "fc_w": "fc.w", "fc_b": "fc.b",
               "fcproj_w": "fcproj.w", "fcproj_b": "fcproj.b"}
        for l in range(self.cfg.n_layer):
            for f in LAYER_FIELDS:
                P["l%d.%s" % (l, f)].copy_(tensors["blk%d.%s" % (l, ren[f])])
        P["lnf_w"].copy_(tensors["lnf.w"])
        P["lnf_b"].copy_(tensors["lnf.b"])
        self.params.sync_compute_copy()

    def sync_bf16(self):
        self.params.sync_compute_copy()

    def zero_grads(self):
        self.params.g.zero_()

    # ------------------------------------------------------------------ inputs
    def set_input(self, idx, tgt, slot=0):
        s = self.slots[slot]
        s.tok.copy_(idx.reshape(-1), non_blocking=True)
        if tgt is not None:
            s.tgt.copy_(tgt.reshape(-1), non_blocking=True)

    # ------------------------------------------------------------------ forward
    def _ar(self, t):
        if self.tp_allreduce is not None:
            ops.plan_call(self.tp_allreduce, t)

    def _row_parallel(self, a, w, out, bias=None, resid=None, b_mn=False):
        """out = sum over the TP group of a @ op(w) (+ bias + resid).  Single rank: one GEMM with a
        fused epilogue.  TP: the fused GEMM + all-reduce kernel when installed, otherwise the
        baseline -- rank 0 folds bias + residual into its partial product and an NCCL all-reduce
        sums the partials (src/core/gpt.c:686-687)."""
        if self.tp > 1 and self.fused_tp is not None:
            self.fused_tp.gemm_ar(a, w, out, b_mn=b_mn, bias=bias, resid=resid)
            return
        if bias is not None and self.tp_rank == 0:
            ops.gemm(a, w, out, b_mn=b_mn, epi=ops.EPI_BIAS_RESID, bias=bias, aux=resid)
        else:
            ops.gemm(a, w, out, b_mn=b_mn)
        self._ar(out)

    def forward_layers(self, s: _Slot):
        cfg, tp = self.cfg, self.tp
        B, T, Hl, hd = cfg.batch, cfg.seq, cfg.n_head // tp, cfg.head_dim
        for l in range(cfg.n_layer):
            a = s.layers[l]
            x = s.x[l]
            ops.layernorm_fwd(x, self.L(l, "ln1_w"), self.L(l, "ln1_b"), a["ln1"], a["mean1"], a["rstd1"])
            ops.gemm(a["ln1"], self.L(l, "qkv_w"), a["qkv"], epi=ops.EPI_BIAS, bias=self.L(l, "qkv_b"))
            ops.flash_fwd(a["qkv"], a["att"], a["lse"], B, T, Hl, hd)
            self._row_parallel(a["att"], self.L(l, "proj_w"), a["xmid"], self.L(l, "proj_b"), x)
            ops.layernorm_fwd(a["xmid"], self.L(l, "ln2_w"), self.L(l, "ln2_b"), a["ln2"], a["mean2"], a["rstd2"])
            ops.gemm(a["ln2"], self.L(l, "fc_w"), a["act"], epi=ops.EPI_BIAS_GELU, bias=self.L(l, "fc_b"), aux=a["pre"])
            self._row_parallel(a["act"], self.L(l, "fcproj_w"), s.x[l + 1], self.L(l, "fcproj_b"), a["xmid"])

    def head_weight(self):
        return self.params.c["head_w"] if self.has_head else self.params.c["wte"]

    def head_grad(self):
        return self.params.grad["head_w"] if self.has_head else self.params.grad["wte"]

    def enable_vocab_parallel(self, group, src_ranks):
        """Split the head over the TP group by vocabulary rows: every rank computes the logits, the
        softmax gradient and the head's weight gradient only for its own slice [v0, v1); the softmax
        statistics are combined across ranks and the input gradient is summed like any other
        row-parallel product.  ``src_ranks[r]`` is the global rank of TP rank r (for the per-step
        exchange of head-gradient blocks, ``sync_head_grad``).  The reference replicates the head on
        every TP rank (src/core/gpt.c:16)."""
        assert self.last and self.tp > 1
        vs = (self.cfg.vocab + self.tp - 1) // self.tp
        self.v0 = min(self.cfg.vocab, self.tp_rank * vs)
        self.v1 = min(self.cfg.vocab, self.v0 + vs)
        self.vp_group, self.vp_src, self.vp_block = group, list(src_ranks), vs

    def _vp_stats_combine(self, s):
        """Global row maximum, sum and loss from the ranks' vocabulary-slice statistics: one kernel over
        peer memory when the fused operators are installed, else ``_vp_combine`` (collective + PyTorch)."""
        f = self.fused_tp
        if f is not None and hasattr(f, "vp_combine") and s.stats.is_cuda:
            f.vp_combine(s.stats, s.tgt, s.gmax, s.gsum, s.rowloss)
        else:
            ops.plan_call(self._vp_combine, s)

    def _vp_combine(self, s):
        import torch.distributed as dist
        dist.all_gather([s.stats_all[r] for r in range(self.tp)], s.stats, group=self.vp_group)
        m, sm, xt = s.stats_all[..., 0], s.stats_all[..., 1], s.stats_all[..., 2]
        gm = m.max(0).values
        gs = (sm * torch.exp(m - gm)).sum(0)
        s.gmax.copy_(gm)
        s.gsum.copy_(gs)
        s.rowloss.copy_(torch.where(s.tgt >= 0, torch.log(gs) + gm - xt.max(0).values, torch.zeros_like(gm)))

    def sync_head_grad(self):
        """Vocabulary-parallel head: every TP rank holds the head gradient of its own row block only;
        exchange the blocks so that the replicated matrix receives the same full gradient everywhere."""
        if self.vp_group is None:
            return
        import torch.distributed as dist
        g = self.head_grad()
        for r in range(self.tp):
            lo = min(self.cfg.vocab, r * self.vp_block)
            hi = min(self.cfg.vocab, lo + self.vp_block)
            if hi > lo:
                dist.broadcast(g[lo:hi], src=self.vp_src[r], group=self.vp_group)

    def forward_layers_sp(self, s: _Slot):
        """Sequence-parallel layers: x, xmid are row shards; LayerNorm writes this rank's rows of a
        symmetric [R, d] buffer that the column-parallel product gathers; the row-parallel products
        reduce-scatter (+ bias + residual on the shard)."""
        cfg, tp, f = self.cfg, self.tp, self.sp
        B, T, Hl, hd = cfg.batch, cfg.seq, cfg.n_head // tp, cfg.head_dim
        for l in range(cfg.n_layer):
            a = s.layers[l]
            x = s.x[l]
            ops.layernorm_fwd(x, self.L(l, "ln1_w"), self.L(l, "ln1_b"), a["sym_ln1"].mine, a["mean1"], a["rstd1"])
            f.ag_gemm_sym(a["sym_ln1"], self.L(l, "qkv_w"), a["qkv"], epi=ops.EPI_BIAS, bias=self.L(l, "qkv_b"))
            ops.flash_fwd(a["qkv"], a["att"], a["lse"], B, T, Hl, hd)
            f.gemm_rs(a["att"], self.L(l, "proj_w"), a["xmid"], bias=self.L(l, "proj_b"), resid=x)
            ops.layernorm_fwd(a["xmid"], self.L(l, "ln2_w"), self.L(l, "ln2_b"), a["sym_ln2"].mine, a["mean2"], a["rstd2"])
            f.ag_gemm_sym(a["sym_ln2"], self.L(l, "fc_w"), a["act"], epi=ops.EPI_BIAS_GELU, bias=self.L(l, "fc_b"),
                          aux=a["pre"])
            f.gemm_rs(a["act"], self.L(l, "fcproj_w"), s.x[l + 1], bias=self.L(l, "fcproj_b"), resid=a["xmid"])

    def forward_head(self, s: _Slot):
        cfg = self.cfg
        w = self.head_weight()[self.v0:self.v1]
        if self.sp is not None:
            ops.layernorm_fwd(s.x[cfg.n_layer], self.params.c["lnf_w"], self.params.c["lnf_b"], s.sym_lnf.mine, s.meanf,
                              s.rstdf)
            self.sp.ag_gemm_sym(s.sym_lnf, w, s.logits[:, :self.v1 - self.v0])
            return
        ops.layernorm_fwd(s.x[cfg.n_layer], self.params.c["lnf_w"], self.params.c["lnf_b"], s.lnf, s.meanf, s.rstdf)
        ops.gemm(s.lnf, w, s.logits[:, :self.v1 - self.v0])

    def forward(self, slot=0, x_in=None, loss_scale=1.0, accumulate_loss=False, compute_loss=True):
        """Forward of one micro-batch.  First stage embeds ``tok``; other stages take ``x_in``
        ([R, d], copied into the stash).  On the last stage the logits are left in the stash and
        the mean cross-entropy times ``loss_scale`` is added to / stored in ``loss_acc``; returns
        the stage output otherwise."""
        s = self.slots[slot]
        cfg = self.cfg
        if self.first:
            tok = s.tok
            if self.sp is not None:         # this rank's sequences only (a shard is a whole number of sequences)
                rs = tok.numel() // self.tp
                tok = tok[self.tp_rank * rs:(self.tp_rank + 1) * rs]
            ops.embed_fwd(tok, None, self.params.c["wte"], self.params.c["wpe"], s.x[0], cfg.seq)
        else:
            ops.plan_call(s.x[0].copy_, x_in)
        if self.sp is not None:
            self.forward_layers_sp(s)
        else:
            self.forward_layers(s)
        if not self.last:
            return s.x[cfg.n_layer]
        self.forward_head(s)
        if compute_loss and not self.skip_loss:
            assert self.vp_group is None, "with a vocabulary-parallel head the loss comes out of backward()"
            R = cfg.batch * cfg.seq
            ops.xent(s.logits, cfg.vocab, s.tgt, rowloss=s.rowloss, write_grad=False)
            ops.sum_f32(s.rowloss, self.loss_acc, scale=loss_scale / R, accumulate=accumulate_loss)
        return None

    def loss(self) -> float:
        """Host read of the accumulated loss (the only device->host sync of a step)."""
        return float(self.loss_acc.item())

    # ------------------------------------------------------------------ backward
    def backward(self, slot=0, dx_out=None, inv_mb=1.0, coef=None, loss_scale=None, accumulate_loss=False):
        """Backward of one micro-batch; gradients accumulate into the fp32 arena.  Last stage
        starts from the loss (``inv_mb`` = 1/M scales it; ``coef`` [R] replaces the uniform
        cross-entropy weight for GRPO, src/core/gpt.c:558); other stages take ``dx_out``.  Returns
        the gradient w.r.t. the stage input (None on the first stage).  With ``loss_scale`` the
        same pass over the logits also produces the loss (mean CE x loss_scale into ``loss_acc``),
        so a training step reads the logits once."""
        if self.sp is not None:
            return self._backward_sp(slot, dx_out, inv_mb, coef, loss_scale, accumulate_loss)
        s = self.slots[slot]
        cfg, tp = self.cfg, self.tp
        R, V = cfg.batch * cfg.seq, cfg.vocab
        B, T, Hl, hd = cfg.batch, cfg.seq, cfg.n_head // tp, cfg.head_dim
        P, Gd = self.params.c, self.params.grad
        dx, other = self.s_dx
        defer = self.group is not None
        if defer:       # the gradient w.r.t. the stage output lands in the top layer's stash
            dx = s.layers[cfg.n_layer - 1]["d_out"]
        if self.last:
            want_loss = loss_scale is not None and not self.skip_loss
            if self.vp_group is None:
                ops.xent(s.logits, V, s.tgt, coef=coef, uniform=inv_mb / R, write_grad=True,
                         rowloss=s.rowloss if want_loss else None)
                dl = s.logits[:, :V]
                ops.gemm(dl, self.head_weight(), self.s_dln, b_mn=True)
                ops.gemm(dl, s.lnf, self.head_grad(), a_mn=True, b_mn=True, accumulate=True)
            else:
                v0, v1 = self.v0, self.v1
                ops.xent_stats(s.logits, v1 - v0, s.tgt, v0, s.stats)
                self._vp_stats_combine(s)
                ops.xent_grad(s.logits, v1 - v0, s.tgt, v0, s.gmax, s.gsum, coef=coef, uniform=inv_mb / R)
                dl = s.logits[:, :v1 - v0]
                self._row_parallel(dl, self.head_weight()[v0:v1], self.s_dln, b_mn=True)
                ops.gemm(dl, s.lnf, self.head_grad()[v0:v1], a_mn=True, b_mn=True, accumulate=True)
            if want_loss:
                ops.sum_f32(s.rowloss, self.loss_acc, scale=loss_scale / R, accumulate=accumulate_loss)
            ops.layernorm_bwd(self.s_dln, s.x[cfg.n_layer], P["lnf_w"], s.meanf, s.rstdf, None, dx, Gd["lnf_w"],
                              Gd["lnf_b"], self.s_lnpart)
        else:
            ops.plan_call(dx.copy_, dx_out)
        if defer:
            for l in reversed(range(cfg.n_layer)):
                a = s.layers[l]
                nxt = s.layers[l - 1]["d_out"] if l > 0 else self.s_dx[0]
                ops.gemm(a["d_out"], self.L(l, "fcproj_w"), a["d_pre"], b_mn=True, epi=ops.EPI_DGELU, aux=a["pre"])
                self._row_parallel(a["d_pre"], self.L(l, "fc_w"), self.s_dln, b_mn=True)
                ops.layernorm_bwd(self.s_dln, a["xmid"], self.L(l, "ln2_w"), a["mean2"], a["rstd2"], a["d_out"],
                                  a["d_mid"], self.G(l, "ln2_w"), self.G(l, "ln2_b"), self.s_lnpart)
                ops.gemm(a["d_mid"], self.L(l, "proj_w"), self.s_datt, b_mn=True)
                ops.flash_bwd(a["qkv"], a["att"], self.s_datt, a["lse"], a["d_qkv"], self.s_delta, B, T, Hl, hd)
                self._row_parallel(a["d_qkv"], self.L(l, "qkv_w"), self.s_dln, b_mn=True)
                ops.layernorm_bwd(self.s_dln, s.x[l], self.L(l, "ln1_w"), a["mean1"], a["rstd1"], a["d_mid"], nxt,
                                  self.G(l, "ln1_w"), self.G(l, "ln1_b"), self.s_lnpart)
            dx = self.s_dx[0]
            if self.first:
                ops.embed_bwd(s.tok, dx, Gd["wte"], Gd["wpe"], B, T, table=self.s_table)
                return None
            return dx
        for l in reversed(range(cfg.n_layer)):
            a = s.layers[l]
            # x[l+1] = xmid + act @ Wfp^T + b
            ops.gemm(dx, a["act"], self.G(l, "fcproj_w"), a_mn=True, b_mn=True, accumulate=True, colsum=self.G(l, "fcproj_b"))
            ops.gemm(dx, self.L(l, "fcproj_w"), self.s_dpre, b_mn=True, epi=ops.EPI_DGELU, aux=a["pre"])
            ops.gemm(self.s_dpre, a["ln2"], self.G(l, "fc_w"), a_mn=True, b_mn=True, accumulate=True, colsum=self.G(l, "fc_b"))
            self._row_parallel(self.s_dpre, self.L(l, "fc_w"), self.s_dln, b_mn=True)
            ops.layernorm_bwd(self.s_dln, a["xmid"], self.L(l, "ln2_w"), a["mean2"], a["rstd2"], dx, other,
                              self.G(l, "ln2_w"), self.G(l, "ln2_b"), self.s_lnpart)
            dx, other = other, dx
            # xmid = x + att @ Wp^T + b
            ops.gemm(dx, a["att"], self.G(l, "proj_w"), a_mn=True, b_mn=True, accumulate=True, colsum=self.G(l, "proj_b"))
            ops.gemm(dx, self.L(l, "proj_w"), self.s_datt, b_mn=True)
            ops.flash_bwd(a["qkv"], a["att"], self.s_datt, a["lse"], self.s_dqkv, self.s_delta, B, T, Hl, hd)
            ops.gemm(self.s_dqkv, a["ln1"], self.G(l, "qkv_w"), a_mn=True, b_mn=True, accumulate=True, colsum=self.G(l, "qkv_b"))
            self._row_parallel(self.s_dqkv, self.L(l, "qkv_w"), self.s_dln, b_mn=True)
            ops.layernorm_bwd(self.s_dln, s.x[l], self.L(l, "ln1_w"), a["mean1"], a["rstd1"], dx, other,
                              self.G(l, "ln1_w"), self.G(l, "ln1_b"), self.s_lnpart)
            dx, other = other, dx
            if self.on_layer_grads is not None:
                ops.plan_call_host(self.on_layer_grads, l)
        if self.first:
            ops.embed_bwd(s.tok, dx, Gd["wte"], Gd["wpe"], B, T, table=self.s_table)
            return None
        return dx

    def _backward_sp(self, slot, dx_out, inv_mb, coef, loss_scale, accumulate_loss):
        """Backward of one micro-batch with sequence-parallel layers.  Gradients of the residual stream are
        row shards; each is written into this rank's rows of a symmetric [R, d] buffer, gathered by the
        input-gradient product of the row-parallel layer (all-gather -> GEMM, which leaves the full matrix
        behind for the weight gradient), and the input gradients of the column-parallel layers come back
        as shards (GEMM -> reduce-scatter)."""
        s = self.slots[slot]
        cfg, tp, f = self.cfg, self.tp, self.sp
        R, V = cfg.batch * cfg.seq, cfg.vocab
        B, T, Hl, hd = cfg.batch, cfg.seq, cfg.n_head // tp, cfg.head_dim
        P, Gd = self.params.c, self.params.grad
        defer = self.group is not None
        L = cfg.n_layer
        # gathered-gradient buffers: per layer and slot under deferred weight gradients, else two shared ones
        d_out = (lambda l: s.layers[l]["sym_d_out"]) if defer else (lambda l: self.sym_dx[1])
        d_mid = (lambda l: s.layers[l]["sym_d_mid"]) if defer else (lambda l: self.sym_dx[2])
        top = d_out(L - 1)
        if self.last:
            want_loss = loss_scale is not None and not self.skip_loss
            if self.vp_group is None:
                ops.xent(s.logits, V, s.tgt, coef=coef, uniform=inv_mb / R, write_grad=True,
                         rowloss=s.rowloss if want_loss else None)
                dl = s.logits[:, :V]
                # replicated head: every rank holds the full input gradient, its own rows are the shard
                ops.gemm(dl, self.head_weight(), self.s_dln_full, b_mn=True)
                rs = R // tp
                ops.plan_call(self.s_dln.copy_, self.s_dln_full[self.tp_rank * rs:(self.tp_rank + 1) * rs])
                ops.gemm(dl, s.lnf, self.head_grad(), a_mn=True, b_mn=True, accumulate=True)
            else:
                v0, v1 = self.v0, self.v1
                ops.xent_stats(s.logits, v1 - v0, s.tgt, v0, s.stats)
                self._vp_stats_combine(s)
                ops.xent_grad(s.logits, v1 - v0, s.tgt, v0, s.gmax, s.gsum, coef=coef, uniform=inv_mb / R)
                dl = s.logits[:, :v1 - v0]
                f.gemm_rs(dl, self.head_weight()[v0:v1], self.s_dln, b_mn=True)
                ops.gemm(dl, s.lnf, self.head_grad()[v0:v1], a_mn=True, b_mn=True, accumulate=True)
            if want_loss:
                ops.sum_f32(s.rowloss, self.loss_acc, scale=loss_scale / R, accumulate=accumulate_loss)
            ops.layernorm_bwd(self.s_dln, s.x[L], P["lnf_w"], s.meanf, s.rstdf, None, top.mine, Gd["lnf_w"],
                              Gd["lnf_b"], self.s_lnpart)
        else:
            ops.plan_call(top.mine.copy_, dx_out)
        for l in reversed(range(L)):
            a = s.layers[l]
            so, sm = d_out(l), d_mid(l)
            nxt = d_out(l - 1) if l > 0 else self.sym_dx[0]
            d_pre = a["d_pre"] if defer else self.s_dpre
            d_qkv = a["d_qkv"] if defer else self.s_dqkv
            # x[l+1] = xmid + act @ Wfp^T + b: gather d x[l+1], d_pre = (dx Wfp) * gelu'(pre)
            f.ag_gemm_sym(so, self.L(l, "fcproj_w"), d_pre, b_mn=True, epi=ops.EPI_DGELU, aux=a["pre"])
            if not defer:
                ops.gemm(so.t, a["act"], self.G(l, "fcproj_w"), a_mn=True, b_mn=True, accumulate=True,
                         colsum=self.G(l, "fcproj_b"))
                ops.gemm(d_pre, a["ln2"], self.G(l, "fc_w"), a_mn=True, b_mn=True, accumulate=True, colsum=self.G(l, "fc_b"))
            f.gemm_rs(d_pre, self.L(l, "fc_w"), self.s_dln, b_mn=True)
            ops.layernorm_bwd(self.s_dln, a["xmid"], self.L(l, "ln2_w"), a["mean2"], a["rstd2"], so.mine, sm.mine,
                              self.G(l, "ln2_w"), self.G(l, "ln2_b"), self.s_lnpart)
            # xmid = x + att @ Wp^T + b
            f.ag_gemm_sym(sm, self.L(l, "proj_w"), self.s_datt, b_mn=True)
            if not defer:
                ops.gemm(sm.t, a["att"], self.G(l, "proj_w"), a_mn=True, b_mn=True, accumulate=True,
                         colsum=self.G(l, "proj_b"))
            ops.flash_bwd(a["qkv"], a["att"], self.s_datt, a["lse"], d_qkv, self.s_delta, B, T, Hl, hd)
            if not defer:
                ops.gemm(d_qkv, a["ln1"], self.G(l, "qkv_w"), a_mn=True, b_mn=True, accumulate=True,
                         colsum=self.G(l, "qkv_b"))
            f.gemm_rs(d_qkv, self.L(l, "qkv_w"), self.s_dln, b_mn=True)
            ops.layernorm_bwd(self.s_dln, s.x[l], self.L(l, "ln1_w"), a["mean1"], a["rstd1"], sm.mine, nxt.mine,
                              self.G(l, "ln1_w"), self.G(l, "ln1_b"), self.s_lnpart)
            if not defer and self.on_layer_grads is not None:
                ops.plan_call_host(self.on_layer_grads, l)
        dx = self.sym_dx[0]
        if self.first:
            # the embedding backward is replicated (no gradient exchange for wte / wpe): gather dx first
            f.all_gather_rows(dx)
            ops.embed_bwd(s.tok, dx.t, Gd["wte"], Gd["wpe"], B, T, table=self.s_table)
            return None
        return dx.mine

    def sp_partial_grads(self):
        """Gradients of the replicated parameters that each rank formed from its own rows only under
        sequence parallelism (LayerNorm gains and biases): to be summed over the TP group once per step."""
        names = ["lnf_w", "lnf_b"] if self.last else []
        for l in range(self.cfg.n_layer):
            names += ["l%d.%s" % (l, n) for n in ("ln1_w", "ln1_b", "ln2_w", "ln2_b")]
        return [self.params.grad[n] for n in names]

    def flush_dw(self, lo=0, hi=None):
        """Weight and bias gradients of all layers from the stashed output gradients of micro-batch
        slots [lo, hi): one product over (hi - lo) * R rows per weight instead of one per
        micro-batch (the reference forms them inside every micro-batch's backward,
        src/core/gpt.c:726-761)."""
        g = self.group
        hi = g.n if hi is None else hi
        if hi <= lo:
            return
        pairs = (("d_out", "act", "fcproj"), ("d_pre", "ln2", "fc"), ("d_mid", "att", "proj"), ("d_qkv", "ln1", "qkv"))
        for l in reversed(range(self.cfg.n_layer)):
            for dy, x, name in pairs:
                dyr, xr = g.rows(l, dy, lo, hi), g.rows(l, x, lo, hi)
                ops.gemm(dyr, xr, self.G(l, name + "_w"), a_mn=True, b_mn=True, accumulate=True,
                         colsum=self.G(l, name + "_b"))
            if hi == g.n and self.on_layer_grads is not None:
                ops.plan_call_host(self.on_layer_grads, l)

    def gather_prob(self, slot=0):
        """p(target) per row from the logits of the last forward (src/core/kernels.cu:372-378)."""
        s = self.slots[slot]
        ops.xent(s.logits, self.cfg.vocab, s.tgt, prob=s.prob, write_grad=False)
        return s.prob

    # ------------------------------------------------------------------ optimizer
    def adamw_step(self, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, grad_scale=1.0, lo=0, hi=None, advance=True):
        """Fused AdamW over the flat arena (src/core/adamw.c:9-16), or over elements [lo, hi) of it; also
        refreshes the bf16 compute copy and clears the gradients for the next accumulation.  The update
        is elementwise, so any partition of the arena into ranges gives the same bits as one sweep."""
        if advance:
            self.step += 1
        ps = self.params
        hi = ps.w.numel() if hi is None else hi
        if hi <= lo:
            return
        wb = None if ps.wb is ps.w else ps.wb[lo:hi]
        ops.adamw(ps.w[lo:hi], ps.g[lo:hi], ps.m[lo:hi], ps.v[lo:hi], wb, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                  wd=wd, step=self.step, grad_scale=grad_scale, zero_grad=True)

    def layer_range(self, l):
        """Elements [lo, hi) of the flat arena that belong to layer l (alignment gaps included)."""
        off = self.params.offsets
        lo = off["l%d.ln1_w" % l]
        hi = off["l%d.ln1_w" % (l + 1)] if l + 1 < self.cfg.n_layer else off["lnf_w"]
        return lo, hi

    # ------------------------------------------------------------------ checkpoint
    def save(self, path, rng_state=0, moments=None):
        from ..utils import ckpt
        ps = self.params
        m, v = moments if moments is not None else (ps.m[:ps.n_flat], ps.v[:ps.n_flat])
        ckpt.save(path, self.cfg.as_list(), self.step, rng_state, ps.w[:ps.n_flat], m, v)

    def load(self, path, moments=None):
        from ..utils import ckpt
        ps = self.params
        m, v = moments if moments is not None else (ps.m[:ps.n_flat], ps.v[:ps.n_flat])
        self.step, rng = ckpt.load(path, self.cfg.as_list(), ps.w[:ps.n_flat], m, v)
        ps.sync_compute_copy()
        return rng

    def memory_bytes(self):
        ps = self.params
        tot = sum(t.numel() * t.element_size() for t in (ps.w, ps.g, ps.m, ps.v))
        if ps.wb is not ps.w:
            tot += ps.wb.numel() * ps.wb.element_size()
        return tot
