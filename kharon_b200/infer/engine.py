"""Paged-KV inference engine: continuous batching, copy-on-write prefix sharing, on-device
sampling, CUDA-graph decode steps.

Division of labour:

* native scheduler (csrc/runtime/kharon_rt.cpp, ``kh_eng_*``): reference-counted block pool
  with a LIFO free list, per-sequence block tables, admission of waiting sequences, the flat
  token list of each mixed prefill+decode step, copy-on-write of shared blocks, retirement;
* this module: device buffers, one packed host->device metadata copy per step, the forward
  pass on the native kernels, the sampler, one small device->host copy of the sampled ids.

Differences from the reference engine (src/core/infer.c): sampling runs on the GPU, so a step
moves ``n_seq`` ints to the host instead of ``n_seq x vocab`` logits (:183-195); block sharing
is reference-counted and lazy (a shared block is copied when a sequence first writes into
it) instead of an eager copy of the partial block at fork time (:315-387); decode steps of a
fixed batch size replay a captured CUDA graph; no fixed-size stack arrays (:231-233,280,323).
Accounting (tokens_decoded counts one token per active sequence per step, the prefill step
included) follows infer.c:295 so that tok/s is comparable.
"""
from __future__ import annotations

import ctypes as C
import os
import time

import torch

from .. import _native, ops
from ..models import GPT


class InferStats(dict):
    pass


class InferEngine:
    def __init__(self, model: GPT, block_size=16, n_blocks=None, max_tokens=None, max_seqs=33, use_graphs=True,
                 persistent_decode=None, attn_splits=None, flash_prefill=True):
        cfg = model.cfg
        self.model, self.cfg = model, cfg
        self.dev, self.dt = model.device, model.dtype
        self.tp = model.tp
        self.bs = block_size
        self.max_lb = (cfg.seq + block_size - 1) // block_size
        self.max_seqs = max_seqs
        self.n_blocks = n_blocks if n_blocks is not None else max_seqs * self.max_lb + 16
        self.max_tokens = max_tokens if max_tokens is not None else max(cfg.seq, max_seqs) + 64
        self.Hl, self.hd = cfg.n_head // self.tp, cfg.head_dim
        lib = _native.rt()
        self._h = lib.kh_eng_create(self.bs, self.n_blocks, max_seqs, self.max_lb)
        if not self._h:
            raise _native.NativeError(lib.kh_last_error().decode())
        L, d, dl, fo = cfg.n_layer, cfg.d_model, cfg.d_model // self.tp, 4 * cfg.d_model // self.tp
        z = dict(device=self.dev)
        self.kc = torch.zeros(L, self.n_blocks, self.bs, self.Hl, self.hd, dtype=self.dt, **z)
        self.vc = torch.zeros_like(self.kc)
        # packed step metadata: tok | pos | slot | rows | btab | pairs
        mt, ms_ = self.max_tokens, max_seqs
        self._o_tok, self._o_pos, self._o_slot = 0, mt, 2 * mt
        self._o_rows = 3 * mt
        self._o_btab = 3 * mt + ms_
        self._o_pairs = self._o_btab + ms_ * self.max_lb
        self._o_step = self._o_pairs + 2 * ms_ * 4          # the step number: sampled steps replayed from a graph read it here
        self._n_meta = self._o_step + 4                      # {step number, seed low, seed high, unused}
        pin = self.dev.type == "cuda"
        self.h_meta = torch.zeros(self._n_meta, dtype=torch.int32, pin_memory=pin)
        self.h_seq_ids = torch.zeros(ms_, dtype=torch.int32)
        self.d_meta = torch.zeros(self._n_meta, dtype=torch.int32, **z)
        v = lambda t, o, n: t[o:o + n]
        self.d_tok, self.d_pos, self.d_slot = v(self.d_meta, 0, mt), v(self.d_meta, mt, mt), v(self.d_meta, 2 * mt, mt)
        self.d_rows = v(self.d_meta, self._o_rows, ms_)
        self.d_btab = v(self.d_meta, self._o_btab, ms_ * self.max_lb).view(ms_, self.max_lb)
        self.d_pairs = v(self.d_meta, self._o_pairs, 2 * ms_ * 4)
        self.d_stepno = v(self.d_meta, self._o_step, 3)
        e = lambda *s: torch.empty(*s, dtype=self.dt, **z)
        self.x = [e(mt, d), e(mt, d)]
        self.xmid, self.ln, self.qkv, self.att = e(mt, d), e(mt, d), e(mt, 3 * dl), e(mt, dl)
        self.pre, self.act = e(mt, fo), e(mt, fo)
        self.last = e(ms_, d)
        self.lnf = e(ms_, d)
        self.logits = torch.zeros(ms_, model.Vp, dtype=self.dt, **z)
        self.d_out = torch.zeros(ms_ * 64, dtype=torch.int32, **z)
        self.h_out = torch.zeros(ms_ * 64, dtype=torch.int32, pin_memory=pin)
        # decode steps (few rows) use the weight-streaming split-K GEMM; its scratch covers every shape used
        self.skinny = None
        if self.dev.type == "cuda":
            shapes = [(3 * dl, d), (d, dl), (fo, d), (d, fo), (cfg.vocab, d)]
            n = max(ops.gemm_skinny_scratch_elems(ops.SKINNY_MAX_ROWS, N, K) for N, K in shapes)
            self.skinny = torch.zeros(n, dtype=torch.float32, **z)
        # Decode steps of up to ``persistent_max`` sequences run all layers and the head in one persistent kernel
        # when the shape allows it (ops.decode_layers); KHARON_PERSISTENT_DECODE=0 or persistent_decode=False keeps
        # the five-kernel chain.  Measured on B200 (L24 d1024): 945 / 6407 / 9614 tok/s against 728 / 4201 / 7301 at
        # G = 1 / 8 / 16; at G = 32 the chain's 128-row tensor-core tiles win (15.9k against 13.3k), hence 16.
        if persistent_decode is None:
            persistent_decode = os.environ.get("KHARON_PERSISTENT_DECODE", "1") != "0"
        self.persistent = bool(persistent_decode and self.skinny is not None and self.tp == 1 and self.dt == torch.bfloat16
                               and ops.decode_layers_ok(1, d, cfg.n_head, cfg.head_dim, cfg.seq))
        self.persistent_max = int(os.environ.get("KHARON_PERSISTENT_MAX_G", "16"))
        if self.persistent:
            names = ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "ln2_w", "ln2_b", "fc_w", "fc_b",
                     "fcproj_w", "fcproj_b")
            self.layer_table = torch.tensor([[model.L(l, n).data_ptr() for n in names] for l in range(L)],
                                            dtype=torch.int64, device=self.dev)
            self.grid_bar = torch.zeros(4, dtype=torch.int32, **z)
        # Contexts beyond 2048 positions: the keys of a token are cut into ranges with a CTA each (split-KV) and merged
        self.attn_splits = int(attn_splits) if attn_splits else (1 if cfg.seq <= 2048 else min(16, (cfg.seq + 2047) // 2048))
        self.attn_scratch = None
        if self.attn_splits > 1 and self.dev.type == "cuda":
            self.attn_scratch = torch.zeros(self.max_tokens * self.Hl * self.attn_splits * (self.hd + 1), dtype=torch.float32, **z)
        # Steps made of whole fresh prompts (every listed token belongs to a sequence that starts at position 0 in this
        # step) run their attention on the tensor cores with the training forward kernel, one launch per prompt;
        # everything else (decode steps, chunked prompts, mixed steps) goes through the paged kernel.
        self.flash_prefill = bool(flash_prefill and self.dev.type == "cuda" and self.dt == torch.bfloat16
                                  and self.hd in (64, 128))
        self.lse_buf = torch.zeros(self.Hl * self.max_tokens, dtype=torch.float32, **z) if self.flash_prefill else None
        self._fresh = None
        self.temperature, self.seed, self.step_no = 0.0, 0, 0
        # under TP the captured step contains the fused GEMM + all-reduce kernels (their call counter
        # is a device word); the NCCL seam is left to eager launches
        self.use_graphs = bool(use_graphs and self.dev.type == "cuda" and self.dt == torch.bfloat16
                               and (self.tp == 1 or getattr(model, "fused_tp", None) is not None))
        self.graphs = {}
        self._warm = set()
        self.d_step = None
        self.launches = 0

    def close(self):
        if self._h:
            _native.rt().kh_eng_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_sampling(self, temperature: float, seed: int):
        """temperature <= 0: greedy.  Otherwise categorical draws seeded by (seed, step, row)."""
        self.temperature, self.seed = float(temperature), int(seed)       # (captured steps are keyed by the temperature;
                                                                          #  seed and step number travel in d_meta)

    def set_eos(self, eos: int):
        _native.rt().kh_eng_set_eos(self._h, eos)

    # ------------------------------------------------------------------ forward
    def _forward(self, ntok, nseq, rep=1):
        m, cfg = self.model, self.cfg
        P = m.params.c
        x, nxt = self.x
        tok, pos, slot = self.d_tok[:ntok], self.d_pos[:ntok], self.d_slot[:ntok]
        xs = x[:ntok]
        ops.embed_fwd(tok, pos, P["wte"], P["wpe"], xs, cfg.seq)
        fused_layers = (self.persistent and ntok == nseq and ntok <= self.persistent_max
                        and ops.decode_layers_ok(ntok, cfg.d_model, cfg.n_head, cfg.head_dim, cfg.seq))
        if fused_layers:      # layers and head in one kernel; only the sampler follows
            ops.decode_layers(xs, self.xmid[:ntok], self.qkv[:ntok], self.att[:ntok], self.act[:ntok], self.layer_table,
                              cfg.n_layer, self.Hl, self.hd, self.kc, self.vc, pos, slot, self.d_btab, self.bs, cfg.seq,
                              self.grid_bar, head_w=m.head_weight(), lnf_w=P["lnf_w"], lnf_b=P["lnf_b"], logits=self.logits,
                              vocab=cfg.vocab, rows=self.d_rows, n_rows=nseq)
            ops.sample(self.logits, cfg.vocab, self.temperature, self.seed, self.step_no, rep, self.d_out, nseq,
                       step_dev=self.d_stepno)
            return
        for l in range(cfg.n_layer):
            ln, qkv, att, xmid = self.ln[:ntok], self.qkv[:ntok], self.att[:ntok], self.xmid[:ntok]
            self._ln_lin(xs, m.L(l, "ln1_w"), m.L(l, "ln1_b"), ln, m.L(l, "qkv_w"), qkv, ops.EPI_BIAS, m.L(l, "qkv_b"))
            decode = ntok == nseq        # one new token per sequence: the attention kernel appends k, v itself
            if not decode:
                ops.append_kv(qkv, self.kc[l], self.vc[l], pos, slot, self.d_btab, self.bs, self.Hl, self.hd, ntok)
            if not decode and self._fresh:
                for r0, T in self._fresh:
                    ops.flash_fwd(qkv[r0:r0 + T], att[r0:r0 + T], self.lse_buf, 1, T, self.Hl, self.hd)
            else:
                ops.paged_attn(qkv, self.kc[l], self.vc[l], att, pos, slot, self.d_btab, self.bs, self.Hl, self.hd, ntok,
                               cfg.seq, append=decode, n_split=self.attn_splits, scratch=self.attn_scratch)
            # row-parallel products: one GEMM, or under TP the fused GEMM + all-reduce kernel / NCCL seam
            self._row(att, m.L(l, "proj_w"), xmid, m.L(l, "proj_b"), xs)
            self._ln_lin(xmid, m.L(l, "ln2_w"), m.L(l, "ln2_b"), ln, m.L(l, "fc_w"), self.act[:ntok], ops.EPI_BIAS_GELU,
                         m.L(l, "fc_b"), self.pre[:ntok])
            ys = nxt[:ntok]
            self._row(self.act[:ntok], m.L(l, "fcproj_w"), ys, m.L(l, "fcproj_b"), xmid)
            x, nxt = nxt, x
            xs = ys
        ops.gather_rows(xs, self.d_rows, self.last, nseq)
        self._ln_lin(self.last[:nseq], P["lnf_w"], P["lnf_b"], self.lnf[:nseq], m.head_weight(),
                     self.logits[:nseq, :cfg.vocab])
        ops.sample(self.logits, cfg.vocab, self.temperature, self.seed, self.step_no, rep, self.d_out, nseq,
                       step_dev=self.d_stepno)

    def _lin(self, x, w, out, epi=ops.EPI_NONE, bias=None, aux=None):
        """Column-parallel / replicated linear layer: skinny kernel for decode-sized inputs."""
        if self.skinny is not None and x.shape[0] <= ops.SKINNY_BEST_ROWS:
            ops.gemm_skinny(x, w, out, self.skinny, epi=epi, bias=bias, aux=aux, weights_static=True)
        else:
            ops.gemm(x, w, out, epi=epi, bias=bias, aux=aux)

    def _ln_lin(self, x, ln_w, ln_b, ln_out, w, out, epi=ops.EPI_NONE, bias=None, aux=None):
        """LayerNorm followed by a linear layer: for decode-sized inputs the skinny kernel normalises
        the rows itself (no LayerNorm launch, ``ln_out`` stays unused)."""
        if self.skinny is not None and x.shape[0] <= ops.SKINNY_BEST_ROWS and x.shape[1] % 8 == 0:
            ops.gemm_skinny(x, w, out, self.skinny, epi=epi, bias=bias, aux=aux, ln_w=ln_w, ln_b=ln_b, weights_static=True)
        else:
            ops.layernorm_fwd(x, ln_w, ln_b, ln_out)
            self._lin(ln_out, w, out, epi, bias, aux)

    def _row(self, x, w, out, bias, resid):
        """Row-parallel linear layer (+ bias + residual); summed over the TP group when there is one."""
        if self.tp == 1:
            self._lin(x, w, out, ops.EPI_BIAS_RESID, bias, resid)
        else:
            self.model._row_parallel(x, w, out, bias, resid)

    def _fresh_prompts(self, ntok, nseq):
        """[(first row, length)] when every token of the step belongs to a prompt that starts at position 0 and is
        listed whole and contiguously; None otherwise (read from the host copy of the step's metadata)."""
        if not self.flash_prefill or ntok == nseq:
            return None
        pos = self.h_meta[self._o_pos:self._o_pos + ntok]
        slot = self.h_meta[self._o_slot:self._o_slot + ntok]
        cuts = [0] + (torch.nonzero(slot[1:] != slot[:-1]).flatten() + 1).tolist() + [ntok]
        out = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            if int(pos[a]) != 0 or int(pos[b - 1]) != b - a - 1 or b - a < 64:     # (short prompts: not worth a launch each)
                return None
            out.append((a, b - a))
        return out if len(out) == nseq else None

    def _run(self, ntok, nseq, rep=1):
        """Metadata is already in ``h_meta``; runs one step and returns the sampled ids (host)."""
        self._fresh = self._fresh_prompts(ntok, nseq)
        sd = self.seed & 0xFFFFFFFFFFFFFFFF
        to_i32 = lambda u: u - (1 << 32) if u >= (1 << 31) else u
        self.h_meta[self._o_step] = self.step_no & 0x7FFFFFFF
        self.h_meta[self._o_step + 1] = to_i32(sd & 0xFFFFFFFF)
        self.h_meta[self._o_step + 2] = to_i32(sd >> 32)
        self.d_meta.copy_(self.h_meta, non_blocking=True)
        key = (ntok, nseq, rep, self.temperature)
        if self.use_graphs and ntok == nseq:           # greedy and sampled steps alike: the step number lives in d_meta
            g = self.graphs.get(key)
            if g is None and key in self._warm:
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._forward(ntok, nseq, rep)
                self.graphs[key] = g
            if g is not None:
                g.replay()
            else:
                self._forward(ntok, nseq, rep)
                self._warm.add(key)
        else:
            self._forward(ntok, nseq, rep)
        self.step_no += 1
        n = nseq * rep
        self.h_out[:n].copy_(self.d_out[:n], non_blocking=True)
        if self.dev.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return self.h_out[:n]

    # ------------------------------------------------------------------ scheduling
    def _plan(self, max_active):
        lib, hm = _native.rt(), self.h_meta
        base = hm.data_ptr()
        n_tok, n_seq, n_pairs = C.c_int32(), C.c_int32(), C.c_int32()
        rc = lib.kh_eng_plan(self._h, max_active, self.max_tokens, base + 4 * self._o_tok, base + 4 * self._o_pos,
                             base + 4 * self._o_slot, base + 4 * self._o_rows, self.h_seq_ids.data_ptr(),
                             base + 4 * self._o_btab, C.byref(n_tok), C.byref(n_seq), base + 4 * self._o_pairs,
                             self.max_seqs * 4, C.byref(n_pairs))
        _native.rt_check(rc)
        return rc, n_tok.value, n_seq.value, n_pairs.value

    def _step(self, max_active):
        rc, ntok, nseq, npairs = self._plan(max_active)
        if rc == 1 or nseq == 0:
            return False
        if npairs:
            self.d_meta.copy_(self.h_meta, non_blocking=True)
            ops.copy_blocks(self.kc, self.vc, self.d_pairs, npairs)
        out = self._run(ntok, nseq)
        _native.rt_check(_native.rt().kh_eng_commit(self._h, out.data_ptr(), nseq))
        return True

    def _stats(self):
        st = (C.c_int64 * 4)()
        _native.rt().kh_eng_stats(self._h, st)
        return InferStats(blocks_total=st[0], blocks_peak=st[1], tokens_decoded=st[2], prefix_blocks_saved=st[3])

    def _tokens(self, sid):
        lib = _native.rt()
        n = lib.kh_eng_seq_len(self._h, sid)
        buf = torch.empty(n, dtype=torch.int32)
        lib.kh_eng_seq_tokens(self._h, sid, buf.data_ptr(), n)
        return buf.tolist()

    def _timer(self):
        if self.dev.type == "cuda":
            torch.cuda.synchronize()
        return time.perf_counter()

    def generate(self, prompts, n_new, max_active=None):
        """Independent generations with continuous batching: at most ``max_active`` sequences in
        flight, waiting ones are admitted as soon as a slot and blocks are free
        (infer_generate, src/core/infer.c:264-313).  Returns (token lists, stats, ms)."""
        lib = _native.rt()
        lib.kh_eng_reset(self._h)
        n = len(prompts)
        news = [n_new] * n if isinstance(n_new, int) else list(n_new)
        max_active = max_active or min(n, self.max_seqs)
        pending = list(range(n))
        sid_of = {}
        outs = [None] * n
        t0 = self._timer()
        while True:
            # feed the scheduler as sequence slots free up
            while pending:
                i = pending[0]
                p = torch.tensor(prompts[i], dtype=torch.int32)
                sid = lib.kh_eng_add(self._h, p.data_ptr(), len(prompts[i]), news[i])
                if sid < 0:
                    if not sid_of:
                        _native.rt_check(sid)
                    break
                sid_of[sid] = i
                pending.pop(0)
            progressed = self._step(max_active)
            for sid, i in list(sid_of.items()):
                if lib.kh_eng_seq_done(self._h, sid):
                    outs[i] = self._tokens(sid)
                    lib.kh_eng_release(self._h, sid)
                    del sid_of[sid]
            if not progressed and not pending and not sid_of:
                break
            if not progressed and not sid_of and pending:
                raise _native.NativeError("generate: cannot admit the next sequence")
        ms = (self._timer() - t0) * 1e3
        return outs, self._stats(), ms

    def generate_group(self, prompt, G, n_new):
        """G samples from one shared prompt: the prompt is prefilled once, all of its blocks are
        shared by reference, the first token of every sample is drawn from the single prefill
        logits row, and a block is copied only when a sample first writes into it
        (infer_generate_group, src/core/infer.c:315-387)."""
        lib = _native.rt()
        lib.kh_eng_reset(self._h)
        t0 = self._timer()
        p = torch.tensor(prompt, dtype=torch.int32)
        parent = _native.rt_check(lib.kh_eng_add(self._h, p.data_ptr(), len(prompt), 0))
        rc, ntok, nseq, npairs = self._plan(1)
        first = self._run(ntok, nseq, rep=G).clone()
        _native.rt_check(lib.kh_eng_commit(self._h, first.data_ptr(), nseq))
        kids = torch.zeros(G, dtype=torch.int32)
        _native.rt_check(lib.kh_eng_fork(self._h, parent, G, n_new, kids.data_ptr()))
        lib.kh_eng_release(self._h, parent)
        for g in range(G):
            _native.rt_check(lib.kh_eng_push(self._h, int(kids[g]), int(first[g])))
        while self._step(G):
            pass
        outs = [self._tokens(int(k)) for k in kids]
        for k in kids:
            lib.kh_eng_release(self._h, int(k))
        ms = (self._timer() - t0) * 1e3
        return outs, self._stats(), ms

    def generate_groups(self, prompts, G, n_new):
        """``generate_group`` for several prompts at once (one GRPO rollout batch): all prompts are
        prefilled in one step, each is forked G ways with its first tokens drawn from its own
        logits row, then all len(prompts) * G samples decode together.  Returns
        ([prompt][g] -> tokens, stats, ms)."""
        lib = _native.rt()
        lib.kh_eng_reset(self._h)
        t0 = self._timer()
        parents = []
        for pr in prompts:
            p = torch.tensor(pr, dtype=torch.int32)
            parents.append(_native.rt_check(lib.kh_eng_add(self._h, p.data_ptr(), len(pr), 0)))
        rc, ntok, nseq, npairs = self._plan(len(prompts))
        assert nseq == len(prompts), "prefill of all prompts must fit one step"
        order = self.h_seq_ids[:nseq].tolist()
        first = self._run(ntok, nseq, rep=G).clone()
        _native.rt_check(lib.kh_eng_commit(self._h, first.data_ptr(), nseq))
        kids_of = {}
        kids = torch.zeros(G, dtype=torch.int32)
        for row, parent in enumerate(order):
            _native.rt_check(lib.kh_eng_fork(self._h, parent, G, n_new, kids.data_ptr()))
            lib.kh_eng_release(self._h, parent)
            kids_of[parent] = kids.tolist()
            for g in range(G):
                _native.rt_check(lib.kh_eng_push(self._h, int(kids[g]), int(first[row * G + g])))
        while self._step(len(prompts) * G):
            pass
        outs = [[self._tokens(k) for k in kids_of[p]] for p in parents]
        for p in parents:
            for k in kids_of[p]:
                lib.kh_eng_release(self._h, k)
        ms = (self._timer() - t0) * 1e3
        return outs, self._stats(), ms

    def kv_bytes_per_position(self):
        return 2 * self.cfg.n_layer * self.Hl * self.hd * self.kc.element_size()


def smoke_decode():
    """Tiny paged decode on cuda:0 (part of the driver's smoke check)."""
    from ..models import Config
    cfg = Config(2, 128, 2, 512, 128, 1)
    m = GPT(cfg, "cuda:0", torch.bfloat16)
    m.init_weights(1234)
    eng = InferEngine(m, block_size=16, max_seqs=5)
    prompt = [(i * 131 + 7) % cfg.vocab for i in range(20)]
    outs, st, ms = eng.generate_group(prompt, 4, 12)
    assert all(len(o) == 32 for o in outs) and all(o == outs[0] for o in outs)
    ops.check_device_status()
    print("smoke: paged decode 4 x 12 tokens, %d blocks peak, %d prefix blocks shared" % (st["blocks_peak"],
                                                                                      st["prefix_blocks_saved"]))
    # a width the persistent decode kernel takes (all layers and the head of a step in one launch)
    cfg = Config(2, 512, 8, 512, 128, 1)
    m = GPT(cfg, "cuda:0", torch.bfloat16)
    m.init_weights(1234)
    eng = InferEngine(m, block_size=16, max_seqs=5)
    outs, st, ms = eng.generate_group(prompt, 4, 12)
    assert eng.persistent and all(len(o) == 32 for o in outs) and all(o == outs[0] for o in outs)
    ops.check_device_status()
    print("smoke: persistent decode kernel, 4 x 12 tokens")
