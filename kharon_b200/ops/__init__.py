"""Operator layer: thin Python wrappers over the hand-written sm_100a kernels.

Every function works in place on caller-supplied tensors (the model owns flat arenas and
stashes, nothing here allocates on the hot path).  On CUDA tensors the native kernel runs
on the current stream; a missing library is an error, never a fallback.  On CPU tensors
the same operation is evaluated with PyTorch in fp32 (``reference.py``) -- that path is the
numerical oracle of the GPU tests and what the CPU test tier exercises.
"""
from __future__ import annotations

import math

import torch

from .. import _native
from . import reference as ref

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESID, EPI_DGELU, EPI_RESID = range(6)

#: number of native kernel launches issued through this module (bench.py reports it)
launch_count = 0


class KernelError(RuntimeError):
    pass


def _lib():
    return _native.cuda()


def _stream():
    return torch.cuda.current_stream().cuda_stream


#: when a list, every native call is also appended as (function, args, launches) -- see ``LaunchPlan``
_recording = None


def _chk(rc, n=1):
    global launch_count
    if rc != 0:
        raise KernelError(_lib().kh_cuda_last_error().decode())
    launch_count += n


def _call(fn, n, *args):
    """Invoke a native entry point; remember the exact call when a plan is being recorded."""
    if _recording is not None:
        _recording.append((fn, args, n))
    _chk(fn(*args), n)


class LaunchPlan:
    """Record-and-replay of a fixed sequence of native calls.

    A training micro-batch issues the same kernels on the same static buffers every step, so
    the Python-side argument marshalling (shape checks, data_ptr/stride lookups) only needs to
    happen once: ``with plan.record():`` runs the code normally while logging each native call
    (and any host callable registered through ``plan_call``, e.g. a collective); ``plan.replay()``
    re-issues exactly those calls.  The stream handle is part of the recorded arguments, so a
    plan must be replayed on the stream it was recorded on.
    """

    def __init__(self):
        self.calls = None

    def record(self):
        plan = self

        class _Ctx:
            def __enter__(self_):
                global _recording
                assert _recording is None, "nested launch-plan recording"
                _recording = []

            def __exit__(self_, et, ev, tb):
                global _recording
                calls, _recording = _recording, None
                if et is None:
                    plan.calls = calls
                return False
        return _Ctx()

    def replay(self):
        global launch_count
        err = 0
        for fn, args, n in self.calls:
            if n < 0:
                fn(*args)            # host callable
            else:
                err |= fn(*args)
                launch_count += n
        if err:
            raise KernelError(_lib().kh_cuda_last_error().decode())


def plan_call(fn, *args):
    """Run a host-side callable (a collective, a copy) and make it part of the plan being recorded."""
    if _recording is not None:
        _recording.append((fn, args, -1))
    fn(*args)


def plan_call_host(fn, *args):
    """Like ``plan_call`` for a host callable that itself issues native calls whose arguments change
    from step to step (an optimizer bucket: the bias corrections depend on the step number): the plan
    keeps the callable and calls it again on every replay; what it launches is not recorded."""
    global _recording
    rec = _recording
    if rec is not None:
        rec.append((fn, args, -1))
    _recording = None
    try:
        fn(*args)
    finally:
        _recording = rec


def _p(t):
    return 0 if t is None else t.data_ptr()


def _use_reference(t):
    """CPU tensors and fp32 activations on a GPU take the PyTorch fp32 evaluation of the operator
    (``reference.py``; its matrix products run on the native fp32 kernel on a GPU).  fp32 storage is
    the oracle configuration of the reference (src/core/gpt.c:332-371), not a throughput path."""
    return (not t.is_cuda) or t.dtype == torch.float32


def error_word(reset: bool = True) -> int:
    """Device-side status word: 0, or the code of the first bounded wait that ran out."""
    return int(_lib().kh_cuda_error_word(1 if reset else 0))


def check_device_status():
    w = error_word()
    if w != 0:
        raise KernelError("a kernel gave up a bounded wait (code %d)" % w)


# ----------------------------------------------------------------------------------- GEMM
def _matmul_f32(A, B):
    """A @ B for fp32 CUDA tensors (any strides) on the native CUDA-core kernel (csrc/kernels/gemm_f32.cu)."""
    M, K = A.shape
    N = B.shape[1]
    out = torch.empty(M, N, dtype=torch.float32, device=A.device)
    _call(_lib().kh_gemm_f32, 1, A.data_ptr(), A.stride(0), A.stride(1), B.data_ptr(), B.stride(0), B.stride(1),
          out.data_ptr(), N, M, N, K, _stream())
    return out


ref.matmul_f32 = _matmul_f32


def gemm(a, b, out, *, a_mn=False, b_mn=False, accumulate=False, epi=EPI_NONE, bias=None, aux=None,
         alpha=1.0, block_n=0, max_ctas=0, colsum=None):
    """out[M,N] (+)= alpha * op(a) @ op(b) with a fused epilogue.

    ``a`` is [M,K] (or [K,M] when ``a_mn``), ``b`` is [N,K] (or [K,N] when ``b_mn``); both
    bf16, row-major, last dim contiguous.  ``out`` is bf16 or fp32 (``accumulate`` only fp32).
    Epilogues: bias add; bias+GELU (``aux`` receives the pre-activation); bias+residual and
    residual (``aux`` is the residual); dGELU (``out = acc * gelu'(aux)``).
    ``colsum`` (fp32 [M], needs ``a_mn``): also receives the column sums of ``a`` -- the bias gradient
    of a weight-gradient product dW = dY^T X -- added to its content when ``accumulate``, formed from
    the operand tiles the kernel already holds in shared memory.
    """
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    assert (b.shape[0] if b_mn else b.shape[1]) == K, "gemm: inner dimensions differ"
    assert out.shape[0] == M and out.shape[1] == N
    assert colsum is None or a_mn, "gemm: column sums need the M-major A of a weight-gradient product"
    if _use_reference(a):
        if colsum is not None:
            ref.colsum(a, colsum, accumulate)
        return ref.gemm(a, b, out, a_mn, b_mn, accumulate, epi, bias, aux, alpha)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    _call(_lib().kh_gemm_bf16_colsum, 1, a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn),
                             out.data_ptr(), out.stride(0), M, N, K, int(out.dtype == torch.float32),
                             int(accumulate), epi, _p(bias), _p(aux), aux.stride(0) if aux is not None else 0,
                             float(alpha), block_n, max_ctas, _p(colsum), _stream())
    return out


SKINNY_MAX_ROWS = 64          # what the kernel accepts
SKINNY_BEST_ROWS = 16         # above this the 128-row tile kernel is faster (measured on B200)


def decode_layers_ok(G, d, H, hd, max_ctx):
    """Whether the persistent decode kernel (all layers of a step in one launch) takes this shape."""
    return bool(torch.cuda.is_available() and _lib().kh_decode_layers_ok(G, d, H, hd, max_ctx))


def decode_layers(x, xmid, qkv, att, act, layers, n_layer, H, hd, kc, vc, pos, slot, btab, bs, max_ctx, bar, *,
                  head_w=None, lnf_w=None, lnf_b=None, logits=None, vocab=0, rows=None, n_rows=0):
    """All transformer layers of one decode step (one new token per sequence) in one persistent kernel:
    ``x [G, d]`` holds the embedded tokens on entry and the last layer's output on return; k and v of the
    new tokens are appended to the paged cache ``kc``, ``vc`` ``[L, blocks, bs, H, hd]``.  ``layers`` is the
    int64 device table of twelve bf16 pointers per layer, ``bar`` four zeroed int32 words.  With ``head_w``
    the kernel also writes ``logits[i, :vocab] = LayerNorm_f(x[rows[i]]) @ head_w^T`` for ``i < n_rows``."""
    G, d = x.shape
    _call(_lib().kh_decode_layers, 1, x.data_ptr(), xmid.data_ptr(), qkv.data_ptr(), att.data_ptr(), act.data_ptr(),
          layers.data_ptr(), n_layer, G, d, H, hd, kc.data_ptr(), vc.data_ptr(), kc.stride(0), pos.data_ptr(),
          slot.data_ptr(), btab.data_ptr(), btab.shape[1], bs, max_ctx, 1.0 / float(hd) ** 0.5,
          _p(head_w), _p(lnf_w), _p(lnf_b), _p(logits), logits.stride(0) if logits is not None else 0, vocab,
          _p(rows), n_rows, bar.data_ptr(), _stream())


def gemm_skinny_scratch_elems(M, N, K):
    return int(_lib().kh_gemm_skinny_scratch_elems(M, N, K)) if torch.cuda.is_available() else 0


def gemm_skinny(x, w, out, scratch, *, epi=EPI_NONE, bias=None, aux=None, ln_w=None, ln_b=None, weights_static=False):
    """out[M,N] = x[M,K] @ w[N,K]^T (+ epilogue) for M <= 64: the weight-streaming split-K kernel used
    by decode steps.  ``scratch`` (gemm_skinny_scratch_elems fp32, zeroed once) holds ticket counters
    and split-K partials.  Epilogues: EPI_NONE, EPI_BIAS, EPI_BIAS_GELU (aux = pre-activation out),
    EPI_BIAS_RESID (aux = residual in).  With ``ln_w``/``ln_b`` (M <= SKINNY_BEST_ROWS) the product is
    taken of LayerNorm(x) * ln_w + ln_b, normalised inside the kernel.  ``weights_static``: the kernel
    launched just before this one on the stream does not write ``w`` (always true inside a decode step);
    the weight stream then starts under that kernel's tail."""
    M, K = x.shape
    N = w.shape[0]
    if _use_reference(x):
        if ln_w is not None:
            y = torch.empty_like(x)
            ref.layernorm_fwd(x, ln_w, ln_b, y, None, None)
            x = y
        return ref.gemm(x, w, out, False, False, False, epi, bias, aux, 1.0)
    _call(_lib().kh_gemm_skinny2, 1, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
          M, N, K, epi, _p(bias), _p(aux), aux.stride(0) if aux is not None else 0, scratch.data_ptr(), _p(ln_w),
          _p(ln_b), int(weights_static), _stream())
    return out


# ------------------------------------------------------------------------------ embedding
def embed_fwd(tok, pos, wte, wpe, out, T):
    if _use_reference(out):
        return ref.embed_fwd(tok, pos, wte, wpe, out, T)
    rows, d = out.shape
    _call(_lib().kh_embed_fwd, 1, tok.data_ptr(), _p(pos), wte.data_ptr(), wpe.data_ptr(), out.data_ptr(), rows, d,
                             wpe.shape[0] if pos is not None else T, wte.shape[0], _stream())
    return out


_scratch = {}


def _scratch_buf(device, nbytes, tag="colsum"):
    """Small per-device, per-purpose scratch for callers that do not pass their own (tests,
    one-off calls).  Buffers that hold ticket counters must not be shared with other uses."""
    key = (device.index, tag)
    t = _scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = t
    return t


def embed_bwd(tok, dx, dwte, dwpe, B, T, table=None):
    """dwte[tok[r]] += dx[r]; dwpe[t] += sum_b dx[b, t] (fp32 grads, deterministic).  ``table`` is
    int32 scratch of 2 * vocab entries."""
    if _use_reference(dx):
        return ref.embed_bwd(tok, dx, dwte, dwpe, B, T)
    d = dx.shape[1]
    V = dwte.shape[0] if dwte is not None else 0
    if table is None and dwte is not None:
        table = _scratch_buf(dx.device, 8 * V, "embed")
    _call(_lib().kh_embed_bwd, 3, tok.data_ptr(), dx.data_ptr(), _p(dwte), _p(dwpe), _p(table), B, T, d, V, _stream())


def colsum_scratch_elems(rows, N):
    return int(_lib().kh_colsum_scratch_elems(rows, N)) if torch.cuda.is_available() else 0


def colsum(x, out, accumulate=True, scratch=None):
    """out[j] (+)= sum_r x[r, j]; ``scratch`` (colsum_scratch_elems fp32, zero-initialised once and
    left zeroed by every call) holds ticket counters and partial rows."""
    if _use_reference(x):
        return ref.colsum(x, out, accumulate)
    rows, N = x.shape
    if scratch is None:
        scratch = _scratch_buf(x.device, 4 * colsum_scratch_elems(rows, N))
    _call(_lib().kh_colsum, 1, x.data_ptr(), x.stride(0), out.data_ptr(), scratch.data_ptr(), rows, N, int(accumulate),
                          _stream())


# ------------------------------------------------------------------------------ LayerNorm
def layernorm_fwd(x, w, b, y, mean=None, rstd=None):
    if _use_reference(x):
        return ref.layernorm_fwd(x, w, b, y, mean, rstd)
    rows, d = x.shape
    _call(_lib().kh_layernorm_fwd, 1, x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), _p(mean), _p(rstd), rows, d,
                                 _stream())
    return y


def layernorm_bwd_scratch_elems(rows, d):
    """fp32 elements of the scratch that ``layernorm_bwd`` needs (ticket counters + partial sums;
    zero-initialised once, every call leaves the counters at zero)."""
    if not torch.cuda.is_available():
        return 2 * d
    return int(_lib().kh_layernorm_bwd_scratch_elems(rows, d))


def layernorm_bwd(dy, x, w, mean, rstd, dres, dx, dw, db, partials):
    """dx = LN'(dy) (+ dres); dw += ..., db += ... (fp32, deterministic two-stage reduction)."""
    if _use_reference(x):
        return ref.layernorm_bwd(dy, x, w, mean, rstd, dres, dx, dw, db)
    rows, d = x.shape
    assert partials.numel() >= layernorm_bwd_scratch_elems(rows, d)
    _call(_lib().kh_layernorm_bwd, 2, dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                 _p(dres), dx.data_ptr(), dw.data_ptr(), db.data_ptr(), partials.data_ptr(), rows, d,
                                 _stream())


# -------------------------------------------------------------------------- cross-entropy
def xent(logits, V, target, *, coef=None, uniform=1.0, rowloss=None, prob=None, write_grad=True):
    """Fused softmax-cross-entropy over bf16 logits [R, ld]; optionally overwrites the logits
    with ``scale_r * (softmax - onehot)`` (scale_r = coef[r] or ``uniform``)."""
    if _use_reference(logits):
        return ref.xent(logits, V, target, coef, uniform, rowloss, prob, write_grad)
    _call(_lib().kh_xent, 1, logits.data_ptr(), logits.stride(0), V, target.data_ptr(), _p(coef), float(uniform),
                        _p(rowloss), _p(prob), int(write_grad), logits.shape[0], _stream())


def xent_stats(logits, V, target, v0, stats):
    """Vocabulary-parallel cross-entropy, stage 1: per row (max, sum exp(x - max), target logit or -inf)
    over this rank's vocabulary slice [v0, v0 + V); ``stats`` is fp32 [R, 3]."""
    if _use_reference(logits):
        return ref.xent_stats(logits, V, target, v0, stats)
    _call(_lib().kh_xent_stats, 1, logits.data_ptr(), logits.stride(0), V, target.data_ptr(), int(v0), stats.data_ptr(),
          logits.shape[0], _stream())


def xent_grad(logits, V, target, v0, gmax, gsum, *, coef=None, uniform=1.0):
    """Stage 2: overwrite the local logits with ``scale_r * (exp(x - gmax) / gsum - onehot)`` given the
    statistics combined over all vocabulary slices."""
    if _use_reference(logits):
        return ref.xent_grad(logits, V, target, v0, gmax, gsum, coef, uniform)
    _call(_lib().kh_xent_grad, 1, logits.data_ptr(), logits.stride(0), V, target.data_ptr(), int(v0), gmax.data_ptr(),
          gsum.data_ptr(), _p(coef), float(uniform), logits.shape[0], _stream())


def sum_f32(x, out, scale=1.0, accumulate=False):
    if not x.is_cuda:
        s = x.double().sum().float() * scale
        out[0] = out[0] + s if accumulate else s
        return
    _call(_lib().kh_sum_f32, 1, x.data_ptr(), x.numel(), float(scale), out.data_ptr(), int(accumulate), _stream())


# ----------------------------------------------------------------------------------- GRPO
def grpo_advantages(rew, n_groups, group, eps, out):
    """out[g, i] = (rew[g, i] - mean_g) / (population std_g + eps) (src/core/grpo.c:7-20), where the rewards live."""
    if not rew.is_cuda:
        _native.rt().kh_grpo_advantages(rew.data_ptr(), n_groups, group, eps, out.data_ptr())
        return out
    _call(_lib().kh_grpo_advantages_dev, 1, rew.data_ptr(), out.data_ptr(), n_groups, group, float(eps), _stream())
    return out


def grpo_coef(adv, p_cur, p_ref, rows, T, t0, t1, beta, out):
    """Per-token coefficient of the GRPO gradient (src/grpo_train.c:164-174): for the completion positions
    t0..t1 (adv[row] - beta (1 - p_ref / max(p_cur, 1e-8))) / (rows (t1 - t0 + 1)), zero elsewhere."""
    if not adv.is_cuda:
        _native.rt().kh_grpo_coef(adv.data_ptr(), p_cur.data_ptr(), p_ref.data_ptr(), rows, T, t0, t1, beta, out.data_ptr())
        return out
    _call(_lib().kh_grpo_coef_dev, 1, adv.data_ptr(), p_cur.data_ptr(), p_ref.data_ptr(), out.data_ptr(), rows, T, t0, t1,
          float(beta), _stream())
    return out


# ---------------------------------------------------------------------------------- AdamW
def adamw(p, g, m, v, pb, *, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, zero_grad=True):
    """One fused pass: moments, decoupled decay on every element, fp32 master update, bf16
    compute copy (``pb``, may be None) and gradient clear.  ``step`` is 1-based."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not p.is_cuda:
        return ref.adamw(p, g, m, v, pb, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, zero_grad)
    _call(_lib().kh_adamw, 1, p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _p(pb), p.numel(), lr, beta1, beta2,
                         eps, wd, bc1, bc2, grad_scale, int(zero_grad), _stream())


def cast_f32_bf16(x, y):
    if not x.is_cuda or y.dtype == torch.float32:
        y.copy_(x)
        return
    _call(_lib().kh_cast_f32_bf16, 1, x.data_ptr(), y.data_ptr(), x.numel(), _stream())


def add_bf16(a, b, c):
    if _use_reference(a):
        c.copy_((a.float() + b.float()))
        return
    _call(_lib().kh_add_bf16, 1, a.data_ptr(), b.data_ptr(), c.data_ptr(), a.numel(), _stream())


def flush_l2(buf):
    """Overwrite ``buf`` (a CUDA tensor larger than L2) so the next kernel starts cold."""
    _call(_lib().kh_fill_u32, 1, buf.data_ptr(), buf.numel() * buf.element_size() // 4, 0, _stream())


# ------------------------------------------------------------------------------ attention
_pad_cache = {}


def _pad_bufs(qkv, B, T, H, hd, hp):
    """Head dims below 64 run on the 64-wide kernel: q, k, v are zero-padded per head into cached
    side buffers (zero columns change neither the scores nor the outputs)."""
    key = (qkv.device.index, B, T, H, hd)
    bufs = _pad_cache.get(key)
    if bufs is None:
        R, dp = B * T, H * hp
        z = dict(device=qkv.device, dtype=qkv.dtype)
        bufs = dict(qkv=torch.zeros(R, 3 * dp, **z), out=torch.zeros(R, dp, **z), dout=torch.zeros(R, dp, **z),
                    dqkv=torch.zeros(R, 3 * dp, **z))
        _pad_cache[key] = bufs
    return bufs


def _pad_in(src, dst, parts, H, hd, hp):
    R = src.shape[0]
    dst.view(R, parts, H, hp)[:, :, :, :hd].copy_(src[:, :parts * H * hd].reshape(R, parts, H, hd))


def _pad_out(src, dst, parts, H, hd, hp):
    R = src.shape[0]
    dst[:, :parts * H * hd].copy_(src.view(R, parts, H, hp)[:, :, :, :hd].reshape(R, parts * H * hd))


def flash_fwd(qkv, out, lse, B, T, H, hd):
    """Causal attention over the fused projection ``qkv`` [B*T, 3*H*hd] (q | k | v blocks,
    head-major inside each); writes ``out`` [B*T, H*hd] and ``lse`` [B, H, T] (fp32)."""
    if _use_reference(qkv):
        return ref.flash_fwd(qkv, out, lse, B, T, H, hd)
    scale = 1.0 / math.sqrt(hd)
    if hd not in (64, 128):
        assert hd < 64, "head dims other than 64/128 must be below 64"
        pb = _pad_bufs(qkv, B, T, H, hd, 64)
        plan_call(_pad_in, qkv, pb["qkv"], 3, H, hd, 64)
        _call(_lib().kh_flash_fwd, 1, pb["qkv"].data_ptr(), pb["out"].data_ptr(), lse.data_ptr(), B, T, H, 64,
              pb["qkv"].stride(0), scale, _stream())
        plan_call(_pad_out, pb["out"], out, 1, H, hd, 64)
        return
    _call(_lib().kh_flash_fwd, 1, qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, H, hd, qkv.stride(0), scale,
          _stream())


def flash_bwd(qkv, out, dout, lse, dqkv, delta, B, T, H, hd):
    """Gradient of ``flash_fwd`` w.r.t. the fused projection: fills ``dqkv`` [B*T, 3*H*hd].
    ``delta`` [B, H, T] fp32 is scratch for rowsum(dO * O)."""
    if _use_reference(qkv):
        return ref.flash_bwd(qkv, out, dout, lse, dqkv, B, T, H, hd)
    scale = 1.0 / math.sqrt(hd)
    if hd not in (64, 128):
        pb = _pad_bufs(qkv, B, T, H, hd, 64)
        plan_call(_pad_in, qkv, pb["qkv"], 3, H, hd, 64)
        plan_call(_pad_in, out, pb["out"], 1, H, hd, 64)
        plan_call(_pad_in, dout, pb["dout"], 1, H, hd, 64)
        _call(_lib().kh_flash_bwd, 3, pb["qkv"].data_ptr(), pb["out"].data_ptr(), pb["dout"].data_ptr(), lse.data_ptr(),
              pb["dqkv"].data_ptr(), delta.data_ptr(), B, T, H, 64, pb["qkv"].stride(0), scale, _stream())
        plan_call(_pad_out, pb["dqkv"], dqkv, 3, H, hd, 64)
        return
    _call(_lib().kh_flash_bwd, 3, qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), dqkv.data_ptr(),
          delta.data_ptr(), B, T, H, hd, qkv.stride(0), scale, _stream())


def merge_attention(o1, lse1, o2, lse2):
    """Combine two attention results computed over disjoint key sets (same queries): the hook for
    context parallelism -- each rank (or each KV chunk of a ring pass) runs ``flash_fwd`` on its keys
    and the partial outputs are merged with their log-sum-exps.  ``o*``: [..., hd] , ``lse*``: [...]
    (natural log).  Returns (o, lse) in fp32.  Not used by the built-in trainers (no sequence beyond
    one GPU's memory is configured); the reference has no counterpart."""
    l1, l2 = lse1.float(), lse2.float()
    m = torch.maximum(l1, l2)
    w1, w2 = torch.exp(l1 - m), torch.exp(l2 - m)
    den = w1 + w2
    o = (o1.float() * w1.unsqueeze(-1) + o2.float() * w2.unsqueeze(-1)) / den.unsqueeze(-1)
    return o, m + torch.log(den)


def wait_probe(flag, target: int, limit_ms: int, status):
    """Launch the bounded-wait probe on ``flag`` (uint32/int32 CUDA tensor); see csrc/comm/wait_probe.cu."""
    _call(_lib().kh_wait_probe, 1, flag.data_ptr(), int(target), int(limit_ms), status.data_ptr(), _stream())


def p2p_put(src, dst_ptr: int, flag_ptr: int, state):
    """Push ``src`` (contiguous) to device address ``dst_ptr`` (normally a peer's mailbox slot) and then
    store-release the next sequence number to ``flag_ptr``; ``state`` = two zero-initialised int32
    device words of this slot (csrc/comm/p2p_mailbox.cu)."""
    _call(_lib().kh_p2p_put, 1, src.data_ptr(), int(dst_ptr), src.numel() * src.element_size(), int(flag_ptr),
          state.data_ptr(), _stream())


def p2p_wait(flag_ptr: int, expected, limit_ms: int):
    """Stream-ordered bounded wait until the counter at ``flag_ptr`` reaches the next expected value
    (``expected`` = one int32 device word, advanced on success); code 7 in the error word on time-out."""
    _call(_lib().kh_p2p_wait, 1, int(flag_ptr), expected.data_ptr(), int(limit_ms), _stream())


# ------------------------------------------------------------------------------ paged KV
def append_kv(qkv, kc, vc, pos, slot, btab, bs, H, hd, ntok):
    """Scatter k, v of each new token into its block: pool layout [n_blocks, bs, H, hd]."""
    if _use_reference(qkv):
        return ref.append_kv(qkv, kc, vc, pos, slot, btab, bs, H, hd, ntok)
    _call(_lib().kh_append_kv, 1, qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(),
                             slot.data_ptr(), btab.data_ptr(), btab.stride(0), bs, H, hd, ntok, _stream())


def paged_attn(qkv, kc, vc, out, pos, slot, btab, bs, H, hd, ntok, max_ctx, append=False, n_split=1, scratch=None):
    """Causal attention of each listed token over positions 0..pos of its own sequence, K/V read
    through the block table.  ``append``: the kernel itself stores each token's k, v into the cache
    first (valid when no two listed tokens belong to one sequence, i.e. decode steps); otherwise
    ``append_kv`` must have run.  ``n_split`` > 1 (long contexts): the keys are cut into that many equal
    ranges of ``max_ctx``, each handled by its own CTA, and merged by their log-sum-exps; ``scratch`` is a
    float32 buffer of at least ``ntok * H * n_split * (hd + 1)`` elements."""
    if _use_reference(qkv):
        if append:
            ref.append_kv(qkv, kc, vc, pos, slot, btab, bs, H, hd, ntok)
        return ref.paged_attn(qkv, kc, vc, out, pos, slot, btab, bs, H, hd, ntok)
    if n_split > 1:
        n_o = ntok * H * n_split * hd
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= n_o + ntok * H * n_split
        _call(_lib().kh_paged_attn_split, 1, qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
              scratch.data_ptr(), scratch.data_ptr() + 4 * n_o, pos.data_ptr(), slot.data_ptr(), btab.data_ptr(),
              btab.stride(0), bs, H, hd, 1.0 / math.sqrt(hd), ntok, max_ctx, n_split, int(append), _stream())
        return
    _call(_lib().kh_paged_attn, 1, qkv.data_ptr(), qkv.stride(0), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                              pos.data_ptr(), slot.data_ptr(), btab.data_ptr(), btab.stride(0), bs, H, hd,
                              1.0 / math.sqrt(hd), ntok, max_ctx, int(append), _stream())


def gather_rows(x, rows, out, nseq):
    if _use_reference(x):
        out[:nseq].copy_(x[rows[:nseq].long()])
        return
    _call(_lib().kh_gather_rows, 1, x.data_ptr(), rows.data_ptr(), out.data_ptr(), nseq, x.shape[1], _stream())


def copy_blocks(kc, vc, pairs, npairs):
    """kc, vc: [n_layer, n_blocks, bs, H, hd]; copies block pairs[2i] -> pairs[2i+1] in all layers."""
    if npairs == 0:
        return
    if _use_reference(kc):
        for i in range(npairs):
            s, d = int(pairs[2 * i]), int(pairs[2 * i + 1])
            kc[:, d].copy_(kc[:, s])
            vc[:, d].copy_(vc[:, s])
        return
    _call(_lib().kh_copy_blocks, 1, kc.data_ptr(), vc.data_ptr(), pairs.data_ptr(), npairs, kc.shape[0],
                               kc[0, 0].numel(), kc[0].numel(), _stream())


def sample(logits, V, temperature, seed, step, rep, out, nseq, step_dev=None):
    """Greedy argmax (temperature <= 0) or a categorical draw from softmax(logits / T), on device.  With
    ``step_dev`` (three int32 words on the device: step number, low and high half of the seed) both are read
    from device memory at launch time, so a captured step can be replayed with fresh random numbers."""
    if _use_reference(logits):
        return ref.sample(logits, V, temperature, seed, step, rep, out, nseq)
    _call(_lib().kh_sample2, 1, logits.data_ptr(), logits.stride(0), V, float(temperature), int(seed), int(step),
                           _p(step_dev), rep, out.data_ptr(), nseq, _stream())
