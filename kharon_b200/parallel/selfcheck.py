"""Small correctness checks of every in-kernel collective a mesh uses, against the NCCL / PyTorch
evaluation of the same operation.  ``bench.py`` runs them before its timed region on the very
ranks, GPUs and process groups that are then timed, so a record of the multi-GPU kernels exists
wherever the benchmark ran, not only where the 2-GPU test suite did.

``fused_check(mesh, device)`` returns ``{family: max relative error, ...,
"bitwise_equal_across_ranks": bool, "error_word": int}`` reduced over all ranks:

* ``gemm_ar`` / ``gemm_rs`` / ``ag_gemm``  (tp > 1) 1024 x 512 x 384 products, both operand layouts
  of B, with and without bias + residual, two calls each so that both staging parities are used;
  ``vp_combine``: the vocabulary-parallel softmax statistics kernel against all_gather + PyTorch;
* ``zero1_step``  (dp > 1) two optimizer steps of a small arena: fused pull-reduce + AdamW + bf16
  push kernel against reduce_scatter / AdamW kernel / all_gather over NCCL;
* ``mailbox``  (pp > 1) a message put into the next stage's slot against an NCCL send / recv.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _tp_checks(mesh, device, out):
    from .fused import FusedTP
    c, grp = mesh.c, mesh.tp_group
    tp, r = c.tp, c.tp_rank
    f = FusedTP(mesh, device)
    g = torch.Generator(device=device)
    g.manual_seed(1000 + c.rank)
    gs = torch.Generator(device=device)           # same stream on every rank of the TP group
    gs.manual_seed(77 + c.rank // tp)
    M, N, K = 1024, 512, 384
    rn = lambda *s, gen=g: torch.randn(*s, device=device, generator=gen)
    e_ar, e_rs, e_ag, same = 0.0, 0.0, 0.0, True
    src0 = dist.get_global_rank(grp, 0)
    for it in range(2):
        for b_mn in (False, True):
            a = (rn(M, K) * 0.5).bfloat16()
            b = (rn(K, N) if b_mn else rn(N, K)).mul(0.1).bfloat16()
            bias, resid = rn(N, gen=gs).bfloat16(), rn(M, N, gen=gs).bfloat16()
            use = it == 0
            want = (a.float() @ (b.float() if b_mn else b.float().t())).to(torch.bfloat16).float()
            dist.all_reduce(want, group=grp)
            if use:
                want = want + bias.float() + resid.float()
            got = torch.zeros(M, N, device=device, dtype=torch.bfloat16)
            f.gemm_ar(a, b, got, b_mn=b_mn, bias=bias if use else None, resid=resid if use else None)
            e_ar = max(e_ar, _rel(got, want))
            other = got.clone()
            dist.broadcast(other, src0, group=grp)
            same = same and bool(torch.equal(other, got))
            rows = M // tp
            shard = torch.zeros(rows, N, device=device, dtype=torch.bfloat16)
            f.gemm_rs(a, b, shard, b_mn=b_mn, bias=bias if use else None,
                      resid=resid[r * rows:(r + 1) * rows] if use else None)
            e_rs = max(e_rs, _rel(shard, want[r * rows:(r + 1) * rows]))
    rows = 512
    sh, ptrs, h = f.symmetric_rows(rows, K)
    for it in range(2):
        sh.copy_((rn(rows, K) * 0.5).bfloat16())
        w = (rn(N, K, gen=gs) * 0.1).bfloat16()
        got = torch.zeros(rows * tp, N, device=device, dtype=torch.bfloat16)
        f.ag_gemm(ptrs, K, rows, w, got)
        full = [torch.empty_like(sh) for _ in range(tp)]
        dist.all_gather(full, sh.contiguous(), group=grp)
        e_ag = max(e_ag, _rel(got, torch.cat(full, 0).float() @ w.float().t()))
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)          # peers have finished reading this shard before it is rewritten
    # epilogues of the all-gather form, operand in a SymRows buffer (the sequence-parallel layer's use)
    from . import fused as fused_mod
    e_epi = 0.0
    (grp_syms, _) = f.sym_rows(rows * tp, K, count=1)
    sym = grp_syms[0][0]
    for it in range(2):
        sym.mine.copy_((rn(rows, K) * 0.5).bfloat16())
        w = (rn(N, K, gen=gs) * 0.1).bfloat16()
        bias = rn(N, gen=gs).bfloat16()
        full = [torch.empty(rows, K, device=device, dtype=torch.bfloat16) for _ in range(tp)]
        dist.all_gather(full, sym.mine.contiguous(), group=grp)
        a_full = torch.cat(full, 0).float()
        pre_want = (a_full @ w.float().t() + bias.float()).to(torch.bfloat16)
        got = torch.zeros(rows * tp, N, device=device, dtype=torch.bfloat16)
        pre = torch.zeros_like(got)
        f.ag_gemm_sym(sym, w, got, epi=ops.EPI_BIAS_GELU, bias=bias, aux=pre)
        from ..ops import reference as ref
        e_epi = max(e_epi, _rel(pre, pre_want), _rel(got, ref.gelu(pre_want.float())), _rel(sym.t, a_full))
        got2 = torch.zeros_like(got)
        f.ag_gemm_sym(sym, w, got2, epi=ops.EPI_DGELU, aux=pre)
        e_epi = max(e_epi, _rel(got2, (a_full @ w.float().t()) * ref.gelu_grad(pre.float())))
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
    # vocabulary-parallel softmax statistics: exchange + combine kernel against all_gather + PyTorch
    e_vp = 0.0
    for it in range(2):
        R = 1000
        st = rn(R, 3)
        st[:, 1] = st[:, 1].abs() + 0.1
        tg = torch.randint(0, 2 * tp, (R,), device=device, dtype=torch.int32, generator=gs)
        st[:, 2] = torch.where(tg % tp == r, st[:, 2], torch.full_like(st[:, 2], float("-inf")))
        gm, gsum, rl = (torch.zeros(R, device=device) for _ in range(3))
        f.vp_combine(st, tg, gm, gsum, rl)
        allst = [torch.empty_like(st) for _ in range(tp)]
        dist.all_gather(allst, st, group=grp)
        allst = torch.stack(allst)
        m, sm, xt = allst[..., 0], allst[..., 1], allst[..., 2]
        wm = m.max(0).values
        ws = (sm * torch.exp(m - wm)).sum(0)
        wl = torch.log(ws) + wm - xt.max(0).values
        e_vp = max(e_vp, float((gm - wm).abs().max()), float(((gsum - ws) / ws).abs().max()), float((rl - wl).abs().max()))
    out.update(gemm_ar=e_ar, gemm_rs=e_rs, ag_gemm=e_ag, ag_gemm_epilogues=e_epi, vp_combine=e_vp)
    return same


def _zero_check(mesh, device, out):
    """Two ZeRO-1 steps of a 1 Mi-element arena, fused kernel against the NCCL sequence."""
    from .zero_fused import ZeroFused
    c, grp = mesh.c, mesh.dp_group
    dp, r = c.dp, c.dp_rank
    n = 1 << 20
    shard = n // dp
    opt = dict(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
    zf = ZeroFused(mesh, device)
    g_f = zf.alloc("g", n, torch.float32)
    wb_f = zf.alloc("wb", n, torch.bfloat16)
    zf.finalize()
    gen = torch.Generator(device=device)
    gen.manual_seed(5 + c.rank % (c.tp * c.pp))           # identical start on the ranks of one DP group
    w0 = torch.randn(n, device=device, generator=gen) * 0.02
    w_f, w_n = w0.clone(), w0.clone()
    m_f, v_f = torch.zeros(shard, device=device), torch.zeros(shard, device=device)
    m_n, v_n = torch.zeros(shard, device=device), torch.zeros(shard, device=device)
    wb_n = torch.zeros(n, device=device, dtype=torch.bfloat16)
    gen.manual_seed(900 + c.rank)

    class _PS:          # the three fields ZeroFused.step reads
        pass

    ps = _PS()
    ps.w, ps.m, ps.v = w_f, m_f, v_f
    lo = r * shard
    same = True
    for step in (1, 2):
        grad = torch.randn(n, device=device, generator=gen) * 1e-2
        g_f.copy_(grad)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
        zf.step(ps, shard, step, opt)
        gs = torch.empty(shard, device=device)
        dist.reduce_scatter_tensor(gs, grad.clone(), op=dist.ReduceOp.AVG, group=grp)
        ops.adamw(w_n[lo:lo + shard], gs, m_n, v_n, wb_n[lo:lo + shard], lr=opt["lr"], beta1=opt["beta1"],
                  beta2=opt["beta2"], eps=opt["eps"], wd=opt["wd"], step=step, zero_grad=False)
        dist.all_gather_into_tensor(wb_n, wb_n[lo:lo + shard].clone(), group=grp)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
    err = max(_rel(wb_f, wb_n), _rel(w_f[lo:lo + shard], w_n[lo:lo + shard]))
    other = wb_f.clone()
    dist.broadcast(other, dist.get_global_rank(grp, 0), group=grp)
    same = bool(torch.equal(other, wb_f)) and float(g_f.abs().max()) == 0.0
    out["zero1_step"] = err
    return same


def _mailbox_check(mesh, device, out):
    from . import p2p
    c = mesh.c
    rows, cols = 256, 512
    box = p2p.Mailbox(mesh, device, 2, rows, cols, torch.bfloat16)
    gen = torch.Generator(device=device)
    gen.manual_seed(31 + c.rank)
    err = 0.0
    for i in range(2):
        msg = torch.randn(rows, cols, device=device, generator=gen).bfloat16()
        want = torch.empty_like(msg)
        reqs = []
        if not c.last:
            box.send_act(i, msg)
            reqs.append(dist.P2POp(dist.isend, msg, c.next_rank))
        if not c.first:
            reqs.append(dist.P2POp(dist.irecv, want, c.prev_rank))
        for w in dist.batch_isend_irecv(reqs):
            w.wait()
        if not c.first:
            box.wait_act(i)
            torch.cuda.synchronize(device)
            err = max(err, float((box.act_in(i).float() - want.float()).abs().max()))
    out["mailbox"] = err
    return True


def fused_check(mesh, device):
    """Run the checks that apply to ``mesh`` and reduce the results over all ranks (max of the
    errors, AND of the equalities, OR of the error words).  Collective: every rank must call it."""
    c = mesh.c
    res, same = {}, True
    if c.tp > 1:
        same = _tp_checks(mesh, device, res) and same
    if c.dp > 1:
        same = _zero_check(mesh, device, res) and same
    if c.pp > 1:
        same = _mailbox_check(mesh, device, res) and same
    torch.cuda.synchronize(device)
    word = ops.error_word()
    keys = sorted(res)
    t = torch.tensor([res[k] for k in keys] + [0.0 if same else 1.0, float(word != 0)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vals = t.tolist()
    out = {k: float("%.3g" % v) for k, v in zip(keys, vals)}
    out["bitwise_equal_across_ranks"] = vals[len(keys)] == 0.0
    out["error_word"] = int(vals[len(keys) + 1]) if word == 0 else int(word)
    return out


def passed(result, tol=1e-2):
    return (result.get("bitwise_equal_across_ranks", True) and result.get("error_word", 0) == 0
            and all(v < tol for k, v in result.items() if k not in ("bitwise_equal_across_ranks", "error_word")))
