"""Fused GEMM + collective kernels on 2 GPUs (one process per GPU): results against the NCCL /
PyTorch evaluation of the same product, bit-identical across ranks and across repeated calls,
and the training engine with the fused path against the NCCL baseline path."""
import os
import socket
import sys
import tempfile

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, part):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from kharon_b200 import ops
    from kharon_b200.parallel.mesh import Mesh, init_distributed
    from kharon_b200.parallel.fused import FusedTP
    _, _, dev = init_distributed()
    mesh = Mesh(world, 1, 1, timeout_s=120)
    f = FusedTP(mesh, dev)
    res = {}
    torch.manual_seed(100 + rank)
    M, N, K = 1024, 512, 384
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()

    def reference(a, b, b_mn, bias, resid):
        part = (a.float() @ (b.float() if b_mn else b.float().t())).to(torch.bfloat16).float()
        dist.all_reduce(part)
        if bias is not None:
            part = part + bias.float() + resid.float()
        return part

    errs, errs_rs, errs_ag, same = [], [], [], []
    for it in range(5 if part == "kernels" else 0):                      # repeated calls exercise the staging parity
        for b_mn in (False, True):
            a = (torch.randn(M, K, device=dev) * 0.5).bfloat16()
            b = (torch.randn(K, N, device=dev) if b_mn else torch.randn(N, K, device=dev)).mul(0.1).bfloat16()
            bias = torch.randn(N, device=dev).bfloat16()
            resid = torch.randn(M, N, device=dev).bfloat16()
            dist.broadcast(bias, 0); dist.broadcast(resid, 0)
            use_b = it % 2 == 0
            out = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
            f.gemm_ar(a, b, out, b_mn=b_mn, bias=bias if use_b else None, resid=resid if use_b else None)
            want = reference(a, b, b_mn, bias if use_b else None, resid if use_b else None)
            errs.append(rel(out, want))
            other = out.clone()
            dist.broadcast(other, 0)
            same.append(bool(torch.equal(other, out)))
            # reduce-scatter form: this rank's row block only
            shard = torch.zeros(M // world, N, device=dev, dtype=torch.bfloat16)
            rs = resid[rank * M // world:(rank + 1) * M // world] if use_b else None
            f.gemm_rs(a, b, shard, b_mn=b_mn, bias=bias if use_b else None, resid=rs)
            errs_rs.append(rel(shard, want[rank * M // world:(rank + 1) * M // world]))
    # all-gather -> GEMM: A = concat of per-rank shards in symmetric memory
    rows = 512
    if part == "kernels":
        sh, ptrs, h = f.symmetric_rows(rows, K)
    for it in range(3 if part == "kernels" else 0):
        sh.copy_((torch.randn(rows, K, device=dev) * 0.5).bfloat16())
        w = (torch.randn(N, K, device=dev) * 0.1).bfloat16()
        out = torch.zeros(rows * world, N, device=dev, dtype=torch.bfloat16)
        f.ag_gemm(ptrs, K, rows, w, out)
        full = [torch.empty_like(sh) for _ in range(world)]
        dist.all_gather(full, sh.contiguous())
        want = torch.cat(full, 0).float() @ w.float().t()
        errs_ag.append(rel(out, want))
        torch.cuda.synchronize()
        dist.barrier()          # the shard is rewritten next iteration
    # vocabulary-parallel softmax statistics: exchange + combine kernel against all_gather + PyTorch
    errs_vp = []
    for it in range(3 if part == "kernels" else 0):
        R = 700                                       # three row blocks, the last one partial
        st = torch.randn(R, 3, device=dev)
        st[:, 1] = st[:, 1].abs() + 0.1
        tg = torch.randint(0, 2 * world, (R,), device=dev, dtype=torch.int32)
        dist.broadcast(tg, 0)
        st[:, 2] = torch.where(tg % world == rank, st[:, 2], torch.full_like(st[:, 2], float("-inf")))
        tg = torch.where(tg >= 2 * world - 1, torch.full_like(tg, -1), tg)      # some ignored rows
        gm, gs, rl = (torch.zeros(R, device=dev) for _ in range(3))
        f.vp_combine(st, tg, gm, gs, rl)
        allst = [torch.empty_like(st) for _ in range(world)]
        dist.all_gather(allst, st)
        allst = torch.stack(allst)
        m, sm, xt = allst[..., 0], allst[..., 1], allst[..., 2]
        wm = m.max(0).values
        ws = (sm * torch.exp(m - wm)).sum(0)
        wl = torch.where(tg >= 0, torch.log(ws) + wm - xt.max(0).values, torch.zeros_like(wm))
        torch.cuda.synchronize()
        errs_vp.append(max(float((gm - wm).abs().max()), float(((gs - ws) / ws).abs().max()), float((rl - wl).abs().max())))
    res["errs_vp"] = errs_vp
    torch.cuda.synchronize()
    res["errs"], res["errs_rs"], res["errs_ag"], res["same"], res["word"] = errs, errs_rs, errs_ag, same, ops.error_word()

    from kharon_b200.engine import TrainEngine
    from kharon_b200.utils.rng import Rng
    kw = dict(layers=2, d_model=256, heads=4, vocab=512, seq=128, mbatch=4, n_micro=2, device=dev, lr=1e-3, wd=0.0,
              mesh=mesh)
    if part in ("tp", "all"):
        # engine: fused path vs NCCL baseline path, TP = world
        losses, grads = {}, {}
        for name, opt in (("nccl", dict(fused_comm=False)), ("fused_ar", dict(fused_comm=True, sp=False)),
                          ("fused_sp", dict(fused_comm=True, sp=True))):
            e = TrainEngine(**opt, **kw)
            assert e.sp == (name == "fused_sp")
            idx, tgt = Rng(5).batch(e.tokens_per_step, 512)
            # gradients of the first step, before the optimizer consumes them
            e._upload(idx, tgt)
            m = e.model
            for mb in range(e.M):
                e._stage_input(mb)
                m.forward(slot=0, compute_loss=False)
                m.backward(slot=0, inv_mb=1.0 / e.M, loss_scale=1.0 / e.M, accumulate_loss=mb > 0)
            m.sync_head_grad()
            e._sync_sp_grads()
            torch.cuda.synchronize()
            grads[name] = m.params.g.clone().cpu()
            m.params.g.zero_()
            ls = []
            for _ in range(6):
                e.train_step(idx, tgt)
                ls.append(e.loss())
            losses[name] = ls
        res["losses"] = {False: losses["nccl"], True: losses["fused_ar"]}
        res["losses_sp"] = losses["fused_sp"]
        gn = grads["nccl"].norm()
        res["grad_err_ar"] = ((grads["fused_ar"] - grads["nccl"]).norm() / gn).item()
        res["grad_err_sp"] = ((grads["fused_sp"] - grads["nccl"]).norm() / gn).item()
        # vocabulary-parallel head (the default) against the replicated head, odd vocabulary
        kv = dict(kw, vocab=509)
        vp = {}
        for split in (False, True):
            e = TrainEngine(fused_comm=True, vocab_parallel=split, **kv)
            idx, tgt = Rng(6).batch(e.tokens_per_step, 509)
            ls = []
            for _ in range(5):
                e.train_step(idx, tgt)
                ls.append(e.loss())
            vp[split] = (ls, e.model.params.w.clone().cpu())
        res["vp_losses"] = {k: v[0] for k, v in vp.items()}
        res["vp_werr"] = ((vp[True][1] - vp[False][1]).norm() / vp[False][1].norm()).item()
    if part in ("pp", "all"):
        # pipeline (PP = world): mailbox transport + deferred weight gradients vs blocking NCCL 1F1B
        from kharon_b200.parallel import p2p
        p2p.WAIT_LIMIT_MS = 4000
        mesh_pp = Mesh(1, world, 1, timeout_s=120)
        kp = dict(kw, mesh=mesh_pp, n_micro=4)
        pl = {}
        for name, opt in (("mailbox", dict(fused_comm=True)), ("nccl_deferred", dict(fused_comm=False)),
                          ("nccl_1f1b", dict(fused_comm=False, defer_dw=False)), ("mailbox_again", dict(fused_comm=True))):
            e = TrainEngine(**opt, **kp)
            idx, tgt = Rng(7).batch(e.tokens_per_step, 512)
            ls = []
            for _ in range(5):
                e.train_step(idx, tgt)
                ls.append(e.loss() if mesh_pp.c.last else 0.0)
            pl[name] = ls
        res["pp_losses"] = pl
    if part in ("zero", "all"):
        # ZeRO-1: fused reduce-scatter + AdamW + bf16 all-gather kernel vs the NCCL path, DP = world
        mesh_dp = Mesh(1, 1, world, timeout_s=120)
        kw["mesh"] = mesh_dp
        zl, zw = {}, {}
        for fused in (False, True):
            e = TrainEngine(fused_comm=fused, **kw)
            idx, tgt = Rng(50 + mesh_dp.c.dp_rank).batch(e.tokens_per_step, 512)
            ls = []
            for _ in range(6):
                e.train_step(idx, tgt)
                ls.append(e.loss())
            e.gather_master()
            zl[fused], zw[fused] = ls, e.model.params.w.clone().cpu()
            assert e.model.params.g.abs().max().item() == 0
        res["zero_losses"] = zl
        res["zero_werr"] = ((zw[True] - zw[False]).norm() / zw[False].norm()).item()
    torch.cuda.synchronize()
    res["word2"] = ops.error_word()
    torch.save(res, os.path.join(out_dir, "r%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


def _run(part):
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, _free_port(), d, part), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, "r%d.pt" % r), weights_only=False) for r in range(2)]
    for r in res:
        assert r["word"] == 0 and r["word2"] == 0
    return res


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
def test_fused_tp_kernels_two_gpus():
    for r in _run("kernels"):
        assert max(r["errs"]) < 1e-2, ("gemm_ar", r["errs"])
        assert max(r["errs_rs"]) < 1e-2, ("gemm_rs", r["errs_rs"])
        assert max(r["errs_ag"]) < 1e-2, ("ag_gemm", r["errs_ag"])
        assert max(r["errs_vp"]) < 1e-5, ("vp_combine", r["errs_vp"])
        assert all(r["same"])
        assert r["word"] == 0


@needs2
def test_tp_engine_fused_matches_nccl_two_gpus():
    res = _run("tp")
    for r in res:
        a, b, c = r["losses"][False], r["losses"][True], r["losses_sp"]
        assert max(abs(x - y) for x, y in zip(a, b)) < 3e-2, (a, b)
        assert max(abs(x - y) for x, y in zip(a, c)) < 3e-2, (a, c)
        assert b[-1] < b[0] and c[-1] < c[0]
        # one step's gradients against the NCCL path: bf16 partial sums are the only difference
        assert r["grad_err_ar"] < 1e-2, r["grad_err_ar"]
        assert r["grad_err_sp"] < 1e-2, r["grad_err_sp"]
        va, vb = r["vp_losses"][False], r["vp_losses"][True]
        assert max(abs(x - y) for x, y in zip(va, vb)) < 2e-2, (va, vb)
        assert r["vp_werr"] < 1e-2, r["vp_werr"]      # Adam turns bf16-level gradient noise into sign flips
    assert res[0]["losses"][True] == res[1]["losses"][True]


@needs2
def test_pipeline_mailbox_matches_nccl_two_gpus():
    for r in _run("pp"):
        _check_pp(r)


def _check_zero(r):
    za, zb = r["zero_losses"][False], r["zero_losses"][True]
    assert max(abs(x - y) for x, y in zip(za, zb)) < 2e-2, (za, zb)
    assert r["zero_werr"] < 1e-3, r["zero_werr"]


def _check_pp(r):
    for name in ("nccl_deferred", "nccl_1f1b", "mailbox_again"):
        pa, pb = r["pp_losses"]["mailbox"], r["pp_losses"][name]
        assert max(abs(x - y) for x, y in zip(pa, pb)) < 2e-2, (name, pa, pb)


@needs2
def test_zero1_fused_matches_nccl_two_gpus():
    for r in _run("zero"):
        _check_zero(r)


@needs2
def test_many_engines_in_one_process_two_gpus():
    """Eleven engines on three meshes built and dropped in one process.  Peer-mapped buffers are
    released and allocated again while the other rank's GPU may still be writing into the old ones;
    the allocation-time drain + barrier keeps late writes out of the new buffers."""
    for r in _run("all"):
        _check_pp(r)
        _check_zero(r)


def _decode_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from kharon_b200 import ops
    from kharon_b200.infer import InferEngine
    from kharon_b200.models import GPT, Config
    from kharon_b200.parallel import fused as fused_mod
    from kharon_b200.parallel.mesh import Mesh, init_distributed
    _, _, dev = init_distributed()
    mesh = Mesh(world, 1, 1, timeout_s=120)
    cfg = Config(2, 256, 4, 300, 96, 1)
    prompts = [[5, 17, 3, 9], [9, 1, 44, 23, 8, 61, 2], [70, 1]]
    outs = {}
    for mode in ("single", "nccl", "fused"):
        tp = 1 if mode == "single" else world
        m = GPT(cfg, dev, torch.bfloat16, tp=tp, tp_rank=rank if tp > 1 else 0)
        m.init_weights(1234)
        m.params.w.mul_(6.0)
        m.sync_bf16()
        if tp > 1:
            m.tp_allreduce = lambda t: dist.all_reduce(t, group=mesh.tp_group)
            if mode == "fused":
                fused_mod.install(m, mesh)
        e = InferEngine(m, block_size=8, max_seqs=5)
        toks, _, _ = e.generate(prompts, 10)
        g, st, _ = e.generate_group(prompts[1], 4, 8)
        outs[mode] = (toks, g)
    torch.cuda.synchronize()
    torch.save(dict(outs=outs, word=ops.error_word()), os.path.join(out_dir, "d%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp_decode_fused_allreduce_two_gpus():
    """Tensor-parallel paged decode: the fused GEMM + all-reduce kernel and the NCCL seam give the
    same greedy tokens on both ranks, and (up to bf16 near-ties) the single-GPU tokens."""
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_decode_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, "d%d.pt" % r), weights_only=False) for r in range(2)]
    assert res[0]["word"] == 0 and res[1]["word"] == 0
    assert res[0]["outs"]["fused"] == res[1]["outs"]["fused"], "ranks disagree (fused)"
    assert res[0]["outs"]["nccl"] == res[1]["outs"]["nccl"], "ranks disagree (nccl)"
    single = res[0]["outs"]["single"][0]
    for mode in ("fused", "nccl"):
        got = res[0]["outs"][mode][0]
        assert [len(x) for x in got] == [len(x) for x in single]
        # greedy decoding diverges for good after one bf16 near-tie, so compare the prefix up to the
        # first difference: the prompt plus at least the first generated tokens must agree
        agree = sum(x == y for s, t in zip(single, got) for x, y in zip(s, t)) / sum(len(s) for s in single)
        assert agree > 0.6, (mode, agree, single, got)
        group = res[0]["outs"][mode][1]
        assert all(x == group[0] for x in group), (mode, "group samples differ under greedy decoding")
