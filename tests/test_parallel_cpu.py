"""Distributed code paths on CPU ranks (gloo, one process per rank): tensor, pipeline, ZeRO-1
data parallel and their combination must reproduce the single-process loss trajectory and
weights; per-rank checkpoints must resume bit-exactly; a rank that raises must surface as an
error on its peers instead of a hang.  (The reference could only check this by eye on a cluster,
scripts/ice_m4_tp.sbatch .. ice_m7_3d.sbatch.)"""
import os
import socket
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KW = dict(layers=4, d_model=64, heads=4, vocab=128, seq=16, mbatch=2, n_micro=4, device="cpu", dtype=torch.float32,
          lr=1e-2, wd=0.1, eps=1e-3)   # a large eps keeps Adam from amplifying summation-order noise


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batches(dp_rank, steps, ntok, vocab):
    from kharon_b200.utils.rng import Rng
    r = Rng(100 + dp_rank)
    return [r.batch(ntok, vocab) for _ in range(steps)]


def _single(steps, dp=1):
    """Single-process oracle: with dp replicas the global batch is their concatenation."""
    from kharon_b200.engine import TrainEngine
    kw = dict(KW)
    kw["n_micro"] = KW["n_micro"] * dp
    e = TrainEngine(**kw)
    per = [_batches(r, steps, KW["n_micro"] * KW["mbatch"] * KW["seq"], KW["vocab"]) for r in range(dp)]
    losses = []
    for s in range(steps):
        idx = torch.cat([per[r][s][0] for r in range(dp)])
        tgt = torch.cat([per[r][s][1] for r in range(dp)])
        e.train_step(idx, tgt)
        losses.append(e.loss())
    return e, losses


def _worker(rank, world, port, tp, pp, dp, steps, out_dir, mode):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from kharon_b200.engine import TrainEngine
    from kharon_b200.parallel.mesh import Mesh
    mesh = Mesh(tp, pp, dp, timeout_s=60)
    extra = {}
    if mode == "classic_deferred":      # blocking 1F1B order + one weight-gradient pass at the end
        extra = dict(defer_dw=True, eager_p2p=False)
    elif mode == "not_deferred":
        extra = dict(defer_dw=False)
    elif mode == "pp_fuse":             # pairs of micro-batches travel through the pipeline as one
        extra = dict(pp_fuse=2)
    elif mode == "sp":                  # sequence-parallel layers (collective-based evaluation of the fused operators)
        extra = dict(sp=True)
    elif mode == "sp_not_deferred":
        extra = dict(sp=True, defer_dw=False)
    elif mode == "sp_replicated_head":
        extra = dict(sp=True, vocab_parallel=False)
    e = TrainEngine(mesh=mesh, pp_split="3,1" if mode == "uneven" else None, **extra, **KW)
    data = _batches(mesh.c.dp_rank, steps, e.tokens_per_step, KW["vocab"])
    losses = []
    prefix = os.path.join(out_dir, "ck")
    if mode == "resume":
        e.load(prefix)
    for s in range(e.model.step, steps):
        e.train_step(*data[s])
        losses.append(e.loss() if mesh.c.last else None)
        if mode == "save_half" and e.model.step == steps // 2:
            e.save(prefix)
            break
    e.gather_master()
    torch.save(dict(losses=losses, w=e.model.params.w.clone(), coord=(mesh.c.dp_rank, mesh.c.stage, mesh.c.tp_rank),
                    offsets=e.model.params.offsets, shapes=e.model.params.shapes, step=e.model.step),
               os.path.join(out_dir, "%s_r%d.pt" % (mode, rank)))
    dist.barrier()
    dist.destroy_process_group()


def _launch(tp, pp, dp, steps, out_dir, mode="run"):
    world = tp * pp * dp
    mp.spawn(_worker, args=(world, _free_port(), tp, pp, dp, steps, out_dir, mode), nprocs=world, join=True)
    return [torch.load(os.path.join(out_dir, "%s_r%d.pt" % (mode, r)), weights_only=False) for r in range(world)]


def _view(res, name):
    o = res["offsets"][name]
    shp = res["shapes"][name]
    n = 1
    for k in shp:
        n *= k
    return res["w"][o:o + n].view(shp)


@pytest.mark.parametrize("tp,pp,dp", [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 1), (1, 2, 2), (1, 4, 1)])
def test_mesh_matches_single_process(tp, pp, dp):
    steps = 3
    ref_e, ref_losses = _single(steps, dp)
    with tempfile.TemporaryDirectory() as d:
        res = _launch(tp, pp, dp, steps, d)
    last = [r for r in res if r["coord"][1] == pp - 1]
    for r in last:
        if dp == 1:
            assert max(abs(a - b) for a, b in zip(r["losses"], ref_losses)) < 2e-5
    if dp > 1:   # each replica reports the loss of its own half; their mean is the global loss
        for s in range(steps):
            vals = [r["losses"][s] for r in last if r["coord"][2] == 0]
            assert abs(sum(vals) / len(vals) - ref_losses[s]) < 2e-5
    # weights after 3 steps: compare shards of a few tensors with the single-process model
    P = ref_e.model.params.p
    nl = KW["layers"] // pp
    d_ = KW["d_model"]
    for r in res:
        _, stage, t = r["coord"]
        gl = stage * nl      # global index of the stage's first layer
        q = _view(r, "l0.qkv_w")
        full = P["l%d.qkv_w" % gl]
        want = torch.cat([full[k * d_ + t * d_ // tp: k * d_ + (t + 1) * d_ // tp] for k in range(3)], 0)
        assert torch.allclose(q, want, rtol=1e-4, atol=2e-5)
        fp = _view(r, "l%d.fcproj_w" % (nl - 1))
        want = P["l%d.fcproj_w" % (gl + nl - 1)][:, t * 4 * d_ // tp:(t + 1) * 4 * d_ // tp]
        assert torch.allclose(fp, want, rtol=1e-4, atol=2e-5)
        if stage == 0:
            assert torch.allclose(_view(r, "wte"), P["wte"], rtol=1e-4, atol=2e-5)
        if stage == pp - 1 and pp > 1:      # tied copy on the last stage stays equal to the embedding
            assert torch.allclose(_view(r, "head_w"), P["wte"], rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("tp,pp,mode", [(2, 1, "sp"), (2, 2, "sp"), (2, 2, "sp_not_deferred"), (2, 1, "sp_replicated_head")])
def test_sequence_parallel_matches_single_process(tp, pp, mode):
    """Sequence-parallel tensor parallelism (activations as row shards between the products, all-gather in
    front of the column-parallel products, reduce-scatter behind the row-parallel ones, LayerNorm
    gradients summed over the TP group) trains exactly like one process: losses and weights."""
    steps = 3
    ref_e, ref_losses = _single(steps, 1)
    with tempfile.TemporaryDirectory() as d:
        res = _launch(tp, pp, 1, steps, d, mode)
    P = ref_e.model.params.p
    nl = KW["layers"] // pp
    for r in res:
        _, stage, t = r["coord"]
        if stage == pp - 1:
            assert max(abs(a - b) for a, b in zip(r["losses"], ref_losses)) < 2e-5
        gl = stage * nl
        for name in ("ln1_w", "ln2_b", "proj_b"):          # replicated parameters, gradients from row shards
            assert torch.allclose(_view(r, "l0." + name), P["l%d.%s" % (gl, name)], rtol=1e-4, atol=2e-5), name
        fp = _view(r, "l%d.fcproj_w" % (nl - 1))
        d_ = KW["d_model"]
        want = P["l%d.fcproj_w" % (gl + nl - 1)][:, t * 4 * d_ // tp:(t + 1) * 4 * d_ // tp]
        assert torch.allclose(fp, want, rtol=1e-4, atol=2e-5)
        if stage == 0:
            assert torch.allclose(_view(r, "wte"), P["wte"], rtol=1e-4, atol=2e-5)
            assert torch.allclose(_view(r, "wpe"), P["wpe"], rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("mode", ["classic_deferred", "not_deferred", "pp_fuse"])
def test_pipeline_variants_match_single_process(mode):
    """The default pipeline path defers the weight gradients and sends without waiting; the 1F1B
    order with a final weight-gradient pass and the per-micro-batch form give the same training."""
    steps = 3
    _, ref_losses = _single(steps, 1)
    with tempfile.TemporaryDirectory() as d:
        res = _launch(1, 2, 1, steps, d, mode)
    last = [r for r in res if r["coord"][1] == 1][0]
    assert max(abs(a - b) for a, b in zip(last["losses"], ref_losses)) < 2e-5


def test_paired_microbatches_on_the_3d_mesh_match_single_process():
    """TP2 x PP2 x DP2 with micro-batches travelling through the stages in pairs: losses of the mesh equal the
    single-process run on the concatenated batch (vocabulary-parallel head, ZeRO-1 and tied embedding included)."""
    steps = 3
    _, ref_losses = _single(steps, 2)
    with tempfile.TemporaryDirectory() as d:
        res = _launch(2, 2, 2, steps, d, "pp_fuse")
    last = [r for r in res if r["coord"][1] == 1]
    for s in range(steps):
        vals = [r["losses"][s] for r in last if r["coord"][2] == 0]
        assert len(vals) == 2 and abs(sum(vals) / len(vals) - ref_losses[s]) < 2e-5


def test_deferred_weight_gradients_single_process():
    from kharon_b200.engine import TrainEngine
    out = {}
    for defer in (False, True):
        e = TrainEngine(defer_dw=defer, **KW)
        assert e.defer_dw == defer
        losses = []
        for idx, tgt in _batches(0, 3, e.tokens_per_step, KW["vocab"]):
            e.train_step(idx, tgt)
            losses.append(e.loss())
        out[defer] = (losses, e.model.params.w.clone())
    assert max(abs(a - b) for a, b in zip(out[True][0], out[False][0])) < 2e-5
    assert torch.allclose(out[True][1], out[False][1], rtol=1e-4, atol=2e-5)


def test_uneven_pipeline_split_matches_single_process():
    """3 + 1 layers on two stages (the head-balancing split) trains exactly like one process."""
    steps = 3
    _, ref_losses = _single(steps, 1)
    with tempfile.TemporaryDirectory() as d:
        res = _launch(1, 2, 1, steps, d, "uneven")
    last = [r for r in res if r["coord"][1] == 1][0]
    assert max(abs(a - b) for a, b in zip(last["losses"], ref_losses)) < 2e-5


def test_per_rank_checkpoint_resume_is_bit_exact():
    tp, pp, dp, steps = 1, 2, 2, 4
    with tempfile.TemporaryDirectory() as d:
        full = _launch(tp, pp, dp, steps, d, "run")
        _launch(tp, pp, dp, steps, d, "save_half")
        assert os.path.exists(os.path.join(d, "ck.r3"))
        res = _launch(tp, pp, dp, steps, d, "resume")
    for a, b in zip(full, res):
        assert b["step"] == steps
        assert torch.equal(a["w"], b["w"])
        if a["losses"][-1] is not None:
            assert a["losses"][-1] == b["losses"][-1]


def _leaving_worker(rank, world, port, steps, out_dir):
    """PP2: every rank saves its checkpoint after step steps/2; then the last rank leaves (between steps,
    nothing in flight).  The survivor's next step must end in an exception, not in a blocked send."""
    sys.path.insert(0, ROOT)
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    from kharon_b200.engine import TrainEngine
    from kharon_b200.parallel.mesh import Mesh
    from kharon_b200.utils.watchdog import CollectiveTimeout, Heartbeat, RankFailure
    mesh = Mesh(1, world, 1, timeout_s=30)
    hb = Heartbeat(rank, world, interval_s=0.2, timeout_s=2.0)
    e = TrainEngine(mesh=mesh, heartbeat=hb, **KW)
    e.p2p_timeout_s = 10.0
    data = _batches(0, steps, e.tokens_per_step, KW["vocab"])
    code = 4
    try:
        for s in range(steps):
            e.train_step(*data[s])
            e.loss() if mesh.c.last else None
            if e.model.step == steps // 2:
                e.save(os.path.join(out_dir, "ck"))
                dist.barrier()                       # both files are complete before anybody leaves
                if rank == world - 1:
                    hb.stop()
                    os._exit(3)
                time.sleep(3.0)                      # the peer's heartbeat goes stale
    except (RankFailure, CollectiveTimeout) as ex:
        open(os.path.join(out_dir, "raised_%d" % rank), "w").write("%s at step %d" % (type(ex).__name__, e.model.step))
        code = 0
    except BaseException:
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
    hb.stop()
    os._exit(code)


def test_rank_leaving_after_a_save_is_detected_and_the_job_resumes_bit_exactly():
    tp, pp, dp, steps = 1, 2, 1, 4
    with tempfile.TemporaryDirectory() as d:
        full = _launch(tp, pp, dp, steps, d, "run")
        ctx = mp.spawn(_leaving_worker, args=(2, _free_port(), steps, d), nprocs=2, join=False)
        for p in ctx.processes:
            p.join(120)
        codes = [p.exitcode for p in ctx.processes]
        assert codes == [0, 3], codes
        assert open(os.path.join(d, "raised_0")).read().endswith("at step %d" % (steps // 2))
        assert os.path.exists(os.path.join(d, "ck.r0")) and os.path.exists(os.path.join(d, "ck.r1"))
        res = _launch(tp, pp, dp, steps, d, "resume")          # the restarted job continues from the files
    for a, b in zip(full, res):
        assert b["step"] == steps
        assert torch.equal(a["w"], b["w"])
        if a["losses"][-1] is not None:
            assert a["losses"][-1] == b["losses"][-1]


def _failing_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from kharon_b200.utils.watchdog import Heartbeat
    hb = Heartbeat(rank, world, interval_s=0.2, timeout_s=2.0)
    t = torch.ones(4)
    dist.all_reduce(t)
    if rank == 1:
        hb.stop()
        os._exit(3)               # the rank dies between steps, with nothing in flight
    import time
    deadline = time.time() + 20
    dead = []
    while time.time() < deadline and not dead:
        time.sleep(0.3)
        dead = hb.dead_ranks()
    open(os.path.join(out_dir, "seen_%d" % rank), "w").write(",".join(map(str, dead)))
    hb.stop()
    if rank == 0:                 # rank 0 hosts the store: it stays until the other survivor has reported too
        while time.time() < deadline and not os.path.exists(os.path.join(out_dir, "seen_2")):
            time.sleep(0.1)
    os._exit(0 if dead == [1] else 4)


def test_dead_rank_is_detected_on_the_host():
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.spawn(_failing_worker, args=(3, _free_port(), d), nprocs=3, join=False)
        for p in ctx.processes:
            p.join(60)
        codes = [p.exitcode for p in ctx.processes]
        assert codes[1] == 3 and codes[0] == 0 and codes[2] == 0, codes
        assert open(os.path.join(d, "seen_0")).read() == "1"


def _guard_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from kharon_b200.utils.watchdog import CollectiveTimeout, Heartbeat, RankFailure, guarded
    hb = Heartbeat(rank, world, interval_s=0.2, timeout_s=1.5)
    t = torch.ones(4)
    guarded(dist.all_reduce(t, async_op=True), hb, timeout_s=20)          # a healthy collective passes through
    assert t[0].item() == world
    if rank == 1:
        hb.stop()                 # the rank goes silent between steps and never joins the next collective
        time.sleep(6)
        os._exit(3)
    t0 = time.time()
    try:
        guarded(dist.all_reduce(t, async_op=True), hb, timeout_s=30)
        verdict = "completed"
    except RankFailure as e:
        verdict = "rank_failure:" + str(e)
    except CollectiveTimeout:
        verdict = "timeout"
    open(os.path.join(out_dir, "guard_%d" % rank), "w").write("%s|%.1f" % (verdict, time.time() - t0))
    hb.stop()
    os._exit(0)


def test_guarded_collective_raises_when_a_peer_never_joins():
    """A collective whose peer went silent ends in RankFailure within the heartbeat time-out instead of
    blocking until the process-group time-out (60 s here)."""
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.spawn(_guard_worker, args=(3, _free_port(), d), nprocs=3, join=False)
        for p in ctx.processes:
            p.join(60)
        for r in (0, 2):
            verdict, secs = open(os.path.join(d, "guard_%d" % r)).read().split("|")
            assert verdict.startswith("rank_failure") and "[1]" in verdict, verdict
            assert float(secs) < 10, secs
