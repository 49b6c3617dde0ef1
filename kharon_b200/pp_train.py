"""3-D mesh trainer (tensor x pipeline(1F1B) x ZeRO-1 data parallel); flags of the reference's
``pp_train`` (src/pp_train.c:58-77): ``--tp 1 --dp 1 --layers 8 --d 512 --heads 8 --seq 256 --mbatch 16
--M 16 --steps 200 --log 50 --lr 3e-4 --data <file> --ckpt <prefix>``; pipeline depth =
world / (tp * dp).  Additions: ``--vocab`` (default 256), ``--synthetic``, ``--untied-head`` (the
reference's separate head matrix on the last stage), ``--no-fused-comm`` (NCCL baseline path),
``--resume``.  Launch with torchrun, one rank per GPU.

After training it prints the reference's report (pp_train.c:160-175): bubble vs theory
(P-1)/(M+P-1), tok/s per replica and for the mesh, MFU, per-axis time breakdown obtained by
differential timing (all-reduce seam nulled, one micro-batch vs the full step, optimizer
communication in isolation), memory per rank and optimizer shard size.  All times are CUDA-event
times, maximum over ranks.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

from .engine import TrainEngine
from .models.layout import matmul_params, Config
from .parallel.mesh import Mesh, init_distributed
from .utils.cli import Flags
from .utils.rng import ByteData, SyntheticData


def _max_ms(ms, device, world):
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _timed(fn, n, device, world, warmup=2):
    """Mean device time of ``fn`` over ``n`` calls after ``warmup`` untimed ones (which absorb launch-plan
    recording, tensor-map creation and the first load of kernels a variant uses), maximum over ranks."""
    for _ in range(warmup):
        fn()
    if world > 1:
        dist.barrier()
    if device.type == "cuda":
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
    else:
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        ms = (time.perf_counter() - t0) * 1e3 / n
    return _max_ms(ms, device, world)


def main(argv=None):
    f = Flags(argv, "pp_train")
    tp, dp = f.int("tp", 1), f.int("dp", 1)
    L, d, H = f.int("layers", 8), f.int("d", 512), f.int("heads", 8)
    seq, mb, M = f.int("seq", 256), f.int("mbatch", 16), f.int("M", 16)
    steps, log, lr = f.int("steps", 200), f.int("log", 50), f.float("lr", 3e-4)
    vocab = f.int("vocab", 256)
    data_path, ckpt = f.str("data", "data/input.bin"), f.str("ckpt", "")
    synthetic, untied, resume = f.has("synthetic"), f.has("untied-head"), f.has("resume")
    fused = not f.has("no-fused-comm")
    use_sp = f.has("sp", "sequence-parallel TP layers (all-gather -> GEMM, GEMM -> reduce-scatter) instead of the fused GEMM + all-reduce")
    report = not f.has("no-report")
    dev_flag = f.str("device", "")
    trace = f.has("trace", "print a per-phase device-time table (CUDA events) at the end")
    jsonl = f.str("jsonl", "", "append one JSON object per logged step to this file")
    hb_s = f.float("heartbeat", 0.0, "seconds after which a silent rank counts as dead (0 = off)")
    pp_split = f.str("pp-split", "even", "layers per stage: even | auto | a,b,... (auto balances the head's cost)")
    pp_fuse = f.int("pp-fuse", 1, "micro-batches that travel through the pipeline stages together (identical math)")
    f.maybe_help()
    rank, world, device = init_distributed(dev_flag or None)
    mesh = Mesh(tp, None, dp) if world > 1 else Mesh.single()
    c = mesh.c
    hb = None
    if hb_s > 0 and world > 1:
        from .utils.watchdog import Heartbeat
        hb = Heartbeat(rank, world, interval_s=min(1.0, hb_s / 4), timeout_s=hb_s)
    from .utils.trace import JsonlLogger
    mlog = JsonlLogger(jsonl if rank == world - 1 else "")
    eng = TrainEngine(L, d, H, vocab, seq, mb, M, mesh=mesh, device=device,
                      dtype=torch.bfloat16 if device.type == "cuda" else torch.float32, lr=lr, untied_head=untied,
                      fused_comm=fused, trace=trace, heartbeat=hb, pp_split=pp_split, sp=use_sp, pp_fuse=pp_fuse)
    if synthetic or not os.path.exists(data_path):
        data = SyntheticData(vocab, M * mb, seq, 42)
    else:
        data = ByteData(data_path, M * mb, seq, 42)
    ntok = M * mb * seq
    pin = device.type == "cuda"
    idx = torch.empty(ntok, dtype=torch.int32, pin_memory=pin)
    tgt = torch.empty(ntok, dtype=torch.int32, pin_memory=pin)
    for _ in range(c.dp_rank):               # replica r starts r batches into the stream (pp_train.c:93)
        data.next_into(idx, tgt)
    if resume and ckpt:
        eng.load(ckpt)
    last_rank = world - 1
    while eng.model.step < steps:
        data.next_into(idx, tgt)
        eng.train_step(idx, tgt)
        st = eng.model.step
        if (st % log == 0 or st == steps) and c.last:
            loss = eng.loss()
            if rank == last_rank:
                print("step %5d  loss %.4f" % (st, loss), flush=True)
                mlog.log(step=st, loss=loss)
    if ckpt:
        eng.save(ckpt, 0)
    if trace and rank == 0:
        print("device time per phase on rank 0:\n" + eng.tracer.format())
    if hb is not None:
        hb.stop()
    if not report:
        return eng
    # ---- measurement epilogue (differential timing)
    t_step = _timed(lambda: eng.train_step(idx, tgt), 10, device, world)
    m = eng.model

    def one_micro():
        x = eng.recv_act[0] if not c.first else None
        m.forward(slot=0, x_in=x, compute_loss=False)
        m.backward(slot=0, dx_out=None if c.last else eng.recv_grad[0], inv_mb=1.0 / eng.M, loss_scale=None)

    if c.pp > 1:
        for b in eng.recv_act + eng.recv_grad:
            b.zero_()
    t_micro = _timed(one_micro, 5, device, world)
    saved_ar, saved_fused = m.tp_allreduce, m.fused_tp
    m.tp_allreduce, m.fused_tp = None, None
    t_comp = _timed(one_micro, 5, device, world)
    m.tp_allreduce, m.fused_tp = saved_ar, saved_fused
    m.zero_grads()
    t_dp = _timed(eng.optimizer_step, 5, device, world) if c.dp > 1 else 0.0
    Mt = eng.M                      # pipeline turns per step (M / pp_fuse)
    ideal = Mt * t_micro
    P = c.pp
    tokens_replica = M * mb * seq
    full = t_step
    Np = matmul_params(Config(L, d, H, vocab, seq, mb))
    peak = 1375.8e12
    try:
        peak = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                           "MEASURED_PEAKS.json")))["bf16_tflops_sustained"] * 1e12
    except Exception:
        pass
    flops_gpu = 6.0 * Np * tokens_replica / (tp * P)
    if rank == 0:
        print("bubble %.1f%% (theory %.1f%%)" % (100 * max(0.0, 1 - ideal / t_step), 100 * (P - 1) / (Mt + P - 1)))
        print("tok/s per replica %.0f   mesh %.0f" % (tokens_replica / full * 1e3, dp * tokens_replica / full * 1e3))
        print("params(matmul) %.1fM  MFU %.1f%% of %.0f TFLOP/s per GPU" % (Np / 1e6, 100 * flops_gpu / (full / 1e3) / peak, peak / 1e12))
        print("step %.1f ms = compute %.1f + TP %.1f + PP %.1f ; optimizer+DP comm %.1f (inside the step)" %
              (t_step, Mt * t_comp, Mt * (t_micro - t_comp), max(0.0, t_step - ideal - t_dp), t_dp))
        rep = eng.memory_report()
        print("memory %.2f GB/rank  optimizer state %.0f MB/rank" % (rep.get("cuda_allocated_gb", 0.0), rep["optimizer_state_mb"]))
    if world > 1:
        dist.barrier()
    return eng


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
