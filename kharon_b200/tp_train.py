"""Pure tensor-parallel trainer (TP = world size); flags of the reference's ``tp_train``
(src/tp_train.c:24-34): ``--layers 8 --d 512 --heads 8 --seq 256 --batch 32 --steps 500 --log 50
--lr 3e-4 --data <file>`` (+ ``--vocab``, ``--synthetic``, ``--no-fused-comm``).  Every rank reads the
same batches (same seed); replicated tensors receive identical gradients by construction.  Ends
with the compute-versus-communication timing of tp_train.c:69-88 (all-reduce seam nulled)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .engine import TrainEngine
from .parallel.mesh import Mesh, init_distributed
from .pp_train import _timed
from .utils.cli import Flags
from .utils.rng import ByteData, SyntheticData


def main(argv=None):
    f = Flags(argv, "tp_train")
    L, d, H = f.int("layers", 8), f.int("d", 512), f.int("heads", 8)
    seq, batch, steps = f.int("seq", 256), f.int("batch", 32), f.int("steps", 500)
    log, lr, vocab = f.int("log", 50), f.float("lr", 3e-4), f.int("vocab", 256)
    data_path, synthetic = f.str("data", "data/input.bin"), f.has("synthetic")
    fused = not f.has("no-fused-comm")
    use_sp = f.has("sp")
    hb_s = f.float("heartbeat", 0.0, "seconds after which a silent rank counts as dead (0 = off)")
    dev_flag = f.str("device", "")
    f.maybe_help()
    rank, world, device = init_distributed(dev_flag or None)
    mesh = Mesh(world, 1, 1) if world > 1 else Mesh.single()
    hb = None
    if hb_s > 0 and world > 1:
        from .utils.watchdog import Heartbeat
        hb = Heartbeat(rank, world, interval_s=min(1.0, hb_s / 4), timeout_s=hb_s)
    eng = TrainEngine(L, d, H, vocab, seq, batch, 1, mesh=mesh, device=device,
                      dtype=torch.bfloat16 if device.type == "cuda" else torch.float32, lr=lr, fused_comm=fused, sp=use_sp,
                      heartbeat=hb)
    data = (SyntheticData(vocab, batch, seq, 42) if synthetic or not os.path.exists(data_path)
            else ByteData(data_path, batch, seq, 42))
    pin = device.type == "cuda"
    idx = torch.empty(batch * seq, dtype=torch.int32, pin_memory=pin)
    tgt = torch.empty(batch * seq, dtype=torch.int32, pin_memory=pin)
    while eng.model.step < steps:
        data.next_into(idx, tgt)
        eng.train_step(idx, tgt)
        if eng.model.step % log == 0 and rank == 0:
            print("step %5d  loss %.4f" % (eng.model.step, eng.loss()), flush=True)
    t_full = _timed(lambda: eng.train_step(idx, tgt), 10, device, world)
    m = eng.model
    saved = (m.tp_allreduce, m.fused_tp)
    m.tp_allreduce, m.fused_tp = None, None
    eng.plans.clear()
    t_comp = _timed(lambda: eng.train_step(idx, tgt), 10, device, world)
    m.tp_allreduce, m.fused_tp = saved
    eng.plans.clear()
    if rank == 0:
        print("TP%d: %.0f tok/s   step %.2f ms = compute %.2f + comms %.2f" %
              (world, batch * seq / t_full * 1e3, t_full, t_comp, t_full - t_comp))
    return eng


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
