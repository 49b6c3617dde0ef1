"""Single-GPU bf16 trainer with periodic checkpoints and ``--resume``.

Flags and defaults of the reference's ``train.exe`` (src/train.c:44-57): ``--layers 4 --d 256
--heads 4 --seq 128 --batch 32 --steps 2000 --log 50 --ckptevery 500 --lr 3e-4 --data
data/input.bin --ckpt checkpoints/train.ckpt --resume``.  Additions: ``--vocab`` (default 256,
the byte vocabulary), ``--synthetic`` (uniform random ids from the data seed instead of a
corpus), ``--wd/--beta1/--beta2``, ``--device``.  Seeds: data 42, init 1337.  The log line
``step %5d  loss %.4f  %.0f tok/s`` is the reference's (train.c:95).
"""
from __future__ import annotations

import os
import sys
import time

import torch

from .engine import TrainEngine
from .utils.cli import Flags
from .utils.rng import ByteData, SyntheticData


def main(argv=None):
    f = Flags(argv, "train")
    layers, d, heads = f.int("layers", 4), f.int("d", 256), f.int("heads", 4)
    seq, batch, steps = f.int("seq", 128), f.int("batch", 32), f.int("steps", 2000)
    log, ckptevery = f.int("log", 50), f.int("ckptevery", 500)
    lr, wd = f.float("lr", 3e-4), f.float("wd", 0.1)
    b1, b2 = f.float("beta1", 0.9), f.float("beta2", 0.95)
    vocab = f.int("vocab", 256)
    data_path, ckpt_path = f.str("data", "data/input.bin"), f.str("ckpt", "checkpoints/train.ckpt")
    resume, synthetic = f.has("resume"), f.has("synthetic")
    device = f.str("device", "cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.float32 if f.has("fp32") else torch.bfloat16
    jsonl = f.str("jsonl", "", "append one JSON object per logged step to this file")
    f.maybe_help()
    from .utils.trace import JsonlLogger
    mlog = JsonlLogger(jsonl)

    eng = TrainEngine(layers, d, heads, vocab, seq, batch, 1, device=device, dtype=dtype, lr=lr, beta1=b1, beta2=b2,
                      wd=wd, seed=1337, init="host")
    if synthetic or not os.path.exists(data_path):
        if not synthetic:
            print("train: %s not found, using synthetic uniform ids" % data_path)
        data = SyntheticData(vocab, batch, seq, 42)
    else:
        data = ByteData(data_path, batch, seq, 42)
    if resume:
        data.rng.state = eng.load(ckpt_path)
        print("resumed from %s at step %d" % (ckpt_path, eng.model.step))
    pin = eng.device.type == "cuda"
    idx = torch.empty(batch * seq, dtype=torch.int32, pin_memory=pin)
    tgt = torch.empty(batch * seq, dtype=torch.int32, pin_memory=pin)
    os.makedirs(os.path.dirname(ckpt_path) or ".", exist_ok=True)
    t0, s0 = time.perf_counter(), eng.model.step
    while eng.model.step < steps:
        data.next_into(idx, tgt)
        eng.train_step(idx, tgt)
        st = eng.model.step
        if st % log == 0 or st == steps:
            loss = eng.loss()          # the only host sync
            dt = time.perf_counter() - t0
            tps = (st - s0) * batch * seq / max(dt, 1e-9)
            print("step %5d  loss %.4f  %.0f tok/s" % (st, loss, tps), flush=True)
            mlog.log(step=st, loss=loss, tok_s=tps)
            t0, s0 = time.perf_counter(), st
        if ckptevery > 0 and st % ckptevery == 0:
            eng.save(ckpt_path, data.rng.state)
    eng.save(ckpt_path, data.rng.state)
    return eng


if __name__ == "__main__":
    main()
