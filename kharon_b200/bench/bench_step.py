"""``python -m kharon_b200.bench.bench_step [iters]``: time of one full training step (forward,
backward, AdamW) of the small fixture model L2 d128 h4 V256 seq64 batch8 (reference
bench/bench_step.c) plus arena sizes."""
import json
import sys

import torch

from ..engine import TrainEngine
from ..utils.rng import Rng
from . import time_ms


def main(argv=None):
    a = [int(x) for x in (sys.argv[1:] if argv is None else argv) if x.isdigit()]
    iters = a[0] if a else 50
    eng = TrainEngine(2, 128, 4, 256, 64, 8, 1, device="cuda")
    idx, tgt = Rng(1).batch(eng.tokens_per_step, 256)
    idx, tgt = idx.cuda(), tgt.cuda()
    t = time_ms(lambda: eng.train_step(idx, tgt), iters=iters)
    res = dict(ms_per_step=t, tok_s=eng.tokens_per_step / t * 1e3, **eng.memory_report())
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
